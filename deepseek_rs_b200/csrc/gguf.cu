// GGUF expert-tensor ingestion: the on-disk format that feeds the routed-expert path.
//
// Stands where the reference's GgufFile (engine/src/gguf.rs:23-122: header, metadata skip, tensor table, 32-byte
// aligned data offset) and the verbatim upload of Engine::open (engine/src/engine.rs:77-90, tensor names bound at
// :176-185) stand, for the tensors of this path only: blk.{il}.ffn_{gate,up,down}_exps.weight and, optionally, the
// router matrix, the hash-routing table and the shared expert. Everything is validated before a byte is copied: type
// ids and block sizes (engine/src/model.rs:29-67: F16 = 1 / 2 B, Q8_0 = 8 / 34 B per 32, Q2_K = 10 / 84 B per 256,
// IQ2_XXS = 16 / 66 B per 256, I32 = 26), dimensions against the handle's configuration, and every offset against the
// size of the file, so a truncated or mislabelled file ends in a status code and never in a fault.
// Host code only (plus cudaMemcpyAsync and the re-layout launch); no kernel is defined here.
#include <cerrno>
#include <cstdarg>
#include <cstdio>
#include <cstring>
#include <new>
#include <string>
#include <vector>

#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include "common.cuh"
#include "launch.h"

using namespace dsmoe;

struct dsmoe_gguf {
    const uint8_t *data = nullptr;
    size_t bytes = 0;
    bool mapped = false;  // data came from mmap (else it is borrowed from the caller)
    uint32_t version = 0;
    uint64_t data_offset = 0;
    struct Tensor {
        std::string name;
        uint32_t type = 0, n_dims = 0;
        uint64_t dims[4] = {1, 1, 1, 1};
        uint64_t offset = 0, nbytes = 0;
    };
    std::vector<Tensor> tensors;
    mutable char err[512] = {0};
};

namespace {

int gfail(const dsmoe_gguf *g, int code, const char *fmt, ...)
{
    if (g) {
        va_list ap;
        va_start(ap, fmt);
        vsnprintf(g->err, sizeof(g->err), fmt, ap);
        va_end(ap);
    }
    return code;
}

// bytes per block and elements per block of a tensor type id; false for ids the reference does not know either
// (engine/src/model.rs:41-67)
bool type_info(uint32_t type, uint64_t *block_bytes, uint64_t *block_elems)
{
    switch (type) {
    case DSMOE_GGUF_F32: *block_bytes = 4, *block_elems = 1; return true;
    case DSMOE_GGUF_F16: *block_bytes = 2, *block_elems = 1; return true;
    case DSMOE_GGUF_Q8_0: *block_bytes = 34, *block_elems = 32; return true;
    case DSMOE_GGUF_Q2_K: *block_bytes = 84, *block_elems = 256; return true;
    case DSMOE_GGUF_Q4_K: *block_bytes = 144, *block_elems = 256; return true;
    case DSMOE_GGUF_IQ2_XXS: *block_bytes = 66, *block_elems = 256; return true;
    case DSMOE_GGUF_I32: *block_bytes = 4, *block_elems = 1; return true;
    default: return false;
    }
}

struct Reader {
    const uint8_t *p;
    size_t n, cur = 0;
    bool ok = true;
    bool need(size_t k)
    {
        if (!ok || k > n - cur) ok = false;
        return ok;
    }
    uint32_t u32()
    {
        uint32_t v = 0;
        if (need(4)) memcpy(&v, p + cur, 4), cur += 4;
        return v;
    }
    uint64_t u64()
    {
        uint64_t v = 0;
        if (need(8)) memcpy(&v, p + cur, 8), cur += 8;
        return v;
    }
    bool str(std::string *out)
    {
        const uint64_t len = u64();
        if (!ok || len > n - cur) return ok = false;
        if (out) out->assign(reinterpret_cast<const char *>(p + cur), (size_t)len);
        cur += (size_t)len;
        return true;
    }
    // skips one metadata value of the given type code (engine/src/gguf.rs:207-266)
    bool skip(uint32_t vtype, int depth = 0)
    {
        static const int fixed[13] = {1, 1, 2, 2, 4, 4, 4, 1, -1, -1, 8, 8, 8};
        if (vtype > 12 || depth > 4) return ok = false;
        if (fixed[vtype] > 0) {
            if (need((size_t)fixed[vtype])) cur += (size_t)fixed[vtype];
            return ok;
        }
        if (vtype == 8) return str(nullptr);
        const uint32_t et = u32();
        const uint64_t count = u64();
        if (!ok || et > 12) return ok = false;
        if (fixed[et] > 0) {  // arrays of scalars are skipped in one step
            if (count > (n - cur) / (uint64_t)fixed[et]) return ok = false;
            cur += (size_t)(count * (uint64_t)fixed[et]);
            return true;
        }
        for (uint64_t i = 0; i < count && ok; ++i) skip(et, depth + 1);
        return ok;
    }
};

int parse(dsmoe_gguf *g)
{
    Reader r{g->data, g->bytes};
    const uint32_t magic = r.u32();
    if (!r.ok || magic != 0x46554747u) return gfail(g, DSMOE_ERR_ARG, "not a GGUF file (magic %08x)", magic);
    g->version = r.u32();
    if (!r.ok || g->version < 2 || g->version > 3) return gfail(g, DSMOE_ERR_ARG, "unsupported GGUF version %u", g->version);
    const uint64_t n_tensors = r.u64(), n_kv = r.u64();
    if (!r.ok) return gfail(g, DSMOE_ERR_BOUNDS, "file ends inside the header");
    for (uint64_t i = 0; i < n_kv; ++i) {  // metadata is skipped: the path uses fixed model constants, as the reference does
        r.str(nullptr);
        const uint32_t vtype = r.u32();
        if (!r.ok || !r.skip(vtype)) return gfail(g, DSMOE_ERR_BOUNDS, "file ends inside (or has an unknown type in) metadata entry %llu", (unsigned long long)i);
    }
    if (n_tensors > (g->bytes - r.cur) / 24) return gfail(g, DSMOE_ERR_BOUNDS, "tensor count %llu does not fit the file", (unsigned long long)n_tensors);
    g->tensors.reserve((size_t)n_tensors);
    for (uint64_t i = 0; i < n_tensors; ++i) {
        dsmoe_gguf::Tensor t;
        r.str(&t.name);
        t.n_dims = r.u32();
        if (!r.ok || t.n_dims == 0 || t.n_dims > 4) return gfail(g, DSMOE_ERR_BOUNDS, "tensor %llu: bad or truncated entry", (unsigned long long)i);
        for (uint32_t d = 0; d < t.n_dims; ++d) t.dims[d] = r.u64();
        t.type = r.u32();
        t.offset = r.u64();
        if (!r.ok) return gfail(g, DSMOE_ERR_BOUNDS, "file ends inside the entry of tensor '%s'", t.name.c_str());
        uint64_t bb, be;
        if (!type_info(t.type, &bb, &be)) return gfail(g, DSMOE_ERR_ARG, "unknown tensor type %u for '%s'", t.type, t.name.c_str());
        uint64_t elems = 1;
        for (uint32_t d = 0; d < t.n_dims; ++d) {
            if (t.dims[d] != 0 && elems > UINT64_MAX / t.dims[d]) return gfail(g, DSMOE_ERR_ARG, "tensor '%s': element count overflows", t.name.c_str());
            elems *= t.dims[d];
        }
        t.nbytes = (elems + be - 1) / be * bb;
        g->tensors.push_back(std::move(t));
    }
    g->data_offset = ((uint64_t)r.cur + 31u) & ~(uint64_t)31u;  // engine/src/gguf.rs:101-102
    for (const auto &t : g->tensors)
        if (g->data_offset > g->bytes || t.offset > g->bytes - g->data_offset || t.nbytes > g->bytes - g->data_offset - t.offset)
            return gfail(g, DSMOE_ERR_BOUNDS, "tensor '%s' (%llu bytes at offset %llu) runs past the end of the file", t.name.c_str(),
                         (unsigned long long)t.nbytes, (unsigned long long)t.offset);
    return DSMOE_OK;
}

void fill(const dsmoe_gguf *g, const dsmoe_gguf::Tensor &t, dsmoe_gguf_tensor *out)
{
    out->name = t.name.c_str();
    out->type = t.type;
    out->n_dims = t.n_dims;
    for (int d = 0; d < 4; ++d) out->dims[d] = t.dims[d];
    out->offset = t.offset;
    out->bytes = t.nbytes;
    out->host_data = g->data + g->data_offset + t.offset;
}

const dsmoe_gguf::Tensor *find(const dsmoe_gguf *g, const std::string &name)
{
    for (const auto &t : g->tensors)
        if (t.name == name) return &t;
    return nullptr;
}

}  // namespace

extern "C" {

int dsmoe_gguf_open_memory(const void *data, size_t bytes, dsmoe_gguf **out)
{
    if (!data || !out) return DSMOE_ERR_ARG;
    dsmoe_gguf *g = new (std::nothrow) dsmoe_gguf();
    if (!g) return DSMOE_ERR_NOMEM;
    g->data = static_cast<const uint8_t *>(data);
    g->bytes = bytes;
    *out = g;  // returned even on a parse error, so that the caller can read the message; close it either way
    return parse(g);
}

int dsmoe_gguf_open(const char *path, dsmoe_gguf **out)
{
    if (!path || !out) return DSMOE_ERR_ARG;
    dsmoe_gguf *g = new (std::nothrow) dsmoe_gguf();
    if (!g) return DSMOE_ERR_NOMEM;
    *out = g;
    const int fd = open(path, O_RDONLY);
    if (fd < 0) return gfail(g, DSMOE_ERR_ARG, "cannot open %s: %s", path, strerror(errno));
    struct stat st;
    if (fstat(fd, &st) != 0 || st.st_size <= 0) {
        close(fd);
        return gfail(g, DSMOE_ERR_ARG, "cannot stat %s (or it is empty)", path);
    }
    void *m = mmap(nullptr, (size_t)st.st_size, PROT_READ, MAP_PRIVATE, fd, 0);
    close(fd);
    if (m == MAP_FAILED) return gfail(g, DSMOE_ERR_NOMEM, "mmap of %s failed: %s", path, strerror(errno));
    g->data = static_cast<const uint8_t *>(m);
    g->bytes = (size_t)st.st_size;
    g->mapped = true;
    return parse(g);
}

int dsmoe_gguf_close(dsmoe_gguf *g)
{
    if (!g) return DSMOE_OK;
    if (g->mapped && g->data) munmap(const_cast<uint8_t *>(g->data), g->bytes);
    delete g;
    return DSMOE_OK;
}

const char *dsmoe_gguf_last_error(const dsmoe_gguf *g) { return g ? g->err : "null gguf"; }
uint64_t dsmoe_gguf_tensor_count(const dsmoe_gguf *g) { return g ? g->tensors.size() : 0; }
uint64_t dsmoe_gguf_data_offset(const dsmoe_gguf *g) { return g ? g->data_offset : 0; }

int dsmoe_gguf_tensor_at(const dsmoe_gguf *g, uint64_t index, dsmoe_gguf_tensor *out)
{
    if (!g || !out) return DSMOE_ERR_ARG;
    if (index >= g->tensors.size()) return gfail(g, DSMOE_ERR_BOUNDS, "tensor index %llu of %zu", (unsigned long long)index, g->tensors.size());
    fill(g, g->tensors[(size_t)index], out);
    return DSMOE_OK;
}

int dsmoe_gguf_find_tensor(const dsmoe_gguf *g, const char *name, dsmoe_gguf_tensor *out)
{
    if (!g || !name || !out) return DSMOE_ERR_ARG;
    const dsmoe_gguf::Tensor *t = find(g, name);
    if (!t) return gfail(g, DSMOE_ERR_STATE, "no tensor named '%s'", name);
    fill(g, *t, out);
    return DSMOE_OK;
}

int dsmoe_gguf_expert_shard_bytes(const dsmoe_config *cfg, uint32_t expert_count, uint64_t *gate_up_bytes, uint64_t *down_bytes)
{
    if (!cfg || !gate_up_bytes || !down_bytes || cfg->n_embd % QK_K || cfg->n_ff % QK_K) return DSMOE_ERR_ARG;
    *gate_up_bytes = (uint64_t)expert_count * cfg->n_ff * (cfg->n_embd / QK_K) * IQ2XXS_BYTES;
    *down_bytes = (uint64_t)expert_count * cfg->n_embd * (cfg->n_ff / QK_K) * Q2K_BYTES;
    return DSMOE_OK;
}

int dsmoe_gguf_upload_experts(const dsmoe_gguf *g, const dsmoe_config *cfg, dsmoe_stream stream, uint32_t gguf_layer,
                              uint32_t expert_begin, uint32_t expert_count, int layout, uint8_t *gate_dev, uint8_t *up_dev,
                              uint8_t *down_dev, uint8_t *staging_dev)
{
    if (!g || !cfg) return DSMOE_ERR_ARG;
    if (layout != DSMOE_LAYOUT_NATIVE && layout != DSMOE_LAYOUT_ROWSOA) return gfail(g, DSMOE_ERR_ARG, "unknown layout %d", layout);
    if (!gate_dev || !up_dev || !down_dev || (layout == DSMOE_LAYOUT_ROWSOA && !staging_dev))
        return gfail(g, DSMOE_ERR_ARG, "upload_experts: null device buffer%s", layout == DSMOE_LAYOUT_ROWSOA ? " (ROWSOA needs a staging buffer)" : "");
    if (cfg->n_embd == 0 || cfg->n_embd % QK_K || cfg->n_ff == 0 || cfg->n_ff % QK_K) return gfail(g, DSMOE_ERR_ARG, "upload_experts: bad configuration");
    if (expert_count == 0 || (uint64_t)expert_begin + expert_count > cfg->n_expert)
        return gfail(g, DSMOE_ERR_BOUNDS, "upload_experts: experts [%u, %u) outside 0..%u", expert_begin, expert_begin + expert_count, cfg->n_expert);
    const uintptr_t al = layout == DSMOE_LAYOUT_ROWSOA ? 15 : 3;
    if ((((uintptr_t)gate_dev | (uintptr_t)up_dev | (uintptr_t)down_dev | (uintptr_t)staging_dev) & al) != 0)
        return gfail(g, DSMOE_ERR_ARG, "upload_experts: device buffers must be %zu-byte aligned for this layout", (size_t)al + 1);
    cudaStream_t st = (cudaStream_t)stream;
    const uint32_t xb = cfg->n_embd / QK_K, mb = cfg->n_ff / QK_K;
    struct Part {
        const char *suffix;
        uint32_t type;
        uint64_t in_dim, out_dim, row_bytes;
        uint8_t *dst;
        bool iq2;
    } parts[3] = {{"ffn_gate_exps.weight", DSMOE_GGUF_IQ2_XXS, cfg->n_embd, cfg->n_ff, (uint64_t)xb * IQ2XXS_BYTES, gate_dev, true},
                  {"ffn_up_exps.weight", DSMOE_GGUF_IQ2_XXS, cfg->n_embd, cfg->n_ff, (uint64_t)xb * IQ2XXS_BYTES, up_dev, true},
                  {"ffn_down_exps.weight", DSMOE_GGUF_Q2_K, cfg->n_ff, cfg->n_embd, (uint64_t)mb * Q2K_BYTES, down_dev, false}};
    // validate all three before the first copy
    const dsmoe_gguf::Tensor *found[3];
    for (int i = 0; i < 3; ++i) {
        char name[128];
        snprintf(name, sizeof(name), "blk.%u.%s", gguf_layer, parts[i].suffix);
        const dsmoe_gguf::Tensor *t = find(g, name);
        if (!t) return gfail(g, DSMOE_ERR_STATE, "no tensor named '%s'", name);
        if (t->type != parts[i].type) return gfail(g, DSMOE_ERR_ARG, "'%s' has type id %u, expected %u", name, t->type, parts[i].type);
        // GGUF lists the fastest dimension first: [in, out, experts]
        if (t->n_dims != 3 || t->dims[0] != parts[i].in_dim || t->dims[1] != parts[i].out_dim || t->dims[2] != cfg->n_expert)
            return gfail(g, DSMOE_ERR_ARG, "'%s' has dims [%llu, %llu, %llu], expected [%llu, %llu, %u]", name,
                         (unsigned long long)t->dims[0], (unsigned long long)t->dims[1], (unsigned long long)t->dims[2],
                         (unsigned long long)parts[i].in_dim, (unsigned long long)parts[i].out_dim, cfg->n_expert);
        if (t->nbytes != (uint64_t)cfg->n_expert * parts[i].out_dim * parts[i].row_bytes)
            return gfail(g, DSMOE_ERR_ARG, "'%s' has %llu bytes, the block format implies another size", name, (unsigned long long)t->nbytes);
        found[i] = t;
    }
    for (int i = 0; i < 3; ++i) {
        const uint64_t expert_bytes = parts[i].out_dim * parts[i].row_bytes, bytes = (uint64_t)expert_count * expert_bytes;
        const uint8_t *src = g->data + g->data_offset + found[i]->offset + (uint64_t)expert_begin * expert_bytes;
        uint8_t *first = layout == DSMOE_LAYOUT_ROWSOA ? staging_dev : parts[i].dst;
        if (cudaMemcpyAsync(first, src, bytes, cudaMemcpyHostToDevice, st) != cudaSuccess)
            return gfail(g, DSMOE_ERR_CUDA, "upload_experts: copy of blk.%u.%s failed: %s", gguf_layer, parts[i].suffix, cudaGetErrorString(cudaGetLastError()));
        if (layout == DSMOE_LAYOUT_ROWSOA) {  // the staging buffer is reused by the next tensor: stream order keeps that safe
            const uint64_t rows = (uint64_t)expert_count * parts[i].out_dim;
            if (parts[i].iq2) launch_relayout_iq2xxs(st, staging_dev, parts[i].dst, rows, xb, 0);
            else launch_relayout_q2k(st, staging_dev, parts[i].dst, rows, mb, 0);
            if (cudaGetLastError() != cudaSuccess) return gfail(g, DSMOE_ERR_CUDA, "upload_experts: re-layout launch failed");
        }
    }
    return DSMOE_OK;
}

}  // extern "C"
