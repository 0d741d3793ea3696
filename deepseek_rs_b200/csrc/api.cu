// The C ABI of libdsmoe: handle, argument checks, tier-1 launch wrappers and the tier-2 layer call.
#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <new>

#include "async.cuh"
#include "common.cuh"
#include "launch.h"

using namespace dsmoe;

struct dsmoe_layer_slot {
    const uint8_t *gate, *up, *down;
    int layout;
    bool set;
};

struct dsmoe_handle {
    dsmoe_config cfg;
    int device;
    mutable char err[512];
    uint64_t launches;
    dsmoe_layer_slot *layers;
    // library-owned scratch for the tier-2 call, sized by cfg.max_tokens
    float *probs, *weights, *mid;
    int32_t *selected;
    uint8_t *xq, *midq;
    // staging for the host-buffer call
    cudaStream_t hstream;
    float *d_x, *d_logits, *d_out;
    int *d_status;  // device status block (STATUS_WORDS ints, async.cuh): [0] first device-side error code, [1] wait limit
    bool use_tma;   // stage packed rows with bulk asynchronous copies where the shapes allow (default on)
    // batched (tcgen05 grouped GEMM) path: used by the tier-2 call from prefill_min_tokens tokens upwards (default:
    // 4.5 pairs per expert; DSMOE_PREFILL_MIN_TOKENS overrides)
    uint8_t *pf_scratch;
    PrefillScratch pf_lay;
    uint32_t prefill_min_tokens;
    cudaEvent_t phase_events[6];
    bool phase_events_set;
    // scratch of the shared-expert call, for sh_chunk tokens at a time
    uint32_t sh_chunk;
    int8_t *sh_xq;
    float *sh_xscale, *sh_gate, *sh_up, *sh_mid;
};

namespace {

int fail(const dsmoe_handle *h, int code, const char *fmt, ...)
{
    if (h) {
        va_list ap;
        va_start(ap, fmt);
        vsnprintf(h->err, sizeof(h->err), fmt, ap);
        va_end(ap);
    }
    return code;
}

int check_launch(dsmoe_handle *h, const char *what, int n_launched)
{
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return fail(h, DSMOE_ERR_CUDA, "%s: %s", what, cudaGetErrorString(e));
    h->launches += (uint64_t)n_launched;
    return DSMOE_OK;
}

bool aligned(const void *p, size_t a) { return ((uintptr_t)p & (a - 1)) == 0; }

// A handle's pointers and streams belong to its device: a call made while another device is current would launch
// there with this device's pointers. Such calls are refused.
int check_device(const dsmoe_handle *h);

int check_layout(const dsmoe_handle *h, int layout)
{
    if (layout != DSMOE_LAYOUT_NATIVE && layout != DSMOE_LAYOUT_ROWSOA)
        return fail(h, DSMOE_ERR_ARG, "unknown layout %d", layout);
    return DSMOE_OK;
}

template <typename T>
cudaError_t dev_alloc(T **p, size_t n)
{
    *p = nullptr;
    return n ? cudaMalloc((void **)p, n * sizeof(T)) : cudaSuccess;
}

#define DSMOE_ENTER(h)                              \
    do {                                            \
        if (!(h)) return DSMOE_ERR_ARG;             \
        if (int rc_ = check_device(h)) return rc_;  \
    } while (0)

#define DSMOE_REQUIRE(h, cond, ...) \
    do {                            \
        if (!(cond)) return fail((h), DSMOE_ERR_ARG, __VA_ARGS__); \
    } while (0)

int check_device(const dsmoe_handle *h)
{
    int cur = -1;
    if (cudaGetDevice(&cur) != cudaSuccess) return fail(h, DSMOE_ERR_CUDA, "cudaGetDevice failed");
    if (cur != h->device)
        return fail(h, DSMOE_ERR_STATE, "the handle belongs to device %d but device %d is current", h->device, cur);
    return DSMOE_OK;
}

}  // namespace

extern "C" {

const char *dsmoe_version(void) { return "dsmoe 0.1 (sm_100a)"; }

void dsmoe_default_config(dsmoe_config *cfg)
{
    if (!cfg) return;
    cfg->n_embd = 4096;
    cfg->n_ff = 2048;
    cfg->n_expert = 256;
    cfg->n_expert_used = 6;
    cfg->swiglu_clamp = 10.0f;
    cfg->route_scale = 1.5f;
    cfg->f16_ieee = 0;
    cfg->max_tokens = 64;
    cfg->max_layers = 1;
}

int dsmoe_create(const dsmoe_config *cfg, int device, dsmoe_handle **out)
{
    if (!cfg || !out) return DSMOE_ERR_ARG;
    *out = nullptr;
    if (cfg->n_embd == 0 || cfg->n_embd % QK_K || cfg->n_ff == 0 || cfg->n_ff % QK_K) return DSMOE_ERR_ARG;
    if (cfg->n_expert == 0 || cfg->n_expert % 32 || cfg->n_expert > 512) return DSMOE_ERR_ARG;
    if (cfg->n_expert_used == 0 || cfg->n_expert_used > MAX_K || cfg->n_expert_used > cfg->n_expert) return DSMOE_ERR_ARG;
    if (!(cfg->route_scale > 0.0f)) return DSMOE_ERR_ARG;

    int count = 0;
    if (cudaGetDeviceCount(&count) != cudaSuccess || device < 0 || device >= count) return DSMOE_ERR_CUDA;
    cudaDeviceProp prop;
    if (cudaGetDeviceProperties(&prop, device) != cudaSuccess) return DSMOE_ERR_CUDA;
    if (prop.major != 10) return DSMOE_ERR_CUDA;  // the kernels are sm_100a machine code only
    int caller_device = -1;
    cudaGetDevice(&caller_device);
    if (cudaSetDevice(device) != cudaSuccess) return DSMOE_ERR_CUDA;
    struct RestoreDevice {  // the caller's current device is put back on every way out
        int d;
        ~RestoreDevice() { if (d >= 0) cudaSetDevice(d); }
    } restore{caller_device};

    dsmoe_handle *h = new (std::nothrow) dsmoe_handle();
    if (!h) return DSMOE_ERR_NOMEM;
    memset(h, 0, sizeof(*h));
    h->cfg = *cfg;
    h->device = device;
    const size_t T = cfg->max_tokens, k = cfg->n_expert_used;
    const size_t L = cfg->max_layers ? cfg->max_layers : 1;
    h->layers = new (std::nothrow) dsmoe_layer_slot[L]();
    bool ok = h->layers != nullptr;
    ok = ok && dev_alloc(&h->probs, T * cfg->n_expert) == cudaSuccess;
    ok = ok && dev_alloc(&h->weights, T * k) == cudaSuccess;
    ok = ok && dev_alloc(&h->selected, T * k) == cudaSuccess;
    ok = ok && dev_alloc(&h->xq, T * (cfg->n_embd / QK_K) * Q8K_BYTES) == cudaSuccess;
    ok = ok && dev_alloc(&h->mid, T * k * cfg->n_ff) == cudaSuccess;
    ok = ok && dev_alloc(&h->midq, T * k * (cfg->n_ff / QK_K) * Q8K_BYTES) == cudaSuccess;
    ok = ok && dev_alloc(&h->d_x, T * cfg->n_embd) == cudaSuccess;
    ok = ok && dev_alloc(&h->d_logits, T * cfg->n_expert) == cudaSuccess;
    ok = ok && dev_alloc(&h->d_out, T * cfg->n_embd) == cudaSuccess;
    {
        h->sh_chunk = cfg->max_tokens < 1024u ? cfg->max_tokens : 1024u;
        if (h->sh_chunk == 0) h->sh_chunk = 1;  // a handle for the tier-1 calls only may be created with max_tokens 0
        const size_t C = h->sh_chunk, wide = cfg->n_embd > cfg->n_ff ? cfg->n_embd : cfg->n_ff;
        ok = ok && dev_alloc(&h->sh_xq, C * wide) == cudaSuccess;
        ok = ok && dev_alloc(&h->sh_xscale, C * ((wide + 31) / 32)) == cudaSuccess;
        ok = ok && dev_alloc(&h->sh_gate, C * cfg->n_ff) == cudaSuccess;
        ok = ok && dev_alloc(&h->sh_up, C * cfg->n_ff) == cudaSuccess;
        ok = ok && dev_alloc(&h->sh_mid, C * cfg->n_ff) == cudaSuccess;
    }
    ok = ok && cudaStreamCreateWithFlags(&h->hstream, cudaStreamNonBlocking) == cudaSuccess;
    ok = ok && dev_alloc(&h->d_status, STATUS_WORDS) == cudaSuccess &&
         cudaMemset(h->d_status, 0, STATUS_WORDS * sizeof(int)) == cudaSuccess;
    {
        const size_t pf_bytes = prefill_scratch_bytes(cfg->max_tokens, cfg->n_expert_used, cfg->n_expert, cfg->n_embd,
                                                      cfg->n_ff, &h->pf_lay);
        ok = ok && dev_alloc(&h->pf_scratch, pf_bytes) == cudaSuccess;
        const char *pm = getenv("DSMOE_PREFILL_MIN_TOKENS");
        // The grouped GEMM costs about 9.4 us per token tile (every tile decodes its expert's weights once, however
        // few rows it holds), the decode kernels about 1.9 us per (token, slot) pair, both measured on a B200. With
        // every expert hit, the batched path wins from about 4.5 pairs per expert upwards.
        const uint32_t by_occupancy = (9u * cfg->n_expert + 2u * cfg->n_expert_used - 1u) / (2u * cfg->n_expert_used);
        h->prefill_min_tokens = pm ? (uint32_t)strtoul(pm, nullptr, 10) : by_occupancy;
    }
    const char *no_tma = getenv("DSMOE_DISABLE_TMA");
    h->use_tma = !(no_tma && no_tma[0] == '1');
    if (!ok) {
        cudaGetLastError();
        dsmoe_destroy(h);
        return DSMOE_ERR_NOMEM;
    }
    *out = h;
    return DSMOE_OK;
}

int dsmoe_destroy(dsmoe_handle *h)
{
    if (!h) return DSMOE_OK;
    int caller_device = -1;
    cudaGetDevice(&caller_device);
    cudaSetDevice(h->device);
    if (h->hstream) cudaStreamDestroy(h->hstream);
    cudaFree(h->probs);
    cudaFree(h->weights);
    cudaFree(h->selected);
    cudaFree(h->xq);
    cudaFree(h->mid);
    cudaFree(h->midq);
    cudaFree(h->d_x);
    cudaFree(h->d_logits);
    cudaFree(h->d_out);
    cudaFree(h->d_status);
    cudaFree(h->pf_scratch);
    cudaFree(h->sh_xq);
    cudaFree(h->sh_xscale);
    cudaFree(h->sh_gate);
    cudaFree(h->sh_up);
    cudaFree(h->sh_mid);
    delete[] h->layers;
    delete h;
    if (caller_device >= 0) cudaSetDevice(caller_device);
    return DSMOE_OK;
}

const char *dsmoe_last_error(const dsmoe_handle *h) { return h ? h->err : "null handle"; }

int dsmoe_set_phase_events(dsmoe_handle *h, void **events, int n_events)
{
    DSMOE_ENTER(h);
    if (!events || n_events == 0) {
        h->phase_events_set = false;
        return DSMOE_OK;
    }
    if (n_events != 6) return fail(h, DSMOE_ERR_ARG, "set_phase_events: expected 6 events, got %d", n_events);
    for (int i = 0; i < 6; ++i) h->phase_events[i] = (cudaEvent_t)events[i];
    h->phase_events_set = true;
    return DSMOE_OK;
}

int dsmoe_device_status(dsmoe_handle *h, dsmoe_stream stream, int *code_out)
{
    if (!h || !code_out) return DSMOE_ERR_ARG;
    if (int rc = check_device(h)) return rc;
    cudaError_t e = cudaMemcpyAsync(code_out, h->d_status, sizeof(int), cudaMemcpyDeviceToHost, (cudaStream_t)stream);
    if (e == cudaSuccess) e = cudaStreamSynchronize((cudaStream_t)stream);
    if (e != cudaSuccess) return fail(h, DSMOE_ERR_CUDA, "device_status: %s", cudaGetErrorString(e));
    if (*code_out != 0) return fail(h, DSMOE_ERR_TIMEOUT, "a bounded device-side wait expired (code %d)", *code_out);
    return DSMOE_OK;
}
uint64_t dsmoe_launch_count(const dsmoe_handle *h) { return h ? h->launches : 0; }

int dsmoe_debug_set(dsmoe_handle *h, int what, int value)
{
    DSMOE_ENTER(h);
    DSMOE_REQUIRE(h, what == DSMOE_DEBUG_WAIT_LIMIT_KCLOCKS || what == DSMOE_DEBUG_DROP_ONE_COPY || what == DSMOE_DEBUG_CLEAR_STATUS,
                  "debug_set: unknown item %d", what);
    DSMOE_REQUIRE(h, value >= 0, "debug_set: negative value");
    const int word = what == DSMOE_DEBUG_WAIT_LIMIT_KCLOCKS ? 1 : what == DSMOE_DEBUG_DROP_ONE_COPY ? 2 : 0;
    if (what == DSMOE_DEBUG_CLEAR_STATUS) value = 0;
    if (cudaDeviceSynchronize() != cudaSuccess ||
        cudaMemcpy(h->d_status + word, &value, sizeof(int), cudaMemcpyHostToDevice) != cudaSuccess)
        return fail(h, DSMOE_ERR_CUDA, "debug_set: %s", cudaGetErrorString(cudaGetLastError()));
    return DSMOE_OK;
}

// ---------------------------------------------------------------------------------------------------------------
// tier 1
// ---------------------------------------------------------------------------------------------------------------

int dsmoe_q8k_quantize(dsmoe_handle *h, dsmoe_stream stream, const float *x, uint8_t *out, uint32_t in_dim,
                       uint32_t n_rows)
{
    DSMOE_ENTER(h);
    DSMOE_REQUIRE(h, in_dim % QK_K == 0, "q8k_quantize: in_dim %u is not a multiple of 256", in_dim);
    if (n_rows == 0 || in_dim == 0) return DSMOE_OK;
    DSMOE_REQUIRE(h, x && out, "q8k_quantize: null pointer");
    DSMOE_REQUIRE(h, aligned(x, 16) && aligned(out, 4), "q8k_quantize: x must be 16-byte and out 4-byte aligned");
    launch_q8k_quantize((cudaStream_t)stream, x, out, in_dim, n_rows);
    return check_launch(h, "q8k_quantize", 1);
}

int dsmoe_router_select(dsmoe_handle *h, dsmoe_stream stream, const float *logits, const float *bias,
                        const int32_t *hash, const int32_t *tokens, float *probs, int32_t *selected, float *weights,
                        int32_t token_scalar, uint32_t hash_rows, uint32_t n_tokens, uint32_t has_bias,
                        uint32_t hash_mode)
{
    DSMOE_ENTER(h);
    if (n_tokens == 0) return DSMOE_OK;
    DSMOE_REQUIRE(h, logits && probs && selected && weights, "router_select: null pointer");
    DSMOE_REQUIRE(h, !has_bias || bias, "router_select: has_bias set but bias is null");
    DSMOE_REQUIRE(h, !hash_mode || (hash && hash_rows > 0), "router_select: hash_mode set but no hash table");
    launch_router_select((cudaStream_t)stream, logits, has_bias ? bias : nullptr, hash_mode ? hash : nullptr, tokens,
                         probs, selected, weights, token_scalar, hash_rows, n_tokens, has_bias != 0, hash_mode != 0,
                         (int)h->cfg.n_expert_used, (int)h->cfg.n_expert, h->cfg.route_scale);
    return check_launch(h, "router_select", 1);
}

int dsmoe_gate_up_mid(dsmoe_handle *h, dsmoe_stream stream, const uint8_t *gate_base, const uint8_t *up_base,
                      const uint8_t *xq, const int32_t *selected, const float *weights, float *gate_out, float *up_out,
                      float *mid_out, uint64_t gate_expert_bytes, uint64_t gate_row_bytes, uint32_t xq_blocks,
                      uint32_t expert_mid_dim, uint32_t n_expert_used, uint32_t n_tokens, float clamp, int layout)
{
    DSMOE_ENTER(h);
    if (int rc = check_layout(h, layout)) return rc;
    if (n_tokens == 0 || expert_mid_dim == 0) return DSMOE_OK;
    DSMOE_REQUIRE(h, gate_base && up_base && xq && selected && weights && mid_out, "gate_up_mid: null pointer");
    DSMOE_REQUIRE(h, n_expert_used >= 1 && n_expert_used <= MAX_K, "gate_up_mid: n_expert_used %u out of 1..8", n_expert_used);
    DSMOE_REQUIRE(h, xq_blocks >= 1 && gate_row_bytes >= (uint64_t)xq_blocks * IQ2XXS_BYTES,
                  "gate_up_mid: row stride %llu shorter than %u blocks", (unsigned long long)gate_row_bytes, xq_blocks);
    DSMOE_REQUIRE(h, aligned(gate_base, 2) && aligned(up_base, 2) && gate_row_bytes % 2 == 0 && gate_expert_bytes % 2 == 0,
                  "gate_up_mid: packed rows must be 2-byte aligned");
    DSMOE_REQUIRE(h, aligned(xq, 4), "gate_up_mid: xq must be 4-byte aligned");
    GateUpArgs a = {gate_base, up_base, xq, selected, weights, gate_out, up_out, mid_out, gate_expert_bytes,
                    gate_row_bytes, xq_blocks, expert_mid_dim, n_expert_used, n_tokens, clamp, layout,
                    (int)h->cfg.f16_ieee};
    DSMOE_REQUIRE(h, (uint64_t)n_tokens * n_expert_used <= 65535u, "gate_up_mid: n_tokens*k exceeds 65535");
    int n = (h->use_tma && gate_up_tma_eligible(a)) ? launch_gate_up_mid_tma((cudaStream_t)stream, a, h->d_status)
                                                    : launch_gate_up_mid((cudaStream_t)stream, a);
    return check_launch(h, "gate_up_mid", n);
}

static int down_common(dsmoe_handle *h, dsmoe_stream stream, const uint8_t *down_base, const uint8_t *midq,
                       const int32_t *selected, float *out, uint64_t down_expert_bytes, uint64_t down_row_bytes,
                       uint32_t midq_blocks, uint32_t out_dim, uint32_t n_expert_used, uint32_t n_tokens, int layout,
                       int sum_slots)
{
    DSMOE_ENTER(h);
    if (int rc = check_layout(h, layout)) return rc;
    if (n_tokens == 0 || out_dim == 0) return DSMOE_OK;
    DSMOE_REQUIRE(h, down_base && midq && selected && out, "down: null pointer");
    DSMOE_REQUIRE(h, n_expert_used >= 1 && n_expert_used <= MAX_K, "down: n_expert_used %u out of 1..8", n_expert_used);
    DSMOE_REQUIRE(h, midq_blocks >= 1 && down_row_bytes >= (uint64_t)midq_blocks * Q2K_BYTES,
                  "down: row stride %llu shorter than %u blocks", (unsigned long long)down_row_bytes, midq_blocks);
    DSMOE_REQUIRE(h, aligned(down_base, 4) && down_row_bytes % 4 == 0 && down_expert_bytes % 4 == 0 && aligned(midq, 4),
                  "down: packed rows and midq must be 4-byte aligned");
    DSMOE_REQUIRE(h, n_tokens <= 65535u, "down: n_tokens exceeds 65535");
    DownArgs a = {down_base, midq, selected, out, down_expert_bytes, down_row_bytes, midq_blocks, out_dim,
                  n_expert_used, n_tokens, layout, (int)h->cfg.f16_ieee, sum_slots};
    int n = (h->use_tma && down_tma_eligible(a)) ? launch_down_tma((cudaStream_t)stream, a, h->d_status)
                                                 : launch_down((cudaStream_t)stream, a);
    return check_launch(h, sum_slots ? "down_sum" : "down", n);
}

int dsmoe_down(dsmoe_handle *h, dsmoe_stream stream, const uint8_t *down_base, const uint8_t *midq,
               const int32_t *selected, float *down_out, uint64_t down_expert_bytes, uint64_t down_row_bytes,
               uint32_t midq_blocks, uint32_t out_dim, uint32_t n_expert_used, uint32_t n_tokens, int layout)
{
    return down_common(h, stream, down_base, midq, selected, down_out, down_expert_bytes, down_row_bytes, midq_blocks,
                       out_dim, n_expert_used, n_tokens, layout, 0);
}

int dsmoe_down_sum(dsmoe_handle *h, dsmoe_stream stream, const uint8_t *down_base, const uint8_t *midq,
                   const int32_t *selected, float *out, uint64_t down_expert_bytes, uint64_t down_row_bytes,
                   uint32_t midq_blocks, uint32_t out_dim, uint32_t n_expert_used, uint32_t n_tokens, int layout)
{
    return down_common(h, stream, down_base, midq, selected, out, down_expert_bytes, down_row_bytes, midq_blocks,
                       out_dim, n_expert_used, n_tokens, layout, 1);
}

int dsmoe_moe_sum(dsmoe_handle *h, dsmoe_stream stream, const float *down, float *out, uint32_t out_dim,
                  uint32_t n_expert_used, uint32_t n_tokens)
{
    DSMOE_ENTER(h);
    if (n_tokens == 0 || out_dim == 0) return DSMOE_OK;
    DSMOE_REQUIRE(h, down && out, "moe_sum: null pointer");
    launch_moe_sum((cudaStream_t)stream, down, nullptr, out, out_dim, n_expert_used, n_tokens);
    return check_launch(h, "moe_sum", 1);
}

int dsmoe_moe_sum_indexed(dsmoe_handle *h, dsmoe_stream stream, const float *rows, const int32_t *pos, float *out,
                          uint32_t out_dim, uint32_t n_expert_used, uint32_t n_tokens)
{
    DSMOE_ENTER(h);
    if (n_tokens == 0 || out_dim == 0) return DSMOE_OK;
    DSMOE_REQUIRE(h, rows && pos && out, "moe_sum_indexed: null pointer");
    launch_moe_sum((cudaStream_t)stream, rows, pos, out, out_dim, n_expert_used, n_tokens);
    return check_launch(h, "moe_sum_indexed", 1);
}

int dsmoe_quantize_q8_0(dsmoe_handle *h, dsmoe_stream stream, const float *x, int8_t *xq, float *xscale, uint64_t in_dim,
                        uint64_t n_tokens)
{
    DSMOE_ENTER(h);
    if (n_tokens == 0 || in_dim == 0) return DSMOE_OK;
    DSMOE_REQUIRE(h, x && xq && xscale, "quantize_q8_0: null pointer");
    launch_quantize_q8_0((cudaStream_t)stream, x, xq, xscale, in_dim, n_tokens);
    return check_launch(h, "quantize_q8_0", 1);
}

int dsmoe_matmul_q8_0(dsmoe_handle *h, dsmoe_stream stream, const uint8_t *w, const int8_t *xq, const float *xscale,
                      float *out, uint64_t in_dim, uint64_t out_dim, uint64_t n_tokens)
{
    DSMOE_ENTER(h);
    if (n_tokens == 0 || out_dim == 0) return DSMOE_OK;
    DSMOE_REQUIRE(h, w && xq && xscale && out, "matmul_q8_0: null pointer");
    DSMOE_REQUIRE(h, ((uintptr_t)w & 3) == 0 && ((uintptr_t)xq & 15) == 0, "matmul_q8_0: w needs 4-byte, xq 16-byte alignment");
    launch_matmul_q8_0((cudaStream_t)stream, w, xq, xscale, out, in_dim, out_dim, n_tokens);
    return check_launch(h, "matmul_q8_0", 1);
}

int dsmoe_swiglu(dsmoe_handle *h, dsmoe_stream stream, const float *gate, const float *up, float *out, uint64_t n,
                 float clamp, float weight)
{
    DSMOE_ENTER(h);
    if (n == 0) return DSMOE_OK;
    DSMOE_REQUIRE(h, gate && up && out, "swiglu: null pointer");
    launch_swiglu((cudaStream_t)stream, gate, up, out, n, clamp, weight);
    return check_launch(h, "swiglu", 1);
}

int dsmoe_matmul_f16(dsmoe_handle *h, dsmoe_stream stream, const uint16_t *w, const float *x, float *out, uint64_t in_dim,
                     uint64_t out_dim, uint64_t n_tokens)
{
    DSMOE_ENTER(h);
    if (n_tokens == 0 || out_dim == 0) return DSMOE_OK;
    DSMOE_REQUIRE(h, w && x && out, "matmul_f16: null pointer");
    DSMOE_REQUIRE(h, n_tokens <= 65535, "matmul_f16: at most 65535 tokens per call");
    launch_matmul_f16((cudaStream_t)stream, w, x, out, in_dim, out_dim, n_tokens);
    return check_launch(h, "matmul_f16", 1);
}

int dsmoe_shared_expert(dsmoe_handle *h, dsmoe_stream stream, const uint8_t *gate_w, const uint8_t *up_w,
                        const uint8_t *down_w, const float *x, uint32_t n_tokens, float *out)
{
    DSMOE_ENTER(h);
    if (n_tokens == 0) return DSMOE_OK;
    DSMOE_REQUIRE(h, gate_w && up_w && down_w && x && out, "shared_expert: null pointer");
    DSMOE_REQUIRE(h, (((uintptr_t)gate_w | (uintptr_t)up_w | (uintptr_t)down_w) & 3) == 0, "shared_expert: weights need 4-byte alignment");
    const dsmoe_config &c = h->cfg;
    cudaStream_t st = (cudaStream_t)stream;
    int n = 0;
    if (shared_fused_eligible(c.n_embd, c.n_ff, n_tokens) && n_tokens <= h->sh_chunk) {
        n = launch_shared_fused(st, gate_w, up_w, down_w, x, h->sh_mid, out, c.n_embd, c.n_ff, n_tokens, c.swiglu_clamp);
        return check_launch(h, "shared_expert", n);
    }
    for (uint32_t t0 = 0; t0 < n_tokens; t0 += h->sh_chunk) {
        const uint32_t T = n_tokens - t0 < h->sh_chunk ? n_tokens - t0 : h->sh_chunk;
        const float *xc = x + (size_t)t0 * c.n_embd;
        launch_quantize_q8_0(st, xc, h->sh_xq, h->sh_xscale, c.n_embd, T);
        launch_matmul_q8_0(st, gate_w, h->sh_xq, h->sh_xscale, h->sh_gate, c.n_embd, c.n_ff, T);
        launch_matmul_q8_0(st, up_w, h->sh_xq, h->sh_xscale, h->sh_up, c.n_embd, c.n_ff, T);
        launch_swiglu(st, h->sh_gate, h->sh_up, h->sh_mid, (uint64_t)T * c.n_ff, c.swiglu_clamp, 1.0f);
        launch_quantize_q8_0(st, h->sh_mid, h->sh_xq, h->sh_xscale, c.n_ff, T);
        launch_matmul_q8_0(st, down_w, h->sh_xq, h->sh_xscale, out + (size_t)t0 * c.n_embd, c.n_ff, c.n_embd, T);
        n += 6;
    }
    return check_launch(h, "shared_expert", n);
}

int dsmoe_dequant_iq2xxs(dsmoe_handle *h, dsmoe_stream stream, const uint8_t *blocks, uint64_t n_blocks, float *out)
{
    DSMOE_ENTER(h);
    if (n_blocks == 0) return DSMOE_OK;
    DSMOE_REQUIRE(h, blocks && out && aligned(blocks, 2), "dequant_iq2xxs: null or misaligned pointer");
    launch_dequant_iq2xxs((cudaStream_t)stream, blocks, n_blocks, out, (int)h->cfg.f16_ieee);
    return check_launch(h, "dequant_iq2xxs", 1);
}

int dsmoe_dequant_q2k(dsmoe_handle *h, dsmoe_stream stream, const uint8_t *blocks, uint64_t n_blocks, float *out)
{
    DSMOE_ENTER(h);
    if (n_blocks == 0) return DSMOE_OK;
    DSMOE_REQUIRE(h, blocks && out && aligned(blocks, 2), "dequant_q2k: null or misaligned pointer");
    launch_dequant_q2k((cudaStream_t)stream, blocks, n_blocks, out, (int)h->cfg.f16_ieee);
    return check_launch(h, "dequant_q2k", 1);
}

int dsmoe_relayout_iq2xxs(dsmoe_handle *h, dsmoe_stream stream, const uint8_t *src, uint8_t *dst, uint64_t n_rows,
                          uint32_t blocks_per_row, int inverse)
{
    DSMOE_ENTER(h);
    if (n_rows == 0 || blocks_per_row == 0) return DSMOE_OK;
    DSMOE_REQUIRE(h, src && dst && src != dst && aligned(src, 2) && aligned(dst, 2),
                  "relayout_iq2xxs: null, aliased or misaligned pointer");
    launch_relayout_iq2xxs((cudaStream_t)stream, src, dst, n_rows, blocks_per_row, inverse);
    return check_launch(h, "relayout_iq2xxs", 1);
}

int dsmoe_relayout_q2k(dsmoe_handle *h, dsmoe_stream stream, const uint8_t *src, uint8_t *dst, uint64_t n_rows,
                       uint32_t blocks_per_row, int inverse)
{
    DSMOE_ENTER(h);
    if (n_rows == 0 || blocks_per_row == 0) return DSMOE_OK;
    DSMOE_REQUIRE(h, src && dst && src != dst && aligned(src, 4) && aligned(dst, 4),
                  "relayout_q2k: null, aliased or misaligned pointer");
    launch_relayout_q2k((cudaStream_t)stream, src, dst, n_rows, blocks_per_row, inverse);
    return check_launch(h, "relayout_q2k", 1);
}

// ---------------------------------------------------------------------------------------------------------------
// FP8 block-scaled projection
// ---------------------------------------------------------------------------------------------------------------

int dsmoe_fp8_quantize(dsmoe_handle *h, dsmoe_stream stream, const float *x, uint8_t *codes, float *scales,
                       uint32_t rows, uint32_t cols, int rows_per_block)
{
    DSMOE_ENTER(h);
    DSMOE_REQUIRE(h, rows_per_block == 1 || rows_per_block == 128, "fp8_quantize: rows_per_block must be 1 or 128");
    DSMOE_REQUIRE(h, cols % 128 == 0, "fp8_quantize: cols %u is not a multiple of 128", cols);
    if (rows == 0 || cols == 0) return DSMOE_OK;
    DSMOE_REQUIRE(h, x && codes && scales && aligned(x, 16) && aligned(codes, 4), "fp8_quantize: null or misaligned pointer");
    launch_fp8_quantize((cudaStream_t)stream, x, codes, scales, rows, cols, rows_per_block);
    return check_launch(h, "fp8_quantize", 1);
}

int dsmoe_fp8_linear(dsmoe_handle *h, dsmoe_stream stream, const uint8_t *a_fp8, const float *a_scale,
                     const uint8_t *w_fp8, const float *w_scale, void *out_bf16, uint32_t M, uint32_t N, uint32_t K)
{
    DSMOE_ENTER(h);
    DSMOE_REQUIRE(h, K % 128 == 0 && N % 128 == 0 && K > 0, "fp8_linear: N %u and K %u must be multiples of 128", N, K);
    if (M == 0 || N == 0) return DSMOE_OK;
    DSMOE_REQUIRE(h, a_fp8 && a_scale && w_fp8 && w_scale && out_bf16, "fp8_linear: null pointer");
    DSMOE_REQUIRE(h, aligned(a_fp8, 16) && aligned(w_fp8, 16) && aligned(out_bf16, 4), "fp8_linear: misaligned pointer");
    int n = launch_fp8_linear((cudaStream_t)stream, a_fp8, a_scale, w_fp8, w_scale, out_bf16, M, N, K, h->d_status);
    return check_launch(h, "fp8_linear", n);
}

// ---------------------------------------------------------------------------------------------------------------
// tier 2
// ---------------------------------------------------------------------------------------------------------------

int dsmoe_layer_register(dsmoe_handle *h, uint32_t layer, const uint8_t *gate, const uint8_t *up, const uint8_t *down,
                         int layout)
{
    DSMOE_ENTER(h);
    if (int rc = check_layout(h, layout)) return rc;
    const uint32_t L = h->cfg.max_layers ? h->cfg.max_layers : 1;
    DSMOE_REQUIRE(h, layer < L, "layer_register: layer %u beyond max_layers %u", layer, L);
    DSMOE_REQUIRE(h, gate && up && down, "layer_register: null tensor");
    const size_t al = layout == DSMOE_LAYOUT_ROWSOA ? 16 : 4;
    DSMOE_REQUIRE(h, aligned(gate, al) && aligned(up, al) && aligned(down, al),
                  "layer_register: tensors must be %zu-byte aligned for this layout", al);
    h->layers[layer] = {gate, up, down, layout, true};
    return DSMOE_OK;
}

// Everything after the router and the Q8_K of x: gate/up/SwiGLU -> Q8_K(mid) -> down -> slot sum, on the decode
// kernels or, from prefill_min_tokens rows upwards, on the grouped GEMM.
static int expert_ffn_impl(dsmoe_handle *h, cudaStream_t st, const dsmoe_layer_slot &ly, const uint8_t *xq,
                           const int32_t *sel, const float *wts, uint32_t n_tokens, float *out, int n, const char *what)
{
    const dsmoe_config &c = h->cfg;
    const uint32_t k = c.n_expert_used, xb = c.n_embd / QK_K, mb = c.n_ff / QK_K;
    if (n_tokens >= h->prefill_min_tokens && prefill_eligible(c.n_embd, c.n_ff, ly.gate, ly.up, ly.down, ly.layout)) {
        PrefillArgs p = {ly.gate, ly.up, ly.down, xq, sel, wts, h->mid, h->midq, out, h->pf_scratch, h->pf_lay,
                         n_tokens, k, c.n_expert, c.n_embd, c.n_ff, c.swiglu_clamp, ly.layout, (int)c.f16_ieee,
                         h->d_status, h->phase_events_set ? h->phase_events : nullptr};
        n += launch_prefill_experts(st, p);
        return check_launch(h, what, n);
    }
    if ((uint64_t)n_tokens * k > 65535u) return fail(h, DSMOE_ERR_BOUNDS, "%s: n_tokens*k exceeds 65535 on the decode kernels", what);
    GateUpArgs g = {ly.gate, ly.up, xq, sel, wts, nullptr, nullptr, h->mid, (uint64_t)c.n_ff * xb * IQ2XXS_BYTES,
                    (uint64_t)xb * IQ2XXS_BYTES, xb, c.n_ff, k, n_tokens, c.swiglu_clamp, ly.layout, (int)c.f16_ieee};
    n += ((h->use_tma && gate_up_tma_eligible(g)) ? launch_gate_up_mid_tma(st, g, h->d_status)
                                                  : launch_gate_up_mid(st, g));
    if (int rc = check_launch(h, what, n)) return rc;
    n = 1;
    launch_q8k_quantize(st, h->mid, h->midq, c.n_ff, n_tokens * k);
    if (int rc = check_launch(h, what, n)) return rc;
    n = 0;
    DownArgs d = {ly.down, h->midq, sel, out, (uint64_t)c.n_embd * mb * Q2K_BYTES, (uint64_t)mb * Q2K_BYTES, mb,
                  c.n_embd, k, n_tokens, ly.layout, (int)c.f16_ieee, 1};
    n += ((h->use_tma && down_tma_eligible(d)) ? launch_down_tma(st, d, h->d_status) : launch_down(st, d));
    return check_launch(h, what, n);
}

int dsmoe_moe_forward(dsmoe_handle *h, dsmoe_stream stream, uint32_t layer, const float *x, const float *logits,
                      uint32_t n_tokens, float *out, int32_t *selected_out, float *weights_out)
{
    DSMOE_ENTER(h);
    const dsmoe_config &c = h->cfg;
    const uint32_t L = c.max_layers ? c.max_layers : 1;
    if (layer >= L || !h->layers[layer].set) return fail(h, DSMOE_ERR_STATE, "moe_forward: layer %u not registered", layer);
    if (n_tokens > c.max_tokens)
        return fail(h, DSMOE_ERR_BOUNDS, "moe_forward: n_tokens %u exceeds max_tokens %u", n_tokens, c.max_tokens);
    if (n_tokens == 0) return DSMOE_OK;
    DSMOE_REQUIRE(h, x && logits && out, "moe_forward: null pointer");
    DSMOE_REQUIRE(h, aligned(x, 16), "moe_forward: x must be 16-byte aligned");
    const dsmoe_layer_slot &ly = h->layers[layer];
    cudaStream_t st = (cudaStream_t)stream;
    const uint32_t k = c.n_expert_used;
    int32_t *sel = selected_out ? selected_out : h->selected;
    float *wts = weights_out ? weights_out : h->weights;

    int n = 0;
    if (c.n_expert <= 256) {
        launch_router_q8k_fused(st, logits, x, h->probs, sel, wts, h->xq, n_tokens, (int)k, (int)c.n_expert, c.n_embd,
                                c.route_scale);
        n = 1;
    } else {
        launch_router_select(st, logits, nullptr, nullptr, nullptr, h->probs, sel, wts, 0, 0, n_tokens, 0, 0, (int)k,
                             (int)c.n_expert, c.route_scale);
        launch_q8k_quantize(st, x, h->xq, c.n_embd, n_tokens);
        n = 2;
    }
    return expert_ffn_impl(h, st, ly, h->xq, sel, wts, n_tokens, out, n, "moe_forward");
}

int dsmoe_expert_ffn(dsmoe_handle *h, dsmoe_stream stream, uint32_t layer, const uint8_t *xq, const int32_t *selected,
                     const float *weights, uint32_t n_tokens, float *out)
{
    DSMOE_ENTER(h);
    const dsmoe_config &c = h->cfg;
    const uint32_t L = c.max_layers ? c.max_layers : 1;
    if (layer >= L || !h->layers[layer].set) return fail(h, DSMOE_ERR_STATE, "expert_ffn: layer %u not registered", layer);
    if (n_tokens > c.max_tokens)
        return fail(h, DSMOE_ERR_BOUNDS, "expert_ffn: n_tokens %u exceeds max_tokens %u", n_tokens, c.max_tokens);
    if (n_tokens == 0) return DSMOE_OK;
    DSMOE_REQUIRE(h, xq && selected && weights && out, "expert_ffn: null pointer");
    DSMOE_REQUIRE(h, aligned(xq, 16), "expert_ffn: xq must be 16-byte aligned");
    return expert_ffn_impl(h, (cudaStream_t)stream, h->layers[layer], xq, selected, weights, n_tokens, out, 0, "expert_ffn");
}

int dsmoe_host_synchronize(dsmoe_handle *h)
{
    DSMOE_ENTER(h);
    const cudaError_t e = cudaStreamSynchronize(h->hstream);
    if (e != cudaSuccess) return fail(h, DSMOE_ERR_CUDA, "host_synchronize: %s", cudaGetErrorString(e));
    return DSMOE_OK;
}

int dsmoe_moe_forward_host(dsmoe_handle *h, uint32_t layer, const float *x_host, const float *logits_host,
                           uint32_t n_tokens, float *out_host, int32_t *selected_out_host, float *weights_out_host)
{
    const int rc = dsmoe_moe_forward_host_async(h, layer, x_host, logits_host, n_tokens, out_host, selected_out_host,
                                                weights_out_host);
    return rc != DSMOE_OK ? rc : dsmoe_host_synchronize(h);
}

int dsmoe_moe_forward_host_async(dsmoe_handle *h, uint32_t layer, const float *x_host, const float *logits_host,
                                 uint32_t n_tokens, float *out_host, int32_t *selected_out_host, float *weights_out_host)
{
    DSMOE_ENTER(h);
    const dsmoe_config &c = h->cfg;
    if (n_tokens > c.max_tokens)
        return fail(h, DSMOE_ERR_BOUNDS, "moe_forward_host: n_tokens %u exceeds max_tokens %u", n_tokens, c.max_tokens);
    if (n_tokens == 0) return DSMOE_OK;
    DSMOE_REQUIRE(h, x_host && logits_host && out_host, "moe_forward_host: null pointer");
    cudaStream_t st = h->hstream;
    const size_t k = c.n_expert_used;
    cudaError_t e = cudaMemcpyAsync(h->d_x, x_host, (size_t)n_tokens * c.n_embd * 4, cudaMemcpyHostToDevice, st);
    if (e == cudaSuccess)
        e = cudaMemcpyAsync(h->d_logits, logits_host, (size_t)n_tokens * c.n_expert * 4, cudaMemcpyHostToDevice, st);
    if (e != cudaSuccess) return fail(h, DSMOE_ERR_CUDA, "moe_forward_host: copy in: %s", cudaGetErrorString(e));
    int rc = dsmoe_moe_forward(h, st, layer, h->d_x, h->d_logits, n_tokens, h->d_out, h->selected, h->weights);
    if (rc != DSMOE_OK) return rc;
    e = cudaMemcpyAsync(out_host, h->d_out, (size_t)n_tokens * c.n_embd * 4, cudaMemcpyDeviceToHost, st);
    if (e == cudaSuccess && selected_out_host)
        e = cudaMemcpyAsync(selected_out_host, h->selected, n_tokens * k * 4, cudaMemcpyDeviceToHost, st);
    if (e == cudaSuccess && weights_out_host)
        e = cudaMemcpyAsync(weights_out_host, h->weights, n_tokens * k * 4, cudaMemcpyDeviceToHost, st);
    if (e != cudaSuccess) return fail(h, DSMOE_ERR_CUDA, "moe_forward_host: copy out: %s", cudaGetErrorString(e));
    return DSMOE_OK;
}

}  // extern "C"
