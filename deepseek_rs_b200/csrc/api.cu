// The C ABI of libdsmoe: handle, argument checks, tier-1 launch wrappers and the tier-2 layer call.
#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <new>

#include "async.cuh"
#include "common.cuh"
#include "ep.h"
#include "launch.h"

using namespace dsmoe;

struct dsmoe_layer_slot {
    const uint8_t *gate, *up, *down;
    int layout;
    bool set;
    // the tensors beside the routed experts (dsmoe_layer_register_extras); any of them may be null
    const uint16_t *router_f16;
    const float *router_bias;
    const int32_t *hash_table;
    uint32_t hash_rows;
    const uint8_t *sh_gate, *sh_up, *sh_down;
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
    int32_t *pair_order;  // pairs sorted by expert for the decode gate/up kernel at 16 tokens and more
    uint32_t *blk_rows;   // rows stored so far per 256-row block of mid (decode gate/up kernel); zero between calls
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
    // dsmoe_ffn_forward: logits computed here, shared-expert output when the caller does not want it, widened bf16 input;
    // the shared expert runs on a side stream between two events
    float *ffn_logits, *ffn_shared, *ffn_x32;
    cudaStream_t sstream;
    cudaEvent_t ev_fork, ev_join;
    // expert-parallel state (dsmoe_ep_init), or null
    EpState *ep;
    cudaEvent_t ep_events[6];
    bool ep_events_set;
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

const char *dsmoe_version(void)
{
#ifdef DSMOE_BOUNDS
    return "dsmoe 0.2 (sm_100a, checked build)";
#else
    return "dsmoe 0.2 (sm_100a)";
#endif
}

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
    ok = ok && dev_alloc(&h->pair_order, T * k) == cudaSuccess;
    ok = ok && dev_alloc(&h->blk_rows, T * k * (cfg->n_ff / QK_K) + 1) == cudaSuccess &&
         cudaMemset(h->blk_rows, 0, (T * k * (cfg->n_ff / QK_K) + 1) * sizeof(uint32_t)) == cudaSuccess;
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
    ok = ok && dev_alloc(&h->ffn_logits, T * cfg->n_expert) == cudaSuccess;
    ok = ok && dev_alloc(&h->ffn_shared, T * cfg->n_embd) == cudaSuccess;
    ok = ok && dev_alloc(&h->ffn_x32, T * cfg->n_embd) == cudaSuccess;
    ok = ok && cudaStreamCreateWithFlags(&h->sstream, cudaStreamNonBlocking) == cudaSuccess;
    ok = ok && cudaEventCreateWithFlags(&h->ev_fork, cudaEventDisableTiming) == cudaSuccess;
    ok = ok && cudaEventCreateWithFlags(&h->ev_join, cudaEventDisableTiming) == cudaSuccess;
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
    if (h->ep) ep_destroy(h->ep);
    if (h->hstream) cudaStreamDestroy(h->hstream);
    if (h->sstream) cudaStreamDestroy(h->sstream);
    if (h->ev_fork) cudaEventDestroy(h->ev_fork);
    if (h->ev_join) cudaEventDestroy(h->ev_join);
    cudaFree(h->ffn_logits);
    cudaFree(h->ffn_shared);
    cudaFree(h->ffn_x32);
    cudaFree(h->probs);
    cudaFree(h->weights);
    cudaFree(h->selected);
    cudaFree(h->pair_order);
    cudaFree(h->blk_rows);
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
    if (*code_out == DEV_ERR_INDEX_RANGE)
        return fail(h, DSMOE_ERR_BOUNDS, "an expert index outside the layer was replaced by 0 (checked build, code %d)", *code_out);
    if (*code_out != 0) {
        // a kernel that gave up may have left the row counters of its unfinished blocks behind
        if (h->blk_rows)
            cudaMemsetAsync(h->blk_rows, 0, ((size_t)h->cfg.max_tokens * h->cfg.n_expert_used * (h->cfg.n_ff / QK_K) + 1) * sizeof(uint32_t),
                            (cudaStream_t)stream);
        return fail(h, DSMOE_ERR_TIMEOUT, "a bounded device-side wait expired (code %d)", *code_out);
    }
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
    const bool tma = h->use_tma && gate_up_tma_eligible(a);
    int n = 0;
    // the same pair sorting as in the whole-layer call, when the handle's buffer holds this many pairs
    if (tma && n_tokens >= 16 && (uint64_t)n_tokens * n_expert_used <= (uint64_t)h->cfg.max_tokens * h->cfg.n_expert_used &&
        launch_pair_order((cudaStream_t)stream, selected, n_tokens * n_expert_used, h->cfg.n_expert, h->pair_order)) {
        a.order = h->pair_order;
        n += 1;
    }
    n += tma ? launch_gate_up_mid_tma((cudaStream_t)stream, a, h->d_status) : launch_gate_up_mid((cudaStream_t)stream, a);
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

static int shared_expert_impl(dsmoe_handle *h, cudaStream_t st, const uint8_t *gate_w, const uint8_t *up_w,
                              const uint8_t *down_w, const float *x, uint32_t n_tokens, float *out);

int dsmoe_shared_expert(dsmoe_handle *h, dsmoe_stream stream, const uint8_t *gate_w, const uint8_t *up_w,
                        const uint8_t *down_w, const float *x, uint32_t n_tokens, float *out)
{
    DSMOE_ENTER(h);
    if (n_tokens == 0) return DSMOE_OK;
    DSMOE_REQUIRE(h, gate_w && up_w && down_w && x && out, "shared_expert: null pointer");
    DSMOE_REQUIRE(h, (((uintptr_t)gate_w | (uintptr_t)up_w | (uintptr_t)down_w) & 3) == 0, "shared_expert: weights need 4-byte alignment");
    return shared_expert_impl(h, (cudaStream_t)stream, gate_w, up_w, down_w, x, n_tokens, out);
}

static int shared_expert_impl(dsmoe_handle *h, cudaStream_t st, const uint8_t *gate_w, const uint8_t *up_w,
                              const uint8_t *down_w, const float *x, uint32_t n_tokens, float *out)
{
    const dsmoe_config &c = h->cfg;
    int n = 0;
    // up to four tokens every CTA quantises the activations itself (two launches); above that, when the tensors can be
    // staged by bulk copies, quantising once and working through tiles of eight tokens is cheaper (four launches)
    const bool tiles = shared_tiles_eligible(gate_w, up_w, down_w, h->sh_xq, h->sh_xscale, c.n_embd, c.n_ff);
    if (n_tokens <= (tiles ? 4u : 8u) && shared_fused_eligible(c.n_embd, c.n_ff, n_tokens) && n_tokens <= h->sh_chunk) {
        n = launch_shared_fused(st, gate_w, up_w, down_w, x, h->sh_mid, out, c.n_embd, c.n_ff, n_tokens, c.swiglu_clamp,
                                h->d_status);
        return check_launch(h, "shared_expert", n);
    }
    for (uint32_t t0 = 0; t0 < n_tokens; t0 += h->sh_chunk) {
        const uint32_t T = n_tokens - t0 < h->sh_chunk ? n_tokens - t0 : h->sh_chunk;
        const float *xc = x + (size_t)t0 * c.n_embd;
        if (tiles) {
            n += launch_shared_tiles(st, gate_w, up_w, down_w, xc, h->sh_xq, h->sh_xscale, h->sh_mid, out + (size_t)t0 * c.n_embd,
                                     c.n_embd, c.n_ff, T, c.swiglu_clamp, h->d_status);
            continue;
        }
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
    dsmoe_layer_slot &ly = h->layers[layer];
    ly.gate = gate, ly.up = up, ly.down = down, ly.layout = layout, ly.set = true;
    return DSMOE_OK;
}

int dsmoe_layer_register_extras(dsmoe_handle *h, uint32_t layer, const uint16_t *router_f16, const float *router_bias,
                                const int32_t *hash_table, uint32_t hash_rows, const uint8_t *shared_gate,
                                const uint8_t *shared_up, const uint8_t *shared_down)
{
    DSMOE_ENTER(h);
    const uint32_t L = h->cfg.max_layers ? h->cfg.max_layers : 1;
    DSMOE_REQUIRE(h, layer < L, "layer_register_extras: layer %u beyond max_layers %u", layer, L);
    DSMOE_REQUIRE(h, (hash_table == nullptr) == (hash_rows == 0), "layer_register_extras: hash table and hash_rows must come together");
    const bool any_sh = shared_gate || shared_up || shared_down, all_sh = shared_gate && shared_up && shared_down;
    DSMOE_REQUIRE(h, any_sh == all_sh, "layer_register_extras: the shared expert needs all three tensors");
    DSMOE_REQUIRE(h, (((uintptr_t)shared_gate | (uintptr_t)shared_up | (uintptr_t)shared_down) & 3) == 0 && aligned(router_f16, 2),
                  "layer_register_extras: shared-expert tensors need 4-byte, the router 2-byte alignment");
    dsmoe_layer_slot &ly = h->layers[layer];
    ly.router_f16 = router_f16, ly.router_bias = router_bias, ly.hash_table = hash_table, ly.hash_rows = hash_rows;
    ly.sh_gate = shared_gate, ly.sh_up = shared_up, ly.sh_down = shared_down;
    return DSMOE_OK;
}

// Everything after the router and the Q8_K of x: gate/up/SwiGLU -> Q8_K(mid) -> down -> slot sum, on the decode
// kernels or, from prefill_min_tokens rows upwards, on the grouped GEMM.
static int expert_ffn_impl(dsmoe_handle *h, cudaStream_t st, const dsmoe_layer_slot &ly, const uint8_t *xq,
                           const int32_t *sel, const float *wts, uint32_t n_tokens, float *out, int n, const char *what,
                           const HcEpilogue *hc = nullptr, cudaEvent_t before_sum = nullptr, float *const *row_ptr = nullptr)
{
    const dsmoe_config &c = h->cfg;
    const uint32_t k = c.n_expert_used, xb = c.n_embd / QK_K, mb = c.n_ff / QK_K;
#ifdef DSMOE_BOUNDS
    // checked build: the kernels only ever see indices inside the layer (a copy in the handle's own selection buffer)
    launch_sanitize_indices(st, sel, h->selected, (uint64_t)n_tokens * k, (int32_t)c.n_expert, h->d_status);
    sel = h->selected;
    n += 1;
#endif
    if (n_tokens >= h->prefill_min_tokens && prefill_eligible(c.n_embd, c.n_ff, ly.gate, ly.up, ly.down, ly.layout)) {
        PrefillArgs p = {ly.gate, ly.up, ly.down, xq, sel, wts, h->mid, h->midq, out, h->pf_scratch, h->pf_lay,
                         n_tokens, k, c.n_expert, c.n_embd, c.n_ff, c.swiglu_clamp, ly.layout, (int)c.f16_ieee,
                         h->d_status, h->phase_events_set ? h->phase_events : nullptr, hc, before_sum, row_ptr};
        n += launch_prefill_experts(st, p);
        return check_launch(h, what, n);
    }
    if ((uint64_t)n_tokens * k > 65535u) return fail(h, DSMOE_ERR_BOUNDS, "%s: n_tokens*k exceeds 65535 on the decode kernels", what);
    GateUpArgs g = {ly.gate, ly.up, xq, sel, wts, nullptr, nullptr, h->mid, (uint64_t)c.n_ff * xb * IQ2XXS_BYTES,
                    (uint64_t)xb * IQ2XXS_BYTES, xb, c.n_ff, k, n_tokens, c.swiglu_clamp, ly.layout, (int)c.f16_ieee};
    const bool gu_tma = h->use_tma && gate_up_tma_eligible(g);
    // from 16 tokens on, experts repeat among the pairs often enough to pay for sorting them (one small launch)
    if (gu_tma && n_tokens >= 16 && launch_pair_order(st, sel, n_tokens * k, c.n_expert, h->pair_order)) {
        g.order = h->pair_order;
        n += 1;
    }
    // the TMA kernel quantises mid itself (a block as soon as its last row is stored): one launch less
    const bool fused_q8k = gu_tma && c.n_ff % QK_K == 0;
    if (fused_q8k) g.midq_out = h->midq, g.blk_rows = h->blk_rows;
    n += gu_tma ? launch_gate_up_mid_tma(st, g, h->d_status) : launch_gate_up_mid(st, g);
    if (int rc = check_launch(h, what, n)) return rc;
    n = 0;
    if (!fused_q8k) {
        launch_q8k_quantize(st, h->mid, h->midq, c.n_ff, n_tokens * k);
        if (int rc = check_launch(h, what, 1)) return rc;
    }
    DownArgs d = {ly.down, h->midq, sel, out, (uint64_t)c.n_embd * mb * Q2K_BYTES, (uint64_t)mb * Q2K_BYTES, mb,
                  c.n_embd, k, n_tokens, ly.layout, (int)c.f16_ieee, 1};
    n += ((h->use_tma && down_tma_eligible(d)) ? launch_down_tma(st, d, h->d_status) : launch_down(st, d));
    if (before_sum) cudaStreamWaitEvent(st, before_sum, 0);
    if (hc && hc->out_hc) {
        launch_hc_expand(st, out, c.n_embd, n_tokens, *hc);
        n += 1;
    }
    if (row_ptr) {  // the decode kernels wrote `out`; the rows go to their destinations with a copy kernel
        launch_scatter_rows(st, out, row_ptr, c.n_embd, n_tokens);
        n += 1;
    }
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

int dsmoe_hc_expand(dsmoe_handle *h, dsmoe_stream stream, const float *block_out, const float *block_add,
                    const float *residual_hc, const float *split, float *out_hc, uint32_t n_embd, uint32_t n_hc,
                    uint32_t n_tokens, uint32_t mix_hc, uint32_t has_add)
{
    DSMOE_ENTER(h);
    if (n_tokens == 0 || n_embd == 0 || n_hc == 0) return DSMOE_OK;
    DSMOE_REQUIRE(h, block_out && residual_hc && split && out_hc && (!has_add || block_add), "hc_expand: null pointer");
    DSMOE_REQUIRE(h, mix_hc >= 2 * n_hc + n_hc * n_hc, "hc_expand: mix_hc %u shorter than pre + post + comb of n_hc %u", mix_hc, n_hc);
    const HcEpilogue hc = {block_out, residual_hc, split, out_hc, n_hc, mix_hc};
    launch_hc_expand((cudaStream_t)stream, has_add ? block_add : nullptr, n_embd, n_tokens, hc);
    return check_launch(h, "hc_expand", 1);
}

int dsmoe_hc_split_weighted_sum_norm(dsmoe_handle *h, dsmoe_stream stream, const float *mix, const float *scale,
                                     const float *base, const float *residual_hc, const float *norm_w, float *split,
                                     float *out, float *norm_out, uint32_t n_embd, uint32_t n_hc, uint32_t n_rows,
                                     uint32_t sinkhorn_iters, float epsv, float norm_eps)
{
    DSMOE_ENTER(h);
    if (n_rows == 0 || n_embd == 0) return DSMOE_OK;
    DSMOE_REQUIRE(h, n_hc == 4, "hc_split_weighted_sum_norm: n_hc must be 4 (the reference kernel returns early otherwise)");
    DSMOE_REQUIRE(h, mix && scale && base && residual_hc && norm_w && split && out && norm_out, "hc_split_weighted_sum_norm: null pointer");
    launch_hc_split_weighted_sum_norm((cudaStream_t)stream, mix, scale, base, residual_hc, norm_w, split, out, norm_out,
                                      n_embd, n_rows, sinkhorn_iters, epsv, norm_eps);
    return check_launch(h, "hc_split_weighted_sum_norm", 1);
}

int dsmoe_ffn_forward(dsmoe_handle *h, dsmoe_stream stream, uint32_t layer, const dsmoe_ffn_args *a)
{
    DSMOE_ENTER(h);
    DSMOE_REQUIRE(h, a != nullptr, "ffn_forward: null arguments");
    const dsmoe_config &c = h->cfg;
    const uint32_t L = c.max_layers ? c.max_layers : 1;
    if (layer >= L || !h->layers[layer].set) return fail(h, DSMOE_ERR_STATE, "ffn_forward: layer %u not registered", layer);
    const dsmoe_layer_slot &ly = h->layers[layer];
    const uint32_t T = a->n_tokens, k = c.n_expert_used;
    if (T > c.max_tokens) return fail(h, DSMOE_ERR_BOUNDS, "ffn_forward: n_tokens %u exceeds max_tokens %u", T, c.max_tokens);
    if (T == 0) return DSMOE_OK;
    DSMOE_REQUIRE(h, a->x && a->routed_out, "ffn_forward: x and routed_out are required");
    DSMOE_REQUIRE(h, a->x_dtype == DSMOE_DTYPE_F32 || a->x_dtype == DSMOE_DTYPE_BF16, "ffn_forward: unknown x_dtype %d", a->x_dtype);
    DSMOE_REQUIRE(h, a->logits || ly.router_f16, "ffn_forward: no logits given and no router matrix registered");
    DSMOE_REQUIRE(h, !a->hash_mode || ly.hash_table, "ffn_forward: hash_mode set but the layer has no hash table");
    const bool want_shared = a->shared_out != nullptr || a->out_hc != nullptr;
    DSMOE_REQUIRE(h, !want_shared || ly.sh_gate, "ffn_forward: shared-expert output wanted but no shared expert registered");
    DSMOE_REQUIRE(h, !a->out_hc || (a->residual_hc && a->hc_split && a->n_hc > 0 && a->mix_hc >= 2 * a->n_hc + a->n_hc * a->n_hc),
                  "ffn_forward: the hyper-connection merge needs residual_hc, hc_split, n_hc and mix_hc >= 2 n_hc + n_hc^2");
    cudaStream_t st = (cudaStream_t)stream;
    int n = 0;

    // hidden states: f32 as the reference keeps them, or bf16 widened exactly
    const float *x = static_cast<const float *>(a->x);
    if (a->x_dtype == DSMOE_DTYPE_BF16) {
        DSMOE_REQUIRE(h, aligned(a->x, 2), "ffn_forward: bf16 x must be 2-byte aligned");
        launch_bf16_to_f32(st, static_cast<const uint16_t *>(a->x), h->ffn_x32, (uint64_t)T * c.n_embd);
        x = h->ffn_x32;
        n += 1;
    } else {
        DSMOE_REQUIRE(h, aligned(a->x, 16), "ffn_forward: x must be 16-byte aligned");
    }

    // shared expert on the side stream (engine/src/session.rs:1894-1987), concurrent with the routed path
    float *shared = a->shared_out ? a->shared_out : h->ffn_shared;
    if (want_shared) {
        if (cudaEventRecord(h->ev_fork, st) != cudaSuccess || cudaStreamWaitEvent(h->sstream, h->ev_fork, 0) != cudaSuccess)
            return fail(h, DSMOE_ERR_CUDA, "ffn_forward: fork: %s", cudaGetErrorString(cudaGetLastError()));
        if (int rc = shared_expert_impl(h, h->sstream, ly.sh_gate, ly.sh_up, ly.sh_down, x, T, shared)) return rc;
        if (cudaEventRecord(h->ev_join, h->sstream) != cudaSuccess)
            return fail(h, DSMOE_ERR_CUDA, "ffn_forward: join: %s", cudaGetErrorString(cudaGetLastError()));
    }

    // router logits (engine/src/session.rs:1995-2008) unless the caller brings them
    const float *logits = a->logits;
    if (!logits) {
        DSMOE_REQUIRE(h, T <= 65535u, "ffn_forward: at most 65535 tokens per call when the logits are computed here");
        launch_matmul_f16(st, ly.router_f16, x, h->ffn_logits, c.n_embd, c.n_expert, T);
        logits = h->ffn_logits;
        n += 1;
    }
    int32_t *sel = a->selected_out ? a->selected_out : h->selected;
    float *wts = a->weights_out ? a->weights_out : h->weights;
    const bool plain_router = !ly.router_bias && !a->hash_mode && c.n_expert <= 256;
    if (plain_router) {
        launch_router_q8k_fused(st, logits, x, h->probs, sel, wts, h->xq, T, (int)k, (int)c.n_expert, c.n_embd, c.route_scale);
        n += 1;
    } else {  // bias and / or hash routing (engine/src/kernels/moe.rs:211-228)
        launch_router_select(st, logits, ly.router_bias, a->hash_mode ? ly.hash_table : nullptr, a->tokens, h->probs, sel, wts,
                             a->token_scalar, a->hash_mode ? ly.hash_rows : 0, T, ly.router_bias != nullptr, a->hash_mode != 0,
                             (int)k, (int)c.n_expert, c.route_scale);
        launch_q8k_quantize(st, x, h->xq, c.n_embd, T);
        n += 2;
    }
    HcEpilogue hc = {shared, a->residual_hc, a->hc_split, a->out_hc, a->n_hc, a->mix_hc};
    const int rc = expert_ffn_impl(h, st, ly, h->xq, sel, wts, T, a->routed_out, n, "ffn_forward", a->out_hc ? &hc : nullptr,
                                   want_shared ? h->ev_join : nullptr);
    return rc;
}

// ---------------------------------------------------------------------------------------------------------------
// expert parallel
// ---------------------------------------------------------------------------------------------------------------

int dsmoe_ep_get_unique_id(uint8_t *id128)
{
    if (!id128) return DSMOE_ERR_ARG;
    return ep_get_unique_id(id128);
}

static int ep_init_common(dsmoe_handle *h, const uint8_t *id128, void *comm, int rank, int world, uint32_t max_replicas,
                          uint32_t recv_capacity_rows)
{
    DSMOE_ENTER(h);
    if (h->ep) return fail(h, DSMOE_ERR_STATE, "ep_init: already initialised");
    DSMOE_REQUIRE(h, id128 || comm, "ep_init: neither a unique id nor a communicator");
    char msg[384] = {0};
    const int rc = ep_create(h->cfg, h->device, id128, comm, rank, world, max_replicas, recv_capacity_rows, &h->ep, msg, sizeof(msg));
    if (rc != DSMOE_OK) return fail(h, rc, "%s", msg);
    return DSMOE_OK;
}

int dsmoe_ep_init(dsmoe_handle *h, const uint8_t *id128, int rank, int world, uint32_t max_replicas,
                  uint32_t recv_capacity_rows)
{
    return ep_init_common(h, id128, nullptr, rank, world, max_replicas, recv_capacity_rows);
}

int dsmoe_ep_init_comm(dsmoe_handle *h, void *nccl_comm, int rank, int world, uint32_t max_replicas,
                       uint32_t recv_capacity_rows)
{
    return ep_init_common(h, nullptr, nccl_comm, rank, world, max_replicas, recv_capacity_rows);
}

#define DSMOE_NEED_EP(h, what) \
    do {                       \
        if (!(h)->ep) return fail((h), DSMOE_ERR_STATE, "%s: dsmoe_ep_init has not run on this handle", what); \
    } while (0)

int dsmoe_ep_layer_register(dsmoe_handle *h, uint32_t layer, const uint8_t *gate, const uint8_t *up, const uint8_t *down,
                            int layout)
{
    DSMOE_ENTER(h);
    DSMOE_NEED_EP(h, "ep_layer_register");
    dsmoe_handle *o = ep_owner(h->ep);
    const int rc = dsmoe_layer_register(o, layer, gate, up, down, layout);
    if (rc != DSMOE_OK) return fail(h, rc, "ep_layer_register: %s", dsmoe_last_error(o));
    return DSMOE_OK;
}

int dsmoe_ep_set_replicas(dsmoe_handle *h, const int32_t *expert_ids, uint32_t n)
{
    DSMOE_ENTER(h);
    DSMOE_NEED_EP(h, "ep_set_replicas");
    DSMOE_REQUIRE(h, n == 0 || expert_ids, "ep_set_replicas: null list");
    const int rc = ep_set_replicas(h->ep, h->cfg.n_expert, expert_ids, n);
    if (rc != DSMOE_OK) return fail(h, rc, "%s", ep_last_error(h->ep));
    return DSMOE_OK;
}

int dsmoe_ep_expert_counts(dsmoe_handle *h, dsmoe_stream stream, uint64_t *counts_host, int reset)
{
    DSMOE_ENTER(h);
    DSMOE_NEED_EP(h, "ep_expert_counts");
    DSMOE_REQUIRE(h, counts_host, "ep_expert_counts: null pointer");
    const int rc = ep_expert_counts(h->ep, (cudaStream_t)stream, h->cfg.n_expert, counts_host, reset);
    if (rc != DSMOE_OK) return fail(h, rc, "%s", ep_last_error(h->ep));
    return DSMOE_OK;
}

int dsmoe_ep_last_recv_rows(dsmoe_handle *h, int32_t *rows_per_rank)
{
    DSMOE_ENTER(h);
    DSMOE_NEED_EP(h, "ep_last_recv_rows");
    DSMOE_REQUIRE(h, rows_per_rank, "ep_last_recv_rows: null pointer");
    return ep_last_recv_rows(h->ep, rows_per_rank);
}

int dsmoe_ep_combine_is_fused(dsmoe_handle *h)
{
    if (!h || !h->ep) return 0;
    return ep_p2p_combine(h->ep);
}

int dsmoe_ep_set_phase_events(dsmoe_handle *h, void **events, int n_events)
{
    DSMOE_ENTER(h);
    if (!events || n_events == 0) {
        h->ep_events_set = false;
        return DSMOE_OK;
    }
    if (n_events != 6) return fail(h, DSMOE_ERR_ARG, "ep_set_phase_events: expected 6 events, got %d", n_events);
    for (int i = 0; i < 6; ++i) h->ep_events[i] = (cudaEvent_t)events[i];
    h->ep_events_set = true;
    return DSMOE_OK;
}

int dsmoe_moe_forward_ep(dsmoe_handle *h, dsmoe_stream stream, uint32_t layer, const float *x, const float *logits,
                         uint32_t n_tokens, float *out, int32_t *selected_out, float *weights_out)
{
    DSMOE_ENTER(h);
    DSMOE_NEED_EP(h, "moe_forward_ep");
    const dsmoe_config &c = h->cfg;
    if (n_tokens > c.max_tokens)
        return fail(h, DSMOE_ERR_BOUNDS, "moe_forward_ep: n_tokens %u exceeds max_tokens %u", n_tokens, c.max_tokens);
    DSMOE_REQUIRE(h, n_tokens == 0 || (x && logits && out), "moe_forward_ep: null pointer");
    DSMOE_REQUIRE(h, aligned(x, 16), "moe_forward_ep: x must be 16-byte aligned");
    DSMOE_REQUIRE(h, c.n_expert <= 256, "moe_forward_ep: at most 256 experts");
    cudaStream_t st = (cudaStream_t)stream;
    int32_t *sel = selected_out ? selected_out : h->selected;
    float *wts = weights_out ? weights_out : h->weights;
    int n = 0;
    if (n_tokens) {  // the same router kernel on the same logits as the single-GPU call: routing is bit-identical
        launch_router_q8k_fused(st, logits, x, h->probs, sel, wts, h->xq, n_tokens, (int)c.n_expert_used, (int)c.n_expert,
                                c.n_embd, c.route_scale);
        n = 1;
    }
    // a rank without tokens still takes part in the exchanges
    const int rc = ep_forward(h->ep, st, layer, h->xq, sel, wts, n_tokens, c.n_expert_used, c.n_embd, out, &n,
                              h->ep_events_set ? h->ep_events : nullptr);
    if (rc != DSMOE_OK) return fail(h, rc, "%s", ep_last_error(h->ep));
    return check_launch(h, "moe_forward_ep", n);
}

// Internal (expert parallel): dsmoe_expert_ffn for a k = 1 handle whose result rows go to row_ptr[i] instead of a local
// array; `out` ([n_tokens][n_embd]) is scratch for the case that the decode kernels run. Not part of the C ABI.
int dsmoe_expert_ffn_rows(dsmoe_handle *h, cudaStream_t st, uint32_t layer, const uint8_t *xq, const int32_t *selected,
                          const float *weights, uint32_t n_tokens, float *out, float *const *row_ptr)
{
    DSMOE_ENTER(h);
    const dsmoe_config &c = h->cfg;
    const uint32_t L = c.max_layers ? c.max_layers : 1;
    if (layer >= L || !h->layers[layer].set) return fail(h, DSMOE_ERR_STATE, "expert_ffn: layer %u not registered", layer);
    if (n_tokens > c.max_tokens) return fail(h, DSMOE_ERR_BOUNDS, "expert_ffn: n_tokens %u exceeds max_tokens %u", n_tokens, c.max_tokens);
    if (c.n_expert_used != 1) return fail(h, DSMOE_ERR_STATE, "expert_ffn_rows: needs a handle with n_expert_used = 1");
    if (n_tokens == 0) return DSMOE_OK;
    return expert_ffn_impl(h, st, h->layers[layer], xq, selected, weights, n_tokens, out, 0, "expert_ffn", nullptr, nullptr, row_ptr);
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
