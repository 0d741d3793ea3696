// Host-side launchers shared between the kernel files and the C ABI. Each launches on the given stream and returns
// without synchronising; the caller checks cudaGetLastError().
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

namespace dsmoe {

// Per-device host state. Function attributes (the dynamic shared-memory limit of a kernel) and device properties
// belong to one device, while a process may create handles on several: everything cached on the host is therefore
// kept per device ordinal, looked up from the CURRENT device at the time of the launch.
constexpr int MAX_DEVICES = 64;
inline int current_device_slot()
{
    int d = 0;
    if (cudaGetDevice(&d) != cudaSuccess || d < 0 || d >= MAX_DEVICES) d = 0;
    return d;
}
// True the first time it is asked on each device.
struct OncePerDevice {
    bool done[MAX_DEVICES] = {};
    bool first()
    {
        const int d = current_device_slot();
        if (done[d]) return false;
        done[d] = true;
        return true;
    }
};
// Multiprocessor count of the current device (cached per device).
inline int sm_count_current()
{
    static int n[MAX_DEVICES] = {};
    const int d = current_device_slot();
    if (n[d] == 0) {
        cudaDeviceGetAttribute(&n[d], cudaDevAttrMultiProcessorCount, d);
        if (n[d] <= 0) n[d] = 148;
    }
    return n[d];
}

// Launch with the programmatic-serialisation attribute (see pdl_wait() in async.cuh): the kernel may be scheduled
// while its predecessor in the stream drains, and must call pdl_wait() before touching that kernel's data.
template <typename... KArgs, typename... Args>
inline cudaError_t launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st, Args... args)
{
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

void launch_q8k_quantize(cudaStream_t st, const float *x, uint8_t *out, uint32_t in_dim, uint32_t n_rows);
// mid = swiglu(clamped gate, clamped up) * weight[row] (engine/src/kernels/moe.rs:692-710) quantised to Q8_K on the fly
// (quantize.rs:309-417): gate / up f32 [n_rows][in_dim], weight f32 [n_rows], out Q8_K [n_rows][in_dim / 256].
void launch_swiglu_q8k(cudaStream_t st, const float *gate, const float *up, const float *weight, uint8_t *out,
                       uint32_t in_dim, uint32_t n_rows, float clamp);

void launch_router_select(cudaStream_t st, const float *logits, const float *bias, const int32_t *hash,
                          const int32_t *tokens, float *probs, int32_t *selected, float *weights, int32_t token_scalar,
                          uint32_t hash_rows, uint32_t n_tokens, int has_bias, int hash_mode, int k, int n_expert,
                          float route_scale);

// Router (no bias / hash) and Q8_K of x in one launch; n_expert <= 256.
void launch_router_q8k_fused(cudaStream_t st, const float *logits, const float *x, float *probs, int32_t *selected,
                             float *weights, uint8_t *xq, uint32_t n_tokens, int k, int n_expert, uint32_t n_embd,
                             float route_scale);

void launch_dequant_iq2xxs(cudaStream_t st, const uint8_t *blocks, uint64_t n_blocks, float *out, int ieee);
void launch_dequant_q2k(cudaStream_t st, const uint8_t *blocks, uint64_t n_blocks, float *out, int ieee);
void launch_relayout_iq2xxs(cudaStream_t st, const uint8_t *src, uint8_t *dst, uint64_t n_rows, uint32_t xb, int inverse);
void launch_relayout_q2k(cudaStream_t st, const uint8_t *src, uint8_t *dst, uint64_t n_rows, uint32_t mb, int inverse);
// Operands of the hyper-connection merge that follows the routed experts in the reference (hc_expand,
// engine/src/kernels/hc.rs:212-251). out_hc == nullptr: no merge.
struct HcEpilogue {
    const float *shared;     // block_out: the shared expert's output [n_tokens][n_embd]
    const float *residual;   // residual_hc [n_tokens][n_hc][n_embd]
    const float *split;      // [n_tokens][mix_hc]: pre (n_hc), post (n_hc), comb (n_hc * n_hc)
    float *out_hc;           // [n_tokens][n_hc][n_embd]
    uint32_t n_hc, mix_hc;
};
void launch_moe_sum(cudaStream_t st, const float *down, const int32_t *pos, float *out, uint32_t out_dim, uint32_t k,
                    uint32_t n_tokens, const HcEpilogue *hc = nullptr);
void launch_hc_expand(cudaStream_t st, const float *block_add, uint32_t n_embd, uint32_t n_tokens, const HcEpilogue &hc);
void launch_bf16_to_f32(cudaStream_t st, const uint16_t *in, float *out, uint64_t n);
// dst[i][0 .. n_embd) = rows[i][0 .. n_embd) for i < n_rows; the destinations may lie in another GPU's memory.
void launch_scatter_rows(cudaStream_t st, const float *rows, float *const *dst, uint32_t n_embd, uint32_t n_rows);
// dst[i] = src[i] < hi ? src[i] : 0, recording DEV_ERR_INDEX_RANGE in *status on a replacement (checked build).
void launch_sanitize_indices(cudaStream_t st, const int32_t *src, int32_t *dst, uint64_t n, int32_t hi, int *status);
// hc_split_weighted_sum_norm_fused (engine/src/kernels/hc.rs:313-394), n_hc = 4: split [n_rows][24], out and norm_out
// [n_rows][n_embd].
void launch_hc_split_weighted_sum_norm(cudaStream_t st, const float *mix, const float *scale, const float *base,
                                       const float *residual_hc, const float *norm_w, float *split, float *out,
                                       float *norm_out, uint32_t n_embd, uint32_t n_rows, uint32_t iters, float epsv,
                                       float norm_eps);

// Router logits and shared expert (shared.cu)
void launch_quantize_q8_0(cudaStream_t st, const float *x, int8_t *xq, float *xscale, uint64_t in_dim, uint64_t n_tok);
void launch_matmul_q8_0(cudaStream_t st, const uint8_t *w, const int8_t *xq, const float *xscale, float *out,
                        uint64_t in_dim, uint64_t out_dim, uint64_t n_tok);
void launch_swiglu(cudaStream_t st, const float *gate, const float *up, float *out, uint64_t n, float clamp, float weight);
// The shared expert in two launches for up to 4 tokens (mid: f32 [n_tokens][n_ff] scratch). Returns the launch count.
bool shared_fused_eligible(uint32_t n_embd, uint32_t n_ff, uint32_t n_tokens);
int launch_shared_fused(cudaStream_t st, const uint8_t *gate_w, const uint8_t *up_w, const uint8_t *down_w, const float *x,
                        float *mid, float *out, uint32_t n_embd, uint32_t n_ff, uint32_t n_tokens, float clamp,
                        int *status);
// More than eight tokens (any count): quantise, gate + up + SwiGLU, quantise, down, the two matrix kernels with weight
// rows and activation tiles staged in shared memory by bulk copies. Needs what shared_tiles_eligible checks. 4 launches.
bool shared_tiles_eligible(const uint8_t *gate_w, const uint8_t *up_w, const uint8_t *down_w, const int8_t *xq,
                           const float *xs, uint32_t n_embd, uint32_t n_ff);
int launch_shared_tiles(cudaStream_t st, const uint8_t *gate_w, const uint8_t *up_w, const uint8_t *down_w, const float *x,
                        int8_t *xq, float *xs, float *mid, float *out, uint32_t n_embd, uint32_t n_ff, uint32_t n_tokens,
                        float clamp, int *status);
void launch_matmul_f16(cudaStream_t st, const uint16_t *w, const float *x, float *out, uint64_t in_dim, uint64_t out_dim,
                       uint64_t n_tok);

struct GateUpArgs {
    const uint8_t *gate_base, *up_base, *xq;
    const int32_t *selected;
    const float *weights;
    float *gate_out, *up_out, *mid_out;
    uint64_t expert_bytes, row_bytes;
    uint32_t xq_blocks, mid_dim, k, n_tokens;
    float clamp;
    int layout, ieee;
    // TMA kernel only, optional: the pairs sorted by expert (order[position] = pair, from launch_pair_order); pairs of
    // one expert are then streamed together and the second one finds the weights in L2. Results do not depend on it.
    const int32_t *order = nullptr;
    // TMA kernel only, optional: the kernel also writes Q8_K(mid) ([pair][mid_dim / 256] blocks), each block by the warp
    // that stores its last row; blk_rows is one zeroed counter per block, which the kernel leaves zeroed. mid_dim must
    // be a multiple of 256.
    uint8_t *midq_out = nullptr;
    uint32_t *blk_rows = nullptr;
};
// Returns the number of kernels launched.
int launch_gate_up_mid(cudaStream_t st, const GateUpArgs &a);
// order[position] = pair, positions sorted by selected[pair]; 0 launches (and `order` untouched) above 4096 experts.
int launch_pair_order(cudaStream_t st, const int32_t *selected, uint32_t n_pairs, uint32_t n_expert, int32_t *order);

struct DownArgs {
    const uint8_t *down_base, *midq;
    const int32_t *selected;
    float *out;  // [n_tokens*k][out_dim] when sum_slots == 0, [n_tokens][out_dim] otherwise
    uint64_t expert_bytes, row_bytes;
    uint32_t midq_blocks, out_dim, k, n_tokens;
    int layout, ieee, sum_slots;
};
int launch_down(cudaStream_t st, const DownArgs &a);

// Variants that stage the packed rows through shared memory with bulk asynchronous copies (reference shapes only).
// status points at a device int that receives a non-zero code if a bounded wait expires.
bool gate_up_tma_eligible(const GateUpArgs &a);
int launch_gate_up_mid_tma(cudaStream_t st, const GateUpArgs &a, int *status);
bool down_tma_eligible(const DownArgs &a);
int launch_down_tma(cudaStream_t st, const DownArgs &a, int *status);

// Batched path (tcgen05 grouped GEMM). Scratch is one device buffer carved up by prefill_scratch_bytes().
struct PrefillScratch {
    uint32_t r_cap, tile_cap;
    size_t counts, offsets, sorted, tile_expert, tile_start, tile_rows, tile_boff, plan, bx, sx, bm, sm, bs, down_pair, up_rows;
};
size_t prefill_scratch_bytes(uint32_t max_tokens, uint32_t k, uint32_t n_expert, uint32_t n_embd, uint32_t n_ff,
                             PrefillScratch *lay);
bool prefill_eligible(uint32_t n_embd, uint32_t n_ff, const uint8_t *gate, const uint8_t *up, const uint8_t *down,
                      int layout);
struct PrefillArgs {
    const uint8_t *gate, *up, *down;   // one layer's expert tensors
    const uint8_t *xq;                 // Q8_K of x, [n_tokens][n_embd/256]
    const int32_t *selected;           // [n_tokens][k]
    const float *weights;              // [n_tokens][k]
    float *mid;                        // [n_tokens*k][n_ff] f32 (scratch, also an output)
    uint8_t *midq;                     // [n_tokens*k][n_ff/256] Q8_K (scratch)
    float *out;                        // [n_tokens][n_embd]
    uint8_t *scratch;
    PrefillScratch lay;
    uint32_t n_tokens, k, n_expert, n_embd, n_ff;
    float clamp;
    int layout, ieee;
    int *status;
    cudaEvent_t *phase_events;         // optional, 6 events: start, grouped+gathered, gate/up, q8k+gather, down, sum
    const HcEpilogue *hc;              // optional: hc_expand fused into the slot sum
    cudaEvent_t before_sum;            // optional: the stream waits for this event before the slot sum (shared expert done)
    float *const *row_ptr;             // optional (k == 1): row_ptr[pair] receives the pair's down row; no slot sum then
};
// Everything after the router and the Q8_K of x. Returns the number of kernels launched.
int launch_prefill_experts(cudaStream_t st, const PrefillArgs &p);

// FP8 E4M3 block-scaled projection. rows_per_block = 1 (activations, 1 x 128 blocks) or 128 (weights, 128 x 128).
void launch_fp8_quantize(cudaStream_t st, const float *x, uint8_t *codes, float *scales, uint32_t rows, uint32_t cols,
                         int rows_per_block);
int launch_fp8_linear(cudaStream_t st, const uint8_t *a, const float *a_scale, const uint8_t *w, const float *w_scale,
                      void *out_bf16, uint32_t M, uint32_t N, uint32_t K, int *status);

}  // namespace dsmoe
