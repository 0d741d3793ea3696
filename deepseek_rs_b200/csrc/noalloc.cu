// dsmoe_moe_forward_noalloc: the routed-expert step for callers that must not allocate device memory.
//
// Some hosts of this library run where cudaMalloc is off limits: a decode loop that has already handed every free
// byte of the device to its KV cache and weight arena, a plugin loaded into a process whose allocator owns the whole
// device and forbids side allocations, or a latency-critical thread that may not take the driver's allocation lock.
// dsmoe_create() allocates the scratch of dsmoe_moe_forward() with cudaMalloc, so those callers cannot even obtain a
// handle. This entry point needs no handle: its scratch is a fixed array in the library's own device image, which
// every GPU that loads the library carries from load until the process exits.
#include "async.cuh"
#include "common.cuh"
#include "launch.h"

using namespace dsmoe;

namespace {

// Reference model constants (engine/src/model.rs:4, 15-18; engine/src/session.rs:21; engine/src/kernels/moe.rs:284).
constexpr uint32_t NA_EMBD = 4096, NA_FF = 2048, NA_EXPERT = 256, NA_K = 6;
constexpr float NA_CLAMP = 10.0f, NA_ROUTE_SCALE = 1.5f;
constexpr uint32_t NA_XB = NA_EMBD / QK_K, NA_MB = NA_FF / QK_K;
constexpr uint32_t NA_T = DSMOE_NOALLOC_MAX_TOKENS;

// Scratch layout (byte offsets, all multiples of 256): the intermediates of one call for up to NA_T tokens.
constexpr size_t OFF_STATUS = 0;                                              // STATUS_WORDS ints, bounded-wait status block
constexpr size_t OFF_PROBS = 256;                                             // f32 [T][256]
constexpr size_t OFF_SEL = OFF_PROBS + (size_t)NA_T * NA_EXPERT * 4;          // i32 [T][6] (padded)
constexpr size_t OFF_WTS = OFF_SEL + 256;                                     // f32 [T][6] (padded)
constexpr size_t OFF_XQ = OFF_WTS + 256;                                      // Q8_K [T][16]
constexpr size_t OFF_MID = OFF_XQ + (((size_t)NA_T * NA_XB * Q8K_BYTES + 255) & ~(size_t)255);   // f32 [T*6][2048]
constexpr size_t OFF_MIDQ = OFF_MID + (size_t)NA_T * NA_K * NA_FF * 4;        // Q8_K [T*6][8]
constexpr size_t SCRATCH_BYTES = OFF_MIDQ + (((size_t)NA_T * NA_K * NA_MB * Q8K_BYTES + 255) & ~(size_t)255);
static_assert(NA_T * NA_K * 4 <= 256, "selection / weight slots are 256 bytes");

// About 0.55 MB. In host code this name is only a stand-in for the symbol, never a device address.
static __device__ __align__(256) unsigned char g_noalloc_scratch[SCRATCH_BYTES];

unsigned char *g_scratch_ptr[MAX_DEVICES] = {};  // per device: the array's device address, looked up once

}  // namespace

extern "C" int dsmoe_moe_forward_noalloc(dsmoe_stream stream, const uint8_t *gate, const uint8_t *up,
                                         const uint8_t *down, int layout, const float *x, const float *logits,
                                         uint32_t n_tokens, float *out, int32_t *selected_out, float *weights_out)
{
    if (layout != DSMOE_LAYOUT_NATIVE && layout != DSMOE_LAYOUT_ROWSOA) return DSMOE_ERR_ARG;
    if (n_tokens > NA_T) return DSMOE_ERR_BOUNDS;  // the static scratch holds DSMOE_NOALLOC_MAX_TOKENS tokens
    if (n_tokens == 0) return DSMOE_OK;
    if (!gate || !up || !down || !x || !logits || !out) return DSMOE_ERR_ARG;
    const uintptr_t al = layout == DSMOE_LAYOUT_ROWSOA ? 15 : 3;
    if ((((uintptr_t)gate | (uintptr_t)up | (uintptr_t)down) & al) || ((uintptr_t)x & 15)) return DSMOE_ERR_ARG;

    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= MAX_DEVICES) return DSMOE_ERR_CUDA;
    if (!g_scratch_ptr[dev]) {
        // set-up, once per device, with that device current: resolve the array's address on THIS device
        cudaDeviceProp prop;
        if (cudaGetDeviceProperties(&prop, dev) != cudaSuccess || prop.major != 10) return DSMOE_ERR_CUDA;
        unsigned char *p = nullptr;
        if (cudaGetSymbolAddress((void **)&p, g_noalloc_scratch) != cudaSuccess || !p) {
            cudaGetLastError();
            return DSMOE_ERR_CUDA;
        }
        g_scratch_ptr[dev] = p;
    }
    unsigned char *s = g_scratch_ptr[dev];
    cudaStream_t st = (cudaStream_t)stream;
    int *status = reinterpret_cast<int *>(s + OFF_STATUS);
    float *probs = reinterpret_cast<float *>(s + OFF_PROBS);
    int32_t *sel = selected_out ? selected_out : reinterpret_cast<int32_t *>(s + OFF_SEL);
    float *wts = weights_out ? weights_out : reinterpret_cast<float *>(s + OFF_WTS);
    uint8_t *xq = s + OFF_XQ;
    float *mid = reinterpret_cast<float *>(s + OFF_MID);
    uint8_t *midq = s + OFF_MIDQ;

    // The status block is the only part of the array that must start at zero: every other region is completely
    // rewritten for rows [0, n_tokens) before it is read.
    if (cudaMemsetAsync(status, 0, STATUS_WORDS * sizeof(int), st) != cudaSuccess) return DSMOE_ERR_CUDA;
    launch_router_q8k_fused(st, logits, x, probs, sel, wts, xq, n_tokens, (int)NA_K, (int)NA_EXPERT, NA_EMBD,
                            NA_ROUTE_SCALE);
    GateUpArgs g = {gate, up, xq, sel, wts, nullptr, nullptr, mid, (uint64_t)NA_FF * NA_XB * IQ2XXS_BYTES,
                    (uint64_t)NA_XB * IQ2XXS_BYTES, NA_XB, NA_FF, NA_K, n_tokens, NA_CLAMP, layout, 0};
    if (gate_up_tma_eligible(g)) launch_gate_up_mid_tma(st, g, status);
    else launch_gate_up_mid(st, g);
    launch_q8k_quantize(st, mid, midq, NA_FF, n_tokens * NA_K);
    DownArgs d = {down, midq, sel, out, (uint64_t)NA_EMBD * NA_MB * Q2K_BYTES, (uint64_t)NA_MB * Q2K_BYTES, NA_MB,
                  NA_EMBD, NA_K, n_tokens, layout, 0, 1};
    if (down_tma_eligible(d)) launch_down_tma(st, d, status);
    else launch_down(st, d);
    return cudaGetLastError() == cudaSuccess ? DSMOE_OK : DSMOE_ERR_CUDA;
}

extern "C" int dsmoe_noalloc_device_status(dsmoe_stream stream, int *code_out)
{
    if (!code_out) return DSMOE_ERR_ARG;
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= MAX_DEVICES) return DSMOE_ERR_CUDA;
    if (!g_scratch_ptr[dev]) return DSMOE_ERR_STATE;  // the entry point has not run on this device
    cudaStream_t st = (cudaStream_t)stream;
    cudaError_t e = cudaMemcpyAsync(code_out, g_scratch_ptr[dev] + OFF_STATUS, sizeof(int), cudaMemcpyDeviceToHost, st);
    if (e == cudaSuccess) e = cudaStreamSynchronize(st);
    if (e != cudaSuccess) return DSMOE_ERR_CUDA;
    return *code_out == 0 ? DSMOE_OK : DSMOE_ERR_TIMEOUT;
}
