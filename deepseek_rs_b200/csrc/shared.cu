// The steps that run on the same normalised activations right beside the routed experts: router logits (f16 weights),
// and the shared expert (Q8_0 weights x Q8_0 activations, SwiGLU between). Kernel for kernel these stand where
//   quantize_q8_0            engine/src/kernels/quantize.rs:147-225
//   matmul_q8_0_preq_warp8   engine/src/kernels/matmul.rs:357-405 (and its batched twin)
//   swiglu                   engine/src/kernels/utils.rs:141-163
//   matmul_f16               engine/src/kernels/matmul.rs:57-105
// stand in engine/src/session.rs:1894-2008. The arithmetic order of each (which partial sums exist and in which order
// they are added) is kept, so the results equal the CPU oracle bit for bit; the thread mapping is new.
#include <cuda_fp16.h>

#include "async.cuh"
#include "common.cuh"
#include "launch.h"

namespace dsmoe {

constexpr int Q8_0_BYTES = 34;  // f16 scale + 32 int8

// ---------------------------------------------------------------------------------------------------------------
// quantize_q8_0: one warp per 32-element block, one element per lane. d = amax / 127, id = 1 / d (0 when d is 0),
// q = trunc(x * id +/- 0.5) clamped to int8; lanes past the end of the row write 0.
// ---------------------------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256) quantize_q8_0_kernel(const float *__restrict__ x, int8_t *__restrict__ xq,
                                                             float *__restrict__ xscale, uint64_t in_dim, uint64_t blocks,
                                                             uint64_t n_units)
{
    const uint64_t unit = (uint64_t)blockIdx.x * 8 + (threadIdx.x >> 5);  // (token, block)
    if (unit >= n_units) return;
    const uint32_t lane = threadIdx.x & 31;
    const uint64_t tok = unit / blocks, b = unit - tok * blocks, i = b * 32 + lane;
    const float v = i < in_dim ? x[tok * in_dim + i] : 0.0f;
    float amax = v < 0.0f ? -v : v;
#pragma unroll
    for (int m = 16; m > 0; m >>= 1) {
        const float o = __shfl_xor_sync(FULL, amax, m);
        amax = o > amax ? o : amax;
    }
    const float d = __fdiv_rn(amax, 127.0f), id = d != 0.0f ? __fdiv_rn(1.0f, d) : 0.0f;
    if (lane == 0) xscale[unit] = d;
    int q = 0;
    if (i < in_dim) {
        const float raw = __fmul_rn(v, id);
        q = raw >= 0.0f ? (int)__fadd_rn(raw, 0.5f) : (int)__fsub_rn(raw, 0.5f);
        q = q > 127 ? 127 : (q < -128 ? -128 : q);
    }
    xq[unit * 32 + lane] = (int8_t)q;
}

// ---------------------------------------------------------------------------------------------------------------
// matmul_q8_0: out[tok][row] = sum over blocks of (scale_w * xscale[b]) * dot_int8. One warp per (row, tile of TOK
// tokens); lane l takes blocks l, l+32, ... in ascending order (the reference's lane partials), then the xor
// butterfly 16, 8, 4, 2, 1. A 34-byte block starts on a 2-byte boundary: it is fetched as nine aligned words and, for
// odd blocks, realigned with funnel shifts. The weight words of a block are reused for all TOK tokens of the tile.
// ---------------------------------------------------------------------------------------------------------------
template <int TOK>
__global__ void __launch_bounds__(256) matmul_q8_0_kernel(const uint8_t *__restrict__ w, const int8_t *__restrict__ xq,
                                                           const float *__restrict__ xscale, float *__restrict__ out,
                                                           uint64_t out_dim, uint64_t blocks, uint64_t n_tok)
{
    const uint64_t row = (uint64_t)blockIdx.x * 8 + (threadIdx.x >> 5);
    if (row >= out_dim) return;
    const uint32_t lane = threadIdx.x & 31;
    const uint64_t tok0 = (uint64_t)blockIdx.y * TOK;
    const uint8_t *wrow = w + row * blocks * Q8_0_BYTES;  // rows are 2-byte aligned at least
    float acc[TOK];
#pragma unroll
    for (int t = 0; t < TOK; ++t) acc[t] = 0.0f;
    // four blocks per lane and round: all their words are requested before any is used
    for (uint64_t b0 = lane; b0 < blocks; b0 += 128) {
        uint32_t raw[4][9];
        bool odd[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const uint64_t b = b0 + 32 * u;
            if (b >= blocks) break;
            const uint8_t *blk = wrow + b * Q8_0_BYTES;
            const uintptr_t addr = reinterpret_cast<uintptr_t>(blk);
            const uint32_t *aw = reinterpret_cast<const uint32_t *>(addr & ~(uintptr_t)3);  // aligned words covering the block
            odd[u] = (addr & 2) != 0;
#pragma unroll
            for (int i = 0; i < 8; ++i) raw[u][i] = aw[i];
            // the ninth word: an even block only owns its low half (never read past the tensor)
            raw[u][8] = odd[u] ? aw[8] : (uint32_t)*reinterpret_cast<const uint16_t *>(blk + 32);
        }
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const uint64_t b = b0 + 32 * u;
            if (b >= blocks) break;
            uint32_t wq[8], scale_bits;
            if (!odd[u]) {  // [scale | q0 q1] [q2..q5] ... : the int8 data starts in the upper half of word 0
                scale_bits = raw[u][0] & 0xFFFFu;
#pragma unroll
                for (int i = 0; i < 8; ++i) wq[i] = __funnelshift_r(raw[u][i], raw[u][i + 1], 16);
            } else {        // [.. | scale] [q0..q3] ...
                scale_bits = raw[u][0] >> 16;
#pragma unroll
                for (int i = 0; i < 8; ++i) wq[i] = raw[u][i + 1];
            }
            const float sw = f16_bits_to_f32(scale_bits, false);
#pragma unroll
            for (int t = 0; t < TOK; ++t) {
                if (tok0 + t >= n_tok) break;
                const uint4 *xv = reinterpret_cast<const uint4 *>(xq + ((tok0 + t) * blocks + b) * 32);
                const uint4 x0 = xv[0], x1 = xv[1];
                int dot = 0;
                dot = __dp4a((int)wq[0], (int)x0.x, dot), dot = __dp4a((int)wq[1], (int)x0.y, dot);
                dot = __dp4a((int)wq[2], (int)x0.z, dot), dot = __dp4a((int)wq[3], (int)x0.w, dot);
                dot = __dp4a((int)wq[4], (int)x1.x, dot), dot = __dp4a((int)wq[5], (int)x1.y, dot);
                dot = __dp4a((int)wq[6], (int)x1.z, dot), dot = __dp4a((int)wq[7], (int)x1.w, dot);
                const float sc = __fmul_rn(sw, xscale[(tok0 + t) * blocks + b]);
                acc[t] = __fadd_rn(acc[t], __fmul_rn(sc, (float)dot));
            }
        }
    }
#pragma unroll
    for (int t = 0; t < TOK; ++t) {
        float v = acc[t];
#pragma unroll
        for (int m = 16; m > 0; m >>= 1) v = __fadd_rn(v, __shfl_xor_sync(FULL, v, m));
        if (lane == 0 && tok0 + t < n_tok) out[(tok0 + t) * out_dim + row] = v;
    }
}

// ---------------------------------------------------------------------------------------------------------------
// swiglu: out = ((g / (1 + exp(-g))) * u) * weight with g clamped from above and u to [-clamp, clamp]
// ---------------------------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256) swiglu_kernel(const float *__restrict__ gate, const float *__restrict__ up,
                                                      float *__restrict__ out, uint64_t n, float clamp, float weight)
{
    const uint64_t i = (uint64_t)blockIdx.x * 256 + threadIdx.x;
    if (i >= n) return;
    float g = gate[i], u = up[i];
    if (clamp > 1.0e-6f) {
        if (g > clamp) g = clamp;
        if (u > clamp) u = clamp;
        if (u < -clamp) u = -clamp;
    }
    out[i] = swiglu_weighted(g, u, weight);
}

// ---------------------------------------------------------------------------------------------------------------
// matmul_f16: out[tok][row] = dot(w[row], x[tok]). The reference sums with 256 threads striding the row (thread tx adds
// elements tx, tx+256, ... in order) and a shared-memory halving tree. Here one warp does a (row, token): lane l owns
// the partial sums of threads 8l .. 8l+7, whose elements at every step are 8 contiguous f16 (one 16-byte load). The
// tree's strides 128 .. 8 pair lane l with lane l + stride/8 (shuffles), strides 4, 2, 1 fold the lane's own eight.
// ---------------------------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(64) matmul_f16_kernel(const uint16_t *__restrict__ w, const float *__restrict__ x,
                                                         float *__restrict__ out, uint64_t in_dim, uint64_t out_dim,
                                                         uint64_t n_tok)
{
    const uint64_t row = (uint64_t)blockIdx.x * 2 + (threadIdx.x >> 5), tok = blockIdx.y;
    if (row >= out_dim || tok >= n_tok) return;
    const uint32_t lane = threadIdx.x & 31;
    const uint16_t *wr = w + row * in_dim;
    const float *xr = x + tok * in_dim;
    float p[8];
#pragma unroll
    for (int k = 0; k < 8; ++k) p[k] = 0.0f;
    const bool vec = (in_dim & 7) == 0 && ((reinterpret_cast<uintptr_t>(wr) | reinterpret_cast<uintptr_t>(xr)) & 15) == 0;
    if (vec) {
        for (uint64_t base0 = 8 * lane; base0 < in_dim; base0 += 1024) {  // four rounds of loads in flight
            uint4 wv[4];
            float4 xa[4], xb[4];
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const uint64_t base = base0 + 256 * u;
                if (base < in_dim) {
                    wv[u] = *reinterpret_cast<const uint4 *>(wr + base);
                    xa[u] = *reinterpret_cast<const float4 *>(xr + base);
                    xb[u] = *reinterpret_cast<const float4 *>(xr + base + 4);
                }
            }
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                if (base0 + 256 * u >= in_dim) break;
                const uint32_t ww[4] = {wv[u].x, wv[u].y, wv[u].z, wv[u].w};
                const float xs[8] = {xa[u].x, xa[u].y, xa[u].z, xa[u].w, xb[u].x, xb[u].y, xb[u].z, xb[u].w};
#pragma unroll
                for (int k = 0; k < 8; ++k)
                    p[k] = __fadd_rn(p[k], __fmul_rn(f16_bits_to_f32((ww[k >> 1] >> (16 * (k & 1))) & 0xFFFFu, false), xs[k]));
            }
        }
    } else {
        for (uint64_t base = 8 * lane; base < in_dim; base += 256)
#pragma unroll
            for (int k = 0; k < 8; ++k)
                if (base + k < in_dim) p[k] = __fadd_rn(p[k], __fmul_rn(f16_bits_to_f32(wr[base + k], false), xr[base + k]));
    }
#pragma unroll
    for (int m = 16; m > 0; m >>= 1)  // strides 128, 64, 32, 16, 8 of the tree; lanes below m hold its values
#pragma unroll
        for (int k = 0; k < 8; ++k) p[k] = __fadd_rn(p[k], __shfl_down_sync(FULL, p[k], m));
#pragma unroll
    for (int k = 0; k < 4; ++k) p[k] = __fadd_rn(p[k], p[k + 4]);  // stride 4
    p[0] = __fadd_rn(p[0], p[2]), p[1] = __fadd_rn(p[1], p[3]);    // stride 2
    if (lane == 0) out[tok * out_dim + row] = __fadd_rn(p[0], p[1]);  // stride 1
}

// The common shape (rows of at most 4096 values, a multiple of 256, 16-byte aligned): every weight load of the row is
// requested at once, and the CTA's four rows share one copy of the token's activations in shared memory. Same
// partial sums and tree as above.
constexpr int MF_MAX_IN = 4096;

__global__ void __launch_bounds__(128) matmul_f16_staged_kernel(const uint16_t *__restrict__ w, const float *__restrict__ x,
                                                                float *__restrict__ out, uint32_t in_dim, uint32_t out_dim)
{
    __shared__ __align__(16) float s_x[MF_MAX_IN];
    const uint32_t lane = threadIdx.x & 31, row = blockIdx.x * 4 + (threadIdx.x >> 5), tok = blockIdx.y;
    const uint32_t rounds = in_dim / 256;
    const bool has = row < out_dim;
    const uint16_t *wr = w + (size_t)(has ? row : 0) * in_dim + 8 * lane;
    uint4 wv[MF_MAX_IN / 256];
#pragma unroll
    for (int u = 0; u < MF_MAX_IN / 256; ++u)
        if (has && (uint32_t)u < rounds) wv[u] = *reinterpret_cast<const uint4 *>(wr + 256 * u);
    const float4 *xr = reinterpret_cast<const float4 *>(x + (size_t)tok * in_dim);
    for (uint32_t i = threadIdx.x; i < in_dim / 4; i += 128) reinterpret_cast<float4 *>(s_x)[i] = xr[i];
    __syncthreads();
    if (!has) return;
    float p[8];
#pragma unroll
    for (int k = 0; k < 8; ++k) p[k] = 0.0f;
#pragma unroll
    for (int u = 0; u < MF_MAX_IN / 256; ++u) {
        if ((uint32_t)u >= rounds) break;
        const float4 xa = *reinterpret_cast<const float4 *>(s_x + 256 * u + 8 * lane);
        const float4 xb = *reinterpret_cast<const float4 *>(s_x + 256 * u + 8 * lane + 4);
        const uint32_t ww[4] = {wv[u].x, wv[u].y, wv[u].z, wv[u].w};
        const float xs[8] = {xa.x, xa.y, xa.z, xa.w, xb.x, xb.y, xb.z, xb.w};
#pragma unroll
        for (int k = 0; k < 8; ++k)
            p[k] = __fadd_rn(p[k], __fmul_rn(f16_bits_to_f32((ww[k >> 1] >> (16 * (k & 1))) & 0xFFFFu, false), xs[k]));
    }
#pragma unroll
    for (int m = 16; m > 0; m >>= 1)
#pragma unroll
        for (int k = 0; k < 8; ++k) p[k] = __fadd_rn(p[k], __shfl_down_sync(FULL, p[k], m));
#pragma unroll
    for (int k = 0; k < 4; ++k) p[k] = __fadd_rn(p[k], p[k + 4]);
    p[0] = __fadd_rn(p[0], p[2]), p[1] = __fadd_rn(p[1], p[3]);
    if (lane == 0) out[(size_t)tok * out_dim + row] = __fadd_rn(p[0], p[1]);
}

// ---------------------------------------------------------------------------------------------------------------
// Small batches: the shared expert in two launches instead of six. Every CTA quantises the token's activation row to
// Q8_0 itself, into shared memory (the same arithmetic as quantize_q8_0_kernel, so the same codes), and then its eight
// warps each take one output row. FIRST: gate row r and up row r of the same warp meet in the SwiGLU, out = mid.
// Otherwise: the down projection. Results equal the six-launch path bit for bit.
// ---------------------------------------------------------------------------------------------------------------
__device__ __forceinline__ void q8_0_block_words(const uint8_t *blk, uint32_t (&wq)[8], float &scale)
{
    const uintptr_t addr = reinterpret_cast<uintptr_t>(blk);
    const uint32_t *aw = reinterpret_cast<const uint32_t *>(addr & ~(uintptr_t)3);
    uint32_t raw[9];
#pragma unroll
    for (int i = 0; i < 8; ++i) raw[i] = aw[i];
    if (addr & 2) {
        raw[8] = aw[8];
        scale = f16_bits_to_f32(raw[0] >> 16, false);
#pragma unroll
        for (int i = 0; i < 8; ++i) wq[i] = raw[i + 1];
    } else {
        raw[8] = (uint32_t)*reinterpret_cast<const uint16_t *>(blk + 32);
        scale = f16_bits_to_f32(raw[0] & 0xFFFFu, false);
#pragma unroll
        for (int i = 0; i < 8; ++i) wq[i] = __funnelshift_r(raw[i], raw[i + 1], 16);
    }
}

__device__ __forceinline__ int q8_0_dot32(const uint32_t (&wq)[8], const int8_t *xq_blk)
{
    const uint4 x0 = reinterpret_cast<const uint4 *>(xq_blk)[0], x1 = reinterpret_cast<const uint4 *>(xq_blk)[1];
    int dot = 0;
    dot = __dp4a((int)wq[0], (int)x0.x, dot), dot = __dp4a((int)wq[1], (int)x0.y, dot);
    dot = __dp4a((int)wq[2], (int)x0.z, dot), dot = __dp4a((int)wq[3], (int)x0.w, dot);
    dot = __dp4a((int)wq[4], (int)x1.x, dot), dot = __dp4a((int)wq[5], (int)x1.y, dot);
    dot = __dp4a((int)wq[6], (int)x1.z, dot), dot = __dp4a((int)wq[7], (int)x1.w, dot);
    return dot;
}

constexpr int SHF_MAX_IN = 4096;  // widest activation row the fused kernels hold in shared memory

template <bool FIRST>
__global__ void __launch_bounds__(256) shared_fused_kernel(const uint8_t *__restrict__ w0, const uint8_t *__restrict__ w1,
                                                            const float *__restrict__ x, float *__restrict__ out,
                                                            uint32_t in_dim, uint32_t out_dim, float clamp)
{
    __shared__ __align__(16) int8_t s_xq[SHF_MAX_IN];
    __shared__ float s_xs[SHF_MAX_IN / 32];
    const uint32_t lane = threadIdx.x & 31, warp = threadIdx.x >> 5, tok = blockIdx.y, blocks = in_dim / 32;
    pdl_launch_dependents();
    pdl_wait();
    const float *xr = x + (size_t)tok * in_dim;
    // quantize_q8_0 of blocks warp, warp + 8, ...: all of the warp's values are requested first
    float xv[SHF_MAX_IN / 256];
#pragma unroll
    for (int i = 0; i < SHF_MAX_IN / 256; ++i) {
        const uint32_t b = warp + 8 * i;
        xv[i] = b < blocks ? xr[b * 32 + lane] : 0.0f;
    }
#pragma unroll
    for (int i = 0; i < SHF_MAX_IN / 256; ++i) {
        const uint32_t b = warp + 8 * i;
        if (b >= blocks) break;
        const float v = xv[i];
        float amax = v < 0.0f ? -v : v;
#pragma unroll
        for (int m = 16; m > 0; m >>= 1) {
            const float o = __shfl_xor_sync(FULL, amax, m);
            amax = o > amax ? o : amax;
        }
        const float d = __fdiv_rn(amax, 127.0f), id = d != 0.0f ? __fdiv_rn(1.0f, d) : 0.0f;
        const float raw = __fmul_rn(v, id);
        int q = raw >= 0.0f ? (int)__fadd_rn(raw, 0.5f) : (int)__fsub_rn(raw, 0.5f);
        q = q > 127 ? 127 : (q < -128 ? -128 : q);
        s_xq[b * 32 + lane] = (int8_t)q;
        if (lane == 0) s_xs[b] = d;
    }
    __syncthreads();
    const uint32_t row = blockIdx.x * 8 + warp;
    if (row >= out_dim) return;
    const uint8_t *r0 = w0 + (size_t)row * blocks * Q8_0_BYTES, *r1 = FIRST ? w1 + (size_t)row * blocks * Q8_0_BYTES : nullptr;
    float a0 = 0.0f, a1 = 0.0f;
    // ascending blocks per lane (the reference's lane partials), four at a time with all their words requested first
    for (uint32_t b0 = lane; b0 < blocks; b0 += 128) {
        uint32_t wq0[4][8], wq1[4][8];
        float sw0[4], sw1[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const uint32_t b = b0 + 32 * u;
            if (b >= blocks) break;
            q8_0_block_words(r0 + (size_t)b * Q8_0_BYTES, wq0[u], sw0[u]);
            if (FIRST) q8_0_block_words(r1 + (size_t)b * Q8_0_BYTES, wq1[u], sw1[u]);
        }
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const uint32_t b = b0 + 32 * u;
            if (b >= blocks) break;
            a0 = __fadd_rn(a0, __fmul_rn(__fmul_rn(sw0[u], s_xs[b]), (float)q8_0_dot32(wq0[u], s_xq + b * 32)));
            if (FIRST) a1 = __fadd_rn(a1, __fmul_rn(__fmul_rn(sw1[u], s_xs[b]), (float)q8_0_dot32(wq1[u], s_xq + b * 32)));
        }
    }
#pragma unroll
    for (int m = 16; m > 0; m >>= 1) {
        a0 = __fadd_rn(a0, __shfl_xor_sync(FULL, a0, m));
        if (FIRST) a1 = __fadd_rn(a1, __shfl_xor_sync(FULL, a1, m));
    }
    if (lane == 0) {
        if (FIRST) {
            float g = a0, u = a1;
            if (clamp > 1.0e-6f) {
                if (g > clamp) g = clamp;
                if (u > clamp) u = clamp;
                if (u < -clamp) u = -clamp;
            }
            out[(size_t)tok * out_dim + row] = swiglu_weighted(g, u, 1.0f);
        } else {
            out[(size_t)tok * out_dim + row] = a0;
        }
    }
}

// ---------------------------------------------------------------------------------------------------------------
// The same two launches with the weight rows staged through shared memory by bulk asynchronous copies: a warp's two
// rows (gate row r and up row r; or two adjacent down rows) arrive as whole 16-byte-aligned rows while the CTA
// quantises the activations, instead of as 4-byte loads at a 34-byte lane stride. All TOK tokens of the call share
// one pass over the weights. The second launch requests its rows before it waits for the first launch to finish
// (the weights are never written by these kernels). Needs 16-byte aligned tensors and in_dim a multiple of 256.
// Lane partials over ascending blocks and the xor butterfly are those of the kernels above: same bits.
// ---------------------------------------------------------------------------------------------------------------
constexpr int SHS_MAX_TOK = 8;

// PREQ: the activations arrive quantised (xq, xs in global memory, from quantize_q8_0_kernel) and the CTA takes the
// tile of TOK tokens blockIdx.y, fetched by two more bulk copies instead of being quantised here; this is the form
// for more than SHS_MAX_TOK tokens, where quantising in every CTA would cost more than the weights.
template <bool FIRST, int TOK, bool PREQ>
__global__ void __launch_bounds__(256) shared_staged_kernel(const uint8_t *__restrict__ w0, const uint8_t *__restrict__ w1,
                                                             const float *__restrict__ x, const int8_t *__restrict__ xq,
                                                             const float *__restrict__ xs, float *__restrict__ out,
                                                             uint32_t in_dim, uint32_t out_dim, uint32_t n_tok_all, float clamp,
                                                             int *status)
{
    extern __shared__ __align__(128) uint8_t smem[];
    const uint32_t lane = threadIdx.x & 31, warp = threadIdx.x >> 5, blocks = in_dim / 32;
    const uint32_t row_bytes = blocks * Q8_0_BYTES;
    uint8_t *wst = smem + (size_t)warp * 2 * row_bytes;
    int8_t *s_xq = reinterpret_cast<int8_t *>(smem + (size_t)16 * row_bytes);
    float *s_xs = reinterpret_cast<float *>(s_xq + (size_t)TOK * in_dim);
    uint64_t *bars = reinterpret_cast<uint64_t *>(s_xs + (size_t)TOK * blocks), *bar = bars + warp, *tile_bar = bars + 8;
    const uint32_t tok0 = PREQ ? blockIdx.y * TOK : 0u;
    const uint32_t n_tok = n_tok_all - tok0 < (uint32_t)TOK ? n_tok_all - tok0 : (uint32_t)TOK;
    // FIRST: rows r of both tensors; otherwise rows r, r + 1 of the one tensor (adjacent in memory: one copy)
    const uint32_t row = FIRST ? blockIdx.x * 8 + warp : blockIdx.x * 16 + 2 * warp;
    const uint32_t n_rows = row >= out_dim ? 0u : (FIRST ? 2u : (out_dim - row < 2u ? out_dim - row : 2u));
    if (lane == 0) {
        mbar_init(bar, 1);
        if (PREQ && warp == 0) mbar_init(tile_bar, 1);
        fence_async_smem();
    }
    auto request_rows = [&]() {
        if (lane != 0 || n_rows == 0) return;
        mbar_expect_tx(bar, n_rows * row_bytes);
        if (FIRST) {
            bulk_g2s(wst, w0 + (size_t)row * row_bytes, row_bytes, bar);
            bulk_g2s(wst + row_bytes, w1 + (size_t)row * row_bytes, row_bytes, bar);
        } else {
            bulk_g2s(wst, w0 + (size_t)row * row_bytes, n_rows * row_bytes, bar);
        }
    };
    if (!FIRST) request_rows();
    pdl_launch_dependents();
    pdl_wait();
    if (FIRST) request_rows();
    if (PREQ) {
        if (threadIdx.x == 0) {
            mbar_expect_tx(tile_bar, n_tok * in_dim + n_tok * blocks * 4);
            bulk_g2s(s_xq, xq + (size_t)tok0 * in_dim, n_tok * in_dim, tile_bar);
            bulk_g2s(s_xs, xs + (size_t)tok0 * blocks, n_tok * blocks * 4, tile_bar);
        }
    } else {
        // quantize_q8_0 of every token's row: a thread takes 16 adjacent values, two neighbouring lanes share a block
        // (its largest magnitude is the larger of the two halves'; the maximum does not depend on the order)
        const uint32_t halves = in_dim / 16, total = n_tok * halves;
        for (uint32_t base = 0; base < total; base += 256) {
            const uint32_t u = base + threadIdx.x;
            const bool active = u < total;
            const uint32_t t = active ? u / halves : 0, h = active ? u - t * halves : 0;
            const float4 *src = reinterpret_cast<const float4 *>(x + (size_t)t * in_dim + h * 16);
            float v[16];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const float4 f = active ? src[i] : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
                v[4 * i] = f.x, v[4 * i + 1] = f.y, v[4 * i + 2] = f.z, v[4 * i + 3] = f.w;
            }
            float amax = 0.0f;
#pragma unroll
            for (int i = 0; i < 16; ++i) {
                const float m = v[i] < 0.0f ? -v[i] : v[i];
                amax = m > amax ? m : amax;
            }
            const float o = __shfl_xor_sync(FULL, amax, 1);
            amax = o > amax ? o : amax;
            const float d = __fdiv_rn(amax, 127.0f), id = d != 0.0f ? __fdiv_rn(1.0f, d) : 0.0f;
            uint32_t pk[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                pk[i] = 0;
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const float raw = __fmul_rn(v[4 * i + j], id);
                    int q = raw >= 0.0f ? (int)__fadd_rn(raw, 0.5f) : (int)__fsub_rn(raw, 0.5f);
                    q = q > 127 ? 127 : (q < -128 ? -128 : q);
                    pk[i] |= ((uint32_t)q & 0xFFu) << (8 * j);
                }
            }
            if (active) {
                *reinterpret_cast<uint4 *>(s_xq + (size_t)t * in_dim + h * 16) = make_uint4(pk[0], pk[1], pk[2], pk[3]);
                if (!(h & 1)) s_xs[t * blocks + (h >> 1)] = d;
            }
        }
    }
    __syncthreads();
    if (n_rows == 0) return;
    if (PREQ && !mbar_wait_bounded(tile_bar, 0, status)) return;
    if (!mbar_wait_bounded(bar, 0, status)) return;
    float acc[2][TOK];
#pragma unroll
    for (int t = 0; t < TOK; ++t) acc[0][t] = acc[1][t] = 0.0f;
    for (uint32_t b = lane; b < blocks; b += 32) {
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            if ((uint32_t)r >= n_rows) break;
            // A block starts on a 2-byte boundary: nine aligned words from its first 4-byte boundary at or after the
            // scale's, shifted by 16 bits when the block itself is aligned (its int8 data then starts mid-word). No
            // branch on the block's parity, which alternates across the lanes. The ninth word of a block that is not
            // aligned belongs to whatever follows it in shared memory and is shifted out.
            const uint8_t *blk = wst + (size_t)r * row_bytes + (size_t)b * Q8_0_BYTES;
            const uint32_t odd = (uint32_t)(b & 1);  // rows start 16-byte aligned and a block has 34 bytes
            const uint32_t *aw = reinterpret_cast<const uint32_t *>(blk + 2 * odd);
            const uint32_t shift = odd ? 0u : 16u;
            uint32_t raw[9], wq[8];
#pragma unroll
            for (int i = 0; i < 9; ++i) raw[i] = aw[i];
#pragma unroll
            for (int i = 0; i < 8; ++i) wq[i] = __funnelshift_r(raw[i], raw[i + 1], shift);
            const float sw = f16_bits_to_f32(*reinterpret_cast<const uint16_t *>(blk), false);
#pragma unroll
            for (int t = 0; t < TOK; ++t) {
                if ((uint32_t)t >= n_tok) break;
                const int dot = q8_0_dot32(wq, s_xq + (size_t)t * in_dim + b * 32);
                acc[r][t] = __fadd_rn(acc[r][t], __fmul_rn(__fmul_rn(sw, s_xs[t * blocks + b]), (float)dot));
            }
        }
    }
    // after the xor butterfly every lane holds the sums; lane t keeps token t's pair and finishes it
    float g = 0.0f, u = 0.0f;
#pragma unroll
    for (int t = 0; t < TOK; ++t) {
        if ((uint32_t)t >= n_tok) break;
        float a0 = acc[0][t], a1 = acc[1][t];
#pragma unroll
        for (int m = 16; m > 0; m >>= 1) {
            a0 = __fadd_rn(a0, __shfl_xor_sync(FULL, a0, m));
            a1 = __fadd_rn(a1, __shfl_xor_sync(FULL, a1, m));
        }
        if (lane == (uint32_t)t) g = a0, u = a1;
    }
    if (lane >= n_tok || lane >= (uint32_t)TOK) return;
    if (FIRST) {
        if (clamp > 1.0e-6f) {
            if (g > clamp) g = clamp;
            if (u > clamp) u = clamp;
            if (u < -clamp) u = -clamp;
        }
        out[(size_t)(tok0 + lane) * out_dim + row] = swiglu_weighted(g, u, 1.0f);
    } else {
        out[(size_t)(tok0 + lane) * out_dim + row] = g;
        if (n_rows == 2) out[(size_t)(tok0 + lane) * out_dim + row + 1] = u;
    }
}

static size_t shared_staged_smem(uint32_t in_dim, int tok)
{
    const size_t blocks = in_dim / 32;
    return 16 * blocks * Q8_0_BYTES + (size_t)tok * in_dim + (size_t)tok * blocks * 4 + 16 * sizeof(uint64_t);
}

template <int TOK>
static void launch_shared_staged(cudaStream_t st, const uint8_t *gate_w, const uint8_t *up_w, const uint8_t *down_w,
                                 const float *x, float *mid, float *out, uint32_t n_embd, uint32_t n_ff, uint32_t n_tokens,
                                 float clamp, int *status)
{
    static OncePerDevice attr;  // one per template instance
    if (attr.first()) {
        cudaFuncSetAttribute(shared_staged_kernel<true, TOK, false>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             (int)shared_staged_smem(SHF_MAX_IN, TOK));
        cudaFuncSetAttribute(shared_staged_kernel<false, TOK, false>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             (int)shared_staged_smem(SHF_MAX_IN, TOK));
    }
    launch_pdl(shared_staged_kernel<true, TOK, false>, dim3((n_ff + 7) / 8), dim3(256), shared_staged_smem(n_embd, TOK), st,
               gate_w, up_w, x, (const int8_t *)nullptr, (const float *)nullptr, mid, n_embd, n_ff, n_tokens, clamp, status);
    launch_pdl(shared_staged_kernel<false, TOK, false>, dim3((n_embd + 15) / 16), dim3(256), shared_staged_smem(n_ff, TOK), st,
               down_w, (const uint8_t *)nullptr, (const float *)mid, (const int8_t *)nullptr, (const float *)nullptr, out, n_ff,
               n_embd, n_tokens, clamp, status);
}

// More than SHS_MAX_TOK tokens: quantise, gate + up + SwiGLU over tiles of eight tokens, quantise, down over tiles.
bool shared_tiles_eligible(const uint8_t *gate_w, const uint8_t *up_w, const uint8_t *down_w, const int8_t *xq,
                           const float *xs, uint32_t n_embd, uint32_t n_ff)
{
    return n_embd % 256 == 0 && n_ff % 256 == 0 && n_embd <= (uint32_t)SHF_MAX_IN && n_ff <= (uint32_t)SHF_MAX_IN &&
           ((reinterpret_cast<uintptr_t>(gate_w) | reinterpret_cast<uintptr_t>(up_w) | reinterpret_cast<uintptr_t>(down_w) |
             reinterpret_cast<uintptr_t>(xq) | reinterpret_cast<uintptr_t>(xs)) & 15) == 0;
}

int launch_shared_tiles(cudaStream_t st, const uint8_t *gate_w, const uint8_t *up_w, const uint8_t *down_w, const float *x,
                        int8_t *xq, float *xs, float *mid, float *out, uint32_t n_embd, uint32_t n_ff, uint32_t n_tokens,
                        float clamp, int *status)
{
    constexpr int TOK = SHS_MAX_TOK;
    static OncePerDevice attr;
    if (attr.first()) {
        cudaFuncSetAttribute(shared_staged_kernel<true, TOK, true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             (int)shared_staged_smem(SHF_MAX_IN, TOK));
        cudaFuncSetAttribute(shared_staged_kernel<false, TOK, true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             (int)shared_staged_smem(SHF_MAX_IN, TOK));
    }
    const unsigned tiles = (n_tokens + TOK - 1) / TOK;
    launch_quantize_q8_0(st, x, xq, xs, n_embd, n_tokens);
    launch_pdl(shared_staged_kernel<true, TOK, true>, dim3((n_ff + 7) / 8, tiles), dim3(256), shared_staged_smem(n_embd, TOK), st,
               gate_w, up_w, (const float *)nullptr, (const int8_t *)xq, (const float *)xs, mid, n_embd, n_ff, n_tokens, clamp,
               status);
    launch_quantize_q8_0(st, mid, xq, xs, n_ff, n_tokens);
    launch_pdl(shared_staged_kernel<false, TOK, true>, dim3((n_embd + 15) / 16, tiles), dim3(256), shared_staged_smem(n_ff, TOK),
               st, down_w, (const uint8_t *)nullptr, (const float *)nullptr, (const int8_t *)xq, (const float *)xs, out, n_ff,
               n_embd, n_tokens, clamp, status);
    return 4;
}

// The staged form needs whole rows that bulk copies can take: 16-byte aligned tensors, rows a multiple of 16 bytes.
static bool shared_staged_eligible(const uint8_t *gate_w, const uint8_t *up_w, const uint8_t *down_w, const float *x,
                                   const float *mid, uint32_t n_embd, uint32_t n_ff, uint32_t n_tokens)
{
    return n_tokens <= (uint32_t)SHS_MAX_TOK && n_embd % 256 == 0 && n_ff % 256 == 0 && n_embd <= (uint32_t)SHF_MAX_IN &&
           n_ff <= (uint32_t)SHF_MAX_IN &&
           ((reinterpret_cast<uintptr_t>(gate_w) | reinterpret_cast<uintptr_t>(up_w) | reinterpret_cast<uintptr_t>(down_w) |
             reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(mid)) & 15) == 0;
}

bool shared_fused_eligible(uint32_t n_embd, uint32_t n_ff, uint32_t n_tokens)
{
    return n_tokens <= (uint32_t)SHS_MAX_TOK && n_embd % 32 == 0 && n_ff % 32 == 0 && n_embd <= (uint32_t)SHF_MAX_IN &&
           n_ff <= (uint32_t)SHF_MAX_IN;
}

int launch_shared_fused(cudaStream_t st, const uint8_t *gate_w, const uint8_t *up_w, const uint8_t *down_w, const float *x,
                        float *mid, float *out, uint32_t n_embd, uint32_t n_ff, uint32_t n_tokens, float clamp, int *status)
{
    if (shared_staged_eligible(gate_w, up_w, down_w, x, mid, n_embd, n_ff, n_tokens)) {
        if (n_tokens == 1) launch_shared_staged<1>(st, gate_w, up_w, down_w, x, mid, out, n_embd, n_ff, n_tokens, clamp, status);
        else if (n_tokens == 2) launch_shared_staged<2>(st, gate_w, up_w, down_w, x, mid, out, n_embd, n_ff, n_tokens, clamp, status);
        else if (n_tokens <= 4) launch_shared_staged<4>(st, gate_w, up_w, down_w, x, mid, out, n_embd, n_ff, n_tokens, clamp, status);
        else launch_shared_staged<8>(st, gate_w, up_w, down_w, x, mid, out, n_embd, n_ff, n_tokens, clamp, status);
        return 2;
    }
    launch_pdl(shared_fused_kernel<true>, dim3((n_ff + 7) / 8, n_tokens), dim3(256), 0, st, gate_w, up_w, x, mid, n_embd, n_ff,
               clamp);
    launch_pdl(shared_fused_kernel<false>, dim3((n_embd + 7) / 8, n_tokens), dim3(256), 0, st, down_w,
               (const uint8_t *)nullptr, (const float *)mid, out, n_ff, n_embd, clamp);
    return 2;
}

// ---------------------------------------------------------------------------------------------------------------
void launch_quantize_q8_0(cudaStream_t st, const float *x, int8_t *xq, float *xscale, uint64_t in_dim, uint64_t n_tok)
{
    const uint64_t blocks = (in_dim + 31) / 32, units = blocks * n_tok;
    if (units == 0) return;
    quantize_q8_0_kernel<<<(unsigned)((units + 7) / 8), 256, 0, st>>>(x, xq, xscale, in_dim, blocks, units);
}

void launch_matmul_q8_0(cudaStream_t st, const uint8_t *w, const int8_t *xq, const float *xscale, float *out,
                        uint64_t in_dim, uint64_t out_dim, uint64_t n_tok)
{
    const uint64_t blocks = (in_dim + 31) / 32;
    if (out_dim == 0 || n_tok == 0) return;
    const unsigned gx = (unsigned)((out_dim + 7) / 8);
    if (n_tok == 1) matmul_q8_0_kernel<1><<<dim3(gx, 1), 256, 0, st>>>(w, xq, xscale, out, out_dim, blocks, n_tok);
    else matmul_q8_0_kernel<4><<<dim3(gx, (unsigned)((n_tok + 3) / 4)), 256, 0, st>>>(w, xq, xscale, out, out_dim, blocks, n_tok);
}

void launch_swiglu(cudaStream_t st, const float *gate, const float *up, float *out, uint64_t n, float clamp, float weight)
{
    if (n == 0) return;
    swiglu_kernel<<<(unsigned)((n + 255) / 256), 256, 0, st>>>(gate, up, out, n, clamp, weight);
}

void launch_matmul_f16(cudaStream_t st, const uint16_t *w, const float *x, float *out, uint64_t in_dim, uint64_t out_dim,
                       uint64_t n_tok)
{
    if (out_dim == 0 || n_tok == 0) return;
    if (in_dim <= (uint64_t)MF_MAX_IN && in_dim % 256 == 0 && out_dim < (1ull << 31) &&
        ((reinterpret_cast<uintptr_t>(w) | reinterpret_cast<uintptr_t>(x)) & 15) == 0) {
        matmul_f16_staged_kernel<<<dim3((unsigned)((out_dim + 3) / 4), (unsigned)n_tok), 128, 0, st>>>(w, x, out, (uint32_t)in_dim,
                                                                                                     (uint32_t)out_dim);
        return;
    }
    matmul_f16_kernel<<<dim3((unsigned)((out_dim + 1) / 2), (unsigned)n_tok), 64, 0, st>>>(w, x, out, in_dim, out_dim, n_tok);
}

}  // namespace dsmoe
