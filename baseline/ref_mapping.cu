// A CUDA C++ restatement of the THREAD MAPPING and memory access pattern of the reference's routed-expert kernels,
// written to have a GPU number to put beside the product's on the same B200. It is NOT the reference's binary (its
// cuda-oxide toolchain is not available) and not part of the product: only tests and the bench load it.
//
// Two forms are restated. The LIVE form: one kernel each, launched as the reference launches them, i.e. once per token:
//   q8k_quantize             engine/src/kernels/quantize.rs:309-417   CTA per 256-block, shared-memory max tree
//   moe_gate_up_mid_qwarp32  engine/src/kernels/moe.rs:622-715        8 lanes per row, 4 rows per quarter-warp, lane b
//                                                                     walks blocks b, b+8; tables in global memory
//   moe_down_sum6_qwarp32    engine/src/kernels/moe.rs:922-970        8 lanes per row, the 6 slots in sequence
// The BATCHED form, which the reference contains but never calls (its only formulation of a whole chunk at once):
//   moe_count / prefix / scatter_sorted_pairs  moe.rs:299-362  histogram with global atomics, serial 256-prefix,
//                                                              atomic-cursor scatter of pair ids into expert order
//   moe_gate_up_mid_sorted_qwarp32             moe.rs:721-815  the gate/up kernel with the pair read from sorted_pairs
//   moe_down_sorted_qwarp32 + moe_sum          moe.rs:871-916, 983-1005
// Both with the block dots of engine/src/kernels/quantize.rs:763-901 in scalar form (byte loads, no dp4a, no vector
// loads), and the f16 conversion of engine/src/kernels/utils.rs:16-29 (subnormals flush to zero). Arithmetic order is
// the reference's, each f32 operation rounded separately, so the results equal the CPU oracle bit for bit.
#include <cuda_runtime.h>
#include <stdint.h>

#include "../include/dsmoe_iq2_tables.h"

namespace refmap {

constexpr int IQ2_BYTES = 66, Q2K_BYTES = 84, Q8K_BYTES = 292;

// the two lookup tables live in global memory, as the reference passes them to every launch as device slices
__device__ const uint64_t g_grid[256] = {DSMOE_IQ2XXS_GRID_VALUES};
__device__ uint8_t g_signs[128];

__global__ void fill_signs_kernel()
{
    if (threadIdx.x < 128) g_signs[threadIdx.x] = (uint8_t)dsmoe_iq2_sign_byte(threadIdx.x);
}

__device__ __forceinline__ uint32_t rd16(const uint8_t *p) { return (uint32_t)p[0] | ((uint32_t)p[1] << 8); }
__device__ __forceinline__ float rdf32(const uint8_t *p)
{
    return __uint_as_float((uint32_t)p[0] | ((uint32_t)p[1] << 8) | ((uint32_t)p[2] << 16) | ((uint32_t)p[3] << 24));
}
__device__ __forceinline__ int rdi16(const uint8_t *p) { return (int)(int16_t)(uint16_t)rd16(p); }

// f16 bits -> f32, subnormal inputs give zero
__device__ __forceinline__ float half_bits(uint32_t h)
{
    const uint32_t sign = (h & 0x8000u) << 16, ex = (h >> 10) & 31u, man = h & 0x3FFu;
    if (ex == 0) return __uint_as_float(sign);
    if (ex == 31) return __uint_as_float(sign | 0x7F800000u | (man << 13));
    return __uint_as_float(sign | ((ex + 112u) << 23) | (man << 13));
}

// eight codebook magnitudes (bytes of g) with sign bits s against eight int8 activations, one element at a time
__device__ __forceinline__ int dot8_signed(uint64_t g, uint32_t s, const int8_t *q)
{
    int acc = 0;
    for (int j = 0; j < 8; ++j) {
        const int mag = (int)((g >> (8 * j)) & 0xFFu);
        acc += ((s >> j) & 1u) ? -mag * (int)q[j] : mag * (int)q[j];
    }
    return acc;
}

__device__ float dot_iq2xxs(const uint8_t *w, const uint8_t *a)
{
    const float dw = half_bits(rd16(w)), da = rdf32(a);
    const int8_t *q = reinterpret_cast<const int8_t *>(a + 4);
    int total = 0;
    for (int grp = 0; grp < 8; ++grp) {
        const uint8_t *p = w + 2 + 8 * grp;
        const uint32_t lo = rd16(p) | (rd16(p + 2) << 16), hi = rd16(p + 4) | (rd16(p + 6) << 16);
        const int scale = (int)(2u * (hi >> 28) + 1u);
        int part = 0;
        for (int u = 0; u < 4; ++u)
            part += dot8_signed(g_grid[(lo >> (8 * u)) & 255u], g_signs[(hi >> (7 * u)) & 127u], q + 32 * grp + 8 * u);
        total += part * scale;
    }
    return __fmul_rn(__fmul_rn(__fmul_rn(0.125f, dw), da), (float)total);
}

__device__ __forceinline__ int dot16_2bit(const uint8_t *q2, const int8_t *q8, int shift)
{
    int acc = 0;
    for (int i = 0; i < 16; ++i) acc += (int)((q2[i] >> shift) & 3u) * (int)q8[i];
    return acc;
}

__device__ float dot_q2k(const uint8_t *w, const uint8_t *a)
{
    const float da = rdf32(a);
    const float dall = __fmul_rn(da, half_bits(rd16(w + 80))), dmin = __fmul_rn(da, half_bits(rd16(w + 82)));
    const int8_t *q8 = reinterpret_cast<const int8_t *>(a + 4);
    int mins = 0;
    for (int j = 0; j < 16; ++j) mins += rdi16(a + 260 + 2 * j) * (int)(w[j] >> 4);
    int isum = 0, sub = 0;
    for (int half = 0; half < 2; ++half)
        for (int f = 0; f < 4; ++f) {
            const uint8_t *q2 = w + 16 + 32 * half;
            const int8_t *x = q8 + 128 * half + 32 * f;
            isum += (int)(w[sub] & 15u) * dot16_2bit(q2, x, 2 * f);
            isum += (int)(w[sub + 1] & 15u) * dot16_2bit(q2 + 16, x + 16, 2 * f);
            sub += 2;
        }
    return __fsub_rn(__fmul_rn(dall, (float)isum), __fmul_rn(dmin, (float)mins));
}

__device__ __forceinline__ float sum8(float v)
{
    v = __fadd_rn(v, __shfl_xor_sync(0xFFFFFFFFu, v, 4));
    v = __fadd_rn(v, __shfl_xor_sync(0xFFFFFFFFu, v, 2));
    v = __fadd_rn(v, __shfl_xor_sync(0xFFFFFFFFu, v, 1));
    return v;
}

// grid (in_dim / 256, n_rows), 256 threads: one CTA per block of one row
__global__ void __launch_bounds__(256) q8k_quantize_kernel(const float *x, uint8_t *out, uint32_t in_dim, uint32_t n_rows)
{
    __shared__ float s_abs[256], s_val[256];
    const uint32_t blk = blockIdx.x, row = blockIdx.y, n_blocks = in_dim / 256, t = threadIdx.x;
    if (row >= n_rows || blk >= n_blocks) return;
    const float *src = x + (size_t)row * in_dim + (size_t)blk * 256;
    const float v = src[t];
    s_abs[t] = v < 0.0f ? -v : v;
    s_val[t] = v;
    __syncthreads();
    for (uint32_t stride = 128; stride > 0; stride >>= 1) {
        if (t < stride && s_abs[t + stride] > s_abs[t]) {
            s_abs[t] = s_abs[t + stride];
            s_val[t] = s_val[t + stride];
        }
        __syncthreads();
    }
    uint8_t *dst = out + ((size_t)row * n_blocks + blk) * Q8K_BYTES;
    if (s_abs[0] == 0.0f) {
        if (t == 0) *reinterpret_cast<float *>(dst) = 0.0f;
        dst[4 + t] = 0;
        if (t < 16) *reinterpret_cast<int16_t *>(dst + 260 + 2 * t) = 0;
        return;
    }
    const float inv = __fdiv_rn(-127.0f, s_val[0]);
    if (t == 0) *reinterpret_cast<float *>(dst) = __fdiv_rn(1.0f, inv);
    __syncthreads();
    const float scaled = __fmul_rn(inv, src[t]);
    int q = scaled >= 0.0f ? (int)__fadd_rn(scaled, 0.5f) : (int)__fsub_rn(scaled, 0.5f);
    q = q > 127 ? 127 : (q < -128 ? -128 : q);
    reinterpret_cast<int8_t *>(dst + 4)[t] = (int8_t)q;
    __syncthreads();
    if (t < 16) {
        int s = 0;
        for (int k = 0; k < 16; ++k) s += (int)reinterpret_cast<const int8_t *>(dst + 4)[16 * t + k];
        *reinterpret_cast<int16_t *>(dst + 260 + 2 * t) = (int16_t)s;
    }
}

// grid (ceil(mid_dim / 128), n_tokens * k), 256 threads: quarter-warp per row, rows r, r+32, r+64, r+96 of the CTA's 128
__global__ void __launch_bounds__(256) gate_up_mid_kernel(const uint8_t *gate, const uint8_t *up, const uint8_t *xq,
                                                           const int32_t *selected, const float *weights, float *gate_out,
                                                           float *up_out, float *mid_out, uint64_t expert_bytes,
                                                           uint64_t row_bytes, uint32_t xq_blocks, uint32_t mid_dim,
                                                           uint32_t k, float clamp, const uint32_t *sorted_pairs)
{
    // sorted_pairs != null: moe_gate_up_mid_sorted_qwarp32 (moe.rs:721), which differs only in where the pair id comes from
    const uint32_t lane = threadIdx.x & 7, rlane = threadIdx.x >> 3, pair = sorted_pairs ? sorted_pairs[blockIdx.y] : blockIdx.y;
    const uint32_t tok = pair / k;
    const int32_t e = selected[pair];
    const uint64_t expert = e < 0 ? 0u : (uint64_t)e;
    const uint8_t *act = xq + (size_t)tok * xq_blocks * Q8K_BYTES;
    for (uint32_t rr = 0; rr < 4; ++rr) {
        const uint32_t row = blockIdx.x * 128 + rlane + 32 * rr;
        if (row >= mid_dim) continue;
        const size_t off = expert * expert_bytes + (size_t)row * row_bytes;
        float g = 0.0f, u = 0.0f;
        for (uint32_t b = lane; b < xq_blocks; b += 8) {
            g = __fadd_rn(g, dot_iq2xxs(gate + off + (size_t)b * IQ2_BYTES, act + (size_t)b * Q8K_BYTES));
            u = __fadd_rn(u, dot_iq2xxs(up + off + (size_t)b * IQ2_BYTES, act + (size_t)b * Q8K_BYTES));
        }
        g = sum8(g);
        u = sum8(u);
        if (lane == 0) {
            if (clamp > 1.0e-6f) {
                if (g > clamp) g = clamp;
                if (u > clamp) u = clamp;
                if (u < -clamp) u = -clamp;
            }
            const size_t o = (size_t)pair * mid_dim + row;
            if (gate_out) gate_out[o] = g;
            if (up_out) up_out[o] = u;
            // exp as a correctly rounded f32 operation, the definition the oracle and the product share
            const float ex = (float)exp((double)-g);
            mid_out[o] = __fmul_rn(__fmul_rn(__fdiv_rn(g, __fadd_rn(1.0f, ex)), u), weights[pair]);
        }
    }
}

// grid (ceil(out_dim / 32)), 256 threads: quarter-warp per output row, the token's 6 slots one after the other
__global__ void __launch_bounds__(256) down_sum6_kernel(const uint8_t *down, const uint8_t *midq, const int32_t *selected,
                                                         float *out, uint64_t expert_bytes, uint64_t row_bytes,
                                                         uint32_t midq_blocks, uint32_t out_dim)
{
    const uint32_t lane = threadIdx.x & 7, row = blockIdx.x * 32 + (threadIdx.x >> 3);
    if (row >= out_dim) return;
    float total = 0.0f;
    for (uint32_t slot = 0; slot < 6; ++slot) {
        const int32_t e = selected[slot];
        const size_t off = (e < 0 ? 0u : (uint64_t)e) * expert_bytes + (size_t)row * row_bytes;
        const uint8_t *act = midq + (size_t)slot * midq_blocks * Q8K_BYTES;
        float acc = 0.0f;
        for (uint32_t b = lane; b < midq_blocks; b += 8)
            acc = __fadd_rn(acc, dot_q2k(down + off + (size_t)b * Q2K_BYTES, act + (size_t)b * Q8K_BYTES));
        acc = sum8(acc);
        if (lane == 0) total = __fadd_rn(total, acc);
    }
    if (lane == 0) out[row] = total;
}

// ---- the batched form (engine/src/kernels/moe.rs:299-362, 871-916, 983-1005) -----------------------------------
__global__ void count_sorted_pairs_kernel(const int32_t *selected, uint32_t *counts, uint32_t pair_count)
{
    const uint32_t pair = blockIdx.x * blockDim.x + threadIdx.x;
    if (pair >= pair_count) return;
    const int32_t e = selected[pair];
    atomicAdd(&counts[e < 0 ? 0 : e], 1u);
}

__global__ void prefix_sorted_pairs_kernel(const uint32_t *counts, uint32_t *offsets, uint32_t *cursors)
{
    if (threadIdx.x != 0) return;
    uint32_t sum = 0;
    for (int e = 0; e < 256; ++e) {
        offsets[e] = sum;
        cursors[e] = sum;
        sum += counts[e];
    }
    offsets[256] = sum;
}

__global__ void scatter_sorted_pairs_kernel(const int32_t *selected, uint32_t *cursors, uint32_t *sorted_pairs, uint32_t pair_count)
{
    const uint32_t pair = blockIdx.x * blockDim.x + threadIdx.x;
    if (pair >= pair_count) return;
    const int32_t e = selected[pair];
    sorted_pairs[atomicAdd(&cursors[e < 0 ? 0 : e], 1u)] = pair;
}

// grid (ceil(out_dim / 32), n_pairs), 256 threads: quarter-warp per output row of one pair
__global__ void __launch_bounds__(256) down_sorted_kernel(const uint8_t *down, const uint8_t *midq, const uint32_t *sorted_pairs,
                                                           const int32_t *selected, float *down_out, uint64_t expert_bytes,
                                                           uint64_t row_bytes, uint32_t midq_blocks, uint32_t out_dim)
{
    const uint32_t lane = threadIdx.x & 7, row = blockIdx.x * 32 + (threadIdx.x >> 3);
    if (row >= out_dim) return;
    const uint32_t pair = sorted_pairs[blockIdx.y];
    const int32_t e = selected[pair];
    const size_t off = (e < 0 ? 0u : (uint64_t)e) * expert_bytes + (size_t)row * row_bytes;
    const uint8_t *act = midq + (size_t)pair * midq_blocks * Q8K_BYTES;
    float acc = 0.0f;
    for (uint32_t b = lane; b < midq_blocks; b += 8)
        acc = __fadd_rn(acc, dot_q2k(down + off + (size_t)b * Q2K_BYTES, act + (size_t)b * Q8K_BYTES));
    acc = sum8(acc);
    if (lane == 0) down_out[(size_t)pair * out_dim + row] = acc;
}

// moe_sum (moe.rs:983-1005): one thread per (token, row), slots added in slot order
__global__ void __launch_bounds__(256) moe_sum_kernel(const float *down, float *out, uint32_t out_dim, uint32_t k, uint64_t n)
{
    const uint64_t gid = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (gid >= n) return;
    const uint64_t tok = gid / out_dim, row = gid - tok * out_dim;
    float acc = 0.0f;
    for (uint32_t slot = 0; slot < k; ++slot) acc = __fadd_rn(acc, down[(tok * k + slot) * out_dim + row]);
    out[gid] = acc;
}

}  // namespace refmap

#define REFMAP_API extern "C" __attribute__((visibility("default")))

REFMAP_API int refmap_init(void *stream)
{
    refmap::fill_signs_kernel<<<1, 128, 0, (cudaStream_t)stream>>>();
    return (int)cudaGetLastError();
}

REFMAP_API int refmap_q8k_quantize(void *stream, const float *x, uint8_t *out, uint32_t in_dim, uint32_t n_rows)
{
    if (n_rows == 0 || in_dim < 256) return 0;
    refmap::q8k_quantize_kernel<<<dim3(in_dim / 256, n_rows), 256, 0, (cudaStream_t)stream>>>(x, out, in_dim, n_rows);
    return (int)cudaGetLastError();
}

REFMAP_API int refmap_gate_up_mid(void *stream, const uint8_t *gate, const uint8_t *up, const uint8_t *xq,
                                  const int32_t *selected, const float *weights, float *gate_out, float *up_out,
                                  float *mid_out, uint64_t expert_bytes, uint64_t row_bytes, uint32_t xq_blocks,
                                  uint32_t mid_dim, uint32_t k, uint32_t n_tokens, float clamp)
{
    if (n_tokens == 0) return 0;
    refmap::gate_up_mid_kernel<<<dim3((mid_dim + 127) / 128, n_tokens * k), 256, 0, (cudaStream_t)stream>>>(
        gate, up, xq, selected, weights, gate_out, up_out, mid_out, expert_bytes, row_bytes, xq_blocks, mid_dim, k, clamp, nullptr);
    return (int)cudaGetLastError();
}

REFMAP_API int refmap_down_sum6(void *stream, const uint8_t *down, const uint8_t *midq, const int32_t *selected, float *out,
                                uint64_t expert_bytes, uint64_t row_bytes, uint32_t midq_blocks, uint32_t out_dim)
{
    refmap::down_sum6_kernel<<<(out_dim + 31) / 32, 256, 0, (cudaStream_t)stream>>>(down, midq, selected, out, expert_bytes,
                                                                                     row_bytes, midq_blocks, out_dim);
    return (int)cudaGetLastError();
}

// The routed-expert part of the reference's per-token FFN (engine/src/session.rs:2062-2153), for n_tokens tokens one
// after the other as its prefill does (engine/src/session.rs:795-895): Q8_K of x, gate/up/mid, Q8_K of mid, down + sum.
// selected / weights: [n_tokens][6] from a router run beforehand. xq, mid, midq: scratch for ONE token.
REFMAP_API int refmap_tokens(void *stream, const uint8_t *gate, const uint8_t *up, const uint8_t *down, const float *x,
                             const int32_t *selected, const float *weights, uint8_t *xq, float *mid, uint8_t *midq,
                             float *out, uint32_t n_embd, uint32_t n_ff, uint32_t n_tokens, float clamp)
{
    const uint32_t xb = n_embd / 256, mb = n_ff / 256;
    for (uint32_t t = 0; t < n_tokens; ++t) {
        refmap_q8k_quantize(stream, x + (size_t)t * n_embd, xq, n_embd, 1);
        refmap_gate_up_mid(stream, gate, up, xq, selected + 6 * t, weights + 6 * t, nullptr, nullptr, mid,
                           (uint64_t)n_ff * xb * refmap::IQ2_BYTES, (uint64_t)xb * refmap::IQ2_BYTES, xb, n_ff, 6, 1, clamp);
        refmap_q8k_quantize(stream, mid, midq, n_ff, 6);
        refmap_down_sum6(stream, down, midq, selected + 6 * t, out + (size_t)t * n_embd,
                         (uint64_t)n_embd * mb * refmap::Q2K_BYTES, (uint64_t)mb * refmap::Q2K_BYTES, mb, n_embd);
    }
    return (int)cudaGetLastError();
}

// The batched form for one chunk of n_tokens tokens: pairs counted, prefixed and scattered into expert order, then one
// launch each of Q8_K(x), sorted gate/up/mid, Q8_K(mid), sorted down and the slot sum. Scratch (device): xq
// [n_tokens][n_embd/256][292], mid f32 [n_tokens*6][n_ff], midq [n_tokens*6][n_ff/256][292], down_rows f32
// [n_tokens*6][n_embd], idx u32 [257 + 257 + 256 + n_tokens*6] (counts, offsets, cursors, sorted pairs).
REFMAP_API int refmap_batched(void *stream, const uint8_t *gate, const uint8_t *up, const uint8_t *down, const float *x,
                              const int32_t *selected, const float *weights, uint8_t *xq, float *mid, uint8_t *midq,
                              float *down_rows, uint32_t *idx, float *out, uint32_t n_embd, uint32_t n_ff, uint32_t n_tokens,
                              float clamp)
{
    if (n_tokens == 0) return 0;
    cudaStream_t st = (cudaStream_t)stream;
    const uint32_t xb = n_embd / 256, mb = n_ff / 256, k = 6, P = n_tokens * k;
    uint32_t *counts = idx, *offsets = idx + 257, *cursors = idx + 514, *sorted = idx + 770;
    cudaMemsetAsync(counts, 0, 257 * sizeof(uint32_t), st);
    refmap::count_sorted_pairs_kernel<<<(P + 255) / 256, 256, 0, st>>>(selected, counts, P);
    refmap::prefix_sorted_pairs_kernel<<<1, 1, 0, st>>>(counts, offsets, cursors);
    refmap::scatter_sorted_pairs_kernel<<<(P + 255) / 256, 256, 0, st>>>(selected, cursors, sorted, P);
    refmap_q8k_quantize(stream, x, xq, n_embd, n_tokens);
    refmap::gate_up_mid_kernel<<<dim3((n_ff + 127) / 128, P), 256, 0, st>>>(
        gate, up, xq, selected, weights, nullptr, nullptr, mid, (uint64_t)n_ff * xb * refmap::IQ2_BYTES,
        (uint64_t)xb * refmap::IQ2_BYTES, xb, n_ff, k, clamp, sorted);
    refmap_q8k_quantize(stream, mid, midq, n_ff, P);
    refmap::down_sorted_kernel<<<dim3((n_embd + 31) / 32, P), 256, 0, st>>>(down, midq, sorted, selected, down_rows,
                                                                             (uint64_t)n_embd * mb * refmap::Q2K_BYTES,
                                                                             (uint64_t)mb * refmap::Q2K_BYTES, mb, n_embd);
    const uint64_t n = (uint64_t)n_tokens * n_embd;
    refmap::moe_sum_kernel<<<(unsigned)((n + 255) / 256), 256, 0, st>>>(down_rows, out, n_embd, k, n);
    return (int)cudaGetLastError();
}
