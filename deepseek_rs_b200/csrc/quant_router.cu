// Q8_K activation quantiser, router top-k, dequantisers, upload-time re-layout and the slot sum.
#include "async.cuh"
#include "common.cuh"
#include "launch.h"
#include "q8k.cuh"

namespace dsmoe {

// ---------------------------------------------------------------------------------------------------------------
// Q8_K quantiser: one warp per 256-element block, lane l owns elements 8l..8l+7.
//
// Result is bit-identical to the reference kernel (engine/src/kernels/quantize.rs:309-417). Its shared-memory
// halving tree keeps the lower slot on equal magnitudes, level by level from stride 128 down to 1, so among equal
// maxima the element with the smallest bit-reversed index wins; using (|x|, bit-reversed index) as the reduction key
// reproduces that choice (and hence the sign of d) in any reduction order.
// ---------------------------------------------------------------------------------------------------------------
__device__ __forceinline__ void q8k_quantize_block(const float *__restrict__ xb, uint8_t *__restrict__ yb, int lane)
{
    const float4 *src = reinterpret_cast<const float4 *>(xb + 8 * lane);
    const float4 v0 = src[0], v1 = src[1];
    const float v[8] = {v0.x, v0.y, v0.z, v0.w, v1.x, v1.y, v1.z, v1.w};
    q8k_quantize_vals(v, yb, lane);
}

// The batched path's step between its two grouped GEMMs: the gate and up row totals become mid = silu(gate) * up * w with
// the reference's clamps and operation order (engine/src/kernels/moe.rs:692-710), and mid is quantised to Q8_K in the
// same warp without ever being stored as f32. One warp per 256-element block.
__global__ void __launch_bounds__(256) swiglu_q8k_kernel(const float *__restrict__ gate, const float *__restrict__ up,
                                                          const float *__restrict__ weight, uint8_t *__restrict__ out,
                                                          uint32_t blocks_per_row, uint64_t n_blocks_total, float clamp)
{
    const int lane = threadIdx.x & 31;
    const uint64_t blk = (uint64_t)blockIdx.x * 8 + (threadIdx.x >> 5);
    if (blk >= n_blocks_total) return;
    const uint64_t row = blk / blocks_per_row;
    const float w = weight[row];
    const float4 *gs = reinterpret_cast<const float4 *>(gate + blk * QK_K + 8 * lane);
    const float4 *us = reinterpret_cast<const float4 *>(up + blk * QK_K + 8 * lane);
    const float4 g0 = gs[0], g1 = gs[1], u0 = us[0], u1 = us[1];
    const float g[8] = {g0.x, g0.y, g0.z, g0.w, g1.x, g1.y, g1.z, g1.w}, u[8] = {u0.x, u0.y, u0.z, u0.w, u1.x, u1.y, u1.z, u1.w};
    float v[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        float gg = g[i], uu = u[i];
        if (clamp > 1.0e-6f) {
            if (gg > clamp) gg = clamp;
            if (uu > clamp) uu = clamp;
            if (uu < -clamp) uu = -clamp;
        }
        v[i] = swiglu_weighted(gg, uu, w);
    }
    q8k_quantize_vals(v, out + blk * Q8K_BYTES, lane);
}

void launch_swiglu_q8k(cudaStream_t st, const float *gate, const float *up, const float *weight, uint8_t *out,
                       uint32_t in_dim, uint32_t n_rows, float clamp)
{
    const uint64_t nb = (uint64_t)(in_dim / QK_K) * n_rows;
    if (nb == 0) return;
    swiglu_q8k_kernel<<<(unsigned)((nb + 7) / 8), 256, 0, st>>>(gate, up, weight, out, in_dim / QK_K, nb, clamp);
}

__global__ void __launch_bounds__(256) q8k_quantize_kernel(const float *__restrict__ x, uint8_t *__restrict__ out,
                                                            uint64_t n_blocks_total)
{
    const int lane = threadIdx.x & 31;
    const uint64_t blk = (uint64_t)blockIdx.x * 8 + (threadIdx.x >> 5);
    pdl_launch_dependents();
    pdl_wait();
    if (blk >= n_blocks_total) return;
    q8k_quantize_block(x + blk * QK_K, out + blk * Q8K_BYTES, lane);
}

void launch_q8k_quantize(cudaStream_t st, const float *x, uint8_t *out, uint32_t in_dim, uint32_t n_rows)
{
    uint64_t nb = (uint64_t)(in_dim / QK_K) * n_rows;
    if (nb == 0) return;
    launch_pdl(q8k_quantize_kernel, dim3((unsigned)((nb + 7) / 8)), dim3(256), 0, st, x, out, nb);
}

// ---------------------------------------------------------------------------------------------------------------
// Router: one warp per token. probs = sqrt(softplus(logit)); k rounds of warp arg-max with the reference's order
// (higher score first, lower index on equal scores), which yields the same list as its insertion scan
// (engine/src/kernels/moe.rs:239-263). Scores that are not greater than -inf (NaN, -inf) are never selected, as in
// the reference, and leave -1 in the list.
// ---------------------------------------------------------------------------------------------------------------
constexpr int ROUTER_MAX_PER_LANE = 16;  // up to 512 experts

__global__ void __launch_bounds__(128) router_select_kernel(const float *__restrict__ logits,
                                                             const float *__restrict__ bias,
                                                             const int32_t *__restrict__ hash,
                                                             const int32_t *__restrict__ tokens,
                                                             float *__restrict__ probs, int32_t *__restrict__ selected,
                                                             float *__restrict__ weights, int32_t token_scalar,
                                                             uint32_t hash_rows, uint32_t n_tokens, int has_bias,
                                                             int hash_mode, int k, int n_expert, float route_scale)
{
    const int lane = threadIdx.x & 31;
    const uint32_t t = blockIdx.x * 4 + (threadIdx.x >> 5);
    if (t >= n_tokens) return;
    const int per_lane = n_expert >> 5;
    float p[ROUTER_MAX_PER_LANE], sc[ROUTER_MAX_PER_LANE];
#pragma unroll
    for (int j = 0; j < ROUTER_MAX_PER_LANE; ++j) {
        p[j] = 0.0f;
        sc[j] = -INFINITY;
        if (j < per_lane) {
            int e = lane + 32 * j;
            float pe = sqrtf(softplus_ref(logits[(size_t)t * n_expert + e]));
            p[j] = pe;
            sc[j] = has_bias ? __fadd_rn(pe, bias[e]) : pe;
            probs[(size_t)t * n_expert + e] = pe;
        }
    }

    int sel_mine = -1;     // lane j keeps the j-th selection
    float w_mine = 0.0f;   // and its un-biased probability
    if (hash_mode) {
        int32_t raw = tokens ? tokens[t] : token_scalar;
        size_t tok = (raw < 0 || (uint32_t)raw >= hash_rows) ? 0 : (size_t)raw;
        if (lane < k) sel_mine = hash[tok * k + lane];
        // fetch the probability of an arbitrary expert id from the lane that owns it
        for (int j = 0; j < k; ++j) {
            int e = __shfl_sync(FULL, sel_mine, j);
            bool ok = e >= 0 && e < n_expert;
            int owner = ok ? (e & 31) : 0, slot = ok ? (e >> 5) : 0;
            float mine = 0.0f;
#pragma unroll
            for (int q = 0; q < ROUTER_MAX_PER_LANE; ++q)
                if (q == slot) mine = p[q];
            float pv = __shfl_sync(FULL, mine, owner);
            if (lane == j) w_mine = ok ? pv : 0.0f;
        }
    } else {
        for (int r = 0; r < k; ++r) {
            float bs = -INFINITY, bp = 0.0f;
            int bi = -1;
#pragma unroll
            for (int j = 0; j < ROUTER_MAX_PER_LANE; ++j)
                if (j < per_lane && sc[j] > -INFINITY) {
                    int e = lane + 32 * j;
                    if (bi < 0 || sc[j] > bs) {  // ascending e within the lane: strict > keeps the lower index
                        bs = sc[j];
                        bp = p[j];
                        bi = e;
                    }
                }
#pragma unroll
            for (int m = 16; m > 0; m >>= 1) {
                float os = __shfl_xor_sync(FULL, bs, m);
                float op = __shfl_xor_sync(FULL, bp, m);
                int oi = __shfl_xor_sync(FULL, bi, m);
                bool take = oi >= 0 && (bi < 0 || os > bs || (os == bs && oi < bi));
                if (take) {
                    bs = os;
                    bp = op;
                    bi = oi;
                }
            }
            if (bi >= 0 && (bi & 31) == lane) {
#pragma unroll
                for (int j = 0; j < ROUTER_MAX_PER_LANE; ++j)
                    if (j == (bi >> 5)) sc[j] = -INFINITY;
            }
            if (lane == r) {
                sel_mine = bi;
                w_mine = bi >= 0 ? bp : 0.0f;
            }
        }
    }
    // sum in slot order, floor at 2^-14, w /= (sum / route_scale)   (engine/src/kernels/moe.rs:266-286)
    float sum = 0.0f;
    for (int j = 0; j < k; ++j) sum = __fadd_rn(sum, __shfl_sync(FULL, w_mine, j));
    if (sum < 6.103515625e-5f) sum = 6.103515625e-5f;
    float div = __fdiv_rn(sum, route_scale);
    if (lane < k) {
        selected[(size_t)t * k + lane] = sel_mine;
        weights[(size_t)t * k + lane] = __fdiv_rn(w_mine, div);
    }
}

void launch_router_select(cudaStream_t st, const float *logits, const float *bias, const int32_t *hash,
                          const int32_t *tokens, float *probs, int32_t *selected, float *weights, int32_t token_scalar,
                          uint32_t hash_rows, uint32_t n_tokens, int has_bias, int hash_mode, int k, int n_expert,
                          float route_scale)
{
    if (n_tokens == 0) return;
    router_select_kernel<<<(n_tokens + 3) / 4, 128, 0, st>>>(logits, bias, hash, tokens, probs, selected, weights,
                                                             token_scalar, hash_rows, n_tokens, has_bias, hash_mode, k,
                                                             n_expert, route_scale);
}

// ---------------------------------------------------------------------------------------------------------------
// Router and Q8_K of the same token in one launch (no bias, no hash table): per token one 256-thread CTA routes, one
// expert per thread, so the double-precision exp/ln of all experts run side by side, and the CTAs beside it
// (blockIdx.y = 1 ..) quantise the token's hidden row, one block per warp, at the same time. Same results as
// router_select_kernel + q8k_quantize_kernel.
// Selection key: order-preserving integer image of the score in the high word, inverted expert index in the low
// word, so an integer maximum picks the highest score and, among equals, the lowest index; key 0 = not selectable.
// ---------------------------------------------------------------------------------------------------------------
__device__ __forceinline__ unsigned long long router_key(float score, int e)
{
    if (!(score > -INFINITY)) return 0ull;
    uint32_t b = __float_as_uint(score);
    b = (b & 0x80000000u) ? ~b : (b | 0x80000000u);
    return ((unsigned long long)b << 32) | (uint32_t)(0xFFFFFFFFu - (uint32_t)e);
}

__global__ void __launch_bounds__(256) router_q8k_fused_kernel(const float *__restrict__ logits,
                                                                const float *__restrict__ x, float *__restrict__ probs,
                                                                int32_t *__restrict__ selected, float *__restrict__ weights,
                                                                uint8_t *__restrict__ xq, int k, int n_expert,
                                                                uint32_t n_embd, float route_scale)
{
    __shared__ unsigned long long s_warp_best[8];
    __shared__ float s_w[MAX_K];
    __shared__ int s_sel[MAX_K];
    pdl_launch_dependents();  // the expert kernel behind this one may set up its tables meanwhile
    pdl_wait();
    const uint32_t t = blockIdx.x;
    const int e = threadIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if (blockIdx.y > 0) {  // CTAs 1.. of a token quantise its row, eight blocks each, beside CTA 0's routing
        const uint32_t n_blocks = n_embd / QK_K, b = (blockIdx.y - 1) * 8 + warp;
        if (b < n_blocks)
            q8k_quantize_block(x + (size_t)t * n_embd + (size_t)b * QK_K, xq + ((size_t)t * n_blocks + b) * Q8K_BYTES, lane);
        return;
    }
    float p = 0.0f;
    unsigned long long key = 0ull;
    if (e < n_expert) {
        p = sqrtf(softplus_ref(logits[(size_t)t * n_expert + e]));
        probs[(size_t)t * n_expert + e] = p;
        key = router_key(p, e);
    }
    for (int r = 0; r < k; ++r) {
        unsigned long long best = key;
#pragma unroll
        for (int m = 16; m > 0; m >>= 1) {
            unsigned long long o = __shfl_xor_sync(FULL, best, m);
            best = o > best ? o : best;
        }
        if (lane == 0) s_warp_best[warp] = best;
        __syncthreads();
        unsigned long long top = s_warp_best[0];
#pragma unroll
        for (int w = 1; w < 8; ++w) top = s_warp_best[w] > top ? s_warp_best[w] : top;
        if (top == 0ull) {
            if (e == 0) {
                s_sel[r] = -1;
                s_w[r] = 0.0f;
            }
        } else if (key == top) {
            s_sel[r] = e;
            s_w[r] = p;
            key = 0ull;  // taken
        }
        __syncthreads();
    }
    if (e == 0) {
        float sum = 0.0f;
        for (int j = 0; j < k; ++j) sum = __fadd_rn(sum, s_w[j]);
        if (sum < 6.103515625e-5f) sum = 6.103515625e-5f;
        const float div = __fdiv_rn(sum, route_scale);
        for (int j = 0; j < k; ++j) {
            selected[(size_t)t * k + j] = s_sel[j];
            weights[(size_t)t * k + j] = __fdiv_rn(s_w[j], div);
        }
    }
}

void launch_router_q8k_fused(cudaStream_t st, const float *logits, const float *x, float *probs, int32_t *selected,
                             float *weights, uint8_t *xq, uint32_t n_tokens, int k, int n_expert, uint32_t n_embd,
                             float route_scale)
{
    if (n_tokens == 0) return;
    const unsigned q_ctas = (n_embd / QK_K + 7) / 8;
    router_q8k_fused_kernel<<<dim3(n_tokens, 1 + q_ctas), 256, 0, st>>>(logits, x, probs, selected, weights, xq, k, n_expert,
                                                                        n_embd, route_scale);
}

// ---------------------------------------------------------------------------------------------------------------
// Dequantisers (NATIVE block order). One thread per 8 weights.
// ---------------------------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256) dequant_iq2xxs_kernel(const uint8_t *__restrict__ blocks, uint64_t n_units,
                                                              float *__restrict__ out, int ieee)
{
    uint64_t u = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;  // unit = (block, ib32, k)
    if (u >= n_units) return;
    uint64_t b = u >> 5;
    int ib32 = (int)(u >> 2) & 7, k = (int)u & 3;
    const uint8_t *blk = blocks + b * IQ2XXS_BYTES;
    const uint16_t *q2 = reinterpret_cast<const uint16_t *>(blk + 2 + 8 * ib32);
    uint32_t aux0 = (uint32_t)q2[0] | ((uint32_t)q2[1] << 16);
    uint32_t aux1 = (uint32_t)q2[2] | ((uint32_t)q2[3] << 16);
    float d = __fmul_rn(0.125f, f16_bits_to_f32(ld_u16(blk), ieee != 0));
    int ls = (int)(2u * (aux1 >> 28) + 1u);
    uint64_t g = c_iq2xxs_grid[(aux0 >> (8 * k)) & 255u];
    uint32_t sb = dsmoe_iq2_sign_byte((aux1 >> (7 * k)) & 127u);
    float *o = out + b * QK_K + 32 * ib32 + 8 * k;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        int mag = (int)((g >> (8 * j)) & 0xFFu);
        int code = ls * (((sb >> j) & 1u) ? -mag : mag);
        o[j] = __fmul_rn(d, (float)code);
    }
}

__global__ void __launch_bounds__(256) dequant_q2k_kernel(const uint8_t *__restrict__ blocks, uint64_t n_elems,
                                                           float *__restrict__ out, int ieee)
{
    uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n_elems) return;
    uint64_t b = i >> 8;
    int e = (int)i & 255, h = e >> 7, j = (e >> 5) & 3, ii = e & 31;
    const uint8_t *blk = blocks + b * Q2K_BYTES;
    int sb = 8 * h + 2 * j + (ii >> 4);
    int q = (blk[16 + 32 * h + ii] >> (2 * j)) & 3;
    float d = f16_bits_to_f32(ld_u16(blk + 80), ieee != 0), dmin = f16_bits_to_f32(ld_u16(blk + 82), ieee != 0);
    float a = __fmul_rn(d, (float)((blk[sb] & 0x0F) * q));
    float m = __fmul_rn(dmin, (float)(blk[sb] >> 4));
    out[i] = __fsub_rn(a, m);
}

void launch_dequant_iq2xxs(cudaStream_t st, const uint8_t *blocks, uint64_t n_blocks, float *out, int ieee)
{
    uint64_t units = n_blocks * 32;
    if (units == 0) return;
    dequant_iq2xxs_kernel<<<(unsigned)((units + 255) / 256), 256, 0, st>>>(blocks, units, out, ieee);
}

void launch_dequant_q2k(cudaStream_t st, const uint8_t *blocks, uint64_t n_blocks, float *out, int ieee)
{
    uint64_t n = n_blocks * QK_K;
    if (n == 0) return;
    dequant_q2k_kernel<<<(unsigned)((n + 255) / 256), 256, 0, st>>>(blocks, n, out, ieee);
}

// ---------------------------------------------------------------------------------------------------------------
// Row re-layout NATIVE <-> ROWSOA: a byte permutation inside each row, done once at upload.
// IQ2_XXS rows move in 2-byte units (33 per block), Q2_K rows in 4-byte units (21 per block).
// ---------------------------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256) relayout_iq2xxs_kernel(const uint16_t *__restrict__ src,
                                                               uint16_t *__restrict__ dst, uint64_t n_rows, uint32_t xb,
                                                               int inverse)
{
    const uint64_t per_row = 33ull * xb, total = n_rows * per_row;
    for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (uint64_t)gridDim.x * blockDim.x) {
        uint64_t row = i / per_row;
        uint32_t s = (uint32_t)(i - row * per_row);  // position in ROWSOA order
        uint32_t n = s < xb ? 33u * s : 33u * ((s - xb) >> 5) + 1u + ((s - xb) & 31u);  // position in NATIVE order
        if (inverse) dst[row * per_row + n] = src[row * per_row + s];
        else dst[row * per_row + s] = src[row * per_row + n];
    }
}

__global__ void __launch_bounds__(256) relayout_q2k_kernel(const uint32_t *__restrict__ src, uint32_t *__restrict__ dst,
                                                            uint64_t n_rows, uint32_t mb, int inverse)
{
    const uint64_t per_row = 21ull * mb, total = n_rows * per_row;
    for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (uint64_t)gridDim.x * blockDim.x) {
        uint64_t row = i / per_row;
        uint32_t s = (uint32_t)(i - row * per_row), n;
        if (s < 4u * mb) n = 21u * (s >> 2) + (s & 3u);
        else if (s < 20u * mb) n = 21u * ((s - 4u * mb) >> 4) + 4u + ((s - 4u * mb) & 15u);
        else n = 21u * (s - 20u * mb) + 20u;
        if (inverse) dst[row * per_row + n] = src[row * per_row + s];
        else dst[row * per_row + s] = src[row * per_row + n];
    }
}

void launch_relayout_iq2xxs(cudaStream_t st, const uint8_t *src, uint8_t *dst, uint64_t n_rows, uint32_t xb, int inverse)
{
    uint64_t total = n_rows * 33ull * xb;
    if (total == 0) return;
    unsigned grid = (unsigned)(((total + 255) / 256) < 148ull * 64 ? ((total + 255) / 256) : 148ull * 64);
    relayout_iq2xxs_kernel<<<grid, 256, 0, st>>>(reinterpret_cast<const uint16_t *>(src),
                                                 reinterpret_cast<uint16_t *>(dst), n_rows, xb, inverse);
}

void launch_relayout_q2k(cudaStream_t st, const uint8_t *src, uint8_t *dst, uint64_t n_rows, uint32_t mb, int inverse)
{
    uint64_t total = n_rows * 21ull * mb;
    if (total == 0) return;
    unsigned grid = (unsigned)(((total + 255) / 256) < 148ull * 64 ? ((total + 255) / 256) : 148ull * 64);
    relayout_q2k_kernel<<<grid, 256, 0, st>>>(reinterpret_cast<const uint32_t *>(src), reinterpret_cast<uint32_t *>(dst),
                                              n_rows, mb, inverse);
}

// ---------------------------------------------------------------------------------------------------------------
// Slot sum (engine/src/kernels/moe.rs:983-1005): out[t][row] = sum over slots, in slot order, starting from 0.
// ---------------------------------------------------------------------------------------------------------------
// out[tok] = ((0 + r_0) + r_1) + ... over the token's k slot rows, r_e = down[pos ? pos[tok*k+e] : tok*k+e].
// VEC = 4: one float4 per thread (out_dim a multiple of 4, pointers 16-byte aligned); VEC = 1 otherwise.
// With hc.out_hc set, the hyper-connection merge that consumes the sum in the reference (hc_expand,
// engine/src/kernels/hc.rs:212-251; call engine/src/session.rs:2162-2175) runs in the same thread, so the routed sum
// is not read back from memory: block_v = shared[t][d] + routed[t][d];
// out_hc[t][dst][d] = block_v * post[dst] + sum over src of comb[dst + src * n_hc] * residual[t][src][d], post and comb
// taken from the token's split row at offsets n_hc and 2 n_hc, every multiplication and addition rounded on its own.
__device__ __forceinline__ void hc_expand_elem(const HcEpilogue &hc, uint64_t tok, uint64_t d, uint32_t n_embd, float routed)
{
    const float block_v = __fadd_rn(hc.shared[tok * n_embd + d], routed);
    const float *sp = hc.split + tok * hc.mix_hc;
    for (uint32_t dst = 0; dst < hc.n_hc; ++dst) {
        float acc = __fmul_rn(block_v, sp[hc.n_hc + dst]);
        for (uint32_t src = 0; src < hc.n_hc; ++src)
            acc = __fadd_rn(acc, __fmul_rn(sp[2 * hc.n_hc + dst + src * hc.n_hc],
                                           hc.residual[(tok * hc.n_hc + src) * n_embd + d]));
        hc.out_hc[(tok * hc.n_hc + dst) * n_embd + d] = acc;
    }
}

template <int VEC>
__global__ void __launch_bounds__(256) moe_sum_kernel(const float *__restrict__ down, const int32_t *__restrict__ pos,
                                                       float *__restrict__ out, uint32_t out_dim, uint32_t k, uint64_t n,
                                                       HcEpilogue hc)
{
    const uint64_t gid = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (gid >= n) return;
    const uint32_t per_row = out_dim / VEC;
    const uint64_t tok = gid / per_row, col = (gid - tok * per_row) * VEC;
    float acc[VEC];
#pragma unroll
    for (int i = 0; i < VEC; ++i) acc[i] = 0.0f;
    for (uint32_t e = 0; e < k; ++e) {
        const uint64_t row = pos ? (uint64_t)(uint32_t)pos[tok * k + e] : tok * k + e;
        const float *src = down + row * out_dim + col;
        if (VEC == 4) {
            const float4 v = *reinterpret_cast<const float4 *>(src);
            acc[0] = __fadd_rn(acc[0], v.x), acc[1] = __fadd_rn(acc[1], v.y);
            acc[2] = __fadd_rn(acc[2], v.z), acc[3] = __fadd_rn(acc[3], v.w);
        } else {
            acc[0] = __fadd_rn(acc[0], src[0]);
        }
    }
    if (VEC == 4) *reinterpret_cast<float4 *>(out + tok * out_dim + col) = make_float4(acc[0], acc[1], acc[2], acc[3]);
    else out[tok * out_dim + col] = acc[0];
    if (hc.out_hc != nullptr) {
#pragma unroll
        for (int i = 0; i < VEC; ++i) hc_expand_elem(hc, tok, col + i, out_dim, acc[i]);
    }
}

void launch_moe_sum(cudaStream_t st, const float *down, const int32_t *pos, float *out, uint32_t out_dim, uint32_t k,
                    uint32_t n_tokens, const HcEpilogue *hc)
{
    if (n_tokens == 0 || out_dim == 0) return;
    HcEpilogue h = {};
    if (hc) h = *hc;
    const bool vec = out_dim % 4 == 0 && (((uintptr_t)down | (uintptr_t)out) & 15) == 0;
    const uint64_t n = (uint64_t)n_tokens * (vec ? out_dim / 4 : out_dim);
    if (vec) moe_sum_kernel<4><<<(unsigned)((n + 255) / 256), 256, 0, st>>>(down, pos, out, out_dim, k, n, h);
    else moe_sum_kernel<1><<<(unsigned)((n + 255) / 256), 256, 0, st>>>(down, pos, out, out_dim, k, n, h);
}

// hc_expand on its own (engine/src/kernels/hc.rs:212-251): one thread per (token, d); block_add may be null
// (has_add == 0: the routed experts did not run).
__global__ void __launch_bounds__(256) hc_expand_kernel(const float *__restrict__ block_add, uint32_t n_embd, uint64_t n,
                                                         HcEpilogue hc)
{
    const uint64_t gid = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (gid >= n) return;
    const uint64_t tok = gid / n_embd, d = gid - tok * n_embd;
    if (block_add != nullptr) {
        hc_expand_elem(hc, tok, d, n_embd, block_add[gid]);
        return;
    }
    const float block_v = hc.shared[gid];
    const float *sp = hc.split + tok * hc.mix_hc;
    for (uint32_t dst = 0; dst < hc.n_hc; ++dst) {
        float acc = __fmul_rn(block_v, sp[hc.n_hc + dst]);
        for (uint32_t src = 0; src < hc.n_hc; ++src)
            acc = __fadd_rn(acc, __fmul_rn(sp[2 * hc.n_hc + dst + src * hc.n_hc],
                                           hc.residual[(tok * hc.n_hc + src) * n_embd + d]));
        hc.out_hc[(tok * hc.n_hc + dst) * n_embd + d] = acc;
    }
}

void launch_hc_expand(cudaStream_t st, const float *block_add, uint32_t n_embd, uint32_t n_tokens, const HcEpilogue &hc)
{
    const uint64_t n = (uint64_t)n_tokens * n_embd;
    if (n == 0) return;
    hc_expand_kernel<<<(unsigned)((n + 255) / 256), 256, 0, st>>>(block_add, n_embd, n, hc);
}

// ---------------------------------------------------------------------------------------------------------------
// FFN pre-norm producer: hc_split_weighted_sum_norm_fused (engine/src/kernels/hc.rs:313-394) with hc4_split_one
// (hc.rs:17-100). One CTA of 256 threads per row, as the reference launches it (engine/src/session.rs:1865-1892).
// Thread 0 computes the 24-value split (4 pre-weights: sigmoid + eps; 4 post-weights: 2 sigmoid; 4 x 4 comb matrix: row
// softmax + eps, then Sinkhorn normalisation), all threads the weighted sum over the 4 residual streams, then the RMS
// norm with the reference's 256-wide halving tree. Every operation is rounded on its own and in the reference's order;
// exp is the correctly rounded f32 exponential this library uses everywhere (the reference's comes from its compiler's
// math library, whose rounding no test pins).
// ---------------------------------------------------------------------------------------------------------------
__device__ void hc4_split_one(float *out, const float *mix, const float *scale, const float *base, uint32_t iters, float epsv)
{
    const float pre_s = scale[0], post_s = scale[1], comb_s = scale[2];
    for (int i = 0; i < 4; ++i) {
        const float z = __fadd_rn(__fmul_rn(mix[i], pre_s), base[i]);
        out[i] = __fadd_rn(__fdiv_rn(1.0f, __fadd_rn(1.0f, expf_cr(-z))), epsv);
    }
    for (int i = 0; i < 4; ++i) {
        const float z = __fadd_rn(__fmul_rn(mix[4 + i], post_s), base[4 + i]);
        out[4 + i] = __fdiv_rn(2.0f, __fadd_rn(1.0f, expf_cr(-z)));
    }
    float c[16];
    for (int r = 0; r < 4; ++r) {
        float m = -INFINITY;
        for (int col = 0; col < 4; ++col) {
            const float v = __fadd_rn(__fmul_rn(mix[8 + r * 4 + col], comb_s), base[8 + r * 4 + col]);
            c[r * 4 + col] = v;
            if (v > m) m = v;
        }
        float sum = 0.0f;
        for (int col = 0; col < 4; ++col) {
            const float v = expf_cr(__fsub_rn(c[r * 4 + col], m));
            c[r * 4 + col] = v;
            sum = __fadd_rn(sum, v);
        }
        for (int col = 0; col < 4; ++col) c[r * 4 + col] = __fadd_rn(__fdiv_rn(c[r * 4 + col], sum), epsv);
    }
    for (int col = 0; col < 4; ++col) {
        float sum = epsv;
        for (int r = 0; r < 4; ++r) sum = __fadd_rn(sum, c[r * 4 + col]);
        for (int r = 0; r < 4; ++r) c[r * 4 + col] = __fdiv_rn(c[r * 4 + col], sum);
    }
    for (uint32_t it = 1; it < iters; ++it) {
        for (int r = 0; r < 4; ++r) {
            float sum = epsv;
            for (int col = 0; col < 4; ++col) sum = __fadd_rn(sum, c[r * 4 + col]);
            for (int col = 0; col < 4; ++col) c[r * 4 + col] = __fdiv_rn(c[r * 4 + col], sum);
        }
        for (int col = 0; col < 4; ++col) {
            float sum = epsv;
            for (int r = 0; r < 4; ++r) sum = __fadd_rn(sum, c[r * 4 + col]);
            for (int r = 0; r < 4; ++r) c[r * 4 + col] = __fdiv_rn(c[r * 4 + col], sum);
        }
    }
    for (int i = 0; i < 16; ++i) out[8 + i] = c[i];
}

__global__ void __launch_bounds__(256) hc_split_weighted_sum_norm_kernel(
    const float *__restrict__ mix, const float *__restrict__ scale, const float *__restrict__ base,
    const float *__restrict__ residual_hc, const float *__restrict__ norm_w, float *__restrict__ split,
    float *__restrict__ out, float *__restrict__ norm_out, uint32_t n_embd, uint32_t iters, float epsv, float norm_eps)
{
    __shared__ float s_split[24];
    __shared__ float s_partial[256];
    const uint32_t t = blockIdx.x, d = threadIdx.x;
    if (d == 0) {
        hc4_split_one(s_split, mix + (size_t)t * 24, scale, base, iters, epsv);
        for (int i = 0; i < 24; ++i) split[(size_t)t * 24 + i] = s_split[i];
    }
    __syncthreads();
    float sum_sq = 0.0f;
    for (uint32_t col = d; col < n_embd; col += 256) {
        float acc = 0.0f;
        for (uint32_t h = 0; h < 4; ++h)
            acc = __fadd_rn(acc, __fmul_rn(residual_hc[((size_t)t * 4 + h) * n_embd + col], s_split[h]));
        out[(size_t)t * n_embd + col] = acc;
        sum_sq = __fadd_rn(sum_sq, __fmul_rn(acc, acc));
    }
    s_partial[d] = sum_sq;
    __syncthreads();
    for (uint32_t stride = 128; stride > 0; stride >>= 1) {
        if (d < stride) s_partial[d] = __fadd_rn(s_partial[d], s_partial[d + stride]);
        __syncthreads();
    }
    const float norm_scale = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fdiv_rn(s_partial[0], (float)n_embd), norm_eps)));
    for (uint32_t col = d; col < n_embd; col += 256) {
        const size_t off = (size_t)t * n_embd + col;
        norm_out[off] = __fmul_rn(__fmul_rn(out[off], norm_scale), norm_w[col]);
    }
}

void launch_hc_split_weighted_sum_norm(cudaStream_t st, const float *mix, const float *scale, const float *base,
                                       const float *residual_hc, const float *norm_w, float *split, float *out,
                                       float *norm_out, uint32_t n_embd, uint32_t n_rows, uint32_t iters, float epsv,
                                       float norm_eps)
{
    if (n_rows == 0) return;
    hc_split_weighted_sum_norm_kernel<<<n_rows, 256, 0, st>>>(mix, scale, base, residual_hc, norm_w, split, out, norm_out,
                                                              n_embd, iters, epsv, norm_eps);
}

// Checked build (-DDSMOE_BOUNDS): expert indices are copied before use, any index >= hi is replaced by 0 and recorded in
// the status word, so an index that would address memory outside the registered tensors never reaches a kernel.
// Negative indices are left alone: the kernels map them to expert 0 as the reference does (moe.rs:645-648).
__global__ void __launch_bounds__(256) sanitize_indices_kernel(const int32_t *src, int32_t *dst,  // may alias
                                                                uint64_t n, int32_t hi, int *status)
{
    const uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    int32_t v = src[i];
    if (v >= hi) {
        v = 0;
        if (status) atomicCAS(status, 0, 2 /* DEV_ERR_INDEX_RANGE */);
    }
    dst[i] = v;
}

void launch_sanitize_indices(cudaStream_t st, const int32_t *src, int32_t *dst, uint64_t n, int32_t hi, int *status)
{
    if (n == 0) return;
    sanitize_indices_kernel<<<(unsigned)((n + 255) / 256), 256, 0, st>>>(src, dst, n, hi, status);
}

// Copies row i to dst[i] (expert-parallel combine on the decode path: plain 16-byte stores, possibly across NVLink).
__global__ void __launch_bounds__(256) scatter_rows_kernel(const float *__restrict__ rows, float *const *__restrict__ dst,
                                                            uint32_t n_embd, uint32_t n_rows)
{
    const uint32_t row = blockIdx.x;
    if (row >= n_rows) return;
    const float4 *src = reinterpret_cast<const float4 *>(rows + (size_t)row * n_embd);
    float4 *d = reinterpret_cast<float4 *>(dst[row]);
    for (uint32_t i = threadIdx.x; i < n_embd / 4; i += 256) d[i] = src[i];
}

void launch_scatter_rows(cudaStream_t st, const float *rows, float *const *dst, uint32_t n_embd, uint32_t n_rows)
{
    if (n_rows == 0) return;
    scatter_rows_kernel<<<n_rows, 256, 0, st>>>(rows, dst, n_embd, n_rows);
}

// bf16 -> f32, exact (the bf16 bit pattern is the upper half of the f32 one)
__global__ void __launch_bounds__(256) bf16_to_f32_kernel(const uint16_t *__restrict__ in, float *__restrict__ out, uint64_t n)
{
    const uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) out[i] = __uint_as_float((uint32_t)in[i] << 16);
}

void launch_bf16_to_f32(cudaStream_t st, const uint16_t *in, float *out, uint64_t n)
{
    if (n == 0) return;
    bf16_to_f32_kernel<<<(unsigned)((n + 255) / 256), 256, 0, st>>>(in, out, n);
}

}  // namespace dsmoe
