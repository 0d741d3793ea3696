// FP8 E4M3 block-scaled dense projection: C[m][n] = bf16( sum_kb s_a[m][kb] * s_w[n/128][kb] * sum_{k in kb} a * w ).
//
// The reference has no FP8 GEMM (its dense projections are Q8_0 x Q8_0 matvecs, engine/src/kernels/matmul.rs:357-603;
// E4M3 appears only as a rounding of KV rows, engine/src/kernels/quantize.rs:10-134), so this follows the definition
// the CPU oracle states: scales max(amax, 1e-4) / 448 per 1x128 activation block and per 128x128 weight block, codes
// = round-to-nearest-even, saturating E4M3 of x / s (the semantics of e4m3fn_dequant, quantize.rs:24-53, which is what
// cvt.rn.satfinite.e4m3x2.f32 does). Parity is unpinned; the test tolerance is rel 2e-2 against the oracle in f64.
//
//   fp8_quantize_kernel   one warp per 1x128 block (activations) / one CTA per 128x128 block (weights)
//   fp8_gemm_kernel       tcgen05 kind::f8f6f4, 128x128 output tile per CTA; a stage is one 128-wide K block (four
//                         K=32 MMAs) whose TMEM accumulator is drained with the block's scale product (one FMA per
//                         element: s_w is one scalar per tile and K block, s_a one per row) while the next block's
//                         MMAs run. Operands reach shared memory by 16-byte cp.async in core-matrix order.
//   fp8_matvec_kernel     M <= 8: bandwidth-bound, one warp per output feature, f32 accumulate.
#include <cuda_bf16.h>
#include <cuda_fp8.h>

#include "common.cuh"
#include "launch.h"
#include "tc05.cuh"

namespace dsmoe {

__device__ __forceinline__ uint8_t fp8_encode(float v)
{
    return (uint8_t)__nv_cvt_float_to_fp8(v, __NV_SATFINITE, __NV_E4M3);
}

__device__ __forceinline__ float fp8_decode(uint8_t c)
{
    const __half_raw h = __nv_cvt_fp8_to_halfraw((__nv_fp8_storage_t)c, __NV_E4M3);
    return __half2float(*reinterpret_cast<const __half *>(&h));
}

// rows_per_block == 1: one warp per (row, 128-column block). rows_per_block == 128: one CTA (256 threads) per block.
__global__ void __launch_bounds__(256) fp8_quantize_kernel(const float *__restrict__ x, uint8_t *__restrict__ codes,
                                                            float *__restrict__ scales, uint32_t rows, uint32_t cols,
                                                            int rows_per_block)
{
    const uint32_t cb = cols / 128;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if (rows_per_block == 1) {
        const uint64_t blk = (uint64_t)blockIdx.x * 8 + warp;
        if (blk >= (uint64_t)rows * cb) return;
        const uint32_t r = (uint32_t)(blk / cb), bc = (uint32_t)(blk % cb);
        const float4 v = *reinterpret_cast<const float4 *>(x + (size_t)r * cols + bc * 128 + 4 * lane);
        float amax = fmaxf(fmaxf(fabsf(v.x), fabsf(v.y)), fmaxf(fabsf(v.z), fabsf(v.w)));
#pragma unroll
        for (int m = 16; m > 0; m >>= 1) amax = fmaxf(amax, __shfl_xor_sync(FULL, amax, m));
        const float s = __fdiv_rn(fmaxf(amax, 1.0e-4f), 448.0f);
        if (lane == 0) scales[(size_t)r * cb + bc] = s;
        const uint32_t packed = (uint32_t)fp8_encode(__fdiv_rn(v.x, s)) | ((uint32_t)fp8_encode(__fdiv_rn(v.y, s)) << 8) |
                                ((uint32_t)fp8_encode(__fdiv_rn(v.z, s)) << 16) | ((uint32_t)fp8_encode(__fdiv_rn(v.w, s)) << 24);
        *reinterpret_cast<uint32_t *>(codes + (size_t)r * cols + bc * 128 + 4 * lane) = packed;
        return;
    }
    __shared__ float s_red[8];
    const uint32_t br = blockIdx.x / cb, bc = blockIdx.x % cb;
    const uint32_t r0 = br * 128, r1 = min(rows, r0 + 128);
    float amax = 0.0f;
    for (uint32_t i = threadIdx.x; i < (r1 - r0) * 128; i += 256)
        amax = fmaxf(amax, fabsf(x[(size_t)(r0 + i / 128) * cols + bc * 128 + (i & 127)]));
#pragma unroll
    for (int m = 16; m > 0; m >>= 1) amax = fmaxf(amax, __shfl_xor_sync(FULL, amax, m));
    if (lane == 0) s_red[warp] = amax;
    __syncthreads();
    amax = s_red[0];
#pragma unroll
    for (int w = 1; w < 8; ++w) amax = fmaxf(amax, s_red[w]);
    const float s = __fdiv_rn(fmaxf(amax, 1.0e-4f), 448.0f);
    if (threadIdx.x == 0) scales[(size_t)br * cb + bc] = s;
    for (uint32_t i = threadIdx.x; i < (r1 - r0) * 128; i += 256) {
        const size_t o = (size_t)(r0 + i / 128) * cols + bc * 128 + (i & 127);
        codes[o] = fp8_encode(__fdiv_rn(x[o], s));
    }
}

void launch_fp8_quantize(cudaStream_t st, const float *x, uint8_t *codes, float *scales, uint32_t rows, uint32_t cols,
                         int rows_per_block)
{
    if (rows == 0 || cols == 0) return;
    const uint32_t cb = cols / 128;
    if (rows_per_block == 1) {
        const uint64_t nb = (uint64_t)rows * cb;
        fp8_quantize_kernel<<<(unsigned)((nb + 7) / 8), 256, 0, st>>>(x, codes, scales, rows, cols, 1);
    } else {
        fp8_quantize_kernel<<<((rows + 127) / 128) * cb, 256, 0, st>>>(x, codes, scales, rows, cols, 128);
    }
}

// ---------------------------------------------------------------------------------------------------------------
// M <= 8: one warp per output feature n; lane l covers bytes 16 l .. 16 l + 15 of each 512-byte stretch of K.
// ---------------------------------------------------------------------------------------------------------------
constexpr int FP8_MV_MAX_M = 8;

__global__ void __launch_bounds__(256) fp8_matvec_kernel(const uint8_t *__restrict__ a, const float *__restrict__ a_scale,
                                                          const uint8_t *__restrict__ w, const float *__restrict__ w_scale,
                                                          __nv_bfloat16 *__restrict__ out, uint32_t M, uint32_t N, uint32_t K)
{
    const int lane = threadIdx.x & 31;
    const uint32_t n = blockIdx.x * 8 + (threadIdx.x >> 5);
    if (n >= N) return;
    const uint32_t kbn = K / 128;
    float acc[FP8_MV_MAX_M];
#pragma unroll
    for (int m = 0; m < FP8_MV_MAX_M; ++m) acc[m] = 0.0f;
    for (uint32_t k0 = 16 * lane; k0 < K; k0 += 512) {
        const uint32_t kb = k0 >> 7;
        const uint4 wv = ld_stream_16B(w + (size_t)n * K + k0);
        const float sw = w_scale[(size_t)(n >> 7) * kbn + kb];
        const uint32_t ww[4] = {wv.x, wv.y, wv.z, wv.w};
        float wf[16];
#pragma unroll
        for (int i = 0; i < 16; ++i) wf[i] = fp8_decode((uint8_t)(ww[i >> 2] >> (8 * (i & 3))));
#pragma unroll
        for (int m = 0; m < FP8_MV_MAX_M; ++m) {
            if (m < (int)M) {
                const uint4 av = *reinterpret_cast<const uint4 *>(a + (size_t)m * K + k0);
                const uint32_t aw[4] = {av.x, av.y, av.z, av.w};
                float p = 0.0f;
#pragma unroll
                for (int i = 0; i < 16; ++i) p = fmaf(fp8_decode((uint8_t)(aw[i >> 2] >> (8 * (i & 3)))), wf[i], p);
                acc[m] = fmaf(a_scale[(size_t)m * kbn + kb] * sw, p, acc[m]);
            }
        }
    }
#pragma unroll
    for (int m = 0; m < FP8_MV_MAX_M; ++m) {
        float v = acc[m];
#pragma unroll
        for (int s = 16; s > 0; s >>= 1) v += __shfl_xor_sync(FULL, v, s);
        if (lane == 0 && m < (int)M) out[(size_t)m * N + n] = __float2bfloat16_rn(v);
    }
}

// ---------------------------------------------------------------------------------------------------------------
// GEMM: 128 (rows of A) x 128 (rows of W) output tile per CTA, 256 threads.
// ---------------------------------------------------------------------------------------------------------------
constexpr int F8_STAGES = 4;
constexpr int F8_TILE = 128 * 128;            // bytes of one operand stage (128 rows x 128 K, one byte each)
constexpr int F8_SBO = (128 / 16) * 128;      // 1024: byte distance between 8-row groups
constexpr int F8_SMEM = 2 * F8_STAGES * F8_TILE + 64;

__device__ __forceinline__ void cp_async_16(uint32_t dst_smem, const void *src, uint32_t src_bytes)
{
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst_smem), "l"(src), "r"(src_bytes) : "memory");
}

__global__ void __launch_bounds__(256, 1) fp8_gemm_kernel(const uint8_t *__restrict__ a, const float *__restrict__ a_scale,
                                                           const uint8_t *__restrict__ w, const float *__restrict__ w_scale,
                                                           __nv_bfloat16 *__restrict__ out, uint32_t M, uint32_t N, uint32_t K,
                                                           int *status)
{
    extern __shared__ __align__(1024) uint8_t smem[];
    uint64_t *bar_mma = reinterpret_cast<uint64_t *>(smem + 2 * F8_STAGES * F8_TILE);  // [2]
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(bar_mma + 2);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const uint32_t n0 = blockIdx.x * 128, m0 = blockIdx.y * 128, nkb = K / 128;

    if (warp == 0) tc05_alloc(tmem_slot, 256);
    if (tid == 0) {
        mbar_init(&bar_mma[0], 1);
        mbar_init(&bar_mma[1], 1);
        fence_async_smem();
    }
    tc05_fence_before_sync();
    __syncthreads();
    tc05_fence_after_sync();
    const uint32_t tmem = *tmem_slot;

    // this thread's four 16-byte chunks of a stage: 8 rows x 64 bytes per warp instruction
    auto load_stage = [&](uint32_t kb) {
        const uint32_t st = kb % F8_STAGES;
        const uint32_t sa = smem_u32(smem + st * F8_TILE), sb = smem_u32(smem + (F8_STAGES + st) * F8_TILE);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const uint32_t q = i * 256 + tid, r = ((q >> 6) << 3) + (q & 7), c = (((q >> 5) & 1) << 2) + ((q >> 3) & 3);
            const uint32_t dst = (r >> 3) * F8_SBO + c * 128 + (r & 7) * 16;
            const uint32_t m = m0 + r;
            cp_async_16(sa + dst, a + (size_t)(m < M ? m : 0) * K + kb * 128 + 16 * c, m < M ? 16u : 0u);
            cp_async_16(sb + dst, w + (size_t)(n0 + r) * K + kb * 128 + 16 * c, 16u);
        }
    };
#pragma unroll
    for (int s = 0; s < F8_STAGES - 1; ++s) {
        if ((uint32_t)s < nkb) load_stage(s);
        asm volatile("cp.async.commit_group;" ::: "memory");
    }

    const uint32_t arow = 32 * (warp & 3) + lane, acol0 = 64 * (warp >> 2), tlane = (32u * (warp & 3)) << 16;
    const uint32_t mrow = m0 + arow;
    const uint32_t idesc = tc05_idesc_e4m3(128, 128);
    float acc[64];
#pragma unroll
    for (int i = 0; i < 64; ++i) acc[i] = 0.0f;
    bool ok = true;

    auto drain = [&](uint32_t kb) {
        const float scale = mrow < M ? a_scale[(size_t)mrow * nkb + kb] * w_scale[(size_t)blockIdx.x * nkb + kb] : 0.0f;
#pragma unroll
        for (int c0 = 0; c0 < 64; c0 += 16) {
            float v[16];
            tc05_ld16(tmem + tlane + (kb & 1) * 128 + acol0 + c0, v);
            tc05_wait_ld16(v);
#pragma unroll
            for (int i = 0; i < 16; ++i) acc[c0 + i] = fmaf(scale, v[i], acc[c0 + i]);
        }
    };

    for (uint32_t kb = 0; kb < nkb; ++kb) {
        asm volatile("cp.async.wait_group %0;" ::"n"(F8_STAGES - 2) : "memory");  // this thread's part of stage kb landed
        fence_async_smem();
        tc05_fence_before_sync();
        ok = __syncthreads_and(ok);
        if (!ok) break;
        if (tid == 0) {
            tc05_fence_after_sync();
            const uint32_t st = kb % F8_STAGES;
            const uint32_t sa = smem_u32(smem + st * F8_TILE), sb = smem_u32(smem + (F8_STAGES + st) * F8_TILE);
#pragma unroll
            for (int ks = 0; ks < 4; ++ks)
                tc05_mma_f8(tmem + (kb & 1) * 128, tc05_smem_desc(sa + ks * 256, 128, F8_SBO),
                            tc05_smem_desc(sb + ks * 256, 128, F8_SBO), idesc, ks != 0);
            tc05_commit(&bar_mma[kb & 1]);
        }
        if (kb >= 1) {
            // the previous block's MMAs have retired: its stage may be refilled and its accumulator drained
            ok = mbar_wait_bounded(&bar_mma[(kb - 1) & 1], ((kb - 1) >> 1) & 1, status);
            tc05_fence_after_sync();
        }
        if (ok && kb + F8_STAGES - 1 < nkb) load_stage(kb + F8_STAGES - 1);
        asm volatile("cp.async.commit_group;" ::: "memory");
        if (ok && kb >= 1) drain(kb - 1);
    }
    if (ok && nkb > 0) {
        ok = mbar_wait_bounded(&bar_mma[(nkb - 1) & 1], ((nkb - 1) >> 1) & 1, status);
        tc05_fence_after_sync();
        if (ok) drain(nkb - 1);
    }
    asm volatile("cp.async.wait_group 0;" ::: "memory");
    if (ok && mrow < M) {
        __nv_bfloat162 *o = reinterpret_cast<__nv_bfloat162 *>(out + (size_t)mrow * N + n0 + acol0);
#pragma unroll
        for (int i = 0; i < 32; ++i) o[i] = __floats2bfloat162_rn(acc[2 * i], acc[2 * i + 1]);
    }
    tc05_fence_before_sync();
    __syncthreads();
    if (warp == 0) tc05_dealloc(tmem, 256);
}

int launch_fp8_linear(cudaStream_t st, const uint8_t *a, const float *a_scale, const uint8_t *w, const float *w_scale,
                      void *out_bf16, uint32_t M, uint32_t N, uint32_t K, int *status)
{
    if (M == 0 || N == 0) return 0;
    __nv_bfloat16 *out = reinterpret_cast<__nv_bfloat16 *>(out_bf16);
    if (M <= FP8_MV_MAX_M) {
        fp8_matvec_kernel<<<(N + 7) / 8, 256, 0, st>>>(a, a_scale, w, w_scale, out, M, N, K);
        return 1;
    }
    static bool attr_set = false;
    if (!attr_set) {
        cudaFuncSetAttribute(fp8_gemm_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, F8_SMEM);
        attr_set = true;
    }
    fp8_gemm_kernel<<<dim3(N / 128, (M + 127) / 128), 256, F8_SMEM, st>>>(a, a_scale, w, w_scale, out, M, N, K, status);
    return 1;
}

}  // namespace dsmoe
