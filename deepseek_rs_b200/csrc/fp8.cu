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
#include <stdlib.h>
#include <string.h>

#include <cuda.h>
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

// Four e4m3 codes (byte 0 first) to f32, two per conversion instruction; the values are exact.
__device__ __forceinline__ void fp8x4_decode(uint32_t c, float *f)
{
    const __half2_raw lo = __nv_cvt_fp8x2_to_halfraw2((__nv_fp8x2_storage_t)(c & 0xFFFFu), __NV_E4M3);
    const __half2_raw hi = __nv_cvt_fp8x2_to_halfraw2((__nv_fp8x2_storage_t)(c >> 16), __NV_E4M3);
    const float2 a = __half22float2(*reinterpret_cast<const __half2 *>(&lo));
    const float2 b = __half22float2(*reinterpret_cast<const __half2 *>(&hi));
    f[0] = a.x, f[1] = a.y, f[2] = b.x, f[3] = b.y;
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

template <int MM, int DEPTH>  // MM: rows handled (M <= MM); DEPTH: 512-byte stretches of the weight row in flight
__global__ void __launch_bounds__(256, 4) fp8_matvec_kernel(const uint8_t *__restrict__ a, const float *__restrict__ a_scale,
                                                          const uint8_t *__restrict__ w, const float *__restrict__ w_scale,
                                                          __nv_bfloat16 *__restrict__ out, uint32_t M, uint32_t N, uint32_t K)
{
    const int lane = threadIdx.x & 31;
    const uint32_t n = blockIdx.x * 8 + (threadIdx.x >> 5);
    if (n >= N) return;
    const uint32_t kbn = K / 128;
    float acc[MM];
#pragma unroll
    for (int m = 0; m < MM; ++m) acc[m] = 0.0f;
    // DEPTH stretches of the row per round, all requested before any is used; four CTAs per SM, so that the 512 CTAs
    // of a 4096-feature projection are resident at once
    for (uint32_t kr = 16 * lane; kr < K; kr += DEPTH * 512) {
        uint4 wq[DEPTH];
#pragma unroll
        for (int u = 0; u < DEPTH; ++u)
            if (kr + 512 * u < K) wq[u] = ld_stream_16B(w + (size_t)n * K + kr + 512 * u);
#pragma unroll
        for (int u = 0; u < DEPTH; ++u) {
            const uint32_t k0 = kr + 512 * u;
            if (k0 >= K) break;
            const uint32_t kb = k0 >> 7;
            const float sw = w_scale[(size_t)(n >> 7) * kbn + kb];
            float wf[16];
            fp8x4_decode(wq[u].x, wf), fp8x4_decode(wq[u].y, wf + 4), fp8x4_decode(wq[u].z, wf + 8), fp8x4_decode(wq[u].w, wf + 12);
#pragma unroll
            for (int m = 0; m < MM; ++m) {
                if (m < (int)M) {
                    const uint4 av = *reinterpret_cast<const uint4 *>(a + (size_t)m * K + k0);
                    float af[16];
                    fp8x4_decode(av.x, af), fp8x4_decode(av.y, af + 4), fp8x4_decode(av.z, af + 8), fp8x4_decode(av.w, af + 12);
                    float p = 0.0f;
#pragma unroll
                    for (int i = 0; i < 16; ++i) p = fmaf(af[i], wf[i], p);
                    acc[m] = fmaf(a_scale[(size_t)m * kbn + kb] * sw, p, acc[m]);
                }
            }
        }
    }
#pragma unroll
    for (int m = 0; m < MM; ++m) {
        float v = acc[m];
#pragma unroll
        for (int s = 16; s > 0; s >>= 1) v += __shfl_xor_sync(FULL, v, s);
        if (lane == 0 && m < (int)M) out[(size_t)m * N + n] = __float2bfloat16_rn(v);
    }
}

// ---------------------------------------------------------------------------------------------------------------
// GEMM: 128 (rows of A) x 128 (rows of W) output tile per CTA, 256 threads.
// ---------------------------------------------------------------------------------------------------------------
#ifndef F8_STAGES_N
#define F8_STAGES_N 3
#define F8_CTAS_PER_SM 2
#endif
constexpr int F8_STAGES = F8_STAGES_N;  // 3 stages x 32 KB: two CTAs share an SM and fill each other's waits
constexpr int F8_TILE = 128 * 128;            // bytes of one operand stage (128 rows x 128 K, one byte each)
constexpr int F8_SBO = (128 / 16) * 128;      // 1024: byte distance between 8-row groups
constexpr int F8_SMEM = 2 * F8_STAGES * F8_TILE + 64;

__device__ __forceinline__ void cp_async_16(uint32_t dst_smem, const void *src, uint32_t src_bytes)
{
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst_smem), "l"(src), "r"(src_bytes) : "memory");
}

__global__ void __launch_bounds__(256, F8_CTAS_PER_SM) fp8_gemm_kernel(const uint8_t *__restrict__ a, const float *__restrict__ a_scale,
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

// ---------------------------------------------------------------------------------------------------------------
// Large M: persistent, warp-specialised. One CTA per SM walks 128 x 256 output tiles; per 128-wide K block
//   warps 8-11  producers  16-byte cp.async of the A (128 rows) and W (256 rows) blocks into a 4-stage ring in
//                          core-matrix order, completion counted on the stage's "full" mbarrier;
//   warp 12     issuer     four K=32 MMAs (M 128, N 256) into one of two TMEM accumulators, committed to the stage's
//                          "free" and the accumulator's "full" mbarriers;
//   warps 0-7   consumers  drain the accumulator (tcgen05.ld), hand it back, apply s_a[row][kb] * s_w[n/128][kb] with
//                          one FMA per element into 128 registers; after the last K block write the bf16 row segment.
// Registers move to the consumers with setmaxnreg. Every wait is bounded; the common exit frees TMEM.
// ---------------------------------------------------------------------------------------------------------------
constexpr int F8W_STAGES = 4, F8W_TN = 256, F8W_THREADS = 512, F8W_MAX_KB = 32;
constexpr int F8W_STAGE_A = 128 * 128, F8W_STAGE_B = F8W_TN * 128;
constexpr int F8W_SMEM_B = F8W_STAGES * F8W_STAGE_A;
constexpr int F8W_SMEM_SA = F8W_SMEM_B + F8W_STAGES * F8W_STAGE_B;   // [kb][128 rows] activation scales of the tile
constexpr int F8W_SMEM_SW = F8W_SMEM_SA + F8W_MAX_KB * 128 * 4;      // [2][kb] weight scales of the tile's two blocks
constexpr int F8W_SMEM_BAR = F8W_SMEM_SW + 2 * F8W_MAX_KB * 4;
constexpr int F8W_SMEM = F8W_SMEM_BAR + 128;
static_assert(F8W_SMEM <= 232448, "shared memory per CTA");
// compiled for 128 registers (512 threads); 8 warps release 56 each, the 8 consumer warps take them
constexpr int F8W_REG_LAUNCH = 128, F8W_REG_CONSUMER = 184, F8W_REG_OTHER = 72;
static_assert(256 * (F8W_REG_CONSUMER - F8W_REG_LAUNCH) <= 256 * (F8W_REG_LAUNCH - F8W_REG_OTHER), "setmaxnreg budget");

// Tensor-map (TMA) tile load into shared memory, completion counted in bytes on the mbarrier. Coordinates: x = byte
// column (a multiple of 16), y = row. Rows outside the tensor arrive as zeros. Local memory only.
__device__ __forceinline__ void tma_load_2d(void *dst_smem, const CUtensorMap *map, uint32_t x, uint32_t y, uint64_t *bar)
{
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(
                     smem_u32(dst_smem)),
                 "l"(reinterpret_cast<uint64_t>(map)), "r"(x), "r"(y), "r"(smem_u32(bar))
                 : "memory");
}

// Shared-memory descriptor of a K-major operand tile written by a 128-byte-swizzled tensor-map load: rows of 128
// bytes, 8-row groups 1024 bytes apart, layout type 2 (128-byte swizzle), version 1. The tile must start on a
// 1024-byte boundary; K advances inside the swizzle atom by adding the byte offset to the start address.
__device__ __forceinline__ uint64_t tc05_smem_desc_sw128(uint32_t smem_addr)
{
    uint64_t d = 0;
    d |= (uint64_t)((smem_addr >> 4) & 0x3FFFu);
    d |= (uint64_t)1 << 16;
    d |= (uint64_t)(1024u >> 4) << 32;
    d |= 1ull << 46;
    d |= 2ull << 61;
    return d;
}

// TMA = true: one producer warp issues two tensor-map loads per stage (128-byte swizzle). TMA = false: four producer
// warps copy 16 bytes at a time with cp.async into the unswizzled core-matrix order.
template <bool TMA>
__global__ void __launch_bounds__(F8W_THREADS, 1) fp8_gemm_ws_kernel(const uint8_t *__restrict__ a,
                                                                     const float *__restrict__ a_scale,
                                                                     const uint8_t *__restrict__ w,
                                                                     const float *__restrict__ w_scale,
                                                                     __nv_bfloat16 *__restrict__ out, uint32_t M, uint32_t N,
                                                                     uint32_t K, int *status,
                                                                     const __grid_constant__ CUtensorMap map_a,
                                                                     const __grid_constant__ CUtensorMap map_w)
{
    extern __shared__ __align__(1024) uint8_t smem[];
    uint64_t *bar_full = reinterpret_cast<uint64_t *>(smem + F8W_SMEM_BAR);  // [4] stage landed (128 producer threads)
    uint64_t *bar_free = bar_full + F8W_STAGES;                               // [4] stage's MMAs retired
    uint64_t *bar_acc_full = bar_free + F8W_STAGES;                           // [2]
    uint64_t *bar_acc_free = bar_acc_full + 2;                                // [2] drained (8 warps)
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(bar_acc_free + 2);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const uint32_t nkb = K / 128, n_nt = N / F8W_TN, n_tiles = ((M + 127) / 128) * n_nt;

    if (warp == 0) tc05_alloc(tmem_slot, 512);
    if (tid == 0) {
        for (int i = 0; i < F8W_STAGES; ++i) {
            mbar_init(&bar_full[i], TMA ? 1 : 128);
            mbar_init(&bar_free[i], 1);
        }
        for (int i = 0; i < 2; ++i) {
            mbar_init(&bar_acc_full[i], 1);
            mbar_init(&bar_acc_free[i], 8);
        }
        fence_async_smem();
    }
    tc05_fence_before_sync();
    __syncthreads();
    tc05_fence_after_sync();
    const uint32_t tmem = *tmem_slot;

    if (warp < 8) {
        // ------------------------------------------------------------------------------------------- consumers
        reg_alloc<F8W_REG_CONSUMER>();
        const uint32_t arow = 32 * (warp & 3) + lane, half = warp >> 2, acol0 = 128 * half, tlane = (32u * (warp & 3)) << 16;
        float *sA = reinterpret_cast<float *>(smem + F8W_SMEM_SA), *sW = reinterpret_cast<float *>(smem + F8W_SMEM_SW);
        uint32_t g = 0;  // K blocks drained so far (accumulator buffer and mbarrier phase)
        bool ok = true;
        for (uint32_t tile = blockIdx.x; tile < n_tiles; tile += gridDim.x) {
            const uint32_t mt = tile / n_nt, nt = tile - mt * n_nt, m0 = mt * 128, n0 = nt * F8W_TN, mrow = m0 + arow;
            // the tile's scale tables, rewritten once every consumer warp is done with the previous tile's
            ok = named_barrier_and(1, 256, ok);
            if (!ok) break;
            for (uint32_t i = tid; i < nkb * 128; i += 256) {
                const uint32_t kb = i >> 7, r = i & 127;
                sA[i] = m0 + r < M ? a_scale[(size_t)(m0 + r) * nkb + kb] : 0.0f;
            }
            for (uint32_t i = tid; i < 2 * nkb; i += 256) sW[i] = w_scale[(size_t)(2 * nt + i / nkb) * nkb + i % nkb];
            named_barrier_sync(1, 256);
            float acc[128];
#pragma unroll
            for (int i = 0; i < 128; ++i) acc[i] = 0.0f;
            for (uint32_t kb = 0; kb < nkb; ++kb, ++g) {
                if (!ok) break;
                const uint32_t buf = g & 1u;
                const float scale = sA[kb * 128 + arow] * sW[half * nkb + kb];
                ok = mbar_wait_bounded(&bar_acc_full[buf], (g >> 1) & 1u, status);
                ok = __all_sync(FULL, ok);
                if (!ok) break;
                tc05_fence_after_sync();
#pragma unroll
                for (int c0 = 0; c0 < 128; c0 += 16) {
                    float v[16];
                    tc05_ld16(tmem + tlane + buf * F8W_TN + acol0 + c0, v);
                    tc05_wait_ld16(v);
                    if (c0 == 112) {  // everything of this accumulator is in registers: hand it back
                        tc05_fence_before_sync();
                        __syncwarp();
                        if (lane == 0) mbar_arrive(&bar_acc_free[buf]);
                    }
#pragma unroll
                    for (int i = 0; i < 16; ++i) acc[c0 + i] = fmaf(scale, v[i], acc[c0 + i]);
                }
            }
            if (!ok) continue;
            if (mrow < M) {
                uint4 *o = reinterpret_cast<uint4 *>(out + (size_t)mrow * N + n0 + acol0);
#pragma unroll
                for (int i = 0; i < 16; ++i) {
                    __nv_bfloat162 p[4];
#pragma unroll
                    for (int j = 0; j < 4; ++j) p[j] = __floats2bfloat162_rn(acc[8 * i + 2 * j], acc[8 * i + 2 * j + 1]);
                    o[i] = *reinterpret_cast<uint4 *>(p);
                }
            }
        }
    } else {
        reg_dealloc<F8W_REG_OTHER>();
        if (TMA && warp == 8) {
            // ------------------------------------------------------------------------------------------- producer (TMA)
            uint32_t g = 0;
            bool ok = true;
            for (uint32_t tile = blockIdx.x; ok && tile < n_tiles; tile += gridDim.x) {
                const uint32_t mt = tile / n_nt, nt = tile - mt * n_nt, m0 = mt * 128, n0 = nt * F8W_TN;
                for (uint32_t kb = 0; kb < nkb; ++kb, ++g) {
                    const uint32_t s = g % F8W_STAGES, use = g / F8W_STAGES;
                    if (use >= 1) ok = mbar_wait_bounded(&bar_free[s], (use - 1) & 1u, status);
                    ok = __all_sync(FULL, ok);
                    if (!ok) break;
                    if (lane == 0) {
                        mbar_expect_tx(&bar_full[s], F8W_STAGE_A + F8W_STAGE_B);
                        tma_load_2d(smem + s * F8W_STAGE_A, &map_a, kb * 128, m0, &bar_full[s]);
                        tma_load_2d(smem + F8W_SMEM_B + s * F8W_STAGE_B, &map_w, kb * 128, n0, &bar_full[s]);
                    }
                    __syncwarp();
                }
            }
        } else if (!TMA && warp < 12) {
            // ------------------------------------------------------------------------------------------- producers
            const uint32_t ptid = tid - 256;
            uint32_t g = 0;
            bool ok = true;
            for (uint32_t tile = blockIdx.x; ok && tile < n_tiles; tile += gridDim.x) {
                const uint32_t mt = tile / n_nt, nt = tile - mt * n_nt, m0 = mt * 128, n0 = nt * F8W_TN;
                for (uint32_t kb = 0; kb < nkb; ++kb, ++g) {
                    const uint32_t s = g % F8W_STAGES, use = g / F8W_STAGES;
                    if (use >= 1) ok = mbar_wait_bounded(&bar_free[s], (use - 1) & 1u, status);
                    ok = __all_sync(FULL, ok);
                    if (!ok) break;
                    const uint32_t sa = smem_u32(smem + s * F8W_STAGE_A), sb = smem_u32(smem + F8W_SMEM_B + s * F8W_STAGE_B);
                    // chunk q of an operand block: row r = q / 8, 16-byte column c = q % 8; a warp instruction
                    // covers 4 rows x 128 contiguous bytes
#pragma unroll
                    for (int i = 0; i < 8; ++i) {
                        const uint32_t q = i * 128 + ptid, r = q >> 3, c = q & 7, m = m0 + r;
                        cp_async_16(sa + (r >> 3) * F8_SBO + c * 128 + (r & 7) * 16,
                                    a + (size_t)(m < M ? m : 0) * K + kb * 128 + 16 * c, m < M ? 16u : 0u);
                    }
#pragma unroll
                    for (int i = 0; i < 16; ++i) {
                        const uint32_t q = i * 128 + ptid, r = q >> 3, c = q & 7;
                        cp_async_16(sb + (r >> 3) * F8_SBO + c * 128 + (r & 7) * 16, w + (size_t)(n0 + r) * K + kb * 128 + 16 * c,
                                    16u);
                    }
                    // arrives on the barrier when this thread's copies above have landed
                    asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(smem_u32(&bar_full[s])) : "memory");
                }
            }
            asm volatile("cp.async.wait_all;" ::: "memory");
        } else if (warp == 12) {
            // ------------------------------------------------------------------------------------------- issuer
            const uint32_t idesc = tc05_idesc_e4m3(128, F8W_TN);
            uint32_t g = 0;
            bool ok = true;
            for (uint32_t tile = blockIdx.x; ok && tile < n_tiles; tile += gridDim.x) {
                for (uint32_t kb = 0; kb < nkb; ++kb, ++g) {
                    const uint32_t s = g % F8W_STAGES, buf = g & 1u;
                    ok = mbar_wait_bounded(&bar_full[s], (g / F8W_STAGES) & 1u, status);
                    if (g >= 2) ok = ok && mbar_wait_bounded(&bar_acc_free[buf], ((g >> 1) - 1) & 1u, status);
                    ok = __all_sync(FULL, ok);
                    fence_async_smem();  // the copies were written through the generic proxy
                    tc05_fence_after_sync();
                    if (elect_one()) {
                        if (ok) {
                            const uint32_t pa = smem_u32(smem + s * F8W_STAGE_A), pb = smem_u32(smem + F8W_SMEM_B + s * F8W_STAGE_B);
                            // unswizzled: K = 32 is two 128-byte core matrices = 256 bytes; swizzled: 32 bytes in the row
                            const uint64_t da = TMA ? tc05_smem_desc_sw128(pa) : tc05_smem_desc(pa, 128, F8_SBO);
                            const uint64_t db = TMA ? tc05_smem_desc_sw128(pb) : tc05_smem_desc(pb, 128, F8_SBO);
                            const uint32_t kstep = TMA ? 2u : 16u;
#pragma unroll
                            for (int ks = 0; ks < 4; ++ks)
                                tc05_mma_f8(tmem + buf * F8W_TN, da + kstep * ks, db + kstep * ks, idesc, ks != 0);
                        }
                        tc05_commit(&bar_free[s]);
                        tc05_commit(&bar_acc_full[buf]);
                    }
                    __syncwarp();
                    if (!ok) break;
                }
            }
        }
    }
    tc05_fence_before_sync();
    __syncthreads();
    if (warp == 0) tc05_dealloc(tmem, 512);
}

static bool fp8_ws_as_planned()
{
    static int state = -1;
    if (state < 0) {
        cudaFuncAttributes f;
        cudaFuncAttributes f2;
        state = cudaFuncGetAttributes(&f, fp8_gemm_ws_kernel<false>) == cudaSuccess && f.numRegs == F8W_REG_LAUNCH &&
                        cudaFuncGetAttributes(&f2, fp8_gemm_ws_kernel<true>) == cudaSuccess && f2.numRegs == F8W_REG_LAUNCH
                    ? 1 : 0;
    }
    return state == 1;
}

// Tensor maps are encoded on the host by a driver function, looked up once through the runtime (no link-time
// dependency on the driver library). Encoding allocates nothing and touches no device memory.
typedef CUresult (*tensor_map_encode_fn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                         const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                         CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static tensor_map_encode_fn tensor_map_encoder()
{
    static tensor_map_encode_fn fn = nullptr;
    static bool looked = false;
    if (!looked) {
        looked = true;
        void *p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<tensor_map_encode_fn>(p);
        cudaGetLastError();
    }
    return fn;
}

// bytes [rows][K] row-major, tiles of box_rows x 128 bytes, 128-byte swizzle, rows past the end read as zero
static bool encode_u8_rows(CUtensorMap *map, const uint8_t *base, uint32_t rows, uint32_t K, uint32_t box_rows)
{
    tensor_map_encode_fn enc = tensor_map_encoder();
    if (!enc || ((uintptr_t)base & 15) != 0 || K % 16 != 0) return false;
    const cuuint64_t dims[2] = {K, rows}, strides[1] = {K};
    const cuuint32_t box[2] = {128, box_rows}, estr[2] = {1, 1};
    return enc(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<uint8_t *>(base), dims, strides, box, estr,
               CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
               CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

int launch_fp8_linear(cudaStream_t st, const uint8_t *a, const float *a_scale, const uint8_t *w, const float *w_scale,
                      void *out_bf16, uint32_t M, uint32_t N, uint32_t K, int *status)
{
    if (M == 0 || N == 0) return 0;
    __nv_bfloat16 *out = reinterpret_cast<__nv_bfloat16 *>(out_bf16);
    if (M <= FP8_MV_MAX_M) {
        if (M == 1) fp8_matvec_kernel<1, 8><<<(N + 7) / 8, 256, 0, st>>>(a, a_scale, w, w_scale, out, M, N, K);
        else fp8_matvec_kernel<FP8_MV_MAX_M, 4><<<(N + 7) / 8, 256, 0, st>>>(a, a_scale, w, w_scale, out, M, N, K);
        return 1;
    }
    static OncePerDevice attr;
    if (attr.first()) {
        cudaFuncSetAttribute(fp8_gemm_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, F8_SMEM);
        cudaFuncSetAttribute(fp8_gemm_ws_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, F8W_SMEM);
        cudaFuncSetAttribute(fp8_gemm_ws_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, F8W_SMEM);
    }
    const int sms = sm_count_current();
    const char *no_ws = getenv("DSMOE_FP8_NO_WS"), *no_tma = getenv("DSMOE_FP8_NO_TMA");
    const uint32_t tiles = ((M + 127) / 128) * (N / F8W_TN);
    if (N % F8W_TN == 0 && K / 128 <= (uint32_t)F8W_MAX_KB && fp8_ws_as_planned() && !(no_ws && no_ws[0] == '1')) {
        const unsigned grid = tiles < (uint32_t)sms ? tiles : (uint32_t)sms;
        CUtensorMap map_a, map_w;
        memset(&map_a, 0, sizeof(map_a));
        memset(&map_w, 0, sizeof(map_w));
        // with tensor-map loads the persistent kernel wins at every M (even on a handful of tiles it finishes a tile in
        // half the lock-step kernel's time); with cp.async producers only when the tiles fill at least half the SMs
        if (!(no_tma && no_tma[0] == '1') && encode_u8_rows(&map_a, a, M, K, 128) && encode_u8_rows(&map_w, w, N, K, F8W_TN)) {
            fp8_gemm_ws_kernel<true><<<grid, F8W_THREADS, F8W_SMEM, st>>>(a, a_scale, w, w_scale, out, M, N, K, status, map_a, map_w);
            return 1;
        }
        if (M > 256 && tiles >= (uint32_t)sms / 2) {
            fp8_gemm_ws_kernel<false><<<grid, F8W_THREADS, F8W_SMEM, st>>>(a, a_scale, w, w_scale, out, M, N, K, status, map_a, map_w);
            return 1;
        }
    }
    fp8_gemm_kernel<<<dim3(N / 128, (M + 127) / 128), 256, F8_SMEM, st>>>(a, a_scale, w, w_scale, out, M, N, K, status);
    return 1;
}

}  // namespace dsmoe
