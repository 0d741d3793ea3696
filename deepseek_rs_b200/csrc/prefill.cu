// Batched (prefill) routed experts: pairs grouped by expert, then one grouped GEMM per projection on the tcgen05
// tensor cores.
//
// The reference runs the expert FFN one token at a time even in prefill (engine/src/session.rs:795-895); its
// sorted-pair and tile-list helpers (engine/src/kernels/moe.rs:299-362, 547-596) were written for a grouped GEMM that
// was never added. This file is that GEMM. To stay within rel 1e-3 of the reference, the contraction consumes what
// the reference's integer block dots consume: the Q8_K int8 activations and the integer weight codes
// (IQ2_XXS: ls * (+/-g), |code| <= 1333; Q2_K: sc_lo * q <= 45), both exact in f16, accumulated in f32 in TMEM per
// 256-wide superblock and scaled by d_w * d_x when the accumulator is drained — the same factorisation as
// engine/src/kernels/quantize.rs:811 and :900.
//
// Pipeline (all on the caller's stream, no host synchronisation):
//   1 pair_count / pair_plan / pair_place   stable counting sort of (token, slot) pairs by expert + token-tile list
//   2 gather_acts                           Q8_K rows of each tile -> f16 operand tiles in the tensor-core layout
//   3 grouped_gemm<IQ2>                     gate & up (64 + 64 rows per tile) -> gate and up row totals f32
//   4 swiglu_q8k, gather_acts               clamp, SwiGLU, router weight, Q8_K of mid in one pass; tiles of it
//   5 grouped_gemm<Q2K>                     down, min-term as a second K=16 MMA -> per-pair rows
//   6 moe_sum                               slots summed in slot order
#include <cuda_fp16.h>

#include "common.cuh"
#include "launch.h"
#include "tc05.cuh"

namespace dsmoe {

constexpr int PF_TN = 128;       // token rows per tile (MMA N), padded to a multiple of 16
constexpr int PF_KS = 128;       // K elements per pipeline stage (half a superblock)
constexpr int PF_STAGE_A = 128 * PF_KS * 2;  // 32 KB: 128 weight rows
constexpr int PF_SBO = (PF_KS / 8) * 128;    // 2048: byte distance between 8-row groups in a stage
constexpr int PF_DRAIN_WARPS = 8;    // consumers: two per TMEM lane quadrant, each draining PF_COLS accumulator columns
constexpr int PF_DECODE_WARPS = 16;  // producers: 8 weight rows each
constexpr int PF_AUX_WARPS = 4;      // MMA issuer, activation loader, two idle (register reallocation works on 4 warps)
constexpr int PF_THREADS = 32 * (PF_DRAIN_WARPS + PF_DECODE_WARPS + PF_AUX_WARPS);
constexpr int PF_COLS = PF_TN / (PF_DRAIN_WARPS / 4);
static_assert(PF_COLS == 64, "the drain reads its 64 TMEM columns per thread with two 32-column loads");
// Registers per thread. The kernel is compiled for PF_REG_LAUNCH (the most 896 threads can have); after the role
// split the producers and the auxiliary warps release registers and the consumers take them (setmaxnreg). An
// increase blocks until the CTA's warps have RELEASED as many registers as it asks for (registers the CTA never
// allocated do not count), so the released total must cover the request or the consumers would wait for ever.
constexpr int PF_REG_LAUNCH = 72;
#ifndef PF_REG_CONSUMER
#define PF_REG_CONSUMER 152
#define PF_REG_PRODUCER 40
#define PF_REG_AUX 32
#endif
static_assert(32 * PF_DRAIN_WARPS * (PF_REG_CONSUMER - PF_REG_LAUNCH) <=
                  32 * PF_DECODE_WARPS * (PF_REG_LAUNCH - PF_REG_PRODUCER) + 32 * PF_AUX_WARPS * (PF_REG_LAUNCH - PF_REG_AUX),
              "setmaxnreg: the consumers ask for more registers than the other roles release");
static_assert(PF_THREADS * PF_REG_LAUNCH <= 65536, "register file");

// ---------------------------------------------------------------------------------------------------------------
// 1. grouping: deterministic and stable (pairs of an expert keep ascending pair order), unlike the reference's
//    atomic-cursor scatter (engine/src/kernels/moe.rs:341-362)
// ---------------------------------------------------------------------------------------------------------------
__device__ __forceinline__ int pf_expert_of(const int32_t *selected, uint32_t p)
{
    const int32_t e = selected[p];
    return e < 0 ? 0 : e;  // engine/src/kernels/moe.rs:645-648
}

// counts[e] = number of pairs routed to e. One CTA per expert.
__global__ void __launch_bounds__(256) pf_count_kernel(const int32_t *__restrict__ selected, uint32_t n_pairs,
                                                        uint32_t *__restrict__ counts)
{
    __shared__ uint32_t s_warp[8];
    const int e = blockIdx.x;
    uint32_t c = 0;
    for (uint32_t p = threadIdx.x; p < n_pairs; p += 256) c += pf_expert_of(selected, p) == e;
#pragma unroll
    for (int m = 16; m > 0; m >>= 1) c += __shfl_xor_sync(FULL, c, m);
    if ((threadIdx.x & 31) == 0) s_warp[threadIdx.x >> 5] = c;
    __syncthreads();
    if (threadIdx.x == 0) {
        uint32_t t = 0;
        for (int w = 0; w < 8; ++w) t += s_warp[w];
        counts[e] = t;
    }
}

// offsets (exclusive prefix of counts) and the tile list: expert e contributes ceil(count / PF_TN) tiles.
// plan[0] = n_tiles, plan[1] = total padded rows. One warp: lane l owns a run of consecutive experts; three warp scans
// (pairs, tiles, padded rows) give each lane the bases its experts' entries start from.
__global__ void __launch_bounds__(32) pf_plan_kernel(const uint32_t *__restrict__ counts, int n_expert,
                                                      uint32_t *__restrict__ offsets, uint32_t *__restrict__ tile_expert,
                                                      uint32_t *__restrict__ tile_start, uint32_t *__restrict__ tile_rows,
                                                      uint32_t *__restrict__ tile_boff, uint32_t *__restrict__ plan)
{
    if (blockIdx.x != 0) return;
    const int lane = threadIdx.x, per = (n_expert + 31) / 32, e0 = lane * per, e1 = min(n_expert, e0 + per);
    uint32_t pairs = 0, tiles = 0, padded = 0;
    for (int e = e0; e < e1; ++e) {
        const uint32_t c = counts[e];
        pairs += c;
        tiles += (c + PF_TN - 1) / PF_TN;
        const uint32_t tail = c % PF_TN;
        padded += (c / PF_TN) * PF_TN + ((tail + 15u) & ~15u);
    }
    uint32_t sp = pairs, st = tiles, sb = padded;  // inclusive scans
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
        const uint32_t a = __shfl_up_sync(FULL, sp, d), b = __shfl_up_sync(FULL, st, d), c = __shfl_up_sync(FULL, sb, d);
        if (lane >= d) sp += a, st += b, sb += c;
    }
    uint32_t sum = sp - pairs, nt = st - tiles, boff = sb - padded;
    for (int e = e0; e < e1; ++e) {
        offsets[e] = sum;
        const uint32_t c = counts[e];
        for (uint32_t s0 = 0; s0 < c; s0 += PF_TN) {
            const uint32_t rows = min((uint32_t)PF_TN, c - s0);
            tile_expert[nt] = (uint32_t)e;
            tile_start[nt] = sum + s0;
            tile_rows[nt] = rows;
            tile_boff[nt] = boff;
            boff += (rows + 15u) & ~15u;
            ++nt;
        }
        sum += c;
    }
    if (lane == 31) {
        offsets[n_expert] = sp;
        tile_boff[st] = sb;
        plan[0] = st;
        plan[1] = sb;
    }
}

// sorted[offsets[e] + rank] = pair, rank = number of earlier pairs of the same expert. One CTA per expert; warp w
// owns the w-th contiguous eighth of the pairs: a first pass counts its hits, a prefix over the eight counts gives its
// base, a second pass places them (ballot ranks inside the warp, running count across its rounds).
__global__ void __launch_bounds__(256) pf_place_kernel(const int32_t *__restrict__ selected, uint32_t n_pairs,
                                                        const uint32_t *__restrict__ offsets,
                                                        uint32_t *__restrict__ sorted)
{
    __shared__ uint32_t s_warp[8];
    const int e = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const uint32_t seg = ((n_pairs + 7) / 8 + 31) & ~31u, p_lo = min(n_pairs, warp * seg), p_hi = min(n_pairs, p_lo + seg);
    uint32_t cnt = 0;
    for (uint32_t p0 = p_lo; p0 < p_hi; p0 += 32) {
        const uint32_t p = p0 + lane;
        cnt += __popc(__ballot_sync(FULL, p < p_hi && pf_expert_of(selected, p) == e));
    }
    if (lane == 0) s_warp[warp] = cnt;
    __syncthreads();
    uint32_t base = offsets[e];
    for (int w = 0; w < warp; ++w) base += s_warp[w];
    for (uint32_t p0 = p_lo; p0 < p_hi; p0 += 32) {
        const uint32_t p = p0 + lane;
        const bool hit = p < p_hi && pf_expert_of(selected, p) == e;
        const uint32_t ballot = __ballot_sync(FULL, hit);
        if (hit) sorted[base + __popc(ballot & ((1u << lane) - 1u))] = p;
        base += __popc(ballot);
    }
}

// ---------------------------------------------------------------------------------------------------------------
// 2. activation tiles. For tile t (rows16 = padded row count, boff = first padded row) the f16 operand occupies
//    rows16 * kblocks * 512 bytes at B + boff * kblocks * 512, ordered [stage = k / 128][row / 8][k % 128 / 8][row % 8]
//    [k % 8] so that one stage is one contiguous block in the layout the MMA descriptor describes.
//    Scales: S[kb * r_cap + boff + row] = d of the row's Q8_K block kb. bsums (Q2_K min term) as f16:
//    BS[(kb * r_cap + boff + row) * 16 + j], stored per tile in core-matrix order [kb][row / 8][j / 8][row % 8][j % 8].
//    src_row(p) = p / div_k (gate/up: the token's row) or p (down: the pair's row).
// ---------------------------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256) pf_gather_kernel(const uint8_t *__restrict__ q8k, uint32_t kblocks,
                                                         uint32_t div_k, const uint32_t *__restrict__ sorted,
                                                         const uint32_t *__restrict__ tile_start,
                                                         const uint32_t *__restrict__ tile_rows,
                                                         const uint32_t *__restrict__ tile_boff,
                                                         const uint32_t *__restrict__ plan, uint8_t *__restrict__ B,
                                                         float *__restrict__ S, __half *__restrict__ BS, uint32_t r_cap,
                                                         uint32_t perm)
{
    const uint32_t n_tiles = plan[0];
    // one warp per (tile, group of 8 padded rows, Q8_K block): lane = (row of the group r8, quarter q); in round j the
    // lane converts elements 8c..8c+7, c = q + 4j, so that the eight rows' pieces of one core matrix (128 contiguous
    // bytes of the operand tile) leave the warp together
    const uint32_t lane = threadIdx.x & 31, r8 = lane & 7, q = lane >> 3;
    for (uint32_t t = blockIdx.y; t < n_tiles; t += gridDim.y) {
        const uint32_t rows = tile_rows[t], rows16 = (rows + 15u) & ~15u, boff = tile_boff[t], start = tile_start[t];
        const uint32_t units = (rows16 >> 3) * kblocks;
        const size_t tile_base = (size_t)boff * kblocks * 512;
        for (uint32_t u = blockIdx.x * 8 + (threadIdx.x >> 5); u < units; u += gridDim.x * 8) {
            const uint32_t g8 = u / kblocks, kb = u - g8 * kblocks, r = 8 * g8 + r8;
            const bool valid = r < rows;
            const uint8_t *blk = valid ? q8k + ((size_t)(sorted[start + r] / div_k) * kblocks + kb) * Q8K_BYTES : q8k;
            const uint32_t *qs = reinterpret_cast<const uint32_t *>(blk + 4);
            const __half2 off = __floats2half2_rn(1152.0f, 1152.0f);
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const uint32_t c = q + 4 * j;
                uint32_t w0 = valid ? qs[2 * c] : 0u, w1 = valid ? qs[2 * c + 1] : 0u;
                // int8 -> f16 exactly: byte ^ 0x80 is the value + 128; 0x6400 | b is 1024 + b as f16
                w0 ^= 0x80808080u;
                w1 ^= 0x80808080u;
                uint32_t h[4] = {__byte_perm(w0, 0x64646464u, 0x4140u), __byte_perm(w0, 0x64646464u, 0x4342u),
                                 __byte_perm(w1, 0x64646464u, 0x4140u), __byte_perm(w1, 0x64646464u, 0x4342u)};
                uint4 o;
                uint32_t *op = reinterpret_cast<uint32_t *>(&o);
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    __half2 v = __hsub2(*reinterpret_cast<__half2 *>(&h[i]), off);
                    op[i] = *reinterpret_cast<uint32_t *>(&v);
                }
                // element k = 256 kb + 8 c. Plain order: stage 2 kb + c / 16, core column c % 16. Interleaved order
                // (perm, for the IQ2_XXS GEMM): the superblock's eight 32-element groups g = c / 4 alternate between its
                // two stages, group g in stage g % 2 at position g / 2, so that the two groups a decoding thread needs in
                // one superblock (2 j and 2 j + 1) are 16 adjacent bytes of the packed row. The order inside a superblock
                // does not matter to the contraction: its products are exact integers.
                const uint32_t st_half = perm ? ((c >> 2) & 1u) : (c >> 4), col = perm ? (4u * (c >> 3) + (c & 3u)) : (c & 15u);
                const size_t off_b = tile_base + (size_t)(2 * kb + st_half) * rows16 * 256 + (size_t)g8 * PF_SBO + col * 128 + r8 * 16;
                *reinterpret_cast<uint4 *>(B + off_b) = o;
            }
            if (q == 0) S[(size_t)kb * r_cap + boff + r] = valid ? *reinterpret_cast<const float *>(blk) : 0.0f;
            if (BS) {  // bsums 4q .. 4q+3 of the row, as f16, in core-matrix order [row / 8][j / 8][row % 8][j % 8]
                const uint32_t *bp = reinterpret_cast<const uint32_t *>(blk + 260);  // 4-byte aligned, not 8
                const uint2 raw = valid ? make_uint2(bp[2 * q], bp[2 * q + 1]) : make_uint2(0u, 0u);
                const __half2 lo = __halves2half2(__short2half_rn((short)(raw.x & 0xFFFFu)), __short2half_rn((short)(raw.x >> 16)));
                const __half2 hi = __halves2half2(__short2half_rn((short)(raw.y & 0xFFFFu)), __short2half_rn((short)(raw.y >> 16)));
                const size_t bs_tile = ((size_t)kb * r_cap + boff) * 16;
                uint2 out2;
                out2.x = *reinterpret_cast<const uint32_t *>(&lo);
                out2.y = *reinterpret_cast<const uint32_t *>(&hi);
                *reinterpret_cast<uint2 *>(BS + bs_tile + (size_t)g8 * 128 + (q >> 1) * 64 + r8 * 8 + (q & 1) * 4) = out2;
            }
        }
    }
}

// ---------------------------------------------------------------------------------------------------------------
// 3 / 5. grouped GEMM on tcgen05, warp-specialised
//
// One persistent CTA per SM (896 threads) walks items = (token tile, M tile). Four roles run asynchronously and meet
// only on mbarriers:
//   warps 8-23  producers  decode 128 weight rows x 128 K per stage (half a superblock) into a two-stage ring as
//                          exact f16 integers. Q2_K: the ring is in shared memory, 8 rows per warp. IQ2_XXS: the ring
//                          is in TENSOR memory (the MMA takes its A operand from there): a thread owns one row
//                          (= its TMEM lane), decodes one 32-weight group per stage in registers and writes it with
//                          one tcgen05.st, so the decoded weights never cross the shared-memory pipe, which the
//                          codebook lookups already keep busy;
//   warp 25     loader     bulk-copies the matching activation blocks (already f16, already in operand layout) into a
//                          three-stage ring, running ahead of the decode;
//   warp 24     issuer     one elected lane issues the stage's eight K=16 MMAs once both operands are there, and
//                          commits them to the rings' "free" mbarriers and, at the end of a superblock, to the
//                          accumulator's "full" mbarrier;
//   warps 0-7   consumers  drain the accumulator of a superblock (tcgen05.ld -> scale by d_w * d_x -> add to 64 f32
//                          registers per thread), hand the TMEM buffer back ("accumulator free") and write the item's
//                          result while the other roles already work on the next item.
// Registers move between the roles with setmaxnreg.
// TMEM (512 columns). Q2_K: two accumulator buffers (D at 0/128, min-term D2 at 256/384), so superblock j is drained
// while j+1 is contracted. IQ2_XXS: two accumulator buffers as well (columns 0-127 and 128-255), one spill set X
// (256..) and the two-stage ring of decoded weights (384.., 64 columns = 128 f16 per row and stage). The reference's
// reduction tree needs up to three spill sets, private to the draining thread: X, a second one (Y) in shared memory
// (64 KB, where the Q2_K kernel has its weight ring), and a third only while the tree's last leaf is being contracted:
// for that window (the last two superblocks of an item; the last one when a row has 8 blocks) accumulator buffer 1 is
// the spill set and buffer 0 works alone.
// IQ2_XXS tile rows: row 2r is gate row r and row 2r+1 the same row of up, so the two inputs of SwiGLU sit in
// neighbouring lanes of one warp and are exchanged with shuffles.
// Q2_K: the min term -dmin * d_x * sum_j bsums[j] * sc_hi[j] is a second accumulator fed by one K=16 MMA per
// superblock (A = sc_hi, B = bsums, both exact in f16).
// Every wait is bounded; on expiry the error is recorded and all threads leave through the common exit that frees
// TMEM. Consumers agree on the error at the item barrier, so nobody is left waiting on it.
// ---------------------------------------------------------------------------------------------------------------
struct PfGemmArgs {
    const uint8_t *w0, *w1;  // IQ2: gate, up tensors; Q2K: down tensor (w1 unused)
    uint64_t expert_bytes;
    const uint8_t *B;        // f16 activation tiles
    const float *S;          // [kblocks][r_cap] Q8_K scales
    const __half *BS;        // Q2K: bsums tiles
    uint32_t r_cap;
    const uint32_t *sorted, *tile_expert, *tile_start, *tile_rows, *tile_boff, *plan;
    const float *weights;    // IQ2: router weight per pair
    float *out;              // IQ2: gate row totals [pair][out_dim]; Q2K: per-pair down rows [pair][out_dim]
    float *out_u;            // IQ2: up row totals [pair][out_dim]
    float *const *row_ptr;   // Q2K, optional: row_ptr[pair] is where that pair's down row goes instead (it may point into
                             // another GPU's memory: the expert-parallel combine fused into this kernel's epilogue)
    uint32_t out_dim, kblocks;
    float clamp;
    int ieee, layout;
    int *status;
};

constexpr int PF_A_STAGES = 2, PF_B_STAGES = 3;
constexpr int PF_SMEM_A = 0;                                          // Q2K: 2 x 32 KB decoded weights; IQ2: spill set Y
constexpr uint32_t PF_TMEM_X = 256, PF_TMEM_A = 384;                    // IQ2: TMEM columns of spill set X and of the weight ring
constexpr uint32_t PF_TMEM_A_STAGE = PF_KS / 2;                          // 64 columns: 128 f16 per row
constexpr int PF_SMEM_B = PF_A_STAGES * PF_STAGE_A;                   // 3 x 32 KB activations
constexpr int PF_SMEM_LUT = PF_SMEM_B + PF_B_STAGES * PF_STAGE_A;     // IQ2: codebook magnitudes as f16 (32 KB: 8 copies of 256 entries)
constexpr int PF_SMEM_A2 = PF_SMEM_LUT;                               // Q2K (no tables): 2 x 4 KB sc_hi tile, one per TMEM buffer
constexpr int PF_SMEM_B2 = PF_SMEM_A2 + 8192;                         // Q2K: 2 x 4 KB bsums tile
constexpr int PF_SMEM_S = PF_SMEM_LUT + 49152;                        // per-item tables: 16 x 128 f32 activation scales,
constexpr int PF_SMEM_D = PF_SMEM_S + 16 * PF_TN * 4;                 //   16 x 128 raw weight-scale words,
constexpr int PF_SMEM_P = PF_SMEM_D + 16 * PF_TN * 4;                 //   128 pair ids,
constexpr int PF_SMEM_W = PF_SMEM_P + PF_TN * 4;                      //   128 router weights
constexpr int PF_SMEM_BAR = PF_SMEM_W + PF_TN * 4;
constexpr int PF_SMEM_TOTAL = PF_SMEM_BAR + 128;
static_assert(PF_SMEM_TOTAL <= 232448, "shared memory per CTA");

enum { PF_IQ2 = 0, PF_Q2K = 1 };

// 8 unsigned bytes (two words) -> 8 exact f16 integers; 0x6400 | b is 1024 + b
__device__ __forceinline__ uint4 pf_bytes_to_f16x8(uint32_t lo, uint32_t hi)
{
    const __half2 off = __floats2half2_rn(1024.0f, 1024.0f);
    uint32_t h[4] = {__byte_perm(lo, 0x64646464u, 0x4140u), __byte_perm(lo, 0x64646464u, 0x4342u),
                     __byte_perm(hi, 0x64646464u, 0x4140u), __byte_perm(hi, 0x64646464u, 0x4342u)};
    uint4 o;
    uint32_t *op = reinterpret_cast<uint32_t *>(&o);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        __half2 v = __hsub2(*reinterpret_cast<__half2 *>(&h[i]), off);
        op[i] = *reinterpret_cast<uint32_t *>(&v);
    }
    return o;
}

__device__ __forceinline__ uint32_t pf_hmul2(uint32_t a, uint32_t b)
{
    __half2 r = __hmul2(*reinterpret_cast<__half2 *>(&a), *reinterpret_cast<__half2 *>(&b));
    return *reinterpret_cast<uint32_t *>(&r);
}

// packed bytes of one (row, stage, quarter): IQ2: one 32-weight group (aux0, aux1); Q2K: 8 quant bytes
template <int KIND>
__device__ __forceinline__ uint2 pf_load_packed(const uint8_t *row, int layout, uint32_t kb, uint32_t half, uint32_t c)
{
    if (KIND == PF_IQ2) {  // stage `half` of a superblock holds groups half, 2 + half, 4 + half, 6 + half (see pf_gather_kernel)
        if (layout == DSMOE_LAYOUT_ROWSOA) return *reinterpret_cast<const uint2 *>(row + 32 + 64 * kb + 8 * (2 * c + half));
        const uint16_t *p = reinterpret_cast<const uint16_t *>(row + IQ2XXS_BYTES * kb + 2 + 8 * (2 * c + half));
        return make_uint2((uint32_t)p[0] | ((uint32_t)p[1] << 16), (uint32_t)p[2] | ((uint32_t)p[3] << 16));
    }
    if (layout == DSMOE_LAYOUT_ROWSOA) return *reinterpret_cast<const uint2 *>(row + 128 + 64 * kb + 32 * half + 8 * c);
    const uint32_t *p = reinterpret_cast<const uint32_t *>(row + Q2K_BYTES * kb + 16 + 32 * half + 8 * c);
    return make_uint2(p[0], p[1]);
}

// the 8 scale bytes of sub-blocks 8*half .. 8*half+7 of Q2_K block kb
__device__ __forceinline__ uint2 pf_load_q2k_scales(const uint8_t *row, int layout, uint32_t kb, uint32_t half)
{
    const uint8_t *p = layout == DSMOE_LAYOUT_ROWSOA ? row + 16 * kb + 8 * half : row + Q2K_BYTES * kb + 8 * half;
    const uint32_t *q = reinterpret_cast<const uint32_t *>(p);
    return make_uint2(q[0], q[1]);
}

// the 16 scale bytes of Q2_K block kb
__device__ __forceinline__ uint4 pf_load_q2k_scales16(const uint8_t *row, int layout, uint32_t kb)
{
    if (layout == DSMOE_LAYOUT_ROWSOA) return *reinterpret_cast<const uint4 *>(row + 16 * kb);
    const uint32_t *q = reinterpret_cast<const uint32_t *>(row + Q2K_BYTES * kb);
    return make_uint4(q[0], q[1], q[2], q[3]);
}

// IQ2_XXS for the tensor-memory ring: decode one 32-weight group into 16 words (f16 pairs in K order).
// Magnitudes: one 16-byte lookup per 8 weights in a table of f16 magnitudes (8 copies of every entry, entry stride 128
// bytes, copy = lane & 7, so the eight lanes of a 128-bit shared-memory wavefront never share a bank group), scaled by
// ls with one packed multiply per two weights. Signs are computed: the sign byte of a 7-bit index is the index with
// its parity as bit 7 (engine/src/kernels/quantize.rs:693-708), and one multiplication by 2^(15-2i) + 2^(30-2i) moves
// bits 2i and 2i+1 of that byte to the f16 sign positions 15 and 31 of word i, where one logic operation flips the two
// magnitudes. (A byte-wide table with a PRMT + fused multiply-add conversion reads a quarter of the shared-memory
// wavefronts but costs four more instructions per 8 weights; the kernel is bound by instruction issue, so this form wins.)
__device__ __forceinline__ void pf_decode_iq2_regs(uint2 pk, uint32_t (&w)[16], const uint4 *lut_grid, uint32_t lane7)
{
    const uint32_t aux0 = pk.x, aux1 = pk.y;
    const __half2 ls = __float2half2_rn((float)(2u * (aux1 >> 28) + 1u));
    const uint32_t ls2 = *reinterpret_cast<const uint32_t *>(&ls);
#pragma unroll
    for (int u = 0; u < 4; ++u) {
        const uint4 g = lut_grid[((aux0 >> (8 * u)) & 255u) * 8 + lane7];
        const uint32_t idx = (aux1 >> (7 * u)) & 127u, sb = idx | ((__popc(idx) & 1u) << 7);
        w[4 * u + 0] = pf_hmul2(g.x, ls2) ^ ((sb * 0x40008000u) & 0x80008000u);
        w[4 * u + 1] = pf_hmul2(g.y, ls2) ^ ((sb * 0x10002000u) & 0x80008000u);
        w[4 * u + 2] = pf_hmul2(g.z, ls2) ^ ((sb * 0x04000800u) & 0x80008000u);
        w[4 * u + 3] = pf_hmul2(g.w, ls2) ^ ((sb * 0x01000200u) & 0x80008000u);
    }
}

// Q2_K: 8 quant bytes (quarter c of half-block `half`) -> units j = 0..3 (k = 32 j + 8 c + i), value sc_lo[j] * q,
// at dst + j * 512. sc8 = the 8 scale bytes of sub-blocks 8*half .. +7; sub-block of unit j is 2 j + c / 2.
__device__ __forceinline__ void pf_decode_q2k(uint2 pk, uint2 sc8, uint32_t c, uint8_t *dst)
{
    const uint32_t sc4 = __byte_perm(sc8.x, sc8.y, (c & 2) ? 0x7531u : 0x6420u) & 0x0F0F0F0Fu;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        const uint32_t sc = (sc4 >> (8 * j)) & 0xFFu;
        const uint32_t lo = ((pk.x >> (2 * j)) & 0x03030303u) * sc, hi = ((pk.y >> (2 * j)) & 0x03030303u) * sc;
        *reinterpret_cast<uint4 *>(dst + j * 512) = pf_bytes_to_f16x8(lo, hi);
    }
}

// Order in which the superblocks of a row are contracted. Q2_K: ascending. IQ2_XXS: the post-order of the reference's
// reduction tree, so that the f32 partial sums can be folded exactly as the reference folds them
// (engine/src/kernels/moe.rs:37-42, 661-690: lane partial a_l = (0 + dot_l) + dot_(l+8), then
// ((a0+a4)+(a2+a6)) + ((a1+a5)+(a3+a7))) with only two live register sets. Leaf order l = 0,4,2,6,1,5,3,7; with 16
// blocks per row visit j covers block l(j/2) + 8 (j%2), with 8 blocks visit j covers block l(j).
template <int KIND>
__device__ __forceinline__ uint32_t pf_visit_block(uint32_t kblocks, uint32_t j)
{
    if (KIND == PF_Q2K) return j;
    const uint32_t leaf = kblocks == 16 ? (j >> 1) : j;
    const uint32_t l = (0x73516240u >> (4 * leaf)) & 7u;
    return kblocks == 16 ? l + 8 * (j & 1) : l;
}

// Accumulator buffer (0 or 1) that superblock j of an item is contracted into. gsb = superblocks this CTA has started
// before it. Q2_K alternates for ever. IQ2_XXS alternates inside an item up to the blocks of the tree's last leaf,
// which use buffer 0 only: buffer 1 then holds a spill set (see the TMEM note above).
template <int KIND>
__device__ __forceinline__ uint32_t pf_acc_buf(uint32_t kblocks, uint32_t j, uint32_t gsb)
{
    if (KIND == PF_Q2K) return gsb & 1u;
    const uint32_t single_from = kblocks == 16 ? 14u : kblocks - 1u;
    return j < single_from ? (j & 1u) : 0u;
}
// IQ2_XXS: the last superblock of an item that is contracted into buffer 1. The consumers hand buffer 1 back only at
// the end of the item, after the spill set parked in it has been read.
__device__ __forceinline__ uint32_t pf_last_buf1_block(uint32_t kblocks) { return kblocks == 16 ? 13u : kblocks - 3u; }

// Weight row behind row `rl` of an item's 128-row operand tile.
template <int KIND>
__device__ __forceinline__ const uint8_t *pf_tile_row(const PfGemmArgs &a, uint64_t ebase, uint32_t mt, uint32_t rl,
                                                      uint32_t row_bytes)
{
    if (KIND == PF_IQ2) return ((rl & 1u) ? a.w1 : a.w0) + ebase + (uint64_t)(mt * 64 + (rl >> 1)) * row_bytes;
    return a.w0 + ebase + (uint64_t)(mt * 128 + rl) * row_bytes;
}

// Asks L2 for the weight rows of an item (contiguous per tensor) so that the decode loads and the scale loads of the
// item find them there. `t` of `nt` threads share the lines.
template <int KIND>
__device__ __forceinline__ void pf_prefetch_item(const PfGemmArgs &a, uint32_t item, uint32_t n_mtiles, uint32_t row_bytes,
                                                 uint32_t t, uint32_t nt)
{
    const uint32_t tile = item / n_mtiles, mt = item - tile * n_mtiles;
    const uint64_t ebase = (uint64_t)a.tile_expert[tile] * a.expert_bytes;
    const uint32_t m_out = KIND == PF_IQ2 ? 64u : 128u, bytes = m_out * row_bytes;
    const uint8_t *p0 = a.w0 + ebase + (uint64_t)mt * bytes;
    for (uint32_t o = t * 128u; o < bytes; o += nt * 128u) asm volatile("prefetch.global.L2 [%0];" ::"l"(p0 + o));
    if (KIND == PF_IQ2) {
        const uint8_t *p1 = a.w1 + ebase + (uint64_t)mt * bytes;
        for (uint32_t o = t * 128u; o < bytes; o += nt * 128u) asm volatile("prefetch.global.L2 [%0];" ::"l"(p1 + o));
    }
}

template <int KIND>
__global__ void __launch_bounds__(PF_THREADS, 1) pf_grouped_gemm_kernel(PfGemmArgs a)
{
    extern __shared__ __align__(1024) uint8_t smem[];
    uint64_t *bar_a_full = reinterpret_cast<uint64_t *>(smem + PF_SMEM_BAR);  // [2] weight stage decoded (16 warps)
    uint64_t *bar_a_free = bar_a_full + 2;                                     // [2] its MMAs retired
    uint64_t *bar_b_full = bar_a_full + 4;                                     // [3] activation stage landed
    uint64_t *bar_b_free = bar_a_full + 7;                                     // [3] its MMAs retired
    uint64_t *bar_acc_full = bar_a_full + 10;                                  // [2] superblock contracted
    uint64_t *bar_acc_free = bar_a_full + 12;                                  // [2] accumulator drained (8 warps)
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(bar_a_full + 14);
    uint4 *lut_grid = reinterpret_cast<uint4 *>(smem + PF_SMEM_LUT);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    constexpr uint32_t TMEM_COLS = 512u;
    constexpr uint32_t M_OUT = KIND == PF_IQ2 ? 64u : 128u;  // output rows per tile
    const bool ieee = a.ieee != 0;

    if (KIND == PF_IQ2) {
        for (int i = tid; i < 256 * 8; i += PF_THREADS) {
            const uint64_t g = c_iq2xxs_grid[i >> 3];
            lut_grid[i] = pf_bytes_to_f16x8((uint32_t)g, (uint32_t)(g >> 32));
        }
    }
    if (warp == 0) tc05_alloc(tmem_slot, TMEM_COLS);
    if (tid == 0) {
        for (int i = 0; i < PF_A_STAGES; ++i) {
            mbar_init(&bar_a_full[i], PF_DECODE_WARPS);
            mbar_init(&bar_a_free[i], 1);
        }
        for (int i = 0; i < PF_B_STAGES; ++i) {
            mbar_init(&bar_b_full[i], 1);
            mbar_init(&bar_b_free[i], 1);
        }
        for (int i = 0; i < 2; ++i) {
            mbar_init(&bar_acc_full[i], 1);
            mbar_init(&bar_acc_free[i], PF_DRAIN_WARPS);
        }
        fence_async_smem();
    }
    tc05_fence_before_sync();
    __syncthreads();
    tc05_fence_after_sync();
    const uint32_t tmem = *tmem_slot;

    const uint32_t n_tiles = a.plan[0], n_mtiles = a.out_dim / M_OUT, n_items = n_tiles * n_mtiles;
    const uint32_t n_stages = 2 * a.kblocks;
    const uint32_t row_bytes = (KIND == PF_IQ2 ? IQ2XXS_BYTES : Q2K_BYTES) * a.kblocks;

    if (warp < PF_DRAIN_WARPS) {
        // ------------------------------------------------------------------------------------------- consumers
        reg_alloc<PF_REG_CONSUMER>();
        // accumulator row (TMEM lane) and column half of this thread
        const uint32_t arow = 32 * (warp & 3) + lane, acol0 = PF_COLS * (warp >> 2);
        const uint32_t tlane = (32u * (warp & 3)) << 16;
        uint32_t gsb = 0, use0 = 0, use1 = 0;  // superblocks drained so far, and per accumulator buffer (mbarrier phase)
        bool ok = true;

        for (uint32_t item = blockIdx.x; item < n_items; item += gridDim.x) {
            const uint32_t tile = item / n_mtiles, mt = item - tile * n_mtiles;
            const uint32_t rows = a.tile_rows[tile], rows16 = (rows + 15u) & ~15u, boff = a.tile_boff[tile];
            const uint32_t start = a.tile_start[tile];
            const uint64_t ebase = (uint64_t)a.tile_expert[tile] * a.expert_bytes;
            const uint8_t *srow = pf_tile_row<KIND>(a, ebase, mt, arow, row_bytes);  // the row whose scales apply here

            // per-item tables: activation scales, this tile's weight scales (raw bits: IQ2 d as f16, Q2K d | dmin << 16),
            // pair ids. They are rewritten once every warp is done with the previous item's.
            float *sS = reinterpret_cast<float *>(smem + PF_SMEM_S);
            uint32_t *sD = reinterpret_cast<uint32_t *>(smem + PF_SMEM_D);
            uint32_t *sP = reinterpret_cast<uint32_t *>(smem + PF_SMEM_P);
            ok = named_barrier_and(1, 32 * PF_DRAIN_WARPS, ok);
            if (!ok) break;  // the same decision in all consumer warps
            if ((uint32_t)(tid & (PF_TN - 1)) < rows16)
                for (uint32_t kb = tid / PF_TN; kb < a.kblocks; kb += 32 * PF_DRAIN_WARPS / PF_TN)
                    sS[kb * PF_TN + (tid & (PF_TN - 1))] = a.S[(size_t)kb * a.r_cap + boff + (tid & (PF_TN - 1))];
            for (uint32_t kb = tid / PF_TN; kb < a.kblocks; kb += 32 * PF_DRAIN_WARPS / PF_TN) {  // row arow = tid % 128
                uint32_t bits;
                if (KIND == PF_IQ2) bits = a.layout == DSMOE_LAYOUT_ROWSOA ? ld_u16(srow + 2 * kb) : ld_u16(srow + IQ2XXS_BYTES * kb);
                else bits = a.layout == DSMOE_LAYOUT_ROWSOA ? ld_u32(srow + 80 * a.kblocks + 4 * kb) : ld_u32(srow + Q2K_BYTES * kb + 80);
                sD[kb * PF_TN + arow] = bits;
            }
            if ((uint32_t)tid < rows) {
                const uint32_t pair = a.sorted[start + tid];
                sP[tid] = pair;

            }
            named_barrier_sync(1, 32 * PF_DRAIN_WARPS);

            // Q2K: running sum. IQ2: the current leaf's partial a_l, after the last leaf the row total
            float acc[PF_COLS];
#pragma unroll
            for (int i = 0; i < PF_COLS; ++i) acc[i] = 0.0f;

            for (uint32_t j = 0; j < a.kblocks; ++j) {
                if (!ok) break;  // keeps walking the items, so that every warp reaches the item barriers
                const uint32_t buf = pf_acc_buf<KIND>(a.kblocks, j, gsb), use = buf ? use1 : use0;
                const uint32_t kb = pf_visit_block<KIND>(a.kblocks, j);
                // IQ2: buffer 1 stays with the consumers after its last superblock of the item (it becomes a spill set)
                const bool keep_buf = KIND == PF_IQ2 && j == pf_last_buf1_block(a.kblocks);
                // IQ2: position of this block in the reference's reduction tree
                const uint32_t leaf = a.kblocks == 16 ? (j >> 1) : j;
                const bool first_of_leaf = a.kblocks == 16 ? (j & 1) == 0 : true;
                const bool last_of_leaf = a.kblocks == 16 ? (j & 1) == 1 : true;
                const uint32_t sc_bits = sD[kb * PF_TN + arow];
                ok = mbar_wait_bounded(&bar_acc_full[buf], use & 1u, a.status);
                ok = __all_sync(FULL, ok);
                if (!ok) break;
                tc05_fence_after_sync();
                float dw, dmin = 0.0f;
                if (KIND == PF_IQ2) {
                    dw = __fmul_rn(0.125f, f16_bits_to_f32(sc_bits, ieee));
                } else {
                    dw = f16_bits_to_f32(sc_bits & 0xFFFFu, ieee);
                    dmin = f16_bits_to_f32(sc_bits >> 16, ieee);
                }
                const float4 *sx4 = reinterpret_cast<const float4 *>(sS + kb * PF_TN + acol0);
                if (KIND == PF_IQ2) {
                    // One accumulator buffer: it goes back to the issuer as soon as this thread's columns are in
                    // registers, so that the next superblock's MMAs overlap the arithmetic.
                    // ((0.125 d_w) d_x) bsum is added to 0 (first block of a leaf) or to the leaf's first block.
                    auto release = [&]() {
                        if (keep_buf) return;
                        tc05_fence_before_sync();
                        __syncwarp();
                        if (lane == 0) mbar_arrive(&bar_acc_free[buf]);
                    };
                    auto scaled = [&](int c0, const float *v, bool first) {  // 16 columns from c0; v = their bsums
                        float dxs[16];
#pragma unroll
                        for (int i = 0; i < 4; ++i) {
                            const float4 t = sx4[(c0 >> 2) + i];
                            dxs[4 * i] = t.x, dxs[4 * i + 1] = t.y, dxs[4 * i + 2] = t.z, dxs[4 * i + 3] = t.w;
                        }
#pragma unroll
                        // The two multiplications run two columns per instruction; the addition stays scalar, because
                        // the assembler contracts a packed multiply feeding a packed add into a fused multiply-add
                        // (measured: one sample in ten then differs from the separately rounded result).
#pragma unroll
                        for (int i = 0; i < 16; i += 2) {
                            const f32x2 t = fmul2_rn(fmul2_rn(f32x2{dw, dw}, f32x2{dxs[i], dxs[i + 1]}), f32x2{v[i], v[i + 1]});
                            acc[c0 + i] = __fadd_rn(first ? 0.0f : acc[c0 + i], t.x);
                            acc[c0 + i + 1] = __fadd_rn(first ? 0.0f : acc[c0 + i + 1], t.y);
                        }
                    };
                    if (first_of_leaf) {  // acc is dead: load all 64 columns into it, release, scale in place
                        if (acol0 < rows16) {  // warp-uniform: columns beyond the padded tile hold nothing
                            tc05_ld32(tmem + tlane + buf * PF_TN + acol0, acc);
                            if (acol0 + 32 < rows16) tc05_ld32(tmem + tlane + buf * PF_TN + acol0 + 32, acc + 32);
                            tc05_wait_ld32(acc);
                            tc05_wait_ld32(acc + 32);
                        }
                        release();
#pragma unroll
                        for (int c0 = 0; c0 < PF_COLS; c0 += 16) {
                            if (acol0 + c0 >= rows16) break;
                            scaled(c0, acc + c0, true);
                        }
                    } else {              // acc is live: two halves through 32 registers
                        float v[32];
#pragma unroll
                        for (int h = 0; h < 2; ++h) {
                            if (acol0 + 32 * h < rows16) {
                                tc05_ld32(tmem + tlane + buf * PF_TN + acol0 + 32 * h, v);
                                tc05_wait_ld32(v);
                            }
                            if (h == 1) release();
#pragma unroll
                            for (int c0 = 32 * h; c0 < 32 * h + 32; c0 += 16) {
                                if (acol0 + c0 >= rows16) break;
                                scaled(c0, v + (c0 - 32 * h), false);
                            }
                        }
                    }
                } else {
#pragma unroll
                    for (int c0 = 0; c0 < PF_COLS; c0 += 16) {
                        if (acol0 + c0 >= rows16) break;
                        float v[16], v2[16];
                        tc05_ld16(tmem + tlane + buf * PF_TN + acol0 + c0, v);
                        tc05_ld16(tmem + tlane + 256u + buf * PF_TN + acol0 + c0, v2);
                        tc05_wait_ld16(v);
                        tc05_wait_ld16(v2);
                        float dxs[16];
#pragma unroll
                        for (int i = 0; i < 4; ++i) {
                            const float4 t = sx4[(c0 >> 2) + i];
                            dxs[4 * i] = t.x, dxs[4 * i + 1] = t.y, dxs[4 * i + 2] = t.z, dxs[4 * i + 3] = t.w;
                        }
#pragma unroll
                        for (int i = 0; i < 16; i += 2) {  // packed multiplications, scalar subtraction and addition
                            const f32x2 dx = f32x2{dxs[i], dxs[i + 1]};
                            const f32x2 p = fmul2_rn(fmul2_rn(dx, f32x2{dw, dw}), f32x2{v[i], v[i + 1]});
                            const f32x2 m = fmul2_rn(fmul2_rn(dx, f32x2{dmin, dmin}), f32x2{v2[i], v2[i + 1]});
                            acc[c0 + i] = __fadd_rn(acc[c0 + i], __fsub_rn(p.x, m.x));
                            acc[c0 + i + 1] = __fadd_rn(acc[c0 + i + 1], __fsub_rn(p.y, m.y));
                        }
                    }
                    // both accumulators have been read: hand the buffer back to the issuer
                    tc05_fence_before_sync();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(&bar_acc_free[buf]);
                }
                ++gsb;
                if (buf) ++use1;
                else ++use0;

                if (KIND == PF_IQ2 && last_of_leaf) {
                    // Fold the finished leaf a_l (in acc) into the tree ((a0+a4)+(a2+a6)) + ((a1+a5)+(a3+a7)); the
                    // leaves arrive in the order 0 4 2 6 1 5 3 7. Spill sets of this thread: X in its TMEM lane, Y in
                    // shared memory (column-major, so that the 32 lanes of a warp touch 32 different banks), and for
                    // the last leaf accumulator buffer 1, whose last superblock of the item has been drained by then.
                    // Stores to the spill sets are only waited for here, right before the next access to them.
                    float *ys = reinterpret_cast<float *>(smem + PF_SMEM_A) + arow;
                    tc05_wait_st();
#pragma unroll
                    for (int c0 = 0; c0 < PF_COLS; c0 += 32) {
                        if (acol0 + c0 >= rows16) break;
                        const uint32_t tx = tmem + tlane + PF_TMEM_X + acol0 + c0, tz = tmem + tlane + PF_TN + acol0 + c0;
                        float *y = ys + (acol0 + c0) * 128;
                        float e[32];
                        if (leaf == 0 || leaf == 6) {              // a0 -> X, a3 -> buffer 1
                            tc05_st32(leaf == 0 ? tx : tz, acc + c0);
                        } else if (leaf == 2 || leaf == 4) {       // a2 -> Y, a1 -> Y
#pragma unroll
                            for (int i = 0; i < 32; ++i) y[i * 128] = acc[c0 + i];
                        } else if (leaf == 1) {                    // X = a0 + a4
                            tc05_ld32(tx, e);
                            tc05_wait_ld32(e);
#pragma unroll
                            for (int i = 0; i < 32; ++i) e[i] = __fadd_rn(e[i], acc[c0 + i]);
                            tc05_st32(tx, e);
                        } else if (leaf == 5) {                    // Y = a1 + a5
#pragma unroll
                            for (int i = 0; i < 32; ++i) y[i * 128] = __fadd_rn(y[i * 128], acc[c0 + i]);
                        } else if (leaf == 3) {                    // X = (a0 + a4) + (a2 + a6): the even half
                            tc05_ld32(tx, e);
                            tc05_wait_ld32(e);
#pragma unroll
                            for (int i = 0; i < 32; ++i) e[i] = __fadd_rn(e[i], __fadd_rn(y[i * 128], acc[c0 + i]));
                            tc05_st32(tx, e);
                        } else {                                   // row total = X + ((a1 + a5) + (a3 + a7))
                            tc05_ld32(tz, e);
                            tc05_wait_ld32(e);
#pragma unroll
                            for (int i = 0; i < 32; ++i) acc[c0 + i] = __fadd_rn(y[i * 128], __fadd_rn(e[i], acc[c0 + i]));
                            tc05_ld32(tx, e);
                            tc05_wait_ld32(e);
#pragma unroll
                            for (int i = 0; i < 32; ++i) acc[c0 + i] = __fadd_rn(e[i], acc[c0 + i]);
                        }
                    }
                }
                if (KIND == PF_IQ2 && last_of_leaf && leaf == 7) {
                    // the spill set in buffer 1 has been read: the issuer may have the buffer again
                    tc05_fence_before_sync();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(&bar_acc_free[1]);
                }
            }
            if (!ok) continue;

            // the item's result
            if (KIND == PF_IQ2) {
                // Lanes 2r / 2r+1 hold gate / up of output row r. The row totals go out as they are, gate rows to
                // a.out and up rows to a.out_u: clamp, SwiGLU, router weight and the Q8_K quantisation of the result
                // run in the kernel that follows (swiglu_q8k_kernel), at full occupancy instead of on these eight warps.
                float *dst = ((lane & 1) ? a.out_u : a.out) + mt * 64 + (arow >> 1);
#pragma unroll
                for (int i0 = 0; i0 < PF_COLS; i0 += 8) {
                    if (acol0 + i0 >= rows) break;
                    uint32_t pr[8];
#pragma unroll
                    for (int q = 0; q < 2; ++q) {
                        const uint4 t = *reinterpret_cast<const uint4 *>(sP + acol0 + i0 + 4 * q);
                        pr[4 * q] = t.x, pr[4 * q + 1] = t.y, pr[4 * q + 2] = t.z, pr[4 * q + 3] = t.w;
                    }
#pragma unroll
                    for (int k = 0; k < 8; ++k)
                        if (acol0 + i0 + k < rows) dst[(size_t)pr[k] * a.out_dim] = acc[i0 + k];
                }
            } else {
                float *orow = a.out + mt * 128 + arow;
#pragma unroll
                for (int i0 = 0; i0 < PF_COLS; i0 += 8) {
                    if (acol0 + i0 >= rows) break;
                    uint32_t pr[8];
#pragma unroll
                    for (int q = 0; q < 2; ++q) {
                        const uint4 t = *reinterpret_cast<const uint4 *>(sP + acol0 + i0 + 4 * q);
                        pr[4 * q] = t.x, pr[4 * q + 1] = t.y, pr[4 * q + 2] = t.z, pr[4 * q + 3] = t.w;
                    }
                    if (a.row_ptr != nullptr) {
                        // plain stores through the row's own pointer: the 32 lanes of a warp write 128 contiguous bytes
                        // of one row, local or across NVLink
#pragma unroll
                        for (int k = 0; k < 8; ++k)
                            if (acol0 + i0 + k < rows) a.row_ptr[pr[k]][mt * 128 + arow] = acc[i0 + k];
                    } else {
#pragma unroll
                        for (int k = 0; k < 8; ++k)
                            if (acol0 + i0 + k < rows) orow[(size_t)pr[k] * a.out_dim] = acc[i0 + k];
                    }
                }
            }
        }
    } else if (warp < PF_DRAIN_WARPS + PF_DECODE_WARPS) {
        // ------------------------------------------------------------------------------------------- producers
        reg_dealloc<PF_REG_PRODUCER>();
        const uint32_t dwarp = warp - PF_DRAIN_WARPS, dtid = tid - 32 * PF_DRAIN_WARPS;
        // This thread in the decode. Q2_K: lane = c * 8 + r8 -> quarter c of the stage, tile row 8 dwarp + r8.
        // IQ2_XXS: a warp can only write the TMEM lanes of its own quadrant (warp index mod 4), so the thread's row is
        // 32 * (warp % 4) + lane and the warp's quarter of the stage is dwarp / 4.
        const uint32_t dc = KIND == PF_IQ2 ? (dwarp >> 2) : (lane >> 3), dr8 = lane & 7;
        const uint32_t rl = KIND == PF_IQ2 ? 32u * (warp & 3u) + lane : 8 * dwarp + dr8;
        uint32_t gs = 0, gsb = 0;  // stages / superblocks started so far by this CTA (ring slot and mbarrier phase)
        bool ok = true;

        // Row pointer of this thread in an item's operand tile
        auto item_row = [&](uint32_t item) -> const uint8_t * {
            const uint32_t tile = item / n_mtiles, mt = item - tile * n_mtiles;
            return pf_tile_row<KIND>(a, (uint64_t)a.tile_expert[tile] * a.expert_bytes, mt, rl, row_bytes);
        };
        // Packed bytes (and Q2_K scale bytes) are requested one whole superblock ahead, across item boundaries too, and
        // BEFORE the wait for a free ring slot: a load from L2 takes about as long as a stage, so a request made only
        // once the slot is free would sit on the critical path of every stage. Two register sets (A: even superblocks,
        // B: odd ones; a row has an even number of superblocks) alternate, so that a fetched value is first touched by
        // the decode that needs it.
        uint2 pA0 = make_uint2(0, 0), pA1 = pA0, pB0 = pA0, pB1 = pA0;
        uint4 scA = make_uint4(0, 0, 0, 0), scB = scA;
        const uint8_t *drow = nullptr;
        if (blockIdx.x < n_items) {
            pf_prefetch_item<KIND>(a, blockIdx.x, n_mtiles, row_bytes, dtid, 32 * PF_DECODE_WARPS);
            drow = item_row(blockIdx.x);
            const uint32_t kb0 = pf_visit_block<KIND>(a.kblocks, 0);
            pA0 = pf_load_packed<KIND>(drow, a.layout, kb0, 0, dc);
            pA1 = pf_load_packed<KIND>(drow, a.layout, kb0, 1, dc);
            if (KIND == PF_Q2K) scA = pf_load_q2k_scales16(drow, a.layout, kb0);
        }
        for (uint32_t item = blockIdx.x; ok && item < n_items; item += gridDim.x) {
            const bool has_next = item + gridDim.x < n_items;
            if (has_next) pf_prefetch_item<KIND>(a, item + gridDim.x, n_mtiles, row_bytes, dtid, 32 * PF_DECODE_WARPS);
            const uint8_t *drow_next = has_next ? item_row(item + gridDim.x) : nullptr;

            auto stage = [&](uint32_t s, const uint2 &cur, const uint4 &sc) -> bool {
                const uint32_t b = gs & 1u, half = s & 1u;
                // the ring slot is free once the MMAs of the stage issued two stages ago have retired
                if (gs >= 2) ok = mbar_wait_bounded(&bar_a_free[b], ((gs >> 1) - 1) & 1u, a.status);
                ok = __all_sync(FULL, ok);
                if (!ok) return false;
                if (KIND == PF_IQ2) tc05_fence_after_sync();  // the MMAs that read this TMEM stage have retired
                uint8_t *dst = smem + PF_SMEM_A + b * PF_STAGE_A + (rl >> 3) * PF_SBO + (rl & 7) * 16;
                if (KIND == PF_IQ2) {
                    // group dc of the stage -> K elements 32 dc .. 32 dc + 31 -> 16 columns of this row's TMEM lane
                    uint32_t wreg[16];
                    pf_decode_iq2_regs(cur, wreg, lut_grid, dr8);
                    tc05_st16_u32(tmem + ((32u * (warp & 3u)) << 16) + PF_TMEM_A + b * PF_TMEM_A_STAGE + 16u * dc, wreg);
                    tc05_wait_st();
                    tc05_fence_before_sync();
                } else {
                    pf_decode_q2k(cur, half ? make_uint2(sc.z, sc.w) : make_uint2(sc.x, sc.y), dc, dst + dc * 128);
                    if (half == 0 && dc < 2) {  // sc_hi of sub-blocks 8 dc .. 8 dc + 7 -> min-term operand, core dc
                        const uint2 sh = dc ? make_uint2(sc.z, sc.w) : make_uint2(sc.x, sc.y);
                        *reinterpret_cast<uint4 *>(smem + PF_SMEM_A2 + (gsb & 1u) * 4096 + (rl >> 3) * 256 + dc * 128 +
                                                   (rl & 7) * 16) =
                            pf_bytes_to_f16x8((sh.x >> 4) & 0x0F0F0F0Fu, (sh.y >> 4) & 0x0F0F0F0Fu);
                    }
                }
                // generic-proxy writes -> visible to the tensor core (async proxy); this warp's share is done
                if (KIND == PF_Q2K) fence_async_smem();
                __syncwarp();
                if (lane == 0) mbar_arrive(&bar_a_full[b]);
                if (half == 1) ++gsb;
                ++gs;
                return true;
            };
            // superblock j from the register set (c0, c1, sc_cur); the other set is filled for superblock j + 1 of this
            // item or superblock 0 of the next
            auto superblock = [&](uint32_t j, const uint2 &c0, const uint2 &c1, const uint4 &sc_cur, uint2 &n0, uint2 &n1,
                                  uint4 &sc_nxt) -> bool {
                const uint8_t *nrow = j + 1 < a.kblocks ? drow : drow_next;
                if (nrow != nullptr) {
                    const uint32_t kbn = pf_visit_block<KIND>(a.kblocks, j + 1 < a.kblocks ? j + 1 : 0);
                    if (KIND == PF_IQ2 && a.layout == DSMOE_LAYOUT_ROWSOA) {  // both stages' groups in one 16-byte load
                        const uint4 t = *reinterpret_cast<const uint4 *>(nrow + 32 + 64 * kbn + 16 * dc);
                        n0 = make_uint2(t.x, t.y), n1 = make_uint2(t.z, t.w);
                    } else {
                        n0 = pf_load_packed<KIND>(nrow, a.layout, kbn, 0, dc);
                        n1 = pf_load_packed<KIND>(nrow, a.layout, kbn, 1, dc);
                    }
                    if (KIND == PF_Q2K) sc_nxt = pf_load_q2k_scales16(nrow, a.layout, kbn);
                }
                return stage(2 * j, c0, sc_cur) && stage(2 * j + 1, c1, sc_cur);
            };
            for (uint32_t j = 0; j < a.kblocks; j += 2) {
                if (!superblock(j, pA0, pA1, scA, pB0, pB1, scB)) break;
                if (!superblock(j + 1, pB0, pB1, scB, pA0, pA1, scA)) break;
            }
            drow = drow_next;
        }
    } else {
        // ------------------------------------------------------------------------------------ issuer and loader
        reg_dealloc<PF_REG_AUX>();
        const uint32_t awarp = warp - PF_DRAIN_WARPS - PF_DECODE_WARPS;
        if (awarp == 0) {
            // issuer: the whole warp walks the stages, one elected lane issues
            uint32_t gs = 0, gsb = 0, use0 = 0, use1 = 0, bslot = 0, bpar = 0;
            bool ok = true;
            for (uint32_t item = blockIdx.x; ok && item < n_items; item += gridDim.x) {
                const uint32_t tile = item / n_mtiles;
                const uint32_t rows16 = (a.tile_rows[tile] + 15u) & ~15u;
                const uint32_t idesc = tc05_idesc_f16(128, rows16);
                for (uint32_t s = 0; s < n_stages; ++s, ++gs) {
                    const uint32_t b = gs & 1u, half = s & 1u;
                    const uint32_t buf = pf_acc_buf<KIND>(a.kblocks, s >> 1, gsb), use = buf ? use1 : use0;
                    ok = mbar_wait_bounded(&bar_a_full[b], (gs >> 1) & 1u, a.status);
                    ok = ok && mbar_wait_bounded(&bar_b_full[bslot], bpar, a.status);
                    // at the start of a superblock the consumers must have handed the accumulator buffer back
                    if (half == 0 && use >= 1u) ok = ok && mbar_wait_bounded(&bar_acc_free[buf], (use - 1u) & 1u, a.status);
                    ok = __all_sync(FULL, ok);
                    tc05_fence_after_sync();
                    if (elect_one()) {
                        if (ok) {
                            const uint32_t d_tmem = tmem + buf * PF_TN;
                            const uint64_t da = tc05_smem_desc(smem_u32(smem + PF_SMEM_A + b * PF_STAGE_A), 128, PF_SBO);
                            const uint64_t db = tc05_smem_desc(smem_u32(smem + PF_SMEM_B + bslot * PF_STAGE_A), 128, PF_SBO);
#pragma unroll
                            for (int ks = 0; ks < PF_KS / 16; ++ks) {  // K advances 256 bytes = 16 descriptor units
                                if (KIND == PF_IQ2)  // A from tensor memory: 16 f16 = 8 columns per K step
                                    tc05_mma_f16_ts(d_tmem, tmem + PF_TMEM_A + b * PF_TMEM_A_STAGE + 8u * ks, db + 16u * ks, idesc,
                                                    (half | ks) != 0);
                                else
                                    tc05_mma_f16(d_tmem, da + 16u * ks, db + 16u * ks, idesc, (half | ks) != 0);
                            }
                            if (KIND == PF_Q2K && half == 1)
                                tc05_mma_f16(tmem + 256u + buf * PF_TN,
                                             tc05_smem_desc(smem_u32(smem + PF_SMEM_A2 + (gsb & 1u) * 4096), 128, 256),
                                             tc05_smem_desc(smem_u32(smem + PF_SMEM_B2 + (gsb & 1u) * 4096), 128, 256), idesc, 0);
                        }
                        // the commits also arrive when a wait above gave up, so nobody waits on them for ever
                        tc05_commit(&bar_a_free[b]);
                        tc05_commit(&bar_b_free[bslot]);
                        if (half == 1) tc05_commit(&bar_acc_full[buf]);
                    }
                    __syncwarp();
                    if (half == 1) {
                        ++gsb;
                        if (buf) ++use1;
                        else ++use0;
                    }
                    if (++bslot == PF_B_STAGES) bslot = 0, bpar ^= 1u;
                    if (!ok) break;
                }
            }
        } else if (awarp == 1) {
            // loader: activation blocks (and, for Q2_K, the superblock's bsums tile) into the three-stage ring
            uint32_t gs = 0, gsb = 0, bslot = 0, bpar = 0;
            bool ok = true;
            for (uint32_t item = blockIdx.x; ok && item < n_items; item += gridDim.x) {
                const uint32_t tile = item / n_mtiles;
                const uint32_t rows16 = (a.tile_rows[tile] + 15u) & ~15u, boff = a.tile_boff[tile];
                const uint8_t *btile = a.B + (size_t)boff * a.kblocks * 512;
                for (uint32_t s = 0; s < n_stages; ++s, ++gs) {
                    const uint32_t kb = pf_visit_block<KIND>(a.kblocks, s >> 1), half = s & 1u;
                    // the slot (and the bsums slot of two superblocks ago) is free once the stage that used it last
                    // has retired
                    if (gs >= PF_B_STAGES) ok = mbar_wait_bounded(&bar_b_free[bslot], bpar ^ 1u, a.status);
                    ok = __all_sync(FULL, ok);
                    if (!ok) break;
                    if (lane == 0) {
                        uint32_t bytes = rows16 * 256u;
                        if (KIND == PF_Q2K && half == 0) bytes += rows16 * 32u;
                        mbar_expect_tx(&bar_b_full[bslot], bytes);
                        bulk_g2s(smem + PF_SMEM_B + bslot * PF_STAGE_A, btile + (size_t)(2 * kb + half) * rows16 * 256,
                                 rows16 * 256u, &bar_b_full[bslot]);
                        if (KIND == PF_Q2K && half == 0)
                            bulk_g2s(smem + PF_SMEM_B2 + (gsb & 1u) * 4096, a.BS + ((size_t)kb * a.r_cap + boff) * 16,
                                     rows16 * 32u, &bar_b_full[bslot]);
                    }
                    __syncwarp();
                    if (half == 1) ++gsb;
                    if (++bslot == PF_B_STAGES) bslot = 0, bpar ^= 1u;
                }
            }
        }
    }

    // common exit: every MMA has retired (the consumers waited for the last accumulator) or an error is recorded
    tc05_fence_before_sync();
    __syncthreads();
    if (warp == 0) tc05_dealloc(tmem, TMEM_COLS);
}

// ---------------------------------------------------------------------------------------------------------------
// launchers
// ---------------------------------------------------------------------------------------------------------------
size_t prefill_scratch_bytes(uint32_t max_tokens, uint32_t k, uint32_t n_expert, uint32_t n_embd, uint32_t n_ff,
                             PrefillScratch *lay)
{
    const size_t P = (size_t)max_tokens * k;
    const size_t tl = P / PF_TN + n_expert + 1;          // tiles: full ones plus one partial per expert
    const size_t r_cap = ((P + 15 * (tl < P ? tl : P) + 15) & ~(size_t)15) + 16;  // padded rows over all tiles
    size_t off = 0;
    auto take = [&](size_t bytes) {
        const size_t o = off;
        off += (bytes + 255) & ~(size_t)255;
        return o;
    };
    PrefillScratch L;
    L.r_cap = (uint32_t)r_cap;
    L.tile_cap = (uint32_t)tl;
    L.counts = take(4 * (size_t)n_expert);
    L.offsets = take(4 * ((size_t)n_expert + 1));
    L.sorted = take(4 * P);
    L.tile_expert = take(4 * tl);
    L.tile_start = take(4 * tl);
    L.tile_rows = take(4 * tl);
    L.tile_boff = take(4 * (tl + 1));
    L.plan = take(16);
    L.bx = take(r_cap * (size_t)n_embd * 2);
    L.sx = take(r_cap * (size_t)(n_embd / QK_K) * 4);
    L.bm = take(r_cap * (size_t)n_ff * 2);
    L.sm = take(r_cap * (size_t)(n_ff / QK_K) * 4);
    L.bs = take(r_cap * (size_t)(n_ff / QK_K) * 16 * 2);
    L.down_pair = take(P * (size_t)n_embd * 4);
    L.up_rows = take(P * (size_t)n_ff * 4);
    if (lay) *lay = L;
    return off;
}

// The register reallocation inside the grouped GEMM is only safe if the kernels were compiled with exactly the
// register count the split was computed for.
static bool pf_kernels_as_planned()
{
    static int state = -1;
    if (state < 0) {
        cudaFuncAttributes f0, f1;
        const bool got = cudaFuncGetAttributes(&f0, pf_grouped_gemm_kernel<PF_IQ2>) == cudaSuccess &&
                         cudaFuncGetAttributes(&f1, pf_grouped_gemm_kernel<PF_Q2K>) == cudaSuccess;
        state = got && f0.numRegs == PF_REG_LAUNCH && f1.numRegs == PF_REG_LAUNCH ? 1 : 0;
    }
    return state == 1;
}

bool prefill_eligible(uint32_t n_embd, uint32_t n_ff, const uint8_t *gate, const uint8_t *up, const uint8_t *down,
                      int layout)
{
    if (!pf_kernels_as_planned()) return false;
    const uintptr_t al = layout == DSMOE_LAYOUT_ROWSOA ? 15 : 3;
    return n_embd % QK_K == 0 && n_ff % QK_K == 0 && n_ff % 64 == 0 && n_embd % 128 == 0 && (n_embd / QK_K == 16 || n_embd / QK_K == 8) &&
           n_ff / QK_K <= 16 && (((uintptr_t)gate | (uintptr_t)up | (uintptr_t)down) & al) == 0 &&
           (layout == DSMOE_LAYOUT_NATIVE || ((n_embd / QK_K * IQ2XXS_BYTES) % 16 == 0 && (n_ff / QK_K * Q2K_BYTES) % 16 == 0));
}

int launch_prefill_experts(cudaStream_t st, const PrefillArgs &p)
{
    uint8_t *w = p.scratch;
    const PrefillScratch &L = p.lay;
    auto u32p = [&](size_t o) { return reinterpret_cast<uint32_t *>(w + o); };
    const uint32_t P = p.n_tokens * p.k, xb = p.n_embd / QK_K, mb = p.n_ff / QK_K;
    static OncePerDevice attr;
    if (attr.first()) {
        cudaFuncSetAttribute(pf_grouped_gemm_kernel<PF_IQ2>, cudaFuncAttributeMaxDynamicSharedMemorySize, PF_SMEM_TOTAL);
        cudaFuncSetAttribute(pf_grouped_gemm_kernel<PF_Q2K>, cudaFuncAttributeMaxDynamicSharedMemorySize, PF_SMEM_TOTAL);
    }
    const int sms = sm_count_current();
    int n = 0;
    auto mark = [&](int i) {
        if (p.phase_events) cudaEventRecord(p.phase_events[i], st);
    };
    mark(0);
    // 1. group pairs by expert
    pf_count_kernel<<<p.n_expert, 256, 0, st>>>(p.selected, P, u32p(L.counts));
    pf_plan_kernel<<<1, 32, 0, st>>>(u32p(L.counts), (int)p.n_expert, u32p(L.offsets), u32p(L.tile_expert),
                                     u32p(L.tile_start), u32p(L.tile_rows), u32p(L.tile_boff), u32p(L.plan));
    pf_place_kernel<<<p.n_expert, 256, 0, st>>>(p.selected, P, u32p(L.offsets), u32p(L.sorted));
    n += 3;
    // 2. activation tiles of x
    const dim3 ggrid(32, (unsigned)(L.tile_cap < 1024u ? L.tile_cap : 1024u));
    pf_gather_kernel<<<ggrid, 256, 0, st>>>(p.xq, xb, p.k, u32p(L.sorted), u32p(L.tile_start), u32p(L.tile_rows),
                                            u32p(L.tile_boff), u32p(L.plan), w + L.bx,
                                            reinterpret_cast<float *>(w + L.sx), nullptr, L.r_cap, 1u);
    mark(1);
    // 3. gate / up / SwiGLU
    PfGemmArgs g = {};
    g.w0 = p.gate, g.w1 = p.up, g.expert_bytes = (uint64_t)p.n_ff * xb * IQ2XXS_BYTES;
    g.B = w + L.bx, g.S = reinterpret_cast<const float *>(w + L.sx), g.BS = nullptr, g.r_cap = L.r_cap;
    g.sorted = u32p(L.sorted), g.tile_expert = u32p(L.tile_expert), g.tile_start = u32p(L.tile_start);
    g.tile_rows = u32p(L.tile_rows), g.tile_boff = u32p(L.tile_boff), g.plan = u32p(L.plan);
    g.weights = p.weights, g.out = p.mid, g.out_u = reinterpret_cast<float *>(w + L.up_rows), g.out_dim = p.n_ff, g.kblocks = xb;
    g.clamp = p.clamp, g.ieee = p.ieee;
    g.layout = p.layout, g.status = p.status;
    pf_grouped_gemm_kernel<PF_IQ2><<<sms, PF_THREADS, PF_SMEM_TOTAL, st>>>(g);
    mark(2);
    // 4. clamp, SwiGLU, router weight and Q8_K of the result in one pass over the gate / up rows; tiles of it (with bsums)
    launch_swiglu_q8k(st, p.mid, reinterpret_cast<const float *>(w + L.up_rows), p.weights, p.midq, p.n_ff, P, p.clamp);
    pf_gather_kernel<<<ggrid, 256, 0, st>>>(p.midq, mb, 1, u32p(L.sorted), u32p(L.tile_start), u32p(L.tile_rows),
                                            u32p(L.tile_boff), u32p(L.plan), w + L.bm,
                                            reinterpret_cast<float *>(w + L.sm), reinterpret_cast<__half *>(w + L.bs),
                                            L.r_cap, 0u);
    mark(3);
    // 5. down
    PfGemmArgs d = g;
    d.w0 = p.down, d.w1 = nullptr, d.expert_bytes = (uint64_t)p.n_embd * mb * Q2K_BYTES;
    d.B = w + L.bm, d.S = reinterpret_cast<const float *>(w + L.sm), d.BS = reinterpret_cast<const __half *>(w + L.bs);
    d.weights = nullptr, d.out = reinterpret_cast<float *>(w + L.down_pair), d.out_dim = p.n_embd, d.kblocks = mb;
    d.row_ptr = p.row_ptr;
    pf_grouped_gemm_kernel<PF_Q2K><<<sms, PF_THREADS, PF_SMEM_TOTAL, st>>>(d);
    mark(4);
    // 6. slots summed in slot order (not when the rows went to their own destinations: the receiver sums them)
    if (p.before_sum) cudaStreamWaitEvent(st, p.before_sum, 0);
    if (!p.row_ptr)
        launch_moe_sum(st, reinterpret_cast<const float *>(w + L.down_pair), nullptr, p.out, p.n_embd, p.k, p.n_tokens, p.hc);
    mark(5);
    return n + (p.row_ptr ? 5 : 6);
}

}  // namespace dsmoe
