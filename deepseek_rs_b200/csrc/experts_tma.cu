// Decode kernels for the reference shapes (n_embd 4096, n_ff 2048) with the packed rows staged through shared memory
// by bulk asynchronous copies (TMA, untiled), so that every SM keeps tens of kilobytes of HBM reads in flight
// without holding them in registers.
//
// Both kernels are limited by instruction issue, not by HBM, at small batch: B200 delivers about 5.8 packed bytes per
// issued warp instruction at full bandwidth, i.e. about 22 IQ2_XXS or 18 Q2_K weights. The mapping therefore gives
// each lane a whole 256-weight block (as the reference's quarter-warp kernels do), which removes every integer
// cross-lane reduction; only the reference's own f32 butterfly remains. The int8 activations of the lane's block
// live in registers for the lifetime of the (token, slot) pair.
//
//   gate/up: persistent CTAs, one per SM. A warp item is two consecutive rows (half-warp per row, lane = block).
//            Lane 0 issues the four 1056-byte bulk copies of an item onto the stage's mbarrier; the warp consumes the
//            stage one item later (the kernel is issue-bound, a depth of one item per warp keeps ~60 KB in flight). Codebook and sign masks are replicated in shared memory so that every 64-bit
//            lookup is conflict-free. Clamp, SwiGLU and the stores run once per 32 finished rows, one row per lane.
//   down:    one CTA per (token, chunk of output rows), one warp per routed slot, four rows per warp step (quarter-warp
//            per row, lane = block); lane 0 fetches the warp's whole chunk of that expert's rows (contiguous) with
//            one bulk copy and the pair's Q8_K activations with another. Slot results meet in shared memory and
//            are summed in slot order.
//
// Lanes read their 64-byte block from the staged row in a rotated 16-byte order ((j + block/2) mod 4) so that the
// eight lanes of a shared-memory wavefront hit eight different bank groups; the activation registers are loaded in
// the same rotated order, which keeps all register indexing static.
//
// Arithmetic and summation order are those of the reference kernels (engine/src/kernels/moe.rs:622-715, 922-970), so
// results stay bit-identical to the CPU oracle.
#include "async.cuh"
#include "common.cuh"
#include "launch.h"
#include "q8k.cuh"

namespace dsmoe {

// The codebook in global memory (read coalesced when filling shared memory; constant memory would serialise the
// per-thread indices).
__device__ const uint64_t g_iq2xxs_grid[DSMOE_IQ2XXS_GRID_ENTRIES] = {DSMOE_IQ2XXS_GRID_VALUES};

constexpr int GU_STAGES = 2;
constexpr int GU_ROW_BYTES = 16 * IQ2XXS_BYTES;  // 1056
constexpr int GU_STAGE_BYTES = 2 * GU_ROW_BYTES; // gate row + up row of one output row
// Lookup tables, replicated so that every lane of a warp (codebook, 32 copies, 256-byte entry stride) or of a
// half-warp (sign masks, 16 copies, 128-byte stride) reads its own bank pair: each 64-bit lookup costs the minimum of
// two shared-memory wavefronts, and the codebook address is assembled from the packed index byte by one PRMT.
constexpr int GU_GRID_TABLE_BYTES = DSMOE_IQ2XXS_GRID_ENTRIES * 256;  // 65536
constexpr int GU_SIGN_TABLE_BYTES = DSMOE_IQ2_SIGN_ENTRIES * 128;     // 16384
constexpr int GU_TABLE_BYTES = GU_GRID_TABLE_BYTES + GU_SIGN_TABLE_BYTES;
constexpr int GU_MAX_WARPS = 16;  // register file: 16 warps x 128 registers; 80 KB tables + 16 rings of 2 x 4224 B

// Integer dot of one 32-weight group; tables addressed as described above. lane8 = 8 * lane,
// sbase = GU_GRID_TABLE_BYTES + 8 * (lane & 15). Signs by the identity sum(+/-g*q) = dp4a(g^m, q) - dp4a(m, q).
__device__ __forceinline__ int iq2_group_dot_rep(uint32_t aux0, uint32_t aux1, const int *q, const uint8_t *tbl,
                                                 uint32_t lane8, uint32_t sbase)
{
    int pos = 0, neg = 0;
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        // (index byte k) << 8 | 8*lane: byte 0 from lane8, byte 1 from aux0, bytes 2-3 zero (lane8 bytes 1, 2)
        const uint32_t goff = __byte_perm(aux0, lane8, 0x6504u | ((uint32_t)k << 4));
        const int sh = 7 - 7 * k;  // bring the 7-bit sign index to bits 7..13
        const uint32_t sraw = sh >= 0 ? (aux1 << sh) : (aux1 >> (-sh));
        const uint32_t soff = (sraw & 0x3F80u) + sbase;
        const uint2 g = *reinterpret_cast<const uint2 *>(tbl + goff);
        const uint2 m = *reinterpret_cast<const uint2 *>(tbl + soff);
        pos = __dp4a((int)(g.x ^ m.x), q[2 * k], pos);
        pos = __dp4a((int)(g.y ^ m.y), q[2 * k + 1], pos);
        neg = __dp4a((int)m.x, q[2 * k], neg);
        neg = __dp4a((int)m.y, q[2 * k + 1], neg);
    }
    return (pos - neg) * (int)(2u * (aux1 >> 28) + 1u);
}

constexpr int GU_ITEM_ROWS = 2;
constexpr int GU_ITEM_BYTES = GU_ITEM_ROWS * GU_STAGE_BYTES;  // gate,up of row r then gate,up of row r+1

// 16-byte piece c (groups 2c, 2c+1) of block blk of a staged row
template <int LAYOUT>
__device__ __forceinline__ uint4 gu_smem_piece(const uint8_t *row, int blk, int c)
{
    if (LAYOUT == DSMOE_LAYOUT_ROWSOA) return *reinterpret_cast<const uint4 *>(row + 32 + 64 * blk + 16 * c);
    return ld_16B_align2(row + IQ2XXS_BYTES * blk + 2 + 16 * c);
}

// ((0.125 * d_w) * d_x) * (float)bsum, engine/src/kernels/quantize.rs:811
__device__ __forceinline__ float iq2_block_scale(uint32_t dbits, float yd, int bsum, bool ieee)
{
    return __fmul_rn(__fmul_rn(__fmul_rn(0.125f, f16_bits_to_f32(dbits, ieee)), yd), (float)bsum);
}

// lane partial a_l = (0 + dot_l) + dot_(l+8), then the butterfly xor 4, 2, 1 (engine/src/kernels/moe.rs:37-42,
// 661-690), over the 16 lanes of a half-warp (lane = block)
__device__ __forceinline__ float gu_row_total(float dot)
{
    const float other = __shfl_xor_sync(FULL, dot, 8);
    const bool low = (threadIdx.x & 8) == 0;
    float a = __fadd_rn(__fadd_rn(0.0f, low ? dot : other), low ? other : dot);
    a = __fadd_rn(a, __shfl_xor_sync(FULL, a, 4));
    a = __fadd_rn(a, __shfl_xor_sync(FULL, a, 2));
    a = __fadd_rn(a, __shfl_xor_sync(FULL, a, 1));
    return a;
}

template <int LAYOUT>
__global__ void __launch_bounds__(32 * GU_MAX_WARPS, 1)
    gate_up_x16_tma_kernel(const uint8_t *__restrict__ gate_base, const uint8_t *__restrict__ up_base,
                           const uint8_t *__restrict__ xq, const int32_t *__restrict__ selected,
                           const float *__restrict__ weights, float *__restrict__ gate_out, float *__restrict__ up_out,
                           float *__restrict__ mid_out, uint64_t expert_bytes, uint32_t mid_dim, uint32_t k,
                           uint32_t n_items, float clamp, int ieee_i, int *status, const int32_t *__restrict__ order,
                           uint32_t parts, uint8_t *__restrict__ midq_out, uint32_t *__restrict__ blk_rows)
{
    extern __shared__ __align__(128) uint8_t smem[];
    const int wpc = blockDim.x >> 5, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    uint8_t *ring = smem + GU_TABLE_BYTES + (size_t)warp * GU_STAGES * GU_ITEM_BYTES;
    uint64_t *bars = reinterpret_cast<uint64_t *>(smem + GU_TABLE_BYTES + (size_t)wpc * GU_STAGES * GU_ITEM_BYTES) +
                     warp * GU_STAGES;

    // fill the replicated tables, 16 bytes (two copies of one entry) per store
    for (int i = threadIdx.x; i < GU_GRID_TABLE_BYTES / 16; i += blockDim.x) {
        const uint64_t g = g_iq2xxs_grid[i >> 4];
        reinterpret_cast<uint4 *>(smem)[i] = make_uint4((uint32_t)g, (uint32_t)(g >> 32), (uint32_t)g, (uint32_t)(g >> 32));
    }
    for (int i = threadIdx.x; i < GU_SIGN_TABLE_BYTES / 16; i += blockDim.x) {
        const uint32_t sb = dsmoe_iq2_sign_byte((uint32_t)(i >> 3));
        const uint32_t lo = nibble_to_bytemask(sb), hi = nibble_to_bytemask(sb >> 4);
        reinterpret_cast<uint4 *>(smem + GU_GRID_TABLE_BYTES)[i] = make_uint4(lo, hi, lo, hi);
    }
    if (lane == 0) {
#pragma unroll
        for (int s = 0; s < GU_STAGES; ++s) mbar_init(&bars[s], 1);
        fence_async_smem();
    }
    // the tables above depend on nothing; activations, routing and the output buffers do
    pdl_launch_dependents();
    pdl_wait();
    __syncthreads();

    // Items: item i covers rows 2i, 2i+1 of the flattened [pair position][row] space (mid_dim is even). Without `order`
    // a warp takes one contiguous run of items and pair position = pair. With `order` (pair positions sorted by expert,
    // order[position] = pair) every pair's items are cut into `parts` runs at the same rows, run = task, and warps take
    // tasks position-major: pairs of one expert stream the same rows at the same time, so the second one finds them
    // in L2 instead of reading DRAM again.
    const uint32_t n_warps = gridDim.x * wpc, gw = blockIdx.x * wpc + warp;
    const bool ieee = ieee_i != 0;
    const uint32_t lane8 = 8u * lane, sbase = GU_GRID_TABLE_BYTES + 8u * (lane & 15);
    const int sub = lane >> 4, blk = lane & 15, rot = blk >> 1;
    const uint32_t items_per_pair = mid_dim / GU_ITEM_ROWS;
    const uint32_t n_tasks = order ? (n_items / items_per_pair) * parts : 1u;
    int q[64];  // activations of block blk, 16-byte pieces in rotated order: q[16j ..] belongs to piece (j + rot) & 3
    float yd = 0.0f;
    uint32_t cur_tok = 0xFFFFFFFFu;
    uint32_t it = 0;  // items consumed so far: ring stage and mbarrier phase follow it across tasks

    // tasks go to the CTAs round-robin, so that when there are fewer tasks than warps every SM keeps about as many
    for (uint32_t task = order ? warp * gridDim.x + blockIdx.x : 0u; task < n_tasks; task += n_warps) {
        uint32_t begin, end;
        if (order) {
            const uint32_t pos = task / parts, part = task - pos * parts;
            begin = pos * items_per_pair + (uint32_t)(((uint64_t)part * items_per_pair) / parts);
            end = pos * items_per_pair + (uint32_t)(((uint64_t)(part + 1) * items_per_pair) / parts);
        } else {
            const uint32_t chunk = (n_items + n_warps - 1) / n_warps;
            begin = min(n_items, gw * chunk), end = min(n_items, begin + chunk);
        }
        if (begin >= end) continue;

        uint32_t f_item = begin, f_pair = begin / items_per_pair, f_row = (begin - f_pair * items_per_pair) * GU_ITEM_ROWS;
        auto issue_next = [&](int stage) {
            if (lane == 0) {
                const int32_t e = selected[order ? (uint32_t)order[f_pair] : f_pair];
                const uint64_t off = (e < 0 ? 0u : (uint64_t)e) * expert_bytes + (uint64_t)f_row * GU_ROW_BYTES;
                uint8_t *dst = ring + stage * GU_ITEM_BYTES;
                mbar_expect_tx(&bars[stage], GU_ITEM_BYTES);
                // rows f_row and f_row+1 are adjacent in each tensor: one copy per tensor; gate rows first, then up rows
                bulk_g2s(dst, gate_base + off, GU_ITEM_ROWS * GU_ROW_BYTES, &bars[stage]);
                bulk_g2s(dst + GU_ITEM_ROWS * GU_ROW_BYTES, up_base + off, GU_ITEM_ROWS * GU_ROW_BYTES, &bars[stage]);
            }
            ++f_item;
            f_row += GU_ITEM_ROWS;
            if (f_row == mid_dim) {
                f_row = 0;
                ++f_pair;
            }
        };
        if (it > 0) fence_async_smem();  // the stages were read by the task before
#pragma unroll
        for (int j = 0; j < GU_STAGES - 1; ++j)
            if (f_item < end) issue_next((it + j) % GU_STAGES);

        uint32_t pos = begin / items_per_pair, row = (begin - pos * items_per_pair) * GU_ITEM_ROWS;
        uint32_t pair = order ? (uint32_t)order[pos] : pos;
        float keep_g = 0.0f, keep_u = 0.0f;  // lane L keeps row (2 * flush_base + L) of the flattened [position][row] space
        uint32_t flush_base = begin;
        for (uint32_t item = begin; item < end; ++item, ++it) {
            const int stage = it % GU_STAGES;
            const uint32_t tok = pair / k;
            if (tok != cur_tok) {  // new token: reload this lane's block of its Q8_K row
                cur_tok = tok;
                const uint8_t *xb = xq + ((size_t)tok * 16 + blk) * Q8K_BYTES;
                yd = *reinterpret_cast<const float *>(xb);
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const int *pq = reinterpret_cast<const int *>(xb + 4 + 64 * ((j + rot) & 3));
#pragma unroll
                    for (int i = 0; i < 16; ++i) q[16 * j + i] = pq[i];
                }
            }
            if (f_item < end) {  // refill the stage consumed one iteration ago
                fence_async_smem();
                issue_next((it + GU_STAGES - 1) % GU_STAGES);
            }
            if (!mbar_wait_bounded(&bars[stage], (it / GU_STAGES) & 1, status)) return;
            const uint8_t *grow = ring + stage * GU_ITEM_BYTES + sub * GU_ROW_BYTES;
            const uint8_t *urow = grow + GU_ITEM_ROWS * GU_ROW_BYTES;
            int sg = 0, su = 0;
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const int c = (j + rot) & 3;
                const uint4 gp = gu_smem_piece<LAYOUT>(grow, blk, c), up = gu_smem_piece<LAYOUT>(urow, blk, c);
                sg += iq2_group_dot_rep(gp.x, gp.y, q + 16 * j, smem, lane8, sbase);
                sg += iq2_group_dot_rep(gp.z, gp.w, q + 16 * j + 8, smem, lane8, sbase);
                su += iq2_group_dot_rep(up.x, up.y, q + 16 * j, smem, lane8, sbase);
                su += iq2_group_dot_rep(up.z, up.w, q + 16 * j + 8, smem, lane8, sbase);
            }
            const uint32_t dstep = LAYOUT == DSMOE_LAYOUT_ROWSOA ? 2 : IQ2XXS_BYTES;
            const uint32_t dg = ld_u16(grow + dstep * blk), du = ld_u16(urow + dstep * blk);
            __syncwarp();  // every lane has finished reading the stage
            const float g = gu_row_total(iq2_block_scale(dg, yd, sg, ieee));  // all 16 lanes of the half hold the row total
            const float u = gu_row_total(iq2_block_scale(du, yd, su, ieee));
            const float g_o = __shfl_xor_sync(FULL, g, 16), u_o = __shfl_xor_sync(FULL, u, 16);
            if ((uint32_t)(lane >> 1) == item - flush_base) {  // lane L keeps sub-row L & 1 of this item
                keep_g = (lane & 1) == sub ? g : g_o;
                keep_u = (lane & 1) == sub ? u : u_o;
            }
            if (item - flush_base == 15 || item + 1 == end) {
                // clamp + SwiGLU + stores for up to 32 finished rows at once, one per lane
                const uint32_t mine = GU_ITEM_ROWS * flush_base + lane;  // flattened [position][row] index
                const bool wrote = mine < GU_ITEM_ROWS * (item + 1);
                size_t dst = 0;
                if (wrote) {
                    float gg = keep_g, uu = keep_u;
                    if (clamp > 1.0e-6f) {
                        if (gg > clamp) gg = clamp;
                        if (uu > clamp) uu = clamp;
                        if (uu < -clamp) uu = -clamp;
                    }
                    const uint32_t mpos = mine / mid_dim, mpair = order ? (uint32_t)order[mpos] : mpos;
                    dst = (size_t)mpair * mid_dim + (mine - mpos * mid_dim);
                    if (gate_out) gate_out[dst] = gg;
                    if (up_out) up_out[dst] = uu;
                    mid_out[dst] = swiglu_weighted(gg, uu, weights[mpair]);
                }
                if (midq_out) {
                    // Q8_K of mid, block by block as the blocks fill up: the rows just stored are counted into their
                    // 256-row blocks (32 adjacent rows touch at most two), and the warp whose rows complete a block
                    // quantises it (mid_dim is a multiple of 256, so a block never spans two pairs). The counter goes
                    // back to 0 for the next call. Nobody waits: whoever arrives last does the work.
                    __threadfence();
                    const uint32_t gb = wrote ? (uint32_t)(dst >> 8) : 0xFFFFFFFFu;
                    const uint32_t any = __ballot_sync(FULL, wrote);
                    const uint32_t gb_a = __shfl_sync(FULL, gb, __ffs(any) - 1);
                    const uint32_t in_b = __ballot_sync(FULL, wrote && gb != gb_a);
                    const uint32_t gb_b = in_b ? __shfl_sync(FULL, gb, __ffs(in_b) - 1) : 0xFFFFFFFFu;
                    uint32_t done = 0;
                    if (lane == 0) {
                        const uint32_t n_a = __popc(any & ~in_b), n_b = __popc(in_b);
                        if (atomicAdd(&blk_rows[gb_a], n_a) + n_a == 256u) done |= 1u;
                        if (in_b && atomicAdd(&blk_rows[gb_b], n_b) + n_b == 256u) done |= 2u;
                    }
                    done = __shfl_sync(FULL, done, 0);
#pragma unroll
                    for (int which = 0; which < 2; ++which) {
                        if (!(done & (1u << which))) continue;
                        const uint32_t b = which ? gb_b : gb_a;
                        __threadfence();
                        const float4 *src = reinterpret_cast<const float4 *>(mid_out + (size_t)b * QK_K + 8 * lane);
                        const float4 v0 = __ldcg(src), v1 = __ldcg(src + 1);
                        const float v[8] = {v0.x, v0.y, v0.z, v0.w, v1.x, v1.y, v1.z, v1.w};
                        q8k_quantize_vals(v, midq_out + (size_t)b * Q8K_BYTES, lane);
                        if (lane == 0) blk_rows[b] = 0;
                    }
                }
                flush_base = item + 1;
            }
            row += GU_ITEM_ROWS;
            if (row == mid_dim) {
                row = 0;
                ++pos;
                if (item + 1 < end) pair = order ? (uint32_t)order[pos] : pos;
            }
        }
    }
}

// ---------------------------------------------------------------------------------------------------------------

constexpr int DN_ROW_BYTES = 8 * Q2K_BYTES;  // 672
constexpr int DN_ROWS_MAX = 16;
constexpr int DN_STAGES = DN_ROWS_MAX / 4;
constexpr int DN_ACT_BYTES = 8 * Q8K_BYTES;  // 2336: one (token, slot) mid row as Q8_K blocks

// 16 quant bytes (piece c = 2h + half: sub-blocks 8h + half + {0,2,4,6}) of block blk of a staged Q2_K row
template <int LAYOUT>
__device__ __forceinline__ uint4 dn_smem_piece(const uint8_t *row, int blk, int c)
{
    const uint8_t *p = q2k_qs_ptr<LAYOUT>(row, 8, blk) + 16 * c;
    if (LAYOUT == DSMOE_LAYOUT_ROWSOA) return *reinterpret_cast<const uint4 *>(p);
    return ld_16B_align4(p);
}

template <int LAYOUT, bool SUM>
__global__ void __launch_bounds__(256, 2) down_m8_tma_kernel(const uint8_t *__restrict__ down_base,
                                                           const uint8_t *__restrict__ midq,
                                                           const int32_t *__restrict__ selected, float *__restrict__ out,
                                                           uint64_t expert_bytes, uint32_t out_dim, uint32_t k, int ieee_i,
                                                           int rows_per_cta, int *status)
{
    extern __shared__ __align__(128) uint8_t smem[];
    const bool ieee = ieee_i != 0;
    const int lane = threadIdx.x & 31, slot = threadIdx.x >> 5;
    uint8_t *wbuf = smem + (size_t)slot * rows_per_cta * DN_ROW_BYTES;
    uint8_t *abuf = smem + (size_t)k * rows_per_cta * DN_ROW_BYTES + (size_t)slot * DN_ACT_BYTES;  // this pair's Q8_K row
    float *s_part = reinterpret_cast<float *>(smem + (size_t)k * (rows_per_cta * DN_ROW_BYTES + DN_ACT_BYTES));
    uint64_t *bars = reinterpret_cast<uint64_t *>(s_part + MAX_K * DN_ROWS_MAX) + slot * DN_STAGES;

    // tokens run fastest over the grid: the CTAs resident at one time cover every token at a few row groups, so tokens
    // that share an expert ask for the same rows at the same time and all but the first are served by L2
    const uint32_t tok = blockIdx.x, pair = tok * k + slot;
    const uint32_t row_begin = blockIdx.y * rows_per_cta;
    const uint32_t n_rows = min((uint32_t)rows_per_cta, out_dim - row_begin);
    pdl_launch_dependents();
    pdl_wait();
    if (lane == 0) {
        const int32_t e = selected[pair];
        const uint64_t ex = e < 0 ? 0u : (uint64_t)e;
        const uint8_t *src = down_base + ex * expert_bytes + (uint64_t)row_begin * DN_ROW_BYTES;
#pragma unroll
        for (int s = 0; s < DN_STAGES; ++s) mbar_init(&bars[s], 1);
        fence_async_smem();
        // everything is requested up front, four rows per mbarrier, so that the first rows can be consumed while
        // the later ones are still arriving
        // test hook (status[2], normally 0): the second group of rows is never requested, so the wait for it runs out
        const bool drop_one = status != nullptr && *reinterpret_cast<volatile int *>(status + 2) != 0;
        for (uint32_t s = 0; 4 * s < n_rows; ++s) {
            const uint32_t rows = min(4u, n_rows - 4 * s), bytes = rows * DN_ROW_BYTES + (s == 0 ? DN_ACT_BYTES : 0);
            if (drop_one && s == 1) continue;
            mbar_expect_tx(&bars[s], bytes);
            if (s == 0) bulk_g2s(abuf, midq + (size_t)pair * DN_ACT_BYTES, DN_ACT_BYTES, &bars[0]);
            bulk_g2s(wbuf + 4 * s * DN_ROW_BYTES, src + (uint64_t)4 * s * DN_ROW_BYTES, rows * DN_ROW_BYTES, &bars[s]);
        }
    }
    // lane = (row of the current group of four, block): the block's 256 activations stay in registers, 16-byte
    // pieces in rotated order (piece (j + rot) & 3 at step j), bsums likewise
    const int sub = lane >> 3, blk = lane & 7, rot = blk >> 1;
    __syncwarp();  // the barrier lane 0 initialised is now visible to the whole warp
    bool ok = mbar_wait_bounded(&bars[0], 0, status);
    const uint8_t *mq = abuf + blk * Q8K_BYTES;
    const float yd = *reinterpret_cast<const float *>(mq);
    int q[4][4][4];      // [step j][sub-block jj][word]
    uint32_t bs[4][2];   // [step j]: bsums of sub-blocks (jj = 0,1) and (2,3) as int16 pairs
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        const int c = (j + rot) & 3, h = c >> 1, half = c & 1;
#pragma unroll
        for (int jj = 0; jj < 4; ++jj) {
            const int *pq = reinterpret_cast<const int *>(mq + 4 + 128 * h + 32 * jj + 16 * half);
#pragma unroll
            for (int w = 0; w < 4; ++w) q[j][jj][w] = pq[w];
        }
        const uint16_t *pb = reinterpret_cast<const uint16_t *>(mq + 260) + 8 * h + half;
        bs[j][0] = (uint32_t)pb[0] | ((uint32_t)pb[2] << 16);
        bs[j][1] = (uint32_t)pb[4] | ((uint32_t)pb[6] << 16);
    }

    for (uint32_t r0 = 0; ok && r0 < n_rows; r0 += 4) {
        if (r0 > 0 && !(ok = mbar_wait_bounded(&bars[r0 >> 2], 0, status))) break;
        const uint32_t r = r0 + sub;
        const bool valid = r < n_rows;
        const uint8_t *rowp = wbuf + (valid ? r : r0) * DN_ROW_BYTES;
        // the 16 scale bytes of the block
        uint32_t sc[4];
        {
            const uint8_t *sp = q2k_scales_ptr<LAYOUT>(rowp, 8, blk);
            if (LAYOUT == DSMOE_LAYOUT_ROWSOA) {
                const uint4 v = *reinterpret_cast<const uint4 *>(sp);
                sc[0] = v.x, sc[1] = v.y, sc[2] = v.z, sc[3] = v.w;
            } else {
                sc[0] = ld_u32(sp), sc[1] = ld_u32(sp + 4), sc[2] = ld_u32(sp + 8), sc[3] = ld_u32(sp + 12);
            }
        }
        const uint32_t dd = ld_u32(q2k_dd_ptr<LAYOUT>(rowp, 8, blk));
        int isum = 0, summs = 0;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int c = (j + rot) & 3;
            const uint4 qs = dn_smem_piece<LAYOUT>(rowp, blk, c);
            const uint32_t lo_w = (c & 2) ? sc[2] : sc[0], hi_w = (c & 2) ? sc[3] : sc[1];
            const uint32_t sc4 = __byte_perm(lo_w, hi_w, (c & 1) ? 0x7531u : 0x6420u);
            int is, sm;
            q2k_quarter_dot(qs, q[j], sc4, bs[j][0], bs[j][1], is, sm);
            isum += is;
            summs += sm;
        }
        // dall * isum - dmin * summs (engine/src/kernels/quantize.rs:856-900); one block per lane = the reference's
        // lane partial, then its butterfly xor 4, 2, 1 over the quarter-warp
        const float dall = __fmul_rn(yd, f16_bits_to_f32(dd & 0xFFFFu, ieee));
        const float dmin = __fmul_rn(yd, f16_bits_to_f32(dd >> 16, ieee));
        float a = __fadd_rn(0.0f, __fsub_rn(__fmul_rn(dall, (float)isum), __fmul_rn(dmin, (float)summs)));
        a = __fadd_rn(a, __shfl_xor_sync(FULL, a, 4));
        a = __fadd_rn(a, __shfl_xor_sync(FULL, a, 2));
        a = __fadd_rn(a, __shfl_xor_sync(FULL, a, 1));
        if (blk == 0 && valid) {
            if (SUM) s_part[slot * DN_ROWS_MAX + r] = a;
            else out[(size_t)pair * out_dim + row_begin + r] = a;
        }
    }
    if (SUM) {
        __syncthreads();
        if (threadIdx.x < n_rows) {
            float total = 0.0f;
            for (uint32_t s = 0; s < k; ++s) total = __fadd_rn(total, s_part[s * DN_ROWS_MAX + threadIdx.x]);
            out[(size_t)tok * out_dim + row_begin + threadIdx.x] = total;
        }
    }
}

// ---------------------------------------------------------------------------------------------------------------
// launchers
// ---------------------------------------------------------------------------------------------------------------

bool gate_up_tma_eligible(const GateUpArgs &a)
{
    return a.xq_blocks == 16 && a.row_bytes == (uint64_t)GU_ROW_BYTES && a.mid_dim % GU_ITEM_ROWS == 0 &&
           (((uintptr_t)a.gate_base | (uintptr_t)a.up_base | a.expert_bytes) & 15) == 0;
}

// Pair positions sorted by expert for the gate/up kernel: order[position] = pair. One CTA: counts in shared memory,
// an exclusive scan, placement (the order inside an expert's run does not matter: every pair is computed on its own).
constexpr int PO_MAX_EXPERTS = 4096;

__global__ void __launch_bounds__(1024) pair_order_kernel(const int32_t *__restrict__ selected, uint32_t n_pairs,
                                                           uint32_t n_expert, int32_t *__restrict__ order)
{
    extern __shared__ uint32_t po_count[];  // n_expert counts, then n_expert cursors
    uint32_t *cursor = po_count + n_expert;
    pdl_launch_dependents();
    for (uint32_t e = threadIdx.x; e < n_expert; e += blockDim.x) po_count[e] = 0;
    pdl_wait();
    __syncthreads();
    auto bin = [&](uint32_t p) {
        const int32_t e = selected[p];
        return e < 0 ? 0u : ((uint32_t)e < n_expert ? (uint32_t)e : n_expert - 1);
    };
    for (uint32_t p = threadIdx.x; p < n_pairs; p += blockDim.x) atomicAdd(&po_count[bin(p)], 1u);
    __syncthreads();
    if (threadIdx.x < 32) {  // exclusive scan by one warp, 32 experts per round
        uint32_t run = 0;
        for (uint32_t e0 = 0; e0 < n_expert; e0 += 32) {
            const uint32_t e = e0 + threadIdx.x, c = e < n_expert ? po_count[e] : 0u;
            uint32_t inc = c;
#pragma unroll
            for (int m = 1; m < 32; m <<= 1) {
                const uint32_t o = __shfl_up_sync(FULL, inc, m);
                if ((int)threadIdx.x >= m) inc += o;
            }
            if (e < n_expert) cursor[e] = run + inc - c;
            run += __shfl_sync(FULL, inc, 31);
        }
    }
    __syncthreads();
    for (uint32_t p = threadIdx.x; p < n_pairs; p += blockDim.x) order[atomicAdd(&cursor[bin(p)], 1u)] = (int32_t)p;
}

int launch_pair_order(cudaStream_t st, const int32_t *selected, uint32_t n_pairs, uint32_t n_expert, int32_t *order)
{
    if (n_pairs == 0 || n_expert == 0 || n_expert > (uint32_t)PO_MAX_EXPERTS) return 0;
    launch_pdl(pair_order_kernel, dim3(1), dim3(1024), (size_t)2 * n_expert * sizeof(uint32_t), st, selected, n_pairs, n_expert,
               order);
    return 1;
}

template <int LAYOUT>
static void launch_gu_tma(cudaStream_t st, const GateUpArgs &a, int *status)
{
    const uint32_t items_per_pair = a.mid_dim / GU_ITEM_ROWS, n_pairs = a.n_tokens * a.k;
    const uint32_t n_items = n_pairs * items_per_pair;
    const int sms = sm_count_current();
    int best_w = GU_MAX_WARPS;
    uint32_t parts = 1;
    if (a.order) {
        // warps per CTA and runs per pair: the fewest items for the busiest warp, a run's start (an empty ring to
        // fill) counted as eight items; ties go to more warps, fewer runs
        uint64_t best_cost = ~0ull;
        for (int w = GU_MAX_WARPS; w >= 8; --w) {
            const uint32_t nw = (uint32_t)sms * w;
            for (uint32_t pr = 1; pr <= items_per_pair && pr <= 256; ++pr) {
                const uint64_t tasks = (uint64_t)n_pairs * pr, rounds = (tasks + nw - 1) / nw;
                const uint64_t cost = rounds * ((items_per_pair + pr - 1) / pr + 8);
                if (cost < best_cost) best_cost = cost, best_w = w, parts = pr;
            }
        }
    } else {
        // warps per CTA: as many as fit, unless a smaller count wastes clearly fewer warp-slots in the last round of items
        auto eff_of = [&](int w) {
            const uint32_t nw = (uint32_t)sms * w, chunk = (n_items + nw - 1) / nw;
            return (double)n_items / ((double)chunk * nw);
        };
        for (int w = GU_MAX_WARPS - 1; w >= 8; --w)
            if (eff_of(w) > eff_of(best_w) + 0.08) best_w = w;
    }
    const size_t smem = GU_TABLE_BYTES + (size_t)best_w * GU_STAGES * GU_ITEM_BYTES + (size_t)best_w * GU_STAGES * 8;
    static OncePerDevice attr;  // one per template instance
    if (attr.first())
        cudaFuncSetAttribute(gate_up_x16_tma_kernel<LAYOUT>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             GU_TABLE_BYTES + GU_MAX_WARPS * GU_STAGES * (GU_ITEM_BYTES + 8));
    const uint32_t want = (n_items + best_w - 1) / best_w;
    const uint32_t grid = want < (uint32_t)sms ? want : (uint32_t)sms;
    launch_pdl(gate_up_x16_tma_kernel<LAYOUT>, dim3(grid), dim3(32 * best_w), smem, st, a.gate_base, a.up_base, a.xq,
               a.selected, a.weights, a.gate_out, a.up_out, a.mid_out, a.expert_bytes, a.mid_dim, a.k, n_items, a.clamp,
               a.ieee, status, a.order, parts, a.midq_out, a.blk_rows);
}

int launch_gate_up_mid_tma(cudaStream_t st, const GateUpArgs &a, int *status)
{
    if (a.n_tokens == 0 || a.mid_dim == 0) return 0;
    if (a.layout == DSMOE_LAYOUT_ROWSOA) launch_gu_tma<DSMOE_LAYOUT_ROWSOA>(st, a, status);
    else launch_gu_tma<DSMOE_LAYOUT_NATIVE>(st, a, status);
    return 1;
}

bool down_tma_eligible(const DownArgs &a)
{
    return a.midq_blocks == 8 && a.row_bytes == (uint64_t)DN_ROW_BYTES &&
           (((uintptr_t)a.down_base | (uintptr_t)a.midq | a.expert_bytes) & 15) == 0;
}

template <int LAYOUT, bool SUM>
static void launch_dn_tma(cudaStream_t st, const DownArgs &a, int *status)
{
    // small batches: short chunks so that one wave of CTAs covers all rows; large batches: longer chunks
    const int rows_per_cta = 16;  // 256 CTAs per token at out_dim 4096: one wave at two CTAs per SM
    const size_t smem = (size_t)a.k * (rows_per_cta * DN_ROW_BYTES + DN_ACT_BYTES) + MAX_K * DN_ROWS_MAX * 4 + MAX_K * DN_STAGES * 8;
    static OncePerDevice attr;  // one per template instance
    if (attr.first())
        cudaFuncSetAttribute(down_m8_tma_kernel<LAYOUT, SUM>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             MAX_K * (DN_ROWS_MAX * DN_ROW_BYTES + DN_ACT_BYTES) + MAX_K * DN_ROWS_MAX * 4 + MAX_K * DN_STAGES * 8);
    dim3 grid(a.n_tokens, (a.out_dim + rows_per_cta - 1) / rows_per_cta);
    launch_pdl(down_m8_tma_kernel<LAYOUT, SUM>, grid, dim3(32 * a.k), smem, st, a.down_base, a.midq, a.selected, a.out,
               a.expert_bytes, a.out_dim, a.k, a.ieee, rows_per_cta, status);
}

int launch_down_tma(cudaStream_t st, const DownArgs &a, int *status)
{
    if (a.n_tokens == 0 || a.out_dim == 0) return 0;
    if (a.layout == DSMOE_LAYOUT_ROWSOA) {
        if (a.sum_slots) launch_dn_tma<DSMOE_LAYOUT_ROWSOA, true>(st, a, status);
        else launch_dn_tma<DSMOE_LAYOUT_ROWSOA, false>(st, a, status);
    } else {
        if (a.sum_slots) launch_dn_tma<DSMOE_LAYOUT_NATIVE, true>(st, a, status);
        else launch_dn_tma<DSMOE_LAYOUT_NATIVE, false>(st, a, status);
    }
    return 1;
}

}  // namespace dsmoe
