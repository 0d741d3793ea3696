// Routed-expert matvec kernels for decode: IQ2_XXS gate/up + SwiGLU, Q2_K down + slot sum.
//
// Both are streaming decode-and-dot kernels bounded by HBM bandwidth on the packed weight bytes (66 B resp. 84 B per
// 256 weights). A warp owns a weight row; each lane keeps the int8 activations of its fixed K-slice in registers, so
// per row a lane only loads its 16-byte pieces of the packed row. Integer block sums are reduced across the lanes
// that share a 256-weight block, then scaled and added in exactly the order of the reference kernels
// (engine/src/kernels/moe.rs:622-715, 922-970: lane partials over blocks l, l+8, ..; butterfly xor 4, 2, 1), which
// makes the f32 results bit-identical to the CPU oracle.
#include "common.cuh"
#include "launch.h"

namespace dsmoe {

// ===============================================================================================================
// gate / up / mid, n_embd = 4096 (16 blocks per row)
// ===============================================================================================================
//
// Lane l loads 16-byte chunk l (block l/4, groups 2(l%4), 2(l%4)+1) and chunk l+32 (block 8 + l/4) of the gate row
// and of the up row: four fully coalesced 512-byte warp loads per row pair. The four lanes l/4 share a block; its
// integer sum is completed with two xor-shuffles, after which every lane of the quad holds
// dot(b) + dot(b+8) = the reference's lane partial a_b, b = l/4. Shuffles xor 16, 8, 4 then play the reference's
// xor 4, 2, 1.

struct GuRow {
    uint4 g0, g1, u0, u1;
    uint32_t dg, du;  // f16 d of blocks b | (b+8) << 16
};

template <int LAYOUT>
__device__ __forceinline__ GuRow gu_load_row(const uint8_t *grow, const uint8_t *urow, int lane)
{
    GuRow r;
    r.g0 = iq2_row_chunk<LAYOUT>(grow, 16, lane);
    r.g1 = iq2_row_chunk<LAYOUT>(grow, 16, lane + 32);
    r.u0 = iq2_row_chunk<LAYOUT>(urow, 16, lane);
    r.u1 = iq2_row_chunk<LAYOUT>(urow, 16, lane + 32);
    const int b = lane >> 2;
    r.dg = iq2_row_d<LAYOUT>(grow, b) | (iq2_row_d<LAYOUT>(grow, b + 8) << 16);
    r.du = iq2_row_d<LAYOUT>(urow, b) | (iq2_row_d<LAYOUT>(urow, b + 8) << 16);
    return r;
}

__device__ __forceinline__ float iq2_two_block_partial(int s0, int s1, uint32_t dbits, float yd0, float yd1, bool ieee)
{
    s0 += __shfl_xor_sync(FULL, s0, 1);
    s1 += __shfl_xor_sync(FULL, s1, 1);
    s0 += __shfl_xor_sync(FULL, s0, 2);
    s1 += __shfl_xor_sync(FULL, s1, 2);
    // ((0.125 * d_w) * d_x) * (float)bsum, engine/src/kernels/quantize.rs:811
    float d0 = __fmul_rn(__fmul_rn(__fmul_rn(0.125f, f16_bits_to_f32(dbits & 0xFFFFu, ieee)), yd0), (float)s0);
    float d1 = __fmul_rn(__fmul_rn(__fmul_rn(0.125f, f16_bits_to_f32(dbits >> 16, ieee)), yd1), (float)s1);
    float a = __fadd_rn(__fadd_rn(0.0f, d0), d1);
    a = __fadd_rn(a, __shfl_xor_sync(FULL, a, 16));
    a = __fadd_rn(a, __shfl_xor_sync(FULL, a, 8));
    a = __fadd_rn(a, __shfl_xor_sync(FULL, a, 4));
    return a;
}

template <int LAYOUT>
__global__ void __launch_bounds__(256) gate_up_x16_kernel(const uint8_t *__restrict__ gate_base,
                                                           const uint8_t *__restrict__ up_base,
                                                           const uint8_t *__restrict__ xq,
                                                           const int32_t *__restrict__ selected,
                                                           const float *__restrict__ weights, float *__restrict__ gate_out,
                                                           float *__restrict__ up_out, float *__restrict__ mid_out,
                                                           uint64_t expert_bytes, uint64_t row_bytes, uint32_t mid_dim,
                                                           uint32_t k, float clamp, int ieee_i, int rows_per_cta)
{
    __shared__ uint2 s_grid[DSMOE_IQ2XXS_GRID_ENTRIES];
    __shared__ uint2 s_sign[DSMOE_IQ2_SIGN_ENTRIES];
    fill_iq2_tables(s_grid, s_sign, threadIdx.x, 256);
    __syncthreads();

    const bool ieee = ieee_i != 0;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const uint32_t pair = blockIdx.y, tok = pair / k;
    const int32_t e = selected[pair];
    const uint64_t ex = e < 0 ? 0u : (uint64_t)e;
    const float w = weights[pair];

    // activations of this lane's K-slice: 64 int8 of block b and 64 of block b+8
    const int b = lane >> 2, part = lane & 3;
    const uint8_t *xt = xq + (size_t)tok * 16 * Q8K_BYTES;
    int qa[16], qb[16];
    {
        const int *pa = reinterpret_cast<const int *>(xt + Q8K_BYTES * b + 4 + 64 * part);
        const int *pb = reinterpret_cast<const int *>(xt + Q8K_BYTES * (b + 8) + 4 + 64 * part);
#pragma unroll
        for (int i = 0; i < 16; ++i) {
            qa[i] = pa[i];
            qb[i] = pb[i];
        }
    }
    const float yd0 = *reinterpret_cast<const float *>(xt + Q8K_BYTES * b);
    const float yd1 = *reinterpret_cast<const float *>(xt + Q8K_BYTES * (b + 8));

    const uint32_t row_begin = blockIdx.x * rows_per_cta;
    const uint32_t row_end = min(mid_dim, row_begin + rows_per_cta);
    uint32_t row = row_begin + warp;
    if (row >= row_end) return;
    const uint8_t *gexp = gate_base + ex * expert_bytes, *uexp = up_base + ex * expert_bytes;
    GuRow cur = gu_load_row<LAYOUT>(gexp + (uint64_t)row * row_bytes, uexp + (uint64_t)row * row_bytes, lane);
    for (; row < row_end; row += 8) {
        const uint32_t nrow = row + 8;
        GuRow nxt = cur;
        if (nrow < row_end)
            nxt = gu_load_row<LAYOUT>(gexp + (uint64_t)nrow * row_bytes, uexp + (uint64_t)nrow * row_bytes, lane);

        int sg0 = iq2_group_dot(cur.g0.x, cur.g0.y, qa, s_grid, s_sign) +
                  iq2_group_dot(cur.g0.z, cur.g0.w, qa + 8, s_grid, s_sign);
        int sg1 = iq2_group_dot(cur.g1.x, cur.g1.y, qb, s_grid, s_sign) +
                  iq2_group_dot(cur.g1.z, cur.g1.w, qb + 8, s_grid, s_sign);
        int su0 = iq2_group_dot(cur.u0.x, cur.u0.y, qa, s_grid, s_sign) +
                  iq2_group_dot(cur.u0.z, cur.u0.w, qa + 8, s_grid, s_sign);
        int su1 = iq2_group_dot(cur.u1.x, cur.u1.y, qb, s_grid, s_sign) +
                  iq2_group_dot(cur.u1.z, cur.u1.w, qb + 8, s_grid, s_sign);
        float g = iq2_two_block_partial(sg0, sg1, cur.dg, yd0, yd1, ieee);
        float u = iq2_two_block_partial(su0, su1, cur.du, yd0, yd1, ieee);
        if (lane == 0) {
            if (clamp > 1.0e-6f) {
                if (g > clamp) g = clamp;
                if (u > clamp) u = clamp;
                if (u < -clamp) u = -clamp;
            }
            const size_t off = (size_t)pair * mid_dim + row;
            if (gate_out) gate_out[off] = g;
            if (up_out) up_out[off] = u;
            mid_out[off] = swiglu_weighted(g, u, w);
        }
        cur = nxt;
    }
}

// ===============================================================================================================
// gate / up / mid, any number of blocks per row (correctness path for other shapes)
// ===============================================================================================================
//
// Lane l takes 32-weight groups l, l+32, ...: group g lies in block g/8, so eight consecutive lanes share a block
// (three xor-shuffles complete its integer sum) and in step i lane group c = l/8 holds block 4i + c, which feeds the
// reference's lane partial a_(c) for even i and a_(c+4) for odd i, in ascending block order.
template <int LAYOUT>
__global__ void __launch_bounds__(256) gate_up_generic_kernel(const uint8_t *__restrict__ gate_base,
                                                               const uint8_t *__restrict__ up_base,
                                                               const uint8_t *__restrict__ xq,
                                                               const int32_t *__restrict__ selected,
                                                               const float *__restrict__ weights,
                                                               float *__restrict__ gate_out, float *__restrict__ up_out,
                                                               float *__restrict__ mid_out, uint64_t expert_bytes,
                                                               uint64_t row_bytes, uint32_t xb, uint32_t mid_dim,
                                                               uint32_t k, float clamp, int ieee_i)
{
    __shared__ uint2 s_grid[DSMOE_IQ2XXS_GRID_ENTRIES];
    __shared__ uint2 s_sign[DSMOE_IQ2_SIGN_ENTRIES];
    fill_iq2_tables(s_grid, s_sign, threadIdx.x, 256);
    __syncthreads();

    const bool ieee = ieee_i != 0;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const uint32_t pair = blockIdx.y, tok = pair / k;
    const uint32_t row = blockIdx.x * 8 + warp;
    if (row >= mid_dim) return;
    const int32_t e = selected[pair];
    const uint64_t ex = e < 0 ? 0u : (uint64_t)e;
    const uint8_t *rows[2] = {gate_base + ex * expert_bytes + (uint64_t)row * row_bytes,
                              up_base + ex * expert_bytes + (uint64_t)row * row_bytes};
    const uint8_t *xt = xq + (size_t)tok * xb * Q8K_BYTES;
    const int grp = lane & 7, c = lane >> 3;
    float acc[2][2] = {{0.0f, 0.0f}, {0.0f, 0.0f}};  // [matrix][a_c, a_(c+4)]
    const uint32_t steps = (xb + 3) / 4;
    for (uint32_t i = 0; i < steps; ++i) {
        const uint32_t blk = 4 * i + c;
        const bool valid = blk < xb;
        int q[8];
        float yd = 0.0f;
        if (valid) {
            const int *qp = reinterpret_cast<const int *>(xt + Q8K_BYTES * blk + 4 + 32 * grp);
#pragma unroll
            for (int j = 0; j < 8; ++j) q[j] = qp[j];
            yd = *reinterpret_cast<const float *>(xt + Q8K_BYTES * blk);
        } else {
#pragma unroll
            for (int j = 0; j < 8; ++j) q[j] = 0;
        }
#pragma unroll
        for (int m = 0; m < 2; ++m) {
            int s = 0;
            uint32_t dbits = 0;
            if (valid) {
                const uint8_t *gp = LAYOUT == DSMOE_LAYOUT_ROWSOA ? rows[m] + 2 * xb + 64 * blk + 8 * grp
                                                                  : rows[m] + IQ2XXS_BYTES * blk + 2 + 8 * grp;
                const uint16_t *hp = reinterpret_cast<const uint16_t *>(gp);
                uint32_t aux0 = (uint32_t)hp[0] | ((uint32_t)hp[1] << 16);
                uint32_t aux1 = (uint32_t)hp[2] | ((uint32_t)hp[3] << 16);
                s = iq2_group_dot(aux0, aux1, q, s_grid, s_sign);
                dbits = iq2_row_d<LAYOUT>(rows[m], blk);
            }
            s += __shfl_xor_sync(FULL, s, 1);
            s += __shfl_xor_sync(FULL, s, 2);
            s += __shfl_xor_sync(FULL, s, 4);
            if (valid) {
                float d = __fmul_rn(__fmul_rn(__fmul_rn(0.125f, f16_bits_to_f32(dbits, ieee)), yd), (float)s);
                acc[m][i & 1] = __fadd_rn(acc[m][i & 1], d);
            }
        }
    }
    float r[2];
#pragma unroll
    for (int m = 0; m < 2; ++m) {
        float a = __fadd_rn(acc[m][0], acc[m][1]);  // a_c + a_(c+4)
        a = __fadd_rn(a, __shfl_xor_sync(FULL, a, 16));
        a = __fadd_rn(a, __shfl_xor_sync(FULL, a, 8));
        r[m] = a;
    }
    if (lane == 0) {
        float g = r[0], u = r[1];
        if (clamp > 1.0e-6f) {
            if (g > clamp) g = clamp;
            if (u > clamp) u = clamp;
            if (u < -clamp) u = -clamp;
        }
        const size_t off = (size_t)pair * mid_dim + row;
        if (gate_out) gate_out[off] = g;
        if (up_out) up_out[off] = u;
        mid_out[off] = swiglu_weighted(g, u, weights[pair]);
    }
}

int launch_gate_up_mid(cudaStream_t st, const GateUpArgs &a)
{
    const uint32_t pairs = a.n_tokens * a.k;
    if (pairs == 0 || a.mid_dim == 0) return 0;
    const bool fast = a.xq_blocks == 16 && (a.layout == DSMOE_LAYOUT_NATIVE ||
                                            (((uintptr_t)a.gate_base | (uintptr_t)a.up_base | a.expert_bytes | a.row_bytes) & 15) == 0);
    if (fast) {
        // keep at least ~4 CTAs per SM in flight for small batches, fewer and longer CTAs for large ones
        int rows_per_cta = pairs <= 8 ? 32 : (pairs <= 64 ? 64 : 128);
        dim3 grid((a.mid_dim + rows_per_cta - 1) / rows_per_cta, pairs);
        if (a.layout == DSMOE_LAYOUT_ROWSOA)
            gate_up_x16_kernel<DSMOE_LAYOUT_ROWSOA><<<grid, 256, 0, st>>>(
                a.gate_base, a.up_base, a.xq, a.selected, a.weights, a.gate_out, a.up_out, a.mid_out, a.expert_bytes,
                a.row_bytes, a.mid_dim, a.k, a.clamp, a.ieee, rows_per_cta);
        else
            gate_up_x16_kernel<DSMOE_LAYOUT_NATIVE><<<grid, 256, 0, st>>>(
                a.gate_base, a.up_base, a.xq, a.selected, a.weights, a.gate_out, a.up_out, a.mid_out, a.expert_bytes,
                a.row_bytes, a.mid_dim, a.k, a.clamp, a.ieee, rows_per_cta);
    } else {
        dim3 grid((a.mid_dim + 7) / 8, pairs);
        if (a.layout == DSMOE_LAYOUT_ROWSOA)
            gate_up_generic_kernel<DSMOE_LAYOUT_ROWSOA><<<grid, 256, 0, st>>>(
                a.gate_base, a.up_base, a.xq, a.selected, a.weights, a.gate_out, a.up_out, a.mid_out, a.expert_bytes,
                a.row_bytes, a.xq_blocks, a.mid_dim, a.k, a.clamp, a.ieee);
        else
            gate_up_generic_kernel<DSMOE_LAYOUT_NATIVE><<<grid, 256, 0, st>>>(
                a.gate_base, a.up_base, a.xq, a.selected, a.weights, a.gate_out, a.up_out, a.mid_out, a.expert_bytes,
                a.row_bytes, a.xq_blocks, a.mid_dim, a.k, a.clamp, a.ieee);
    }
    return 1;
}

// ===============================================================================================================
// down projection (+ slot sum)
// ===============================================================================================================
//
// One CTA per (token, chunk of R output rows), one warp per routed slot. Lane l of a slot's warp owns quarter l%4 of
// block l/4 of the mid row (n_ff = 2048 -> 8 blocks -> exactly 32 quarters), keeps those 64 activations in registers
// and, per output row, loads 16 quant bytes, 8 scale bytes and the f16 pair. Two xor-shuffles complete a block's
// integer sums; xor 16, 8, 4 reproduce the reference's quarter-warp butterfly. Slot results meet in shared memory and
// are summed in slot order (engine/src/kernels/moe.rs:937-968).

struct DnRow {
    uint4 qs;
    uint2 sc;
    uint32_t dd;
};

template <int LAYOUT>
__device__ __forceinline__ DnRow dn_load_row(const uint8_t *rowp, int mb, int b, int c)
{
    DnRow r;
    const uint8_t *qp = q2k_qs_ptr<LAYOUT>(rowp, mb, b) + 16 * c;
    const uint8_t *sp = q2k_scales_ptr<LAYOUT>(rowp, mb, b) + 8 * (c >> 1);
    if (LAYOUT == DSMOE_LAYOUT_ROWSOA) {
        r.qs = ld_stream_16B(qp);
        r.sc = ld_stream_8B(sp);
    } else {
        r.qs = ld_16B_align4(qp);
        r.sc = make_uint2(ld_u32(sp), ld_u32(sp + 4));
    }
    r.dd = ld_u32(q2k_dd_ptr<LAYOUT>(rowp, mb, b));
    return r;
}

// Block dot from the lane's quarter: completes the integer sums over the quad and applies
// dall*isum - dmin*summs (engine/src/kernels/quantize.rs:856-900).
__device__ __forceinline__ float q2k_block_dot(const DnRow &r, const int (&q)[4][4], uint32_t bs01, uint32_t bs23,
                                               float yd, int half, bool ieee)
{
    uint32_t sc4 = __byte_perm(r.sc.x, r.sc.y, half ? 0x7531u : 0x6420u);
    int isum, summs;
    q2k_quarter_dot(r.qs, q, sc4, bs01, bs23, isum, summs);
    isum += __shfl_xor_sync(FULL, isum, 1);
    summs += __shfl_xor_sync(FULL, summs, 1);
    isum += __shfl_xor_sync(FULL, isum, 2);
    summs += __shfl_xor_sync(FULL, summs, 2);
    float dall = __fmul_rn(yd, f16_bits_to_f32(r.dd & 0xFFFFu, ieee));
    float dmin = __fmul_rn(yd, f16_bits_to_f32(r.dd >> 16, ieee));
    return __fsub_rn(__fmul_rn(dall, (float)isum), __fmul_rn(dmin, (float)summs));
}


constexpr int DOWN_ROWS_MAX = 32;

template <int LAYOUT, bool SUM>
__global__ void __launch_bounds__(256) down_m8_kernel(const uint8_t *__restrict__ down_base,
                                                       const uint8_t *__restrict__ midq,
                                                       const int32_t *__restrict__ selected, float *__restrict__ out,
                                                       uint64_t expert_bytes, uint64_t row_bytes, uint32_t out_dim,
                                                       uint32_t k, int ieee_i, int rows_per_cta)
{
    __shared__ float s_part[MAX_K][DOWN_ROWS_MAX];
    const bool ieee = ieee_i != 0;
    const int lane = threadIdx.x & 31, slot = threadIdx.x >> 5;
    const uint32_t tok = blockIdx.y, pair = tok * k + slot;
    const int32_t e = selected[pair];
    const uint64_t ex = e < 0 ? 0u : (uint64_t)e;
    const int b = lane >> 2, c = lane & 3;

    int q[4][4];
    uint32_t bs01, bs23;
    float yd;
    q2k_load_acts(midq + ((size_t)pair * 8 + b) * Q8K_BYTES, c, q, bs01, bs23, yd);

    const uint32_t row_begin = blockIdx.x * rows_per_cta;
    const uint32_t n_rows = min((uint32_t)rows_per_cta, out_dim - row_begin);
    const uint8_t *wexp = down_base + ex * expert_bytes + (uint64_t)row_begin * row_bytes;
    DnRow cur = dn_load_row<LAYOUT>(wexp, 8, b, c);
    for (uint32_t r = 0; r < n_rows; ++r) {
        DnRow nxt = cur;
        if (r + 1 < n_rows) nxt = dn_load_row<LAYOUT>(wexp + (uint64_t)(r + 1) * row_bytes, 8, b, c);
        float a = __fadd_rn(0.0f, q2k_block_dot(cur, q, bs01, bs23, yd, c & 1, ieee));
        a = __fadd_rn(a, __shfl_xor_sync(FULL, a, 16));
        a = __fadd_rn(a, __shfl_xor_sync(FULL, a, 8));
        a = __fadd_rn(a, __shfl_xor_sync(FULL, a, 4));
        if (lane == 0) {
            if (SUM) s_part[slot][r] = a;
            else out[(size_t)pair * out_dim + row_begin + r] = a;
        }
        cur = nxt;
    }
    if (SUM) {
        __syncthreads();
        if (threadIdx.x < n_rows) {
            float total = 0.0f;
            for (uint32_t s = 0; s < k; ++s) total = __fadd_rn(total, s_part[s][threadIdx.x]);
            out[(size_t)tok * out_dim + row_begin + threadIdx.x] = total;
        }
    }
}

// Any number of blocks per mid row: lane l takes quarters l, l+32, ... (block q/4), so in step i lane quad l/4 holds
// block 8i + l/4, the reference's lane partial a_(l/4), in ascending block order.
template <int LAYOUT, bool SUM>
__global__ void __launch_bounds__(256) down_generic_kernel(const uint8_t *__restrict__ down_base,
                                                            const uint8_t *__restrict__ midq,
                                                            const int32_t *__restrict__ selected,
                                                            float *__restrict__ out, uint64_t expert_bytes,
                                                            uint64_t row_bytes, uint32_t mb, uint32_t out_dim, uint32_t k,
                                                            int ieee_i, int rows_per_cta)
{
    __shared__ float s_part[MAX_K][DOWN_ROWS_MAX];
    const bool ieee = ieee_i != 0;
    const int lane = threadIdx.x & 31, slot = threadIdx.x >> 5;
    const uint32_t tok = blockIdx.y, pair = tok * k + slot;
    const int32_t e = selected[pair];
    const uint64_t ex = e < 0 ? 0u : (uint64_t)e;
    const int c = lane & 3;
    const uint32_t row_begin = blockIdx.x * rows_per_cta;
    const uint32_t n_rows = min((uint32_t)rows_per_cta, out_dim - row_begin);
    const uint32_t steps = (mb + 7) / 8;
    for (uint32_t r = 0; r < n_rows; ++r) {
        const uint8_t *rowp = down_base + ex * expert_bytes + (uint64_t)(row_begin + r) * row_bytes;
        float a = 0.0f;
        for (uint32_t i = 0; i < steps; ++i) {
            const uint32_t blk = 8 * i + (lane >> 2);
            const bool valid = blk < mb;
            int q[4][4] = {};
            uint32_t bs01 = 0, bs23 = 0;
            float yd = 0.0f;
            DnRow d = {make_uint4(0, 0, 0, 0), make_uint2(0, 0), 0};
            if (valid) {
                q2k_load_acts(midq + ((size_t)pair * mb + blk) * Q8K_BYTES, c, q, bs01, bs23, yd);
                const uint8_t *qp = q2k_qs_ptr<LAYOUT>(rowp, mb, blk) + 16 * c;
                const uint8_t *sp = q2k_scales_ptr<LAYOUT>(rowp, mb, blk) + 8 * (c >> 1);
                d.qs = ld_16B_align4(qp);
                d.sc = make_uint2(ld_u32(sp), ld_u32(sp + 4));
                d.dd = ld_u32(q2k_dd_ptr<LAYOUT>(rowp, mb, blk));
            }
            float dot = q2k_block_dot(d, q, bs01, bs23, yd, c & 1, ieee);
            if (valid) a = __fadd_rn(a, dot);
        }
        a = __fadd_rn(a, __shfl_xor_sync(FULL, a, 16));
        a = __fadd_rn(a, __shfl_xor_sync(FULL, a, 8));
        a = __fadd_rn(a, __shfl_xor_sync(FULL, a, 4));
        if (lane == 0) {
            if (SUM) s_part[slot][r] = a;
            else out[(size_t)pair * out_dim + row_begin + r] = a;
        }
    }
    if (SUM) {
        __syncthreads();
        if (threadIdx.x < n_rows) {
            float total = 0.0f;
            for (uint32_t s = 0; s < k; ++s) total = __fadd_rn(total, s_part[s][threadIdx.x]);
            out[(size_t)tok * out_dim + row_begin + threadIdx.x] = total;
        }
    }
}

template <int LAYOUT, bool SUM>
static void launch_down_t(cudaStream_t st, const DownArgs &a, bool fast, int rows_per_cta)
{
    dim3 grid((a.out_dim + rows_per_cta - 1) / rows_per_cta, a.n_tokens);
    if (fast)
        down_m8_kernel<LAYOUT, SUM><<<grid, 32 * a.k, 0, st>>>(a.down_base, a.midq, a.selected, a.out, a.expert_bytes,
                                                               a.row_bytes, a.out_dim, a.k, a.ieee, rows_per_cta);
    else
        down_generic_kernel<LAYOUT, SUM><<<grid, 32 * a.k, 0, st>>>(a.down_base, a.midq, a.selected, a.out,
                                                                    a.expert_bytes, a.row_bytes, a.midq_blocks,
                                                                    a.out_dim, a.k, a.ieee, rows_per_cta);
}

int launch_down(cudaStream_t st, const DownArgs &a)
{
    if (a.n_tokens == 0 || a.out_dim == 0) return 0;
    const bool fast = a.midq_blocks == 8 && (a.layout == DSMOE_LAYOUT_NATIVE ||
                                             (((uintptr_t)a.down_base | a.expert_bytes | a.row_bytes) & 15) == 0);
    const int rows_per_cta = a.n_tokens <= 2 ? 8 : (a.n_tokens <= 16 ? 16 : 32);
    if (a.layout == DSMOE_LAYOUT_ROWSOA) {
        if (a.sum_slots) launch_down_t<DSMOE_LAYOUT_ROWSOA, true>(st, a, fast, rows_per_cta);
        else launch_down_t<DSMOE_LAYOUT_ROWSOA, false>(st, a, fast, rows_per_cta);
    } else {
        if (a.sum_slots) launch_down_t<DSMOE_LAYOUT_NATIVE, true>(st, a, fast, rows_per_cta);
        else launch_down_t<DSMOE_LAYOUT_NATIVE, false>(st, a, fast, rows_per_cta);
    }
    return 1;
}

}  // namespace dsmoe
