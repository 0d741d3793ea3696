// Decode kernels for the reference shapes (n_embd 4096, n_ff 2048) with the packed rows staged through shared memory
// by bulk asynchronous copies (TMA, untiled), so that every SM keeps tens of kilobytes of HBM reads in flight
// without holding them in registers.
//
//   gate/up: persistent CTAs, one per SM. Each warp owns a contiguous run of (pair, row) items and a private ring of
//            GU_STAGES stages; lane 0 issues two 1056-byte bulk copies (gate row, up row) per stage onto the stage's
//            mbarrier, the warp consumes the stage two items later. The codebook and the sign masks are replicated
//            16x in shared memory, one copy per lane of a half-warp, which makes every 64-bit lookup conflict-free.
//   down:    one CTA per (token, chunk of output rows), one warp per routed slot; lane 0 fetches the warp's whole
//            chunk of that expert's rows (contiguous) with a single bulk copy while the other lanes load the int8
//            activations of their K-slice into registers.
//
// Arithmetic and summation order are those of experts.cu (and of the reference kernels), so results stay
// bit-identical to the CPU oracle.
#include "async.cuh"
#include "common.cuh"
#include "launch.h"

namespace dsmoe {

// The codebook in global memory (read coalesced when filling shared memory; constant memory would serialise the
// per-thread indices).
__device__ const uint64_t g_iq2xxs_grid[DSMOE_IQ2XXS_GRID_ENTRIES] = {DSMOE_IQ2XXS_GRID_VALUES};

constexpr int GU_STAGES = 3;
constexpr int GU_ROW_BYTES = 16 * IQ2XXS_BYTES;  // 1056
constexpr int GU_STAGE_BYTES = 2 * GU_ROW_BYTES; // gate row + up row
constexpr int GU_TABLE_BYTES = (DSMOE_IQ2XXS_GRID_ENTRIES + DSMOE_IQ2_SIGN_ENTRIES) * 16 * 8;  // 49152
constexpr int GU_MAX_WARPS = 16;

// conflict-free variant of iq2_group_dot: tg / ts point at this lane's copy (entry stride 16 uint2)
__device__ __forceinline__ int iq2_group_dot_rep(uint32_t aux0, uint32_t aux1, const int *q, const uint2 *tg,
                                                 const uint2 *ts)
{
    int pos = 0, neg = 0;
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        uint2 g = tg[((aux0 >> (8 * k)) & 255u) * 16];
        uint2 m = ts[((aux1 >> (7 * k)) & 127u) * 16];
        pos = __dp4a((int)(g.x ^ m.x), q[2 * k], pos);
        pos = __dp4a((int)(g.y ^ m.y), q[2 * k + 1], pos);
        neg = __dp4a((int)m.x, q[2 * k], neg);
        neg = __dp4a((int)m.y, q[2 * k + 1], neg);
    }
    return (pos - neg) * (int)(2u * (aux1 >> 28) + 1u);
}

template <int LAYOUT>
__device__ __forceinline__ uint4 gu_smem_chunk(const uint8_t *row, int c)
{
    if (LAYOUT == DSMOE_LAYOUT_ROWSOA) return *reinterpret_cast<const uint4 *>(row + 32 + 16 * c);
    return ld_16B_align2(row + IQ2XXS_BYTES * (c >> 2) + 2 + 16 * (c & 3));
}

__device__ __forceinline__ float gu_reduce(int s0, int s1, uint32_t d0, uint32_t d1, float yd0, float yd1, bool ieee)
{
    s0 += __shfl_xor_sync(FULL, s0, 1);
    s1 += __shfl_xor_sync(FULL, s1, 1);
    s0 += __shfl_xor_sync(FULL, s0, 2);
    s1 += __shfl_xor_sync(FULL, s1, 2);
    float p0 = __fmul_rn(__fmul_rn(__fmul_rn(0.125f, f16_bits_to_f32(d0, ieee)), yd0), (float)s0);
    float p1 = __fmul_rn(__fmul_rn(__fmul_rn(0.125f, f16_bits_to_f32(d1, ieee)), yd1), (float)s1);
    float a = __fadd_rn(__fadd_rn(0.0f, p0), p1);
    a = __fadd_rn(a, __shfl_xor_sync(FULL, a, 16));
    a = __fadd_rn(a, __shfl_xor_sync(FULL, a, 8));
    a = __fadd_rn(a, __shfl_xor_sync(FULL, a, 4));
    return a;
}

template <int LAYOUT>
__global__ void __launch_bounds__(32 * GU_MAX_WARPS, 1)
    gate_up_x16_tma_kernel(const uint8_t *__restrict__ gate_base, const uint8_t *__restrict__ up_base,
                           const uint8_t *__restrict__ xq, const int32_t *__restrict__ selected,
                           const float *__restrict__ weights, float *__restrict__ gate_out, float *__restrict__ up_out,
                           float *__restrict__ mid_out, uint64_t expert_bytes, uint32_t mid_dim, uint32_t k,
                           uint32_t n_items, float clamp, int ieee_i, int *status)
{
    extern __shared__ __align__(128) uint8_t smem[];
    uint2 *s_grid = reinterpret_cast<uint2 *>(smem);
    uint2 *s_sign = s_grid + DSMOE_IQ2XXS_GRID_ENTRIES * 16;
    const int wpc = blockDim.x >> 5, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    uint8_t *ring = smem + GU_TABLE_BYTES + (size_t)warp * GU_STAGES * GU_STAGE_BYTES;
    uint64_t *bars = reinterpret_cast<uint64_t *>(smem + GU_TABLE_BYTES + (size_t)wpc * GU_STAGES * GU_STAGE_BYTES) +
                     warp * GU_STAGES;

    for (int i = threadIdx.x; i < DSMOE_IQ2XXS_GRID_ENTRIES * 16; i += blockDim.x) {
        uint64_t g = g_iq2xxs_grid[i >> 4];
        s_grid[i] = make_uint2((uint32_t)g, (uint32_t)(g >> 32));
    }
    for (int i = threadIdx.x; i < DSMOE_IQ2_SIGN_ENTRIES * 16; i += blockDim.x) {
        uint32_t sb = dsmoe_iq2_sign_byte((uint32_t)(i >> 4));
        s_sign[i] = make_uint2(nibble_to_bytemask(sb), nibble_to_bytemask(sb >> 4));
    }
    if (lane == 0) {
#pragma unroll
        for (int s = 0; s < GU_STAGES; ++s) mbar_init(&bars[s], 1);
        fence_async_smem();
    }
    __syncthreads();

    // this warp's run of items; item = pair * mid_dim + row
    const uint32_t n_warps = gridDim.x * wpc, gw = blockIdx.x * wpc + warp;
    const uint32_t chunk = (n_items + n_warps - 1) / n_warps;
    const uint32_t begin = min(n_items, gw * chunk), end = min(n_items, begin + chunk);
    if (begin >= end) return;
    const bool ieee = ieee_i != 0;
    const uint2 *tg = s_grid + (lane & 15), *ts = s_sign + (lane & 15);
    const int b = lane >> 2, part = lane & 3;

    auto issue = [&](uint32_t item, int stage) {
        if (lane == 0) {
            const uint32_t pair = item / mid_dim, row = item - pair * mid_dim;
            const int32_t e = selected[pair];
            const uint64_t off = (e < 0 ? 0u : (uint64_t)e) * expert_bytes + (uint64_t)row * GU_ROW_BYTES;
            uint8_t *dst = ring + stage * GU_STAGE_BYTES;
            mbar_expect_tx(&bars[stage], GU_STAGE_BYTES);
            bulk_g2s(dst, gate_base + off, GU_ROW_BYTES, &bars[stage]);
            bulk_g2s(dst + GU_ROW_BYTES, up_base + off, GU_ROW_BYTES, &bars[stage]);
        }
    };
#pragma unroll
    for (int j = 0; j < GU_STAGES - 1; ++j)
        if (begin + j < end) issue(begin + j, j);

    int qa[16], qb[16];
    float yd0 = 0.0f, yd1 = 0.0f, w = 0.0f;
    uint32_t cur_pair = 0xFFFFFFFFu;
    uint32_t it = 0;
    for (uint32_t item = begin; item < end; ++item, ++it) {
        const int stage = it % GU_STAGES;
        const uint32_t pair = item / mid_dim, row = item - pair * mid_dim;
        if (pair != cur_pair) {  // new (token, slot): reload this lane's slice of the token's Q8_K row
            cur_pair = pair;
            const uint8_t *xt = xq + (size_t)(pair / k) * 16 * Q8K_BYTES;
            const int *pa = reinterpret_cast<const int *>(xt + Q8K_BYTES * b + 4 + 64 * part);
            const int *pb = reinterpret_cast<const int *>(xt + Q8K_BYTES * (b + 8) + 4 + 64 * part);
#pragma unroll
            for (int i = 0; i < 16; ++i) {
                qa[i] = pa[i];
                qb[i] = pb[i];
            }
            yd0 = *reinterpret_cast<const float *>(xt + Q8K_BYTES * b);
            yd1 = *reinterpret_cast<const float *>(xt + Q8K_BYTES * (b + 8));
            w = weights[pair];
        }
        // refill the stage consumed one iteration ago (all lanes finished reading it before the __syncwarp below)
        if (item + GU_STAGES - 1 < end) {
            fence_async_smem();
            issue(item + GU_STAGES - 1, (it + GU_STAGES - 1) % GU_STAGES);
        }
        if (!mbar_wait_bounded(&bars[stage], (it / GU_STAGES) & 1, status)) return;
        const uint8_t *grow = ring + stage * GU_STAGE_BYTES, *urow = grow + GU_ROW_BYTES;
        const uint4 g0 = gu_smem_chunk<LAYOUT>(grow, lane), g1 = gu_smem_chunk<LAYOUT>(grow, lane + 32);
        const uint4 u0 = gu_smem_chunk<LAYOUT>(urow, lane), u1 = gu_smem_chunk<LAYOUT>(urow, lane + 32);
        const uint32_t dstep = LAYOUT == DSMOE_LAYOUT_ROWSOA ? 2 : IQ2XXS_BYTES;
        const uint32_t dg0 = ld_u16(grow + dstep * b), dg1 = ld_u16(grow + dstep * (b + 8));
        const uint32_t du0 = ld_u16(urow + dstep * b), du1 = ld_u16(urow + dstep * (b + 8));
        __syncwarp();

        int sg0 = iq2_group_dot_rep(g0.x, g0.y, qa, tg, ts) + iq2_group_dot_rep(g0.z, g0.w, qa + 8, tg, ts);
        int sg1 = iq2_group_dot_rep(g1.x, g1.y, qb, tg, ts) + iq2_group_dot_rep(g1.z, g1.w, qb + 8, tg, ts);
        int su0 = iq2_group_dot_rep(u0.x, u0.y, qa, tg, ts) + iq2_group_dot_rep(u0.z, u0.w, qa + 8, tg, ts);
        int su1 = iq2_group_dot_rep(u1.x, u1.y, qb, tg, ts) + iq2_group_dot_rep(u1.z, u1.w, qb + 8, tg, ts);
        float g = gu_reduce(sg0, sg1, dg0, dg1, yd0, yd1, ieee);
        float u = gu_reduce(su0, su1, du0, du1, yd0, yd1, ieee);
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
    }
}

// ---------------------------------------------------------------------------------------------------------------

constexpr int DN_ROW_BYTES = 8 * Q2K_BYTES;  // 672
constexpr int DN_ROWS_MAX = 16;

struct DnRowS {
    uint4 qs;
    uint2 sc;
    uint32_t dd;
};

template <int LAYOUT, bool SUM>
__global__ void __launch_bounds__(256) down_m8_tma_kernel(const uint8_t *__restrict__ down_base,
                                                           const uint8_t *__restrict__ midq,
                                                           const int32_t *__restrict__ selected, float *__restrict__ out,
                                                           uint64_t expert_bytes, uint32_t out_dim, uint32_t k, int ieee_i,
                                                           int rows_per_cta, int *status)
{
    extern __shared__ __align__(128) uint8_t smem[];
    const bool ieee = ieee_i != 0;
    const int lane = threadIdx.x & 31, slot = threadIdx.x >> 5;
    uint8_t *wbuf = smem + (size_t)slot * rows_per_cta * DN_ROW_BYTES;
    float *s_part = reinterpret_cast<float *>(smem + (size_t)k * rows_per_cta * DN_ROW_BYTES);
    uint64_t *bar = reinterpret_cast<uint64_t *>(s_part + MAX_K * DN_ROWS_MAX) + slot;

    const uint32_t tok = blockIdx.y, pair = tok * k + slot;
    const uint32_t row_begin = blockIdx.x * rows_per_cta;
    const uint32_t n_rows = min((uint32_t)rows_per_cta, out_dim - row_begin);
    if (lane == 0) {
        const int32_t e = selected[pair];
        const uint64_t ex = e < 0 ? 0u : (uint64_t)e;
        mbar_init(bar, 1);
        fence_async_smem();
        mbar_expect_tx(bar, n_rows * DN_ROW_BYTES);
        bulk_g2s(wbuf, down_base + ex * expert_bytes + (uint64_t)row_begin * DN_ROW_BYTES, n_rows * DN_ROW_BYTES, bar);
    }
    const int b = lane >> 2, c = lane & 3;
    int q[4][4];
    uint32_t bs01, bs23;
    float yd;
    q2k_load_acts(midq + ((size_t)pair * 8 + b) * Q8K_BYTES, c, q, bs01, bs23, yd);
    __syncwarp();  // the barrier lane 0 initialised is now visible to the whole warp
    const bool ok = mbar_wait_bounded(bar, 0, status);

    for (uint32_t r = 0; ok && r < n_rows; ++r) {
        const uint8_t *rowp = wbuf + r * DN_ROW_BYTES;
        DnRowS d;
        const uint8_t *qp = q2k_qs_ptr<LAYOUT>(rowp, 8, b) + 16 * c;
        const uint8_t *sp = q2k_scales_ptr<LAYOUT>(rowp, 8, b) + 8 * (c >> 1);
        if (LAYOUT == DSMOE_LAYOUT_ROWSOA) {
            d.qs = *reinterpret_cast<const uint4 *>(qp);
            d.sc = *reinterpret_cast<const uint2 *>(sp);
        } else {
            d.qs = ld_16B_align4(qp);
            d.sc = make_uint2(ld_u32(sp), ld_u32(sp + 4));
        }
        d.dd = ld_u32(q2k_dd_ptr<LAYOUT>(rowp, 8, b));

        uint32_t sc4 = __byte_perm(d.sc.x, d.sc.y, (c & 1) ? 0x7531u : 0x6420u);
        int isum, summs;
        q2k_quarter_dot(d.qs, q, sc4, bs01, bs23, isum, summs);
        isum += __shfl_xor_sync(FULL, isum, 1);
        summs += __shfl_xor_sync(FULL, summs, 1);
        isum += __shfl_xor_sync(FULL, isum, 2);
        summs += __shfl_xor_sync(FULL, summs, 2);
        float dall = __fmul_rn(yd, f16_bits_to_f32(d.dd & 0xFFFFu, ieee));
        float dmin = __fmul_rn(yd, f16_bits_to_f32(d.dd >> 16, ieee));
        float a = __fadd_rn(0.0f, __fsub_rn(__fmul_rn(dall, (float)isum), __fmul_rn(dmin, (float)summs)));
        a = __fadd_rn(a, __shfl_xor_sync(FULL, a, 16));
        a = __fadd_rn(a, __shfl_xor_sync(FULL, a, 8));
        a = __fadd_rn(a, __shfl_xor_sync(FULL, a, 4));
        if (lane == 0) {
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

static int g_sm_count = 0;

static int sm_count()
{
    if (g_sm_count == 0) {
        int dev = 0;
        cudaGetDevice(&dev);
        cudaDeviceGetAttribute(&g_sm_count, cudaDevAttrMultiProcessorCount, dev);
        if (g_sm_count <= 0) g_sm_count = 148;
    }
    return g_sm_count;
}

bool gate_up_tma_eligible(const GateUpArgs &a)
{
    return a.xq_blocks == 16 && a.row_bytes == (uint64_t)GU_ROW_BYTES &&
           (((uintptr_t)a.gate_base | (uintptr_t)a.up_base | a.expert_bytes) & 15) == 0;
}

template <int LAYOUT>
static void launch_gu_tma(cudaStream_t st, const GateUpArgs &a, int *status)
{
    const uint32_t n_items = a.n_tokens * a.k * a.mid_dim;
    const int sms = sm_count();
    // warps per CTA: the count in 8..16 that leaves the fewest idle warp-slots in the last round of items
    int best_w = 16;
    double best_eff = 0.0;
    for (int w = 16; w >= 8; --w) {
        const uint32_t nw = (uint32_t)sms * w, chunk = (n_items + nw - 1) / nw;
        const double eff = (double)n_items / ((double)chunk * nw);
        if (eff > best_eff + 1e-9) {
            best_eff = eff;
            best_w = w;
        }
    }
    const size_t smem = GU_TABLE_BYTES + (size_t)best_w * GU_STAGES * GU_STAGE_BYTES + (size_t)best_w * GU_STAGES * 8;
    static bool attr_set[2] = {false, false};
    if (!attr_set[LAYOUT]) {
        cudaFuncSetAttribute(gate_up_x16_tma_kernel<LAYOUT>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             GU_TABLE_BYTES + GU_MAX_WARPS * GU_STAGES * (GU_STAGE_BYTES + 8));
        attr_set[LAYOUT] = true;
    }
    const uint32_t want = (n_items + best_w - 1) / best_w;
    const uint32_t grid = want < (uint32_t)sms ? want : (uint32_t)sms;
    gate_up_x16_tma_kernel<LAYOUT><<<grid, 32 * best_w, smem, st>>>(a.gate_base, a.up_base, a.xq, a.selected, a.weights,
                                                                    a.gate_out, a.up_out, a.mid_out, a.expert_bytes,
                                                                    a.mid_dim, a.k, n_items, a.clamp, a.ieee, status);
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
           (((uintptr_t)a.down_base | a.expert_bytes) & 15) == 0;
}

template <int LAYOUT, bool SUM>
static void launch_dn_tma(cudaStream_t st, const DownArgs &a, int *status)
{
    // small batches: short chunks so that one wave of CTAs covers all rows; large batches: longer chunks
    const int rows_per_cta = a.n_tokens <= 2 ? 6 : (a.n_tokens <= 16 ? 8 : 16);
    const size_t smem = (size_t)a.k * rows_per_cta * DN_ROW_BYTES + MAX_K * DN_ROWS_MAX * 4 + MAX_K * 8;
    static bool attr_set = false;
    if (!attr_set) {
        cudaFuncSetAttribute(down_m8_tma_kernel<LAYOUT, SUM>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             MAX_K * DN_ROWS_MAX * DN_ROW_BYTES + MAX_K * DN_ROWS_MAX * 4 + MAX_K * 8);
        attr_set = true;
    }
    dim3 grid((a.out_dim + rows_per_cta - 1) / rows_per_cta, a.n_tokens);
    down_m8_tma_kernel<LAYOUT, SUM><<<grid, 32 * a.k, smem, st>>>(a.down_base, a.midq, a.selected, a.out, a.expert_bytes,
                                                                  a.out_dim, a.k, a.ieee, rows_per_cta, status);
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
