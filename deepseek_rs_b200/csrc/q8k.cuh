// Q8_K quantisation of one 256-element block by one warp (lane l owns elements 8l .. 8l+7), shared by the quantiser
// kernels and by the decode gate/up kernel, which quantises a block of mid as soon as its last row is stored.
//
// Result is bit-identical to the reference kernel (engine/src/kernels/quantize.rs:309-417). Its shared-memory
// halving tree keeps the lower slot on equal magnitudes, level by level from stride 128 down to 1, so among equal
// maxima the element with the smallest bit-reversed index wins; using (|x|, bit-reversed index) as the reduction key
// reproduces that choice (and hence the sign of d) in any reduction order.
#pragma once

#include "common.cuh"

namespace dsmoe {

// v: the lane's eight elements 8 lane .. 8 lane + 7 of the block
__device__ __forceinline__ void q8k_quantize_vals(const float (&v)[8], uint8_t *__restrict__ yb, int lane)
{

    float best_abs = -1.0f, best_val = 0.0f;
    uint32_t best_rev = 0xFFFFFFFFu;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        float a = v[i] < 0.0f ? -v[i] : v[i];
        uint32_t rev = __brev((uint32_t)(8 * lane + i)) >> 24;
        if (a > best_abs || (a == best_abs && rev < best_rev)) {
            best_abs = a;
            best_val = v[i];
            best_rev = rev;
        }
    }
#pragma unroll
    for (int m = 16; m > 0; m >>= 1) {
        float oa = __shfl_xor_sync(FULL, best_abs, m);
        float ov = __shfl_xor_sync(FULL, best_val, m);
        uint32_t orv = __shfl_xor_sync(FULL, best_rev, m);
        if (oa > best_abs || (oa == best_abs && orv < best_rev)) {
            best_abs = oa;
            best_val = ov;
            best_rev = orv;
        }
    }

    uint32_t *qdst = reinterpret_cast<uint32_t *>(yb + 4 + 8 * lane);
    if (!(best_abs > 0.0f)) {  // amax == 0 (or no finite maximum): all-zero block
        if (lane == 0) *reinterpret_cast<float *>(yb) = 0.0f;
        qdst[0] = 0u;
        qdst[1] = 0u;
        if (lane < 16) reinterpret_cast<uint16_t *>(yb + 260)[lane] = 0;
        return;
    }
    const float iscale = __fdiv_rn(-127.0f, best_val);
    if (lane == 0) *reinterpret_cast<float *>(yb) = __fdiv_rn(1.0f, iscale);

    int q[8], s = 0;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        float raw = __fmul_rn(iscale, v[i]);
        int qi = raw >= 0.0f ? __float2int_rz(__fadd_rn(raw, 0.5f)) : __float2int_rz(__fadd_rn(raw, -0.5f));
        qi = max(-128, min(127, qi));
        q[i] = qi;
        s += qi;
    }
    qdst[0] = (uint32_t)(q[0] & 255) | ((uint32_t)(q[1] & 255) << 8) | ((uint32_t)(q[2] & 255) << 16) |
              ((uint32_t)(q[3] & 255) << 24);
    qdst[1] = (uint32_t)(q[4] & 255) | ((uint32_t)(q[5] & 255) << 8) | ((uint32_t)(q[6] & 255) << 16) |
              ((uint32_t)(q[7] & 255) << 24);
    s += __shfl_xor_sync(FULL, s, 1);  // bsums cover 16 elements = two lanes
    if ((lane & 1) == 0) reinterpret_cast<int16_t *>(yb + 260)[lane >> 1] = (int16_t)s;
}

}  // namespace dsmoe
