/*
 * CPU oracle for the quantized MoE expert path of jbreams/deepseek-rs.
 *
 * TEST INFRASTRUCTURE ONLY. This file restates, in plain C, the arithmetic that the reference engine performs on
 * the routed-expert path so that the CUDA kernels can be diffed against it. Nothing in the shipped library links,
 * loads or calls it; only the test-suite, the smoke check and the benchmark's CPU-baseline leg do.
 *
 * The reference is Rust compiled through cuda-oxide (nightly toolchain plus un-vendored path dependencies), which
 * cannot be built where this oracle is built, so this is a restatement ("port"), not the reference binary. It is
 * pinned against every known answer the reference's own CPU tests hold for the path
 * (engine/tests/quant_cpu.rs:304-364, :391-429, :453-501; engine/tests/kernels_smoke.rs:398-514).
 *
 * Parity status: block dots, Q8_K quantiser, router ordering and SwiGLU are pinned by those known answers.
 * Device transcendental rounding (exp/ln in the router and in SiLU) is unpinned in the reference (it comes from a
 * compiler that is not in its tree); here exp and ln are evaluated as correctly rounded f32 operations, see
 * orc_expf()/orc_logf(). The FP8 block-scaled GEMM has no reference implementation at all: parity unpinned.
 *
 * Every function cites the reference lines it follows. Floating-point contraction must be off when compiling
 * (-ffp-contract=off): the reference's host-side mirror computes each f32 operation separately.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#include "../include/dsmoe_iq2_tables.h"

#if defined(_OPENMP)
#include <omp.h>
#endif

#define ORC_QK_K 256
#define ORC_IQ2XXS_BYTES 66
#define ORC_Q2K_BYTES 84
#define ORC_Q8K_BYTES 292
#define ORC_MAX_K 8

static const uint64_t orc_grid[DSMOE_IQ2XXS_GRID_ENTRIES] = {DSMOE_IQ2XXS_GRID_VALUES};

/* ------------------------------------------------------------------------------------------------------------ */
/* scalar helpers                                                                                                 */
/* ------------------------------------------------------------------------------------------------------------ */

static inline float orc_bits_f32(uint32_t b)
{
    float f;
    memcpy(&f, &b, 4);
    return f;
}

static inline uint32_t orc_f32_bits(float f)
{
    uint32_t b;
    memcpy(&b, &f, 4);
    return b;
}

/*
 * f16 bits -> f32. ieee == 0 follows the device helper f16_bits_to_f32 (engine/src/kernels/utils.rs:16-29): a zero
 * exponent field, i.e. zero AND every f16 subnormal, becomes a signed zero. ieee != 0 converts subnormals exactly
 * (value = mant * 2^-24), which neither the device helper nor the reference's CPU test helper
 * (engine/tests/quant_cpu.rs:11-23) does; it exists so the effect of the flush can be reported.
 */
float orc_f16_to_f32(uint16_t h, int ieee)
{
    uint32_t sign = ((uint32_t)h & 0x8000u) << 16;
    uint32_t exp = ((uint32_t)h >> 10) & 0x1Fu;
    uint32_t mant = (uint32_t)h & 0x3FFu;
    if (exp == 0) {
        if (!ieee || mant == 0) return orc_bits_f32(sign);
        float v = (float)mant * 5.9604644775390625e-08f; /* 2^-24, exact */
        return sign ? -v : v;
    }
    if (exp == 31) return orc_bits_f32(sign | 0x7F800000u | (mant << 13));
    return orc_bits_f32(sign | ((exp + 112u) << 23) | (mant << 13));
}

/*
 * exp and ln as f32 operations. The reference calls f32::exp / f32::ln (engine/src/kernels/moe.rs:16-22, :709;
 * host mirror engine/tests/quant_cpu.rs:433-441) whose device rounding is not pinned by any test. The oracle
 * defines them as the correctly rounded f32 result, obtained by evaluating in double and rounding once; the CUDA
 * kernels do the same, so selection and SiLU agree bit for bit between the two.
 */
float orc_expf(float x) { return (float)exp((double)x); }
float orc_logf(float x) { return (float)log((double)x); }

/* softplus of engine/src/kernels/moe.rs:12-24 */
float orc_softplus(float x)
{
    if (x > 20.0f) return x;
    if (x < -20.0f) return orc_expf(x);
    return orc_logf(1.0f + orc_expf(x));
}

/* router probability of engine/src/kernels/moe.rs:199 */
float orc_router_score(float logit) { return sqrtf(orc_softplus(logit)); }

static inline uint16_t orc_rd_u16(const uint8_t *p) { return (uint16_t)(p[0] | ((uint16_t)p[1] << 8)); }
static inline uint32_t orc_rd_u32(const uint8_t *p)
{
    return (uint32_t)p[0] | ((uint32_t)p[1] << 8) | ((uint32_t)p[2] << 16) | ((uint32_t)p[3] << 24);
}
static inline float orc_rd_f32(const uint8_t *p) { return orc_bits_f32(orc_rd_u32(p)); }
static inline int16_t orc_rd_i16(const uint8_t *p) { return (int16_t)orc_rd_u16(p); }

/* Rust's saturating `as i32` on an f32 (NaN -> 0). */
static inline int32_t orc_f32_as_i32(float v)
{
    if (v != v) return 0;
    if (v >= 2147483648.0f) return INT32_MAX;
    if (v <= -2147483648.0f) return INT32_MIN;
    return (int32_t)v;
}

/* ------------------------------------------------------------------------------------------------------------ */
/* dequantised weights (the bit-exactness target)                                                                 */
/* ------------------------------------------------------------------------------------------------------------ */

/*
 * Signed integer code of one IQ2_XXS superblock: code[e] = ls * (+/- grid byte), the integer that multiplies
 * 0.125 * d in the block dot (engine/src/kernels/quantize.rs:777-811, :716-728).
 */
void orc_iq2xxs_codes(const uint8_t *blk, int32_t *code)
{
    for (int ib32 = 0; ib32 < 8; ++ib32) {
        const uint8_t *q2 = blk + 2 + ib32 * 8;
        uint32_t aux0 = orc_rd_u32(q2);
        uint32_t aux1 = orc_rd_u32(q2 + 4);
        int32_t ls = (int32_t)(2u * (aux1 >> 28) + 1u);
        for (int k = 0; k < 4; ++k) {
            uint64_t g = orc_grid[(aux0 >> (8 * k)) & 255u];
            uint8_t sb = dsmoe_iq2_sign_byte((aux1 >> (7 * k)) & 127u);
            for (int j = 0; j < 8; ++j) {
                int32_t mag = (int32_t)((g >> (8 * j)) & 0xFFu);
                code[ib32 * 32 + k * 8 + j] = ls * (((sb >> j) & 1) ? -mag : mag);
            }
        }
    }
}

/*
 * Dequantised IQ2_XXS weights. The reference never materialises them; the definition follows from the block dot
 * 0.125 * d * d_x * sum(ls * (+/-g) * q8) (engine/src/kernels/quantize.rs:811): w = (0.125 * d) * code. Both
 * products are exact in f32.
 */
void orc_dequant_iq2xxs(const uint8_t *blocks, int64_t n_blocks, float *out, int ieee_f16)
{
    for (int64_t b = 0; b < n_blocks; ++b) {
        const uint8_t *blk = blocks + b * ORC_IQ2XXS_BYTES;
        int32_t code[ORC_QK_K];
        float d = 0.125f * orc_f16_to_f32(orc_rd_u16(blk), ieee_f16);
        orc_iq2xxs_codes(blk, code);
        for (int e = 0; e < ORC_QK_K; ++e) out[b * ORC_QK_K + e] = d * (float)code[e];
    }
}

/*
 * Dequantised Q2_K weights: element e = 128h + 32j + i has q = (qs[32h+i] >> 2j) & 3 and sub-block 8h + 2j + i/16;
 * w = d * (sc_lo * q) - dmin * sc_hi, from dall*isum - dmin*summs (engine/src/kernels/quantize.rs:846-900).
 */
void orc_dequant_q2k(const uint8_t *blocks, int64_t n_blocks, float *out, int ieee_f16)
{
    for (int64_t b = 0; b < n_blocks; ++b) {
        const uint8_t *blk = blocks + b * ORC_Q2K_BYTES;
        float d = orc_f16_to_f32(orc_rd_u16(blk + 80), ieee_f16);
        float dmin = orc_f16_to_f32(orc_rd_u16(blk + 82), ieee_f16);
        for (int h = 0; h < 2; ++h)
            for (int j = 0; j < 4; ++j)
                for (int i = 0; i < 32; ++i) {
                    int sb = 8 * h + 2 * j + i / 16;
                    int q = (blk[16 + 32 * h + i] >> (2 * j)) & 3;
                    float a = d * (float)((blk[sb] & 0x0F) * q);
                    float m = dmin * (float)(blk[sb] >> 4);
                    out[b * ORC_QK_K + 128 * h + 32 * j + i] = a - m;
                }
    }
}

/* ------------------------------------------------------------------------------------------------------------ */
/* Q8_K activation quantiser                                                                                      */
/* ------------------------------------------------------------------------------------------------------------ */

/*
 * q8k_quantize (engine/src/kernels/quantize.rs:309-417). One 256-thread block per (row, 256-element block): a
 * shared-memory tree picks the element of largest magnitude, keeping its signed value; a strictly-greater compare
 * means the lower tree slot wins ties (:338-350). amax == 0 writes an all-zero block (:355-374). Otherwise
 * iscale = -127 / maxval, d = 1 / iscale (:378-381), q = trunc(iscale*x +/- 0.5) clamped to int8 (:389-401), and
 * bsums[j] = sum of 16 consecutive q (:408-416).
 */
void orc_q8k_quantize(const float *x, uint8_t *out, int64_t in_dim, int64_t n_rows)
{
    int64_t n_blocks = in_dim / ORC_QK_K;
    for (int64_t row = 0; row < n_rows; ++row)
        for (int64_t b = 0; b < n_blocks; ++b) {
            const float *xr = x + row * in_dim + b * ORC_QK_K;
            uint8_t *yb = out + (row * n_blocks + b) * ORC_Q8K_BYTES;
            float absp[ORC_QK_K], valp[ORC_QK_K];
            for (int t = 0; t < ORC_QK_K; ++t) {
                float v = xr[t];
                absp[t] = (v < 0.0f) ? -v : v;
                valp[t] = v;
            }
            for (int stride = ORC_QK_K / 2; stride > 0; stride >>= 1)
                for (int t = 0; t < stride; ++t)
                    if (absp[t + stride] > absp[t]) {
                        absp[t] = absp[t + stride];
                        valp[t] = valp[t + stride];
                    }
            float amax = absp[0];
            if (amax == 0.0f) {
                memset(yb, 0, ORC_Q8K_BYTES);
                continue;
            }
            float iscale = -127.0f / valp[0];
            float d = 1.0f / iscale;
            uint32_t db = orc_f32_bits(d);
            yb[0] = (uint8_t)db;
            yb[1] = (uint8_t)(db >> 8);
            yb[2] = (uint8_t)(db >> 16);
            yb[3] = (uint8_t)(db >> 24);
            int8_t *qs = (int8_t *)(yb + 4);
            for (int t = 0; t < ORC_QK_K; ++t) {
                float raw = iscale * xr[t];
                int32_t qv = (raw >= 0.0f) ? orc_f32_as_i32(raw + 0.5f) : orc_f32_as_i32(raw - 0.5f);
                qs[t] = (int8_t)(qv > 127 ? 127 : (qv < -128 ? -128 : qv));
            }
            for (int j = 0; j < 16; ++j) {
                int32_t s = 0;
                for (int k = 0; k < 16; ++k) s += qs[j * 16 + k];
                uint16_t u = (uint16_t)(int16_t)s;
                yb[260 + 2 * j] = (uint8_t)u;
                yb[261 + 2 * j] = (uint8_t)(u >> 8);
            }
        }
}

/* ------------------------------------------------------------------------------------------------------------ */
/* block dots                                                                                                     */
/* ------------------------------------------------------------------------------------------------------------ */

/* integer part of dot_iq2_xxs_q8k: sum over the 8 groups of ls * sumi (engine/src/kernels/quantize.rs:777-810) */
int32_t orc_iq2xxs_q8k_isum(const uint8_t *iq2_blk, const uint8_t *q8k_blk)
{
    const int8_t *q8 = (const int8_t *)(q8k_blk + 4);
    int32_t bsum = 0;
    for (int ib32 = 0; ib32 < 8; ++ib32) {
        const uint8_t *q2 = iq2_blk + 2 + ib32 * 8;
        uint32_t aux0 = orc_rd_u32(q2);
        uint32_t aux1 = orc_rd_u32(q2 + 4);
        int32_t ls = (int32_t)(2u * (aux1 >> 28) + 1u);
        int32_t sumi = 0;
        for (int k = 0; k < 4; ++k) {
            uint64_t g = orc_grid[(aux0 >> (8 * k)) & 255u];
            uint8_t sb = dsmoe_iq2_sign_byte((aux1 >> (7 * k)) & 127u);
            for (int j = 0; j < 8; ++j) {
                int32_t mag = (int32_t)((g >> (8 * j)) & 0xFFu);
                int32_t w = ((sb >> j) & 1) ? -mag : mag;
                sumi += w * (int32_t)q8[ib32 * 32 + k * 8 + j];
            }
        }
        bsum += sumi * ls;
    }
    return bsum;
}

/*
 * dot_iq2_xxs_q8k (engine/src/kernels/quantize.rs:763-812; host mirror engine/tests/quant_cpu.rs:43-87):
 * ((0.125 * d_w) * d_x) * (float)bsum, left to right.
 */
float orc_dot_iq2xxs_q8k(const uint8_t *iq2_blk, const uint8_t *q8k_blk, int ieee_f16)
{
    float xd = orc_f16_to_f32(orc_rd_u16(iq2_blk), ieee_f16);
    float yd = orc_rd_f32(q8k_blk);
    int32_t bsum = orc_iq2xxs_q8k_isum(iq2_blk, q8k_blk);
    float t = 0.125f * xd;
    t = t * yd;
    return t * (float)bsum;
}

/* integer parts of dot_q2k_q8k (engine/src/kernels/quantize.rs:859-899) */
void orc_q2k_q8k_isums(const uint8_t *q2k_blk, const uint8_t *q8k_blk, int32_t *isum_out, int32_t *summs_out)
{
    const uint8_t *scales = q2k_blk;
    const uint8_t *qs = q2k_blk + 16;
    const int8_t *q8 = (const int8_t *)(q8k_blk + 4);
    int32_t summs = 0;
    for (int j = 0; j < 16; ++j) summs += (int32_t)orc_rd_i16(q8k_blk + 260 + 2 * j) * (int32_t)(scales[j] >> 4);
    int32_t isum = 0;
    int is = 0;
    for (int h = 0; h < 2; ++h)
        for (int j = 0; j < 4; ++j)
            for (int half = 0; half < 2; ++half) {
                int32_t sc = scales[is++] & 0x0F;
                int32_t s = 0;
                for (int i = 0; i < 16; ++i) {
                    int q = (qs[32 * h + 16 * half + i] >> (2 * j)) & 3;
                    s += q * (int32_t)q8[128 * h + 32 * j + 16 * half + i];
                }
                isum += sc * s;
            }
    *isum_out = isum;
    *summs_out = summs;
}

/*
 * dot_q2k_q8k (engine/src/kernels/quantize.rs:846-901; host mirror engine/tests/quant_cpu.rs:90-151):
 * dall = d_x * d, dmin = d_x * dmin_w, result = dall * isum - dmin * summs, each operation rounded separately.
 */
float orc_dot_q2k_q8k(const uint8_t *q2k_blk, const uint8_t *q8k_blk, int ieee_f16)
{
    float yd = orc_rd_f32(q8k_blk);
    float dall = yd * orc_f16_to_f32(orc_rd_u16(q2k_blk + 80), ieee_f16);
    float dmin = yd * orc_f16_to_f32(orc_rd_u16(q2k_blk + 82), ieee_f16);
    int32_t isum, summs;
    orc_q2k_q8k_isums(q2k_blk, q8k_blk, &isum, &summs);
    float a = dall * (float)isum;
    float m = dmin * (float)summs;
    return a - m;
}

/* quarter_warp_sum (engine/src/kernels/moe.rs:37-42): butterfly xor 4, 2, 1 over eight lane partials, lane 0. */
static inline float orc_quarter_warp_sum(const float *a)
{
    float s04 = a[0] + a[4], s15 = a[1] + a[5], s26 = a[2] + a[6], s37 = a[3] + a[7];
    float e = s04 + s26, o = s15 + s37;
    return e + o;
}

/* ------------------------------------------------------------------------------------------------------------ */
/* router                                                                                                         */
/* ------------------------------------------------------------------------------------------------------------ */

/*
 * router_select_parallel (engine/src/kernels/moe.rs:177-287; the serial and warp variants :64-169, :376-537 give
 * the same result). probs = sqrt(softplus(logit)); selection score = prob + bias; insertion over experts in
 * ascending order with a strictly-greater compare so ties keep the lower index (:239-263); weights are the
 * un-biased probs of the selected experts, sum floored at 2^-14, then w /= (sum / 1.5) (:266-286). hash_mode
 * copies the selection from a token-indexed table (:211-228). k is 6 in the reference (model.rs:16); the oracle
 * accepts 1..8. n_expert is 256 in the reference.
 */
void orc_router_select(const float *logits, const float *bias, const int32_t *hash, const int32_t *tokens,
                       float *probs, int32_t *selected, float *weights, int32_t token_scalar, uint32_t hash_rows,
                       int64_t n_tokens, int has_bias, int hash_mode, int k, int n_expert)
{
    for (int64_t t = 0; t < n_tokens; ++t) {
        const float *lg = logits + t * n_expert;
        float *pr = probs + t * n_expert;
        int32_t *sel = selected + t * k;
        float *w = weights + t * k;
        for (int e = 0; e < n_expert; ++e) pr[e] = orc_router_score(lg[e]);
        if (hash_mode) {
            int32_t raw = tokens ? tokens[t] : token_scalar;
            int64_t tok = (raw < 0 || (uint32_t)raw >= hash_rows) ? 0 : raw;
            for (int j = 0; j < k; ++j) sel[j] = hash[tok * k + j];
        } else {
            for (int j = 0; j < k; ++j) sel[j] = -1;
            for (int e = 0; e < n_expert; ++e) {
                float score = pr[e] + (has_bias ? bias[e] : 0.0f);
                for (int j = 0; j < k; ++j) {
                    int32_t cur = sel[j];
                    float cur_score = (cur < 0) ? -INFINITY : pr[cur] + (has_bias ? bias[cur] : 0.0f);
                    if (score > cur_score) {
                        for (int m = k - 1; m > j; --m) sel[m] = sel[m - 1];
                        sel[j] = e;
                        break;
                    }
                }
            }
        }
        float sum = 0.0f;
        for (int j = 0; j < k; ++j) {
            int32_t e = sel[j];
            float v = (e >= 0 && e < n_expert) ? pr[e] : 0.0f;
            w[j] = v;
            sum += v;
        }
        if (sum < 6.103515625e-5f) sum = 6.103515625e-5f;
        float div = sum / 1.5f;
        for (int j = 0; j < k; ++j) w[j] = w[j] / div;
    }
}

/*
 * matmul_f16 (engine/src/kernels/matmul.rs:57-105) as used for the router logits (engine/src/session.rs:1995-2008):
 * 256 threads stride the row, each accumulating w*x sequentially, then a shared-memory halving tree.
 */
void orc_matmul_f16(const uint16_t *w, const float *x, float *out, int64_t in_dim, int64_t out_dim, int64_t n_tok)
{
#if defined(_OPENMP)
#pragma omp parallel for collapse(2) schedule(static)
#endif
    for (int64_t tok = 0; tok < n_tok; ++tok)
        for (int64_t row = 0; row < out_dim; ++row) {
            float partial[256];
            for (int tx = 0; tx < 256; ++tx) {
                float sum = 0.0f;
                for (int64_t i = tx; i < in_dim; i += 256) {
                    float p = orc_f16_to_f32(w[row * in_dim + i], 0) * x[tok * in_dim + i];
                    sum = sum + p;
                }
                partial[tx] = sum;
            }
            for (int stride = 128; stride > 0; stride >>= 1)
                for (int tx = 0; tx < stride; ++tx) partial[tx] += partial[tx + stride];
            out[tok * out_dim + row] = partial[0];
        }
}

/* ------------------------------------------------------------------------------------------------------------ */
/* expert projections                                                                                             */
/* ------------------------------------------------------------------------------------------------------------ */

static inline float orc_row_dot_iq2(const uint8_t *row, const uint8_t *xq, uint32_t blocks, int ieee)
{
    float a[8];
    for (uint32_t l = 0; l < 8; ++l) {
        float acc = 0.0f;
        for (uint32_t b = l; b < blocks; b += 8)
            acc += orc_dot_iq2xxs_q8k(row + (size_t)b * ORC_IQ2XXS_BYTES, xq + (size_t)b * ORC_Q8K_BYTES, ieee);
        a[l] = acc;
    }
    return orc_quarter_warp_sum(a);
}

static inline float orc_row_dot_q2k(const uint8_t *row, const uint8_t *xq, uint32_t blocks, int ieee)
{
    float a[8];
    for (uint32_t l = 0; l < 8; ++l) {
        float acc = 0.0f;
        for (uint32_t b = l; b < blocks; b += 8)
            acc += orc_dot_q2k_q8k(row + (size_t)b * ORC_Q2K_BYTES, xq + (size_t)b * ORC_Q8K_BYTES, ieee);
        a[l] = acc;
    }
    return orc_quarter_warp_sum(a);
}

/*
 * Plain matrix-vector products against Q8_K activations, one weight matrix, n_tok activation rows: the unit the
 * reference's CPU tests exercise one block at a time. out[tok][row]. Used for the single-matrix configurations.
 */
void orc_matvec_iq2xxs(const uint8_t *w, const uint8_t *xq, float *out, int64_t n_rows, uint32_t blocks,
                       int64_t n_tok, int ieee)
{
#if defined(_OPENMP)
#pragma omp parallel for collapse(2) schedule(static)
#endif
    for (int64_t t = 0; t < n_tok; ++t)
        for (int64_t r = 0; r < n_rows; ++r)
            out[t * n_rows + r] = orc_row_dot_iq2(w + (size_t)r * blocks * ORC_IQ2XXS_BYTES,
                                                  xq + (size_t)t * blocks * ORC_Q8K_BYTES, blocks, ieee);
}

void orc_matvec_q2k(const uint8_t *w, const uint8_t *xq, float *out, int64_t n_rows, uint32_t blocks, int64_t n_tok,
                    int ieee)
{
#if defined(_OPENMP)
#pragma omp parallel for collapse(2) schedule(static)
#endif
    for (int64_t t = 0; t < n_tok; ++t)
        for (int64_t r = 0; r < n_rows; ++r)
            out[t * n_rows + r] = orc_row_dot_q2k(w + (size_t)r * blocks * ORC_Q2K_BYTES,
                                                  xq + (size_t)t * blocks * ORC_Q8K_BYTES, blocks, ieee);
}

/*
 * moe_gate_up_mid_qwarp32 (engine/src/kernels/moe.rs:622-715). Per pair = tok*k + slot: expert = max(selected,0)
 * (:645-648); each row's gate and up are eight lane partials over blocks l, l+8, ... (:661-688) reduced by the
 * butterfly; clamp gate from above and up on both sides when clamp > 1e-6 (:692-702);
 * mid = ((gate / (1 + exp(-gate))) * up) * w (:703-710). gate_out / up_out may be NULL.
 */
void orc_gate_up_mid(const uint8_t *gate_base, const uint8_t *up_base, const uint8_t *xq, const int32_t *selected,
                     const float *weights, float *gate_out, float *up_out, float *mid_out,
                     uint64_t gate_expert_bytes, uint64_t gate_row_bytes, uint32_t xq_blocks, uint32_t expert_mid_dim,
                     uint32_t k, int64_t n_tokens, float clamp, int ieee)
{
    int64_t n_pairs = n_tokens * k;
#if defined(_OPENMP)
#pragma omp parallel for collapse(2) schedule(static)
#endif
    for (int64_t pair = 0; pair < n_pairs; ++pair)
        for (uint32_t row = 0; row < expert_mid_dim; ++row) {
            int64_t tok = pair / k;
            int32_t e = selected[pair];
            uint64_t ex = e < 0 ? 0u : (uint64_t)e;
            size_t off = (size_t)(ex * gate_expert_bytes + (uint64_t)row * gate_row_bytes);
            const uint8_t *x = xq + (size_t)tok * xq_blocks * ORC_Q8K_BYTES;
            float g = orc_row_dot_iq2(gate_base + off, x, xq_blocks, ieee);
            float u = orc_row_dot_iq2(up_base + off, x, xq_blocks, ieee);
            if (clamp > 1.0e-6f) {
                if (g > clamp) g = clamp;
                if (u > clamp) u = clamp;
                if (u < -clamp) u = -clamp;
            }
            size_t o = (size_t)pair * expert_mid_dim + row;
            if (gate_out) gate_out[o] = g;
            if (up_out) up_out[o] = u;
            float s = g / (1.0f + orc_expf(-g));
            s = s * u;
            mid_out[o] = s * weights[pair];
        }
}

/* moe_down_qwarp32 (engine/src/kernels/moe.rs:821-865): per pair, down_out[pair][row]. */
void orc_down(const uint8_t *down_base, const uint8_t *midq, const int32_t *selected, float *down_out,
              uint64_t down_expert_bytes, uint64_t down_row_bytes, uint32_t midq_blocks, uint32_t out_dim, uint32_t k,
              int64_t n_tokens, int ieee)
{
    int64_t n_pairs = n_tokens * k;
#if defined(_OPENMP)
#pragma omp parallel for collapse(2) schedule(static)
#endif
    for (int64_t pair = 0; pair < n_pairs; ++pair)
        for (uint32_t row = 0; row < out_dim; ++row) {
            int32_t e = selected[pair];
            uint64_t ex = e < 0 ? 0u : (uint64_t)e;
            const uint8_t *w = down_base + (size_t)(ex * down_expert_bytes + (uint64_t)row * down_row_bytes);
            down_out[(size_t)pair * out_dim + row] =
                orc_row_dot_q2k(w, midq + (size_t)pair * midq_blocks * ORC_Q8K_BYTES, midq_blocks, ieee);
        }
}

/*
 * moe_down_sum6_qwarp32 (engine/src/kernels/moe.rs:922-970), generalised from one token to n_tokens and from six
 * slots to k: out[tok][row] = sum over slots, in slot order, of the pair's row dot. moe_down_qwarp32 followed by
 * moe_sum (:983-1005) gives the same numbers.
 */
void orc_down_sum(const uint8_t *down_base, const uint8_t *midq, const int32_t *selected, float *out,
                  uint64_t down_expert_bytes, uint64_t down_row_bytes, uint32_t midq_blocks, uint32_t out_dim,
                  uint32_t k, int64_t n_tokens, int ieee)
{
#if defined(_OPENMP)
#pragma omp parallel for collapse(2) schedule(static)
#endif
    for (int64_t tok = 0; tok < n_tokens; ++tok)
        for (uint32_t row = 0; row < out_dim; ++row) {
            float total = 0.0f;
            for (uint32_t slot = 0; slot < k; ++slot) {
                int64_t pair = tok * k + slot;
                int32_t e = selected[pair];
                uint64_t ex = e < 0 ? 0u : (uint64_t)e;
                const uint8_t *w = down_base + (size_t)(ex * down_expert_bytes + (uint64_t)row * down_row_bytes);
                total += orc_row_dot_q2k(w, midq + (size_t)pair * midq_blocks * ORC_Q8K_BYTES, midq_blocks, ieee);
            }
            out[(size_t)tok * out_dim + row] = total;
        }
}

/* swiglu (engine/src/kernels/utils.rs:141-163), the shared-expert activation; pinned by kernels_smoke.rs:398-514. */
void orc_swiglu(const float *gate, const float *up, float *out, int64_t n, float clamp, float weight)
{
    for (int64_t i = 0; i < n; ++i) {
        float g = gate[i], u = up[i];
        if (clamp > 1.0e-6f) {
            if (g > clamp) g = clamp;
            if (u > clamp) u = clamp;
            if (u < -clamp) u = -clamp;
        }
        float s = g / (1.0f + orc_expf(-g));
        s = s * u;
        out[i] = s * weight;
    }
}

/*
 * The routed-expert step of Session::decode_attn_out_and_ffn (engine/src/session.rs:2010-2155) for n_tokens rows
 * of x (logits are [n_tokens][n_expert]): router_select -> q8k(x) -> gate/up/mid -> q8k(mid) -> down + slot sum. Router logits are an input (the
 * reference computes them with matmul_f16 just before, session.rs:1995-2008). Scratch is allocated here.
 * Returns 0, or -1 when memory runs out.
 */
int orc_moe_layer(const float *x, const float *logits, const uint8_t *gate_base, const uint8_t *up_base,
                  const uint8_t *down_base, float *out, int32_t *selected, float *weights, float *mid_opt,
                  int64_t n_tokens, uint32_t n_embd, uint32_t n_ff, int n_expert, int k, float clamp, int ieee)
{
    uint32_t xb = n_embd / ORC_QK_K, mb = n_ff / ORC_QK_K;
    uint64_t gate_row = (uint64_t)xb * ORC_IQ2XXS_BYTES, gate_exp = (uint64_t)n_ff * gate_row;
    uint64_t down_row = (uint64_t)mb * ORC_Q2K_BYTES, down_exp = (uint64_t)n_embd * down_row;
    int64_t n_pairs = n_tokens * k;
    float *probs = (float *)malloc((size_t)n_tokens * (size_t)n_expert * sizeof(float));
    uint8_t *xq = (uint8_t *)malloc((size_t)n_tokens * xb * ORC_Q8K_BYTES);
    float *mid = mid_opt ? mid_opt : (float *)malloc((size_t)n_pairs * n_ff * sizeof(float));
    uint8_t *midq = (uint8_t *)malloc((size_t)n_pairs * mb * ORC_Q8K_BYTES);
    int rc = -1;
    if (probs && xq && mid && midq) {
        orc_router_select(logits, NULL, NULL, NULL, probs, selected, weights, 0, 0, n_tokens, 0, 0, k, n_expert);
        orc_q8k_quantize(x, xq, n_embd, n_tokens);
        orc_gate_up_mid(gate_base, up_base, xq, selected, weights, NULL, NULL, mid, gate_exp, gate_row, xb, n_ff,
                        (uint32_t)k, n_tokens, clamp, ieee);
        orc_q8k_quantize(mid, midq, n_ff, n_pairs);
        orc_down_sum(down_base, midq, selected, out, down_exp, down_row, mb, n_embd, (uint32_t)k, n_tokens, ieee);
        rc = 0;
    }
    free(probs);
    free(xq);
    if (!mid_opt) free(mid);
    free(midq);
    return rc;
}

/* ------------------------------------------------------------------------------------------------------------ */
/* shared expert (Q8_0)                                                                                           */
/* ------------------------------------------------------------------------------------------------------------ */

/*
 * quantize_q8_0 (engine/src/kernels/quantize.rs:147-225): 32-element blocks, d = amax / 127, id = 1/d (0 when d is
 * 0), q = trunc(x*id +/- 0.5) clamped to int8. xq is [tok][blocks*32] int8, xscale [tok][blocks] f32.
 */
void orc_quantize_q8_0(const float *x, int8_t *xq, float *xscale, int64_t in_dim, int64_t n_tok)
{
    int64_t blocks = (in_dim + 31) / 32;
    for (int64_t t = 0; t < n_tok; ++t)
        for (int64_t b = 0; b < blocks; ++b) {
            int64_t i0 = b * 32;
            int bn = (in_dim - i0 < 32) ? (int)(in_dim - i0) : 32;
            float amax = 0.0f;
            for (int i = 0; i < bn; ++i) {
                float v = x[t * in_dim + i0 + i];
                float a = v < 0.0f ? -v : v;
                if (a > amax) amax = a;
            }
            float d = amax / 127.0f;
            float id = (d != 0.0f) ? 1.0f / d : 0.0f;
            xscale[t * blocks + b] = d;
            for (int i = 0; i < 32; ++i) {
                int8_t q = 0;
                if (i < bn) {
                    float raw = x[t * in_dim + i0 + i] * id;
                    int32_t r = raw >= 0.0f ? orc_f32_as_i32(raw + 0.5f) : orc_f32_as_i32(raw - 0.5f);
                    q = (int8_t)(r > 127 ? 127 : (r < -128 ? -128 : r));
                }
                xq[(t * blocks + b) * 32 + i] = q;
            }
        }
}

/*
 * matmul_q8_0_preq_warp8 (engine/src/kernels/matmul.rs:357-405; row dot mirrored in engine/tests/quant_cpu.rs:29-40):
 * one warp per output row, lane l takes blocks l, l+32, ..., each adding (scale_w * xscale[b]) * (float)dot, then a
 * 32-lane butterfly (xor 16, 8, 4, 2, 1).
 */
void orc_matmul_q8_0(const uint8_t *w, const int8_t *xq, const float *xscale, float *out, int64_t in_dim,
                     int64_t out_dim, int64_t n_tok)
{
    int64_t blocks = in_dim / 32;
#if defined(_OPENMP)
#pragma omp parallel for collapse(2) schedule(static)
#endif
    for (int64_t t = 0; t < n_tok; ++t)
        for (int64_t row = 0; row < out_dim; ++row) {
            float lane[32];
            for (int l = 0; l < 32; ++l) {
                float acc = 0.0f;
                for (int64_t b = l; b < blocks; b += 32) {
                    const uint8_t *blk = w + (size_t)(row * blocks + b) * 34;
                    float sw = orc_f16_to_f32(orc_rd_u16(blk), 0);
                    int32_t dot = 0;
                    for (int i = 0; i < 32; ++i) dot += (int32_t)(int8_t)blk[2 + i] * (int32_t)xq[(t * blocks + b) * 32 + i];
                    float s = sw * xscale[t * blocks + b];
                    acc += s * (float)dot;
                }
                lane[l] = acc;
            }
            for (int m = 16; m > 0; m >>= 1)
                for (int l = 0; l < 32; ++l)
                    if ((l & m) == 0) {
                        float s = lane[l] + lane[l | m];
                        lane[l] = s;
                        lane[l | m] = s;
                    }
            out[t * out_dim + row] = lane[0];
        }
}

/* ------------------------------------------------------------------------------------------------------------ */
/* FP8 E4M3 block-scaled projection (no reference implementation: parity unpinned)                                */
/* ------------------------------------------------------------------------------------------------------------ */

/* e4m3fn_value (engine/src/kernels/quantize.rs:10-18): positive value of code i in 0..126 */
float orc_e4m3_value(int i)
{
    int exp = (i >> 3) & 15, mant = i & 7;
    if (exp == 0) return (float)mant * 0.001953125f;
    return (1.0f + (float)mant * 0.125f) * ldexpf(1.0f, exp - 7);
}

/*
 * e4m3fn_dequant (engine/src/kernels/quantize.rs:24-53) returning the code byte instead of the value: nearest
 * representable magnitude, ties to the even code, saturating at 448 (code 126). Sign goes to bit 7.
 */
uint8_t orc_e4m3_encode(float x)
{
    int neg = x < 0.0f;
    float ax = neg ? -x : x;
    if (!(ax < 448.0f)) ax = 448.0f; /* also maps NaN to the clamp, as the reference's compare does */
    int lo = 0, hi = 126;
    while (lo < hi) {
        int mid = (lo + hi + 1) >> 1;
        if (orc_e4m3_value(mid) <= ax) lo = mid;
        else hi = mid - 1;
    }
    int best = lo;
    if (best < 126) {
        float bd = fabsf(ax - orc_e4m3_value(best));
        float nd = fabsf(ax - orc_e4m3_value(best + 1));
        if (nd < bd || (nd == bd && ((best + 1) & 1) == 0 && (best & 1) != 0)) best += 1;
    }
    return (uint8_t)(best | (neg ? 0x80 : 0));
}

float orc_e4m3_decode(uint8_t c)
{
    float v = orc_e4m3_value(c & 0x7F);
    return (c & 0x80) ? -v : v;
}

/*
 * Block-scaled E4M3 quantisation. Scale per (rows_per_block x 128) tile: s = max(amax, 1e-4) / 448 (the floor is
 * the one fp8_kv_quantize uses, engine/src/kernels/quantize.rs:109-112); codes = encode(x / s). Activations use
 * rows_per_block = 1, weights 128. scales is [ceil(rows/rpb)][cols/128].
 */
void orc_fp8_quantize(const float *x, uint8_t *codes, float *scales, int64_t rows, int64_t cols, int rows_per_block)
{
    int64_t cb = cols / 128, rb = (rows + rows_per_block - 1) / rows_per_block;
#if defined(_OPENMP)
#pragma omp parallel for collapse(2) schedule(static)
#endif
    for (int64_t br = 0; br < rb; ++br)
        for (int64_t bc = 0; bc < cb; ++bc) {
            int64_t r0 = br * rows_per_block, r1 = r0 + rows_per_block;
            if (r1 > rows) r1 = rows;
            float amax = 0.0f;
            for (int64_t r = r0; r < r1; ++r)
                for (int c = 0; c < 128; ++c) {
                    float a = fabsf(x[r * cols + bc * 128 + c]);
                    if (a > amax) amax = a;
                }
            if (amax < 1.0e-4f) amax = 1.0e-4f;
            float s = amax / 448.0f;
            scales[br * cb + bc] = s;
            for (int64_t r = r0; r < r1; ++r)
                for (int c = 0; c < 128; ++c)
                    codes[r * cols + bc * 128 + c] = orc_e4m3_encode(x[r * cols + bc * 128 + c] / s);
        }
}

/*
 * C[m][n] = sum over 128-wide K blocks of s_a[m][kb] * s_w[n/128][kb] * sum_k a*w, evaluated in double; the caller
 * rounds to bf16 when comparing. A is [M][K] codes, W is [N][K] codes.
 */
void orc_fp8_gemm(const uint8_t *a, const float *a_scale, const uint8_t *w, const float *w_scale, float *out,
                  int64_t M, int64_t N, int64_t K)
{
    int64_t kb_n = K / 128;
    float lut[256];
    for (int i = 0; i < 256; ++i) lut[i] = orc_e4m3_decode((uint8_t)i);
#if defined(_OPENMP)
#pragma omp parallel for collapse(2) schedule(static)
#endif
    for (int64_t m = 0; m < M; ++m)
        for (int64_t n = 0; n < N; ++n) {
            double acc = 0.0;
            for (int64_t kb = 0; kb < kb_n; ++kb) {
                double part = 0.0;
                const uint8_t *ar = a + m * K + kb * 128, *wr = w + n * K + kb * 128;
                for (int c = 0; c < 128; ++c) part += (double)lut[ar[c]] * (double)lut[wr[c]];
                acc += (double)a_scale[m * kb_n + kb] * (double)w_scale[(n / 128) * kb_n + kb] * part;
            }
            out[m * N + n] = (float)acc;
        }
}

/* ------------------------------------------------------------------------------------------------------------ */

/* hc_expand, engine/src/kernels/hc.rs:212-251: block_v = block_out (+ block_add); out = block_v * post[dst] +
 * sum over src of comb[dst + src * n_hc] * residual[src], with post at split[n_hc ..] and comb at split[2 n_hc ..] of the
 * token's row of mix_hc floats. Multiplications and additions are separate f32 operations, as in the Rust source. */
void orc_hc_expand(const float *block_out, const float *block_add, const float *residual_hc, const float *split,
                   float *out_hc, int64_t n_embd, int64_t n_hc, int64_t n_tokens, int64_t mix_hc, int has_add)
{
    for (int64_t t = 0; t < n_tokens; ++t)
        for (int64_t dst = 0; dst < n_hc; ++dst)
            for (int64_t d = 0; d < n_embd; ++d) {
                float block_v = block_out[t * n_embd + d];
                if (has_add) block_v += block_add[t * n_embd + d];
                const float *sp = split + t * mix_hc;
                float acc = block_v * sp[n_hc + dst];
                for (int64_t src = 0; src < n_hc; ++src) {
                    const float prod = sp[2 * n_hc + dst + src * n_hc] * residual_hc[(t * n_hc + src) * n_embd + d];
                    acc += prod;
                }
                out_hc[(t * n_hc + dst) * n_embd + d] = acc;
            }
}

/* hc4_split_one, engine/src/kernels/hc.rs:17-100 */
static void orc_hc4_split_one(float *out, const float *mix, const float *scale, const float *base, int iters, float epsv)
{
    const float pre_s = scale[0], post_s = scale[1], comb_s = scale[2];
    for (int i = 0; i < 4; ++i) {
        const float z = mix[i] * pre_s + base[i];
        out[i] = 1.0f / (1.0f + orc_expf(-z)) + epsv;
    }
    for (int i = 0; i < 4; ++i) {
        const float z = mix[4 + i] * post_s + base[4 + i];
        out[4 + i] = 2.0f / (1.0f + orc_expf(-z));
    }
    float c[16];
    for (int r = 0; r < 4; ++r) {
        float m = -INFINITY;
        for (int col = 0; col < 4; ++col) {
            const float v = mix[8 + r * 4 + col] * comb_s + base[8 + r * 4 + col];
            c[r * 4 + col] = v;
            if (v > m) m = v;
        }
        float s = 0.0f;
        for (int col = 0; col < 4; ++col) {
            const float v = orc_expf(c[r * 4 + col] - m);
            c[r * 4 + col] = v;
            s += v;
        }
        for (int col = 0; col < 4; ++col) c[r * 4 + col] = c[r * 4 + col] / s + epsv;
    }
    for (int col = 0; col < 4; ++col) {
        float s = epsv;
        for (int r = 0; r < 4; ++r) s += c[r * 4 + col];
        for (int r = 0; r < 4; ++r) c[r * 4 + col] /= s;
    }
    for (int it = 1; it < iters; ++it) {
        for (int r = 0; r < 4; ++r) {
            float s = epsv;
            for (int col = 0; col < 4; ++col) s += c[r * 4 + col];
            for (int col = 0; col < 4; ++col) c[r * 4 + col] /= s;
        }
        for (int col = 0; col < 4; ++col) {
            float s = epsv;
            for (int r = 0; r < 4; ++r) s += c[r * 4 + col];
            for (int r = 0; r < 4; ++r) c[r * 4 + col] /= s;
        }
    }
    for (int i = 0; i < 16; ++i) out[8 + i] = c[i];
}

/* hc_split_weighted_sum_norm_fused, engine/src/kernels/hc.rs:313-394: 256 "threads" per row, each summing the squares of
 * its columns d, d + 256, ..., then the halving tree over the 256 partial sums. */
void orc_hc_split_weighted_sum_norm(const float *mix, const float *scale, const float *base, const float *residual_hc,
                                    const float *norm_w, float *split, float *out, float *norm_out, int64_t n_embd,
                                    int64_t n_rows, int iters, float epsv, float norm_eps)
{
    for (int64_t t = 0; t < n_rows; ++t) {
        float *sp = split + t * 24;
        orc_hc4_split_one(sp, mix + t * 24, scale, base, iters, epsv);
        float partial[256];
        for (int d = 0; d < 256; ++d) {
            float sum_sq = 0.0f;
            for (int64_t col = d; col < n_embd; col += 256) {
                float acc = 0.0f;
                for (int h = 0; h < 4; ++h) {
                    const float prod = residual_hc[(t * 4 + h) * n_embd + col] * sp[h];
                    acc += prod;
                }
                out[t * n_embd + col] = acc;
                const float sq = acc * acc;
                sum_sq += sq;
            }
            partial[d] = sum_sq;
        }
        for (int stride = 128; stride > 0; stride >>= 1)
            for (int d = 0; d < stride; ++d) partial[d] += partial[d + stride];
        const float norm_scale = 1.0f / sqrtf(partial[0] / (float)n_embd + norm_eps);
        for (int64_t col = 0; col < n_embd; ++col) {
            const float v = out[t * n_embd + col] * norm_scale;
            norm_out[t * n_embd + col] = v * norm_w[col];
        }
    }
}

int orc_num_threads(void)
{
#if defined(_OPENMP)
    return omp_get_max_threads();
#else
    return 1;
#endif
}

void orc_set_num_threads(int n)
{
#if defined(_OPENMP)
    if (n > 0) omp_set_num_threads(n);
#else
    (void)n;
#endif
}

/* ------------------------------------------------------------------------------------------------------------ */
/*
 * Check of the division the CUDA SwiGLU uses in place of the library's (common.cuh, fdiv_rn_swiglu): for b in
 * [1, 2^60) and |a| in [2^-60, 2^60), reciprocal by two Newton steps from an approximation that is off by up to
 * three units in the last place (the hardware's is within one), then q + (a - b q) * y with an exact residual.
 * The engine divides with the host's IEEE division (engine/src/kernels/moe.rs:703-710). Returns the number of
 * operand pairs, out of n pseudo-random ones (one in four with a significand of b next to all ones or all zeros),
 * for which the two differ; pairs whose b has an all-ones significand are counted in *skipped instead, because
 * the CUDA code sends those to the library division.
 */
static inline float orc_u2f(uint32_t u) { float f; memcpy(&f, &u, 4); return f; }
static inline uint32_t orc_f2u(float f) { uint32_t u; memcpy(&u, &f, 4); return u; }

int64_t orc_check_div_rn(int64_t n, uint64_t seed, int64_t *skipped)
{
    int64_t bad = 0, skip = 0;
#if defined(_OPENMP)
#pragma omp parallel for reduction(+ : bad, skip) schedule(static)
#endif
    for (int64_t i = 0; i < n; ++i) {
        uint64_t x = seed + 0x9E3779B97F4A7C15ull * (uint64_t)(2 * i + 1), y;
        x ^= x >> 30, x *= 0xBF58476D1CE4E5B9ull, x ^= x >> 27, x *= 0x94D049BB133111EBull, x ^= x >> 31;
        y = x + 0x9E3779B97F4A7C15ull;
        y ^= y >> 30, y *= 0xBF58476D1CE4E5B9ull, y ^= y >> 27, y *= 0x94D049BB133111EBull, y ^= y >> 31;
        uint32_t mb = (uint32_t)(x & 0x7FFFFF);
        if ((i & 7) == 0) mb = 0x7FFFFF - (uint32_t)((x >> 40) & 3);
        if ((i & 7) == 1) mb = (uint32_t)((x >> 40) & 3);
        float b = orc_u2f(((127u + (uint32_t)((x >> 23) % 60)) << 23) | mb);
        uint32_t ma = (uint32_t)(y & 0x7FFFFF);
        if ((i & 15) == 2) ma = 0x7FFFFF - (uint32_t)((y >> 40) & 3);
        float a = orc_u2f(((uint32_t)((y >> 63) & 1) << 31) | ((67u + (uint32_t)((y >> 23) % 120)) << 23) | ma);
        float r = orc_u2f(orc_f2u(1.0f / b) + (uint32_t)((int)((y >> 50) % 7) - 3));
        float e = fmaf(-b, r, 1.0f);
        r = fmaf(r, e, r);
        e = fmaf(-b, r, 1.0f);
        r = fmaf(r, e, r);
        float q = a * r;
        float got = fmaf(fmaf(-b, q, a), r, q);
        if (orc_f2u(got) != orc_f2u(a / b)) {
            if (mb == 0x7FFFFF) ++skip;
            else ++bad;
        }
    }
    if (skipped) *skipped = skip;
    return bad;
}
