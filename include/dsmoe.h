/*
 * dsmoe — B200-native (sm_100a) kernels for the quantized routed-expert path of the deepseek-rs engine, behind a
 * plain C ABI.
 *
 * Every entry point replaces one kernel launch (tier 1) or one group of launches (tier 2) that the reference's Rust
 * host code makes through its generated `engine.kernels.<module>.<kernel>(&stream, LaunchConfig, args...)` methods
 * (engine/src/engine.rs:16-55). Operand meaning and order follow the reference kernel's parameter list; launch
 * geometry and lookup tables are internal. The reference file:line each one stands in for is cited on its
 * declaration.
 *
 * Conventions
 *   - All pointers are device pointers unless the name ends in `_host`. The library never frees caller memory.
 *   - All calls are asynchronous on the caller's stream (a cudaStream_t passed as void*; NULL = the legacy default
 *     stream) and perform no host synchronisation, except the `_host` calls and create/destroy.
 *   - Every function returns DSMOE_OK or a negative dsmoe_status; dsmoe_last_error() gives the text. Nothing aborts
 *     and nothing throws across the boundary.
 *   - Packed weight pointers must be 16-byte aligned for the ROWSOA layout and 2-byte (IQ2_XXS) / 4-byte (Q2_K)
 *     aligned for the NATIVE layout; Q8_K buffers must be 4-byte aligned.
 *   - A handle belongs to one device and one host thread at a time. Calls that take a handle must be made with the
 *     handle's device current (cudaSetDevice); otherwise they return DSMOE_ERR_STATE. dsmoe_create and dsmoe_destroy
 *     switch to the handle's device themselves and put the caller's current device back before they return.
 *   - The decode kernels index (token, slot) pairs with 16 bits: tier-1 gate/up/down calls and the tier-2 call below
 *     its batched threshold take at most 65535 pairs (n_tokens * n_expert_used) per call and return DSMOE_ERR_ARG /
 *     DSMOE_ERR_BOUNDS beyond that. The batched (grouped GEMM) path has no such limit.
 *
 * Block formats (little-endian): IQ2_XXS 66 B, Q2_K 84 B, Q8_K 292 B per 256 values
 * (engine/src/kernels/moe.rs:601-611).
 */
#ifndef DSMOE_H
#define DSMOE_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#if defined(_WIN32)
#define DSMOE_API
#else
#define DSMOE_API __attribute__((visibility("default")))
#endif

typedef struct dsmoe_handle dsmoe_handle;
typedef void *dsmoe_stream; /* cudaStream_t */

typedef enum dsmoe_status {
    DSMOE_OK = 0,
    DSMOE_ERR_ARG = -1,     /* bad pointer, size, alignment or enum */
    DSMOE_ERR_CUDA = -2,    /* a CUDA runtime call or launch failed */
    DSMOE_ERR_NCCL = -3,    /* an NCCL call failed, or libnccl.so.2 could not be loaded (expert-parallel calls) */
    DSMOE_ERR_TIMEOUT = -4, /* a bounded device-side wait expired */
    DSMOE_ERR_BOUNDS = -5,  /* a size exceeds what the handle was created for */
    DSMOE_ERR_NOMEM = -6,
    DSMOE_ERR_STATE = -7    /* e.g. layer not registered */
} dsmoe_status;

/*
 * Byte order of packed expert rows in device memory. A row keeps its byte count and stride in both layouts, so the
 * expert/row byte strides the reference passes (engine/src/session.rs:2079-2080, 2130-2131) stay valid.
 *   NATIVE: the GGUF order the reference uploads verbatim (engine/src/engine.rs:81-89): block after block.
 *   ROWSOA: a per-row permutation made once at upload by dsmoe_relayout_*: for IQ2_XXS
 *           [d x blocks][qs(64 B) x blocks]; for Q2_K [scales(16 B) x blocks][qs(64 B) x blocks][d,dmin x blocks].
 *           It makes every 16-byte load aligned. Dequantised values are unchanged.
 */
typedef enum dsmoe_layout { DSMOE_LAYOUT_NATIVE = 0, DSMOE_LAYOUT_ROWSOA = 1 } dsmoe_layout;

typedef struct dsmoe_config {
    uint32_t n_embd;        /* hidden size, multiple of 256 (reference: 4096, engine/src/model.rs:4) */
    uint32_t n_ff;          /* expert width, multiple of 256 (2048, model.rs:18) */
    uint32_t n_expert;      /* routed experts, multiple of 32, <= 512 (256, model.rs:15) */
    uint32_t n_expert_used; /* top-k, 1..8 (6, model.rs:16) */
    float swiglu_clamp;     /* 10.0 (engine/src/session.rs:21); <= 1e-6 disables clamping */
    float route_scale;      /* selected weights are renormalised to this sum (1.5, moe.rs:279-285) */
    uint32_t f16_ieee;      /* 0: f16 subnormal scales flush to zero as the reference device code does
                               (engine/src/kernels/utils.rs:16-29); 1: IEEE conversion */
    uint32_t max_tokens;    /* largest n_tokens the tier-2 calls will see; sizes library-owned scratch */
    uint32_t max_layers;    /* layer slots for dsmoe_layer_register */
} dsmoe_config;

DSMOE_API const char *dsmoe_version(void);
DSMOE_API void dsmoe_default_config(dsmoe_config *cfg);

/* Replaces Kernels::load (engine/src/engine.rs:31-54): the kernels are prebuilt sm_100a code inside this library,
 * so nothing is JIT-compiled. Fails with DSMOE_ERR_CUDA when the device is not compute capability 10.x. */
DSMOE_API int dsmoe_create(const dsmoe_config *cfg, int device, dsmoe_handle **out);
DSMOE_API int dsmoe_destroy(dsmoe_handle *h);
DSMOE_API const char *dsmoe_last_error(const dsmoe_handle *h);
/* Waits for the stream and reads the handle's device status word. Kernels that wait on asynchronous copies bound the
 * wait; if one ever expires the kernel records a code and returns instead of hanging. Returns DSMOE_OK with
 * *code_out == 0, or DSMOE_ERR_TIMEOUT with the code. The reference has no device-side error reporting
 * (launch errors only, engine/src/session.rs `?` propagation). */
DSMOE_API int dsmoe_device_status(dsmoe_handle *h, dsmoe_stream stream, int *code_out);
/* Measurement aid with no counterpart in the reference: when six cudaEvent_t are set, the batched (grouped-GEMM) path
 * of dsmoe_moe_forward records them on the stream at: start, pairs grouped + activations gathered, gate/up GEMM done,
 * Q8_K(mid) + gather done, down GEMM done, slot sum done. Pass NULL / 0 to clear. */
DSMOE_API int dsmoe_set_phase_events(dsmoe_handle *h, void **events, int n_events);
/* Number of kernels this handle has launched since creation (bookkeeping for benchmarks). */
DSMOE_API uint64_t dsmoe_launch_count(const dsmoe_handle *h);

/* Test hooks for the bounded-wait error path; no counterpart in the reference (which has no device-side waits).
 * Synchronises the device, then writes one word of the handle's device status block:
 *   DSMOE_DEBUG_WAIT_LIMIT_KCLOCKS  value = limit of every device-side wait in units of 1024 SM clocks (0 = default,
 *                                   about two seconds)
 *   DSMOE_DEBUG_DROP_ONE_COPY       value != 0: the TMA-staged down kernel leaves one of its bulk copies out, so the
 *                                   wait for it runs out; the kernel records the code and returns, nothing hangs
 *   DSMOE_DEBUG_CLEAR_STATUS        clears a recorded error code
 * A test sets a short limit and the drop flag, runs dsmoe_down_sum, and expects dsmoe_device_status to return
 * DSMOE_ERR_TIMEOUT. Production code never calls this. */
enum { DSMOE_DEBUG_WAIT_LIMIT_KCLOCKS = 1, DSMOE_DEBUG_DROP_ONE_COPY = 2, DSMOE_DEBUG_CLEAR_STATUS = 3 };
DSMOE_API int dsmoe_debug_set(dsmoe_handle *h, int what, int value);

/* ------------------------------------------------------------------------------------------------------------ */
/* Tier 1: kernel-for-kernel                                                                                      */
/* ------------------------------------------------------------------------------------------------------------ */

/* q8k_quantize (engine/src/kernels/quantize.rs:309-417; calls engine/src/session.rs:2062-2073, 2115-2126).
 * x: f32 [n_rows][in_dim]; out: Q8_K blocks [n_rows][in_dim/256][292]. Bit-exact. */
DSMOE_API int dsmoe_q8k_quantize(dsmoe_handle *h, dsmoe_stream stream, const float *x, uint8_t *out, uint32_t in_dim,
                                 uint32_t n_rows);

/* router_select_parallel (engine/src/kernels/moe.rs:177-287; call engine/src/session.rs:2038-2057); the serial and
 * warp variants (:64-169, :376-537) compute the same thing. bias, hash, tokens may be NULL. k and the expert count
 * come from the handle's config. logits, probs: f32 [n_tokens][n_expert]; selected: i32 [n_tokens][k];
 * weights: f32 [n_tokens][k]. */
DSMOE_API int dsmoe_router_select(dsmoe_handle *h, dsmoe_stream stream, const float *logits, const float *bias,
                                  const int32_t *hash, const int32_t *tokens, float *probs, int32_t *selected,
                                  float *weights, int32_t token_scalar, uint32_t hash_rows, uint32_t n_tokens,
                                  uint32_t has_bias, uint32_t hash_mode);

/* moe_gate_up_mid_qwarp32 (engine/src/kernels/moe.rs:622-715; call engine/src/session.rs:2088-2111).
 * xq: Q8_K [n_tokens][xq_blocks]; outputs f32 [n_tokens*k][expert_mid_dim]; gate_out / up_out may be NULL (the
 * reference never reads them back). */
DSMOE_API int dsmoe_gate_up_mid(dsmoe_handle *h, dsmoe_stream stream, const uint8_t *gate_base, const uint8_t *up_base,
                                const uint8_t *xq, const int32_t *selected, const float *weights, float *gate_out,
                                float *up_out, float *mid_out, uint64_t gate_expert_bytes, uint64_t gate_row_bytes,
                                uint32_t xq_blocks, uint32_t expert_mid_dim, uint32_t n_expert_used, uint32_t n_tokens,
                                float clamp, int layout);

/* moe_down_qwarp32 (engine/src/kernels/moe.rs:821-865). midq: Q8_K [n_tokens*k][midq_blocks];
 * down_out: f32 [n_tokens*k][out_dim]. */
DSMOE_API int dsmoe_down(dsmoe_handle *h, dsmoe_stream stream, const uint8_t *down_base, const uint8_t *midq,
                         const int32_t *selected, float *down_out, uint64_t down_expert_bytes, uint64_t down_row_bytes,
                         uint32_t midq_blocks, uint32_t out_dim, uint32_t n_expert_used, uint32_t n_tokens, int layout);

/* moe_down_sum6_qwarp32 (engine/src/kernels/moe.rs:922-970; call engine/src/session.rs:2138-2153), generalised to
 * n_tokens rows and k slots: out f32 [n_tokens][out_dim] = slots summed in slot order. */
DSMOE_API int dsmoe_down_sum(dsmoe_handle *h, dsmoe_stream stream, const uint8_t *down_base, const uint8_t *midq,
                             const int32_t *selected, float *out, uint64_t down_expert_bytes, uint64_t down_row_bytes,
                             uint32_t midq_blocks, uint32_t out_dim, uint32_t n_expert_used, uint32_t n_tokens,
                             int layout);

/* moe_sum (engine/src/kernels/moe.rs:983-1005). down: f32 [n_tokens*n_expert_used][out_dim]. */
DSMOE_API int dsmoe_moe_sum(dsmoe_handle *h, dsmoe_stream stream, const float *down, float *out, uint32_t out_dim,
                            uint32_t n_expert_used, uint32_t n_tokens);

/* The same sum (engine/src/kernels/moe.rs:983-1005: 0 + r_0 + r_1 + ... in slot order) over rows that are not stored
 * in pair order: slot e of token t is rows[pos[t*n_expert_used + e]]. No counterpart in the reference, which is
 * single-GPU; the expert-parallel combine uses it to sum the rows in the order they came back from their owners.
 * pos entries must lie in [0, number of rows). */
DSMOE_API int dsmoe_moe_sum_indexed(dsmoe_handle *h, dsmoe_stream stream, const float *rows, const int32_t *pos,
                                    float *out, uint32_t out_dim, uint32_t n_expert_used, uint32_t n_tokens);

/* ---- the steps beside the routed experts: router logits and the shared expert (engine/src/session.rs:1894-2008) ---- */

/* quantize_q8_0 (engine/src/kernels/quantize.rs:147-225; calls engine/src/session.rs:1896-1908, 1960-1972).
 * x: f32 [n_tokens][in_dim] -> xq: int8 [n_tokens][ceil(in_dim/32)*32], xscale: f32 [n_tokens][ceil(in_dim/32)]. */
DSMOE_API int dsmoe_quantize_q8_0(dsmoe_handle *h, dsmoe_stream stream, const float *x, int8_t *xq, float *xscale,
                                  uint64_t in_dim, uint64_t n_tokens);

/* matmul_q8_0_preq_warp8 / matmul_q8_0_preq_batch_warp8 (engine/src/kernels/matmul.rs:357-405 and the batched twin
 * after it; calls engine/src/session.rs:1915-1944, 1973-1984). w: Q8_0 blocks [out_dim][ceil(in_dim/32)][34 bytes],
 * 4-byte aligned; xq 16-byte aligned. out: f32 [n_tokens][out_dim]. */
DSMOE_API int dsmoe_matmul_q8_0(dsmoe_handle *h, dsmoe_stream stream, const uint8_t *w, const int8_t *xq,
                                const float *xscale, float *out, uint64_t in_dim, uint64_t out_dim, uint64_t n_tokens);

/* swiglu (engine/src/kernels/utils.rs:141-163; call engine/src/session.rs:1945-1953). */
DSMOE_API int dsmoe_swiglu(dsmoe_handle *h, dsmoe_stream stream, const float *gate, const float *up, float *out,
                           uint64_t n, float clamp, float weight);

/* matmul_f16 (engine/src/kernels/matmul.rs:57-105; the router-logits call engine/src/session.rs:1995-2008).
 * w: f16 bit patterns [out_dim][in_dim]; x: f32 [n_tokens][in_dim]; out: f32 [n_tokens][out_dim]. */
DSMOE_API int dsmoe_matmul_f16(dsmoe_handle *h, dsmoe_stream stream, const uint16_t *w, const float *x, float *out,
                               uint64_t in_dim, uint64_t out_dim, uint64_t n_tokens);

/* The whole shared expert of engine/src/session.rs:1894-1986 for n_tokens rows (any count; scratch is library-owned):
 * Q8_0 of x -> gate, up -> swiglu(clamp from the config, weight 1) -> Q8_0 -> down. out: f32 [n_tokens][n_embd]. */
DSMOE_API int dsmoe_shared_expert(dsmoe_handle *h, dsmoe_stream stream, const uint8_t *gate_w, const uint8_t *up_w,
                                  const uint8_t *down_w, const float *x, uint32_t n_tokens, float *out);

/* Dequantised weights. The reference has no such kernel; the values are defined by its block dots
 * (engine/src/kernels/quantize.rs:811, :900): IQ2_XXS w = (0.125*d) * (ls * +/-g); Q2_K w = d*(sc*q) - dmin*m.
 * blocks are in NATIVE order; out: f32 [n_blocks][256]. Bit-exact against the CPU oracle. */
DSMOE_API int dsmoe_dequant_iq2xxs(dsmoe_handle *h, dsmoe_stream stream, const uint8_t *blocks, uint64_t n_blocks,
                                   float *out);
DSMOE_API int dsmoe_dequant_q2k(dsmoe_handle *h, dsmoe_stream stream, const uint8_t *blocks, uint64_t n_blocks,
                                float *out);

/* Upload-time row permutation NATIVE -> ROWSOA (replaces the verbatim upload of engine/src/engine.rs:81-89).
 * src and dst must not overlap. inverse != 0 converts back. */
DSMOE_API int dsmoe_relayout_iq2xxs(dsmoe_handle *h, dsmoe_stream stream, const uint8_t *src, uint8_t *dst,
                                    uint64_t n_rows, uint32_t blocks_per_row, int inverse);
DSMOE_API int dsmoe_relayout_q2k(dsmoe_handle *h, dsmoe_stream stream, const uint8_t *src, uint8_t *dst,
                                 uint64_t n_rows, uint32_t blocks_per_row, int inverse);

/* ------------------------------------------------------------------------------------------------------------ */
/* FP8 E4M3 block-scaled dense projection                                                                         */
/* ------------------------------------------------------------------------------------------------------------ */

/* No FP8 GEMM exists in the reference: its dense projections are Q8_0 x Q8_0 matvecs
 * (engine/src/kernels/matmul.rs:357-603) and E4M3 is only used to round KV rows (engine/src/kernels/quantize.rs:10-134,
 * whose rounding rule these codes follow: nearest, ties to the even code, saturating at 448). These two calls stand
 * where quantize_q8_0 + matmul_q8_0_preq_warp8 stand for a projection (engine/src/session.rs:1329-1437).
 *
 * dsmoe_fp8_quantize: x f32 [rows][cols] -> codes u8 [rows][cols], scales f32 [ceil(rows/rpb)][cols/128] with
 * scale = max(amax, 1e-4) / 448 per rpb x 128 block; rows_per_block = 1 for activations, 128 for weights.
 * dsmoe_fp8_linear: out bf16 [M][N] = sum over 128-wide K blocks of a_scale[m][kb] * w_scale[n/128][kb] * (a . w),
 * a: [M][K] codes, w: [N][K] codes; N and K multiples of 128. */
DSMOE_API int dsmoe_fp8_quantize(dsmoe_handle *h, dsmoe_stream stream, const float *x, uint8_t *codes, float *scales,
                                 uint32_t rows, uint32_t cols, int rows_per_block);
DSMOE_API int dsmoe_fp8_linear(dsmoe_handle *h, dsmoe_stream stream, const uint8_t *a_fp8, const float *a_scale,
                               const uint8_t *w_fp8, const float *w_scale, void *out_bf16, uint32_t M, uint32_t N,
                               uint32_t K);

/* ------------------------------------------------------------------------------------------------------------ */
/* Tier 2: the routed-expert step as one call                                                                     */
/* ------------------------------------------------------------------------------------------------------------ */

/* Registers one layer's expert tensors (blk.{il}.ffn_{gate,up,down}_exps.weight, engine/src/engine.rs:180-182),
 * already in device memory in the given layout. The pointers are borrowed for the handle's lifetime. */
DSMOE_API int dsmoe_layer_register(dsmoe_handle *h, uint32_t layer, const uint8_t *gate, const uint8_t *up,
                                   const uint8_t *down, int layout);

/* Steps 2-6 of the routed-expert block of Session::decode_attn_out_and_ffn (engine/src/session.rs:2010-2155) for
 * n_tokens rows: router_select -> q8k(x) -> gate/up/SwiGLU -> q8k(mid) -> down + slot sum.
 * x: f32 [n_tokens][n_embd]; logits: f32 [n_tokens][n_expert]; out: f32 [n_tokens][n_embd];
 * selected_out / weights_out: optional [n_tokens][k]. Scratch is library-owned, sized by max_tokens. */
DSMOE_API int dsmoe_moe_forward(dsmoe_handle *h, dsmoe_stream stream, uint32_t layer, const float *x,
                                const float *logits, uint32_t n_tokens, float *out, int32_t *selected_out,
                                float *weights_out);

/* The part of dsmoe_moe_forward after the router and the Q8_K of x (engine/src/session.rs:2075-2155): gate/up/SwiGLU,
 * Q8_K(mid), down, slot sum, for rows that are already routed and quantised. xq: Q8_K [n_tokens][n_embd/256];
 * selected / weights: [n_tokens][k] with k from the handle's config. This is what an expert-parallel rank runs on the
 * rows it received (with a handle created for n_expert_used = 1 and expert ids local to its shard). */
DSMOE_API int dsmoe_expert_ffn(dsmoe_handle *h, dsmoe_stream stream, uint32_t layer, const uint8_t *xq,
                               const int32_t *selected, const float *weights, uint32_t n_tokens, float *out);

/* The tensors beside the routed experts of one layer, all optional (NULL / 0), borrowed like the expert tensors:
 *   router_f16    blk.{il}.ffn_gate_inp.weight, f16 bit patterns [n_expert][n_embd] (engine/src/engine.rs:178); with it
 *                 dsmoe_ffn_forward computes the logits itself (matmul_f16, engine/src/session.rs:1995-2008)
 *   router_bias   f32 [n_expert], added to the selection score only (engine/src/kernels/moe.rs:229-262); the reference
 *                 binds none for this model (engine/src/engine.rs:179)
 *   hash_table    blk.{il}.ffn_gate_tid2eid, i32 [hash_rows][n_expert_used] (engine/src/engine.rs:177); layers below
 *                 N_HASH_LAYER = 3 carry one (engine/src/model.rs:19)
 *   shared_*      blk.{il}.ffn_{gate,up,down}_shexp.weight, Q8_0 blocks (engine/src/session.rs:1894-1987) */
DSMOE_API int dsmoe_layer_register_extras(dsmoe_handle *h, uint32_t layer, const uint16_t *router_f16,
                                          const float *router_bias, const int32_t *hash_table, uint32_t hash_rows,
                                          const uint8_t *shared_gate, const uint8_t *shared_up,
                                          const uint8_t *shared_down);

enum { DSMOE_DTYPE_F32 = 0, DSMOE_DTYPE_BF16 = 1 };

/* Operands of dsmoe_ffn_forward. Unused optional pointers are NULL. */
typedef struct dsmoe_ffn_args {
    const void *x;             /* hidden states (ffn_norm) [n_tokens][n_embd]: f32 as the reference keeps them, or bf16,
                                  which is widened exactly before the same Q8_K / Q8_0 steps */
    int32_t x_dtype;           /* DSMOE_DTYPE_F32 or DSMOE_DTYPE_BF16 */
    uint32_t n_tokens;
    const float *logits;       /* optional [n_tokens][n_expert]; NULL: computed from the registered router matrix */
    const int32_t *tokens;     /* optional token ids [n_tokens] for hash routing (NULL: token_scalar for every row) */
    int32_t token_scalar;
    uint32_t hash_mode;        /* 0: score routing (what the reference's live call passes, engine/src/session.rs:2056);
                                  1: selected = hash_table[token] (engine/src/kernels/moe.rs:211-228) */
    float *routed_out;         /* required: slot sum of the routed experts [n_tokens][n_embd] (Session::routed_out) */
    float *shared_out;         /* optional: shared-expert output [n_tokens][n_embd] (Session::shared_out) */
    /* optional hyper-connection merge, hc_expand (engine/src/kernels/hc.rs:212-251, call engine/src/session.rs:2162-2175):
     * out_hc[t][dst][d] = (shared + routed)[t][d] * post[dst] + sum_src comb[dst + src * n_hc] * residual_hc[t][src][d],
     * post / comb at offsets n_hc / 2 n_hc of the token's hc_split row. Needs a registered shared expert. */
    const float *residual_hc;  /* [n_tokens][n_hc][n_embd] (Session::after_attn_hc) */
    const float *hc_split;     /* [n_tokens][mix_hc] */
    float *out_hc;             /* [n_tokens][n_hc][n_embd] (Session::after_ffn_hc) */
    uint32_t n_hc, mix_hc;
    int32_t *selected_out;     /* optional [n_tokens][n_expert_used] */
    float *weights_out;        /* optional [n_tokens][n_expert_used] */
} dsmoe_ffn_args;

/* Steps g, h and i of Session::decode_attn_out_and_ffn (engine/src/session.rs:1894-2180) for n_tokens rows in one call:
 * shared expert (on an internal side stream, concurrently with the routed path), router logits, router_select (score,
 * bias or hash mode), Q8_K, routed experts, slot sum and, when out_hc is set, the hyper-connection merge fused into the
 * slot sum (batched path) or run right after it. On return the caller's stream has been made to wait for the side
 * stream, so every output is ordered on `stream` like the other calls. */
DSMOE_API int dsmoe_ffn_forward(dsmoe_handle *h, dsmoe_stream stream, uint32_t layer, const dsmoe_ffn_args *args);

/* hc_expand on its own (engine/src/kernels/hc.rs:212-251): block_out / block_add f32 [n_tokens][n_embd] (block_add is
 * read when has_add != 0), residual_hc [n_tokens][n_hc][n_embd], split [n_tokens][mix_hc], out_hc like residual_hc. */
DSMOE_API int dsmoe_hc_expand(dsmoe_handle *h, dsmoe_stream stream, const float *block_out, const float *block_add,
                              const float *residual_hc, const float *split, float *out_hc, uint32_t n_embd,
                              uint32_t n_hc, uint32_t n_tokens, uint32_t mix_hc, uint32_t has_add);

/* hc_split_weighted_sum_norm_fused (engine/src/kernels/hc.rs:313-394 with hc4_split_one, :17-100; call
 * engine/src/session.rs:1865-1892): the producer of ffn_norm, the input of this path. Per row: the 24-value split
 * (pre = sigmoid + epsv, post = 2 sigmoid, comb = row softmax + epsv then sinkhorn_iters rounds of Sinkhorn
 * normalisation), out = sum over the 4 residual streams weighted by pre, norm_out = out * rsqrt(mean(out^2) + norm_eps)
 * * norm_w. mix [n_rows][24], scale [3], base [24], residual_hc [n_rows][4][n_embd], norm_w [n_embd]; split
 * [n_rows][24] is the hc_split buffer dsmoe_ffn_forward and dsmoe_hc_expand read (mix_hc = 24). n_hc must be 4. */
DSMOE_API int dsmoe_hc_split_weighted_sum_norm(dsmoe_handle *h, dsmoe_stream stream, const float *mix,
                                               const float *scale, const float *base, const float *residual_hc,
                                               const float *norm_w, float *split, float *out, float *norm_out,
                                               uint32_t n_embd, uint32_t n_hc, uint32_t n_rows,
                                               uint32_t sinkhorn_iters, float epsv, float norm_eps);

/* Same with host buffers: copies x and logits in, runs dsmoe_moe_forward on an internal stream, copies out (and the
 * optional routing) back and waits. Host buffers should be page-locked for full copy speed. */
DSMOE_API int dsmoe_moe_forward_host(dsmoe_handle *h, uint32_t layer, const float *x_host, const float *logits_host,
                                     uint32_t n_tokens, float *out_host, int32_t *selected_out_host,
                                     float *weights_out_host);

/* The same without the final wait: the copies and kernels are queued on the handle's internal stream and the call
 * returns; dsmoe_host_synchronize waits for everything queued on that stream. The host buffers must be page-locked and
 * stay untouched until then, and a handle takes one such call at a time (its staging buffers are per handle). Two
 * handles used in turn overlap one chunk's copies with the other's kernels. No counterpart in the reference, which
 * keeps its activations on the device. */
DSMOE_API int dsmoe_moe_forward_host_async(dsmoe_handle *h, uint32_t layer, const float *x_host,
                                           const float *logits_host, uint32_t n_tokens, float *out_host,
                                           int32_t *selected_out_host, float *weights_out_host);
DSMOE_API int dsmoe_host_synchronize(dsmoe_handle *h);

/* ------------------------------------------------------------------------------------------------------------ */
/* Expert parallel: experts sharded over the GPUs of one box, NCCL dispatch and combine                           */
/* ------------------------------------------------------------------------------------------------------------ */

/* No counterpart in the reference, which is single-GPU (one context, one stream: engine/src/engine.rs:73-74); defined by
 * "same result as one GPU". Rank r of `world` owns experts [r * n_expert / world, (r + 1) * n_expert / world) and routes
 * its own tokens with the same router kernel as dsmoe_moe_forward, so routing is bit-identical.
 *
 * Set-up: the handle is created with the MODEL's n_expert / n_expert_used and max_tokens = the most tokens this rank
 * routes per call. Rank 0 calls dsmoe_ep_get_unique_id and hands the 128 bytes to every rank over any host channel;
 * every rank then calls dsmoe_ep_init (it creates the NCCL communicator: collective, all ranks must call it), or
 * dsmoe_ep_init_comm with an ncclComm_t it already has. NCCL is looked up with dlsym in the libnccl.so.2 the process
 * has loaded, so no second NCCL is linked beside the host's. max_replicas: room for that many replicated experts
 * (n_expert / world + max_replicas must be a multiple of 32); recv_capacity_rows: rows this rank can receive per call
 * (0 = twice the pairs it routes itself). dsmoe_ep_layer_register takes the rank's shard in the order
 * [own experts | replicas in dsmoe_ep_set_replicas order], (n_expert / world + max_replicas) experts long.
 *
 * dsmoe_moe_forward_ep is collective: every rank calls it, in the same order, also with n_tokens == 0. It makes ONE host
 * synchronisation per call (it reads the world x world count matrix that sizes the transfers). Every rank sees the whole
 * matrix, so if any rank's receive buffer would overflow, every rank returns DSMOE_ERR_BOUNDS before any data moves and
 * none is left waiting. Operands as in dsmoe_moe_forward. */
#define DSMOE_EP_UNIQUE_ID_BYTES 128
DSMOE_API int dsmoe_ep_get_unique_id(uint8_t *id128);
DSMOE_API int dsmoe_ep_init(dsmoe_handle *h, const uint8_t *id128, int rank, int world, uint32_t max_replicas,
                            uint32_t recv_capacity_rows);
DSMOE_API int dsmoe_ep_init_comm(dsmoe_handle *h, void *nccl_comm, int rank, int world, uint32_t max_replicas,
                                 uint32_t recv_capacity_rows);
DSMOE_API int dsmoe_ep_layer_register(dsmoe_handle *h, uint32_t layer, const uint8_t *gate, const uint8_t *up,
                                      const uint8_t *down, int layout);
/* Experts every rank holds a copy of: their pairs are computed on the rank that routed them and never dispatched, which
 * takes the load of a few very popular experts off their owners. Results do not change. Synchronises the device. */
DSMOE_API int dsmoe_ep_set_replicas(dsmoe_handle *h, const int32_t *expert_ids, uint32_t n);
/* Running count of selections per expert over this rank's dsmoe_moe_forward_ep calls (uint64 [n_expert], copied to the
 * host; reset != 0 clears it): what a server picks its replicas from. Synchronises the stream. */
DSMOE_API int dsmoe_ep_expert_counts(dsmoe_handle *h, dsmoe_stream stream, uint64_t *counts_host, int reset);
/* Rows this rank received from each rank in its most recent dsmoe_moe_forward_ep (int32 [world]). */
DSMOE_API int dsmoe_ep_last_recv_rows(dsmoe_handle *h, int32_t *rows_per_rank);
/* 1 when dispatch and combine go over peer-mapped memory: at dsmoe_ep_init every rank maps the others' receive and
 * return buffers (CUDA IPC). Dispatch is then the row-gather kernel itself, storing each pair's Q8_K row, local expert
 * id and router weight where its owner reads them; combine is the owner's down-projection epilogue, storing each
 * finished row straight into its source rank's buffer. Both are plain global stores over NVLink (no loads from peer
 * memory, no TMA, no multicast), each followed by a four-byte all-gather as the completion signal. 0: rows travel both
 * ways by grouped ncclSend / ncclRecv (DSMOE_EP_NO_P2P=1 in the environment at dsmoe_ep_init, or an IPC mapping failed
 * on some rank - the ranks agree on the mode). Results are identical. */
DSMOE_API int dsmoe_ep_combine_is_fused(dsmoe_handle *h);
/* Measurement aid: six cudaEvent_t recorded at start, plan done, dispatch done, owner compute done, combine done, slot
 * sum done. NULL / 0 clears. */
DSMOE_API int dsmoe_ep_set_phase_events(dsmoe_handle *h, void **events, int n_events);
DSMOE_API int dsmoe_moe_forward_ep(dsmoe_handle *h, dsmoe_stream stream, uint32_t layer, const float *x,
                                   const float *logits, uint32_t n_tokens, float *out, int32_t *selected_out,
                                   float *weights_out);

/* ------------------------------------------------------------------------------------------------------------ */
/* GGUF expert-tensor ingestion                                                                                   */
/* ------------------------------------------------------------------------------------------------------------ */

/* Replaces GgufFile (engine/src/gguf.rs:23-122) and the verbatim tensor upload of Engine::open
 * (engine/src/engine.rs:77-90, names bound at :176-185) for the tensors of this path. Host-side calls; they need no
 * handle and, except dsmoe_gguf_upload_experts, no GPU. Tensor type ids as in engine/src/model.rs:29-39. */
enum { DSMOE_GGUF_F32 = 0, DSMOE_GGUF_F16 = 1, DSMOE_GGUF_Q8_0 = 8, DSMOE_GGUF_Q2_K = 10, DSMOE_GGUF_Q4_K = 12,
       DSMOE_GGUF_IQ2_XXS = 16, DSMOE_GGUF_I32 = 26 };

typedef struct dsmoe_gguf dsmoe_gguf;
typedef struct dsmoe_gguf_tensor {
    const char *name;       /* owned by the dsmoe_gguf object */
    uint32_t type, n_dims;  /* type id as stored in the file */
    uint64_t dims[4];       /* fastest-varying dimension first, as GGUF stores them; unused entries are 1 */
    uint64_t offset;        /* from the start of the data section */
    uint64_t bytes;         /* ceil(elements / block elements) * block bytes (engine/src/model.rs:41-75) */
    const void *host_data;  /* the tensor's bytes inside the mapping */
} dsmoe_gguf_tensor;

/* Maps the file read-only and parses header, metadata (skipped) and tensor table; the data section starts at the next
 * 32-byte boundary (engine/src/gguf.rs:101-102). *out is set even when parsing fails, so that dsmoe_gguf_last_error
 * can be read; close it in either case. DSMOE_ERR_ARG: bad magic, version outside 2..3, unknown tensor type id.
 * DSMOE_ERR_BOUNDS: the file ends inside the header or table, or a tensor's bytes run past its end. */
DSMOE_API int dsmoe_gguf_open(const char *path, dsmoe_gguf **out);
/* The same over bytes the caller keeps alive (the reference's parser tests build their files in memory,
 * engine/tests/gguf_parse.rs:12-77). */
DSMOE_API int dsmoe_gguf_open_memory(const void *data, size_t bytes, dsmoe_gguf **out);
DSMOE_API int dsmoe_gguf_close(dsmoe_gguf *g);
DSMOE_API const char *dsmoe_gguf_last_error(const dsmoe_gguf *g);
DSMOE_API uint64_t dsmoe_gguf_tensor_count(const dsmoe_gguf *g);
DSMOE_API uint64_t dsmoe_gguf_data_offset(const dsmoe_gguf *g);
DSMOE_API int dsmoe_gguf_tensor_at(const dsmoe_gguf *g, uint64_t index, dsmoe_gguf_tensor *out);
/* GgufFile::find (engine/src/gguf.rs:118-121); DSMOE_ERR_STATE when there is no such tensor. */
DSMOE_API int dsmoe_gguf_find_tensor(const dsmoe_gguf *g, const char *name, dsmoe_gguf_tensor *out);

/* Device bytes of expert_count experts of one layer: gate (= up) and down. */
DSMOE_API int dsmoe_gguf_expert_shard_bytes(const dsmoe_config *cfg, uint32_t expert_count, uint64_t *gate_up_bytes,
                                            uint64_t *down_bytes);
/* Validates blk.{gguf_layer}.ffn_{gate,up,down}_exps.weight (type ids 16 / 16 / 10, dims [in, out, n_expert] against
 * cfg, byte sizes against the block formats) and copies experts [expert_begin, expert_begin + expert_count) - one
 * expert-parallel shard, or all of them - into the caller's device buffers on `stream`, permuted to ROWSOA on the way
 * when `layout` says so (staging_dev: a device buffer of at least the down shard's bytes; unused for NATIVE). The
 * buffers are then ready for dsmoe_layer_register. Nothing is copied unless all three tensors validate. */
DSMOE_API int dsmoe_gguf_upload_experts(const dsmoe_gguf *g, const dsmoe_config *cfg, dsmoe_stream stream,
                                        uint32_t gguf_layer, uint32_t expert_begin, uint32_t expert_count, int layout,
                                        uint8_t *gate_dev, uint8_t *up_dev, uint8_t *down_dev, uint8_t *staging_dev);

/* ------------------------------------------------------------------------------------------------------------ */
/* For callers that cannot allocate device memory                                                                 */
/* ------------------------------------------------------------------------------------------------------------ */

#define DSMOE_NOALLOC_MAX_TOKENS 8

/* No counterpart in the reference (its Session owns cudaMalloc'd scratch, engine/src/session.rs:224-271).
 *
 * The routed-expert step of dsmoe_moe_forward without a handle and without any device allocation, for hosts where
 * cudaMalloc is not an option: an engine that has already given the whole device to its own arena, a plugin inside a
 * process whose allocator forbids side allocations, a real-time thread that must not take the driver's allocation
 * lock. The intermediates (probabilities, Q8_K blocks, the f32 mid rows) live in a fixed array of about 0.55 MB inside
 * the library's device image; every GPU that loads the library holds that array until the process exits.
 *
 * Fixed to the reference model: n_embd 4096, n_ff 2048, 256 experts, top-6, clamp 10, weights renormalised to 1.5,
 * f16 subnormals flushed. n_tokens above DSMOE_NOALLOC_MAX_TOKENS returns DSMOE_ERR_BOUNDS. gate / up / down are one
 * layer's expert tensors in `layout`; the other operands are as in dsmoe_moe_forward; selected_out / weights_out may
 * be NULL. Runs on the CURRENT device, asynchronously on `stream`.
 *
 * The first call on a device looks the array's address up (cudaGetSymbolAddress); make that first call outside any
 * stream capture. All calls on a device share the one array, which keeps the previous call's contents: the call
 * clears the one word that must start at zero and overwrites the rest before reading it, but two calls whose kernels
 * overlap on the GPU (different streams, or different host threads) race on it — serialise them. */
DSMOE_API int dsmoe_moe_forward_noalloc(dsmoe_stream stream, const uint8_t *gate, const uint8_t *up,
                                        const uint8_t *down, int layout, const float *x, const float *logits,
                                        uint32_t n_tokens, float *out, int32_t *selected_out, float *weights_out);

/* The device status word of dsmoe_moe_forward_noalloc on the CURRENT device (no counterpart in the reference). The
 * kernels of that call bound their waits on asynchronous copies like every other kernel here; the word lives in the
 * same static array as the scratch, so there is no handle to ask. Waits for `stream`, copies the word back (no
 * allocation: a plain cudaMemcpyAsync from the array's looked-up address) and returns DSMOE_OK with *code_out == 0,
 * or DSMOE_ERR_TIMEOUT with the code if a wait expired during the most recent call (each call clears the word
 * first). Returns DSMOE_ERR_STATE if dsmoe_moe_forward_noalloc has not run on this device yet. */
DSMOE_API int dsmoe_noalloc_device_status(dsmoe_stream stream, int *code_out);

#ifdef __cplusplus
}
#endif
#endif /* DSMOE_H */
