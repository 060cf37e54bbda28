/*
 * buddy_b200 -- the symbols buddy-mlir's compiled code binds.
 *
 * Calling convention (identical to runtime/external_kernels in buddy-mlir):
 * after bufferisation and -llvm-request-c-wrappers (tools/buddy-codegen/
 * compile_pipeline.py:66) a graph-level `func.call @name(tensor...) -> tensor`
 * (frontend/Python/ops/func.py:115-147) becomes
 *     void _mlir_ciface_<name>(ResultDesc *out, ArgDesc *a0, ArgDesc *a1, ...)
 * with every descriptor
 *     { T *allocated; T *aligned; intptr_t offset; intptr_t sizes[R]; intptr_t strides[R]; }
 * (frontend/Interfaces/buddy/Core/Container.h:126-138; the StridedMemRefType
 * of runtime/external_kernels/rng/RNGUtils.cpp:87-118).  Strides are in
 * elements and may be non-contiguous.  `out` arrives uninitialised: the callee
 * mallocs the result and fills every field (RNGUtils.cpp:104-117,
 * runtime/external_kernels/matmul/MatmulTorq.cpp:149-165); the generated code
 * frees it later.  The functions return void; on failure they leave
 * out->allocated = out->aligned = NULL (MatmulTorq.cpp:150-151 returns
 * silently on OOM) and the reason is available from b200_last_error().
 *
 * All buffers here are HOST memory.  Weight operands are uploaded and
 * repacked once and cached by host address; b200_release_cached_weights()
 * drops the cache.
 */
#ifndef BUDDY_B200_MEMREF_H
#define BUDDY_B200_MEMREF_H

#include "buddy_b200.h"

#ifdef __cplusplus
extern "C" {
#endif

#define B200_MEMREF(NAME, T, R)                                                \
  typedef struct {                                                             \
    T *allocated;                                                              \
    T *aligned;                                                                \
    intptr_t offset;                                                           \
    intptr_t sizes[R];                                                         \
    intptr_t strides[R];                                                       \
  } NAME

B200_MEMREF(b200_memref_f32_1, float, 1);
B200_MEMREF(b200_memref_f32_2, float, 2);
B200_MEMREF(b200_memref_f32_3, float, 3);
B200_MEMREF(b200_memref_f32_4, float, 4);
B200_MEMREF(b200_memref_f16_2, uint16_t, 2);
B200_MEMREF(b200_memref_i8_2, int8_t, 2);
B200_MEMREF(b200_memref_i64_1, long long, 1);
B200_MEMREF(b200_memref_i64_2, long long, 2);

/* Same symbol, same signature as runtime/include/buddy/runtime/Matmul.h:35-36
 * (implemented there for RISC-V only, MatmulTorq.cpp:116-166): result = A*B,
 * A [M,K], B [K,N] f32. */
void _mlir_ciface_buddy_matmul_f32(b200_memref_f32_2 *result,
                                   b200_memref_f32_2 *A, b200_memref_f32_2 *B);

/* int8 weight-only decode matmul: C[m,n] = scale[0,n] * sum_k A[m,k]*W[k,n].
 * Replaces the code DequantMatMulVectorizationDecode.cpp:191-366 generates
 * for the chain sitofp(W) * scale -> linalg.matmul. A [M,K] f32, W [K,N]
 * int8, scale [1,N] f32. */
void _mlir_ciface_buddy_gemv_w8_f32(b200_memref_f32_2 *result,
                                    b200_memref_f32_2 *A, b200_memref_i8_2 *W,
                                    b200_memref_f32_2 *scale);

/* W8A8 matmul: what the reference lowers QuantizedMatmulOp to
 * (frontend/Python/ops/linalg.py:12797-12846): dynamic per-tensor int8
 * activations, i8 x i8 -> i32, C[m,n] = float(acc) * (act_scale * scale[0,n]).
 * A [M,K] f32 (K a multiple of 64), W [K,N] int8, scale [1,N] f32.  Runs on the
 * integer tensor cores; bit-identical to the reference arithmetic. */
void _mlir_ciface_buddy_matmul_w8a8_f32(b200_memref_f32_2 *result,
                                        b200_memref_f32_2 *A, b200_memref_i8_2 *W,
                                        b200_memref_f32_2 *scale);

/* packed-int4 decode matmul, f16 in / f16 out
 * (Int4DequantMatMulVectorizationDecode.cpp:320-562): A [M,K] f16,
 * P [K,N/2] signed nibbles, scale [1,N] f16. Accumulates in f32. */
void _mlir_ciface_buddy_gemv_w4_f16(b200_memref_f16_2 *result,
                                    b200_memref_f16_2 *A, b200_memref_i8_2 *P,
                                    b200_memref_f16_2 *scale);

/* group-wise zero-point-8 int4 (this library's format): A [M,K] f32,
 * P [K,N/2] codes, scale [K/G,N] f16; G = K / scale->sizes[0]. */
void _mlir_ciface_buddy_gemv_w4g_f32(b200_memref_f32_2 *result,
                                     b200_memref_f32_2 *A, b200_memref_i8_2 *P,
                                     b200_memref_f16_2 *scale);

/* RMSNorm over the last dim (subgraph0_decode_simplify.mlir:60-72):
 * x [rows,H], w [H]; eps is a one-element memref. */
void _mlir_ciface_buddy_rmsnorm_f32(b200_memref_f32_2 *result,
                                    b200_memref_f32_2 *x, b200_memref_f32_1 *w,
                                    b200_memref_f32_1 *eps);

/* silu(g) * u (subgraph0_decode_simplify.mlir:226-231). */
void _mlir_ciface_buddy_silu_mul_f32(b200_memref_f32_2 *result,
                                     b200_memref_f32_2 *g,
                                     b200_memref_f32_2 *u);

/* RoPE at one position (subgraph0_decode_simplify.mlir:52-59, 86-105):
 * x [1,heads,1,D], inv_freq [D/2], pos [1]. */
void _mlir_ciface_buddy_rope_f32(b200_memref_f32_4 *result,
                                 b200_memref_f32_4 *x,
                                 b200_memref_f32_1 *inv_freq,
                                 b200_memref_i64_1 *pos);

/* GQA decode attention (frontend/Python/ops/tosa.py:13931-14635):
 * q [1,q_heads,1,D], caches [1,kv_heads,max_len,D], pos [1] (rows 0..pos are
 * live; the reference expresses the same thing with its additive mask). */
void _mlir_ciface_buddy_gqa_decode_f32(b200_memref_f32_4 *result,
                                       b200_memref_f32_4 *q,
                                       b200_memref_f32_4 *k_cache,
                                       b200_memref_f32_4 *v_cache,
                                       b200_memref_i64_1 *pos);

void b200_release_cached_weights(void);

/* ------------------------------------------------------------------------
 * Whole-entry model ABI.  The generated ModelSession resolves
 * _mlir_ciface_forward_decode in the model .so by dlsym and calls it with
 *   (DecodeABI *result, MemRef<Tw,1> *w0 [, *w1], MemRef<i64,2> *token,
 *    MemRef<i64,1> *cache_position, KV4 *kv0, KV4 *kv1, Dummy1 *dummy0,
 *    KV4 *kv2, KV4 *kv3, Dummy1 *dummy1, ...)
 * (tools/buddy-codegen/gen_session.py:979-1008, 1381-1414); DecodeABI is
 * { i64_1 cache_position_out; f32_4 kv0, kv1; i64_1 dummy0; f32_4 kv2, kv3;
 *   i64_1 dummy1; ...; f32_3 logits } (gen_session.py:924-972).  Because the
 * arity depends on the model, that symbol lives in a small per-variant shim
 * (buddy_mlir_b200/gen_model_entry.py writes it) which unpacks the
 * descriptors and calls this function.
 *
 * host_kv: 2*n_layers host cache buffers [1,kv_heads,max_len,head_dim], K at
 * even index.  The reference entry is stateless; this one keeps the cache on
 * the device together with a host copy of what the device holds.  Before a
 * step, rows 0, (pos-1)/2 and pos-1 of every host buffer are compared with
 * that copy: if they differ (first decode after a CPU prefill, another
 * sequence, the host-side handleKVCacheOverflow of gen_session.py:1471-1506)
 * or the device holds fewer than `pos` rows, rows [0,pos) are uploaded from
 * host_kv first.
 * Every call writes the new K/V row `pos` back into host_kv, so the host
 * buffers stay what the reference's in-place KV write would have left.
 * logits_out receives a malloc'ed [vocab] f32 buffer the caller frees
 * (gen_session.py:1416-1442 copies it out and destroys the descriptor).
 * ---------------------------------------------------------------------- */
int b200_forward_decode(const b200_model_config *cfg, const char *variant,
                        int all_linear_w8, const void *w0, int64_t n0,
                        const void *w1, int64_t n1, long long token,
                        long long pos, float *const *host_kv,
                        float **logits_out);
/* Prefill counterpart, behind _mlir_ciface_forward_prefill(PrefillABI *result,
 * MemRef<Tw,1> *w0 [, *w1], Text<size_t,2> *tokens)
 * (tools/buddy-codegen/gen_session.py:908-923 PrefillABI = 2*n_layers KV
 * buffers then logits [1,max_len,vocab]; :979-984 the function type;
 * :1345-1373 the call, which copies every result into the session's state).
 * tokens: n_rows ids (the prompt, and the pad rows behind it if the caller
 * wants them computed as the reference does).  Row i is computed at position
 * i over rows [0,i) -- causal, as flash_attention_for_cpu_prefill_op
 * (frontend/Python/ops/tosa.py:4326-4700).  host_kv_out: 2*n_layers buffers
 * [1,kv_heads,max_len,head_dim] that receive rows [0,n_rows) (rows behind them
 * are zeroed); logits_out: [max_len,vocab] f32, rows [0,n_rows) are written.
 * The cache stays on the device: a following b200_forward_decode at any
 * position <= n_rows whose host cache still holds these rows uploads nothing. */
int b200_forward_prefill(const b200_model_config *cfg, const char *variant,
                         int all_linear_w8, const void *w0, int64_t n0,
                         const void *w1, int64_t n1, const long long *tokens,
                         int n_rows, float *const *host_kv_out,
                         float *logits_out);
/* The same two entries for the variants whose cache and logits are f16 on the
 * host (w4a16: tools/buddy-codegen/gen_config.py:37-49; uint16_t holds the IEEE
 * half bits, as in the reference's generated session).  The device session
 * stays f32; rows and logits are rounded to half at the boundary, and the host
 * cache check compares against the rounded rows. */
int b200_forward_decode_f16(const b200_model_config *cfg, const char *variant,
                            int all_linear_w8, const void *w0, int64_t n0,
                            const void *w1, int64_t n1, long long token,
                            long long pos, uint16_t *const *host_kv,
                            uint16_t **logits_out);
int b200_forward_prefill_f16(const b200_model_config *cfg, const char *variant,
                             int all_linear_w8, const void *w0, int64_t n0,
                             const void *w1, int64_t n1, const long long *tokens,
                             int n_rows, uint16_t *const *host_kv_out,
                             uint16_t *logits_out);
/* And with bfloat16 cache and logits, again carried as uint16_t (the bf16
 * variant, tools/buddy-codegen/gen_config.py:40-44; values leave the device
 * session rounded to nearest even). */
int b200_forward_decode_bf16(const b200_model_config *cfg, const char *variant,
                             int all_linear_w8, const void *w0, int64_t n0,
                             const void *w1, int64_t n1, long long token,
                             long long pos, uint16_t *const *host_kv,
                             uint16_t **logits_out);
int b200_forward_prefill_bf16(const b200_model_config *cfg, const char *variant,
                              int all_linear_w8, const void *w0, int64_t n0,
                              const void *w1, int64_t n1, const long long *tokens,
                              int n_rows, uint16_t *const *host_kv_out,
                              uint16_t *logits_out);
/* The same two entries for the tiered-cache spec
 * (models/deepseek_r1/specs/f32_tiered_kv_cache.json; gen_session.py:303-800
 * resolves _mlir_ciface_forward_prefill_<size> / _mlir_ciface_forward_decode_<size>
 * for every cache size and moves the host cache to a larger tier as the
 * sequence grows): host_len = rows per kv head of the host buffers of the tier;
 * the device session keeps max_len rows whatever the tier. */
int b200_forward_decode_tier(const b200_model_config *cfg, const char *variant,
                             int all_linear_w8, const void *w0, int64_t n0,
                             const void *w1, int64_t n1, long long token,
                             long long pos, float *const *host_kv, int host_len,
                             float **logits_out);
int b200_forward_prefill_tier(const b200_model_config *cfg, const char *variant,
                              int all_linear_w8, const void *w0, int64_t n0,
                              const void *w1, int64_t n1, const long long *tokens,
                              int n_rows, float *const *host_kv_out, int host_len,
                              float *logits_out);
/* The entry symbols return void, so a failure cannot be reported through them:
 * the shim prints the reason, hands back zero-filled logits of the right shape
 * (the reference caller copies from the buffer unconditionally,
 * gen_session.py:1416-1418) and this code stays set -- the first failure since
 * the last b200_forward_reset(), 0 if none; b200_last_error() has the text. */
int b200_forward_status(void);
/* Diagnostic: how many times the entry pair has built its device session (upload,
 * quantise, pack) since the last b200_forward_reset().  Variant "f32p32" is the
 * f32 blob with every matmul weight in 32-column panels -- the decode file of the
 * reference's packed-decode spec (pack_decode_weights.py:32-124,
 * gen_session.py:1290-1300,1393): the decode entry receives it while the prefill
 * entry receives the plain blob, and both are recognised as one model. */
int b200_forward_session_builds(void);
/* Drop the session the two entries keep (weights, KV, graph) and the status. */
void b200_forward_reset(void);

#ifdef __cplusplus
}
#endif
#endif
