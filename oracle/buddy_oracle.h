/*
 * CPU restatement of buddy-mlir's LLM decode arithmetic.
 *
 * TEST INFRASTRUCTURE ONLY.  Nothing in the shipped library links or calls
 * this file; it exists so the CUDA kernels can be checked against the
 * arithmetic buddy-mlir's own generated CPU code performs, and so that the
 * same arithmetic can be timed on the host cores as a baseline.
 *
 * Pinning: the GEMV routines reproduce the reference's runnable known-answer
 * examples (examples/BuddyMatmul/dequant-matmul-vectorization-decode.mlir:93-133,
 * examples/BuddyMatmul/int4-dequant-matmul-vectorization-decode.mlir:160-206,
 * examples/BuddyMatmul/dequant-matmul-vectorization-blis-prefill.mlir:113-115),
 * the panel packer reproduces the address math checked by
 * tests/Conversion/matmul-vectorization-decode-packed.mlir:18-28, the argmax
 * and the KV discard/re-rotation are compared with the reference's own
 * Sampler.h / KVCacheManager.h compiled from source, and the float model is
 * compared with HuggingFace Qwen2/Qwen3 eager on the same weights.  The
 * quantiser, RMSNorm, RoPE and end-to-end logits have no golden vectors in
 * the reference: for those, parity is unpinned by the reference's tests and
 * rests on the HuggingFace cross-check.
 *
 * Every routine cites the reference file:line it follows (paths relative to
 * the buddy-mlir source tree).
 */
#ifndef BUDDY_ORACLE_H
#define BUDDY_ORACLE_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ---- quantiser and nibble packing ------------------------------------- */
/* tools/buddy-codegen/import_model.py:830-850.  W is [K,N] row-major f32;
 * one scale per output column n: max(1e-10, absmax_k / qmax); values are
 * clamp(rne(W/scale), lo, hi). bits = 8 -> qmax 127, range -128..127;
 * bits = 4 -> qmax 7, range -8..7 (values returned unpacked, one per byte). */
void orc_quantize_per_channel(const float *W, int64_t K, int64_t N, int bits,
                              int8_t *Q, float *scale);
/* import_model.py:810-815: flat[2i] -> low nibble, flat[2i+1] -> high. */
void orc_pack_int4(const int8_t *flat, int64_t n, int8_t *packed);
/* frontend/Python/ops/tosa.py:12158-12203: low = ((b&0xF)<<4)>>4 (arithmetic),
 * high = b>>4 (arithmetic); output interleaved low, high. */
void orc_unpack_int4(const int8_t *packed, int64_t nbytes, int8_t *flat);
/* Group-wise zero-point-8 quantiser (a superset format defined by this
 * project, not by the reference): groups of G consecutive k per column n,
 * scale = max(1e-10, absmax/7) rounded to f16, u = clamp(rne(W/scale_f16),
 * -8, 7) + 8.  P is [K, N/2] bytes (even column low nibble), scales are
 * [K/G, N] f16 bit patterns. */
void orc_quantize_w4_group(const float *W, int64_t K, int64_t N, int64_t G,
                           uint8_t *P, uint16_t *scale_f16);

/* ---- decode GEMVs (m = 1 .. M rows, each row independent) -------------- */
/* midend/lib/Conversion/MatMulOptimization/DequantMatMulVectorizationDecode.cpp:250-321:
 * acc=0; for k: acc=fma(x[k], float(Q[k,n]), acc); acc*=scale[n]; y[n]+=acc. */
void orc_gemv_w8_f32(const float *x, const int8_t *Q, const float *scale,
                     float *y, int64_t M, int64_t K, int64_t N);
/* Same pass with f16 element type (accumulator = element type of C,
 * DequantMatMulVectorizationDecode.cpp:228-230).  f16 passed as bit patterns. */
void orc_gemv_w8_f16(const uint16_t *x, const int8_t *Q, const uint16_t *scale,
                     uint16_t *y, int64_t M, int64_t K, int64_t N);
/* Int4DequantMatMulVectorizationDecode.cpp:359-430: P is [K,N/2] signed
 * nibbles, everything f16, f16 accumulation. */
void orc_gemv_w4_f16(const uint16_t *x, const int8_t *P, const uint16_t *scale,
                     uint16_t *y, int64_t M, int64_t K, int64_t N);
/* MatMulVectorizationDecode.cpp:94-192: y[n] += sum_k fma(x[k], B[k,n]). */
void orc_gemv_f32(const float *x, const float *B, float *y, int64_t M,
                  int64_t K, int64_t N);
/* Group-wise zp-8 int4 (this project's format, see orc_quantize_w4_group):
 * per group acc_g = sum_k fma(x[k], float(u-8), acc_g); y[n] += acc_g*s_g. */
void orc_gemv_w4g_f32(const float *x, const uint8_t *P,
                      const uint16_t *scale_f16, float *y, int64_t M,
                      int64_t K, int64_t N, int64_t G);
/* frontend/Python/graph/transform/pack_decode_weights.py:32-124 and
 * MatMulVectorizationDecodePacked.cpp:128-266:
 * packed[(n/V)*K*V + k*V + n%V] = B[k,n]. */
void orc_pack_panels_f32(const float *B, int64_t K, int64_t N, int64_t V,
                         float *packed);
void orc_gemv_f32_packed(const float *x, const float *packed, float *y,
                         int64_t K, int64_t N, int64_t V);
/* MatMulBlisVectorization.cpp:367-530 (prefill): w = float(q)*scale is formed
 * before the FMA. C is accumulated into. */
void orc_gemm_w8_prefill_f32(const float *A, const int8_t *Q,
                             const float *scale, float *C, int64_t M,
                             int64_t K, int64_t N);
/* frontend/Python/ops/linalg.py:12728-12846 (w8a8): dynamic per-tensor int8
 * activations, i8 x i8 -> i32, * (act_scale * scale[n]) (+ bias, may be NULL). */
void orc_matmul_w8a8(const float *A, const int8_t *Q, const float *scale,
                     const float *bias, float *C, int64_t M, int64_t K,
                     int64_t N);

/* ---- small ops --------------------------------------------------------- */
/* examples/BuddyDeepSeekR1/subgraph0_decode_simplify.mlir:60-72. */
void orc_rmsnorm(const float *x, const float *w, float *y, int64_t H,
                 float eps);
/* subgraph0_decode_simplify.mlir:52-59 (angles) and :86-105 (apply). */
void orc_rope(float *v, int64_t heads, int64_t head_dim,
              const float *inv_freq, int64_t pos);
/* subgraph0_decode_simplify.mlir:226-231: (g*sigmoid(g))*u. */
void orc_silu_mul(const float *g, const float *u, float *y, int64_t n);
/* runtime/include/buddy/runtime/llm/Sampler.h:101-104: lowest index of max. */
int64_t orc_argmax_first(const float *v, int64_t n);
/* frontend/Python/ops/tosa.py:14130-14600.  q [q_heads, D], K/V caches
 * [kv_heads, max_len, D]; walks all max_len positions with the additive
 * mask (0 for j<=pos, -inf beyond). out [q_heads, D]. */
void orc_gqa_decode(const float *q, const float *Kc, const float *Vc,
                    float *out, int64_t q_heads, int64_t kv_heads,
                    int64_t max_len, int64_t D, int64_t pos);
/* runtime/include/buddy/runtime/llm/KVCacheManager.h:151-273 as driven by
 * tools/buddy-codegen/gen_session.py:1471-1506.  kv = n_buffers pointers
 * (K at even index). Returns the new position (or -1 if no overflow). */
int64_t orc_kv_overflow(float **kv, int64_t n_buffers, int64_t kv_heads,
                        int64_t max_len, int64_t D, int64_t position,
                        int64_t keep, float theta);

/* ---- whole decode step -------------------------------------------------- */
enum { ORC_LIN_F32 = 0, ORC_LIN_W8 = 1, ORC_LIN_W4G = 2, ORC_LIN_W4 = 3, ORC_LIN_W8H = 4, ORC_LIN_W8Q = 5 };   /* W4: signed nibbles, per-channel f16 scale, f16 accumulation (w4a16); W8H: int8, f16 scale, f16 activations and accumulation (w8a16); W8Q: int8 weights and dynamically quantised int8 activations, one scale per activation tensor (w8a8, orc_matmul_w8a8) */

typedef struct {
  int32_t kind;       /* ORC_LIN_* */
  int32_t group;      /* W4G group size */
  int64_t K, N;
  const void *w;      /* [K,N] f32 | [K,N] int8 | [K,N/2] nibbles */
  const void *scale;  /* f32 [N] (W8) | f16 [K/G,N] (W4G) | null */
  const float *bias;  /* [N] or null */
} OrcLinear;

typedef struct {
  const float *in_norm, *post_norm; /* [hidden] */
  const float *q_norm, *k_norm;     /* [head_dim] or null (Qwen3 QK-norm) */
  OrcLinear q, k, v, o, gate, up, down;
} OrcLayer;

typedef struct {
  int64_t hidden, n_layers, q_heads, kv_heads, head_dim, ffn, vocab, max_len;
  float eps;
  const float *embed;     /* [vocab, hidden] */
  const float *inv_freq;  /* [head_dim/2] */
  const OrcLayer *layers;
  const float *final_norm;
  OrcLinear lm_head;
} OrcModel;

/* One decode step of the graph in subgraph0_decode_simplify.mlir:46-260 (+
 * tail). kv: 2*n_layers buffers [kv_heads,max_len,head_dim] (K even, V odd),
 * updated in place at row pos. logits: [vocab]. */
void orc_decode_step(const OrcModel *m, int64_t token, int64_t pos, float **kv,
                     float *logits);
/* The prefill graph over M rows at positions 0..M-1 (the same operations as the
 * decode step, row-batched; tools/buddy-codegen/import_model.py:640-680 builds
 * both graphs from one model).  It differs from M decode steps only where an
 * operation looks at the whole activation tensor: a W8Q projection takes its
 * activation scale over all M rows (frontend/Python/ops/linalg.py:12728-12846).
 * kv rows 0..M-1 are written; logits: [M, vocab]. */
void orc_prefill_rows(const OrcModel *m, const int64_t *tokens, int64_t M,
                      float **kv, float *logits);
/* Number of OpenMP threads the routines above will use. */
int orc_num_threads(void);

#ifdef __cplusplus
}
#endif
#endif
