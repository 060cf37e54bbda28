/*
 * buddy_b200 -- hand-written sm_100a kernels for buddy-mlir's LLM decode path,
 * behind a plain C ABI.
 *
 * Three layers, lowest first:
 *
 *   1. b200_*            device-pointer entry points (weights, activations and
 *                        KV already resident in HBM; every call takes a CUDA
 *                        stream as void*).  This is the performance surface.
 *   2. b200_model_*      a device-resident decode session: weights in the
 *                        packed device layout, KV cache, one CUDA graph per
 *                        decode step.
 *   3. _mlir_ciface_*    the symbols buddy-mlir's compiled code and generated
 *                        ModelSession bind: per-op external kernels in the
 *                        convention of runtime/external_kernels (MemRef
 *                        descriptors on the host, callee-allocated result) and
 *                        the model entry _mlir_ciface_forward_decode.
 *                        Declared in buddy_b200_memref.h.
 *
 * All functions return 0 on success and a negative B200_E* code on failure;
 * b200_last_error() gives the message of the calling thread's last failure.
 * Nothing here falls back to the CPU: without a CUDA device every compute
 * entry point fails with B200_ENODEV.
 */
#ifndef BUDDY_B200_H
#define BUDDY_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define B200_OK 0
#define B200_EINVAL (-1)  /* bad argument (shape, alignment, null pointer) */
#define B200_ECUDA (-2)   /* a CUDA runtime call failed */
#define B200_ENODEV (-3)  /* no usable CUDA device */
#define B200_ENOMEM (-4)  /* device or host allocation failed */
#define B200_ELIMIT (-5)  /* size beyond a documented fixed limit */
#define B200_ESTATE (-6)  /* call sequence error (e.g. decode before load) */

const char *b200_last_error(void);
/* Library version, and the number of kernels launched by this process so far
 * (counted at every launch site; graph replays add the node count). */
const char *b200_version(void);
uint64_t b200_launch_count(void);

/* Element types of activation / scale buffers. */
enum { B200_F32 = 0, B200_F16 = 1, B200_BF16 = 2 };

/* Weight kinds of the packed device layout. */
enum {
  B200_W_F32 = 0, /* f32, row n = output channel, K contiguous            */
  B200_W_I8 = 1,  /* int8, per-output-channel scale                       */
  B200_W_U4 = 2   /* 4-bit, value = nibble - 8, one scale per `group` k    */
};

/* ------------------------------------------------------------------------
 * Packed device layout ("packed decode weights").
 *
 * buddy-mlir keeps every matmul weight as [K,N] row-major after
 * eliminate_transpose (frontend/Python/graph/transform/eliminate_weight_transpose.py:163-219),
 * which its CPU GEMV walks with a stride of N between consecutive k
 * (docs/DecodeWeightPacking.md:27-46), and panel-packs only float weights
 * (frontend/Python/graph/transform/pack_decode_weights.py:32-124).  The device
 * layout here is one row per OUTPUT channel n with the row's K weights
 * contiguous, so that a warp streams one output row with 32 x 16-byte loads.
 * Inside a row, k is permuted within blocks of 32 sixteen-byte units so that
 * the four (int8) or eight (int4) 4-element groups a lane holds are a quarter
 * (an eighth) of a block apart: the activation reads from shared memory are
 * then contiguous across lanes.  b200_packed_offset() states the map.
 * ---------------------------------------------------------------------- */

/* Padded K (elements) and bytes per packed row for a weight kind. */
int64_t b200_packed_k(int kind, int64_t K);
int64_t b200_packed_row_bytes(int kind, int64_t K);
/* Byte offset inside a packed row of element k (for U4: of the byte holding
 * it; *nibble = 0 low, 1 high).  Pure host function. */
int64_t b200_packed_offset(int kind, int64_t K, int64_t k, int *nibble);

/* Reference layout -> device layout.  src is the reference's [K,N] row-major
 * tensor: f32, int8, or nibble-packed [K,N/2] (even column = low nibble,
 * tools/buddy-codegen/import_model.py:810-815).  src_signed = 1 means the
 * nibbles are two's complement (-8..7, the reference's w4a16 format) and are
 * stored as nibble+8; 0 means they already are zero-point-8 codes. */
int b200_pack_weight(int kind, const void *src_kn, int64_t K, int64_t N,
                     int src_signed, void *dst, void *stream);
/* Device layout -> reference layout (exact inverse of b200_pack_weight). */
int b200_unpack_weight(int kind, const void *packed, int64_t K, int64_t N,
                       int dst_signed, void *dst_kn, void *stream);
/* Scales: reference [K/G, N] (or [N] when G == K) -> device [N, K/G]. */
int b200_pack_scales(const void *src, int dtype, int64_t groups, int64_t N,
                     void *dst, void *stream);

/* Replaces extract_quantized_weights (tools/buddy-codegen/import_model.py:790-892):
 * W [K,N] f32 -> Q [K,N] int8 values (bits = 8: -128..127, bits = 4: -8..7)
 * and scale [N] f32 = max(1e-10, absmax_k / qmax). */
int b200_quantize_per_channel(const float *W, int64_t K, int64_t N, int bits,
                              int8_t *Q, float *scale, void *stream);
/* Group-wise zero-point-8 int4 quantiser (this library's superset format):
 * P [K,N/2] nibble codes, scales [K/G,N] f16. */
int b200_quantize_w4_group(const float *W, int64_t K, int64_t N, int64_t G,
                           uint8_t *P, uint16_t *scale_f16, void *stream);
/* Replaces pack_int4_nibbles (import_model.py:810-815) and int4_unpack_op
 * (frontend/Python/ops/tosa.py:12158-12203). */
int b200_pack_int4(const int8_t *flat, int64_t n, int8_t *packed, void *stream);
int b200_unpack_int4(const int8_t *packed, int64_t nbytes, int8_t *flat,
                     void *stream);

/* ------------------------------------------------------------------------
 * Decode GEMV, M = 1..16 activation rows.
 * Replaces the loops emitted by
 *   midend/lib/Conversion/MatMulOptimization/DequantMatMulVectorizationDecode.cpp:191-366      (I8)
 *   midend/lib/Conversion/MatMulOptimization/Int4DequantMatMulVectorizationDecode.cpp:320-562  (U4)
 *   midend/lib/Conversion/MatMulOptimization/MatMulVectorizationDecode.cpp:94-192              (F32)
 * y[m,n] = (accumulate ? y[m,n] : 0) + bias[n] + residual[m,n]
 *          + sum_g scale[n,g] * sum_{k in g} x[m,k] * w[n,k]
 * with f32 accumulation.  When norm_weight != NULL, x is first replaced by
 * norm_weight * (x * rsqrt(mean(x^2) + eps)) (the RMSNorm of
 * examples/BuddyDeepSeekR1/subgraph0_decode_simplify.mlir:60-72).  When
 * silu_pairs != 0 the N rows are (gate_j, up_j) pairs and y has N/2 columns:
 * y[m,j] = silu(row 2j) * row 2j+1 (subgraph0_decode_simplify.mlir:226-231).
 * ---------------------------------------------------------------------- */
typedef struct {
  int32_t kind;        /* B200_W_*                                         */
  int32_t group;       /* U4: k per scale; I8/F32: ignored                 */
  int64_t K, N;
  const void *w;       /* packed device layout                             */
  const void *scale;   /* I8: [N]; U4: [N, K/group]; F32: NULL             */
  int32_t scale_dtype; /* B200_F32 or B200_F16                             */
  int32_t reserved;
  const float *bias;   /* [N] or NULL                                      */
} b200_weight;

typedef struct {
  const void *x;          /* [M,K] activations                             */
  int32_t x_dtype;        /* B200_F32 / F16 / BF16                         */
  int32_t y_dtype;        /* B200_F32 / F16                                */
  int64_t x_ld, y_ld;     /* row strides in elements                       */
  void *y;                /* [M,N] (or [M,N/2] with silu_pairs)            */
  const float *residual;  /* [M,N] f32, stride y_ld, or NULL; may alias y  */
  const float *norm_weight; /* [K] or NULL                                 */
  float norm_eps;
  int32_t M;
  int32_t accumulate;
  int32_t silu_pairs;
} b200_gemv_args;

int b200_gemv(const b200_weight *w, const b200_gemv_args *a, void *stream);

/* Dense weight-only GEMM for prefill and batched decode, on the tcgen05 tensor
 * cores: C[M,N] = A[M,K] * dequant(W)^T (+ bias) (+ residual), or, with
 * silu_pairs, C[M,N/2] = silu(gate) * up over interleaved (gate, up) rows.
 * Replaces the prefill matmul of
 * midend/lib/Conversion/MatMulOptimization/MatMulBlisVectorization.cpp:367-530
 * (dequantisation fused into the B packing; known answer
 * examples/BuddyMatmul/dequant-matmul-vectorization-blis-prefill.mlir:113-115).
 * w: int8 per-channel packed rows as for b200_gemv (f32 scales, optional
 * bias), K a multiple of 64.  A: f32 [M, lda] on the device; norm_weight (or
 * NULL): RMSNorm of every row of A first.  The f32 activations are split into
 * two bf16 terms (16 significant bits), int8 -> bf16 is exact, accumulation is
 * f32 in tensor memory.  workspace: b200_gemm_w8_workspace_bytes(M, K) bytes,
 * 256-byte aligned, owned by the caller (it holds the split activations and an
 * error word).  b200_gemm_w8_status() reports a bounded wait that gave up. */
int64_t b200_gemm_w8_workspace_bytes(int M, int64_t K);
int b200_gemm_w8(const b200_weight *w, const float *A, int M, int64_t lda,
                 float *C, int64_t ldc, const float *residual, int64_t ldr,
                 const float *norm_weight, float norm_eps, int silu_pairs,
                 void *workspace, int64_t workspace_bytes, void *stream);
int b200_gemm_w8_status(void *workspace, void *stream);

/* W8A8 (buddy-mlir's QuantizedMatmulOp / QuantizedAddMMOp,
 * frontend/Python/ops/linalg.py:12728-12910): the activations get one dynamic
 * scale for the whole [M, K] tensor, s = max(absmax / 127, 1e-10), are rounded
 * to int8 (nearest even), contracted exactly with the int8 weights on the
 * integer tensor-core path (tcgen05.mma kind::i8, s32 accumulator in tensor
 * memory), and C[m, n] = float(acc) * (s * scale[n]) (+ w->bias[n]).  Every
 * step follows the reference operation by operation: results are bit-identical
 * to its arithmetic.  w: int8 per-channel weights in the packed device layout,
 * K a multiple of 64.  workspace: b200_gemm_w8a8_workspace_bytes(M, K) bytes,
 * 256-byte aligned; b200_gemm_w8_status() reads its error word as well. */
int64_t b200_gemm_w8a8_workspace_bytes(int M, int64_t K);
int b200_gemm_w8a8(const b200_weight *w, const float *A, int M, int64_t lda,
                   float *C, int64_t ldc, void *workspace,
                   int64_t workspace_bytes, void *stream);

/* ------------------------------------------------------------------------
 * Small fused ops (f32).
 * ---------------------------------------------------------------------- */
/* RMSNorm, subgraph0_decode_simplify.mlir:60-72. x,y [rows,H]. */
int b200_rmsnorm(const float *x, const float *w, float *y, int64_t rows,
                 int64_t H, float eps, void *stream);
/* silu(g) * u, subgraph0_decode_simplify.mlir:226-231. */
int b200_silu_mul(const float *g, const float *u, float *y, int64_t n,
                  void *stream);
/* RoPE on q [q_heads,D] and k [kv_heads,D] in place at position *pos, then
 * write k and v into cache row *pos (subgraph0_decode_simplify.mlir:52-59,
 * 86-142).  Optional per-head RMSNorm of q and k first (Qwen3). pos is a
 * device pointer so the call can live in a CUDA graph. */
int b200_rope_kv_write(float *q, float *k, const float *v, float *k_cache,
                       float *v_cache, const float *inv_freq,
                       const float *q_norm, const float *k_norm, float eps,
                       int q_heads, int kv_heads, int D, int max_len,
                       const int32_t *pos, void *stream);
/* GQA decode attention, frontend/Python/ops/tosa.py:13931-14635: one query
 * row per head against cache rows [0, *pos].  scratch holds the split
 * partials and one arrival counter per kv head: b200_gqa_scratch_floats()
 * floats, zeroed once by the caller before the first call (every call leaves
 * the counters at zero again). */
int64_t b200_gqa_scratch_floats(int q_heads, int D, int splits);
int b200_gqa_decode(const float *q, const float *k_cache, const float *v_cache,
                    float *out, float *scratch, int q_heads, int kv_heads,
                    int D, int max_len, int splits, const int32_t *pos,
                    void *stream);
/* The same attention for callers that must not allocate device memory.
 * (No counterpart in buddy-mlir.)  Some hosts hand every byte of device memory
 * to a planner before inference starts, and some run decode inside loops where
 * a cudaMalloc -- which can stall the whole device -- is not acceptable; such
 * callers have nowhere to get the split-partial scratch from.  This entry point
 * uses an array built into the library image instead: B200_GQA_STATIC_SCRATCH_FLOATS
 * floats (about 1.07 MB, resident on every GPU that loads the library until
 * the process exits).  It calls no cudaMalloc, cudaFree or allocating library
 * routine.  Shapes whose scratch (b200_gqa_scratch_floats) exceeds the array
 * are refused with B200_ELIMIT.  The first call on a device looks up the
 * array's device address; make that first call before any stream capture
 * begins.  All calls share the one array: calls that can overlap on the GPU
 * (different streams, different threads) race and must be serialised by the
 * caller.  Inputs, outputs and results are exactly those of b200_gqa_decode. */
#define B200_GQA_STATIC_SCRATCH_FLOATS (64 * 32 * 130 + 64)
int b200_gqa_decode_static(const float *q, const float *k_cache, const float *v_cache, float *out,
                           int q_heads, int kv_heads, int D, int max_len, int splits,
                           const int32_t *pos, void *stream);
/* Embedding row gather (subgraph0_decode_simplify.mlir:46-49). */
int b200_embed(const float *table, const int32_t *token, float *x, int64_t H,
               void *stream);
/* Greedy sampling: lowest index among equal maxima
 * (runtime/include/buddy/runtime/llm/Sampler.h:101-104). scratch: 2*1024
 * floats. */
int b200_argmax_first(const float *v, int64_t n, int32_t *out, float *scratch,
                      void *stream);
/* KV overflow: discard + move + zero + RoPE re-rotation of K
 * (runtime/include/buddy/runtime/llm/KVCacheManager.h:151-273 as driven by
 * tools/buddy-codegen/gen_session.py:1471-1506).  kv_dev: device array of
 * n_buffers device pointers (K at even index).  Returns new position in
 * *new_position (host), or -1 there when position < max_len. */
int b200_kv_overflow(float **kv_dev, int n_buffers, int kv_heads, int max_len,
                     int D, int position, int keep, float theta,
                     int *new_position, void *stream);

/* ------------------------------------------------------------------------
 * Device-resident decode session.
 * ---------------------------------------------------------------------- */
typedef struct {
  int32_t hidden, n_layers, q_heads, kv_heads, head_dim, ffn, vocab, max_len;
  float eps, rope_theta;
  int32_t qkv_bias; /* Qwen2: 1 */
  int32_t qk_norm;  /* Qwen3: 1 */
  int32_t tp_rank, tp_size; /* tensor parallel shard of this process */
} b200_model_config;

typedef struct b200_model b200_model;

/* Tensor slots for b200_model_set_*; layer = -1 for model-level slots. */
enum {
  B200_T_EMBED = 0, B200_T_INV_FREQ, B200_T_FINAL_NORM, B200_T_LM_HEAD,
  B200_T_IN_NORM, B200_T_POST_NORM, B200_T_Q_NORM, B200_T_K_NORM,
  B200_T_Q, B200_T_K, B200_T_V, B200_T_O, B200_T_GATE, B200_T_UP, B200_T_DOWN,
  B200_T_Q_BIAS, B200_T_K_BIAS, B200_T_V_BIAS
};

int b200_model_create(const b200_model_config *cfg, b200_model **out);
void b200_model_destroy(b200_model *m);
/* Upload a float vector / table from HOST memory (full, unsharded tensor). */
int b200_model_set_vector(b200_model *m, int layer, int slot,
                          const float *host, int64_t n);
/* Upload one linear layer from HOST memory in the reference's layout
 * ([K,N] row-major f32 / int8 / nibble-packed) and repack it on the device.
 * src_kind: B200_W_*; quantize_to: -1 keep, B200_W_I8 / B200_W_U4 quantise an
 * f32 source on the device first (group = U4 group size, 0 = per channel). */
int b200_model_set_linear(b200_model *m, int layer, int slot, int src_kind,
                          const void *host_w, const void *host_scale,
                          int scale_dtype, int src_signed, int64_t K,
                          int64_t N, int quantize_to, int group);
/* Walk buddy-mlir's flat weight blobs (frontend/Python/graph/graph.py:836-863,
 * frontend/Python/graph/transform/quantization/quantize.py:577-589; file
 * table tools/buddy-codegen/gen_config.py:51-71) and load every tensor.
 * Tensor order (Qwen2), as tools/buddy-codegen/import_model.py writes it: the
 * parameters in the order the traced graph first uses them, then the rotary
 * buffer (frontend/Python/frontend.py:922-933): embedding, per layer {input
 * norm, Wq, q bias, Wk, k bias, Wv, v bias, Wo, post-attention norm, Wgate,
 * Wup, Wdown}, final norm, lm_head, inv_freq; every matmul weight [K,N]
 * row-major; the scales of the quantised tensors follow in that tensor order.
 * Qwen3 (no biases, head norms): input norm, Wq, q norm, Wk, k norm, Wv, Wo, ...
 * variant: "f32", "f16" or "bf16" (one blob of f32 / f16 / bf16 elements), "w8a32" (float blob + int8 blob: o, gate, up,
 * down and lm_head quantised, q/k/v float, scales at the end of the float
 * blob), "w8a8" (the files of w8a32; the session then quantises the activations of
 * the int8 projections as well, see b200_model_set_activation_int8), "w8a16"
 * (the same split, the float blob and the scales as f16) or
 * "w4a16" (f16 blob + nibble-packed signed int4 blob, f16 scales); n_float
 * counts elements of the float blob whatever their width. all_linear_w8 != 0 additionally quantises every remaining f32 linear
 * layer to int8 on the device. */
int b200_model_load_blobs(b200_model *m, const char *variant,
                          const void *float_blob, int64_t n_float,
                          const void *int_blob, int64_t n_int,
                          int all_linear_w8);
/* The w8a8 graphs (tools/buddy-codegen/import_model.py:669-675,
 * frontend/Python/graph/transform/quantization/passes.py:54-140): every int8
 * per-channel projection becomes QuantizedMatmulOp: its activation tensor
 * (all rows of a prefill, the one row of a decode step) gets one dynamic int8
 * scale and the contraction runs on the integer tensor cores (b200_gemm_w8a8).
 * enabled != 0 routes prefill, decode and generate of this session through
 * that arithmetic (a decode step quantises each projection's input row and
 * contracts it by dp4a over the int8 weight rows, as a CUDA graph of its own;
 * the persistent decode kernel serves the float-activation variants only).
 * Single-GPU sessions; the batched entry points (b200_batch_*) refuse such a
 * session, since rows of unrelated sequences would share one scale.  Not stored by
 * b200_model_save_packed: set it again after b200_model_load_packed. */
int b200_model_set_activation_int8(b200_model *m, int enabled);
int b200_model_activation_int8(const b200_model *m);
/* Repack cache (the one-time GPU-layout repack of a model's blobs, kept on disk).
 * save_packed writes the packed device layout of every tensor set so far
 * (quantised, sharded for this tensor-parallel rank) to `path`; call it after
 * load_blobs / set_linear / set_vector and BEFORE finalize.  load_packed fills a
 * freshly created model from such a file instead of walking the blobs; the file
 * must have been written for the same configuration, tp_size and tp_rank
 * (B200_EINVAL otherwise).  The file holds nothing but this library's own
 * layout: a new library version may refuse an old file. */
int b200_model_save_packed(b200_model *m, const char *path);
int b200_model_load_packed(b200_model *m, const char *path);
/* Expected element counts of the blobs for a variant (pure host function). */
int b200_blob_elements(const b200_model_config *cfg, const char *variant,
                       int64_t *n_float, int64_t *n_int);
/* Finish loading: fuse q|k|v and gate|up rows, build the decode graph. */
int b200_model_finalize(b200_model *m);
/* Copy KV rows [pos0, pos0 + n_pos) of every head of one cache buffer (index
 * 2*layer + (0 K | 1 V)) between a host buffer laid out like the reference's
 * [1, kv_heads, max_len, head_dim] f32 cache and the device cache. */
int b200_model_kv_upload(b200_model *m, int buffer, const float *host,
                         int pos0, int n_pos);
int b200_model_kv_download(b200_model *m, int buffer, float *host, int pos0,
                           int n_pos);
/* The K and V rows the last decode step wrote, gathered:
 * host [2*n_layers][local kv_heads][head_dim] (K of layer l at index 2l). */
int b200_model_read_new_kv_rows(b200_model *m, float *host);
/* One decode step (the body of _mlir_ciface_forward_decode): token at cache
 * row `pos`.  logits_host (vocab floats, may be NULL) receives the logits;
 * next_token (may be NULL) the device-side greedy argmax. */
int b200_model_decode(b200_model *m, int token, int pos, float *logits_host,
                      int *next_token);
/* Device-resident loop: `steps` greedy decode steps starting from `token` at
 * `pos`, feeding each argmax back without leaving the GPU; tokens_out
 * receives the `steps` generated ids. */
int b200_model_generate(b200_model *m, int token, int pos, int steps,
                        int *tokens_out);
/* Prefill: n_tokens prompt rows at positions pos0 .. pos0 + n_tokens - 1 in one
 * pass (the reference's compiled forward_prefill,
 * tools/buddy-codegen/gen_session.py:1345-1373, pipeline
 * tools/buddy-codegen/compile_pipeline.py:207-220): dense tensor-core GEMMs
 * (b200_gemm_w8) for int8 projections, causal attention over the cache rows
 * written so far (frontend/Python/ops/tosa.py:4326-4700), K/V rows left in the
 * device cache.  logits_host: [n_tokens, vocab] when all_rows != 0, else
 * [vocab] (the last row), or NULL.  next_token (optional): first maximum of
 * the last row.  Single-GPU sessions. */
int b200_model_prefill(b200_model *m, const int32_t *tokens, int n_tokens,
                       int pos0, float *logits_host, int all_rows,
                       int *next_token);

/* Batched decode over a paged KV cache: many sequences of different lengths
 * advance one token per step through the dense tensor-core GEMMs (the weights
 * are read once per step for all of them).  buddy-mlir has no paged cache and
 * no batched decode entry; per sequence the arithmetic is that of
 * b200_model_decode over a contiguous cache (the parity tests compare every
 * sequence with the CPU restatement run on its own).  Pages: page_size
 * positions of all kv heads, per layer and K/V buffer [n_pages][kv_heads]
 * [page_size][head_dim] f32, handed out from a free list as sequences grow and
 * returned by b200_batch_remove; a sequence holds at most max_context
 * positions.  The batch borrows the model's weights and scratch: use one batch
 * (or the model's own session calls) at a time. */
typedef struct b200_batch b200_batch;
int b200_batch_create(b200_model *m, int max_seqs, int page_size, int n_pages,
                      int max_context, b200_batch **out);
void b200_batch_destroy(b200_batch *b);
int b200_batch_add(b200_batch *b, int *seq);
int b200_batch_remove(b200_batch *b, int seq);
int b200_batch_length(const b200_batch *b, int seq);
int b200_batch_free_pages(const b200_batch *b);
/* Append n prompt tokens to one sequence (one dense pass); logits_host: the
 * last row [vocab] or NULL. */
int b200_batch_prefill(b200_batch *b, int seq, const int32_t *tokens, int n,
                       float *logits_host, int *next_token);
/* One token for each of n distinct sequences; logits_host [n, vocab] or NULL,
 * next_tokens [n] (first maximum per row) or NULL. */
int b200_batch_decode(b200_batch *b, int n, const int *seqs,
                      const int32_t *tokens, float *logits_host,
                      int32_t *next_tokens);
float b200_batch_last_ms(const b200_batch *b);
/* Timing of the last decode/generate call, CUDA events on the session's
 * stream (ms). */
float b200_model_last_ms(const b200_model *m);
/* Algorithmic HBM bytes one decode step reads at context length ctx
 * (weights + scales + small tensors + embedding row + live KV rows). */
int64_t b200_model_step_bytes(const b200_model *m, int ctx);
int b200_model_kernels_per_step(const b200_model *m);
/* 1 when decode steps run as the single persistent kernel (batch 1, every
 * linear layer int8, one GPU); 0 when they replay the multi-kernel CUDA graph.
 * The environment variable BUDDY_B200_DECODE=graph forces the graph. */
int b200_model_uses_persistent_kernel(const b200_model *m);
/* Diagnostic: set the persistent kernel's launch counter (the base of the 32-bit
 * tags its CTAs exchange activations under), e.g. just below the wrap of the tag
 * space at 2^32 / (8 * (n_layers + 3)) launches, to cross it in a test. */
int b200_model_set_launch_counter(b200_model *m, uint32_t launches);
/* How the sums of a tensor-parallel model's row-parallel projections are formed:
 * 0 = single GPU, 1 = NCCL all-reduce, 2 = every rank's GEMV stores its partial
 * results straight into all ranks' staging buffers over NVLink (tagged pairs),
 * a small kernel adds them up in rank order. */
int b200_model_tp_sum_kind(const b200_model *m);
/* Tuning aid: with BUDDY_B200_TRACE=<stride> set at load time, every
 * stride-th CTA of the persistent kernel records the SM clock at each phase
 * boundary of the last step: host[cta/stride][layer][32]. Returns the number
 * of values copied (negative on error). */
int b200_model_read_trace(b200_model *m, long long *host, int64_t capacity);
/* Session handle -> device pointers, for tests. */
float *b200_model_kv_ptr(b200_model *m, int buffer);
/* KV overflow on the device-resident cache; see b200_kv_overflow. */
int b200_model_kv_overflow(b200_model *m, int position, int keep, float theta,
                           int *new_position);

/* Tensor parallel plumbing: the caller creates an NCCL unique id
 * (b200_tp_unique_id on rank 0), distributes the 128 bytes with its own
 * transport, and every rank calls b200_tp_init before b200_model_create. */
int b200_tp_unique_id(void *id128);
int b200_tp_init(const void *id128, int rank, int size);
void b200_tp_shutdown(void);

/* ------------------------------------------------------------------------
 * Payload section of a buddy-mlir .rax package, without FlatBuffers
 * (runtime/include/buddy/runtime/core/ModelManifest.h:124-145, 202-310):
 * [manifest "RAX0"][payload blobs][index "RAXIDX01"][64-byte footer
 * "RAXPAY01"].  The manifest is not parsed; the payload entries are named
 * (weight blobs keep their file names), so the weights of a packaged model can
 * be read straight from the package.  A package without a payload opens with
 * zero entries.  Host code; no device is needed.
 * ---------------------------------------------------------------------- */
typedef struct b200_rax b200_rax;
int b200_rax_open(const char *path, b200_rax **out);
void b200_rax_close(b200_rax *r);
int b200_rax_count(const b200_rax *r);
uint64_t b200_rax_manifest_bytes(const b200_rax *r);
int b200_rax_entry(const b200_rax *r, int i, char *name, int name_cap,
                   int *kind, uint64_t *offset, uint64_t *size);
/* Index of the first entry whose name ends with name_suffix, or -1. */
int b200_rax_find(const b200_rax *r, const char *name_suffix);
int b200_rax_read(const b200_rax *r, int i, void *dst, uint64_t bytes);

#ifdef __cplusplus
}
#endif
#endif
