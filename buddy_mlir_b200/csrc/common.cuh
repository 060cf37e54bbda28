// Shared helpers for the sm_100a kernels: status handling, launch counting,
// warp reductions and the packed-row index map.
#pragma once
#include <cuda_fp16.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <atomic>
#include <cstdarg>
#include <cstdio>

#include "../../include/buddy_b200.h"

namespace b200 {

// Message of the calling thread's last failure.
char *error_buffer();
int fail(int code, const char *fmt, ...);
extern std::atomic<uint64_t> g_launches;
inline void count_launch(uint64_t n = 1) {
  g_launches.fetch_add(n, std::memory_order_relaxed);
}
int ensure_device();

#define B200_CUDA(expr)                                                        \
  do {                                                                         \
    cudaError_t e_ = (expr);                                                   \
    if (e_ != cudaSuccess)                                                     \
      return ::b200::fail(B200_ECUDA, "%s: %s (%s:%d)", #expr,                 \
                          cudaGetErrorString(e_), __FILE__, __LINE__);         \
  } while (0)

#define B200_LAUNCH_CHECK()                                                    \
  do {                                                                         \
    ::b200::count_launch();                                                    \
    cudaError_t e_ = cudaGetLastError();                                       \
    if (e_ != cudaSuccess)                                                     \
      return ::b200::fail(B200_ECUDA, "kernel launch: %s (%s:%d)",             \
                          cudaGetErrorString(e_), __FILE__, __LINE__);         \
  } while (0)

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1)
    v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1)
    v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// ---- tensor-parallel sum without a collective library -----------------------
// A row-parallel projection (o, down) leaves a partial sum on every rank.  Its
// GEMV stores each partial result straight into the staging buffers of ALL ranks
// (plain 8-byte peer stores over NVLink) as (value, tag) pairs; the tag numbers
// the reduction (decode step x reductions per step + index), so a receiver just
// polls for the tag: the data's arrival is the synchronisation.  Four regions
// are used in turn; a rank cannot run more than one reduction ahead of the
// slowest one, so a region is never overwritten before it has been read.
constexpr int kTpMaxRanks = 8;
constexpr int kTpRegions = 4;
struct TpPush {
  uint2 *peer[kTpMaxRanks];   // staging buffer of every rank: [kTpRegions][ranks][H] pairs
  int ranks, rank, H;
  const int32_t *step;        // device counter of decode steps (the same on every rank)
  int index, per_step;        // which reduction of the step this is, and how many there are
};
int gemv_run(const b200_weight *w, const b200_gemv_args *a, const TpPush *push, cudaStream_t stream);
__device__ __forceinline__ void tagged_store(uint2 *p, float v, uint32_t tag) {
  asm volatile("st.volatile.global.v2.u32 [%0], {%1, %2};" ::"l"(p), "r"(__float_as_uint(v)),
               "r"(tag)
               : "memory");
}
// two neighbouring pairs in one 16-byte store (p 16-byte aligned): half the packets on the link
__device__ __forceinline__ void tagged_store2(uint2 *p, float v0, float v1, uint32_t tag) {
  asm volatile("st.volatile.global.v4.u32 [%0], {%1, %2, %3, %4};" ::"l"(p), "r"(__float_as_uint(v0)), "r"(tag),
               "r"(__float_as_uint(v1)), "r"(tag)
               : "memory");
}
__device__ __forceinline__ uint2 tagged_load(const uint2 *p) {
  uint2 v;
  asm volatile("ld.volatile.global.v2.u32 {%0, %1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(p) : "memory");
  return v;
}

// ---- packed-row index map -------------------------------------------------
// A packed row is a sequence of blocks of up to 32 sixteen-byte units.  Unit
// (lane) l of a block holds G groups of 4 consecutive k; group j of lane l
// covers k = blk_k0 + j*(Bs/G) + 4*l .. +3, where Bs is the block's element
// count.  G = 4 for int8 (4 B per group), 8 for int4 (2 B per group), 1 for
// f32 (16 B per group).
__host__ __device__ inline int elems_per_unit(int kind) {
  return kind == B200_W_I8 ? 16 : (kind == B200_W_U4 ? 32 : 4);
}
__host__ __device__ inline int groups_per_unit(int kind) {
  return kind == B200_W_I8 ? 4 : (kind == B200_W_U4 ? 8 : 1);
}
__host__ __device__ inline int64_t packed_k(int kind, int64_t K) {
  const int e = elems_per_unit(kind);
  return (K + e - 1) / e * e;
}
__host__ __device__ inline int64_t packed_row_bytes(int kind, int64_t K) {
  return packed_k(kind, K) / elems_per_unit(kind) * 16;
}
// Byte offset (and nibble for U4) of element k inside a packed row.
__host__ __device__ inline int64_t packed_offset(int kind, int64_t K, int64_t k,
                                                 int *nibble) {
  const int e = elems_per_unit(kind), G = groups_per_unit(kind);
  const int64_t Kp = packed_k(kind, K);
  const int64_t blk_elems = 32 * (int64_t)e;
  const int64_t b = k / blk_elems;
  const int64_t k0 = b * blk_elems;
  const int64_t Bs = (Kp - k0) < blk_elems ? (Kp - k0) : blk_elems;
  const int64_t q = Bs / G;  // k distance between a lane's groups
  const int64_t kk = k - k0;
  const int64_t j = kk / q, r = kk % q;
  const int64_t l = r / 4, el = r % 4;
  const int64_t unit_off = b * 512 + l * 16;
  if (nibble)
    *nibble = 0;
  if (kind == B200_W_I8)
    return unit_off + j * 4 + el;
  if (kind == B200_W_U4) {
    if (nibble)
      *nibble = (int)(el & 1);
    return unit_off + j * 2 + el / 2;
  }
  return unit_off + el * 4; // f32: one group of 4 floats, byte offset
}

// prefill.cu: the row-batched small ops around the dense GEMMs
int embed_rows_launch(const float *table, const int32_t *tokens_dev, float *x, int64_t H, int M, cudaStream_t st);
int rope_kv_rows_launch(float *qkv, int64_t ld, float *k_cache, float *v_cache, const float *inv_freq,
                        const float *q_norm, const float *k_norm, float eps, int q_heads, int kv_heads, int D,
                        int max_len, int pos0, int M, cudaStream_t st);
int gqa_prefill_launch(const float *qkv, int64_t ld, const float *kc, const float *vc, float *out, int64_t ldo,
                       int q_heads, int kv_heads, int D, int max_len, int pos0, int M, cudaStream_t st);

int rope_kv_paged_launch(float *qkv, int64_t ld, float *k_pool, float *v_pool, const float *inv_freq,
                         const float *q_norm, const float *k_norm, float eps, int q_heads, int kv_heads, int D,
                         int page, const int32_t *row_seq, const int32_t *row_pos, const int32_t *block_table,
                         int table_stride, int M, cudaStream_t st);
int gqa_paged_launch(const float *qkv, int64_t ld, const float *k_pool, const float *v_pool, float *out, int64_t ldo,
                     int q_heads, int kv_heads, int D, int page, const int32_t *row_seq, const int32_t *row_pos,
                     const int32_t *block_table, int table_stride, int M, float *scratch, int scratch_rows,
                     int max_context, cudaStream_t st);
int gqa_paged_prefill_launch(const float *qkv, int64_t ld, const float *k_pool, const float *v_pool, float *out,
                             int64_t ldo, int q_heads, int kv_heads, int D, int page, const int32_t *seq_table,
                             int pos0, int M, int max_context, cudaStream_t st);
int64_t gqa_paged_scratch_floats(int rows, int q_heads, int D, int max_context);
// gemm_tc.cu: b200_gemm_w8a8 with the residual sum or the SiLU pair folded into the store
int gemm_w8a8_fused(const b200_weight *w, const float *A, int M, int64_t lda, float *C, int64_t ldc,
                    const float *residual, int64_t ldr, int silu_pairs, void *workspace, int64_t workspace_bytes,
                    cudaStream_t stream);
int argmax_rows_launch(const float *v, int64_t n, int rows, int32_t *out, cudaStream_t st);

__device__ __forceinline__ float load_as_float(const void *p, int dtype,
                                               int64_t i) {
  if (dtype == B200_F32)
    return ((const float *)p)[i];
  if (dtype == B200_F16)
    return __half2float(((const __half *)p)[i]);
  return __bfloat162float(((const __nv_bfloat16 *)p)[i]);
}

} // namespace b200
