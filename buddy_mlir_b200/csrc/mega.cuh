// Parameters of the persistent decode-step kernel (mega.cu).
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace b200 {

constexpr int kMegaThreads = 512;      // 16 warps
constexpr int kMegaMaxSlots = 16;
constexpr int kMegaMaxLayerStages = 128;  // ring stages one CTA consumes per layer
constexpr int kMegaTraceSlots = 64;    // trace points per (CTA, layer)
constexpr int kMegaTrailer = 16;       // bytes per row behind every stage: scale, bias, sum of the row's weights
constexpr int kMegaBlockRows = 16;     // rows of one tensor-core row block (the m of mma.m16n8k32)
constexpr int kMegaAccBlocks = 16;     // row blocks per CTA of a projection whose K is split over warps

// One projection.  A CTA's rows are cut into blocks of 16; a block's K bytes are
// cut into `nks` slices of `slice_bytes`; one ring stage = (block, slice) =
// [rows x slice_bytes of int8 weights][rows x 16-byte trailer].  A stage is
// worked on by `nkw` warps, each taking 1/nkw of the slice's k range.
struct MegaPhase {
  int K, N;
  int slice_bytes;  // multiple of 64
  int nks;          // K / slice_bytes
  int nkw;          // warps per stage; divides slice_bytes / 64
  int unit;         // rows are dealt to CTAs in multiples of this (2 keeps gate/up pairs together)
  int swizzle;      // 4 when slice_bytes is a multiple of 128 (odd rows swap the halves of every 128 bytes), else 0
};

struct MegaParams {
  const uint8_t *stream;       // every CTA's private weight stream, back to back
  const int64_t *cta_off;      // [grid] start of each CTA's stream
  MegaPhase phase[5];          // qkv, o, gate|up (interleaved pairs), down, lm_head
  int H, F, V, qh, kvh, L, max_len, splits;
  int slots, slot_bytes;
  int xs_bytes;                // shared-memory scratch: activation planes / attention staging
  int plane_stride;            // bytes between the three activation planes
  float eps;
  const float *embed, *inv_freq, *final_norm;
  const float *const *lvec;    // [4*L]: input norm, post norm, q_norm, k_norm (or null)
  float *const *kv;            // [2*L] cache buffers, K at even index
  // tagged (value, tag) activation buffers, two copies each (layer parity)
  uint2 *ll_qkv;               // [2][QD + 2*KD]
  uint2 *ll_attn;              // [2][QD]
  uint2 *ll_xb;                // [2][H]   residual stream after attention
  uint2 *ll_mid;               // [2][F]   silu(gate) * up
  uint2 *ll_xa;                // [2][H]   residual stream after the MLP
  uint2 *ll_part;              // [2][qh][splits][D + 2] attention split partials
  uint2 *ll_cand;              // [grid][2] per-CTA argmax candidates (value, index)
  float *logits;
  float *kv_stage;             // [2*L][kvh*D] rows written this step
  int32_t *state;              // token, pos, next, count, launches completed
  int32_t *history;
  int history_cap;
  int *error;                  // 0, or the code of the first wait that gave up
  long long *trace;            // optional [grid/stride][L+1][kMegaTraceSlots] SM-clock timeline, or null
  int trace_stride;
};

// Bytes of the (block, slice) stages of `nrows` rows of a projection.
__host__ __device__ inline int64_t mega_rows_bytes(const MegaPhase &ph, int nrows) {
  // every stage carries its rows' trailers
  return (int64_t)nrows * ph.K + (int64_t)nrows * kMegaTrailer * ph.nks;
}

int mega_build_rows(const void *packed, int K, int n_rows, int row_stride, int row_phase,
                    int N_total, const MegaPhase &ph, const float *scale, const float *bias,
                    int grid_ctas, const int64_t *cta_phase_off_dev, void *stream_buf,
                    cudaStream_t st);
size_t mega_fixed_shared_bytes();
int mega_launch(const MegaParams &p, int grid, size_t smem, cudaStream_t st);

} // namespace b200
