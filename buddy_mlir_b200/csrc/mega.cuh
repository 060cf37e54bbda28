// Parameters of the persistent decode-step kernel (mega.cu).
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace b200 {

constexpr int kMegaThreads = 512;      // 16 warps
constexpr int kMegaMaxSlots = 16;
constexpr int kMegaMaxLayerStages = 96;   // ring stages one CTA consumes per layer
constexpr int kMegaTraceSlots = 64;   // trace points per (CTA, layer)
constexpr int kMegaMaxMid = 128;       // SiLU-gated MLP values one CTA produces (and consumes) per layer
constexpr int kMegaTrailer = 16;       // bytes appended to every streamed row: scale, bias

struct MegaPhase {
  int K, N;
  int row_bytes;   // K + trailer
  int rps;         // rows per ring slot (even)
  int mode;        // 0: rows (a warp owns whole rows of a stage); 2: columns
  int unit;        // rows are dealt to CTAs in multiples of this (2 keeps gate/up pairs together)
};

struct MegaParams {
  const uint8_t *stream;       // every CTA's private weight stream, back to back
  const int64_t *cta_off;      // [grid] start of each CTA's stream
  // qkv, o, gate|up (interleaved pairs), down (COLUMNS: K = N = ffn columns dealt to the CTAs,
  // row_bytes = hidden bytes per column, no trailer), lm_head
  MegaPhase phase[5];
  int H, F, V, qh, kvh, L, max_len, splits;
  int slots, slot_bytes;
  int xs_floats;               // shared-memory staging area (activations, attention and column scratch)
  float eps;
  const float *embed, *inv_freq, *final_norm;
  const float *const *lvec;    // [4*L]: input norm, post norm, q_norm, k_norm (or null)
  float *const *kv;            // [2*L] cache buffers, K at even index
  // tagged (value, tag) activation buffers, two copies each (layer parity)
  uint2 *ll_qkv;               // [2][QD + 2*KD]
  uint2 *ll_attn;              // [2][QD]
  uint2 *ll_xb;                // [2][H]   residual stream after attention
  uint2 *ll_dpart;             // [2][grid][H] per-CTA partial sums of the down projection
  const float *const *down_scale;   // [L] per-channel scales of the down projection
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

int mega_build_rows(const void *packed, int K, int n_rows, int row_stride, int row_phase,
                    int N_total, int unit, const float *scale, const float *bias, int grid_ctas,
                    int row_bytes, const int64_t *cta_phase_off_dev, void *stream_buf,
                    cudaStream_t st);
int mega_build_cols(const void *packed, int K, int H, const int32_t *koff_dev, int grid_ctas,
                    const int64_t *cta_phase_off_dev, void *stream_buf, cudaStream_t st);
size_t mega_fixed_shared_bytes();
int mega_launch(const MegaParams &p, int grid, size_t smem, cudaStream_t st);

} // namespace b200
