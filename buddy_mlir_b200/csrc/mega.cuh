// Parameters of the persistent decode-step kernel (mega.cu).
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace b200 {

constexpr int kMegaThreads = 512;      // 16 warps
constexpr int kMegaMaxSlots = 16;
constexpr int kMegaMaxLayerStages = 96;   // ring stages one CTA consumes per layer
constexpr int kMegaTraceSlots = 64;   // trace points per (CTA, layer)
constexpr int kMegaTrailer = 16;       // bytes appended to every streamed row: scale, bias

struct MegaPhase {
  int K, N;
  int row_bytes;   // K + trailer
  int rps;         // rows per ring stage
  int mode;        // unused (0)
  int unit;        // rows are dealt to CTAs in multiples of this (2 keeps gate/up pairs together)
};

struct MegaParams {
  const uint8_t *stream;       // every CTA's private weight stream, back to back
  const int64_t *cta_off;      // [grid] start of each CTA's stream
  MegaPhase phase[5];          // qkv, o, gate|up (interleaved pairs), down, lm_head
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

int mega_build_rows(const void *packed, int K, int n_rows, int row_stride, int row_phase,
                    int N_total, int unit, const float *scale, const float *bias, int grid_ctas,
                    int row_bytes, const int64_t *cta_phase_off_dev, void *stream_buf,
                    cudaStream_t st);
size_t mega_fixed_shared_bytes();
int mega_launch(const MegaParams &p, int grid, size_t smem, cudaStream_t st);

} // namespace b200
