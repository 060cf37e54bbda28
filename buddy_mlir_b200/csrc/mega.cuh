// Parameters of the persistent decode-step kernel (mega.cu).
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace b200 {

constexpr int kMegaThreads = 288;      // 8 consumer warps + 1 producer warp
constexpr int kMegaMaxSlots = 16;
constexpr int kMegaMaxRowsB = 64;      // rows of a shared-row phase finalised per flush
constexpr int kMegaTrailer = 16;       // bytes appended to every streamed row: scale, bias

struct MegaPhase {
  int K, N;
  int row_bytes;   // K + trailer
  int rps;         // rows per ring slot
  int mode;        // 0: a warp owns a row; 1: all consumer threads share each row
};

struct MegaParams {
  const uint8_t *stream;       // every CTA's private weight stream, back to back
  const int64_t *cta_off;      // [grid] start of each CTA's stream
  MegaPhase phase[5];          // qkv, o, gate|up, down, lm_head
  int H, F, V, D, qh, kvh, L, max_len, splits;
  int slots, slot_bytes;
  float eps;
  const float *embed, *inv_freq, *final_norm;
  const float *const *lvec;    // [4*L]: input norm, post norm, q_norm, k_norm (or null)
  float *const *kv;            // [2*L] cache buffers, K at even index
  float *xa, *xb, *qkv, *attn, *gu, *logits;
  float *attn_part;            // split partials [qh][splits][D+2]
  unsigned *attn_count;        // [kvh] arrival counters, zero between launches
  float *kv_stage;             // [2*L][kvh*D] rows written this step
  int32_t *state;              // token, pos, next, count, launches completed
  int32_t *history;
  int history_cap;
  float *cand_val;             // [grid] per-CTA argmax candidates
  int *cand_idx;
  unsigned *barrier;           // grid barrier counter: monotonic, never reset
  int *error;                  // 0, or the code of the first wait that gave up
  long long *trace;            // optional [grid/stride][L+1][12] SM-clock timeline, or null
  int trace_stride;
};

int mega_build_rows(const void *packed, int K, int n_rows, int row_offset, int N_total,
                    const float *scale, const float *bias, int grid_ctas, int row_bytes,
                    const int64_t *cta_phase_off_dev, void *stream_buf, cudaStream_t st);
size_t mega_shared_bytes(int slots, int slot_bytes);
int mega_launch(const MegaParams &p, int grid, size_t smem, cudaStream_t st);

} // namespace b200
