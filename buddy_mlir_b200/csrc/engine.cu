// Device-resident decode session: packed weights, KV cache, and one CUDA graph
// holding every kernel of a decode step.
//
// This is the body that stands behind _mlir_ciface_forward_decode: the op
// sequence is the decode subgraph of
// examples/BuddyDeepSeekR1/subgraph0_decode_simplify.mlir:46-260 (+ tail); the
// weight blobs are walked in the order the reference packs them
// (frontend/Python/graph/graph.py:836-863,
// frontend/Python/graph/transform/quantization/quantize.py:577-589); tensor
// parallel sharding follows examples/BuddyTensorParallel (column-parallel
// q/k/v/gate/up, row-parallel o/down, sum after each, vocab-sharded lm_head;
// buddy-deepseek-r1-distributed.cpp:521-617) with NCCL in place of MPI.
#include "common.cuh"
#include "mega.cuh"

#include <dlfcn.h>

#include <algorithm>
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <string>
#include <vector>

namespace b200 {

int gqa_decode_launch(const float *q, const float *kc, const float *vc,
                      float *out, float *scratch, int q_heads, int kv_heads,
                      int D, int max_len, int splits, const int32_t *pos,
                      cudaStream_t st);
int quantize_row_launch(const float *x, const float *norm_w, float eps, int64_t K, uint32_t *q, float *scale,
                        cudaStream_t st);
int gemv_i8_launch(const b200_weight *w, const uint32_t *q, const float *act_scale, const float *residual, float *y,
                   int silu_pairs, cudaStream_t st);
bool gemv_i8_fusable(int64_t K);
int gemv_i8_fused_launch(const b200_weight *w, const float *x, const float *norm_w, float eps, const float *residual,
                         float *y, int silu_pairs, cudaStream_t st);
int rope_kv_write_launch(float *q, float *k, const float *v, float *k_cache,
                         float *v_cache, const float *inv_freq,
                         const float *q_norm, const float *k_norm, float eps,
                         int q_heads, int kv_heads, int D, int max_len,
                         const int32_t *pos, float *k_stage, float *v_stage,
                         cudaStream_t st);

// ---- NCCL, bound at run time so single-GPU users need no NCCL ---------------
struct Id128 {  // ncclUniqueId: 128 opaque bytes, passed by value
  char bytes[128];
};
struct Nccl {
  void *lib = nullptr;
  void *comm = nullptr;
  int rank = 0, size = 1;
  int (*GetUniqueId)(void *) = nullptr;
  int (*CommInitRank)(void **, int, Id128, int) = nullptr;
  int (*AllReduce)(const void *, void *, size_t, int, int, void *,
                   cudaStream_t) = nullptr;
  int (*AllGather)(const void *, void *, size_t, int, void *,
                   cudaStream_t) = nullptr;
  int (*CommDestroy)(void *) = nullptr;
  const char *(*GetErrorString)(int) = nullptr;
};
static Nccl g_nccl;
constexpr int kNcclFloat = 7;  // ncclFloat32
constexpr int kNcclSum = 0;    // ncclSum

static int nccl_bind() {
  if (g_nccl.lib)
    return B200_OK;
  void *lib = dlopen("libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
  if (!lib)
    return fail(B200_ESTATE, "cannot load libnccl.so.2: %s", dlerror());
  g_nccl.lib = lib;
#define B200_SYM(field, name)                                                  \
  *(void **)(&g_nccl.field) = dlsym(lib, name);                                \
  if (!g_nccl.field)                                                           \
    return fail(B200_ESTATE, "libnccl.so.2 lacks %s", name);
  B200_SYM(GetUniqueId, "ncclGetUniqueId")
  B200_SYM(CommInitRank, "ncclCommInitRank")
  B200_SYM(AllReduce, "ncclAllReduce")
  B200_SYM(AllGather, "ncclAllGather")
  B200_SYM(CommDestroy, "ncclCommDestroy")
  B200_SYM(GetErrorString, "ncclGetErrorString")
#undef B200_SYM
  return B200_OK;
}
#define B200_NCCL(expr)                                                        \
  do {                                                                         \
    int r_ = (expr);                                                           \
    if (r_ != 0)                                                               \
      return fail(B200_ECUDA, "%s: %s", #expr, g_nccl.GetErrorString(r_));     \
  } while (0)

// x += part (after the tensor-parallel sum)
__global__ void add_inplace_kernel(float *x, const float *part, int n) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n)
    x[i] = __fadd_rn(x[i], part[i]);
}
// x[n] += sum over ranks (in rank order, the same on every rank) of the partial
// results that the ranks' GEMVs pushed into this rank's staging buffer.  Every
// wait is bounded (poll count and 10 s of wall time: the ranks are separate
// processes that enter a step at slightly different times); on expiry the
// kernel records code 500 in *err, and later waits of the step fall through.
__global__ void tp_reduce_add_kernel(float *x, const uint2 *buf, int H, int ranks,
                                     const int32_t *step, int index, int per_step, int *err) {
  const int n = blockIdx.x * blockDim.x + threadIdx.x;
  if (n >= H)
    return;
  const uint32_t seq = (uint32_t)(*step) * per_step + index, tag = seq + 1u;
  const uint2 *src = buf + (size_t)(seq % kTpRegions) * ranks * H + n;
  float sum = x[n];
  // every rank's slot is requested before the first one is looked at: the loads overlap instead
  // of costing one memory round trip per rank
  uint2 v[kTpMaxRanks];
#pragma unroll
  for (int r = 0; r < kTpMaxRanks; ++r)
    if (r < ranks)
      v[r] = tagged_load(src + (size_t)r * H);
#pragma unroll
  for (int r = 0; r < kTpMaxRanks; ++r) {
    if (r >= ranks)
      break;
    if (v[r].y != tag) {
      const uint2 *p = src + (size_t)r * H;
      unsigned long long t0 = 0;
      for (uint32_t it = 1; v[r].y != tag; ++it) {
        if ((it & 0xFF) == 0) {
          unsigned long long t;
          asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
          if (t0 == 0)
            t0 = t;
          if (*(volatile int *)err != 0 || t - t0 > 10000000000ull || it > (1u << 30)) {
            atomicCAS(err, 0, 500);
            break;
          }
        }
        __nanosleep(100);
        v[r] = tagged_load(p);
      }
    }
    sum = __fadd_rn(sum, __uint_as_float(v[r].x));   // rank order: every rank forms the same sum
  }
  x[n] = sum;
}
// One-off check of the peer mappings before they are used: every rank stores a
// marker into every rank's buffer (behind the staging regions) and waits, at most
// two seconds, for everybody's marker in its own.  *ok is cleared on expiry.
__global__ void tp_handshake_kernel(TpPush push, size_t at, int *ok) {
  const int t = threadIdx.x;
  const uint32_t tag = 0xFFFFFF00u;
  if (t < push.ranks)
    tagged_store(push.peer[t] + at + push.rank, (float)(push.rank + 1), tag);
  if (t < push.ranks) {
    const uint2 *p = push.peer[push.rank] + at + t;
    unsigned long long t0;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t0));
    for (uint32_t it = 0; it < (1u << 28); ++it) {
      if (tagged_load(p).y == tag)
        return;
      unsigned long long now;
      asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(now));
      if (now - t0 > 2000000000ull)
        break;
      __nanosleep(200);
    }
    *ok = 0;
  }
}
// Greedy token of a vocabulary-sharded lm_head without gathering the logits: every rank
// holds the first maximum of its own shard; it stores (value, tag) and (global index, tag)
// into every rank's buffer, waits (bounded) for all ranks' pairs and keeps the largest
// value, the lowest index among equals: the MAXLOC reduction of
// examples/BuddyTensorParallel/buddy-deepseek-r1-distributed.cpp:211-223,602-613.
// One warp; lane t talks to rank t.  Two slots are used in turn (step parity).
__global__ void tp_argmax_kernel(TpPush push, size_t at, const float *shard, const int32_t *local_idx,
                                 int shard_len, int32_t *next, int *err) {
  const int t = threadIdx.x;
  const uint32_t step = (uint32_t)(*push.step);
  const uint32_t tag = 0x40000000u + step;
  const size_t base = at + (size_t)(step & 1u) * 2 * push.ranks;
  const int li = *local_idx;
  if (t < push.ranks) {
    tagged_store(push.peer[t] + base + 2 * push.rank, shard[li], tag);
    tagged_store(push.peer[t] + base + 2 * push.rank + 1, __int_as_float(li + push.rank * shard_len), tag);
  }
  float bv = -INFINITY;
  int bi = 0x7fffffff;
  if (t < push.ranks) {
    const uint2 *p = push.peer[push.rank] + base + 2 * t;
    uint2 v = tagged_load(p), w = tagged_load(p + 1);
    unsigned long long t0 = 0;
    for (uint32_t it = 1; v.y != tag || w.y != tag; ++it) {
      if ((it & 0xFF) == 0) {
        unsigned long long now;
        asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(now));
        if (t0 == 0)
          t0 = now;
        if (*(volatile int *)err != 0 || now - t0 > 10000000000ull || it > (1u << 30)) {
          atomicCAS(err, 0, 501);
          break;
        }
      }
      v = tagged_load(p);
      w = tagged_load(p + 1);
    }
    bv = __uint_as_float(v.x);
    bi = (int)w.x;
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
    const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
    if (ov > bv || (ov == bv && oi < bi)) {
      bv = ov;
      bi = oi;
    }
  }
  if (t == 0)
    *next = bi == 0x7fffffff ? 0 : bi;
}
// end of a step: feed the argmax back and advance the position
__global__ void advance_kernel(int32_t *token, int32_t *pos,
                               const int32_t *next, int32_t *history,
                               int32_t *count, int cap, int32_t *steps_done) {
  if (threadIdx.x == 0 && blockIdx.x == 0) {
    *steps_done = *steps_done + 1;   // numbers the tensor-parallel reductions
    const int c = *count;
    if (c < cap)
      history[c] = *next;
    *count = c + 1;
    *token = *next;
    *pos = *pos + 1;
  }
}

struct DevLinear {
  b200_weight w{};
  void *w_buf = nullptr, *scale_buf = nullptr;
  float *bias_buf = nullptr;
  bool set = false;
  int64_t bytes() const {
    if (!set)
      return 0;
    int64_t b = packed_row_bytes(w.kind, w.K) * w.N;
    if (w.scale) {
      const int64_t ng =
          (w.kind == B200_W_U4 && w.group > 0 && w.group < w.K) ? w.K / w.group : 1;
      b += w.N * ng * (w.scale_dtype == B200_F32 ? 4 : 2);
    }
    if (w.bias)
      b += w.N * 4;
    return b;
  }
  void release() {
    cudaFree(w_buf);
    cudaFree(scale_buf);
    cudaFree(bias_buf);
    w_buf = scale_buf = nullptr;
    bias_buf = nullptr;
    set = false;
  }
};

struct Layer {
  float *in_norm = nullptr, *post_norm = nullptr, *q_norm = nullptr,
        *k_norm = nullptr;
  DevLinear q, k, v, o, gate, up, down;
  DevLinear qkv, gateup;  // fused at finalize
};

} // namespace b200

using namespace b200;

struct b200_model {
  b200_model_config cfg{};
  int tp = 1, rank = 0;
  int qh = 0, kvh = 0, ffn = 0, vocab = 0;  // local (sharded) sizes
  float *embed = nullptr, *inv_freq = nullptr, *final_norm = nullptr;
  std::vector<Layer> layers;
  DevLinear lm_head;
  std::vector<float *> kv;
  float **kv_dev = nullptr;
  float *x = nullptr, *qkv = nullptr, *attn = nullptr, *mid = nullptr,
        *part = nullptr, *logits = nullptr, *logits_shard = nullptr;
  float *attn_scratch = nullptr, *argmax_scratch = nullptr;
  float *kv_stage = nullptr;  // [2*layers][kv_heads*D]: the rows written this step
  int32_t *d_state = nullptr;  // token, pos, next, count, launches, -, error, -
  int32_t *d_history = nullptr;
  int history_cap = 0;
  int splits = 1;
  cudaStream_t stream = nullptr;
  cudaGraph_t graph = nullptr;
  cudaGraphExec_t exec = nullptr;
  cudaEvent_t ev0 = nullptr, ev1 = nullptr;
  float last_ms = 0.f;
  int kernels_per_step = 0;
  bool finalized = false;
  float *h_logits_pinned = nullptr;
  float *h_rows_pinned = nullptr;   // this step's K/V rows, fetched together with the logits
  bool rows_fresh = false;
  int32_t *h_state_pinned = nullptr;
  // persistent decode-step kernel (batch 1, int8): see mega.cu
  bool mega = false;
  MegaParams mp{};
  int mega_grid = 0;
  size_t mega_smem = 0;
  int64_t mega_stream_bytes = 0;
  uint8_t *mega_stream = nullptr;
  int64_t *mega_offsets = nullptr;   // [(4L+1)+1][grid]: per-phase and per-CTA stream offsets
  const float **lvec_dev = nullptr;
  uint2 *ll_buf = nullptr;           // tagged activation buffers
  long long *d_trace = nullptr;
  // prefill (many rows at once): activations of all rows, grown on demand
  float *pf_x = nullptr, *pf_qkv = nullptr, *pf_att = nullptr, *pf_mid = nullptr, *pf_logits = nullptr;
  float *pf_norm = nullptr;   // W8A8 only: the normalised rows of a projection
  bool act_int8 = false;   // the w8a8 variant: int8 projections quantise their activations per call
  uint32_t *q_row = nullptr;   // decode: the quantised activation row of the current projection
  float *q_scale = nullptr;    //         and its scale
  cudaGraph_t graph_q = nullptr;      // the decode step with int8 activations, captured on first use
  cudaGraphExec_t exec_q = nullptr;
  int kernels_per_step_q = 0;
  void *pf_ws = nullptr;
  int32_t *pf_tokens = nullptr;
  int pf_rows = 0, pf_logit_rows = 0;
  int64_t pf_ws_bytes = 0;
  // tensor-parallel sums by peer stores (see TpPush): this rank's staging buffer and everybody's
  uint2 *tp_ll = nullptr;
  void *tp_opened[kTpMaxRanks] = {};
  TpPush tp_push{};   // ranks == 0: the NCCL all-reduce is used instead
  size_t tp_argmax_at = 0;   // pair offset of the (value, index) exchange slots inside the staging buffers
};

namespace {

int dev_alloc(void **p, size_t bytes) {
  cudaError_t e = cudaMalloc(p, bytes ? bytes : 16);
  if (e != cudaSuccess) {
    (void)cudaGetLastError();
    return fail(B200_ENOMEM, "cudaMalloc(%zu): %s", bytes, cudaGetErrorString(e));
  }
  return B200_OK;
}

DevLinear *linear_slot(b200_model *m, int layer, int slot) {
  if (slot == B200_T_LM_HEAD)
    return &m->lm_head;
  if (layer < 0 || layer >= (int)m->layers.size())
    return nullptr;
  Layer &L = m->layers[layer];
  switch (slot) {
  case B200_T_Q: return &L.q;
  case B200_T_K: return &L.k;
  case B200_T_V: return &L.v;
  case B200_T_O: return &L.o;
  case B200_T_GATE: return &L.gate;
  case B200_T_UP: return &L.up;
  case B200_T_DOWN: return &L.down;
  default: return nullptr;
  }
}

bool is_row_parallel(int slot) { return slot == B200_T_O || slot == B200_T_DOWN; }

// Concatenate (interleave = 0) or row-interleave (interleave = 1, two parts)
// packed linears that share K and kind into one.
int fuse_linears(const std::vector<DevLinear *> &parts, bool interleave,
                 DevLinear *out, cudaStream_t st) {
  const DevLinear &a = *parts[0];
  int64_t N = 0;
  bool bias = false;
  for (auto *p : parts) {
    if (!p->set || p->w.kind != a.w.kind || p->w.K != a.w.K ||
        p->w.group != a.w.group || p->w.scale_dtype != a.w.scale_dtype)
      return fail(B200_EINVAL, "fused projections must share kind, K and scale type");
    N += p->w.N;
    bias = bias || p->w.bias;
  }
  const int64_t rb = packed_row_bytes(a.w.kind, a.w.K);
  const bool grouped = a.w.kind == B200_W_U4 && a.w.group > 0 && a.w.group < a.w.K;
  const int64_t ng = grouped ? a.w.K / a.w.group : 1;
  const int64_t sb = a.w.scale ? ng * (a.w.scale_dtype == B200_F32 ? 4 : 2) : 0;
  if (int rc = dev_alloc(&out->w_buf, rb * N)) return rc;
  if (sb)
    if (int rc = dev_alloc(&out->scale_buf, sb * N)) return rc;
  if (bias) {
    if (int rc = dev_alloc((void **)&out->bias_buf, N * 4)) return rc;
    B200_CUDA(cudaMemsetAsync(out->bias_buf, 0, N * 4, st));
  }
  int64_t row = 0;
  const size_t np = parts.size();
  for (size_t i = 0; i < np; ++i) {
    const DevLinear &p = *parts[i];
    if (interleave) {
      B200_CUDA(cudaMemcpy2DAsync((char *)out->w_buf + i * rb, np * rb, p.w_buf,
                                  rb, rb, p.w.N, cudaMemcpyDeviceToDevice, st));
      if (sb)
        B200_CUDA(cudaMemcpy2DAsync((char *)out->scale_buf + i * sb, np * sb,
                                    p.scale_buf, sb, sb, p.w.N,
                                    cudaMemcpyDeviceToDevice, st));
      if (p.w.bias)
        B200_CUDA(cudaMemcpy2DAsync(out->bias_buf + i, np * 4, p.bias_buf, 4, 4,
                                    p.w.N, cudaMemcpyDeviceToDevice, st));
    } else {
      B200_CUDA(cudaMemcpyAsync((char *)out->w_buf + row * rb, p.w_buf,
                                rb * p.w.N, cudaMemcpyDeviceToDevice, st));
      if (sb)
        B200_CUDA(cudaMemcpyAsync((char *)out->scale_buf + row * sb, p.scale_buf,
                                  sb * p.w.N, cudaMemcpyDeviceToDevice, st));
      if (p.w.bias)
        B200_CUDA(cudaMemcpyAsync(out->bias_buf + row, p.bias_buf, p.w.N * 4,
                                  cudaMemcpyDeviceToDevice, st));
      row += p.w.N;
    }
  }
  out->w = a.w;
  out->w.N = N;
  out->w.w = out->w_buf;
  out->w.scale = out->scale_buf;
  out->w.bias = out->bias_buf;
  out->set = true;
  B200_CUDA(cudaStreamSynchronize(st));
  return B200_OK;
}

int gemv(b200_model *m, const DevLinear &L, const float *x, float *y,
         const float *residual, const float *norm_w, bool silu) {
  b200_gemv_args a{};
  a.x = x;
  a.x_dtype = B200_F32;
  a.y_dtype = B200_F32;
  a.y = y;
  a.residual = residual;
  a.norm_weight = norm_w;
  a.norm_eps = m->cfg.eps;
  a.M = 1;
  a.silu_pairs = silu ? 1 : 0;
  return b200_gemv(&L.w, &a, m->stream);
}

// Row-parallel projection of a tensor-parallel model: x += sum over ranks of (input @ W_rank).
int gemv_tp_sum(b200_model *m, const DevLinear &L, const float *input, int index) {
  const int H = m->cfg.hidden;
  cudaStream_t st = m->stream;
  if (m->tp_push.ranks > 0) {
    b200_gemv_args a{};
    a.x = input;
    a.x_dtype = B200_F32;
    a.y_dtype = B200_F32;
    a.y = m->part;   // not written: the results go to the ranks' staging buffers
    a.M = 1;
    TpPush push = m->tp_push;
    push.index = index;
    if (int rc = gemv_run(&L.w, &a, &push, st)) return rc;
    tp_reduce_add_kernel<<<(H + 127) / 128, 128, 0, st>>>(m->x, m->tp_ll, H, push.ranks, push.step, index,
                                                        push.per_step, m->d_state + 6);
    B200_LAUNCH_CHECK();
    return B200_OK;
  }
  if (int rc = gemv(m, L, input, m->part, nullptr, nullptr, false)) return rc;
  B200_NCCL(g_nccl.AllReduce(m->part, m->part, H, kNcclFloat, kNcclSum, g_nccl.comm, st));
  add_inplace_kernel<<<(H + 255) / 256, 256, 0, st>>>(m->x, m->part, H);
  B200_LAUNCH_CHECK();
  return B200_OK;
}

// One projection of a single-GPU decode step: under the w8a8 arithmetic an int8 per-channel layer
// quantises its input row (after the fused RMSNorm) and contracts in integers; everything else
// takes the float GEMV.
int proj(b200_model *m, const DevLinear &L, const float *x, float *y, const float *residual, const float *norm_w,
         bool silu) {
  if (m->act_int8 && L.w.kind == B200_W_I8 && L.w.scale_dtype == B200_F32) {
    if (L.w.K % 64 != 0)
      return fail(B200_EINVAL, "w8a8 projection: K = %lld is not a multiple of 64", (long long)L.w.K);
    if (gemv_i8_fusable(L.w.K))
      return gemv_i8_fused_launch(&L.w, x, norm_w, m->cfg.eps, residual, y, silu ? 1 : 0, m->stream);
    if (int rc = quantize_row_launch(x, norm_w, m->cfg.eps, L.w.K, m->q_row, m->q_scale, m->stream)) return rc;
    return gemv_i8_launch(&L.w, m->q_row, m->q_scale, residual, y, silu ? 1 : 0, m->stream);
  }
  return gemv(m, L, x, y, residual, norm_w, silu);
}

// Issue every kernel of one decode step on m->stream.
int issue_step(b200_model *m, int *n_kernels) {
  const b200_model_config &c = m->cfg;
  const int D = c.head_dim, H = c.hidden;
  const int QD = m->qh * D, KD = m->kvh * D;
  int32_t *d_token = m->d_state, *d_pos = m->d_state + 1,
          *d_next = m->d_state + 2, *d_count = m->d_state + 3;
  cudaStream_t st = m->stream;
  const uint64_t before = b200_launch_count();
  if (int rc = b200_embed(m->embed, d_token, m->x, H, st)) return rc;
  for (int l = 0; l < c.n_layers; ++l) {
    Layer &L = m->layers[l];
    float *q = m->qkv, *k = m->qkv + QD, *v = m->qkv + QD + KD;
    if (int rc = proj(m, L.qkv, m->x, m->qkv, nullptr, L.in_norm, false)) return rc;
    if (int rc = rope_kv_write_launch(q, k, v, m->kv[2 * l], m->kv[2 * l + 1],
                                      m->inv_freq, L.q_norm, L.k_norm, c.eps,
                                      m->qh, m->kvh, D, c.max_len, d_pos,
                                      m->kv_stage + (size_t)(2 * l) * KD,
                                      m->kv_stage + (size_t)(2 * l + 1) * KD, st))
      return rc;
    if (int rc = gqa_decode_launch(q, m->kv[2 * l], m->kv[2 * l + 1], m->attn,
                                   m->attn_scratch, m->qh, m->kvh, D, c.max_len,
                                   m->splits, d_pos, st))
      return rc;
    if (m->tp == 1) {
      if (int rc = proj(m, L.o, m->attn, m->x, m->x, nullptr, false)) return rc;
    } else {
      if (int rc = gemv_tp_sum(m, L.o, m->attn, 2 * l)) return rc;
    }
    if (int rc = proj(m, L.gateup, m->x, m->mid, nullptr, L.post_norm, true)) return rc;
    if (m->tp == 1) {
      if (int rc = proj(m, L.down, m->mid, m->x, m->x, nullptr, false)) return rc;
    } else {
      if (int rc = gemv_tp_sum(m, L.down, m->mid, 2 * l + 1)) return rc;
    }
  }
  if (m->tp == 1) {
    if (int rc = proj(m, m->lm_head, m->x, m->logits, nullptr, m->final_norm, false))
      return rc;
  } else {
    if (int rc = gemv(m, m->lm_head, m->x, m->logits_shard, nullptr,
                      m->final_norm, false))
      return rc;
    if (m->tp_push.ranks > 0) {
      // (value, index) exchange by peer stores; the full logits are gathered only on request
      if (int rc = b200_argmax_first(m->logits_shard, m->vocab, m->d_state + 5, m->argmax_scratch, st))
        return rc;
      tp_argmax_kernel<<<1, 32, 0, st>>>(m->tp_push, m->tp_argmax_at, m->logits_shard, m->d_state + 5, m->vocab,
                                         d_next, m->d_state + 6);
      B200_LAUNCH_CHECK();
    } else {
      B200_NCCL(g_nccl.AllGather(m->logits_shard, m->logits, m->vocab, kNcclFloat,
                                 g_nccl.comm, st));
    }
  }
  if (m->tp == 1 || m->tp_push.ranks == 0)
    if (int rc = b200_argmax_first(m->logits, c.vocab, d_next, m->argmax_scratch, st))
      return rc;
  advance_kernel<<<1, 32, 0, st>>>(d_token, d_pos, d_next, m->d_history, d_count,
                                   m->history_cap, m->d_state + 7);
  B200_LAUNCH_CHECK();
  if (n_kernels)
    *n_kernels = (int)(b200_launch_count() - before);
  return B200_OK;
}


// ---- persistent-kernel path ------------------------------------------------------
void rows_of_host(int N, int cta, int grid, int &begin, int &count) {  // N in dealing units
  const int base = N / grid, rem = N % grid;
  begin = cta * base + (cta < rem ? cta : rem);
  count = base + (cta < rem ? 1 : 0);
}

bool mega_eligible(const b200_model *m, const Layer &L0) {
  const char *env = std::getenv("BUDDY_B200_DECODE");
  if (env && !strcmp(env, "graph"))
    return false;
  const b200_model_config &c = m->cfg;
  if (m->tp != 1 || c.head_dim != 128)
    return false;
  const int G = c.q_heads / c.kv_heads;
  if (G != 1 && G != 2 && G != 4 && G != 6 && G != 8)
    return false;
  auto ok = [](const DevLinear &l) {
    return l.set && l.w.kind == B200_W_I8 && l.w.scale_dtype == B200_F32 && l.w.K % 16 == 0 &&
           l.w.K <= 12288;
  };
  for (const auto &L : m->layers)
    if (!ok(L.qkv) || !ok(L.o) || !ok(L.gate) || !ok(L.up) || !ok(L.down))
      return false;
  (void)L0;
  return ok(m->lm_head);
}

int build_mega(b200_model *m) {
  const b200_model_config &c = m->cfg;
  int dev = 0, sms = 0, coop = 0;
  B200_CUDA(cudaGetDevice(&dev));
  B200_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
  B200_CUDA(cudaDeviceGetAttribute(&coop, cudaDevAttrCooperativeLaunch, dev));
  const int G = c.q_heads / c.kv_heads;
  const int grid = sms, L = c.n_layers, D = c.head_dim;
  // attention work items: every CTA takes one (kv head, split) pair
  int splits = grid / c.kv_heads;
  if (splits > 128) splits = 128;
  while (splits > 1 && G * splits > 768) --splits;
  // the split fold keeps (outputs per warp) x (splits per lane) partials in registers
  const bool fold_fits =
      splits >= 1 && (((G * D + splits - 1) / splits + 15) / 16) * ((splits + 31) / 32) <= 8;
  if (!coop || !fold_fits)
    return B200_OK;  // stays on the graph path
  const int H = c.hidden, QD = c.q_heads * D, KD = c.kv_heads * D, F = c.ffn, V = c.vocab;
  MegaParams &p = m->mp;
  const int Ks[5] = {H, QD, H, F, H}, Ns[5] = {QD + 2 * KD, H, 2 * F, H, V};
  if (H > 1536 || QD > 1536 || H % 16 != 0 || QD % 16 != 0 || F % 16 != 0)
    return B200_OK;
  int slot_bytes = 0;
  for (int i = 0; i < 5; ++i) {
    if (i == 3)
      continue;
    MegaPhase &ph = p.phase[i];
    ph.K = Ks[i];
    ph.N = Ns[i];
    ph.row_bytes = Ks[i] + kMegaTrailer;
    ph.mode = 0;
    ph.unit = i == 2 ? 2 : 1;
    ph.rps = 16;   // a stage is 16 rows: 16 warps x 1 row, 4 x 4 or 2 x 8
    if (ph.rps * ph.row_bytes > slot_bytes)
      slot_bytes = ph.rps * ph.row_bytes;
  }
  {
    // down projection: long rows, a few per stage, one warp per row
    MegaPhase &ph = p.phase[3];
    ph.K = F;
    ph.N = H;
    ph.row_bytes = F + kMegaTrailer;
    ph.mode = 0;
    ph.unit = 1;
    ph.rps = slot_bytes / ph.row_bytes;
    if (ph.rps > 8) ph.rps = 8;
    if (ph.rps < 1 || (ph.rps & (ph.rps - 1)) != 0) {   // 1, 2, 4 or 8 rows: the warps split evenly over stages
      if (ph.rps >= 4) ph.rps = 4;
      else if (ph.rps >= 2) ph.rps = 2;
      else if (ph.rps < 1) return B200_OK;
    }
  }
  slot_bytes = (slot_bytes + 127) / 128 * 128;
  int xs_floats = H > QD ? H : QD;                          // staged activations of a projection
  if (xs_floats < F) xs_floats = F;
  if (xs_floats < (G + 2 + 7 * G) * D) xs_floats = (G + 2 + 7 * G) * D;   // staged q | k | v + states of the 7 scanning warps
  if (xs_floats < 3 * G * splits + 8) xs_floats = 3 * G * splits + 8;   // split fold: m, l, weights
  xs_floats = (xs_floats + 31) / 32 * 32;
  const size_t fixed = mega_fixed_shared_bytes() + (size_t)xs_floats * 4;
  int slots = (int)((227 * 1024 - (long)fixed) / slot_bytes);
  if (slots > kMegaMaxSlots) slots = kMegaMaxSlots;
  if (slots < 4)
    return B200_OK;
  for (int cta = 0; cta < grid; ++cta) {   // the in-kernel stage table is fixed-size
    int per_layer = 0;
    for (int i = 0; i < 4; ++i) {
      int b, n;
      rows_of_host(p.phase[i].N / p.phase[i].unit, cta, grid, b, n);
      per_layer += (n * p.phase[i].unit + p.phase[i].rps - 1) / p.phase[i].rps;
    }
    if (per_layer > kMegaMaxLayerStages)
      return B200_OK;
  }
  // per-phase, per-CTA stream offsets
  const int nph = 4 * L + 1;
  std::vector<int64_t> table((size_t)(nph + 1) * grid);
  int64_t total = 0;
  for (int cta = 0; cta < grid; ++cta) {
    table[(size_t)nph * grid + cta] = total;  // start of this CTA's stream
    for (int i = 0; i < nph; ++i) {
      const MegaPhase &ph = p.phase[i < 4 * L ? i % 4 : 4];
      int b, n;
      rows_of_host(ph.N / ph.unit, cta, grid, b, n);
      table[(size_t)i * grid + cta] = total;
      total += (int64_t)n * ph.unit * ph.row_bytes;
    }
  }
  if (int rc = dev_alloc((void **)&m->mega_stream, total)) return rc;
  if (int rc = dev_alloc((void **)&m->mega_offsets, table.size() * 8)) return rc;
  B200_CUDA(cudaMemcpy(m->mega_offsets, table.data(), table.size() * 8, cudaMemcpyHostToDevice));
  cudaStream_t st = m->stream;
  for (int l = 0; l < L; ++l) {
    Layer &Ly = m->layers[l];
    const int64_t *o0 = m->mega_offsets + (size_t)(4 * l) * grid;
    if (int rc = mega_build_rows(Ly.qkv.w_buf, H, Ns[0], 1, 0, Ns[0], 1, (const float *)Ly.qkv.scale_buf,
                                 Ly.qkv.bias_buf, grid, p.phase[0].row_bytes, o0, m->mega_stream, st))
      return rc;
    if (int rc = mega_build_rows(Ly.o.w_buf, QD, H, 1, 0, H, 1, (const float *)Ly.o.scale_buf, nullptr,
                                 grid, p.phase[1].row_bytes, o0 + grid, m->mega_stream, st))
      return rc;
    // gate_j -> row 2j, up_j -> row 2j+1: one warp then holds the pair of a SiLU gate
    if (int rc = mega_build_rows(Ly.gate.w_buf, H, F, 2, 0, 2 * F, 2, (const float *)Ly.gate.scale_buf,
                                 nullptr, grid, p.phase[2].row_bytes, o0 + 2 * grid, m->mega_stream, st))
      return rc;
    if (int rc = mega_build_rows(Ly.up.w_buf, H, F, 2, 1, 2 * F, 2, (const float *)Ly.up.scale_buf, nullptr,
                                 grid, p.phase[2].row_bytes, o0 + 2 * grid, m->mega_stream, st))
      return rc;
    if (int rc = mega_build_rows(Ly.down.w_buf, F, H, 1, 0, H, 1, (const float *)Ly.down.scale_buf, nullptr,
                                 grid, p.phase[3].row_bytes, o0 + 3 * grid, m->mega_stream, st))
      return rc;
  }
  if (int rc = mega_build_rows(m->lm_head.w_buf, H, V, 1, 0, V, 1, (const float *)m->lm_head.scale_buf,
                               nullptr, grid, p.phase[4].row_bytes,
                               m->mega_offsets + (size_t)(4 * L) * grid, m->mega_stream, st))
    return rc;
  std::vector<const float *> lvec(4 * L);
  for (int l = 0; l < L; ++l) {
    lvec[4 * l] = m->layers[l].in_norm;
    lvec[4 * l + 1] = m->layers[l].post_norm;
    lvec[4 * l + 2] = m->layers[l].q_norm;
    lvec[4 * l + 3] = m->layers[l].k_norm;
  }
  if (int rc = dev_alloc((void **)&m->lvec_dev, lvec.size() * sizeof(float *))) return rc;
  B200_CUDA(cudaMemcpy(m->lvec_dev, lvec.data(), lvec.size() * sizeof(float *), cudaMemcpyHostToDevice));
  // tagged activation buffers, all in one allocation (zero tags never match)
  const size_t n_qkv = 2 * (size_t)(QD + 2 * KD), n_attn = 2 * (size_t)QD, n_x = 2 * (size_t)H,
               n_mid = 2 * (size_t)F, n_part = 2 * (size_t)c.q_heads * splits * (D + 2),
               n_cand = 2 * (size_t)grid;
  const size_t n_ll = n_qkv + n_attn + 2 * n_x + n_mid + n_part + n_cand + 16;
  if (int rc = dev_alloc((void **)&m->ll_buf, n_ll * sizeof(uint2))) return rc;
  B200_CUDA(cudaMemset(m->ll_buf, 0, n_ll * sizeof(uint2)));
  uint2 *q = m->ll_buf;
  auto take = [&](size_t n) { uint2 *r = q; q += (n + 1) / 2 * 2; return r; };   // keep 16-byte alignment
  p.ll_qkv = take(n_qkv);
  p.ll_attn = take(n_attn);
  p.ll_xb = take(n_x);
  p.ll_mid = take(n_mid);
  p.ll_xa = take(n_x);
  p.ll_part = take(n_part);
  p.ll_cand = take(n_cand);
  p.stream = m->mega_stream;
  p.cta_off = m->mega_offsets + (size_t)nph * grid;
  p.H = H; p.F = F; p.V = V; p.qh = c.q_heads; p.kvh = c.kv_heads; p.L = L;
  p.max_len = c.max_len;
  p.splits = splits;
  p.slots = slots;
  p.slot_bytes = slot_bytes;
  p.xs_floats = xs_floats;
  p.eps = c.eps;
  p.embed = m->embed; p.inv_freq = m->inv_freq; p.final_norm = m->final_norm;
  p.lvec = m->lvec_dev;
  p.kv = m->kv_dev;
  p.logits = m->logits;
  p.kv_stage = m->kv_stage;
  p.state = m->d_state;
  p.history = m->d_history;
  p.history_cap = m->history_cap;
  p.error = m->d_state + 6;
  p.trace = nullptr;
  p.trace_stride = 1;
  if (const char *t = std::getenv("BUDDY_B200_TRACE")) {
    p.trace_stride = std::atoi(t) > 0 ? std::atoi(t) : 1;
    const size_t n = (size_t)(grid / p.trace_stride + 1) * (L + 1) * kMegaTraceSlots;
    if (int rc = dev_alloc((void **)&m->d_trace, n * 8)) return rc;
    B200_CUDA(cudaMemset(m->d_trace, 0, n * 8));
    p.trace = m->d_trace;
  }
  m->mega_grid = grid;
  m->mega_smem = fixed + (size_t)slots * slot_bytes;
  m->mega_stream_bytes = total;
  B200_CUDA(cudaStreamSynchronize(st));
  m->mega = true;
  return B200_OK;
}

int set_state(b200_model *m, int token, int pos);

// The decode step of the w8a8 arithmetic: the same kernels as the float step except for the int8
// projections, captured into a graph of its own the first time it is needed.  The caller has
// set the device state (token, position); the warm-up pass outside capture runs that very step
// (it writes the K/V row the real step writes again), then the state is put back.
int run_step_int8(b200_model *m) {
  if (!m->exec_q) {
    const b200_model_config &c = m->cfg;
    int64_t Kmax = c.hidden > m->ffn ? c.hidden : m->ffn;
    if ((int64_t)m->qh * c.head_dim > Kmax) Kmax = (int64_t)m->qh * c.head_dim;
    if (!m->q_row) {
      if (int rc = dev_alloc((void **)&m->q_row, (size_t)Kmax)) return rc;
      if (int rc = dev_alloc((void **)&m->q_scale, 16)) return rc;
    }
    const int token = m->h_state_pinned[0], pos = m->h_state_pinned[1];
    if (int rc = issue_step(m, &m->kernels_per_step_q)) return rc;
    B200_CUDA(cudaStreamSynchronize(m->stream));
    if (int rc = set_state(m, token, pos)) return rc;
    B200_CUDA(cudaStreamBeginCapture(m->stream, cudaStreamCaptureModeThreadLocal));
    int rc = issue_step(m, nullptr);
    cudaGraph_t g = nullptr;
    cudaError_t e = cudaStreamEndCapture(m->stream, &g);
    if (rc != B200_OK) {
      if (g) cudaGraphDestroy(g);
      return rc;
    }
    if (e != cudaSuccess)
      return fail(B200_ECUDA, "graph capture (w8a8 step): %s", cudaGetErrorString(e));
    m->graph_q = g;
    B200_CUDA(cudaGraphInstantiate(&m->exec_q, m->graph_q, 0));
  }
  B200_CUDA(cudaGraphLaunch(m->exec_q, m->stream));
  count_launch(m->kernels_per_step_q);
  return B200_OK;
}

int run_step(b200_model *m) {
  if (m->act_int8)
    return run_step_int8(m);
  if (m->mega)
    return mega_launch(m->mp, m->mega_grid, m->mega_smem, m->stream);
  B200_CUDA(cudaGraphLaunch(m->exec, m->stream));
  count_launch(m->kernels_per_step);
  return B200_OK;
}

int check_step_error(b200_model *m) {
  // h_state_pinned holds the 8 state words read back after the step
  if (m->h_state_pinned[6] != 0) {
    const int code = m->h_state_pinned[6];
    // clear the flag and move the launch counter on, so that tags written by
    // the failed step can never match a later one
    m->h_state_pinned[6] = 0;
    m->h_state_pinned[4] += 2;
    cudaMemcpyAsync(m->d_state + 4, m->h_state_pinned + 4, 12, cudaMemcpyHostToDevice, m->stream);
    cudaStreamSynchronize(m->stream);
    return fail(B200_ECUDA, "decode step kernel gave up on a bounded wait (code %d)", code);
  }
  return B200_OK;
}

int set_state(b200_model *m, int token, int pos) {
  m->h_state_pinned[0] = token;
  m->h_state_pinned[1] = pos;
  m->h_state_pinned[2] = 0;
  m->h_state_pinned[3] = 0;
  B200_CUDA(cudaMemcpyAsync(m->d_state, m->h_state_pinned, 4 * sizeof(int32_t),
                            cudaMemcpyHostToDevice, m->stream));
  return B200_OK;
}

} // namespace

extern "C" {

int b200_tp_unique_id(void *id128) {
  if (!id128)
    return fail(B200_EINVAL, "tp_unique_id: null");
  if (int rc = nccl_bind()) return rc;
  B200_NCCL(g_nccl.GetUniqueId(id128));
  return B200_OK;
}

int b200_tp_init(const void *id128, int rank, int size) {
  if (!id128 || size < 1 || rank < 0 || rank >= size)
    return fail(B200_EINVAL, "tp_init: bad argument");
  if (int rc = ensure_device()) return rc;
  if (int rc = nccl_bind()) return rc;
  if (g_nccl.comm)
    return fail(B200_ESTATE, "tp_init: already initialised");
  Id128 id;
  memcpy(id.bytes, id128, 128);
  B200_NCCL(g_nccl.CommInitRank(&g_nccl.comm, size, id, rank));
  g_nccl.rank = rank;
  g_nccl.size = size;
  return B200_OK;
}

void b200_tp_shutdown(void) {
  if (g_nccl.comm) {
    g_nccl.CommDestroy(g_nccl.comm);
    g_nccl.comm = nullptr;
  }
  g_nccl.size = 1;
  g_nccl.rank = 0;
}

int b200_model_create(const b200_model_config *cfg, b200_model **out) {
  if (!cfg || !out)
    return fail(B200_EINVAL, "model_create: null argument");
  const b200_model_config &c = *cfg;
  const int tp = c.tp_size < 1 ? 1 : c.tp_size;
  if (c.hidden < 1 || c.n_layers < 1 || c.q_heads < 1 || c.kv_heads < 1 ||
      c.q_heads % c.kv_heads || c.ffn < 1 || c.vocab < 1 || c.max_len < 1 ||
      (c.head_dim != 64 && c.head_dim != 128))
    return fail(B200_EINVAL, "model_create: bad architecture");
  if (c.tp_rank < 0 || c.tp_rank >= tp || c.kv_heads % tp || c.q_heads % tp ||
      c.ffn % tp || c.vocab % tp)
    return fail(B200_EINVAL,
                "model_create: tp_size %d must divide kv_heads, q_heads, ffn and vocab", tp);
  if (tp > 1 && (!g_nccl.comm || g_nccl.size != tp || g_nccl.rank != c.tp_rank))
    return fail(B200_ESTATE, "model_create: call b200_tp_init(rank, size) first");
  if (int rc = ensure_device()) return rc;

  b200_model *m = new b200_model();
  m->cfg = c;
  m->cfg.tp_size = tp;
  m->tp = tp;
  m->rank = c.tp_rank;
  m->qh = c.q_heads / tp;
  m->kvh = c.kv_heads / tp;
  m->ffn = c.ffn / tp;
  m->vocab = c.vocab / tp;
  m->layers.resize(c.n_layers);
  m->kv.assign(2 * c.n_layers, nullptr);
  const int D = c.head_dim;
  // attention splits: about four CTAs per SM over this rank's kv heads, at least 32 rows each
  {
    const int local_kv = c.kv_heads / tp;
    m->splits = (4 * 148 + local_kv - 1) / local_kv;
    if (m->splits > c.max_len / 32) m->splits = c.max_len / 32;
    if (m->splits > 128) m->splits = 128;
    if (m->splits < 1) m->splits = 1;
  }
  m->history_cap = 65536;

  int rc = B200_OK;
  auto A = [&](void **p, size_t bytes) {
    if (rc == B200_OK) {
      rc = dev_alloc(p, bytes);
      if (rc == B200_OK && cudaMemset(*p, 0, bytes ? bytes : 16) != cudaSuccess)
        rc = fail(B200_ECUDA, "cudaMemset failed");
    }
  };
  const size_t kv_bytes = (size_t)m->kvh * c.max_len * D * sizeof(float);
  for (auto &p : m->kv) A((void **)&p, kv_bytes);
  A((void **)&m->kv_dev, m->kv.size() * sizeof(float *));
  A((void **)&m->x, c.hidden * 4);
  A((void **)&m->qkv, (size_t)(m->qh + 2 * m->kvh) * D * 4);
  A((void **)&m->attn, (size_t)m->qh * D * 4);
  A((void **)&m->mid, (size_t)m->ffn * 4);
  A((void **)&m->part, c.hidden * 4);
  A((void **)&m->logits, (size_t)c.vocab * 4);
  A((void **)&m->logits_shard, (size_t)m->vocab * 4);
  A((void **)&m->attn_scratch, b200_gqa_scratch_floats(m->qh, D, m->splits) * 4);
  A((void **)&m->argmax_scratch, 2048 * 4);
  A((void **)&m->kv_stage, (size_t)2 * c.n_layers * m->kvh * D * 4);
  A((void **)&m->d_state, 8 * sizeof(int32_t));
  A((void **)&m->d_history, m->history_cap * sizeof(int32_t));
  if (rc == B200_OK &&
      cudaMemcpy(m->kv_dev, m->kv.data(), m->kv.size() * sizeof(float *),
                 cudaMemcpyHostToDevice) != cudaSuccess)
    rc = fail(B200_ECUDA, "kv pointer table upload failed");
  if (rc == B200_OK && cudaStreamCreateWithFlags(&m->stream, cudaStreamNonBlocking) != cudaSuccess)
    rc = fail(B200_ECUDA, "stream create failed");
  if (rc == B200_OK && (cudaEventCreate(&m->ev0) != cudaSuccess || cudaEventCreate(&m->ev1) != cudaSuccess))
    rc = fail(B200_ECUDA, "event create failed");
  if (rc == B200_OK && (cudaMallocHost((void **)&m->h_logits_pinned, (size_t)c.vocab * 4) != cudaSuccess ||
                        cudaMallocHost((void **)&m->h_rows_pinned,
                                       (size_t)2 * c.n_layers * m->kvh * D * 4) != cudaSuccess ||
                        cudaMallocHost((void **)&m->h_state_pinned, 32) != cudaSuccess))
    rc = fail(B200_ENOMEM, "pinned host allocation failed");
  if (rc != B200_OK) {
    b200_model_destroy(m);
    return rc;
  }
  *out = m;
  return B200_OK;
}

void b200_model_destroy(b200_model *m) {
  if (!m) return;
  if (m->stream) cudaStreamSynchronize(m->stream);
  if (m->exec) cudaGraphExecDestroy(m->exec);
  if (m->graph) cudaGraphDestroy(m->graph);
  for (auto &L : m->layers) {
    cudaFree(L.in_norm); cudaFree(L.post_norm); cudaFree(L.q_norm); cudaFree(L.k_norm);
    L.q.release(); L.k.release(); L.v.release(); L.o.release();
    L.gate.release(); L.up.release(); L.down.release();
    L.qkv.release(); L.gateup.release();
  }
  m->lm_head.release();
  for (auto p : m->kv) cudaFree(p);
  cudaFree(m->kv_dev); cudaFree(m->embed); cudaFree(m->inv_freq); cudaFree(m->final_norm);
  cudaFree(m->x); cudaFree(m->qkv); cudaFree(m->attn); cudaFree(m->mid);
  for (void *p : m->tp_opened)
    if (p) cudaIpcCloseMemHandle(p);
  cudaFree(m->tp_ll);
  cudaFree(m->part); cudaFree(m->logits); cudaFree(m->logits_shard);
  cudaFree(m->attn_scratch); cudaFree(m->argmax_scratch); cudaFree(m->kv_stage);
  cudaFree(m->d_state); cudaFree(m->d_history);
  cudaFree(m->mega_stream); cudaFree(m->mega_offsets); cudaFree(m->lvec_dev);
  cudaFree(m->ll_buf); cudaFree(m->d_trace);
  cudaFree(m->pf_x); cudaFree(m->pf_qkv); cudaFree(m->pf_att); cudaFree(m->pf_mid); cudaFree(m->pf_logits);
  cudaFree(m->pf_ws); cudaFree(m->pf_tokens); cudaFree(m->pf_norm);
  cudaFree(m->q_row); cudaFree(m->q_scale);
  if (m->exec_q) cudaGraphExecDestroy(m->exec_q);
  if (m->graph_q) cudaGraphDestroy(m->graph_q);
  if (m->h_logits_pinned) cudaFreeHost(m->h_logits_pinned);
  if (m->h_rows_pinned) cudaFreeHost(m->h_rows_pinned);
  if (m->h_state_pinned) cudaFreeHost(m->h_state_pinned);
  if (m->ev0) cudaEventDestroy(m->ev0);
  if (m->ev1) cudaEventDestroy(m->ev1);
  if (m->stream) cudaStreamDestroy(m->stream);
  delete m;
}

int b200_model_set_vector(b200_model *m, int layer, int slot, const float *host,
                          int64_t n) {
  if (!m || !host || n < 1)
    return fail(B200_EINVAL, "set_vector: bad argument");
  if (m->finalized)
    return fail(B200_ESTATE, "set_vector: model already finalised");
  const b200_model_config &c = m->cfg;
  float **dst = nullptr;
  int64_t want = 0, off = 0, take = 0;
  DevLinear *bias_of = nullptr;
  switch (slot) {
  case B200_T_EMBED: dst = &m->embed; want = (int64_t)c.vocab * c.hidden; break;
  case B200_T_INV_FREQ: dst = &m->inv_freq; want = c.head_dim / 2; break;
  case B200_T_FINAL_NORM: dst = &m->final_norm; want = c.hidden; break;
  default: break;
  }
  if (!dst && layer >= 0 && layer < c.n_layers) {
    Layer &L = m->layers[layer];
    switch (slot) {
    case B200_T_IN_NORM: dst = &L.in_norm; want = c.hidden; break;
    case B200_T_POST_NORM: dst = &L.post_norm; want = c.hidden; break;
    case B200_T_Q_NORM: dst = &L.q_norm; want = c.head_dim; break;
    case B200_T_K_NORM: dst = &L.k_norm; want = c.head_dim; break;
    case B200_T_Q_BIAS: bias_of = &L.q; want = (int64_t)c.q_heads * c.head_dim; break;
    case B200_T_K_BIAS: bias_of = &L.k; want = (int64_t)c.kv_heads * c.head_dim; break;
    case B200_T_V_BIAS: bias_of = &L.v; want = (int64_t)c.kv_heads * c.head_dim; break;
    default: break;
    }
  }
  if (!dst && !bias_of)
    return fail(B200_EINVAL, "set_vector: unknown slot %d (layer %d)", slot, layer);
  if (n != want)
    return fail(B200_EINVAL, "set_vector: slot %d expects %lld elements, got %lld",
                slot, (long long)want, (long long)n);
  take = want;
  if (bias_of) {  // column-parallel bias: this rank's slice
    take = want / m->tp;
    off = take * m->rank;
    if (!bias_of->set)
      return fail(B200_ESTATE, "set_vector: set the projection before its bias");
    dst = &bias_of->bias_buf;
  }
  if (*dst) { cudaFree(*dst); *dst = nullptr; }
  if (int rc = dev_alloc((void **)dst, take * 4)) return rc;
  B200_CUDA(cudaMemcpy(*dst, host + off, take * 4, cudaMemcpyHostToDevice));
  if (bias_of)
    bias_of->w.bias = *dst;
  return B200_OK;
}

int b200_model_set_linear(b200_model *m, int layer, int slot, int src_kind,
                          const void *host_w, const void *host_scale,
                          int scale_dtype, int src_signed, int64_t K, int64_t N,
                          int quantize_to, int group) {
  if (!m || !host_w || K < 1 || N < 1)
    return fail(B200_EINVAL, "set_linear: bad argument");
  if (m->finalized)
    return fail(B200_ESTATE, "set_linear: model already finalised");
  DevLinear *L = linear_slot(m, layer, slot);
  if (!L)
    return fail(B200_EINVAL, "set_linear: unknown slot %d (layer %d)", slot, layer);
  if (src_kind != B200_W_F32 && quantize_to >= 0)
    return fail(B200_EINVAL, "set_linear: only f32 sources can be quantised");
  if (src_kind != B200_W_F32 && !host_scale)
    return fail(B200_EINVAL, "set_linear: quantised source without scales");
  const int tp = m->tp, rank = m->rank;
  const bool rowp = is_row_parallel(slot);
  if ((rowp && K % tp) || (!rowp && N % tp))
    return fail(B200_EINVAL, "set_linear: shape not divisible by tp_size");
  cudaStream_t st = m->stream;
  L->release();

  const int kind = quantize_to >= 0 ? quantize_to : src_kind;
  if (kind == B200_W_U4 && (N & 1))
    return fail(B200_EINVAL, "set_linear: int4 needs an even N");
  int64_t G = (kind == B200_W_U4 && group > 0 && group < K) ? group : K;
  if (kind == B200_W_U4 && (K % G || (rowp && (K / tp) % G && G != K)))
    return fail(B200_EINVAL, "set_linear: group %lld incompatible with K/tp", (long long)G);
  const int64_t ng = K / G;

  // 1. full tensor in the reference layout on the device
  const int64_t src_elem_bytes = src_kind == B200_W_F32 ? 4 : 1;
  const int64_t src_bytes = src_kind == B200_W_U4 ? K * N / 2 : K * N * src_elem_bytes;
  void *d_src = nullptr, *d_q = nullptr, *d_scale = nullptr, *d_full = nullptr;
  int rc = dev_alloc(&d_src, src_bytes);
  auto cleanup = [&]() { cudaFree(d_src); cudaFree(d_q); cudaFree(d_scale); cudaFree(d_full); };
#define B200_TRY(expr)                                                         \
  do { if (rc == B200_OK) rc = (expr); } while (0)
#define B200_TRYCUDA(expr)                                                     \
  do { if (rc == B200_OK && (expr) != cudaSuccess)                             \
      rc = fail(B200_ECUDA, "%s failed: %s", #expr, cudaGetErrorString(cudaGetLastError())); } while (0)
  B200_TRYCUDA(cudaMemcpyAsync(d_src, host_w, src_bytes, cudaMemcpyHostToDevice, st));

  // 2. quantise on the device when asked; scales end up as [ng, N] (ref layout)
  const void *ref_w = d_src;
  int sdt = scale_dtype;
  if (quantize_to == B200_W_I8) {
    B200_TRY(dev_alloc(&d_q, K * N));
    B200_TRY(dev_alloc(&d_scale, N * 4));
    B200_TRY(b200_quantize_per_channel((const float *)d_src, K, N, 8, (int8_t *)d_q,
                                       (float *)d_scale, st));
    ref_w = d_q;
    sdt = B200_F32;
  } else if (quantize_to == B200_W_U4) {
    B200_TRY(dev_alloc(&d_q, K * N / 2));
    B200_TRY(dev_alloc(&d_scale, ng * N * 2));
    B200_TRY(b200_quantize_w4_group((const float *)d_src, K, N, G, (uint8_t *)d_q,
                                    (uint16_t *)d_scale, st));
    ref_w = d_q;
    sdt = B200_F16;
    src_signed = 0;
  } else if (quantize_to >= 0) {
    rc = fail(B200_EINVAL, "set_linear: cannot quantise to kind %d", quantize_to);
  } else if (kind != B200_W_F32) {
    const int64_t sb = ng * N * (sdt == B200_F32 ? 4 : 2);
    B200_TRY(dev_alloc(&d_scale, sb));
    B200_TRYCUDA(cudaMemcpyAsync(d_scale, host_scale, sb, cudaMemcpyHostToDevice, st));
  }

  // 3. pack this rank's shard
  const int64_t Kl = rowp ? K / tp : K, Nl = rowp ? N : N / tp;
  const int64_t rb = packed_row_bytes(kind, Kl);
  const int64_t ssz = sdt == B200_F32 ? 4 : 2;
  const int64_t ngl = (G == K) ? 1 : Kl / G;
  B200_TRY(dev_alloc(&L->w_buf, rb * Nl));
  if (kind != B200_W_F32)
    B200_TRY(dev_alloc(&L->scale_buf, ngl * Nl * ssz));
  if (rc == B200_OK) {
    if (rowp || tp == 1) {
      // K-slice: rows [rank*Kl, (rank+1)*Kl) of the [K,N] source are contiguous
      const int64_t row_bytes_src = src_bytes / K;
      const int64_t ref_row = (ref_w == d_src) ? row_bytes_src
                                               : (kind == B200_W_U4 ? N / 2 : N);
      const char *shard = (const char *)ref_w + (rowp ? rank * Kl * ref_row : 0);
      B200_TRY(b200_pack_weight(kind, shard, Kl, N, src_signed, L->w_buf, st));
      if (kind != B200_W_F32) {
        // per-channel scales are shared by every K-shard; group scales split by rows
        const char *sshard = (const char *)d_scale +
                             ((rowp && G != K) ? rank * ngl * N * ssz : 0);
        B200_TRY(b200_pack_scales(sshard, sdt, ngl, N, L->scale_buf, st));
      }
    } else {
      // N-slice: pack the full tensor, keep rows [rank*Nl, (rank+1)*Nl)
      B200_TRY(dev_alloc(&d_full, rb * N));
      B200_TRY(b200_pack_weight(kind, ref_w, K, N, src_signed, d_full, st));
      B200_TRYCUDA(cudaMemcpyAsync(L->w_buf, (char *)d_full + rank * Nl * rb, rb * Nl,
                                   cudaMemcpyDeviceToDevice, st));
      if (kind != B200_W_F32) {
        void *d_sfull = nullptr;
        B200_TRY(dev_alloc(&d_sfull, ng * N * ssz));
        B200_TRY(b200_pack_scales(d_scale, sdt, ng, N, d_sfull, st));
        B200_TRYCUDA(cudaMemcpyAsync(L->scale_buf, (char *)d_sfull + rank * Nl * ng * ssz,
                                     ng * Nl * ssz, cudaMemcpyDeviceToDevice, st));
        B200_TRYCUDA(cudaStreamSynchronize(st));
        cudaFree(d_sfull);
      }
    }
  }
  B200_TRYCUDA(cudaStreamSynchronize(st));
#undef B200_TRY
#undef B200_TRYCUDA
  cleanup();
  if (rc != B200_OK) {
    L->release();
    return rc;
  }
  L->w.kind = kind;
  L->w.group = (kind == B200_W_U4 && G != K) ? (int)G : 0;
  L->w.K = Kl;
  L->w.N = Nl;
  L->w.w = L->w_buf;
  L->w.scale = L->scale_buf;
  L->w.scale_dtype = sdt;
  L->w.bias = nullptr;
  L->set = true;
  return B200_OK;
}

int b200_blob_elements(const b200_model_config *cfg, const char *variant,
                       int64_t *n_float, int64_t *n_int) {
  if (!cfg || !variant)
    return fail(B200_EINVAL, "blob_elements: null argument");
  const b200_model_config &c = *cfg;
  const int64_t H = c.hidden, D = c.head_dim, QD = (int64_t)c.q_heads * D,
                KD = (int64_t)c.kv_heads * D, F = c.ffn, V = c.vocab;
  const int64_t qkv = H * QD + 2 * H * KD + (c.qkv_bias ? QD + 2 * KD : 0);
  const int64_t quant_layer = QD * H + 2 * H * F + F * H;
  const int64_t small_layer = 2 * H + (c.qk_norm ? 2 * D : 0);   // the layer norms (+ Qwen3's head norms)
  const int64_t common = V * H + D / 2 + H;  // embedding, inv_freq, final norm
  int64_t nf = 0, ni = 0;
  if (!strcmp(variant, "f32") || !strcmp(variant, "f16") || !strcmp(variant, "bf16") || !strcmp(variant, "f32p32")) {
    // f32p32: the f32 blob with every matmul weight in 32-column panels (the decode file of
    // the packed-decode spec, frontend/Python/graph/transform/pack_decode_weights.py:32-124)
    // f16 / bf16: the same single blob with 16-bit elements (models/deepseek_r1/specs/f16.json;
    // bf16: the module is converted with .bfloat16() before tracing, the writer keeps the high
    // halves of those values, tools/buddy-codegen/import_model.py:118-145, 700-707)
    nf = common + c.n_layers * (small_layer + qkv + quant_layer) + H * V;
  } else if (!strcmp(variant, "w8a32") || !strcmp(variant, "w8a16") || !strcmp(variant, "w8a8")) {
    // w8a16: the same split, n_float counts f16 elements (models/deepseek_r1/specs/w8a16.json);
    // w8a8: the files of w8a32 (tools/buddy-codegen/gen_config.py:63-66), the graph differs
    ni = c.n_layers * quant_layer + H * V;
    nf = common + c.n_layers * (small_layer + qkv) +
         c.n_layers * (H + 2 * F + H) + V;  // + one scale per quantised column
  } else if (!strcmp(variant, "w4a16")) {
    // the same split as w8a32: n_float counts f16 elements, n_int packed bytes (two nibbles each)
    ni = (c.n_layers * quant_layer + H * V) / 2;
    nf = common + c.n_layers * (small_layer + qkv) + c.n_layers * (H + 2 * F + H) + V;
  } else {
    return fail(B200_EINVAL, "blob_elements: unknown variant '%s'", variant);
  }
  if (n_float) *n_float = nf;
  if (n_int) *n_int = ni;
  return B200_OK;
}

int b200_model_load_blobs(b200_model *m, const char *variant,
                          const void *float_blob, int64_t n_float,
                          const void *int_blob, int64_t n_int,
                          int all_linear_w8) {
  if (!m || !variant || !float_blob)
    return fail(B200_EINVAL, "load_blobs: null argument");
  const b200_model_config &c = m->cfg;
  int64_t want_f = 0, want_i = 0;
  if (int rc = b200_blob_elements(&c, variant, &want_f, &want_i)) return rc;
  const bool w8h = !strcmp(variant, "w8a16");
  const bool w8q = !strcmp(variant, "w8a8");
  const bool w8 = !strcmp(variant, "w8a32") || w8h || w8q, w4 = !strcmp(variant, "w4a16");
  if (w8q && m->tp != 1)
    return fail(B200_EINVAL, "load_blobs(w8a8): single-GPU sessions only");
  if (n_float != want_f || ((w8 || w4) && (n_int != want_i || !int_blob)))
    return fail(B200_EINVAL,
                "load_blobs(%s): expected %lld float / %lld int8 elements, got %lld / %lld",
                variant, (long long)want_f, (long long)want_i, (long long)n_float,
                (long long)n_int);
  const int64_t H = c.hidden, D = c.head_dim, QD = (int64_t)c.q_heads * D,
                KD = (int64_t)c.kv_heads * D, F = c.ffn, V = c.vocab;
  // w4a16 / w8a16: the float blob holds f16 values (tools/buddy-codegen/gen_config.py:51-71);
  // they are widened once (exact), so that the rest of the walk is the same for every variant.
  // The int4 scales stay f16 (they follow the float tensors in the same blob); the int8 scales
  // of w8a16 are taken from the widened copy (the same values as f32).
  std::vector<float> widened;
  const uint16_t *f16_blob = (const uint16_t *)float_blob;
  const bool bf16_blob = !strcmp(variant, "bf16");
  const bool half_blob = w4 || w8h || !strcmp(variant, "f16") || bf16_blob;
  if (half_blob) {
    widened.resize((size_t)n_float);
    for (int64_t i = 0; i < n_float; ++i) {
      if (bf16_blob) {
        const uint32_t u = (uint32_t)f16_blob[i] << 16;
        memcpy(&widened[(size_t)i], &u, 4);
      } else {
        widened[(size_t)i] = __half2float(__ushort_as_half(f16_blob[i]));
      }
    }
  }
  const float *fp0 = half_blob ? widened.data() : (const float *)float_blob;
  const float *fp = fp0;
  const int8_t *ip = (const int8_t *)int_blob;
  const int qf = all_linear_w8 ? B200_W_I8 : -1;  // float linears: keep or quantise
  auto takef = [&](int64_t n) { const float *p = fp; fp += n; return p; };
  auto takei = [&](int64_t n) { const int8_t *p = ip; ip += n; return p; };
  struct Pending { int layer, slot; const int8_t *w; int64_t K, N; };
  std::vector<Pending> pend;
  int rc = B200_OK;
#define B200_DO(expr) do { if (rc == B200_OK) rc = (expr); } while (0)
  // Order: the module's parameters as the traced graph first uses them, then its buffers
  // (frontend/Python/frontend.py:922-933): embedding, layers, final norm, lm_head, inv_freq.
  B200_DO(b200_model_set_vector(m, -1, B200_T_EMBED, takef(V * H), V * H));
  // f32p32: Bpacked[n / 32][k][n % 32] == B[k, n]; the panels are undone into a scratch copy
  const bool panels = !strcmp(variant, "f32p32");
  std::vector<float> plain;
  auto flinear = [&](int l, int slot, int64_t K, int64_t N) {
    const float *w = takef(K * N);
    if (panels && rc == B200_OK) {
      if (N % 32 != 0) {
        rc = fail(B200_EINVAL, "load_blobs(f32p32): N = %lld is not a multiple of the panel width", (long long)N);
        return;
      }
      plain.resize((size_t)(K * N));
      for (int64_t pn = 0; pn < N / 32; ++pn)
        for (int64_t k = 0; k < K; ++k)
          memcpy(&plain[(size_t)(k * N + pn * 32)], w + (pn * K + k) * 32, 32 * sizeof(float));
      w = plain.data();
    }
    B200_DO(b200_model_set_linear(m, l, slot, B200_W_F32, w, nullptr, B200_F32, 0, K, N, qf, 0));
  };
  auto qlinear = [&](int l, int slot, int64_t K, int64_t N) {
    if (w8)
      pend.push_back({l, slot, takei(K * N), K, N});
    else if (w4)
      pend.push_back({l, slot, takei(K * N / 2), K, N});
    else
      flinear(l, slot, K, N);
  };
  for (int l = 0; l < c.n_layers && rc == B200_OK; ++l) {
    B200_DO(b200_model_set_vector(m, l, B200_T_IN_NORM, takef(H), H));
    // Qwen3: the head norms follow the projection they normalise (in norm, Wq, q norm, Wk, k norm,
    // Wv, Wo, ...: the importer's order for transformers.Qwen3ForCausalLM)
    flinear(l, B200_T_Q, H, QD);
    if (c.qkv_bias) B200_DO(b200_model_set_vector(m, l, B200_T_Q_BIAS, takef(QD), QD));
    if (c.qk_norm) B200_DO(b200_model_set_vector(m, l, B200_T_Q_NORM, takef(D), D));
    flinear(l, B200_T_K, H, KD);
    if (c.qkv_bias) B200_DO(b200_model_set_vector(m, l, B200_T_K_BIAS, takef(KD), KD));
    if (c.qk_norm) B200_DO(b200_model_set_vector(m, l, B200_T_K_NORM, takef(D), D));
    flinear(l, B200_T_V, H, KD);
    if (c.qkv_bias) B200_DO(b200_model_set_vector(m, l, B200_T_V_BIAS, takef(KD), KD));
    qlinear(l, B200_T_O, QD, H);
    B200_DO(b200_model_set_vector(m, l, B200_T_POST_NORM, takef(H), H));
    qlinear(l, B200_T_GATE, H, F);
    qlinear(l, B200_T_UP, H, F);
    qlinear(l, B200_T_DOWN, F, H);
  }
  B200_DO(b200_model_set_vector(m, -1, B200_T_FINAL_NORM, takef(H), H));
  qlinear(-1, B200_T_LM_HEAD, H, V);
  B200_DO(b200_model_set_vector(m, -1, B200_T_INV_FREQ, takef(D / 2), D / 2));
  // quantize.py:577-589: the scaler params follow every original param, in
  // original-weight order.
  for (auto &p : pend) {
    if (w4) {
      // signed nibbles [K, N/2], per-channel f16 scales straight from the f16 blob
      const uint16_t *sc = f16_blob + (fp - fp0);
      fp += p.N;
      B200_DO(b200_model_set_linear(m, p.layer, p.slot, B200_W_U4, p.w, sc, B200_F16, 1, p.K, p.N, -1, 0));
    } else {
      B200_DO(b200_model_set_linear(m, p.layer, p.slot, B200_W_I8, p.w, takef(p.N),
                                    B200_F32, 1, p.K, p.N, -1, 0));
    }
  }
#undef B200_DO
  if (rc == B200_OK && w8q)
    m->act_int8 = true;
  return rc;
}

int b200_model_set_activation_int8(b200_model *m, int enabled) {
  if (!m)
    return fail(B200_EINVAL, "set_activation_int8: null model");
  if (enabled && m->tp != 1)
    return fail(B200_ESTATE, "set_activation_int8: single-GPU sessions only");
  m->act_int8 = enabled != 0;
  return B200_OK;
}
int b200_model_activation_int8(const b200_model *m) { return m && m->act_int8 ? 1 : 0; }

// Staging buffers for the peer-store sums: allocate this rank's, trade CUDA IPC
// handles through NCCL, map the peers'.  All ranks agree (a min-reduction) on
// whether the path is usable; otherwise every rank keeps the NCCL all-reduce.
static int tp_push_setup(b200_model *m) {
  const int tp = m->tp, H = m->cfg.hidden;
  const char *env = std::getenv("BUDDY_B200_TP_SUM");
  int ok = !(env && !strcmp(env, "nccl")) && tp <= kTpMaxRanks;
  cudaStream_t st = m->stream;
  // + one marker per rank for the handshake + two slots of (value, index) per rank for the argmax
  const size_t pairs = (size_t)kTpRegions * tp * H + kTpMaxRanks + 4 * kTpMaxRanks;
  m->tp_argmax_at = (size_t)kTpRegions * tp * H + kTpMaxRanks;
  char *d_send = nullptr, *d_recv = nullptr;
  float *d_flag = nullptr;
  if (int rc = dev_alloc((void **)&d_send, 64)) return rc;
  if (int rc = dev_alloc((void **)&d_recv, 64 * (size_t)tp)) return rc;
  if (int rc = dev_alloc((void **)&d_flag, 4)) return rc;
  cudaIpcMemHandle_t mine{};
  static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handle size");
  if (ok) {
    if (dev_alloc((void **)&m->tp_ll, pairs * sizeof(uint2)) != B200_OK ||
        cudaMemset(m->tp_ll, 0, pairs * sizeof(uint2)) != cudaSuccess ||
        cudaIpcGetMemHandle(&mine, m->tp_ll) != cudaSuccess) {
      (void)cudaGetLastError();
      ok = 0;
    }
  }
  B200_CUDA(cudaMemcpy(d_send, &mine, 64, cudaMemcpyHostToDevice));
  B200_NCCL(g_nccl.AllGather(d_send, d_recv, 64, 0 /* ncclChar */, g_nccl.comm, st));
  B200_CUDA(cudaStreamSynchronize(st));
  std::vector<cudaIpcMemHandle_t> all(tp);
  B200_CUDA(cudaMemcpy(all.data(), d_recv, 64 * (size_t)tp, cudaMemcpyDeviceToHost));
  TpPush push{};
  if (ok) {
    for (int r = 0; r < tp; ++r) {
      if (r == g_nccl.rank) {
        push.peer[r] = m->tp_ll;
        continue;
      }
      void *p = nullptr;
      if (cudaIpcOpenMemHandle(&p, all[r], cudaIpcMemLazyEnablePeerAccess) != cudaSuccess) {
        (void)cudaGetLastError();
        ok = 0;
        break;
      }
      m->tp_opened[r] = p;
      push.peer[r] = (uint2 *)p;
    }
  }
  if (ok) {
    // try the mappings once: a store to every peer, everybody's store seen here
    int *d_ok = nullptr;
    const int one = 1;
    if (int rc = dev_alloc((void **)&d_ok, 4)) return rc;
    B200_CUDA(cudaMemcpy(d_ok, &one, 4, cudaMemcpyHostToDevice));
    push.ranks = tp;
    push.rank = g_nccl.rank;
    tp_handshake_kernel<<<1, 32, 0, st>>>(push, (size_t)kTpRegions * tp * H, d_ok);
    int seen = 0;
    if (cudaStreamSynchronize(st) != cudaSuccess ||
        cudaMemcpy(&seen, d_ok, 4, cudaMemcpyDeviceToHost) != cudaSuccess) {
      (void)cudaGetLastError();
      seen = 0;
    }
    cudaFree(d_ok);
    ok = seen;
  }
  // every rank must take the same path (this also lines the ranks up before the first step)
  const float mine_ok = ok ? 1.f : 0.f;
  B200_CUDA(cudaMemcpy(d_flag, &mine_ok, 4, cudaMemcpyHostToDevice));
  B200_NCCL(g_nccl.AllReduce(d_flag, d_flag, 1, kNcclFloat, 3 /* ncclMin */, g_nccl.comm, st));
  B200_CUDA(cudaStreamSynchronize(st));
  float all_ok = 0.f;
  B200_CUDA(cudaMemcpy(&all_ok, d_flag, 4, cudaMemcpyDeviceToHost));
  cudaFree(d_send); cudaFree(d_recv); cudaFree(d_flag);
  if (all_ok > 0.5f) {
    push.ranks = tp;
    push.rank = g_nccl.rank;
    push.H = H;
    push.step = m->d_state + 7;
    push.per_step = 2 * m->cfg.n_layers;
    m->tp_push = push;
  } else {
    m->tp_push = TpPush{};
  }
  return B200_OK;
}

// ---- repack cache: the packed device layout of every tensor in one file ---------------------
// Quantising and packing a model's blobs takes seconds; the result depends only on the
// blobs, the configuration and the tensor-parallel rank.  b200_model_save_packed writes what
// set_linear / set_vector left on the device (before finalize, which fuses and frees the
// per-projection buffers); b200_model_load_packed fills a freshly created model from such a
// file, after which finalize runs as usual.  Layout: header {magic "B2PACK01", config bytes,
// tp size and rank, record count}, then records {layer, slot, is_linear, kind, group, K, N,
// scale dtype, byte counts of weights / scales / bias} each followed by its payloads.
namespace {
constexpr char kPackMagic[8] = {'B', '2', 'P', 'A', 'C', 'K', '0', '1'};
struct PackHeader {
  char magic[8];
  uint32_t config_bytes;
  int32_t tp, rank;
  uint32_t records;
  b200_model_config cfg;
};
struct PackRecord {
  int32_t layer, slot, is_linear, kind, group, scale_dtype;
  int64_t K, N;
  uint64_t w_bytes, scale_bytes, bias_bytes;
};

int write_device(FILE *f, const void *dev, uint64_t bytes, std::vector<char> &buf) {
  for (uint64_t off = 0; off < bytes; off += buf.size()) {
    const size_t n = (size_t)std::min<uint64_t>(buf.size(), bytes - off);
    B200_CUDA(cudaMemcpy(buf.data(), (const char *)dev + off, n, cudaMemcpyDeviceToHost));
    if (fwrite(buf.data(), 1, n, f) != n)
      return fail(B200_EINVAL, "save_packed: write failed");
  }
  return B200_OK;
}
int read_device(FILE *f, void **dev, uint64_t bytes, std::vector<char> &buf) {
  if (int rc = dev_alloc(dev, bytes)) return rc;
  for (uint64_t off = 0; off < bytes; off += buf.size()) {
    const size_t n = (size_t)std::min<uint64_t>(buf.size(), bytes - off);
    if (fread(buf.data(), 1, n, f) != n)
      return fail(B200_EINVAL, "load_packed: the file is truncated");
    B200_CUDA(cudaMemcpy((char *)*dev + off, buf.data(), n, cudaMemcpyHostToDevice));
  }
  return B200_OK;
}
struct VecSlot { int layer, slot; float **p; int64_t n; };
std::vector<VecSlot> vector_slots(b200_model *m) {
  const b200_model_config &c = m->cfg;
  std::vector<VecSlot> v = {{-1, B200_T_EMBED, &m->embed, (int64_t)c.vocab * c.hidden},
                            {-1, B200_T_INV_FREQ, &m->inv_freq, c.head_dim / 2},
                            {-1, B200_T_FINAL_NORM, &m->final_norm, c.hidden}};
  for (int l = 0; l < c.n_layers; ++l) {
    Layer &L = m->layers[l];
    v.push_back({l, B200_T_IN_NORM, &L.in_norm, c.hidden});
    v.push_back({l, B200_T_POST_NORM, &L.post_norm, c.hidden});
    v.push_back({l, B200_T_Q_NORM, &L.q_norm, c.head_dim});
    v.push_back({l, B200_T_K_NORM, &L.k_norm, c.head_dim});
  }
  return v;
}
constexpr int kLinearSlots[] = {B200_T_Q, B200_T_K, B200_T_V, B200_T_O, B200_T_GATE, B200_T_UP, B200_T_DOWN};
} // namespace

int b200_model_save_packed(b200_model *m, const char *path) {
  if (!m || !path)
    return fail(B200_EINVAL, "save_packed: null argument");
  if (m->finalized)
    return fail(B200_ESTATE, "save_packed: call it before finalize (finalize frees the per-projection buffers)");
  FILE *f = fopen(path, "wb");
  if (!f)
    return fail(B200_EINVAL, "save_packed: cannot create %s", path);
  std::vector<char> buf((size_t)64 << 20);
  std::vector<std::pair<PackRecord, DevLinear *>> lin;
  std::vector<std::pair<PackRecord, float *>> vec;
  for (const VecSlot &v : vector_slots(m))
    if (*v.p) {
      PackRecord r{};
      r.layer = v.layer; r.slot = v.slot; r.N = v.n; r.w_bytes = (uint64_t)v.n * 4;
      vec.push_back({r, *v.p});
    }
  auto add_linear = [&](int layer, int slot, DevLinear *L) {
    if (!L->set) return;
    PackRecord r{};
    r.layer = layer; r.slot = slot; r.is_linear = 1;
    r.kind = L->w.kind; r.group = L->w.group; r.scale_dtype = L->w.scale_dtype;
    r.K = L->w.K; r.N = L->w.N;
    r.w_bytes = (uint64_t)packed_row_bytes(L->w.kind, L->w.K) * L->w.N;
    const int64_t ng = (L->w.kind == B200_W_U4 && L->w.group > 0 && L->w.group < L->w.K) ? L->w.K / L->w.group : 1;
    r.scale_bytes = L->scale_buf ? (uint64_t)L->w.N * ng * (L->w.scale_dtype == B200_F32 ? 4 : 2) : 0;
    r.bias_bytes = L->bias_buf ? (uint64_t)L->w.N * 4 : 0;
    lin.push_back({r, L});
  };
  for (int l = 0; l < m->cfg.n_layers; ++l)
    for (int slot : kLinearSlots)
      add_linear(l, slot, linear_slot(m, l, slot));
  add_linear(-1, B200_T_LM_HEAD, &m->lm_head);
  PackHeader h{};
  memcpy(h.magic, kPackMagic, 8);
  h.config_bytes = sizeof(b200_model_config);
  h.tp = m->tp;
  h.rank = m->rank;
  h.records = (uint32_t)(vec.size() + lin.size());
  h.cfg = m->cfg;
  int rc = fwrite(&h, sizeof h, 1, f) == 1 ? B200_OK : fail(B200_EINVAL, "save_packed: write failed");
  for (auto &v : vec) {
    if (rc == B200_OK && fwrite(&v.first, sizeof(PackRecord), 1, f) != 1) rc = fail(B200_EINVAL, "save_packed: write failed");
    if (rc == B200_OK) rc = write_device(f, v.second, v.first.w_bytes, buf);
  }
  for (auto &l : lin) {
    if (rc == B200_OK && fwrite(&l.first, sizeof(PackRecord), 1, f) != 1) rc = fail(B200_EINVAL, "save_packed: write failed");
    if (rc == B200_OK) rc = write_device(f, l.second->w_buf, l.first.w_bytes, buf);
    if (rc == B200_OK && l.first.scale_bytes) rc = write_device(f, l.second->scale_buf, l.first.scale_bytes, buf);
    if (rc == B200_OK && l.first.bias_bytes) rc = write_device(f, l.second->bias_buf, l.first.bias_bytes, buf);
  }
  if (fclose(f) != 0 && rc == B200_OK)
    rc = fail(B200_EINVAL, "save_packed: close failed");
  if (rc != B200_OK)
    remove(path);
  return rc;
}

int b200_model_load_packed(b200_model *m, const char *path) {
  if (!m || !path)
    return fail(B200_EINVAL, "load_packed: null argument");
  if (m->finalized)
    return fail(B200_ESTATE, "load_packed: model already finalised");
  FILE *f = fopen(path, "rb");
  if (!f)
    return fail(B200_EINVAL, "load_packed: cannot open %s", path);
  std::vector<char> buf((size_t)64 << 20);
  PackHeader h{};
  int rc = B200_OK;
  if (fread(&h, sizeof h, 1, f) != 1 || memcmp(h.magic, kPackMagic, 8) != 0 ||
      h.config_bytes != sizeof(b200_model_config))
    rc = fail(B200_EINVAL, "load_packed: %s is not a packed-weights file of this library version", path);
  else if (memcmp(&h.cfg, &m->cfg, sizeof(b200_model_config)) != 0 || h.tp != m->tp || h.rank != m->rank)
    rc = fail(B200_EINVAL, "load_packed: the file was written for another configuration or tensor-parallel rank");
  const std::vector<VecSlot> vs = vector_slots(m);
  for (uint32_t i = 0; i < h.records && rc == B200_OK; ++i) {
    PackRecord r{};
    if (fread(&r, sizeof r, 1, f) != 1) {
      rc = fail(B200_EINVAL, "load_packed: the file is truncated");
      break;
    }
    if (!r.is_linear) {
      const VecSlot *slot = nullptr;
      for (const VecSlot &v : vs)
        if (v.layer == r.layer && v.slot == r.slot) slot = &v;
      if (!slot || r.N != slot->n || r.w_bytes != (uint64_t)slot->n * 4) {
        rc = fail(B200_EINVAL, "load_packed: unexpected vector record (layer %d, slot %d)", r.layer, r.slot);
        break;
      }
      if (*slot->p) { cudaFree(*slot->p); *slot->p = nullptr; }
      rc = read_device(f, (void **)slot->p, r.w_bytes, buf);
      continue;
    }
    DevLinear *L = linear_slot(m, r.layer, r.slot);
    if (!L || r.K < 1 || r.N < 1 || r.w_bytes != (uint64_t)packed_row_bytes(r.kind, r.K) * r.N) {
      rc = fail(B200_EINVAL, "load_packed: unexpected linear record (layer %d, slot %d)", r.layer, r.slot);
      break;
    }
    L->release();
    rc = read_device(f, &L->w_buf, r.w_bytes, buf);
    if (rc == B200_OK && r.scale_bytes) rc = read_device(f, &L->scale_buf, r.scale_bytes, buf);
    if (rc == B200_OK && r.bias_bytes) rc = read_device(f, (void **)&L->bias_buf, r.bias_bytes, buf);
    if (rc != B200_OK) { L->release(); break; }
    L->w = b200_weight{};
    L->w.kind = r.kind; L->w.group = r.group; L->w.K = r.K; L->w.N = r.N;
    L->w.w = L->w_buf; L->w.scale = L->scale_buf; L->w.scale_dtype = r.scale_dtype; L->w.bias = L->bias_buf;
    L->set = true;
  }
  fclose(f);
  return rc;
}

int b200_model_finalize(b200_model *m) {
  if (!m)
    return fail(B200_EINVAL, "finalize: null model");
  if (m->finalized)
    return B200_OK;
  const b200_model_config &c = m->cfg;
  if (!m->embed || !m->final_norm || !m->lm_head.set)
    return fail(B200_ESTATE, "finalize: embedding, final norm or lm_head missing");
  if (!m->inv_freq) {
    std::vector<float> f(c.head_dim / 2);
    for (int j = 0; j < c.head_dim / 2; ++j)
      f[j] = (float)(1.0 / std::pow((double)c.rope_theta, (2.0 * j) / c.head_dim));
    if (int rc = b200_model_set_vector(m, -1, B200_T_INV_FREQ, f.data(), f.size()))
      return rc;
  }
  for (int l = 0; l < c.n_layers; ++l) {
    Layer &L = m->layers[l];
    if (!L.in_norm || !L.post_norm || !L.q.set || !L.k.set || !L.v.set ||
        !L.o.set || !L.gate.set || !L.up.set || !L.down.set)
      return fail(B200_ESTATE, "finalize: layer %d is incomplete", l);
    if (c.qk_norm && (!L.q_norm || !L.k_norm))
      return fail(B200_ESTATE, "finalize: layer %d lacks q_norm/k_norm", l);
    if (int rc = fuse_linears({&L.q, &L.k, &L.v}, false, &L.qkv, m->stream)) return rc;
    if (int rc = fuse_linears({&L.gate, &L.up}, true, &L.gateup, m->stream)) return rc;
    L.q.release(); L.k.release(); L.v.release();
  }
  if (mega_eligible(m, m->layers[0]))
    if (int rc = build_mega(m)) return rc;
  for (auto &L : m->layers) { L.gate.release(); L.up.release(); }
  if (m->mega) {
    // warm the kernel once (shared-memory attribute, module load), then clear the row it wrote
    if (int rc = set_state(m, 0, 0)) return rc;
    if (int rc = run_step(m)) return rc;
    B200_CUDA(cudaMemcpyAsync(m->h_state_pinned, m->d_state, 32, cudaMemcpyDeviceToHost, m->stream));
    B200_CUDA(cudaStreamSynchronize(m->stream));
    if (int rc = check_step_error(m)) return rc;
    for (auto p : m->kv)
      B200_CUDA(cudaMemsetAsync(p, 0, (size_t)m->kvh * c.max_len * c.head_dim * 4, m->stream));
    B200_CUDA(cudaStreamSynchronize(m->stream));
    m->kernels_per_step = 1;
    m->finalized = true;
    return B200_OK;
  }
  if (m->tp > 1)
    if (int rc = tp_push_setup(m)) return rc;
  // Warm every kernel once outside capture (sets shared-memory attributes),
  // then capture the step.  This is the float-activation step; the step of the w8a8
  // arithmetic is captured when it is first run.
  struct FloatStep {
    b200_model *m;
    bool saved;
    explicit FloatStep(b200_model *mm) : m(mm), saved(mm->act_int8) { m->act_int8 = false; }
    ~FloatStep() { m->act_int8 = saved; }
  } float_step(m);
  if (int rc = set_state(m, 0, 0)) return rc;
  if (int rc = issue_step(m, &m->kernels_per_step)) return rc;
  B200_CUDA(cudaStreamSynchronize(m->stream));
  for (auto p : m->kv)  // the warm-up wrote row 0
    B200_CUDA(cudaMemsetAsync(p, 0, (size_t)m->kvh * c.max_len * c.head_dim * 4, m->stream));
  B200_CUDA(cudaStreamBeginCapture(m->stream, cudaStreamCaptureModeThreadLocal));
  int rc = issue_step(m, nullptr);
  cudaGraph_t g = nullptr;
  cudaError_t e = cudaStreamEndCapture(m->stream, &g);
  if (rc != B200_OK) {
    if (g) cudaGraphDestroy(g);
    return rc;
  }
  if (e != cudaSuccess)
    return fail(B200_ECUDA, "graph capture: %s", cudaGetErrorString(e));
  m->graph = g;
  B200_CUDA(cudaGraphInstantiate(&m->exec, m->graph, 0));
  B200_CUDA(cudaStreamSynchronize(m->stream));
  m->finalized = true;
  return B200_OK;
}

static int kv_copy(b200_model *m, int buffer, float *host, int pos0, int n_pos,
                   bool upload) {
  if (!m || !host || buffer < 0 || buffer >= (int)m->kv.size() || pos0 < 0 ||
      n_pos < 0 || pos0 + n_pos > m->cfg.max_len)
    return fail(B200_EINVAL, "kv copy: bad argument");
  if (n_pos == 0)
    return B200_OK;
  const int D = m->cfg.head_dim;
  const size_t pitch = (size_t)m->cfg.max_len * D * 4, width = (size_t)n_pos * D * 4;
  // this rank's kv heads out of the host's full [kv_heads, max_len, D]
  float *h0 = host + ((size_t)m->rank * m->kvh * m->cfg.max_len + pos0) * D;
  float *d0 = m->kv[buffer] + (size_t)pos0 * D;
  if (upload)
    B200_CUDA(cudaMemcpy2DAsync(d0, pitch, h0, pitch, width, m->kvh,
                                cudaMemcpyHostToDevice, m->stream));
  else
    B200_CUDA(cudaMemcpy2DAsync(h0, pitch, d0, pitch, width, m->kvh,
                                cudaMemcpyDeviceToHost, m->stream));
  B200_CUDA(cudaStreamSynchronize(m->stream));
  return B200_OK;
}
int b200_model_kv_upload(b200_model *m, int buffer, const float *host, int pos0,
                         int n_pos) {
  return kv_copy(m, buffer, const_cast<float *>(host), pos0, n_pos, true);
}
int b200_model_kv_download(b200_model *m, int buffer, float *host, int pos0,
                           int n_pos) {
  return kv_copy(m, buffer, host, pos0, n_pos, false);
}

int b200_model_decode(b200_model *m, int token, int pos, float *logits_host,
                      int *next_token) {
  if (!m)
    return fail(B200_EINVAL, "decode: null model");
  if (!m->finalized)
    return fail(B200_ESTATE, "decode: call b200_model_finalize first");
  if (token < 0 || token >= m->cfg.vocab || pos < 0 || pos >= m->cfg.max_len)
    return fail(B200_EINVAL, "decode: token %d / position %d out of range", token, pos);
  if (int rc = set_state(m, token, pos)) return rc;
  B200_CUDA(cudaEventRecord(m->ev0, m->stream));
  if (int rc = run_step(m)) return rc;
  B200_CUDA(cudaEventRecord(m->ev1, m->stream));
  m->rows_fresh = false;
  if (logits_host && m->tp > 1 && m->tp_push.ranks > 0)   // the step itself exchanged only (value, index)
    B200_NCCL(g_nccl.AllGather(m->logits_shard, m->logits, m->vocab, kNcclFloat, g_nccl.comm, m->stream));
  if (logits_host) {
    B200_CUDA(cudaMemcpyAsync(m->h_logits_pinned, m->logits, (size_t)m->cfg.vocab * 4,
                              cudaMemcpyDeviceToHost, m->stream));
    // a caller that wants the logits on the host usually mirrors the new K/V rows too:
    // they ride along, so that b200_model_read_new_kv_rows needs no second round trip
    B200_CUDA(cudaMemcpyAsync(m->h_rows_pinned, m->kv_stage,
                              (size_t)2 * m->cfg.n_layers * m->kvh * m->cfg.head_dim * 4,
                              cudaMemcpyDeviceToHost, m->stream));
  }
  B200_CUDA(cudaMemcpyAsync(m->h_state_pinned, m->d_state, 32, cudaMemcpyDeviceToHost, m->stream));
  B200_CUDA(cudaStreamSynchronize(m->stream));
  B200_CUDA(cudaEventElapsedTime(&m->last_ms, m->ev0, m->ev1));
  if (int rc = check_step_error(m)) return rc;
  if (logits_host) {
    memcpy(logits_host, m->h_logits_pinned, (size_t)m->cfg.vocab * 4);
    m->rows_fresh = true;
  }
  if (next_token)
    *next_token = m->h_state_pinned[2];
  return B200_OK;
}

int b200_model_generate(b200_model *m, int token, int pos, int steps,
                        int *tokens_out) {
  if (!m || !tokens_out)
    return fail(B200_EINVAL, "generate: null argument");
  if (!m->finalized)
    return fail(B200_ESTATE, "generate: call b200_model_finalize first");
  if (steps < 1 || steps > m->history_cap || token < 0 || token >= m->cfg.vocab ||
      pos < 0 || pos + steps > m->cfg.max_len)
    return fail(B200_EINVAL, "generate: %d steps from position %d exceed max_len %d",
                steps, pos, m->cfg.max_len);
  m->rows_fresh = false;
  if (int rc = set_state(m, token, pos)) return rc;
  B200_CUDA(cudaEventRecord(m->ev0, m->stream));
  for (int s = 0; s < steps; ++s)
    if (int rc = run_step(m)) return rc;
  B200_CUDA(cudaEventRecord(m->ev1, m->stream));
  B200_CUDA(cudaMemcpyAsync(tokens_out, m->d_history, (size_t)steps * 4,
                            cudaMemcpyDeviceToHost, m->stream));
  B200_CUDA(cudaMemcpyAsync(m->h_state_pinned, m->d_state, 32, cudaMemcpyDeviceToHost, m->stream));
  B200_CUDA(cudaStreamSynchronize(m->stream));
  B200_CUDA(cudaEventElapsedTime(&m->last_ms, m->ev0, m->ev1));
  return check_step_error(m);
}

// A W8A8 projection over M rows (QuantizedMatmulOp / QuantizedAddMMOp of the w8a8 graphs,
// frontend/Python/graph/transform/quantization/passes.py:54-140): the normalised rows are one
// activation tensor with one dynamic scale; the norm is an f32 kernel before it, the residual sum
// or the SiLU pair an f32 operation in the GEMM's store.
static int linear_rows_int8(b200_model *m, const DevLinear &L, const float *X, int64_t ldx, int M, float *Y,
                            int64_t ldy, const float *residual, const float *norm_w, bool silu) {
  cudaStream_t st = m->stream;
  const int64_t K = L.w.K;
  const float *A = X;
  int64_t lda = ldx;
  if (norm_w) {
    if (ldx != K)
      return fail(B200_EINVAL, "w8a8 projection: normalised rows must be contiguous");
    if (int rc = b200_rmsnorm(X, norm_w, m->pf_norm, M, K, m->cfg.eps, st)) return rc;
    A = m->pf_norm;
    lda = K;
  }
  return gemm_w8a8_fused(&L.w, A, M, lda, Y, ldy, residual, ldy, silu ? 1 : 0, m->pf_ws, m->pf_ws_bytes, st);
}

// One projection over M rows: the dense tensor-core GEMM for int8 per-channel
// weights, else the GEMV kernel sixteen rows at a time.
static int linear_rows(b200_model *m, const DevLinear &L, const float *X, int64_t ldx, int M, float *Y,
                       int64_t ldy, const float *residual, const float *norm_w, bool silu) {
  if (m->act_int8 && L.w.kind == B200_W_I8 && L.w.scale_dtype == B200_F32) {
    if (L.w.K % 64 != 0)
      return fail(B200_EINVAL, "w8a8 projection: K = %lld is not a multiple of 64", (long long)L.w.K);
    return linear_rows_int8(m, L, X, ldx, M, Y, ldy, residual, norm_w, silu);
  }
  if (L.w.kind == B200_W_I8 && L.w.scale_dtype == B200_F32 && L.w.K % 64 == 0)
    return b200_gemm_w8(&L.w, X, M, ldx, Y, ldy, residual, ldy, norm_w, m->cfg.eps, silu ? 1 : 0, m->pf_ws,
                        m->pf_ws_bytes, m->stream);
  for (int m0 = 0; m0 < M; m0 += 16) {
    b200_gemv_args a{};
    a.x = X + (int64_t)m0 * ldx;
    a.x_dtype = B200_F32;
    a.y_dtype = B200_F32;
    a.x_ld = ldx;
    a.y_ld = ldy;
    a.y = Y + (int64_t)m0 * ldy;
    a.residual = residual ? residual + (int64_t)m0 * ldy : nullptr;
    a.norm_weight = norm_w;
    a.norm_eps = m->cfg.eps;
    a.M = M - m0 < 16 ? M - m0 : 16;
    a.silu_pairs = silu ? 1 : 0;
    if (int rc = b200_gemv(&L.w, &a, m->stream)) return rc;
  }
  return B200_OK;
}

static int prefill_reserve(b200_model *m, int rows, int logit_rows) {
  const b200_model_config &c = m->cfg;
  const int D = c.head_dim;
  const int64_t QKV = (int64_t)(m->qh + 2 * m->kvh) * D;
  if (m->act_int8 && !m->pf_norm && rows < m->pf_rows)   // switched on after a first pass: regrow with its buffers
    rows = m->pf_rows;
  if (rows > m->pf_rows || (m->act_int8 && !m->pf_norm)) {
    cudaFree(m->pf_x); cudaFree(m->pf_qkv); cudaFree(m->pf_att); cudaFree(m->pf_mid); cudaFree(m->pf_ws);
    cudaFree(m->pf_tokens); cudaFree(m->pf_norm);
    m->pf_x = m->pf_qkv = m->pf_att = m->pf_mid = m->pf_norm = nullptr;
    m->pf_ws = nullptr;
    m->pf_tokens = nullptr;
    m->pf_rows = 0;
    int64_t Kmax = c.hidden > m->ffn ? c.hidden : m->ffn;
    if ((int64_t)m->qh * D > Kmax) Kmax = (int64_t)m->qh * D;
    m->pf_ws_bytes = std::max(b200_gemm_w8_workspace_bytes(rows, Kmax), b200_gemm_w8a8_workspace_bytes(rows, Kmax));
    if (int rc = dev_alloc((void **)&m->pf_x, (size_t)rows * c.hidden * 4)) return rc;
    if (int rc = dev_alloc((void **)&m->pf_qkv, (size_t)rows * QKV * 4)) return rc;
    if (int rc = dev_alloc((void **)&m->pf_att, (size_t)rows * m->qh * D * 4)) return rc;
    if (int rc = dev_alloc((void **)&m->pf_mid, (size_t)rows * m->ffn * 4)) return rc;
    if (int rc = dev_alloc(&m->pf_ws, (size_t)m->pf_ws_bytes)) return rc;
    B200_CUDA(cudaMemset(m->pf_ws, 0, 256));   // the GEMM's error word (float projections never touch it)
    if (int rc = dev_alloc((void **)&m->pf_tokens, (size_t)rows * 4)) return rc;
    if (m->act_int8)
      if (int rc = dev_alloc((void **)&m->pf_norm, (size_t)rows * c.hidden * 4)) return rc;
    m->pf_rows = rows;
  }
  if (logit_rows > m->pf_logit_rows) {
    cudaFree(m->pf_logits);
    m->pf_logits = nullptr;
    m->pf_logit_rows = 0;
    if (int rc = dev_alloc((void **)&m->pf_logits, (size_t)logit_rows * c.vocab * 4)) return rc;
    m->pf_logit_rows = logit_rows;
  }
  return B200_OK;
}

int b200_model_prefill(b200_model *m, const int32_t *tokens, int n_tokens, int pos0, float *logits_host,
                       int all_rows, int *next_token) {
  if (!m || !tokens)
    return fail(B200_EINVAL, "prefill: null argument");
  if (!m->finalized)
    return fail(B200_ESTATE, "prefill: call b200_model_finalize first");
  if (m->tp != 1)
    return fail(B200_ESTATE, "prefill: single-GPU sessions only (tensor-parallel sessions feed the prompt through decode)");
  const b200_model_config &c = m->cfg;
  if (n_tokens < 1 || pos0 < 0 || pos0 + n_tokens > c.max_len)
    return fail(B200_EINVAL, "prefill: %d rows from position %d exceed max_len %d", n_tokens, pos0, c.max_len);
  for (int i = 0; i < n_tokens; ++i)
    if (tokens[i] < 0 || tokens[i] >= c.vocab)
      return fail(B200_EINVAL, "prefill: token %d at row %d out of range", tokens[i], i);
  const int M = n_tokens, D = c.head_dim, H = c.hidden;
  const int64_t QD = (int64_t)m->qh * D, KD = (int64_t)m->kvh * D, QKV = QD + 2 * KD;
  // w8a8: the activation scale of the last projection belongs to all rows, so all of them are computed
  const int logit_rows = ((all_rows && logits_host) || m->act_int8) ? M : 1;
  if (int rc = prefill_reserve(m, M, logit_rows)) return rc;
  cudaStream_t st = m->stream;
  B200_CUDA(cudaEventRecord(m->ev0, st));
  B200_CUDA(cudaMemcpyAsync(m->pf_tokens, tokens, (size_t)M * 4, cudaMemcpyHostToDevice, st));
  if (int rc = embed_rows_launch(m->embed, m->pf_tokens, m->pf_x, H, M, st)) return rc;
  for (int l = 0; l < c.n_layers; ++l) {
    Layer &L = m->layers[l];
    // q | k | v (+ bias) <- RMSNorm(x)
    if (int rc = linear_rows(m, L.qkv, m->pf_x, H, M, m->pf_qkv, QKV, nullptr, L.in_norm, false)) return rc;
    if (int rc = rope_kv_rows_launch(m->pf_qkv, QKV, m->kv[2 * l], m->kv[2 * l + 1], m->inv_freq, L.q_norm,
                                     L.k_norm, c.eps, m->qh, m->kvh, D, c.max_len, pos0, M, st))
      return rc;
    if (int rc = gqa_prefill_launch(m->pf_qkv, QKV, m->kv[2 * l], m->kv[2 * l + 1], m->pf_att, QD, m->qh,
                                    m->kvh, D, c.max_len, pos0, M, st))
      return rc;
    // x1 = x + attn @ Wo ; mid = silu(gate) * up <- RMSNorm(x1) ; x2 = x1 + mid @ Wdown
    if (int rc = linear_rows(m, L.o, m->pf_att, QD, M, m->pf_x, H, m->pf_x, nullptr, false)) return rc;
    if (int rc = linear_rows(m, L.gateup, m->pf_x, H, M, m->pf_mid, m->ffn, nullptr, L.post_norm, true)) return rc;
    if (int rc = linear_rows(m, L.down, m->pf_mid, m->ffn, M, m->pf_x, H, m->pf_x, nullptr, false)) return rc;
  }
  // logits: every row, or the last one only
  const int first = logit_rows == M ? 0 : M - 1;
  if (int rc = linear_rows(m, m->lm_head, m->pf_x + (int64_t)first * H, H, logit_rows, m->pf_logits, c.vocab,
                           nullptr, m->final_norm, false))
    return rc;
  // greedy token of the last row, and the device state a following decode / generate continues from
  const float *last_logits = m->pf_logits + (int64_t)(logit_rows - 1) * c.vocab;
  if (int rc = b200_argmax_first(last_logits, c.vocab, m->d_state + 2, m->argmax_scratch, st)) return rc;
  m->h_state_pinned[0] = 0;
  m->h_state_pinned[1] = pos0 + M;
  B200_CUDA(cudaMemcpyAsync(m->d_state + 1, m->h_state_pinned + 1, 4, cudaMemcpyHostToDevice, st));
  B200_CUDA(cudaEventRecord(m->ev1, st));
  if (logits_host && all_rows)
    B200_CUDA(cudaMemcpyAsync(logits_host, m->pf_logits, (size_t)logit_rows * c.vocab * 4, cudaMemcpyDeviceToHost, st));
  else if (logits_host)
    B200_CUDA(cudaMemcpyAsync(logits_host, last_logits, (size_t)c.vocab * 4, cudaMemcpyDeviceToHost, st));
  B200_CUDA(cudaMemcpyAsync(m->h_state_pinned, m->d_state, 32, cudaMemcpyDeviceToHost, st));
  B200_CUDA(cudaStreamSynchronize(st));
  B200_CUDA(cudaEventElapsedTime(&m->last_ms, m->ev0, m->ev1));
  m->rows_fresh = false;
  if (int rc = b200_gemm_w8_status(m->pf_ws, st)) return rc;
  if (next_token)
    *next_token = m->h_state_pinned[2];
  return B200_OK;
}

// ---- batched decode over a paged KV cache ------------------------------------------------
struct b200_batch {
  b200_model *m = nullptr;
  int max_seqs = 0, page = 0, n_pages = 0, table_stride = 0;
  std::vector<float *> pool;            // [2 * layers] page pools [n_pages][kv_heads][page][D]
  std::vector<int> free_pages;
  std::vector<int> len;                 // per sequence: -1 = unused slot
  std::vector<int32_t> table;           // [max_seqs][table_stride] host mirror
  int32_t *d_table = nullptr, *d_seq = nullptr, *d_pos = nullptr, *d_next = nullptr;
  float *d_part = nullptr;              // attention partials of the key-split scan, for up to part_rows rows
  int part_rows = 0, max_context = 0;
  int rows_cap = 0;
  float last_ms = 0.f;
};

static int batch_rows(b200_batch *b, int M, const int32_t *tokens, const int32_t *row_seq, const int32_t *row_pos,
                      bool all_logits, float *logits_host, int32_t *next_host) {
  b200_model *m = b->m;
  // A w8a8 projection scales its whole activation tensor: rows of unrelated sequences in one
  // batch would share that scale, and each sequence's result would depend on its neighbours.
  if (m->act_int8)
    return fail(B200_ESTATE, "batch: the w8a8 arithmetic is defined per sequence (one prefill or decode tensor at a time)");
  const b200_model_config &c = m->cfg;
  const int D = c.head_dim, H = c.hidden;
  const int64_t QD = (int64_t)m->qh * D, KD = (int64_t)m->kvh * D, QKV = QD + 2 * KD;
  const int logit_rows = all_logits ? M : 1;
  if (int rc = prefill_reserve(m, M, logit_rows)) return rc;
  cudaStream_t st = m->stream;
  if (M > b->rows_cap) {
    cudaFree(b->d_seq); cudaFree(b->d_pos); cudaFree(b->d_next);
    b->d_seq = b->d_pos = b->d_next = nullptr;
    b->rows_cap = 0;
    if (int rc = dev_alloc((void **)&b->d_seq, (size_t)M * 4)) return rc;
    if (int rc = dev_alloc((void **)&b->d_pos, (size_t)M * 4)) return rc;
    if (int rc = dev_alloc((void **)&b->d_next, (size_t)M * 4)) return rc;
    b->rows_cap = M;
  }
  B200_CUDA(cudaEventRecord(m->ev0, st));
  B200_CUDA(cudaMemcpyAsync(m->pf_tokens, tokens, (size_t)M * 4, cudaMemcpyHostToDevice, st));
  B200_CUDA(cudaMemcpyAsync(b->d_seq, row_seq, (size_t)M * 4, cudaMemcpyHostToDevice, st));
  B200_CUDA(cudaMemcpyAsync(b->d_pos, row_pos, (size_t)M * 4, cudaMemcpyHostToDevice, st));
  B200_CUDA(cudaMemcpyAsync(b->d_table, b->table.data(), b->table.size() * 4, cudaMemcpyHostToDevice, st));
  bool one_chunk = M >= 64;
  for (int r = 1; r < M && one_chunk; ++r)
    one_chunk = row_seq[r] == row_seq[0] && row_pos[r] == row_pos[0] + r;
  if (int rc = embed_rows_launch(m->embed, m->pf_tokens, m->pf_x, H, M, st)) return rc;
  for (int l = 0; l < c.n_layers; ++l) {
    Layer &L = m->layers[l];
    if (int rc = linear_rows(m, L.qkv, m->pf_x, H, M, m->pf_qkv, QKV, nullptr, L.in_norm, false)) return rc;
    if (int rc = rope_kv_paged_launch(m->pf_qkv, QKV, b->pool[2 * l], b->pool[2 * l + 1], m->inv_freq, L.q_norm,
                                      L.k_norm, c.eps, m->qh, m->kvh, D, b->page, b->d_seq, b->d_pos, b->d_table,
                                      b->table_stride, M, st))
      return rc;
    int arc = B200_ESTATE;
    if (one_chunk)   // a prefill chunk: consecutive positions of one sequence
      arc = gqa_paged_prefill_launch(m->pf_qkv, QKV, b->pool[2 * l], b->pool[2 * l + 1], m->pf_att, QD, m->qh, m->kvh,
                                     D, b->page, b->d_table + (size_t)row_seq[0] * b->table_stride, row_pos[0], M,
                                     b->max_context, st);
    if (arc == B200_ESTATE)
      arc = gqa_paged_launch(m->pf_qkv, QKV, b->pool[2 * l], b->pool[2 * l + 1], m->pf_att, QD, m->qh, m->kvh, D,
                             b->page, b->d_seq, b->d_pos, b->d_table, b->table_stride, M, b->d_part, b->part_rows,
                             b->max_context, st);
    if (arc)
      return arc;
    if (int rc = linear_rows(m, L.o, m->pf_att, QD, M, m->pf_x, H, m->pf_x, nullptr, false)) return rc;
    if (int rc = linear_rows(m, L.gateup, m->pf_x, H, M, m->pf_mid, m->ffn, nullptr, L.post_norm, true)) return rc;
    if (int rc = linear_rows(m, L.down, m->pf_mid, m->ffn, M, m->pf_x, H, m->pf_x, nullptr, false)) return rc;
  }
  const int first = all_logits ? 0 : M - 1;
  if (int rc = linear_rows(m, m->lm_head, m->pf_x + (int64_t)first * H, H, logit_rows, m->pf_logits, c.vocab, nullptr,
                           m->final_norm, false))
    return rc;
  if (int rc = argmax_rows_launch(m->pf_logits, c.vocab, logit_rows, b->d_next, st)) return rc;
  B200_CUDA(cudaEventRecord(m->ev1, st));
  if (logits_host)
    B200_CUDA(cudaMemcpyAsync(logits_host, m->pf_logits, (size_t)logit_rows * c.vocab * 4, cudaMemcpyDeviceToHost, st));
  if (next_host)
    B200_CUDA(cudaMemcpyAsync(next_host, b->d_next, (size_t)logit_rows * 4, cudaMemcpyDeviceToHost, st));
  B200_CUDA(cudaStreamSynchronize(st));
  B200_CUDA(cudaEventElapsedTime(&b->last_ms, m->ev0, m->ev1));
  return b200_gemm_w8_status(m->pf_ws, st);
}

// pages for positions [len, len + n) of a sequence
static int batch_grow(b200_batch *b, int seq, int n) {
  const int have = (b->len[seq] + b->page - 1) / b->page, want = (b->len[seq] + n + b->page - 1) / b->page;
  if (want > b->table_stride)
    return fail(B200_ELIMIT, "batch: sequence %d would exceed the context limit of %d positions", seq,
                b->table_stride * b->page);
  if (want - have > (int)b->free_pages.size())
    return fail(B200_ENOMEM, "batch: the page pool is exhausted (%d pages)", b->n_pages);
  for (int i = have; i < want; ++i) {
    b->table[(size_t)seq * b->table_stride + i] = b->free_pages.back();
    b->free_pages.pop_back();
  }
  return B200_OK;
}

int b200_batch_create(b200_model *m, int max_seqs, int page_size, int n_pages, int max_context, b200_batch **out) {
  if (!m || !out || max_seqs < 1 || page_size < 1 || n_pages < 1 || max_context < 1)
    return fail(B200_EINVAL, "batch_create: bad argument");
  if (!m->finalized || m->tp != 1)
    return fail(B200_ESTATE, "batch_create: a finalised single-GPU model is required");
  b200_batch *b = new b200_batch();
  b->m = m;
  b->max_seqs = max_seqs;
  b->page = page_size;
  b->n_pages = n_pages;
  b->table_stride = (max_context + page_size - 1) / page_size;
  b->len.assign(max_seqs, -1);
  b->table.assign((size_t)max_seqs * b->table_stride, 0);
  for (int i = n_pages - 1; i >= 0; --i)
    b->free_pages.push_back(i);
  const size_t pool_bytes = (size_t)n_pages * m->kvh * page_size * m->cfg.head_dim * 4;
  b->pool.assign(2 * m->cfg.n_layers, nullptr);
  int rc = B200_OK;
  for (auto &p : b->pool)
    if (rc == B200_OK) rc = dev_alloc((void **)&p, pool_bytes);
  if (rc == B200_OK) rc = dev_alloc((void **)&b->d_table, b->table.size() * 4);
  b->max_context = b->table_stride * page_size;
  b->part_rows = max_seqs;
  if (rc == B200_OK)
    rc = dev_alloc((void **)&b->d_part,
                   (size_t)gqa_paged_scratch_floats(b->part_rows, m->qh, m->cfg.head_dim, b->max_context) * 4);
  if (rc == B200_OK && cudaMemset(b->d_part, 0, (size_t)b->part_rows * m->qh * 4) != cudaSuccess)   // the counters
    rc = fail(B200_ECUDA, "batch_create: cudaMemset failed");
  if (rc != B200_OK) {
    b200_batch_destroy(b);
    return rc;
  }
  *out = b;
  return B200_OK;
}

void b200_batch_destroy(b200_batch *b) {
  if (!b) return;
  for (auto p : b->pool) cudaFree(p);
  cudaFree(b->d_table); cudaFree(b->d_seq); cudaFree(b->d_pos); cudaFree(b->d_next);
  cudaFree(b->d_part);
  delete b;
}

int b200_batch_add(b200_batch *b, int *seq) {
  if (!b || !seq)
    return fail(B200_EINVAL, "batch_add: null argument");
  for (int i = 0; i < b->max_seqs; ++i)
    if (b->len[i] < 0) {
      b->len[i] = 0;
      *seq = i;
      return B200_OK;
    }
  return fail(B200_ELIMIT, "batch_add: all %d sequence slots are in use", b->max_seqs);
}

int b200_batch_remove(b200_batch *b, int seq) {
  if (!b || seq < 0 || seq >= b->max_seqs || b->len[seq] < 0)
    return fail(B200_EINVAL, "batch_remove: no such sequence");
  const int pages = (b->len[seq] + b->page - 1) / b->page;
  for (int i = 0; i < pages; ++i)
    b->free_pages.push_back(b->table[(size_t)seq * b->table_stride + i]);
  b->len[seq] = -1;
  return B200_OK;
}

int b200_batch_length(const b200_batch *b, int seq) {
  return (b && seq >= 0 && seq < b->max_seqs) ? b->len[seq] : -1;
}
int b200_batch_free_pages(const b200_batch *b) { return b ? (int)b->free_pages.size() : 0; }
float b200_batch_last_ms(const b200_batch *b) { return b ? b->last_ms : 0.f; }

int b200_batch_prefill(b200_batch *b, int seq, const int32_t *tokens, int n, float *logits_host, int *next_token) {
  if (!b || !tokens || n < 1 || seq < 0 || seq >= b->max_seqs || b->len[seq] < 0)
    return fail(B200_EINVAL, "batch_prefill: bad argument");
  for (int i = 0; i < n; ++i)
    if (tokens[i] < 0 || tokens[i] >= b->m->cfg.vocab)
      return fail(B200_EINVAL, "batch_prefill: token %d at row %d out of range", tokens[i], i);
  if (int rc = batch_grow(b, seq, n)) return rc;
  std::vector<int32_t> rs((size_t)n, seq), rp((size_t)n);
  for (int i = 0; i < n; ++i)
    rp[(size_t)i] = b->len[seq] + i;
  int32_t nxt = 0;
  if (int rc = batch_rows(b, n, tokens, rs.data(), rp.data(), false, logits_host, &nxt)) return rc;
  b->len[seq] += n;
  if (next_token) *next_token = nxt;
  return B200_OK;
}

int b200_batch_decode(b200_batch *b, int n, const int *seqs, const int32_t *tokens, float *logits_host,
                      int32_t *next_tokens) {
  if (!b || !seqs || !tokens || n < 1 || n > b->max_seqs)
    return fail(B200_EINVAL, "batch_decode: bad argument");
  std::vector<int32_t> rs((size_t)n), rp((size_t)n);
  std::vector<char> seen((size_t)b->max_seqs, 0);
  for (int i = 0; i < n; ++i) {
    const int s = seqs[i];
    if (s < 0 || s >= b->max_seqs || b->len[s] < 0 || seen[(size_t)s])
      return fail(B200_EINVAL, "batch_decode: sequence %d is unknown or listed twice", s);
    if (tokens[i] < 0 || tokens[i] >= b->m->cfg.vocab)
      return fail(B200_EINVAL, "batch_decode: token %d of sequence %d out of range", tokens[i], s);
    seen[(size_t)s] = 1;
  }
  for (int i = 0; i < n; ++i)
    if (int rc = batch_grow(b, seqs[i], 1)) return rc;
  for (int i = 0; i < n; ++i) {
    rs[(size_t)i] = seqs[i];
    rp[(size_t)i] = b->len[seqs[i]];
  }
  if (int rc = batch_rows(b, n, tokens, rs.data(), rp.data(), true, logits_host, next_tokens)) return rc;
  for (int i = 0; i < n; ++i)
    b->len[seqs[i]] += 1;
  return B200_OK;
}

int b200_model_read_new_kv_rows(b200_model *m, float *host) {
  if (!m || !host)
    return fail(B200_EINVAL, "read_new_kv_rows: null argument");
  if (m->rows_fresh) {   // fetched with the last decode's logits
    memcpy(host, m->h_rows_pinned, (size_t)2 * m->cfg.n_layers * m->kvh * m->cfg.head_dim * 4);
    return B200_OK;
  }
  B200_CUDA(cudaMemcpyAsync(host, m->kv_stage,
                            (size_t)2 * m->cfg.n_layers * m->kvh * m->cfg.head_dim * 4,
                            cudaMemcpyDeviceToHost, m->stream));
  B200_CUDA(cudaStreamSynchronize(m->stream));
  return B200_OK;
}

float b200_model_last_ms(const b200_model *m) { return m ? m->last_ms : 0.f; }
int b200_model_kernels_per_step(const b200_model *m) { return m ? m->kernels_per_step : 0; }
float *b200_model_kv_ptr(b200_model *m, int buffer) {
  return (m && buffer >= 0 && buffer < (int)m->kv.size()) ? m->kv[buffer] : nullptr;
}

int b200_model_uses_persistent_kernel(const b200_model *m) { return m && m->mega ? 1 : 0; }
// Diagnostic: move the persistent kernel's launch counter, the base of the 32-bit tags its
// CTAs exchange activations under (tag = (launches + 1) * 8 * (layers + 3) + phase), so that
// the wrap of the tag space (after 2^32 / (8 * (layers + 3)) launches, 17 million tokens for
// 28 layers) can be crossed in a test instead of in the fifth hour of a server's life.
int b200_model_set_launch_counter(b200_model *m, uint32_t launches) {
  if (!m || !m->finalized)
    return fail(B200_ESTATE, "set_launch_counter: a finalised model is required");
  if (!m->mega)
    return fail(B200_ESTATE, "set_launch_counter: the model does not run the persistent kernel");
  B200_CUDA(cudaStreamSynchronize(m->stream));
  m->h_state_pinned[4] = (int32_t)launches;
  B200_CUDA(cudaMemcpyAsync(m->d_state + 4, m->h_state_pinned + 4, 4, cudaMemcpyHostToDevice, m->stream));
  B200_CUDA(cudaStreamSynchronize(m->stream));
  return B200_OK;
}
int b200_model_tp_sum_kind(const b200_model *m) {
  return !m || m->tp <= 1 ? 0 : (m->tp_push.ranks > 0 ? 2 : 1);
}

int b200_model_read_trace(b200_model *m, long long *host, int64_t capacity) {
  if (!m || !host || !m->d_trace)
    return fail(B200_ESTATE, "read_trace: tracing is off (set BUDDY_B200_TRACE=<cta stride>)");
  const int64_t n = (int64_t)(m->mega_grid / m->mp.trace_stride + 1) * (m->cfg.n_layers + 1) * kMegaTraceSlots;
  B200_CUDA(cudaMemcpy(host, m->d_trace, (size_t)(n < capacity ? n : capacity) * 8,
                       cudaMemcpyDeviceToHost));
  return (int)(n < capacity ? n : capacity);
}

int64_t b200_model_step_bytes(const b200_model *m, int ctx) {
  if (!m) return 0;
  const b200_model_config &c = m->cfg;
  int64_t b = 0;
  for (const auto &L : m->layers) {
    b += L.qkv.bytes() + L.o.bytes() + L.gateup.bytes() + L.down.bytes();
    b += 2 * (int64_t)c.hidden * 4;  // two RMSNorm weights
    if (L.q_norm) b += 2 * (int64_t)c.head_dim * 4;
  }
  b += m->lm_head.bytes() + (int64_t)c.hidden * 4;  // final norm
  b += (int64_t)c.hidden * 4 + (int64_t)c.head_dim / 2 * 4;  // embedding row, inv_freq
  // live KV rows read by attention + the row written this step
  b += (int64_t)c.n_layers * 2 * m->kvh * c.head_dim * 4 * ((int64_t)ctx + 1);
  return b;
}

int b200_model_kv_overflow(b200_model *m, int position, int keep, float theta,
                           int *new_position) {
  if (!m || !new_position)
    return fail(B200_EINVAL, "model_kv_overflow: null argument");
  if (int rc = b200_kv_overflow(m->kv_dev, (int)m->kv.size(), m->kvh, m->cfg.max_len,
                                m->cfg.head_dim, position, keep, theta, new_position,
                                m->stream))
    return rc;
  B200_CUDA(cudaStreamSynchronize(m->stream));
  return B200_OK;
}

} // extern "C"
