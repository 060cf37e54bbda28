// Weight preparation on the device: the reference's quantiser, its nibble
// packing, and the repack between the reference's [K,N] layout and the packed
// device layout.  All integer/byte work here is bit-exact against the
// reference's definitions:
//   tools/buddy-codegen/import_model.py:790-892  (scales, rounding, clamping)
//   tools/buddy-codegen/import_model.py:810-815  (two nibbles per byte)
//   frontend/Python/ops/tosa.py:12158-12203      (sign-extending unpack)
#include "common.cuh"

#include <mutex>

namespace b200 {

static thread_local char t_err[512];
char *error_buffer() { return t_err; }
std::atomic<uint64_t> g_launches{0};

int fail(int code, const char *fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(t_err, sizeof(t_err), fmt, ap);
  va_end(ap);
  return code;
}

int ensure_device() {
  static std::once_flag once;
  static int status = B200_OK;
  std::call_once(once, [] {
    int n = 0;
    cudaError_t e = cudaGetDeviceCount(&n);
    if (e != cudaSuccess || n == 0) {
      status = B200_ENODEV;
      (void)cudaGetLastError();
    }
  });
  if (status != B200_OK)
    return fail(B200_ENODEV,
                "no CUDA device: buddy_b200 has no CPU path and cannot run");
  return B200_OK;
}

// ---- per-output-channel quantiser -----------------------------------------
__global__ void absmax_cols_kernel(const float *W, int64_t K, int64_t N,
                                   int64_t rows_per_slice, uint32_t *amax) {
  const int64_t n = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (n >= N)
    return;
  const int64_t k0 = (int64_t)blockIdx.y * rows_per_slice;
  const int64_t k1 = min(K, k0 + rows_per_slice);
  float a = 0.f;
  for (int64_t k = k0; k < k1; ++k)
    a = fmaxf(a, fabsf(W[k * N + n]));
  // non-negative floats order like their bit patterns
  atomicMax(&amax[n], __float_as_uint(a));
}

__global__ void scale_from_amax_kernel(float *scale, int64_t N, float qmax) {
  const int64_t n = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (n < N)
    scale[n] = fmaxf(__fdiv_rn(scale[n], qmax), 1e-10f);
}

__global__ void quantize_cols_kernel(const float *W, const float *scale,
                                     int64_t K, int64_t N, float lo, float hi,
                                     int8_t *Q) {
  const int64_t n = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const int64_t k = blockIdx.y;
  if (n >= N)
    return;
  const float r = rintf(__fdiv_rn(W[k * N + n], scale[n]));
  Q[k * N + n] = (int8_t)fminf(fmaxf(r, lo), hi);
}

// ---- group-wise zero-point-8 int4 quantiser ---------------------------------
__global__ void quantize_w4_group_kernel(const float *W, int64_t K, int64_t N,
                                         int64_t G, uint8_t *P,
                                         __half *scales) {
  const int64_t pair = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const int64_t g = blockIdx.y;
  if (pair >= N / 2)
    return;
  float s[2];
  for (int c = 0; c < 2; ++c) {
    const int64_t n = 2 * pair + c;
    float a = 0.f;
    for (int64_t k = g * G; k < (g + 1) * G; ++k)
      a = fmaxf(a, fabsf(W[k * N + n]));
    __half h = __float2half_rn(fmaxf(__fdiv_rn(a, 7.0f), 1e-10f));
    if (__half2float(h) == 0.0f)
      h = __ushort_as_half((unsigned short)1);
    scales[g * N + n] = h;
    s[c] = __half2float(h);
  }
  for (int64_t k = g * G; k < (g + 1) * G; ++k) {
    uint32_t u[2];
    for (int c = 0; c < 2; ++c) {
      float r = rintf(__fdiv_rn(W[k * N + 2 * pair + c], s[c]));
      r = fminf(fmaxf(r, -8.f), 7.f);
      u[c] = (uint32_t)((int)r + 8) & 0xF;
    }
    P[k * (N / 2) + pair] = (uint8_t)(u[0] | (u[1] << 4));
  }
}

// ---- nibble pack / unpack ----------------------------------------------------
__global__ void pack_int4_kernel(const int8_t *flat, int64_t nbytes,
                                 int8_t *packed) {
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= nbytes)
    return;
  const uint32_t lo = (uint8_t)flat[2 * i] & 0x0Fu;
  const uint32_t hi = ((uint8_t)flat[2 * i + 1] & 0x0Fu) << 4;
  packed[i] = (int8_t)(lo | hi);
}

__global__ void unpack_int4_kernel(const int8_t *packed, int64_t nbytes,
                                   int8_t *flat) {
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= nbytes)
    return;
  const int b = packed[i];
  flat[2 * i] = (int8_t)(((b & 0x0F) ^ 8) - 8);  // sign-extend the low nibble
  flat[2 * i + 1] = (int8_t)(b >> 4);            // arithmetic shift
}

// ---- reference [K,N] <-> packed device rows ---------------------------------
// One thread per (output row n, 16-byte unit); n is the fast index so the
// reads of the [K,N] source are coalesced.
template <int KIND>
__global__ void pack_weight_kernel(const uint8_t *src, int64_t K, int64_t N,
                                   int src_signed, uint8_t *dst,
                                   int64_t row_bytes) {
  constexpr int E = KIND == B200_W_I8 ? 16 : (KIND == B200_W_U4 ? 32 : 4);
  constexpr int G = KIND == B200_W_I8 ? 4 : (KIND == B200_W_U4 ? 8 : 1);
  const int64_t n = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const int64_t unit = blockIdx.y;
  if (n >= N)
    return;
  const int64_t Kp = packed_k(KIND, K);
  const int64_t b = unit / 32, l = unit % 32;
  const int64_t k0 = b * 32 * E;
  const int64_t Bs = min((int64_t)32 * E, Kp - k0);
  const int64_t q = Bs / G;
  uint32_t out[4] = {0, 0, 0, 0};
#pragma unroll
  for (int j = 0; j < G; ++j)
#pragma unroll
    for (int el = 0; el < 4; ++el) {
      const int64_t k = k0 + j * q + 4 * l + el;
      if (KIND == B200_W_I8) {
        const uint32_t v = k < K ? src[k * N + n] : 0u;
        out[j] |= v << (8 * el);
      } else if (KIND == B200_W_U4) {
        uint32_t v = 8u;  // zero-point: contributes nothing
        if (k < K) {
          const uint32_t byte = src[k * (N / 2) + n / 2];
          v = (n & 1) ? (byte >> 4) : (byte & 0xFu);
          if (src_signed)
            v ^= 8u;  // two's complement nibble -> nibble + 8
        }
        out[j >> 1] |= v << (16 * (j & 1) + 4 * el);
      } else {
        out[el] = k < K ? ((const uint32_t *)src)[k * N + n] : 0u;
      }
    }
  uint4 *d = reinterpret_cast<uint4 *>(dst + n * row_bytes + unit * 16);
  *d = make_uint4(out[0], out[1], out[2], out[3]);
}

template <int KIND>
__global__ void unpack_weight_kernel(const uint8_t *packed, int64_t K,
                                     int64_t N, int dst_signed, uint8_t *dst,
                                     int64_t row_bytes) {
  // one thread per destination element (I8 / F32) or destination byte (U4)
  const int64_t c = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const int64_t k = blockIdx.y;
  if (KIND == B200_W_U4) {
    if (c >= N / 2)
      return;
    uint32_t byte = 0;
    for (int h = 0; h < 2; ++h) {
      const int64_t n = 2 * c + h;
      int nib;
      const int64_t off = packed_offset(KIND, K, k, &nib);
      uint32_t v = packed[n * row_bytes + off];
      v = nib ? (v >> 4) : (v & 0xFu);
      if (dst_signed)
        v ^= 8u;
      byte |= v << (4 * h);
    }
    dst[k * (N / 2) + c] = (uint8_t)byte;
  } else {
    if (c >= N)
      return;
    const int64_t off = packed_offset(KIND, K, k, nullptr);
    if (KIND == B200_W_I8)
      dst[k * N + c] = packed[c * row_bytes + off];
    else
      ((uint32_t *)dst)[k * N + c] =
          *(const uint32_t *)(packed + c * row_bytes + off);
  }
}

template <typename T>
__global__ void transpose_scales_kernel(const T *src, int64_t groups,
                                        int64_t N, T *dst) {
  const int64_t n = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const int64_t g = blockIdx.y;
  if (n < N)
    dst[n * groups + g] = src[g * N + n];
}

} // namespace b200

using namespace b200;

extern "C" {

const char *b200_last_error(void) { return error_buffer(); }
const char *b200_version(void) { return "buddy_b200 0.1 (sm_100a)"; }
uint64_t b200_launch_count(void) { return g_launches.load(); }

int64_t b200_packed_k(int kind, int64_t K) { return packed_k(kind, K); }
int64_t b200_packed_row_bytes(int kind, int64_t K) {
  return packed_row_bytes(kind, K);
}
int64_t b200_packed_offset(int kind, int64_t K, int64_t k, int *nibble) {
  return packed_offset(kind, K, k, nibble);
}

static int check_kind(int kind) {
  if (kind != B200_W_F32 && kind != B200_W_I8 && kind != B200_W_U4)
    return fail(B200_EINVAL, "unknown weight kind %d", kind);
  return B200_OK;
}

int b200_pack_weight(int kind, const void *src_kn, int64_t K, int64_t N,
                     int src_signed, void *dst, void *stream) {
  if (int rc = check_kind(kind))
    return rc;
  if (!src_kn || !dst || K < 1 || N < 1)
    return fail(B200_EINVAL, "pack_weight: bad argument");
  if (kind == B200_W_U4 && (N & 1))
    return fail(B200_EINVAL, "pack_weight: int4 needs an even N");
  if (int rc = ensure_device())
    return rc;
  const int64_t rb = packed_row_bytes(kind, K);
  if (rb / 16 > 65535)
    return fail(B200_ELIMIT, "pack_weight: K=%lld too large", (long long)K);
  dim3 grid((unsigned)((N + 127) / 128), (unsigned)(rb / 16));
  cudaStream_t st = (cudaStream_t)stream;
  if (kind == B200_W_I8)
    pack_weight_kernel<B200_W_I8><<<grid, 128, 0, st>>>(
        (const uint8_t *)src_kn, K, N, src_signed, (uint8_t *)dst, rb);
  else if (kind == B200_W_U4)
    pack_weight_kernel<B200_W_U4><<<grid, 128, 0, st>>>(
        (const uint8_t *)src_kn, K, N, src_signed, (uint8_t *)dst, rb);
  else
    pack_weight_kernel<B200_W_F32><<<grid, 128, 0, st>>>(
        (const uint8_t *)src_kn, K, N, src_signed, (uint8_t *)dst, rb);
  B200_LAUNCH_CHECK();
  return B200_OK;
}

int b200_unpack_weight(int kind, const void *packed, int64_t K, int64_t N,
                       int dst_signed, void *dst_kn, void *stream) {
  if (int rc = check_kind(kind))
    return rc;
  if (!packed || !dst_kn || K < 1 || N < 1 || K > 65535)
    return fail(B200_EINVAL, "unpack_weight: bad argument");
  if (int rc = ensure_device())
    return rc;
  const int64_t rb = packed_row_bytes(kind, K);
  const int64_t cols = kind == B200_W_U4 ? N / 2 : N;
  dim3 grid((unsigned)((cols + 127) / 128), (unsigned)K);
  cudaStream_t st = (cudaStream_t)stream;
  if (kind == B200_W_I8)
    unpack_weight_kernel<B200_W_I8><<<grid, 128, 0, st>>>(
        (const uint8_t *)packed, K, N, dst_signed, (uint8_t *)dst_kn, rb);
  else if (kind == B200_W_U4)
    unpack_weight_kernel<B200_W_U4><<<grid, 128, 0, st>>>(
        (const uint8_t *)packed, K, N, dst_signed, (uint8_t *)dst_kn, rb);
  else
    unpack_weight_kernel<B200_W_F32><<<grid, 128, 0, st>>>(
        (const uint8_t *)packed, K, N, dst_signed, (uint8_t *)dst_kn, rb);
  B200_LAUNCH_CHECK();
  return B200_OK;
}

int b200_pack_scales(const void *src, int dtype, int64_t groups, int64_t N,
                     void *dst, void *stream) {
  if (!src || !dst || groups < 1 || groups > 65535 || N < 1)
    return fail(B200_EINVAL, "pack_scales: bad argument");
  if (int rc = ensure_device())
    return rc;
  dim3 grid((unsigned)((N + 127) / 128), (unsigned)groups);
  cudaStream_t st = (cudaStream_t)stream;
  if (dtype == B200_F32)
    transpose_scales_kernel<float>
        <<<grid, 128, 0, st>>>((const float *)src, groups, N, (float *)dst);
  else
    transpose_scales_kernel<uint16_t><<<grid, 128, 0, st>>>(
        (const uint16_t *)src, groups, N, (uint16_t *)dst);
  B200_LAUNCH_CHECK();
  return B200_OK;
}

int b200_quantize_per_channel(const float *W, int64_t K, int64_t N, int bits,
                              int8_t *Q, float *scale, void *stream) {
  if (!W || !Q || !scale || K < 1 || N < 1 || (bits != 8 && bits != 4))
    return fail(B200_EINVAL, "quantize_per_channel: bad argument");
  if (K > 65535)
    return fail(B200_ELIMIT, "quantize_per_channel: K=%lld > 65535",
                (long long)K);
  if (int rc = ensure_device())
    return rc;
  cudaStream_t st = (cudaStream_t)stream;
  B200_CUDA(cudaMemsetAsync(scale, 0, N * sizeof(float), st));
  const int64_t slices = 32;
  const int64_t rows = (K + slices - 1) / slices;
  dim3 g1((unsigned)((N + 255) / 256), (unsigned)slices);
  absmax_cols_kernel<<<g1, 256, 0, st>>>(W, K, N, rows, (uint32_t *)scale);
  B200_LAUNCH_CHECK();
  scale_from_amax_kernel<<<(unsigned)((N + 255) / 256), 256, 0, st>>>(
      scale, N, bits == 4 ? 7.f : 127.f);
  B200_LAUNCH_CHECK();
  dim3 g3((unsigned)((N + 255) / 256), (unsigned)K);
  quantize_cols_kernel<<<g3, 256, 0, st>>>(W, scale, K, N,
                                           bits == 4 ? -8.f : -128.f,
                                           bits == 4 ? 7.f : 127.f, Q);
  B200_LAUNCH_CHECK();
  return B200_OK;
}

int b200_quantize_w4_group(const float *W, int64_t K, int64_t N, int64_t G,
                           uint8_t *P, uint16_t *scale_f16, void *stream) {
  if (!W || !P || !scale_f16 || K < 1 || N < 2 || (N & 1) || G < 1 || K % G)
    return fail(B200_EINVAL, "quantize_w4_group: bad argument");
  if (K / G > 65535)
    return fail(B200_ELIMIT, "quantize_w4_group: too many groups");
  if (int rc = ensure_device())
    return rc;
  dim3 grid((unsigned)((N / 2 + 127) / 128), (unsigned)(K / G));
  quantize_w4_group_kernel<<<grid, 128, 0, (cudaStream_t)stream>>>(
      W, K, N, G, P, (__half *)scale_f16);
  B200_LAUNCH_CHECK();
  return B200_OK;
}

int b200_pack_int4(const int8_t *flat, int64_t n, int8_t *packed,
                   void *stream) {
  if (!flat || !packed || n < 0 || (n & 1))
    return fail(B200_EINVAL, "pack_int4: odd or negative element count");
  if (n == 0)
    return B200_OK;
  if (int rc = ensure_device())
    return rc;
  const int64_t nb = n / 2;
  pack_int4_kernel<<<(unsigned)((nb + 255) / 256), 256, 0,
                     (cudaStream_t)stream>>>(flat, nb, packed);
  B200_LAUNCH_CHECK();
  return B200_OK;
}

int b200_unpack_int4(const int8_t *packed, int64_t nbytes, int8_t *flat,
                     void *stream) {
  if (!flat || !packed || nbytes < 0)
    return fail(B200_EINVAL, "unpack_int4: bad argument");
  if (nbytes == 0)
    return B200_OK;
  if (int rc = ensure_device())
    return rc;
  unpack_int4_kernel<<<(unsigned)((nbytes + 255) / 256), 256, 0,
                       (cudaStream_t)stream>>>(packed, nbytes, flat);
  B200_LAUNCH_CHECK();
  return B200_OK;
}

} // extern "C"
