// Row-wise kernels around the float32 residual stream for blocks whose norm sits on the
// sublayer's OUTPUT (x += mult * w * y / rms(y)) and for embeddings that are a sum of tables.
// Each is instantiated for float (the true 32-bit path) and bfloat16 storage; sums, statistics
// and the stream itself are always float.
#include "common.cuh"

namespace kvcm {

// ------------------------------------------------------------------ embedding as a sum of tables
// x[t] = table[id] + pair[row(prev, id)] + place[pos], every term optional but the first.
//   row(prev, id) = (prev * mul_prev + id * mul_cur) mod buckets, and row `buckets` (the table's
//   last) when the request has no earlier token (prev < 0).
// An id or position outside its table yields a row of NaN: loud, not wrong.  A padding row
// (position < 0) gets the token's row only.  `h` (optional) receives the sum in the storage type.
template <typename T>
__global__ void __launch_bounds__(256)
embed_sum_kernel(const int* __restrict__ ids, const int* __restrict__ prev, const int* __restrict__ positions,
                 const T* __restrict__ table, const T* __restrict__ pair, const T* __restrict__ place,
                 float* __restrict__ x, T* __restrict__ h, int hidden, int vocab, int buckets,
                 long long mul_prev, long long mul_cur, int max_pos) {
  const int t = blockIdx.x;
  const int id = ids[t];
  const int pos = positions[t];
  const bool bad = id < 0 || id >= vocab || (place && pos >= max_pos);
  long long row = buckets;
  if (pair && prev[t] >= 0) {
    row = ((long long)prev[t] * mul_prev + (long long)id * mul_cur) % buckets;
    if (row < 0) row += buckets;                          // the mathematical residue, also for negative multipliers
  }
  for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
    float v;
    if (bad) {
      v = __int_as_float(0x7fc00000);
    } else {
      v = ldf(table + size_t(id) * hidden + i);
      if (pair && pos >= 0) v += ldf(pair + size_t(row) * hidden + i);
      if (place && pos >= 0) v += ldf(place + size_t(pos) * hidden + i);
    }
    x[size_t(t) * hidden + i] = v;
    if (h) stf(h + size_t(t) * hidden + i, v);
  }
}

// ------------------------------------------------------- norm on a sublayer's output + residual
// x[r] += mult * w * (y[r] * inv),  inv = 1 / sqrt(mean(y[r]^2) + eps);  h[r] = storage(x[r]).
// y may be float or the storage type; the weight float or the storage type.
template <typename T, typename Y, typename W>
__global__ void __launch_bounds__(256)
rms_scale_add_kernel(float* __restrict__ x, const Y* __restrict__ y, const W* __restrict__ weight,
                     T* __restrict__ h, int hidden, float eps, float mult) {
  __shared__ float scratch[33];
  extern __shared__ float row_cache[];            // hidden floats: the row of y
  const int r = blockIdx.x;
  const Y* yr = y + size_t(r) * hidden;
  float ss = 0.f;
  for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
    const float v = ldf(yr + i);
    row_cache[i] = v;
    ss += v * v;
  }
  ss = block_sum(ss, scratch);
  const float inv = 1.f / sqrtf(ss / float(hidden) + eps);
  float* xr = x + size_t(r) * hidden;
  for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
    const float v = xr[i] + mult * (ldf(weight + i) * (row_cache[i] * inv));
    xr[i] = v;
    if (h) stf(h + size_t(r) * hidden + i, v);
  }
}

// The same with four elements an access (hidden % 4 == 0, rows 16-byte aligned in every type).
__device__ __forceinline__ float4 ro_load4(const float* p) { return *reinterpret_cast<const float4*>(p); }
__device__ __forceinline__ float4 ro_load4(const bf16* p) {
  const uint2 raw = *reinterpret_cast<const uint2*>(p);
  const __nv_bfloat162 lo = *reinterpret_cast<const __nv_bfloat162*>(&raw.x), hi = *reinterpret_cast<const __nv_bfloat162*>(&raw.y);
  return make_float4(__bfloat162float(lo.x), __bfloat162float(lo.y), __bfloat162float(hi.x), __bfloat162float(hi.y));
}
__device__ __forceinline__ void ro_store4(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
__device__ __forceinline__ void ro_store4(bf16* p, float4 v) {
  const __nv_bfloat162 lo = __floats2bfloat162_rn(v.x, v.y), hi = __floats2bfloat162_rn(v.z, v.w);
  uint2 raw;
  raw.x = *reinterpret_cast<const uint32_t*>(&lo);
  raw.y = *reinterpret_cast<const uint32_t*>(&hi);
  *reinterpret_cast<uint2*>(p) = raw;
}

template <typename T, typename Y, typename W>
__global__ void __launch_bounds__(256)
rms_scale_add_vec_kernel(float* __restrict__ x, const Y* __restrict__ y, const W* __restrict__ weight,
                         T* __restrict__ h, int hidden, float eps, float mult) {
  __shared__ float scratch[33];
  extern __shared__ float row_cache[];
  const int r = blockIdx.x;
  const Y* yr = y + size_t(r) * hidden;
  float ss = 0.f;
  for (int i = threadIdx.x * 4; i < hidden; i += blockDim.x * 4) {
    const float4 v = ro_load4(yr + i);
    *reinterpret_cast<float4*>(row_cache + i) = v;
    ss += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
  }
  ss = block_sum(ss, scratch);
  const float inv = 1.f / sqrtf(ss / float(hidden) + eps);
  float* xr = x + size_t(r) * hidden;
  for (int i = threadIdx.x * 4; i < hidden; i += blockDim.x * 4) {
    const float4 a = ro_load4(xr + i), w = ro_load4(weight + i), v = *reinterpret_cast<const float4*>(row_cache + i);
    const float4 o = make_float4(a.x + mult * (w.x * (v.x * inv)), a.y + mult * (w.y * (v.y * inv)),
                                 a.z + mult * (w.z * (v.z * inv)), a.w + mult * (w.w * (v.w * inv)));
    ro_store4(xr + i, o);
    if (h) ro_store4(h + size_t(r) * hidden + i, o);
  }
}

// out[i] = storage(x[i])
template <typename T>
__global__ void cast_rows_kernel(const float* __restrict__ x, T* __restrict__ out, long long n) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) stf(out + i, x[i]);
}

template <typename T>
int launch_embed_sum(const int* ids, const int* prev, const int* positions, const void* table, const void* pair,
                     const void* place, float* x, void* h, int rows, int hidden, int vocab, int buckets,
                     long long mul_prev, long long mul_cur, int max_pos, cudaStream_t s) {
  if (rows == 0) return 0;
  if (pair && (buckets <= 0 || !prev)) return KVCM_ERR_UNSUPPORTED;
  embed_sum_kernel<T><<<rows, 256, 0, s>>>(ids, prev, positions, (const T*)table, (const T*)pair, (const T*)place, x,
                                           (T*)h, hidden, vocab, buckets, mul_prev, mul_cur, max_pos);
  return KVCM_LAUNCH_RESULT();
}

template <typename T>
int launch_rms_scale_add(float* x, const void* y, int y_f32, const void* w, int w_f32, void* h, int rows, int hidden,
                         float eps, float mult, cudaStream_t s) {
  if (rows == 0) return 0;
  const size_t smem = size_t(hidden) * sizeof(float);
  if (smem > 160 * 1024) return KVCM_ERR_UNSUPPORTED;
  const bool vec = (hidden % 4) == 0 && ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(y) |
                                          reinterpret_cast<uintptr_t>(w) | reinterpret_cast<uintptr_t>(h)) & 15) == 0;
#define KVCM_RSA(Y, W)                                                                                           \
  do {                                                                                                           \
    auto kernel = vec ? rms_scale_add_vec_kernel<T, Y, W> : rms_scale_add_kernel<T, Y, W>;                       \
    if (smem > 48 * 1024) cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);  \
    kernel<<<rows, 256, smem, s>>>(x, (const Y*)y, (const W*)w, (T*)h, hidden, eps, mult);                       \
  } while (0)
  if (y_f32 && w_f32) KVCM_RSA(float, float);
  else if (y_f32) KVCM_RSA(float, T);
  else if (w_f32) KVCM_RSA(T, float);
  else KVCM_RSA(T, T);
#undef KVCM_RSA
  return KVCM_LAUNCH_RESULT();
}

}  // namespace kvcm

using namespace kvcm;

#define KVCM_RESIDUAL_OPS(SUFFIX, T)                                                                              \
  KVCM_API int kvcm_embed_sum_##SUFFIX(const int* ids, const int* prev, const int* positions, const void* table,  \
                                       const void* pair, const void* place, float* x, void* h, int rows,          \
                                       int hidden, int vocab, int buckets, long long mul_prev, long long mul_cur, \
                                       int max_pos, void* stream) {                                               \
    return launch_embed_sum<T>(ids, prev, positions, table, pair, place, x, h, rows, hidden, vocab, buckets,      \
                               mul_prev, mul_cur, max_pos, (cudaStream_t)stream);                                 \
  }                                                                                                               \
  KVCM_API int kvcm_rms_scale_add_##SUFFIX(float* x, const void* y, int y_f32, const void* w, int w_f32, void* h, \
                                           int rows, int hidden, float eps, float mult, void* stream) {           \
    return launch_rms_scale_add<T>(x, y, y_f32, w, w_f32, h, rows, hidden, eps, mult, (cudaStream_t)stream);      \
  }                                                                                                               \
  KVCM_API int kvcm_cast_rows_##SUFFIX(const float* x, void* out, long long n, void* stream) {                    \
    if (n == 0) return 0;                                                                                         \
    cast_rows_kernel<T><<<(unsigned)((n + 255) / 256), 256, 0, (cudaStream_t)stream>>>(x, (T*)out, n);            \
    return KVCM_LAUNCH_RESULT();                                                                                  \
  }

KVCM_RESIDUAL_OPS(f32, float)
KVCM_RESIDUAL_OPS(bf16, bf16)
