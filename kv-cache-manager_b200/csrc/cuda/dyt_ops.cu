// Row-wise kernels of a block whose sublayers all read ONE normalised copy of the residual stream
// and whose outputs are added to the stream together:
//
//   dyt_norm:  x += s0 * p0 + s1 * p1 + s2 * p2   (the sublayers' float outputs of the layer before,
//              any of them absent), then  out = tanh(alpha * x) * w + b  in the storage type.
//              The norm takes no statistics of the row; alpha is one number read from device memory.
//              With `rows` the output rows are gathered from the listed input rows and x is left as it is.
//   relu_sq:   out = max(x, 0)^2, the activation of an ungated feed-forward.
//
// The stream, the sum and the tanh are float in both storage types.
#include "common.cuh"
#include "pdl.cuh"

namespace kvcm {

template <typename T>
__global__ void __launch_bounds__(256)
dyt_norm_kernel(float* __restrict__ x, const float* __restrict__ p0, float s0, const float* __restrict__ p1, float s1,
                const float* __restrict__ p2, float s2, const float* __restrict__ w, const float* __restrict__ b,
                const float* __restrict__ alpha, T* __restrict__ out, const int* __restrict__ rows, int hidden) {
  pdl_launch_dependents();
  pdl_wait();
  const int r = blockIdx.x;
  const int src = rows ? rows[r] : r;
  const float a = alpha[0];
  float* xr = x + size_t(src) * hidden;
  const size_t at = size_t(src) * hidden;
  for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
    float add = 0.f;
    if (p0) add = s0 * p0[at + i];
    if (p1) add = fmaf(s1, p1[at + i], add);
    if (p2) add = fmaf(s2, p2[at + i], add);
    float v = xr[i];
    if (p0 || p1 || p2) {
      v += add;
      if (!rows) xr[i] = v;
    }
    stf(out + size_t(r) * hidden + i, fmaf(tanhf(a * v), w[i], b[i]));
  }
}

// Four elements a thread (hidden % 4 == 0; every row then starts on a 16-byte boundary).
template <typename T>
__global__ void __launch_bounds__(256)
dyt_norm_vec_kernel(float* __restrict__ x, const float* __restrict__ p0, float s0, const float* __restrict__ p1, float s1,
                    const float* __restrict__ p2, float s2, const float* __restrict__ w, const float* __restrict__ b,
                    const float* __restrict__ alpha, T* __restrict__ out, const int* __restrict__ rows, int hidden) {
  pdl_launch_dependents();
  pdl_wait();
  const int r = blockIdx.x;
  const int src = rows ? rows[r] : r;
  const float a = alpha[0];
  const size_t at = size_t(src) * hidden;
  for (int i = 4 * threadIdx.x; i < hidden; i += 4 * blockDim.x) {
    float4 v = *reinterpret_cast<const float4*>(x + at + i);
    if (p0 || p1 || p2) {
      float4 add = make_float4(0.f, 0.f, 0.f, 0.f);
      if (p0) { const float4 t = *reinterpret_cast<const float4*>(p0 + at + i); add.x = s0 * t.x; add.y = s0 * t.y; add.z = s0 * t.z; add.w = s0 * t.w; }
      if (p1) { const float4 t = *reinterpret_cast<const float4*>(p1 + at + i); add.x = fmaf(s1, t.x, add.x); add.y = fmaf(s1, t.y, add.y); add.z = fmaf(s1, t.z, add.z); add.w = fmaf(s1, t.w, add.w); }
      if (p2) { const float4 t = *reinterpret_cast<const float4*>(p2 + at + i); add.x = fmaf(s2, t.x, add.x); add.y = fmaf(s2, t.y, add.y); add.z = fmaf(s2, t.z, add.z); add.w = fmaf(s2, t.w, add.w); }
      v.x += add.x; v.y += add.y; v.z += add.z; v.w += add.w;
      if (!rows) *reinterpret_cast<float4*>(x + at + i) = v;
    }
    const float4 ww = *reinterpret_cast<const float4*>(w + i), bb = *reinterpret_cast<const float4*>(b + i);
    T* o = out + size_t(r) * hidden + i;
    stf(o, fmaf(tanhf(a * v.x), ww.x, bb.x));
    stf(o + 1, fmaf(tanhf(a * v.y), ww.y, bb.y));
    stf(o + 2, fmaf(tanhf(a * v.z), ww.z, bb.z));
    stf(o + 3, fmaf(tanhf(a * v.w), ww.w, bb.w));
  }
}

template <typename T>
__global__ void __launch_bounds__(256)
relu_sq_kernel(const T* in, T* out, long long n) {
  pdl_launch_dependents();
  pdl_wait();
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    const float v = fmaxf(ldf(in + i), 0.f);
    stf(out + i, v * v);
  }
}

// bfloat16, eight elements a thread (16-byte accesses): n % 8 == 0 and aligned pointers.
__global__ void __launch_bounds__(256)
relu_sq_vec_kernel(const uint4* in, uint4* out, long long n8) {
  pdl_launch_dependents();
  pdl_wait();
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n8; i += (long long)gridDim.x * blockDim.x) {
    uint4 v = in[i];
    __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&v);
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      float2 f = __bfloat1622float2(h[k]);
      f.x = fmaxf(f.x, 0.f); f.y = fmaxf(f.y, 0.f);
      h[k] = __floats2bfloat162_rn(f.x * f.x, f.y * f.y);
    }
    out[i] = v;
  }
}

template <typename T>
int launch_dyt_norm(float* x, const float* p0, float s0, const float* p1, float s1, const float* p2, float s2,
                    const float* w, const float* b, const float* alpha, T* out, const int* rows, int n_rows, int hidden,
                    cudaStream_t s) {
  if (n_rows == 0) return 0;
  if (hidden % 4 == 0)
    return pdl_launch(dyt_norm_vec_kernel<T>, dim3(n_rows), dim3(256), 0, s, x, p0, s0, p1, s1, p2, s2, w, b, alpha, out, rows, hidden);
  return pdl_launch(dyt_norm_kernel<T>, dim3(n_rows), dim3(256), 0, s, x, p0, s0, p1, s1, p2, s2, w, b, alpha, out, rows, hidden);
}

}  // namespace kvcm

using namespace kvcm;

KVCM_API int kvcm_dyt_norm_f32(float* x, const float* p0, float s0, const float* p1, float s1, const float* p2, float s2,
                               const float* w, const float* b, const float* alpha, void* out, const int* rows, int n_rows,
                               int hidden, void* stream) {
  return launch_dyt_norm<float>(x, p0, s0, p1, s1, p2, s2, w, b, alpha, (float*)out, rows, n_rows, hidden, (cudaStream_t)stream);
}
KVCM_API int kvcm_dyt_norm_bf16(float* x, const float* p0, float s0, const float* p1, float s1, const float* p2, float s2,
                                const float* w, const float* b, const float* alpha, void* out, const int* rows, int n_rows,
                                int hidden, void* stream) {
  return launch_dyt_norm<bf16>(x, p0, s0, p1, s1, p2, s2, w, b, alpha, (bf16*)out, rows, n_rows, hidden, (cudaStream_t)stream);
}

KVCM_API int kvcm_relu_sq_f32(const void* in, void* out, long long n, void* stream) {
  if (n == 0) return 0;
  const int blocks = int(min((n + 255) / 256, (long long)148 * 16));
  return pdl_launch(relu_sq_kernel<float>, dim3(blocks), dim3(256), 0, (cudaStream_t)stream, (const float*)in, (float*)out, n);
}
KVCM_API int kvcm_relu_sq_bf16(const void* in, void* out, long long n, void* stream) {
  if (n == 0) return 0;
  if (n % 8 == 0 && ((reinterpret_cast<uintptr_t>(in) | reinterpret_cast<uintptr_t>(out)) & 15) == 0) {
    const int vblocks = int(min((n / 8 + 255) / 256, (long long)148 * 16));
    return pdl_launch(relu_sq_vec_kernel, dim3(vblocks), dim3(256), 0, (cudaStream_t)stream, (const uint4*)in, (uint4*)out, n / 8);
  }
  const int blocks = int(min((n + 255) / 256, (long long)148 * 16));
  return pdl_launch(relu_sq_kernel<bf16>, dim3(blocks), dim3(256), 0, (cudaStream_t)stream, (const bf16*)in, (bf16*)out, n);
}
