// A cache of one normalised vector per position (a compressed latent from which keys and values
// of all heads are expanded): c = w * v / sqrt(mean(v^2) + eps), statistics in float, written
// straight into the row's page slot.  The pages have the layout of the key pools,
// [pages, 1, page size, width], so the paged attention kernels read them as one shared head.
#include "common.cuh"

namespace kvcm {

template <typename T>
__global__ void __launch_bounds__(128)
latent_norm_cache_kernel(const T* __restrict__ v, int ldv, const float* __restrict__ weight,
                         const int* __restrict__ slot_mapping, T* __restrict__ cache, int width, float eps) {
  __shared__ float scratch[33];
  const int row = blockIdx.x;
  const int slot = slot_mapping[row];
  if (slot < 0) return;                                   // a padding row holds no page
  const T* src = v + size_t(row) * ldv;
  float ss = 0.f;
  for (int i = threadIdx.x; i < width; i += blockDim.x) {
    const float a = ldf(src + i);
    ss += a * a;
  }
  ss = block_sum(ss, scratch);
  const float inv = 1.f / sqrtf(ss / float(width) + eps);
  T* dst = cache + size_t(slot) * width;
  for (int i = threadIdx.x; i < width; i += blockDim.x) stf(dst + i, weight[i] * (ldf(src + i) * inv));
}

}  // namespace kvcm

using namespace kvcm;

KVCM_API int kvcm_latent_norm_cache_f32(const void* v, int ldv, const float* weight, const int* slot_mapping,
                                        void* cache, int rows, int width, float eps, void* stream) {
  if (rows == 0) return 0;
  latent_norm_cache_kernel<float><<<rows, 128, 0, (cudaStream_t)stream>>>((const float*)v, ldv, weight, slot_mapping,
                                                                         (float*)cache, width, eps);
  return KVCM_LAUNCH_RESULT();
}
KVCM_API int kvcm_latent_norm_cache_bf16(const void* v, int ldv, const float* weight, const int* slot_mapping,
                                         void* cache, int rows, int width, float eps, void* stream) {
  if (rows == 0) return 0;
  latent_norm_cache_kernel<bf16><<<rows, 128, 0, (cudaStream_t)stream>>>((const bf16*)v, ldv, weight, slot_mapping,
                                                                        (bf16*)cache, width, eps);
  return KVCM_LAUNCH_RESULT();
}
