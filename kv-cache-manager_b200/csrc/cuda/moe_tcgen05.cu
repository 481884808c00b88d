// The experts' products of a routed feed-forward on the fifth-generation tensor cores.
//
// The (row, choice) pairs of a step are sorted by expert (csrc/cuda/moe.cu) and the rows of h
// gathered in that order into xs [pairs, K]; a *work tile* is up to 128 consecutive sorted pairs
// of ONE expert.  Both products of an expert are then ordinary tiles of a grouped product:
//     gate/up:  act[place, n] = silu(xs[place] . Wg_e[n]) * (xs[place] . Wu_e[n])     (bfloat16)
//     down:     y[place, n]   = act[place] . Wd_e[n]                                  (float)
// with the expert's matrices addressed inside the stacked tensor ([E * rows_per_expert, K]) by a
// row offset of the tensor-map coordinate.  The kernel is the persistent, warp-specialised one of
// gemm_tcgen05.cu (TMA ring of 128-byte-swizzled [128 x 64] and [256 x 64] pieces, one thread
// issuing tcgen05.mma into two accumulators of tensor memory, four epilogue warps reading them
// back with tcgen05.ld) with two changes: the list of work tiles, and how many there are, is
// read from device memory (nothing about the routing is known on the host, so the step can be
// recorded into a CUDA graph), and the epilogue stores only the tile's own rows: a tile that holds
// fewer than 128 pairs computes on the rows that follow it in xs (other experts' pairs, or zeros
// behind the end) and drops those results.
// Every wait on an mbarrier is bounded; when one runs out the block records it
// (kvcm_moe_tcgen05_error), stops waiting, frees its tensor memory and leaves.
#include "tcgen05_common.cuh"

namespace kvcm {

constexpr int kMeBM = 128, kMeBK = 64, kMeBN = 256;
constexpr int kMeThreads = 192;
constexpr int kMeABytes = kMeBM * kMeBK * 2;
constexpr int kMeBBytes = kMeBN * kMeBK * 2;
constexpr int kMeStageBytes = kMeABytes + kMeBBytes;
constexpr int kMeStages = 4;

__device__ int g_moe_tcgen05_error = 0;

// GATED: an expert has 2N rows in W (N gate rows, then N up rows); a tile's 256 accumulator columns
// are 128 gate columns n0.. and the 128 up columns n0.. of the same expert; OutT = bf16.
// Otherwise an expert has N rows and the tile is 256 output columns wide; OutT = float.
template <typename OutT, bool GATED>
__global__ void __launch_bounds__(kMeThreads)
moe_tcgen05_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_w,
                   OutT* __restrict__ Y, int N, int K, int ldy, const int* __restrict__ tile_expert,
                   const int* __restrict__ tile_begin, const int* __restrict__ tile_rows,
                   const int* __restrict__ num_tiles) {
  constexpr int BNOUT = GATED ? kMeBN / 2 : kMeBN;
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  unsigned char* ring = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  __shared__ __align__(8) uint64_t full[kMeStages], empty[kMeStages], acc_full[2], acc_empty[2];
  __shared__ uint32_t tmem_base;
  __shared__ volatile int abort_flag;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n_tiles = (N + BNOUT - 1) / BNOUT;
  const int rows_per_expert = GATED ? 2 * N : N;
  const int tiles = num_tiles[0] * n_tiles;
  const int nk = (K + kMeBK - 1) / kMeBK;
  const int my_tiles = int(blockIdx.x) < tiles ? (tiles - 1 - int(blockIdx.x)) / int(gridDim.x) + 1 : 0;

  if (threadIdx.x == 0) {
    abort_flag = 0;
    for (int s = 0; s < kMeStages; ++s) {
      tc5::mbar_init(&full[s], 1);
      tc5::mbar_init(&empty[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      tc5::mbar_init(&acc_full[a], 1);
      tc5::mbar_init(&acc_empty[a], 4);                        // four epilogue warps
    }
    tc5::mbar_init_fence();
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(tc5::s32(&tmem_base)), "r"(2 * kMeBN));
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::);
  }
  tc5::fence_before();
  __syncthreads();
  tc5::fence_after();
  const uint32_t tmem = tmem_base;

  if (warp == 0) {
    if (lane == 0) {
      int it = 0;
      for (int tl = 0; tl < my_tiles && !abort_flag; ++tl) {
        const int t = int(blockIdx.x) + tl * int(gridDim.x);
        const int wt = t / n_tiles, n0 = (t % n_tiles) * BNOUT;
        const int m0 = tile_begin[wt];
        const int w0 = tile_expert[wt] * rows_per_expert + n0;
        for (int k = 0; k < nk; ++k, ++it) {
          const int s = it % kMeStages;
          if (!tc5::mbar_wait(&empty[s], ((it / kMeStages) & 1) ^ 1)) {
            atomicExch(&g_moe_tcgen05_error, (1 << 16) | int(blockIdx.x & 0xffff));
            abort_flag = 1;
            break;
          }
          tc5::mbar_expect_tx(&full[s], kMeStageBytes);
          unsigned char* a = ring + s * kMeStageBytes;
          unsigned char* b = a + kMeABytes;
          tc5::tma_load_2d(a, &map_x, &full[s], k * kMeBK, m0);
          if constexpr (GATED) {                                  // the map's box is 128 rows
            tc5::tma_load_2d(b, &map_w, &full[s], k * kMeBK, w0);
            tc5::tma_load_2d(b + kMeBBytes / 2, &map_w, &full[s], k * kMeBK, w0 + N);
          } else {
            tc5::tma_load_2d(b, &map_w, &full[s], k * kMeBK, w0);
          }
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc = tc5::idesc(kMeBM, kMeBN);
      int it = 0;
      for (int tl = 0; tl < my_tiles && !abort_flag; ++tl) {
        const int acc = tl & 1;
        if (!tc5::mbar_wait(&acc_empty[acc], ((tl >> 1) & 1) ^ 1)) {
          atomicExch(&g_moe_tcgen05_error, (4 << 16) | int(blockIdx.x & 0xffff));
          abort_flag = 1;
          break;
        }
        tc5::fence_after();
        const uint32_t d_tmem = tmem + uint32_t(acc * kMeBN);
        for (int k = 0; k < nk; ++k, ++it) {
          const int s = it % kMeStages;
          if (!tc5::mbar_wait(&full[s], (it / kMeStages) & 1)) {
            atomicExch(&g_moe_tcgen05_error, (2 << 16) | int(blockIdx.x & 0xffff));
            abort_flag = 1;
            break;
          }
          tc5::fence_after();
          const uint32_t a_addr = tc5::s32(ring + s * kMeStageBytes);
          const uint64_t da = tc5::smem_desc(a_addr), db = tc5::smem_desc(a_addr + kMeABytes);
#pragma unroll
          for (int j = 0; j < kMeBK / 16; ++j)
            tc5::mma(d_tmem, da + uint64_t(2 * j), db + uint64_t(2 * j), idesc, (k > 0 || j > 0) ? 1u : 0u);
          tc5::commit(&empty[s]);
        }
        if (abort_flag) break;
        tc5::commit(&acc_full[acc]);
      }
    }
  } else {
    const int quarter = warp & 3;
    for (int tl = 0; tl < my_tiles; ++tl) {
      const int acc = tl & 1;
      const int t = int(blockIdx.x) + tl * int(gridDim.x);
      const int wt = t / n_tiles, n0 = (t % n_tiles) * BNOUT;
      if (abort_flag || !tc5::mbar_wait(&acc_full[acc], (tl >> 1) & 1)) {
        if (!abort_flag && lane == 0) atomicExch(&g_moe_tcgen05_error, (3 << 16) | int(blockIdx.x & 0xffff));
        abort_flag = 1;
        break;
      }
      tc5::fence_after();
      const int local = quarter * 32 + lane;
      const bool row_ok = local < tile_rows[wt];
      const size_t row = size_t(tile_begin[wt]) + local;
#pragma unroll 1
      for (int c = 0; c < BNOUT / 32; ++c) {
        const uint32_t taddr = tmem + (uint32_t(quarter * 32) << 16) + uint32_t(acc * kMeBN + c * 32);
        const int col0 = n0 + c * 32;
        if constexpr (GATED) {
          uint32_t g[32], u[32];
          tc5::ld32(taddr, g);
          tc5::ld32(taddr + BNOUT, u);
          tc5::ld_wait();
          if (row_ok) {
            bf16* dst = reinterpret_cast<bf16*>(Y) + row * ldy + col0;
            __nv_bfloat162 h2[16];
#pragma unroll
            for (int i = 0; i < 32; ++i) {
              const float xa = __uint_as_float(g[i]);
              const bf16 y = __float2bfloat16_rn(xa / (1.f + expf(-xa)) * __uint_as_float(u[i]));
              if (i & 1) h2[i / 2].y = y; else h2[i / 2].x = y;
            }
            if (col0 + 32 <= N && (reinterpret_cast<uintptr_t>(dst) & 15) == 0) {
#pragma unroll
              for (int i = 0; i < 4; ++i) reinterpret_cast<uint4*>(dst)[i] = reinterpret_cast<const uint4*>(h2)[i];
            } else {
#pragma unroll
              for (int i = 0; i < 32; ++i)
                if (col0 + i < N) dst[i] = (i & 1) ? h2[i / 2].y : h2[i / 2].x;
            }
          }
        } else {
          uint32_t v[32];
          tc5::ld32(taddr, v);
          tc5::ld_wait();
          if (row_ok) {
            float* dst = reinterpret_cast<float*>(Y) + row * ldy + col0;
            if (col0 + 32 <= N && (reinterpret_cast<uintptr_t>(dst) & 15) == 0) {
#pragma unroll
              for (int i = 0; i < 8; ++i)
                reinterpret_cast<uint4*>(dst)[i] = make_uint4(v[4 * i], v[4 * i + 1], v[4 * i + 2], v[4 * i + 3]);
            } else {
#pragma unroll
              for (int i = 0; i < 32; ++i)
                if (col0 + i < N) dst[i] = __uint_as_float(v[i]);
            }
          }
        }
      }
      tc5::fence_before();
      __syncwarp();
      if (lane == 0) tc5::mbar_arrive(&acc_empty[acc]);
    }
  }
  tc5::fence_before();
  __syncthreads();
  if (warp == 1) {
    tc5::fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem), "r"(2 * kMeBN));
  }
}

// xs[place] = h[pair_of[place] / top]: the rows of h in the order of the sorted pairs.
__global__ void __launch_bounds__(256)
moe_gather_kernel(const bf16* __restrict__ h, int ldh, const int* __restrict__ pair_of, int top, bf16* __restrict__ xs,
                  int D) {
  const int place = blockIdx.x;
  const bf16* src = h + size_t(pair_of[place] / top) * ldh;
  bf16* dst = xs + size_t(place) * D;
  if ((D % 8) == 0 && (ldh % 8) == 0 && (reinterpret_cast<uintptr_t>(h) & 15) == 0) {
    for (int i = threadIdx.x; i < D / 8; i += blockDim.x)
      reinterpret_cast<uint4*>(dst)[i] = reinterpret_cast<const uint4*>(src)[i];
  } else {
    for (int i = threadIdx.x; i < D; i += blockDim.x) dst[i] = src[i];
  }
}

template <typename OutT, bool GATED>
int launch_moe_tcgen05(const void* X, long long x_rows, const void* W, long long w_rows, void* Y, int N, int K, int ldy,
                       const int* tile_expert, const int* tile_begin, const int* tile_rows, const int* num_tiles,
                       int max_work_tiles, cudaStream_t s) {
  CUtensorMap mx, mw;
  int rc = tc5::make_map(&mx, X, x_rows, K, K, kMeBM);
  if (rc) return rc;
  rc = tc5::make_map(&mw, W, w_rows, K, K, GATED ? kMeBN / 2 : kMeBN);
  if (rc) return rc;
  auto kernel = moe_tcgen05_kernel<OutT, GATED>;
  const size_t smem = size_t(kMeStages) * kMeStageBytes + 1024;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem));
    if (e != cudaSuccess) return int(e);
    configured = true;
  }
  constexpr int BNOUT = GATED ? kMeBN / 2 : kMeBN;
  const long long most = (long long)max_work_tiles * ((N + BNOUT - 1) / BNOUT);
  const int sms = tc5::current_sm_count();
  kernel<<<dim3(unsigned(most < sms ? most : sms)), kMeThreads, smem, s>>>(mx, mw, reinterpret_cast<OutT*>(Y), N, K, ldy,
                                                                         tile_expert, tile_begin, tile_rows, num_tiles);
  return KVCM_LAUNCH_RESULT();
}

}  // namespace kvcm

using namespace kvcm;

// Sizes the tensor-core form takes: rows of xs, act and the weights must be 16-byte aligned.
KVCM_API int kvcm_moe_tcgen05_supports(int F, int D) { return F >= 8 && D >= 8 && (F % 8) == 0 && (D % 8) == 0; }

// The three steps after the sort (tiles of 128 pairs): gather, gate/up, down.
//   h [rows, D] bf16 (ldh apart); wgu [E, 2F, D]; wd [E, D, F]; pair_of/tile_*/num_tiles from the sort;
//   xs [pairs, D] and act [pairs, F] bf16 scratch; y [pairs, D] float, in the order of the sorted pairs.
KVCM_API int kvcm_moe_experts_tcgen05_bf16(const void* h, int ldh, const void* wgu, const void* wd, const int* pair_of,
                                           const int* tile_expert, const int* tile_begin, const int* tile_rows,
                                           const int* num_tiles, int pairs, int top, int E, int F, int D, void* xs,
                                           void* act, float* y, void* stream) {
  if (pairs == 0) return 0;
  if (!kvcm_moe_tcgen05_supports(F, D)) return KVCM_ERR_UNSUPPORTED;
  for (const void* p : {h, wgu, wd, (const void*)xs, (const void*)act, (const void*)y})
    if (reinterpret_cast<uintptr_t>(p) & 15) return KVCM_ERR_UNSUPPORTED;
  cudaStream_t s = (cudaStream_t)stream;
  const int max_work_tiles = pairs / kMeBM + E;
  moe_gather_kernel<<<pairs, 256, 0, s>>>((const bf16*)h, ldh, pair_of, top, (bf16*)xs, D);
  int rc = KVCM_LAUNCH_RESULT();
  if (rc) return rc;
  rc = launch_moe_tcgen05<bf16, true>(xs, pairs, wgu, (long long)E * 2 * F, act, F, D, F, tile_expert, tile_begin,
                                      tile_rows, num_tiles, max_work_tiles, s);
  if (rc) return rc;
  return launch_moe_tcgen05<float, false>(act, pairs, wd, (long long)E * D, y, D, F, D, tile_expert, tile_begin, tile_rows,
                                          num_tiles, max_work_tiles, s);
}

KVCM_API const int* kvcm_moe_tcgen05_error_address(void) {
  int* p = nullptr;
  return cudaGetSymbolAddress((void**)&p, g_moe_tcgen05_error) == cudaSuccess ? p : nullptr;
}

// Reads and clears the error word (0 = no bounded wait ever ran out).  Synchronises the device.
KVCM_API int kvcm_moe_tcgen05_error(void) {
  int v = 0, zero = 0;
  if (cudaMemcpyFromSymbol(&v, g_moe_tcgen05_error, sizeof v) != cudaSuccess) return -1;
  if (v != 0) cudaMemcpyToSymbol(g_moe_tcgen05_error, &zero, sizeof zero);
  return v;
}
