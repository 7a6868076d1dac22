// Expert-parallel exchange kernels and their host context. See ep_exchange.cuh.
#include "common.hpp"
#include "ep_exchange.cuh"

namespace ijah {

__device__ __forceinline__ void st_release_sys(uint32_t *p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t *p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
// waits until *flag has reached `epoch`; gives up after about a second, recording `code` in the status word
__device__ __forceinline__ bool wait_epoch(const uint32_t *flag, uint32_t epoch, int *status, int code) {
  for (int i = 0; i < (1 << 22); i++) {
    if ((int32_t)(ld_acquire_sys(flag) - epoch) >= 0) return true;
    __nanosleep(200);
  }
  atomicExch(status, code);
  return false;
}

// CTA d: this rank's packed rows -> rank d's gather buffer, then the flag; afterwards CTA s waits for source s.
__global__ void __launch_bounds__(256) ep_exchange_kernel(const EpDev *ep, const float *pack_own, int rows, uint32_t epoch, int *status) {
  const int d = blockIdx.x, me = ep->rank;
  const int n4 = rows * ep->W / 4;  // W is a multiple of 4
  const float4 *src = reinterpret_cast<const float4 *>(pack_own);
  float4 *dst = reinterpret_cast<float4 *>(ep->gather[d] + (size_t)me * rows * ep->W);
  for (int i = threadIdx.x; i < n4; i += blockDim.x) dst[i] = src[i];
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) {
    st_release_sys(ep->gflag[d] + me, epoch);
    wait_epoch(ep->gflag[me] + d, epoch, status, 21);
  }
}

// y_own[r][c] = sum over source ranks (in rank order) of part[s][r][c], once every source's flag shows this epoch
__global__ void __launch_bounds__(256) ep_sum_kernel(const EpDev *ep, int rows, uint32_t epoch, float *y_own, int *status) {
  __shared__ int ok;
  const int me = ep->rank, world = ep->world, H = ep->H;
  if (threadIdx.x == 0) ok = 1;
  __syncthreads();
  if (threadIdx.x < world && !wait_epoch(ep->pflag[me] + threadIdx.x, epoch, status, 22)) ok = 0;
  __syncthreads();
  if (!ok) return;
  const int n4 = rows * H / 4;
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n4; i += gridDim.x * blockDim.x) {
    float4 acc = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
    for (int s = 0; s < world; s++) {
      const float4 v = __ldcg(reinterpret_cast<const float4 *>(ep->part[me] + (size_t)s * ep->rows_cap * H) + i);
      acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
    }
    reinterpret_cast<float4 *>(y_own)[i] = acc;
  }
}

void launch_ep_exchange(const EpCtx &c, int rows, uint32_t epoch, int *status, cudaStream_t st) {
  ep_exchange_kernel<<<c.host.world, 256, 0, st>>>(c.dev, c.pack_own, rows, epoch, status);
  IJ_CUDA(cudaGetLastError());
}

void launch_ep_sum(const EpCtx &c, int rows, uint32_t epoch, float *y_own, int *status, cudaStream_t st) {
  const int n4 = rows * c.host.H / 4;
  ep_sum_kernel<<<std::max(1, std::min(32, (n4 + 255) / 256)), 256, 0, st>>>(c.dev, rows, epoch, y_own, status);
  IJ_CUDA(cudaGetLastError());
}

}  // namespace ijah
