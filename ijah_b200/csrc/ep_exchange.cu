// Expert-parallel exchange kernels and their host context. See ep_exchange.cuh.
#include <algorithm>

#include "common.hpp"
#include "ep_exchange.cuh"
#include "launch.cuh"

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

// CTA d: this rank's rows, packed as (x row | route row), -> rank d's gather buffer, then the flag; afterwards CTA s waits
// for source s. x_own [rows][H] floats and route_own [rows][2 top_k] words are the router's input and output.
__global__ void __launch_bounds__(256) ep_exchange_kernel(const EpDev *ep, const float *x_own, const uint32_t *route_own, int rows, int *status) {
  pdl_wait();
  pdl_launch();
  const int d = blockIdx.x, me = ep->rank, H4 = ep->H / 4, W4 = ep->W / 4, R4 = W4 - H4;
  const uint32_t epoch = *reinterpret_cast<volatile uint32_t *>(ep->epoch) + 1u;  // every CTA reads it before any CTA can store the new value
  float4 *dst = reinterpret_cast<float4 *>(ep->gather[d] + (size_t)me * rows * ep->W);
  for (int i = threadIdx.x; i < rows * W4; i += blockDim.x) {
    const int r = i / W4, c = i - r * W4;
    dst[i] = c < H4 ? reinterpret_cast<const float4 *>(x_own)[r * H4 + c] : reinterpret_cast<const float4 *>(route_own)[r * R4 + c - H4];
  }
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) {
    st_release_sys(ep->gflag[d] + me, epoch);
    wait_epoch(ep->gflag[me] + d, epoch, status, 21);
    // the last CTA to get here (all have read the old epoch by then) publishes the block's epoch for the kernels that follow
    if (atomicAdd(ep->ticket, 1u) == gridDim.x - 1) {
      *ep->ticket = 0u;
      *reinterpret_cast<volatile uint32_t *>(ep->epoch) = epoch;
    }
  }
}

// y_own[r][c] = sum over source ranks (in rank order) of part[s][r][c], once every source's flag shows this epoch
__global__ void __launch_bounds__(256) ep_sum_kernel(const EpDev *ep, int rows, float *y_own, int *status) {
  __shared__ int ok;
  pdl_wait();
  pdl_launch();
  const int me = ep->rank, world = ep->world, H = ep->H;
  const uint32_t epoch = *reinterpret_cast<volatile uint32_t *>(ep->epoch);
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

void launch_ep_exchange(const EpCtx &c, const float *x_own, const uint32_t *route_own, int rows, int *status, cudaStream_t st) {
  launch_pdl(ep_exchange_kernel, dim3(c.host.world), dim3(256), 0, st, (const EpDev *)c.dev, x_own, route_own, rows, status);
}

void launch_ep_sum(const EpCtx &c, int rows, float *y_own, int *status, cudaStream_t st) {
  const int n4 = rows * c.host.H / 4;
  launch_pdl(ep_sum_kernel, dim3(std::max(1, std::min(32, (n4 + 255) / 256))), dim3(256), 0, st, (const EpDev *)c.dev, rows, y_own, status);
}

}  // namespace ijah
