// Host launcher for stream_gemm_kernel instantiations (included by the .cu files that define a problem type).
#pragma once
#include "common.hpp"
#include "stream_gemm.cuh"

namespace ijah {

// Launch with programmatic stream serialization allowed: the kernel may be scheduled while its predecessor in the
// stream still runs and synchronises with it through pdl_wait() (also valid inside stream capture).
template <class... KArgs, class... Args>
void launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st, Args &&...args) {
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = grid; cfg.blockDim = block; cfg.dynamicSmemBytes = smem; cfg.stream = st;
  cudaLaunchAttribute at[1];
  at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  at[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = at; cfg.numAttrs = 1;
  IJ_CUDA(cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...));
}

template <class P, int MT, bool EX>
static void launch_stream_ex(const P &prob, const StreamLayout &lay, int grid, int *status, cudaStream_t st) {
  // the attribute belongs to the current device's context: set it on every launch (cheap) rather than once per process
  IJ_CUDA(cudaFuncSetAttribute(stream_gemm_kernel<P, MT, EX>, cudaFuncAttributeMaxDynamicSharedMemorySize, 226 * 1024));
  launch_pdl(stream_gemm_kernel<P, MT, EX>, dim3(grid), dim3(SG_THREADS), lay.total(), st, prob, lay, status);
}
// the product mode in force (g_summand_product) picks the kernel; the prepared rows of the same call were written to match
template <class P, int MT>
static void launch_stream_mt(const P &prob, const StreamLayout &lay, int grid, int *status, cudaStream_t st) {
  if (g_summand_product) launch_stream_ex<P, MT, false>(prob, lay, grid, status, st);
  else launch_stream_ex<P, MT, true>(prob, lay, grid, status, st);
}

template <class P>
void launch_stream(const P &prob, int MT, const StreamLayout &lay, int grid, int *status, cudaStream_t st) {
  IJ_CHECK(lay.stages >= 2 && lay.stages <= 16, "bad ring depth %d", lay.stages);
  switch (MT) {
    case 1: launch_stream_mt<P, 1>(prob, lay, grid, status, st); break;
    case 2: launch_stream_mt<P, 2>(prob, lay, grid, status, st); break;
    case 4: launch_stream_mt<P, 4>(prob, lay, grid, status, st); break;
    case 8: launch_stream_mt<P, 8>(prob, lay, grid, status, st); break;
    default: fail("unsupported row tile count %d", MT);
  }
}

}  // namespace ijah
