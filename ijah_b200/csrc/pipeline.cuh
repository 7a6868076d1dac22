// Shared-memory pipeline primitives for sm_100a: mbarriers with transaction counts and 1-D bulk async copies
// (global -> shared, completion signalled on an mbarrier). Every wait is bounded: after WAIT_LIMIT polls the waiter
// gives up, records the fact in a caller-provided status word and returns false, so a kernel can never spin forever.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace ijah {

// try_wait itself blocks for a hardware-defined slice before returning, so this many polls is on the order of a second.
constexpr uint32_t WAIT_LIMIT = 1u << 22;

__device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint64_t *bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_fence_init() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }

// barriers addressed by their 32-bit shared-memory address (the hot loops keep those in registers)
__device__ __forceinline__ void mbar_arrive_a(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx_a(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait_a(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}
// Bounded wait as ONE asm block, so the caller's loop has no control flow of its own around it: polls until the phase
// completes or WAIT_LIMIT polls have passed. Returns 1 (completed) or 0 (gave up).
__device__ __forceinline__ uint32_t mbar_wait_poll(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      ".reg .u32 n;\n\t"
      "mov.u32 n, 0;\n"
      "W:\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "@p bra D;\n\t"
      "add.u32 n, n, 1;\n\t"
      "setp.lt.u32 p, n, %3;\n\t"
      "@p bra W;\n\t"
      "mov.u32 %0, 0;\n\t"
      "bra E;\n"
      "D:\n\t"
      "mov.u32 %0, 1;\n"
      "E:\n\t"
      "}"
      : "=r"(ok)
      : "r"(bar), "r"(parity), "r"(WAIT_LIMIT)
      : "memory");
  return ok;
}
// arrive issued by the lanes whose `pred` is non-zero, as a predicated instruction (no branch)
__device__ __forceinline__ void mbar_arrive_if(uint32_t bar, uint32_t pred) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.u32 p, %1, 0;\n\t"
      "@p mbarrier.arrive.shared::cta.b64 _, [%0];\n\t}" ::"r"(bar), "r"(pred)
      : "memory");
}
// Bounded wait. Returns false (and sets *status = code, if status is given) when the limit is hit.
__device__ __forceinline__ bool mbar_wait_a(uint32_t bar, uint32_t parity, int *status, int code) {
  if (mbar_wait_poll(bar, parity)) return true;
  if (status) atomicExch(status, code);
  return false;
}

// The same for a waiter that is idle by design (a producer far ahead of its consumers): it sleeps between polls so that its
// polling does not take instruction-issue slots from the warps that work. 2^21 sleeps of `ns` bound the wait.
__device__ __forceinline__ bool mbar_wait_sleep(uint64_t *bar, uint32_t parity, int *status, int code, uint32_t ns) {
  const uint32_t a = smem_u32(bar);
  for (uint32_t i = 0; i < (1u << 21); i++) {
    if (mbar_try_wait_a(a, parity)) return true;
    __nanosleep(ns);
  }
  if (status) atomicExch(status, code);
  return false;
}

__device__ __forceinline__ void mbar_arrive(uint64_t *bar) { mbar_arrive_a(smem_u32(bar)); }
__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t *bar, uint32_t bytes) { mbar_arrive_expect_tx_a(smem_u32(bar), bytes); }
__device__ __forceinline__ bool mbar_try_wait(uint64_t *bar, uint32_t parity) { return mbar_try_wait_a(smem_u32(bar), parity); }
__device__ __forceinline__ bool mbar_wait(uint64_t *bar, uint32_t parity, int *status, int code) {
  return mbar_wait_a(smem_u32(bar), parity, status, code);
}

// 1-D bulk copy global -> this CTA's shared memory; src, dst 16-byte aligned, bytes a multiple of 16.
__device__ __forceinline__ void bulk_g2s(void *dst, const void *src, uint32_t bytes, uint64_t *bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                   smem_u32(dst)),
               "l"(src), "r"(bytes), "r"(smem_u32(bar))
               : "memory");
}

// The same with an L2 cache policy. Compressed weights are read exactly once per launch: streamed with evict-first they
// do not push the data that is re-read (activations, partial sums, plans, the kernels' own code) out of L2.
__device__ __forceinline__ uint64_t l2_evict_first_policy() {
  uint64_t pol;
  asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(pol));
  return pol;
}
__device__ __forceinline__ void bulk_g2s_hint(void *dst, const void *src, uint32_t bytes, uint64_t *bar, uint64_t policy) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1], %2, [%3], %4;" ::"r"(
                   smem_u32(dst)),
               "l"(src), "r"(bytes), "r"(smem_u32(bar)), "l"(policy)
               : "memory");
}

// Tiled TMA load of one 3-D box (global -> this CTA's shared memory, no multicast) with an L2 cache policy. `tmap` is the
// generic address of a CUtensorMap in kernel-parameter or global memory; x is the innermost coordinate (x * element size
// must be a multiple of 16 bytes); dst 128-byte aligned. The mbarrier receives the box size in bytes (out-of-range parts
// of the box are zero-filled and counted).
__device__ __forceinline__ void tma_load_3d(uint32_t dst, const void *tmap, int x, int y, int z, uint32_t bar, uint64_t policy) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1, {%2, %3, %4}], [%5], %6;" ::"r"(dst),
      "l"(tmap), "r"(x), "r"(y), "r"(z), "r"(bar), "l"(policy)
      : "memory");
}
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const void *tmap, int x, int y, uint32_t bar, uint64_t policy) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1, {%2, %3}], [%4], %5;" ::"r"(dst),
      "l"(tmap), "r"(x), "r"(y), "r"(bar), "l"(policy)
      : "memory");
}
__device__ __forceinline__ void tma_prefetch_descriptor(const void *tmap) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(tmap) : "memory");
}

__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(addr));
}

// D (16x8, f32) += A (16x16, f16, row) * B (16x8, f16, col)
__device__ __forceinline__ void mma_16816(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// D = A * B (the same shapes, accumulator starts at zero: no registers to clear)
__device__ __forceinline__ void mma_16816_zero(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
      : "=f"(d[0]), "=f"(d[1]), "=f"(d[2]), "=f"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1), "f"(0.0f));
}

// Programmatic dependent launch: a kernel launched with the stream-serialization attribute may start while its
// predecessor in the stream still runs. pdl_wait() blocks until the predecessor has completed and its writes are visible
// (a no-op for a plain launch); pdl_launch() lets the successor's CTAs be scheduled once every CTA of this grid has
// called it or exited. Every kernel of a chain calls pdl_wait() before pdl_launch() and before it touches anything an
// earlier kernel wrote, so completion of one kernel implies completion of all kernels before it.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

}  // namespace ijah
