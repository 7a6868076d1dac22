// ne_exl3_linear_static: the EXL3 Linear for callers that must not allocate.
//
// ne_exl3_linear takes its scratch (k-split partial sums and the prepared fp16 operand) from an arena that the library
// grows with cudaMalloc whenever a call needs more than any earlier one did. Some callers cannot tolerate that: code
// that runs inside a memory-pool or allocator hook, a real-time serving loop that was handed a fixed memory budget at
// start-up, or a host that shares the GPU with another runtime owning all remaining device memory. For them the same
// kernels run here on a fixed scratch area that is part of the library image itself: a file-scope __device__ array,
// resident on every GPU that loads the library until the process exits. Nothing is allocated or freed, by this entry
// point or by any routine it calls, on the first call or later.
//
// The first call on a device looks up the device address of that array (cudaGetSymbolAddress, with the device
// current); make that first call before any stream capture begins. All calls share the one area and it keeps what the
// last call left in it. Nothing in it has to start at zero (every partial sum and operand element a call reads was
// written by the same call), but two calls whose GPU work overlaps -- different streams, or different threads -- race on
// it and corrupt each other's results.
#include "../../include/ijah_b200.h"
#include "common.hpp"
#include "exl3_linear.cuh"

using namespace ijah;

namespace {

constexpr size_t kStaticScratchBytes = 8u << 20;  // 8 MiB; the header says what fits
constexpr int kMaxDevices = 64;

static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];

struct DeviceSlots {
  void *scratch = nullptr;
  int *status = nullptr;  // the library's bounded-wait status word (also part of the image: ne_device_wait_status reads it)
};
DeviceSlots g_slots[kMaxDevices];

// In host code `g_static_scratch` is only a handle for the symbol, not a device address; the address the kernels need
// comes from cudaGetSymbolAddress, asked once per device with that device current.
DeviceSlots &slots_of_current_device() {
  int d = 0;
  IJ_CUDA(cudaGetDevice(&d));
  IJ_CHECK(d >= 0 && d < kMaxDevices, "device ordinal %d not supported by the static scratch table", d);
  DeviceSlots &s = g_slots[d];
  if (s.scratch == nullptr) {
    void *p = nullptr;
    IJ_CUDA(cudaGetSymbolAddress(&p, g_static_scratch));
    s.status = device_status_word();
    s.scratch = p;
  }
  return s;
}

}  // namespace

extern "C" {

NE_API uint64_t ne_exl3_linear_static_capacity(void) { return kStaticScratchBytes; }

NE_API int ne_exl3_linear_static(const ne_exl3_weight *w, const float *x_dev, int rows, float *y_dev, void *stream) {
  return c_call([&] {
    IJ_CHECK(w && w->trellis_dev && w->suh_dev && w->svh_dev && x_dev && y_dev, "null argument");
    IJ_CHECK(((uintptr_t)w->trellis_dev & 15) == 0, "trellis must be 16-byte aligned on the device");
    const LinearPlan p = plan_linear(w->in, w->out, w->K, rows);
    IJ_CHECK(p.scratch_bytes() <= kStaticScratchBytes,
             "ne_exl3_linear_static: %d rows of a %d -> %d Linear need %zu bytes of scratch, the built-in area holds %zu; "
             "use fewer rows per call or ne_exl3_linear",
             rows, w->in, w->out, p.scratch_bytes(), kStaticScratchBytes);
    DeviceSlots &s = slots_of_current_device();
    launch_linear(p, w->trellis_dev, w->suh_dev, w->svh_dev, x_dev, y_dev, s.scratch, s.status, (cudaStream_t)stream);
  });
}

}  // extern "C"
