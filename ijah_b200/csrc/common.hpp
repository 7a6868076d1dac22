// Host-side plumbing shared by the C ABI sources: per-thread error text, exception -> return-code wrapper, CUDA checks,
// and a per-device growable scratch arena. The error convention is the reference's (include/engine.h:3-5 of the
// reference: int functions return 0 / -1, pointer functions NULL, message in ne_last_error(), per thread).
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>

#include <cstdarg>
#include <cstdio>
#include <stdexcept>
#include <string>

namespace ijah {

std::string &last_error_ref();

struct Error : std::runtime_error {
  using std::runtime_error::runtime_error;
};

[[noreturn]] inline void fail(const char *fmt, ...) {
  char buf[1024];
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(buf, sizeof buf, fmt, ap);
  va_end(ap);
  throw Error(buf);
}

// Product mode of the decode-width stream kernels (ne_exl3_set_summand_product): 0 = every weight enters the tensor
// core as fp16(lo + hi), the value the format defines; 1 = as its two fp16 summands, whose sum the fp32 accumulator
// forms unrounded. Read when a call is enqueued (or recorded into a graph), by the operand-prep kernels' launchers and
// the stream kernel's launcher alike.
inline int g_summand_product = 0;

#define IJ_CHECK(cond, ...) \
  do {                      \
    if (!(cond)) ::ijah::fail(__VA_ARGS__); \
  } while (0)

#define IJ_CUDA(expr)                                                                              \
  do {                                                                                             \
    cudaError_t e_ = (expr);                                                                       \
    if (e_ != cudaSuccess) ::ijah::fail("%s: %s (%s:%d)", #expr, cudaGetErrorString(e_), __FILE__, __LINE__); \
  } while (0)

template <class F>
int c_call(F &&f) {
  try {
    f();
    return 0;
  } catch (const std::exception &e) {
    last_error_ref() = e.what();
  } catch (...) {
    last_error_ref() = "unknown error";
  }
  return -1;
}

// Scratch that outlives a call: one arena per device, grown on demand (never shrunk), used by the entry points that
// take no workspace argument. Not thread-safe across concurrent calls on the same device (as the reference: one engine
// thread drives the device, server/ne_server.py:8-9).
void *device_scratch(size_t bytes);
int *device_status_word();   // zero-initialised int the kernels report bounded-wait failures into
void check_status_word();    // throws if a kernel reported a failure (reads the word after a stream sync)
int sm_count();

// Tensor map over an EXL3 trellis for the stream kernels' tiled TMA loads: the trellis of E matrices of IT x OT tiles of
// 32K bytes each is described as a 3-D array of 8-byte elements, x = position along a row of tiles (OT * 4K elements),
// y = k-tile (stride OT * 32K bytes), z = matrix (stride IT * OT * 32K bytes); box = (8 tiles, ks k-tiles, 1). Host-side
// arithmetic only (no allocation, no device work). `base` must be 16-byte aligned.
void make_trellis_map(CUtensorMap *out, const void *base, int E, int IT, int OT, int K, int ks);

}  // namespace ijah
