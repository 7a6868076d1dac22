// Expert-parallel exchange over NVLink peer memory (one process per GPU, buffers shared with CUDA IPC).
//
// The two exchange steps of an expert-parallel MoE block move a few KB per rank, so with a library collective they
// cost launch + protocol latency (about 12 us each at 2 ranks, 22 us at 8). Here the ranks write straight into each
// other's memory with ordinary stores and signal with one flag word per (destination, source):
//   dispatch  ep_exchange_kernel: CTA d writes this rank's rows, packed as (x | route), into rank d's gather buffer, fences,
//             writes the epoch into rank d's flag word of this rank; then CTA s waits for the flag of source s.
//   combine   moe_combine_kernel writes each finished output row into the part buffer of the rank that owns the row
//             (fused with the slot-ordered sum); the last CTA to finish fences and raises this rank's flag on every peer;
//             ep_sum_kernel waits for all sources' flags and adds the partial rows in rank order.
// Every wait is bounded (status word, then the kernel returns). No multicast, no TMA: plain peer stores and
// system-scope release / acquire flag accesses. A buffer is not reused before its readers are done: a rank can only send
// the rows of block b + 1 after it has summed block b, i.e. after every peer has finished all kernels of block b.
#pragma once
#include <stdint.h>

namespace ijah {

constexpr int EP_MAX_RANKS = 16;

struct EpDev {  // lives in device memory of the owning rank; pointers to every rank's exchange buffer (peer mappings)
  int rank, world, rows_cap, H, W;  // W = H + 2 top_k floats per packed row
  float *gather[EP_MAX_RANKS];      // rank d's [world * rows_cap][W]
  float *part[EP_MAX_RANKS];        // rank d's [world][rows_cap][H]
  uint32_t *gflag[EP_MAX_RANKS];    // rank d's [EP_MAX_RANKS] epochs of arrived rows per source
  uint32_t *pflag[EP_MAX_RANKS];    // rank d's [EP_MAX_RANKS] epochs of arrived partial outputs per source
  unsigned *counter;                // local: CTAs of the combine kernel that have finished
  // The epoch of the block in flight lives in device memory, so that a block (and a whole decode step) is the same
  // sequence of launches with the same arguments every time and can be replayed from a CUDA graph: the dispatch kernel
  // works with *epoch + 1 and its last CTA stores that value; the combine and sum kernels of the block then read it.
  uint32_t *epoch;                  // local
  unsigned *ticket;                 // local: CTAs of the dispatch kernel that have read the epoch and sent their rows
};

struct EpCtx {
  EpDev host{};          // host copy of the table
  EpDev *dev = nullptr;  // device copy
  void *local = nullptr; // this rank's exchange buffer (cudaMalloc, exported with cudaIpcGetMemHandle)
  void *peer[EP_MAX_RANKS] = {};
  uint32_t *route_own = nullptr;  // [rows_cap][2 top_k] routes of this rank's rows (the router's output)
  size_t off_gather = 0, off_part = 0, off_flags = 0, bytes = 0;
  int top_k = 0;
  bool connected = false;
};

void launch_ep_exchange(const EpCtx &c, const float *x_own, const uint32_t *route_own, int rows, int *status, cudaStream_t st);
void launch_ep_sum(const EpCtx &c, int rows, float *y_own, int *status, cudaStream_t st);

}  // namespace ijah
