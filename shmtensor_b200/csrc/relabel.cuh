// Shared declarations of the relabel kernels (used by relabel.cu and the fused
// multi-hop sampler).
#pragma once

#include "ctx.cuh"
#include "lookback.cuh"

namespace shmt {

constexpr int kRelThreads = 256;
constexpr int kRelItems = 4;
constexpr int kRelTile = kRelThreads * kRelItems;
constexpr int kMaxParts = 8;

struct Parts {
  const void* ptr[kMaxParts];
  int64_t start[kMaxParts + 1];  // element offset of each part; start[kMaxParts] = total
  int n;
  int is64;
  // Two-part form whose sizes were produced on the device (dev_n1 set): |part 1| = *dev_n1,
  // |part 0| = *dev_n0, or the host's start[1] if dev_n0 is null; the kernels fill start[].
  const int64_t* dev_n0;
  const int64_t* dev_n1;
};

struct RelTable {
  long long* keys;  // cap entries, -1 = empty
  unsigned* first;  // cap entries, smallest input index holding the key (all ones = none)
  unsigned* newid;  // cap entries, dense id of the key (written by the compact kernel)
  uint32_t mask;    // cap - 1
};

// Slots of the table that serves up to `numel_bound` ids.
uint64_t relabel_capacity(int64_t numel_bound);

// Queue the three relabel kernels.  `numel_bound` >= the real element count sizes the
// table and the grids; `newid` is scratch of 4 * relabel_capacity(numel_bound) bytes;
// ticket/status/result are zeroed device words.
int launch_relabel(shmt_ctx* ctx, const Parts& ps, int64_t numel_bound, unsigned* newid,
                   void* out_unique, void* out_relabel, TileStates st, int64_t* ticket,
                   int64_t* status, int64_t* result, cudaStream_t s);

}  // namespace shmt
