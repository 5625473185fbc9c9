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

// One 16-byte slot per distinct id, so that claiming the key and recording the first occurrence
// touch one sector, as do reading the new id and emptying the slot.
struct __align__(16) RelSlot {
  long long key;   // -1 = empty
  unsigned first;  // smallest input index holding the key (all ones = none)
  unsigned newid;  // dense id of the key (written by the compact kernel; needs no initial value)
};

struct RelTable {
  RelSlot* slots;  // cap entries
  uint32_t mask;   // cap - 1
};

#ifdef __CUDACC__
// Hash mask for an input of at most `numel` ids: load <= 0.5, never beyond the table.
__device__ __forceinline__ uint32_t relabel_mask_for(int64_t numel, uint32_t table_mask) {
  if (numel <= 0) return table_mask < 63u ? table_mask : 63u;
  const uint32_t want = numel * 2 <= 64 ? 63u : (0xFFFFFFFFu >> __clz((uint32_t)(numel * 2 - 1)));
  return want < table_mask ? want : table_mask;
}

// Claim (or find) the slot of `key`, record `i` as a candidate first occurrence, and return
// the slot.  Linear probing from mix64(key) & mask; bounded by the table size.
__device__ __forceinline__ uint32_t relabel_insert_one(RelSlot* slots, uint32_t mask, long long key,
                                                       unsigned i, int64_t* status) {
  uint32_t pos = (uint32_t)mix64((uint64_t)key) & mask;
  uint32_t steps = 0;
  while (true) {
    long long cur = __ldcg(&slots[pos].key);
    if (cur == kEmptyKey)
      cur = (long long)atomicCAS(reinterpret_cast<unsigned long long*>(&slots[pos].key),
                                 (unsigned long long)kEmptyKey, (unsigned long long)key);
    if (cur == kEmptyKey || cur == key) break;
    pos = (pos + 1) & mask;
    if (++steps > mask) {  // cannot happen at load <= 0.5; bounded all the same
      atomicMax(reinterpret_cast<unsigned long long*>(status), (unsigned long long)DEV_OVERFLOW);
      break;
    }
  }
  atomicMin(&slots[pos].first, i);
  return pos;
}
#endif

// Slots of the table that serves up to `numel_bound` ids.
uint64_t relabel_capacity(int64_t numel_bound);

// Queue the three relabel kernels.  `numel_bound` >= the real element count sizes the
// table and the grids; ticket/status/result are zeroed device words.
// `pdl`: launch with programmatic stream serialization (see pdl_prologue in common.cuh).
// `inserted`: the slots were already claimed and recorded in out_relabel by the producer
// of the ids (the fused sampling kernel), so only the compact and remap kernels run.
// `post`: the compact kernel hands the result words to the host as soon as the unique count is
// final, i.e. while the remap kernel is still to run (it produces neither sizes nor errors).
int launch_relabel(shmt_ctx* ctx, const Parts& ps, int64_t numel_bound, void* out_unique, void* out_relabel, TileStates st, int64_t* ticket,
                   int64_t* status, int64_t* result, cudaStream_t s, bool inserted = false,
                   bool pdl = false, const HostPost* post = nullptr);

// The context's table for `numel_bound` ids (reserving it).
int relabel_table(shmt_ctx* ctx, int64_t numel_bound, RelTable* t, cudaStream_t s);

}  // namespace shmt
