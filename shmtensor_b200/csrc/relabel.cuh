// Shared declarations of the relabel kernels (used by relabel.cu and the fused
// multi-hop sampler).
#pragma once

#include "ctx.cuh"
#include "lookback.cuh"

namespace shmt {

constexpr int kRelThreads = 256;
// Elements per thread of the compact kernel, and so per tile.  Its tiles hand their counts on
// through a look-back that advances 32 tiles per round trip: for a large input the length of that
// chain, not memory, is what small tiles cost, so inputs of kRelLargeInput elements and more use
// kRelItemsLarge per thread; a small input is a few dependent reads long and wants many CTAs.
// Look-back state is always sized for the small tile.
constexpr int kRelItems = 4;
constexpr int kRelItemsLarge = 16;
constexpr int64_t kRelLargeInput = 4 << 20;
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

// What the inserting pass leaves per element in the output array: the element's slot, plus a mark
// on the elements that are certainly NOT the first occurrence of their id (they met a smaller index
// in the slot), so that the later passes need not look at the slot to know.  64-bit arrays always
// have room for the mark; 32-bit ones as long as the table has fewer than 2^31 slots.
constexpr unsigned long long kRelNotFirst64 = 1ull << 40;
constexpr uint32_t kRelNotFirst32 = 0x80000000u;

__device__ __forceinline__ int64_t relabel_pack(uint32_t pos, bool maybe_first, bool is64, uint32_t table_mask) {
  if (is64) return (int64_t)((unsigned long long)pos | (maybe_first ? 0ull : kRelNotFirst64));
  if (table_mask < kRelNotFirst32 && !maybe_first) pos |= kRelNotFirst32;
  return (int64_t)(int32_t)pos;
}

__device__ __forceinline__ uint32_t relabel_unpack64(unsigned long long raw, bool* maybe_first) {
  *maybe_first = !(raw & kRelNotFirst64);
  return (uint32_t)raw;
}

__device__ __forceinline__ uint32_t relabel_unpack32(uint32_t raw, uint32_t table_mask, bool* maybe_first) {
  if (table_mask < kRelNotFirst32) {
    *maybe_first = !(raw & kRelNotFirst32);
    return raw & ~kRelNotFirst32;
  }
  *maybe_first = true;
  return raw;
}

__device__ __forceinline__ uint32_t relabel_unpack(const void* slot_of, bool is64, int64_t i, uint32_t table_mask,
                                                   bool* maybe_first) {
  if (is64) return relabel_unpack64(reinterpret_cast<const unsigned long long*>(slot_of)[i], maybe_first);
  return relabel_unpack32(reinterpret_cast<const uint32_t*>(slot_of)[i], table_mask, maybe_first);
}

// Claim (or find) the slot of `key`, record `i` as a candidate first occurrence, and return
// the slot.  Linear probing from mix64(key) & mask; bounded by the table size.  *maybe_first is
// false when the slot was seen to hold a smaller index (then `i` cannot be the first occurrence).
// `direct`: every id of the input is known to lie in [0, mask], so the id itself is its slot:
// neighbouring ids share cache lines and nothing collides.
__device__ __forceinline__ uint32_t relabel_insert_one(RelSlot* slots, uint32_t mask, long long key,
                                                       unsigned i, int64_t* status, bool* maybe_first,
                                                       bool direct = false) {
  uint32_t pos = direct ? (uint32_t)key : (uint32_t)mix64((uint64_t)key) & mask;
  uint32_t steps = 0;
  unsigned seen_first;
  while (true) {
    // key and first index come with one 16-byte load
    const uint4 s = __ldcg(reinterpret_cast<const uint4*>(slots + pos));
    long long cur = (long long)(((unsigned long long)s.y << 32) | s.x);
    seen_first = s.z;
    if (cur == kEmptyKey) {
      cur = (long long)atomicCAS(reinterpret_cast<unsigned long long*>(&slots[pos].key),
                                 (unsigned long long)kEmptyKey, (unsigned long long)key);
      seen_first = 0xFFFFFFFFu;  // claimed just now, by this element or by another one of the same id
    }
    if (cur == kEmptyKey || cur == key) break;
    pos = (pos + 1) & mask;
    if (++steps > mask) {  // cannot happen at load <= 0.5; bounded all the same
      atomicMax(reinterpret_cast<unsigned long long*>(status), (unsigned long long)DEV_OVERFLOW);
      break;
    }
  }
  // `first` only ever goes down: when the index seen there is already smaller than this one the
  // atomic would change nothing, and most elements of a frontier are such repeats.  Nothing waits
  // for the atomic's result: an element that lowers the index, or loses to a still smaller one, is
  // simply left among the candidates.
  *maybe_first = seen_first > i;
  if (*maybe_first) atomicMin(&slots[pos].first, i);
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
// `range`: a zeroed device word; when given, a first kernel stores the largest id there and the
// insert kernel uses ids as slots if they all fit the table (see relabel_insert_one).
int launch_relabel(shmt_ctx* ctx, const Parts& ps, int64_t numel_bound, void* out_unique, void* out_relabel, TileStates st, int64_t* ticket,
                   int64_t* status, int64_t* result, cudaStream_t s, bool inserted = false,
                   bool pdl = false, const HostPost* post = nullptr, int64_t* range = nullptr);

// The context's table for `numel_bound` ids (reserving it).
int relabel_table(shmt_ctx* ctx, int64_t numel_bound, RelTable* t, cudaStream_t s);

}  // namespace shmt
