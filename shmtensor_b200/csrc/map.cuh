// Static open-addressing hashmap for sm_100a: device view + cooperative probes.
//
// Layout: 16-byte slots {int64 key, int64 value}, grouped in windows of 4 slots
// (64 bytes, half a cache line).  A key's home window is mulhi(mix64(key),
// n_windows); probing is linear over windows.  A 4-lane tile inspects one
// window per step (each lane one 16-byte load) and votes with a ballot, so a
// warp resolves 8 keys per step and 32 keys with four independent steps in
// flight.  An empty slot ends a probe; an erased slot (key -2) does not, and is
// taken again by a later bulk insert.
// Empty key = -1 (the reference's sentinel, include/cuco_hashmap.cuh:58-59);
// -2 marks an erased slot, so both are reserved (ids are non-negative);
// int32 keys are stored sign-extended, int32 values likewise.
#pragma once

#include "common.cuh"

namespace shmt {

struct __align__(16) Slot {
  long long key;
  long long val;
};

struct MapView {
  Slot* slots;         // nullptr: no map (every lookup misses)
  uint64_t n_windows;  // table holds 4 * n_windows slots
  int key32;           // narrow lookups to int32 first (map built from int32 keys)
};

constexpr int kWindow = 4;
constexpr int64_t kErasedKey = -2;

}  // namespace shmt

struct shmt_map {
  int device = 0;
  shmt::MapView view{nullptr, 0, 0};
  int64_t capacity = 0;  // as requested; what capacity() reports
  int key_dtype = SHMT_I64;
  int val_dtype = SHMT_I64;
  bool owns_table = false;
  size_t table_bytes = 0;
  int64_t* d_meta = nullptr;  // device: [0] status, [1] number of keys stored
  int64_t size = 0;
};

namespace shmt {

inline MapView view_of(const shmt_map* m) {
  return m ? m->view : MapView{nullptr, 0, 0};
}

#ifdef __CUDACC__

__device__ __forceinline__ int64_t narrow_key(const MapView& m, int64_t k) {
  return m.key32 ? (int64_t)(int32_t)k : k;
}

__device__ __forceinline__ bool reserved_key(int64_t k) { return k == kEmptyKey || k == kErasedKey; }

__device__ __forceinline__ uint64_t home_window(const MapView& m, int64_t k) {
  return __umul64hi(mix64((uint64_t)k), m.n_windows);
}

// Look up one key per lane.  All 32 lanes of the warp must call; lanes with
// valid == false take part in the votes only.  Returns the value or -1.
__device__ __forceinline__ int64_t warp_find(const MapView& m, int64_t key, bool valid) {
  const unsigned full = 0xffffffffu;
  const unsigned lane = threadIdx.x & 31, sub = lane & 3, tile = lane >> 2;
  key = narrow_key(m, key);
  if (reserved_key(key)) valid = false;
  const longlong2* slots = reinterpret_cast<const longlong2*>(m.slots);

  longlong2 s[4];
  int64_t kr[4];
  int vr[4];
#pragma unroll
  for (int r = 0; r < 4; ++r) {
    const int src = r * 8 + tile;
    kr[r] = __shfl_sync(full, key, src);
    vr[r] = __shfl_sync(full, (int)valid, src);
    s[r] = make_longlong2(kEmptyKey, -1);
    if (vr[r]) s[r] = __ldg(slots + home_window(m, kr[r]) * kWindow + sub);
  }
  int64_t result = -1;
  int more = 0;
#pragma unroll
  for (int r = 0; r < 4; ++r) {
    const bool match = vr[r] && s[r].x == kr[r];
    const bool empty = !vr[r] || s[r].x == kEmptyKey;
    const unsigned mb = (__ballot_sync(full, match) >> (tile * 4)) & 0xFu;
    const unsigned eb = (__ballot_sync(full, empty) >> (tile * 4)) & 0xFu;
    const int from = mb ? (int)(tile * 4 + __ffs(mb) - 1) : (int)lane;
    const int64_t val = __shfl_sync(full, s[r].y, from);
    const int64_t res = mb ? val : -1;
    const int cont = (!mb && !eb) ? 1 : 0;
    const int64_t rv = __shfl_sync(full, res, (lane & 7) * 4);
    const int rc = __shfl_sync(full, cont, (lane & 7) * 4);
    if ((int)(lane >> 3) == r) {
      result = rv;
      more = rc;
    }
  }
  if (more) {
    // rare: the home window was full of other keys; walk on, one whole window (four
    // independent 16-byte loads) per step
    uint64_t w = home_window(m, key);
    for (uint64_t step = 1; step < m.n_windows; ++step) {
      w = w + 1 == m.n_windows ? 0 : w + 1;
      const longlong2* p = slots + w * kWindow;
      const longlong2 c0 = __ldg(p), c1 = __ldg(p + 1), c2 = __ldg(p + 2), c3 = __ldg(p + 3);
      if (c0.x == key) { result = c0.y; break; }
      if (c1.x == key) { result = c1.y; break; }
      if (c2.x == key) { result = c2.y; break; }
      if (c3.x == key) { result = c3.y; break; }
      if (c0.x == kEmptyKey || c1.x == kEmptyKey || c2.x == kEmptyKey || c3.x == kEmptyKey) break;
    }
  }
  return result;
}

// 16-byte compare-and-swap on one slot (atom.cas.b128, sm_90+): key and value
// become visible together, so no reader ever sees a claimed slot without its value.
__device__ __forceinline__ longlong2 cas_slot(Slot* p, longlong2 expect, longlong2 desired) {
  longlong2 old;
  asm volatile(
      "{\n\t"
      ".reg .b128 c, s, o;\n\t"
      "mov.b128 c, {%2, %3};\n\t"
      "mov.b128 s, {%4, %5};\n\t"
      "atom.global.cas.b128 o, [%6], c, s;\n\t"
      "mov.b128 {%0, %1}, o;\n\t"
      "}"
      : "=l"(old.x), "=l"(old.y)
      : "l"(expect.x), "l"(expect.y), "l"(desired.x), "l"(desired.y), "l"(p)
      : "memory");
  return old;
}

// One thread inserts one (key, value): walk the slots from the start of the home window up to the
// first empty one, which proves the key absent, then claim the first erased slot met on the way,
// else that empty slot, with a 16-byte CAS.  A table that was once full has no empty slot left
// (erasing leaves markers): a whole lap without the key proves it absent just as well, and the
// first erased slot is claimed then.  Occupied slots never change while inserts run, so two
// threads inserting the same key meet at the same slot and one of them sees the other's key.
// Without erased slots this is the placement rule of warp_insert (first empty slot in window
// order), so both can fill one table.  For bulk builds, where every thread has its own key and
// nothing else to wait for, this is faster than the cooperative form.  Must not run concurrently
// with thread_erase.  Returns true if the key is new; *overflow is set if the table is full.
__device__ __forceinline__ bool thread_insert(const MapView& m, int64_t key, int64_t val, bool assign,
                                              bool* overflow) {
  key = narrow_key(m, key);
  if (reserved_key(key)) return false;
  const uint64_t n_slots = m.n_windows * kWindow, none = ~0ULL;
  // a lost race starts the walk again; a few restarts cover any realistic contention
  for (int attempt = 0; attempt < 16; ++attempt) {
    uint64_t pos = home_window(m, key) * kWindow, erased_at = none, target = none;
    for (uint64_t step = 0; step < n_slots; ++step) {
      const long long cur = __ldcg(&m.slots[pos].key);
      if (cur == key) {
        if (assign) m.slots[pos].val = val;
        return false;
      }
      if (cur == kErasedKey && erased_at == none) erased_at = pos;
      if (cur == kEmptyKey) {
        target = erased_at != none ? erased_at : pos;
        break;
      }
      pos = pos + 1 == n_slots ? 0 : pos + 1;
    }
    if (target == none) target = erased_at;  // a whole lap: no empty slot anywhere
    if (target == none) break;               // nor an erased one: the table is full
    const long long expect = target == erased_at ? kErasedKey : kEmptyKey;
    const longlong2 old = cas_slot(m.slots + target, make_longlong2(expect, -1), make_longlong2(key, val));
    if (old.x == expect) return true;
    if (old.x == key) {
      if (assign) m.slots[target].val = val;
      return false;
    }
    // another key took the slot first: walk again
  }
  *overflow = true;
  return false;
}

// One thread erases one key: the slot becomes {-2, -1}.  Returns the value the key had, or -1 if
// it was absent (or another thread of the same launch erased it first).
__device__ __forceinline__ int64_t thread_erase(const MapView& m, int64_t key) {
  key = narrow_key(m, key);
  if (reserved_key(key)) return -1;
  const uint64_t n_slots = m.n_windows * kWindow;
  uint64_t pos = home_window(m, key) * kWindow;
  for (uint64_t step = 0; step < n_slots; ++step) {
    Slot* p = m.slots + pos;
    const long long cur = __ldcg(&p->key);
    if (cur == kEmptyKey) return -1;
    if (cur == key) {
      long long v = __ldcg(&p->val);
      for (int tries = 0; tries < 4; ++tries) {
        const longlong2 old = cas_slot(p, make_longlong2(key, v), make_longlong2(kErasedKey, -1));
        if (old.x != key) return -1;
        if (old.y == v) return v;
        v = old.y;
      }
      return -1;
    }
    pos = pos + 1 == n_slots ? 0 : pos + 1;
  }
  return -1;
}

// Insert one (key, value) per lane; all 32 lanes must call.  A key already in
// the table keeps its slot; its value is replaced only if `assign`.  Returns
// the value now stored for the key (-1 for invalid lanes or on overflow) and
// counts newly stored keys in *n_new (warp total, same on every lane).
// Placement is thread_insert's: the first erased slot met before the first empty one (or, in a
// table without empty slots, in a whole lap), else that empty slot.
__device__ __forceinline__ int64_t warp_insert(const MapView& m, int64_t key, int64_t val,
                                               bool valid, bool assign, int64_t* status_word,
                                               int* n_new) {
  const unsigned full = 0xffffffffu;
  const unsigned lane = threadIdx.x & 31, sub = lane & 3, tile = lane >> 2;
  const uint64_t none = ~0ULL;
  key = narrow_key(m, key);
  if (reserved_key(key)) valid = false;
  int64_t result = -1;
  int added = 0;
#pragma unroll 1
  for (int r = 0; r < 4; ++r) {
    const int src = r * 8 + tile;
    const int64_t k = __shfl_sync(full, key, src);
    const int64_t v = __shfl_sync(full, val, src);
    bool done = !__shfl_sync(full, (int)valid, src);
    uint64_t w = done ? 0 : home_window(m, k);
    uint64_t steps = 0, erased_slot = none;  // same on the four lanes of a tile
    int restarts = 0;
    int64_t res = -1;
    bool newly = false;
    while (__any_sync(full, !done)) {
      Slot* p = m.slots + w * kWindow + sub;
      longlong2 s = make_longlong2(0, 0);
      if (!done) s = __ldcg(reinterpret_cast<const longlong2*>(p));
      const bool match = !done && s.x == k;
      const bool empty = !done && s.x == kEmptyKey;
      const bool erased = !done && s.x == kErasedKey;
      const unsigned mb = (__ballot_sync(full, match) >> (tile * 4)) & 0xFu;
      const unsigned eb = (__ballot_sync(full, empty) >> (tile * 4)) & 0xFu;
      const unsigned rb = (__ballot_sync(full, erased) >> (tile * 4)) & 0xFu;
      if (!done && !mb && erased_slot == none && rb) {
        // only an erased slot in front of the window's first empty one counts
        const unsigned first_r = (unsigned)__ffs(rb) - 1u;
        if (!eb || first_r < (unsigned)__ffs(eb) - 1u) erased_slot = w * kWindow + first_r;
      }
      const bool lap = !done && !mb && !eb && steps + 1 >= m.n_windows;  // the last window of a lap
      // absent for sure (an empty slot, or the whole table seen): pick the slot to claim
      uint64_t target = none;
      long long expect = kEmptyKey;
      if (!done && !mb && (eb || lap)) {
        if (erased_slot != none) {
          target = erased_slot;
          expect = kErasedKey;
        } else if (eb) {
          target = w * kWindow + (unsigned)__ffs(eb) - 1u;
        }
      }
      longlong2 old = make_longlong2(0, 0);
      const bool try_claim = target != none && sub == 0;
      if (try_claim) old = cas_slot(m.slots + target, make_longlong2(expect, -1), make_longlong2(k, v));
      const unsigned okb = (__ballot_sync(full, try_claim && old.x == expect) >> (tile * 4)) & 0xFu;
      const unsigned sameb = (__ballot_sync(full, try_claim && old.x == k) >> (tile * 4)) & 0xFu;
      const int from = mb ? (int)(tile * 4 + __ffs(mb) - 1) : (int)(tile * 4);
      const int64_t exist = __shfl_sync(full, mb ? s.y : old.y, from);
      if (!done) {
        if (mb) {
          if (assign && (int)sub == __ffs(mb) - 1) p->val = v;
          res = assign ? v : exist;
          done = true;
        } else if (okb) {
          res = v;
          newly = true;
          done = true;
        } else if (sameb) {
          // another warp stored this very key into the slot a moment ago
          if (assign && sub == 0) m.slots[target].val = v;
          res = assign ? v : exist;
          done = true;
        } else if (target != none) {
          // the slot went to another key first: walk again from the home window
          w = home_window(m, k);
          steps = 0;
          erased_slot = none;
          if (++restarts > 16) {
            if (sub == 0)
              atomicMax(reinterpret_cast<unsigned long long*>(status_word),
                        (unsigned long long)DEV_OVERFLOW);
            done = true;
          }
        } else if (lap) {
          // a whole lap, no empty and no erased slot: the table is full
          if (sub == 0)
            atomicMax(reinterpret_cast<unsigned long long*>(status_word),
                      (unsigned long long)DEV_OVERFLOW);
          done = true;
        } else {
          w = w + 1 == m.n_windows ? 0 : w + 1;
          ++steps;
        }
      }
    }
    added += __popc(__ballot_sync(full, newly && sub == 0));
    const int64_t rv = __shfl_sync(full, res, (lane & 7) * 4);
    if ((int)(lane >> 3) == r) result = rv;
  }
  *n_new = added;
  return result;
}

#endif  // __CUDACC__

}  // namespace shmt
