// Single-pass prefix hand-off between CTAs (decoupled look-back, Merrill &
// Garland 2016), shared by the scan, the sampling hop and relabel.
//
// Every tile owns one 16-byte descriptor {value, state}, read and written as a single 128-bit
// access, so a reader always sees a value together with the state it belongs to.  Tile t
// publishes its local aggregate (state 1) as soon as it has it, then looks back over its
// predecessors 32 at a time, one load per predecessor, until it meets one whose inclusive prefix
// is known (state 2), and finally replaces its own descriptor by its inclusive prefix.
// Tiles take their index from an atomic ticket, so every predecessor of a running tile has
// already started: no wait depends on an unscheduled CTA.
// Every wait is bounded; a tile that gives up records DEV_TIMEOUT and carries on with what it
// has, so the kernel always terminates.
#pragma once

#include "common.cuh"

namespace shmt {

struct __align__(16) TileDesc {
  long long value;
  unsigned long long state;  // 0 = nothing yet, 1 = value is the aggregate, 2 = the inclusive prefix
};

struct TileStates {
  TileDesc* d;
};

// Bytes of look-back state for n_tiles tiles; they must be zero when the kernel starts.
constexpr size_t tile_state_bytes(int64_t n_tiles) { return (size_t)n_tiles * sizeof(TileDesc); }

inline TileStates carve_tile_states(char* base, int64_t /*n_tiles*/) {  // base: 16-byte aligned
  return TileStates{reinterpret_cast<TileDesc*>(base)};
}

#ifdef __CUDACC__

constexpr int kLookbackSpinLimit = 1 << 22;
constexpr unsigned long long kTileAggregate = 1, kTileInclusive = 2;

__device__ __forceinline__ void st_desc(TileDesc* p, long long value, unsigned long long state) {
  asm volatile(
      "{\n\t"
      ".reg .b128 t;\n\t"
      "mov.b128 t, {%1, %2};\n\t"
      "st.relaxed.gpu.global.b128 [%0], t;\n\t"
      "}" ::"l"(p), "l"(value), "l"(state)
      : "memory");
}

__device__ __forceinline__ void ld_desc(const TileDesc* p, long long* value, unsigned long long* state) {
  asm volatile(
      "{\n\t"
      ".reg .b128 t;\n\t"
      "ld.relaxed.gpu.global.b128 t, [%2];\n\t"
      "mov.b128 {%0, %1}, t;\n\t"
      "}"
      : "=l"(*value), "=l"(*state)
      : "l"(p)
      : "memory");
}

// Ticketed tile index for the calling CTA (call from every thread).
__device__ __forceinline__ int take_tile(int64_t* ticket, int* smem_slot) {
  if (threadIdx.x == 0) *smem_slot = (int)atomicAdd(reinterpret_cast<unsigned long long*>(ticket), 1ULL);
  __syncthreads();
  return *smem_slot;
}

// Exclusive prefix of `tile` given its aggregate.  Must be called by all 32
// lanes of ONE warp of the CTA; every lane gets the result.
__device__ __forceinline__ int64_t lookback_exclusive_prefix(const TileStates& st, int tile,
                                                             int64_t aggregate,
                                                             int64_t* status_word,
                                                             int spin_limit = kLookbackSpinLimit) {
  const unsigned lane = threadIdx.x & 31;
  if (tile == 0) {
    if (lane == 0) st_desc(st.d, aggregate, kTileInclusive);
    return 0;
  }
  if (lane == 0) st_desc(st.d + tile, aggregate, kTileAggregate);
  int64_t prefix = 0;
  int base = tile - 1;
  while (true) {
    const int t = base - (int)lane;
    unsigned long long f = kTileInclusive;
    long long v = 0;
    if (t >= 0) {
      int spins = 0;
      ld_desc(st.d + t, &v, &f);
      while (f == 0ULL && spins < spin_limit) {
        __nanosleep(20);
        ld_desc(st.d + t, &v, &f);
        ++spins;
      }
      if (f == 0ULL) {
        atomicMax(reinterpret_cast<unsigned long long*>(status_word),
                  (unsigned long long)DEV_TIMEOUT);
        f = kTileInclusive;  // give up: treat as a known (zero) prefix so the chain ends here
        v = 0;
      }
    }
    const unsigned known = __ballot_sync(0xffffffffu, f == kTileInclusive);
    // lanes at or before the nearest tile with a known inclusive prefix contribute
    const unsigned upto = known ? (unsigned)(__ffs(known) - 1) : 31u;
    int64_t part = lane <= upto ? (int64_t)v : 0;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) part += __shfl_xor_sync(0xffffffffu, part, o);
    prefix += part;
    if (known) break;
    base -= 32;
  }
  if (lane == 0) st_desc(st.d + tile, prefix + aggregate, kTileInclusive);
  return prefix;
}

// Look-back for a tile whose aggregate has ALREADY been published (state 1, or state 2 for tile
// 0) by an earlier step of the same kernel: returns the exclusive prefix and, if `publish`,
// replaces the descriptor by the inclusive prefix.  Several CTAs that computed one tile together
// (a thread-block cluster) may all call it and get the same prefix; one of them publishes.
// WINDOWS * 32 predecessors are read per step, all loads in flight together: when the sums are
// known to be out already, reading further back costs nothing in waiting and saves round trips
// through L2.  A waiting lane gives up as soon as another tile has recorded a timeout, so a kernel
// whose tile order was broken ends after one bounded wait instead of one per tile.
template <int WINDOWS>
__device__ __forceinline__ int64_t lookback_published(const TileStates& st, int tile, int64_t aggregate,
                                                      bool publish, int64_t* status_word,
                                                      int spin_limit = kLookbackSpinLimit) {
  const unsigned lane = threadIdx.x & 31;
  if (tile == 0) return 0;
  int64_t prefix = 0;
  int base = tile - 1;
  bool done = false;
  while (!done) {
    unsigned long long f[WINDOWS];
    long long v[WINDOWS];
#pragma unroll
    for (int j = 0; j < WINDOWS; ++j) {
      const int t = base - 32 * j - (int)lane;
      f[j] = kTileInclusive;  // before the first tile: a known prefix of zero
      v[j] = 0;
      if (t >= 0) ld_desc(st.d + t, &v[j], &f[j]);
    }
#pragma unroll
    for (int j = 0; j < WINDOWS; ++j) {
      if (done) break;
      const int t = base - 32 * j - (int)lane;
      int spins = 0;
      while (f[j] == 0ULL && spins < spin_limit) {
        __nanosleep(20);
        ld_desc(st.d + t, &v[j], &f[j]);
        if ((++spins & 1023) == 0 && ld_relaxed64(status_word) != DEV_OK) spins = spin_limit;
      }
      if (f[j] == 0ULL) {
        atomicMax(reinterpret_cast<unsigned long long*>(status_word),
                  (unsigned long long)DEV_TIMEOUT);
        f[j] = kTileInclusive;  // give up: treat as a known (zero) prefix so the chain ends here
        v[j] = 0;
      }
      const unsigned known = __ballot_sync(0xffffffffu, f[j] == kTileInclusive);
      // lanes at or before the nearest tile with a known inclusive prefix contribute
      const unsigned upto = known ? (unsigned)(__ffs(known) - 1) : 31u;
      int64_t part = lane <= upto ? (int64_t)v[j] : 0;
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) part += __shfl_xor_sync(0xffffffffu, part, o);
      prefix += part;
      done = known != 0;
    }
    base -= 32 * WINDOWS;
  }
  if (publish && lane == 0) st_desc(st.d + tile, prefix + aggregate, kTileInclusive);
  return prefix;
}

// Block-wide exclusive scan of one int64 per thread (blockDim.x <= 1024,
// multiple of 32).  `warp_sums` is 32 int64 of shared memory.  Returns the
// exclusive prefix of the caller; *total gets the block sum.
__device__ __forceinline__ int64_t block_exclusive_scan(int64_t v, int64_t* warp_sums,
                                                        int64_t* total) {
  const unsigned lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const unsigned n_warps = (blockDim.x + 31) >> 5;
  int64_t inc = v;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const int64_t up = __shfl_up_sync(0xffffffffu, inc, o);
    if (lane >= (unsigned)o) inc += up;
  }
  if (lane == 31) warp_sums[warp] = inc;
  __syncthreads();
  if (warp == 0) {
    int64_t w = lane < n_warps ? warp_sums[lane] : 0;
    int64_t winc = w;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int64_t up = __shfl_up_sync(0xffffffffu, winc, o);
      if (lane >= (unsigned)o) winc += up;
    }
    if (lane < n_warps) warp_sums[lane] = winc - w;  // exclusive prefix of each warp
    if (lane == 31) *total = winc;
  }
  __syncthreads();
  return warp_sums[warp] + inc - v;
}

#endif  // __CUDACC__

}  // namespace shmt
