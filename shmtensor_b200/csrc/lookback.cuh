// Single-pass prefix hand-off between CTAs (decoupled look-back, Merrill &
// Garland 2016), shared by the scan, the sampling hop and relabel.
//
// Tile t publishes its local aggregate (flag 1) as soon as it has it, then looks
// back over its predecessors 32 at a time until it meets one whose inclusive
// prefix is known (flag 2), and finally publishes its own inclusive prefix.
// Tiles take their index from an atomic ticket, so every predecessor of a
// running tile has already started: no wait depends on an unscheduled CTA.
// Every wait is bounded; a tile that gives up records DEV_TIMEOUT and carries on
// with what it has, so the kernel always terminates.
#pragma once

#include "common.cuh"

namespace shmt {

struct TileStates {
  uint32_t* flag;  // 0 = nothing yet, 1 = aggregate valid, 2 = inclusive valid
  int64_t* agg;
  int64_t* inc;
};

constexpr size_t tile_state_bytes(int64_t n_tiles) {
  // flags padded so the two int64 arrays stay 8-byte aligned
  return ((size_t)n_tiles * 4 + 7) / 8 * 8 + (size_t)n_tiles * 16;
}

inline TileStates carve_tile_states(char* base, int64_t n_tiles) {
  TileStates st;
  st.flag = reinterpret_cast<uint32_t*>(base);
  char* p = base + ((size_t)n_tiles * 4 + 7) / 8 * 8;
  st.agg = reinterpret_cast<int64_t*>(p);
  st.inc = st.agg + n_tiles;
  return st;
}

#ifdef __CUDACC__

constexpr int kLookbackSpinLimit = 1 << 22;

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
    if (lane == 0) {
      st_relaxed64(st.inc, aggregate);
      st_release(st.flag, 2u);
    }
    return 0;
  }
  if (lane == 0) {
    st_relaxed64(st.agg + tile, aggregate);
    st_release(st.flag + tile, 1u);
  }
  int64_t prefix = 0;
  int base = tile - 1;
  while (true) {
    const int t = base - (int)lane;
    uint32_t f = 2u;
    int64_t v = 0;
    if (t >= 0) {
      int spins = 0;
      f = ld_acquire(st.flag + t);
      while (f == 0u && spins < spin_limit) {
        __nanosleep(32);
        f = ld_acquire(st.flag + t);
        ++spins;
      }
      if (f == 0u) {
        atomicMax(reinterpret_cast<unsigned long long*>(status_word),
                  (unsigned long long)DEV_TIMEOUT);
        f = 2u;  // give up: treat as a known (zero) prefix so the chain ends here
      } else {
        v = ld_relaxed64((f == 2u ? st.inc : st.agg) + t);
      }
    }
    const unsigned known = __ballot_sync(0xffffffffu, f == 2u);
    // lanes at or before the nearest tile with a known inclusive prefix contribute
    const unsigned upto = known ? (unsigned)(__ffs(known) - 1) : 31u;
    int64_t part = lane <= upto ? v : 0;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) part += __shfl_xor_sync(0xffffffffu, part, o);
    prefix += part;
    if (known) break;
    base -= 32;
  }
  if (lane == 0) {
    st_relaxed64(st.inc + tile, prefix + aggregate);
    st_release(st.flag + tile, 2u);
  }
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
