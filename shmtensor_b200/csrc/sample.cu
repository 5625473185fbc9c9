// One fan-out hop of neighbour sampling over a (partly cached) CSR, as ONE kernel,
// and the sub-CSR builder that fills the cache.
//
// Reference: GetSubIndptr / GetSubIndptrWithCache + CUB scan + host read of nnz +
// CSRWise[Mask]SampleUniform[Replace]Kernel (src/cache_graph_sampling.cu:47-89,
// 222-289, 91-177, 291-380, 179-220, 382-426); CreateCacheCSR (:428-492).
//
// Here a CTA takes a tile of S seeds:
//   1. one seed per thread: cooperative map probe, row bounds from the cached
//      indptr (hit) or the host indptr over UVA (miss), picks = min(deg, k);
//   2. block scan of the picks, decoupled look-back for the tile's offset ->
//      sub_indptr, so no separate scan kernel and no host round trip;
//   3. groups of G = 8/16/32 lanes (smallest power of two >= k) sample one seed
//      each: deg <= k copies the row; otherwise each lane p < k draws
//      t_p ~ U[0, deg-k+p] with Philox4x32-10 and the group resolves Floyd's
//      subset algorithm with k shuffle+ballot steps (O(k) work, exact uniform
//      k-subset; the reference draws O(deg) numbers and uses global atomics).
//      k > 32: one warp per seed draws positions into a shared-memory set until k distinct
//      ones (or, for rows shorter than 2k, the deg-k to leave out) are held: O(k) draws, no
//      global atomics.  Only beyond 1024 picks per seed does it fall back to the reference's
//      reservoir on the output row.
#include "ctx.cuh"
#include "lookback.cuh"
#include "map.cuh"
#include "relabel.cuh"

namespace shmt {

constexpr int kHopThreads = 256;
constexpr int kMaxSeedsPerTile = 1024;

struct HopJob {
  const void* indptr;
  int indptr64;
  const void* indices;      // host / full graph
  const void* gpu_indptr;   // compact cached CSR (nullable)
  const void* gpu_indices;
  MapView map;
  const void* seeds;
  int seeds64;
  int64_t n;
  int64_t k;
  int replace;
  uint64_t rng_seed;
  uint32_t off_lo, off_hi;
  void* sub_indptr;
  void* sub_indices;
  TileStates st;
  int64_t* ticket;        // tile ticket counter (starts at 0)
  int64_t* status;        // device status word
  int64_t* result;        // receives nnz
  const int64_t* n_dev;   // if set, the seed count is read here (it was produced on the device)
  int seeds_per_tile;
  uint32_t set_slots;     // fan-out > 32: words of the per-warp set of chosen positions (0: none)
  // Edge ids (optional): for every sampled neighbour its position in the full `indices` array,
  // in the dtype of indptr.  A cached row's position there is gpu_edge_base[slot] + offset in row.
  void* out_eids;
  const void* gpu_edge_base;
  // Weighted sampling (optional): one positive float per edge, parallel to `indices` (and to
  // gpu_indices for the cached rows).  Always sampled by one warp per seed.
  const float* weights;
  const float* gpu_weights;
  // Fused relabel insert (multi-hop path): the kernel also claims a relabel-table slot for
  // every seed and every sampled neighbour, at its index in [seeds | neighbours], and
  // records the slot in rel_out -- the work of relabel's first kernel, done while this
  // kernel would otherwise wait on memory.  rel_slots == nullptr: off.
  RelSlot* rel_slots;
  uint32_t rel_mask;
  void* rel_out;
  // Single-hop call with a host result: the CTA that finishes its bookkeeping last hands the
  // result words to the host, which returns while the rows are still being written.
  HostPost post;
};

// indptr[i] and indptr[i+1] with one load when the pair is naturally aligned (one request on
// the host link instead of two for a row that lives in host memory).  Alignment is decided on
// the address of element i, so a view that starts at an odd element (indptr[1:], an .npy
// payload at an offset that is no multiple of 16) pairs its odd rows and never issues a
// misaligned vector load.
__device__ __forceinline__ void load_bounds(const void* indptr, int is64, int64_t i, int64_t* b,
                                            int64_t* e) {
  if (is64) {
    const long long* p = reinterpret_cast<const long long*>(indptr) + i;
    if ((reinterpret_cast<uintptr_t>(p) & 15) == 0) {
      const longlong2 v = __ldg(reinterpret_cast<const longlong2*>(p));
      *b = v.x;
      *e = v.y;
      return;
    }
  } else {
    const int* p = reinterpret_cast<const int*>(indptr) + i;
    if ((reinterpret_cast<uintptr_t>(p) & 7) == 0) {
      const int2 v = __ldg(reinterpret_cast<const int2*>(p));
      *b = v.x;
      *e = v.y;
      return;
    }
  }
  *b = load_int(indptr, is64, i);
  *e = load_int(indptr, is64, i + 1);
}

__device__ __forceinline__ uint64_t draw_below(const Philox& rng, uint32_t seed_idx, uint32_t draw,
                                               uint32_t off_lo, uint32_t off_hi, uint64_t range) {
  const uint4 r = rng(seed_idx, draw, off_lo, off_hi);
  return bounded(r.x, r.y, range);
}

template <typename IxT, int G>
__global__ void __launch_bounds__(kHopThreads) sample_hop_kernel(const HopJob job) {
  __shared__ int64_t s_begin[kMaxSeedsPerTile];
  __shared__ int64_t s_deg[kMaxSeedsPerTile];
  __shared__ int64_t s_off[kMaxSeedsPerTile];
  __shared__ uint8_t s_hit[kMaxSeedsPerTile];
  __shared__ int64_t s_eshift[kMaxSeedsPerTile];  // edge id = position read from + this (edge ids only)
  __shared__ int64_t warp_sums[32];
  __shared__ int64_t s_total;
  __shared__ int64_t s_prefix;
  __shared__ int s_tile;

  pdl_prologue();
  const unsigned full = 0xffffffffu;
  const unsigned tid = threadIdx.x, lane = tid & 31;
  const int S = job.seeds_per_tile;
  const int64_t n = job.n_dev ? *job.n_dev : job.n;
  const int64_t n_tiles = (n + S - 1) / S;
  const int tile = take_tile(job.ticket, &s_tile);
  if (tile >= n_tiles) {  // the grid is sized for the largest n the caller allows
    if (n == 0 && tile == 0 && tid == 0) {
      store_int(job.sub_indptr, job.indptr64, 0, 0);
      st_relaxed64(job.result, 0);
      post_to_host(job.post);
    }
    return;
  }
  const int64_t first = (int64_t)tile * S;
  const int rows = (int)min((int64_t)S, n - first);
  const int64_t k = job.k;

  // ---- 1. row bounds and pick counts, one seed per thread
  for (int j0 = (int)(tid & ~31u); j0 < S; j0 += kHopThreads) {
    const int j = j0 + (int)lane;
    const bool valid = j < rows;
    const int64_t row = valid ? load_int(job.seeds, job.seeds64, first + j) : kEmptyKey;
    int64_t slot = -1;
    if (job.map.slots) slot = warp_find(job.map, row, valid);
    int64_t b = 0, e = 0;
    if (valid) {
      if (slot >= 0)
        load_bounds(job.gpu_indptr, job.indptr64, slot, &b, &e);
      else
        load_bounds(job.indptr, job.indptr64, row, &b, &e);
    }
    const int64_t deg = e - b;
    if (job.out_eids && j < S)
      s_eshift[j] = (valid && slot >= 0) ? load_int(job.gpu_edge_base, job.indptr64, slot) - b : 0;
    if (j < S) {
      s_begin[j] = b;
      s_deg[j] = deg;
      s_hit[j] = slot >= 0;
      s_off[j] = !valid ? 0 : (job.replace ? (deg > 0 ? k : 0) : (deg < k ? deg : k));
    }
  }
  __syncthreads();

  constexpr int kGroups = kHopThreads / G;
  constexpr int U = 8;  // seeds per group; a tile never holds more than kGroups * U when k <= G
  const unsigned gl = tid & (G - 1);
  const unsigned gshift = lane & ~(unsigned)(G - 1);  // first lane of my group within the warp
  const unsigned gmask = G == 32 ? full : (((1u << G) - 1u) << gshift);
  const int group = (int)(tid / G);
  const Philox rng(job.rng_seed);
  IxT* out_all = static_cast<IxT*>(job.sub_indices);

  // ---- 2. (k <= G) pick positions and LOAD the neighbours now, before the tile's output
  // offset is known: the loads (often over the host link) then overlap the look-back wait
  // and the other tiles' row-bound reads.  One element per lane and seed; the U seeds of a
  // group are resolved first (arithmetic and shuffles only), then their loads go out back
  // to back.
  const IxT* src[U];
  IxT v[U];
  if (k <= G && !job.weights) {
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int j = u * kGroups + group;
      const bool active = j < rows;
      const int64_t deg = active ? s_deg[j] : 0;
      const uint32_t seed_idx = (uint32_t)(first + j);
      int64_t pos = -1;
      if (job.replace) {
        if (deg > 0 && (int64_t)gl < k)
          pos = (int64_t)draw_below(rng, seed_idx, gl, job.off_lo, job.off_hi, (uint64_t)deg);
      } else {
        if (active && deg <= k && (int64_t)gl < deg) pos = gl;
        const bool pick = active && deg > k;
        // Floyd: step p inserts t_p unless already chosen, then inserts deg-k+p instead
        if (__any_sync(full, pick)) {
          const int64_t top = deg - k + (int64_t)gl;  // largest position step gl may choose
          int64_t t = -1;
          if (pick && (int64_t)gl < k)
            t = (int64_t)draw_below(rng, seed_idx, gl, job.off_lo, job.off_hi, (uint64_t)top + 1);
          int64_t res = -1;
          for (int p = 0; p < (int)k; ++p) {
            const int64_t cand = __shfl_sync(full, t, p, G);
            const bool clash = pick && (int)gl < p && res == cand;
            const unsigned votes = __ballot_sync(full, clash) & gmask;
            if ((int)gl == p) res = votes ? top : cand;
          }
          if (pick && (int64_t)gl < k) pos = res;
        }
      }
      src[u] = nullptr;
      if (pos >= 0)
        src[u] = static_cast<const IxT*>(s_hit[j] ? job.gpu_indices : job.indices) + s_begin[j] + pos;
    }
#pragma unroll
    for (int u = 0; u < U; ++u)
      if (src[u]) v[u] = __ldg(src[u]);
  }

  // ---- 3. offsets: scan inside the tile, look-back across tiles
  {
    const int ch = (S + kHopThreads - 1) / kHopThreads;  // seeds per thread, 1..4
    int64_t c[kMaxSeedsPerTile / kHopThreads];
    int64_t sum = 0;
#pragma unroll
    for (int q = 0; q < kMaxSeedsPerTile / kHopThreads; ++q) {
      const int j = (int)tid * ch + q;
      c[q] = (q < ch && j < S) ? s_off[j] : 0;
      sum += c[q];
    }
    int64_t run = block_exclusive_scan(sum, warp_sums, &s_total);
    if (tid < 32) {
      const int64_t p = lookback_exclusive_prefix(job.st, tile, s_total, job.status);
      if (tid == 0) s_prefix = p;
    }
#pragma unroll
    for (int q = 0; q < kMaxSeedsPerTile / kHopThreads; ++q) {
      const int j = (int)tid * ch + q;
      if (q < ch && j < S) s_off[j] = run;
      run += c[q];
    }
    __syncthreads();
  }
  const int64_t prefix = s_prefix;
  const bool relabel = job.rel_slots != nullptr;
  // ids are hashed into as much of the table as n seeds with k picks each can need
  const uint32_t rel_mask = relabel ? relabel_mask_for(n * (1 + k), job.rel_mask) : 0u;
  for (int j = (int)tid; j < rows; j += kHopThreads) {
    store_int(job.sub_indptr, job.indptr64, first + j, prefix + s_off[j]);
    if (relabel) {
      const int64_t i = first + j;
      bool maybe_first;
      const uint32_t pos = relabel_insert_one(job.rel_slots, rel_mask,
                                              load_int(job.seeds, job.seeds64, i), (unsigned)i,
                                              job.status, &maybe_first);
      store_int(job.rel_out, sizeof(IxT) == 8, i, relabel_pack(pos, maybe_first, sizeof(IxT) == 8, job.rel_mask));
    }
  }
  if (tile == n_tiles - 1 && tid == 0) {
    store_int(job.sub_indptr, job.indptr64, n, prefix + s_total);
    st_relaxed64(job.result, prefix + s_total);
  }
  if (job.post.host) {  // uniform over the grid; the fused path (which may still flag the relabel table) never posts here
    __syncthreads();
    if (tid == 0) post_when_last(job.post, n_tiles);
  }

  // ---- 4. output
  if (k <= G && !job.weights) {
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int j = u * kGroups + group;
      if (src[u]) {
        const int64_t o = prefix + s_off[j] + gl;
        out_all[o] = v[u];
        if (job.out_eids)
          store_int(job.out_eids, job.indptr64, o,
                    (src[u] - static_cast<const IxT*>(s_hit[j] ? job.gpu_indices : job.indices)) + s_eshift[j]);
        if (relabel) {
          bool maybe_first;
          const uint32_t pos = relabel_insert_one(job.rel_slots, rel_mask, (long long)v[u],
                                                  (unsigned)(n + o), job.status, &maybe_first);
          store_int(job.rel_out, sizeof(IxT) == 8, n + o,
                    relabel_pack(pos, maybe_first, sizeof(IxT) == 8, job.rel_mask));
        }
      }
    }
    return;
  }

  // k > 32 (G == 32): one warp per seed
  extern __shared__ uint32_t s_sets[];  // per warp: a set of chosen positions (job.set_slots words)
  const uint32_t set_slots = job.set_slots;
  uint32_t* set = s_sets + (size_t)(tid >> 5) * set_slots;
  for (int j0 = 0; j0 < rows; j0 += kGroups) {
    const int j = j0 + group;
    const bool active = j < rows;
    const int64_t deg = active ? s_deg[j] : 0;
    const IxT* in = nullptr;
    int64_t out_at = 0;
    if (active) {
      in = static_cast<const IxT*>(s_hit[j] ? job.gpu_indices : job.indices) + s_begin[j];
      out_at = prefix + s_off[j];
    }
    const uint32_t seed_idx = (uint32_t)(first + j);
    // one output element: the neighbour at `pos` of the row goes to slot `o` of the output
    auto emit = [&](int64_t o, int64_t pos) {
      const IxT val = __ldg(in + pos);
      out_all[o] = val;
      if (job.out_eids) store_int(job.out_eids, job.indptr64, o, s_begin[j] + pos + s_eshift[j]);
      if (relabel) {
        bool maybe_first;
        const uint32_t slot = relabel_insert_one(job.rel_slots, rel_mask, (long long)val,
                                                 (unsigned)(n + o), job.status, &maybe_first);
        store_int(job.rel_out, sizeof(IxT) == 8, n + o,
                  relabel_pack(slot, maybe_first, sizeof(IxT) == 8, job.rel_mask));
      }
    };
    if (job.weights && deg > 0 && (job.replace || deg > k)) {
      const float* w = (s_hit[j] ? job.gpu_weights : job.weights) + s_begin[j];
      const float tiny = 1.17549435e-38f;  // a weight that is not positive counts as the smallest one
      if (!job.replace) {
        // Efraimidis-Spirakis: every edge gets the key -log(u) / w (an exponential clock of rate
        // w) and the k smallest keys win, which is sampling without replacement with
        // probabilities proportional to the weights.  Lanes 0..k-1 hold the k smallest keys seen
        // so far, ascending; a key below the largest of them is inserted by one shuffle step.
        float best = __int_as_float(0x7f800000);
        int64_t bpos = -1;
        float thr = best;
        for (int64_t p0 = 0; p0 < deg; p0 += 32) {
          const int64_t pos = p0 + gl;
          float key = __int_as_float(0x7f800000);
          if (pos < deg) {
            const uint4 r = rng(seed_idx, (uint32_t)pos, job.off_lo, job.off_hi);
            const float u = ((float)(r.x >> 8) + 1.0f) * (1.0f / 16777216.0f);  // (0, 1]
            key = -__logf(u) / fmaxf(__ldg(w + pos), tiny);
          }
          unsigned cand = __ballot_sync(full, key < thr);
          while (cand) {
            const int from = __ffs(cand) - 1;
            cand &= cand - 1;
            const float ck = __shfl_sync(full, key, from);
            const int64_t cp = __shfl_sync(full, pos, from);
            if (ck < thr) {  // the bound may have dropped since the vote; same on every lane
              const float left_k = __shfl_up_sync(full, best, 1);
              const int64_t left_p = __shfl_up_sync(full, bpos, 1);
              if ((int64_t)gl < k && ck < best) {
                if (gl == 0 || left_k <= ck) {
                  best = ck;
                  bpos = cp;
                } else {
                  best = left_k;
                  bpos = left_p;
                }
              }
              thr = __shfl_sync(full, best, (int)k - 1);
            }
          }
        }
        if ((int64_t)gl < k) emit(out_at + gl, bpos);
      } else {
        // k independent draws proportional to the weights: the row's total, then for 32 draws at
        // a time a second walk that finds where each draw's share of the total falls
        double sum = 0.0;
        for (int64_t p = gl; p < deg; p += 32) sum += (double)fmaxf(__ldg(w + p), tiny);
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(full, sum, o);
        for (int64_t d0 = 0; d0 < k; d0 += 32) {
          const bool mine = d0 + gl < k;
          const uint4 r = rng(seed_idx, (uint32_t)(d0 + gl), job.off_lo, job.off_hi);
          const double target = ((double)r.x + 0.5) * (1.0 / 4294967296.0) * sum;
          int64_t found = -1;
          double base = 0.0;
          for (int64_t p0 = 0; p0 < deg; p0 += 32) {
            const int64_t pos = p0 + gl;
            double inc = pos < deg ? (double)fmaxf(__ldg(w + pos), tiny) : 0.0;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
              const double up = __shfl_up_sync(full, inc, o);
              if (gl >= (unsigned)o) inc += up;
            }
            const double chunk_end = base + __shfl_sync(full, inc, 31);
            const bool here = mine && found < 0 && target < chunk_end;
            if (__any_sync(full, here)) {
              for (int q = 0; q < 32; ++q) {
                const double upto = base + __shfl_sync(full, inc, q);
                if (here && found < 0 && target < upto && p0 + q < deg) found = p0 + q;
              }
            }
            base = chunk_end;
          }
          if (mine) emit(out_at + d0 + gl, found >= 0 ? found : deg - 1);
        }
      }
      continue;
    }
    if (job.replace) {
      if (deg > 0)
        for (int64_t p = gl; p < k; p += 32)
          emit(out_at + p, (int64_t)draw_below(rng, seed_idx, (uint32_t)p, job.off_lo, job.off_hi, (uint64_t)deg));
      continue;
    }
    if (deg <= k) {
      for (int64_t p = gl; p < deg; p += 32) emit(out_at + p, p);
      continue;
    }
    if (set_slots == 0 || deg >= 0xFFFFFFFFll) {
      // fan-outs beyond the shared-memory set (or rows of 2^32 neighbours): the reservoir on the
      // output row, O(deg) draws (src/cache_graph_sampling.cu:329-345)
      IxT* out = out_all + out_at;
      for (int64_t p = gl; p < k; p += 32) out[p] = (IxT)p;
      __syncwarp();
      for (int64_t q = k + gl; q < deg; q += 32) {
        const uint64_t r = draw_below(rng, seed_idx, (uint32_t)q, job.off_lo, job.off_hi, (uint64_t)q + 1);
        if (r < (uint64_t)k) atomicMax(out + r, (IxT)q);
      }
      __syncwarp();
      __threadfence_block();
      for (int64_t p = gl; p < k; p += 32) {
        const IxT pos = *reinterpret_cast<volatile IxT*>(out + p);
        emit(out_at + p, (int64_t)pos);
      }
      continue;
    }
    // A uniform k-subset in O(k) draws, all in shared memory: positions are drawn independently
    // and kept if new, until m distinct ones are held (any rule that treats all positions alike
    // yields every subset with the same probability).  m = k when the row is at least twice the
    // fan-out; otherwise the deg - k positions to LEAVE OUT are drawn, so at most half of the
    // draws are ever rejected.  The set is an open-addressing table of 2^x >= 2k words per warp.
    const bool complement = deg < 2 * k;
    const uint32_t m = (uint32_t)(complement ? deg - k : k);
    const uint32_t smask = set_slots - 1;
    for (uint32_t q = gl; q < set_slots; q += 32) set[q] = 0xFFFFFFFFu;
    __syncwarp();
    uint32_t held = 0, draws = 0;
    // a draw is rejected with probability below 1/2, so a few rounds suffice; the cap only makes
    // the loop provably finite
    for (int round = 0; held < m && round < 256 + (int)(m >> 2); ++round) {
      const bool mine = held + gl < m;
      bool kept = false;
      if (mine) {
        const uint32_t pos = (uint32_t)draw_below(rng, seed_idx, draws + gl, job.off_lo, job.off_hi, (uint64_t)deg);
        uint32_t at = (pos * 0x9E3779B1u) & smask;
        while (true) {
          const uint32_t old = atomicCAS(set + at, 0xFFFFFFFFu, pos);
          if (old == 0xFFFFFFFFu) { kept = true; break; }
          if (old == pos) break;
          at = (at + 1) & smask;
        }
      }
      held += (uint32_t)__popc(__ballot_sync(full, kept));
      draws += 32;
    }
    __syncwarp();
    if (held < m && gl == 0) {
      // never reached in practice: complete the set with the lowest positions not in it
      for (uint32_t pos = 0; held < m && pos < (uint32_t)deg; ++pos) {
        uint32_t at = (pos * 0x9E3779B1u) & smask;
        while (set[at] != 0xFFFFFFFFu && set[at] != pos) at = (at + 1) & smask;
        if (set[at] == 0xFFFFFFFFu) {
          set[at] = pos;
          ++held;
        }
      }
    }
    __syncwarp();
    if (!complement) {
      // the chosen positions, in table order
      uint32_t done = 0;
      for (uint32_t q0 = 0; q0 < set_slots; q0 += 32) {
        const uint32_t pos = set[q0 + gl];
        const unsigned has = __ballot_sync(full, pos != 0xFFFFFFFFu);
        if (pos != 0xFFFFFFFFu) emit(out_at + done + __popc(has & ((1u << gl) - 1u)), (int64_t)pos);
        done += (uint32_t)__popc(has);
      }
    } else {
      // every position that was not drawn, in row order
      uint32_t done = 0;
      for (int64_t p0 = 0; p0 < deg; p0 += 32) {
        const int64_t pos = p0 + gl;
        bool keep = pos < deg;
        if (keep) {
          uint32_t at = ((uint32_t)pos * 0x9E3779B1u) & smask;
          while (true) {
            const uint32_t cur = set[at];
            if (cur == 0xFFFFFFFFu) break;
            if (cur == (uint32_t)pos) { keep = false; break; }
            at = (at + 1) & smask;
          }
        }
        const unsigned has = __ballot_sync(full, keep);
        if (keep) emit(out_at + done + __popc(has & ((1u << gl) - 1u)), pos);
        done += (uint32_t)__popc(has);
      }
    }
    __syncwarp();  // the set is cleared for the next seed only after every lane has read it
  }
}

// ---- sub-CSR ------------------------------------------------------------------

__global__ void subcsr_degree_kernel(const void* __restrict__ indptr, int indptr64,
                                     const void* __restrict__ seeds, int seeds64, int64_t n,
                                     void* __restrict__ out) {
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i <= n; i += stride) {
    int64_t d = 0;
    if (i < n) {
      const int64_t row = load_int(seeds, seeds64, i);
      d = load_int(indptr, indptr64, row + 1) - load_int(indptr, indptr64, row);
    }
    store_int(out, indptr64, i, d);
  }
}

// out[i] = indptr[seeds[i]]: where each selected row starts in the full edge array.
__global__ void subcsr_edge_base_kernel(const void* __restrict__ indptr, int indptr64,
                                        const void* __restrict__ seeds, int seeds64, int64_t n,
                                        void* __restrict__ out) {
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride)
    store_int(out, indptr64, i, load_int(indptr, indptr64, load_int(seeds, seeds64, i)));
}

template <typename IxT>
__global__ void __launch_bounds__(256)
subcsr_fill_kernel(const void* __restrict__ indptr, int indptr64, const IxT* __restrict__ indices,
                   const void* __restrict__ seeds, int seeds64, int64_t n,
                   const void* __restrict__ gpu_indptr, IxT* __restrict__ out) {
  const int64_t warp = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int64_t n_warps = ((int64_t)gridDim.x * blockDim.x) >> 5;
  const unsigned lane = threadIdx.x & 31;
  for (int64_t i = warp; i < n; i += n_warps) {
    const int64_t row = load_int(seeds, seeds64, i);
    const int64_t b = load_int(indptr, indptr64, row);
    const int64_t deg = load_int(indptr, indptr64, row + 1) - b;
    const IxT* src = indices + b;
    IxT* dst = out + load_int(gpu_indptr, indptr64, i);
    int64_t p = lane;
    for (; p + 96 < deg; p += 128) {  // four independent loads per lane in flight
      const IxT a0 = src[p], a1 = src[p + 32], a2 = src[p + 64], a3 = src[p + 96];
      dst[p] = a0;
      dst[p + 32] = a1;
      dst[p + 64] = a2;
      dst[p + 96] = a3;
    }
    for (; p < deg; p += 32) dst[p] = src[p];
  }
}

int launch_scan(shmt_ctx* ctx, void* data, int dtype, int64_t n, int exclusive,
                size_t scratch_off, cudaStream_t stream);
size_t scan_scratch_bytes(int64_t n);

static int pick_seeds_per_tile(int64_t n, int64_t k) {
  int64_t s = (n + (int64_t)sm_count() * 4 - 1) / ((int64_t)sm_count() * 4);
  s = (s + 31) / 32 * 32;
  if (s < 32) s = 32;
  if (s > kMaxSeedsPerTile) s = kMaxSeedsPerTile;
  // with k <= 32 a tile is sampled in one pass of 8 seeds per lane group (see the kernel)
  const int64_t one_pass = k <= 8 ? 256 : (k <= 16 ? 128 : (k <= 32 ? 64 : kMaxSeedsPerTile));
  if (s > one_pass) s = one_pass;
  return (int)s;
}

// Fan-outs above 32 keep a set of chosen positions per warp in shared memory: the smallest
// power of two >= 2k words, for k <= 1024 (64 KB per CTA at most).  0: the fan-out needs none,
// or is too large for it.
constexpr int64_t kMaxSetPicks = 1024;
static uint32_t set_slots_for(int64_t k) {
  if (k <= 32 || k > kMaxSetPicks) return 0;
  uint32_t slots = 128;
  while ((int64_t)slots < 2 * k) slots <<= 1;
  return slots;
}

template <typename IxT>
static cudaError_t launch_hop(HopJob job, int64_t n_tiles, cudaStream_t s, bool pdl = false) {
  const unsigned grid = (unsigned)n_tiles;
  job.set_slots = set_slots_for(job.k);
  if (!job.weights) {
    if (job.k <= 8) return launch_kernel(pdl, sample_hop_kernel<IxT, 8>, grid, kHopThreads, 0, s, job);
    if (job.k <= 16) return launch_kernel(pdl, sample_hop_kernel<IxT, 16>, grid, kHopThreads, 0, s, job);
  }
  const size_t smem = (size_t)job.set_slots * sizeof(uint32_t) * (kHopThreads / 32);
  if (smem > 0) {
    static bool configured[64] = {false};
    int dev = 0;
    if (cudaGetDevice(&dev) == cudaSuccess && dev >= 0 && dev < 64 && !configured[dev]) {
      const cudaError_t e = cudaFuncSetAttribute(sample_hop_kernel<IxT, 32>,
                                                 cudaFuncAttributeMaxDynamicSharedMemorySize,
                                                 (int)(2 * kMaxSetPicks * sizeof(uint32_t) * (kHopThreads / 32)));
      if (e != cudaSuccess) return e;
      configured[dev] = true;
    }
  }
  return launch_kernel(pdl, sample_hop_kernel<IxT, 32>, grid, kHopThreads, smem, s, job);
}

// Scratch layout of a multi-hop mini-batch, from its worst-case sizes (c_0 = n_seeds,
// c_{h+1} = c_h * (1 + fanouts[h])).
constexpr int kMaxHops = 8;
struct MinibatchPlan {
  int64_t cap[kMaxHops + 1], hop_tiles[kMaxHops], rel_tiles[kMaxHops];
  int spt[kMaxHops];
  size_t off_hop[kMaxHops], off_rel[kMaxHops];
  size_t scratch_bytes;
};

static int plan_minibatch(int64_t n_seeds, const int64_t* fanouts, int n_hops, MinibatchPlan* p,
                          bool weighted = false) {
  SHMT_REQUIRE(n_hops >= 1 && n_hops <= kMaxHops, "mini-batch: 1..%d hops", kMaxHops);
  SHMT_REQUIRE(n_seeds >= 1 && n_seeds < ((int64_t)1 << 31), "mini-batch: seed count out of range");
  SHMT_REQUIRE(fanouts != nullptr, "mini-batch: fanouts is null");
  p->cap[0] = n_seeds;
  size_t cursor = ((size_t)(n_hops * 8 + 8) * 8 + 255) & ~(size_t)255;
  for (int h = 0; h < n_hops; ++h) {
    SHMT_REQUIRE(fanouts[h] >= 1 && fanouts[h] < ((int64_t)1 << 20), "mini-batch: fan-out out of range");
    p->cap[h + 1] = p->cap[h] * (1 + fanouts[h]);
    SHMT_REQUIRE(p->cap[h + 1] < ((int64_t)1 << 30), "mini-batch: worst-case frontier too large");
    p->spt[h] = pick_seeds_per_tile(p->cap[h], weighted ? 33 : fanouts[h]);  // weighted: warp-per-seed layout
    p->hop_tiles[h] = (p->cap[h] + p->spt[h] - 1) / p->spt[h];
    p->rel_tiles[h] = (p->cap[h + 1] + kRelTile - 1) / kRelTile;
    p->off_hop[h] = cursor;
    cursor += (tile_state_bytes(p->hop_tiles[h]) + 255) & ~(size_t)255;
    p->off_rel[h] = cursor;
    cursor += (tile_state_bytes(p->rel_tiles[h]) + 255) & ~(size_t)255;
  }
  p->scratch_bytes = cursor;
  return SHMT_OK;
}

}  // namespace shmt

using namespace shmt;

extern "C" {

int shmt_ctx_reserve_minibatch(shmt_ctx* ctx, int64_t n_seeds, const int64_t* fanouts, int n_hops,
                               void* stream) {
  SHMT_REQUIRE(ctx != nullptr, "shmt_ctx_reserve_minibatch: ctx is null");
  MinibatchPlan plan;
  if (int rc = plan_minibatch(n_seeds, fanouts, n_hops, &plan)) return rc;
  DeviceGuard guard(ctx->device);
  if (int rc = ctx_reserve(ctx, plan.scratch_bytes)) return rc;
  RelTable t;
  return relabel_table(ctx, plan.cap[n_hops], &t, static_cast<cudaStream_t>(stream));
}

static int sample_hop_impl(shmt_ctx* ctx, const void* indptr, int indptr_dtype, const void* indices,
                           int indices_dtype, const void* gpu_indptr, const void* gpu_indices,
                           const shmt_map* map, const void* seeds, int seeds_dtype, int64_t n, int64_t k,
                           int replace, uint64_t rng_seed, uint64_t rng_offset, void* out_sub_indptr,
                           void* out_sub_indices, int64_t* nnz_host, void* stream, void* out_eids,
                           const void* gpu_edge_base, const float* weights = nullptr,
                           const float* gpu_weights = nullptr) {
  SHMT_REQUIRE(ctx != nullptr, "shmt_sample_hop: ctx is null");
  SHMT_REQUIRE(valid_int_dtype(indptr_dtype) && valid_int_dtype(indices_dtype) &&
                   valid_int_dtype(seeds_dtype),
               "shmt_sample_hop: ID can only be int32 or int64");
  SHMT_REQUIRE(n >= 0 && n < ((int64_t)1 << 31), "shmt_sample_hop: seed count out of range");
  SHMT_REQUIRE(k >= 0 && k < ((int64_t)1 << 31), "shmt_sample_hop: num_picks out of range");
  SHMT_REQUIRE(out_sub_indptr != nullptr, "shmt_sample_hop: out_sub_indptr is null");
  SHMT_REQUIRE(indptr != nullptr && (indices != nullptr || k == 0), "shmt_sample_hop: CSR is null");
  SHMT_REQUIRE(n == 0 || seeds != nullptr, "shmt_sample_hop: seeds are null");
  SHMT_REQUIRE(map == nullptr || (gpu_indptr != nullptr && gpu_indices != nullptr),
               "shmt_sample_hop: a map needs gpu_indptr and gpu_indices");
  SHMT_REQUIRE(n == 0 || k == 0 || out_sub_indices != nullptr,
               "shmt_sample_hop: out_sub_indices is null");
  DeviceGuard guard(ctx->device);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (n == 0) {
    SHMT_CUDA_TRY(cudaMemsetAsync(out_sub_indptr, 0, int_itemsize(indptr_dtype), s));
    if (nnz_host) {
      SHMT_CUDA_TRY(cudaStreamSynchronize(s));
      *nnz_host = 0;
    }
    return SHMT_OK;
  }
  HopJob job{};
  job.indptr = indptr;
  job.indptr64 = indptr_dtype == SHMT_I64;
  job.indices = indices;
  job.gpu_indptr = gpu_indptr;
  job.gpu_indices = gpu_indices;
  job.map = view_of(map);
  job.seeds = seeds;
  job.seeds64 = seeds_dtype == SHMT_I64;
  job.n = n;
  job.k = k;
  job.replace = replace != 0;
  job.rng_seed = rng_seed;
  job.off_lo = (uint32_t)rng_offset;
  job.off_hi = (uint32_t)(rng_offset >> 32);
  job.sub_indptr = out_sub_indptr;
  job.sub_indices = out_sub_indices;
  job.out_eids = out_eids;
  job.gpu_edge_base = gpu_edge_base;
  job.weights = weights;
  job.gpu_weights = gpu_weights;
  job.seeds_per_tile = pick_seeds_per_tile(n, weights ? 33 : k);  // weighted: the warp-per-seed layout
  const int64_t n_tiles = (n + job.seeds_per_tile - 1) / job.seeds_per_tile;
  if (int rc = ctx_reserve(ctx, tile_state_bytes(n_tiles))) return rc;
  job.st = carve_tile_states(ctx->region(), n_tiles);
  job.ticket = ctx->d_words() + W_TICKET;
  job.status = ctx->d_words() + W_STATUS;
  job.result = ctx->d_words() + W_RESULT;
  job.n_dev = nullptr;
  if (nnz_host) job.post = ctx_begin_post(ctx, ctx->d_words(), 4, ctx->d_words() + W_DONE);
  SHMT_CUDA_TRY(cudaMemsetAsync(ctx->scratch, 0, 256 + tile_state_bytes(n_tiles), s));
  SHMT_CUDA_TRY(indices_dtype == SHMT_I64 ? launch_hop<long long>(job, n_tiles, s)
                                          : launch_hop<int>(job, n_tiles, s));
  SHMT_CUDA_TRY(cudaGetLastError());
  if (nnz_host) {
    if (int rc = ctx_mark_tail(ctx, s)) return rc;
    if (int rc = ctx_await_post(ctx, job.post, s)) return rc;
    if (int rc = ctx_status_of_words(ctx, "shmt_sample_hop")) return rc;
    *nnz_host = ctx->h_words[W_RESULT];
  }
  return SHMT_OK;
}

int shmt_sample_hop(shmt_ctx* ctx, const void* indptr, int indptr_dtype, const void* indices,
                    int indices_dtype, const void* gpu_indptr, const void* gpu_indices,
                    const shmt_map* map, const void* seeds, int seeds_dtype, int64_t n, int64_t k,
                    int replace, uint64_t rng_seed, uint64_t rng_offset, void* out_sub_indptr,
                    void* out_sub_indices, int64_t* nnz_host, void* stream) {
  return sample_hop_impl(ctx, indptr, indptr_dtype, indices, indices_dtype, gpu_indptr, gpu_indices, map,
                         seeds, seeds_dtype, n, k, replace, rng_seed, rng_offset, out_sub_indptr,
                         out_sub_indices, nnz_host, stream, nullptr, nullptr);
}

int shmt_sample_hop_weighted(shmt_ctx* ctx, const void* indptr, int indptr_dtype, const void* indices,
                             int indices_dtype, const float* weights, const void* gpu_indptr,
                             const void* gpu_indices, const float* gpu_weights,
                             const void* gpu_edge_base, const shmt_map* map, const void* seeds,
                             int seeds_dtype, int64_t n, int64_t k, int replace, uint64_t rng_seed,
                             uint64_t rng_offset, void* out_sub_indptr, void* out_sub_indices,
                             void* out_edge_ids, int64_t* nnz_host, void* stream) {
  SHMT_REQUIRE(weights != nullptr || n == 0 || k == 0, "shmt_sample_hop_weighted: weights are null");
  SHMT_REQUIRE(replace || k <= 32,
               "shmt_sample_hop_weighted: without replacement the fan-out is limited to 32 (got %lld)",
               (long long)k);
  SHMT_REQUIRE(map == nullptr || gpu_weights != nullptr,
               "shmt_sample_hop_weighted: a cached graph needs gpu_weights");
  SHMT_REQUIRE(map == nullptr || out_edge_ids == nullptr || gpu_edge_base != nullptr,
               "shmt_sample_hop_weighted: edge ids of a cached graph need gpu_edge_base");
  return sample_hop_impl(ctx, indptr, indptr_dtype, indices, indices_dtype, gpu_indptr, gpu_indices, map,
                         seeds, seeds_dtype, n, k, replace, rng_seed, rng_offset, out_sub_indptr,
                         out_sub_indices, nnz_host, stream, out_edge_ids, gpu_edge_base, weights,
                         gpu_weights);
}

int shmt_sample_hop_eids(shmt_ctx* ctx, const void* indptr, int indptr_dtype, const void* indices,
                         int indices_dtype, const void* gpu_indptr, const void* gpu_indices,
                         const void* gpu_edge_base, const shmt_map* map, const void* seeds,
                         int seeds_dtype, int64_t n, int64_t k, int replace, uint64_t rng_seed,
                         uint64_t rng_offset, void* out_sub_indptr, void* out_sub_indices,
                         void* out_edge_ids, int64_t* nnz_host, void* stream) {
  SHMT_REQUIRE(n == 0 || k == 0 || out_edge_ids != nullptr, "shmt_sample_hop_eids: out_edge_ids is null");
  SHMT_REQUIRE(map == nullptr || gpu_edge_base != nullptr,
               "shmt_sample_hop_eids: a cached graph needs gpu_edge_base (shmt_subcsr_edge_base)");
  return sample_hop_impl(ctx, indptr, indptr_dtype, indices, indices_dtype, gpu_indptr, gpu_indices, map,
                         seeds, seeds_dtype, n, k, replace, rng_seed, rng_offset, out_sub_indptr,
                         out_sub_indices, nnz_host, stream, out_edge_ids, gpu_edge_base);
}

// Multi-hop mini-batch: every hop's sampling kernel and relabel kernels are queued back
// to back; each reads the size of its input from the device word the previous stage
// wrote, with grids sized for the largest frontier the fan-outs allow.  The host waits
// once, at the end, for all the sizes.
static int sample_minibatch_impl(shmt_ctx* ctx, const void* indptr, int indptr_dtype, const void* indices,
                                 int indices_dtype, const void* gpu_indptr, const void* gpu_indices,
                                 const shmt_map* map, const void* seeds, int64_t n_seeds,
                                 const int64_t* fanouts, int n_hops, int replace, uint64_t rng_seed,
                                 uint64_t rng_offset, void* const* out_sub_indptr,
                                 void* const* out_sub_indices, void* const* out_relabel,
                                 void* const* out_frontier, int64_t* sizes_host, void* stream,
                                 const void* gpu_edge_base, void* const* out_edge_ids,
                                 const float* weights = nullptr, const float* gpu_weights = nullptr) {
  SHMT_REQUIRE(ctx != nullptr, "shmt_sample_minibatch: ctx is null");
  SHMT_REQUIRE(valid_int_dtype(indptr_dtype) && valid_int_dtype(indices_dtype),
               "shmt_sample_minibatch: ID can only be int32 or int64");
  SHMT_REQUIRE(n_hops >= 1 && n_hops <= kMaxHops, "shmt_sample_minibatch: 1..%d hops", kMaxHops);
  SHMT_REQUIRE(n_seeds >= 1 && n_seeds < ((int64_t)1 << 31), "shmt_sample_minibatch: seed count out of range");
  SHMT_REQUIRE(indptr && indices && seeds && fanouts && out_sub_indptr && out_sub_indices &&
                   out_relabel && out_frontier && sizes_host,
               "shmt_sample_minibatch: null argument");
  SHMT_REQUIRE(map == nullptr || (gpu_indptr != nullptr && gpu_indices != nullptr),
               "shmt_sample_minibatch: a map needs gpu_indptr and gpu_indices");
  DeviceGuard guard(ctx->device);
  cudaStream_t s = static_cast<cudaStream_t>(stream);

  // worst-case frontier sizes and the scratch plan: [words][per hop: sample tiles | relabel tiles]
  MinibatchPlan plan;
  if (int rc = plan_minibatch(n_seeds, fanouts, n_hops, &plan, weights != nullptr)) return rc;
  for (int h = 0; h < n_hops; ++h)
    SHMT_REQUIRE(out_sub_indptr[h] && out_sub_indices[h] && out_relabel[h] && out_frontier[h],
                 "shmt_sample_minibatch: output buffer of hop %d is null", h);
  const int64_t* cap = plan.cap;
  const int64_t *hop_tiles = plan.hop_tiles, *rel_tiles = plan.rel_tiles;
  const int* spt = plan.spt;
  const size_t *off_hop = plan.off_hop, *off_rel = plan.off_rel;
  const size_t cursor = plan.scratch_bytes;
  if (int rc = ctx_reserve(ctx, cursor)) return rc;
  char* base = ctx->region();
  int64_t* words = reinterpret_cast<int64_t*>(base);
  SHMT_CUDA_TRY(cudaMemsetAsync(base, 0, cursor, s));  // words, tickets and every tile descriptor
  int64_t* status = words + n_hops * 8;

  {  // the relabel table for the largest hop, reserved before anything is queued
    RelTable biggest;
    if (int rc = relabel_table(ctx, cap[n_hops], &biggest, s)) return rc;
  }
  const void* cur_seeds = seeds;
  HostPost post{};
  for (int h = 0; h < n_hops; ++h) {
    int64_t* w = words + h * 8;  // [0] hop ticket, [1] nnz, [2] relabel ticket, [3] n_unique, [4] CTAs done
    HopJob job{};
    job.indptr = indptr;
    job.indptr64 = indptr_dtype == SHMT_I64;
    job.indices = indices;
    job.gpu_indptr = gpu_indptr;
    job.gpu_indices = gpu_indices;
    job.map = view_of(map);
    job.seeds = cur_seeds;
    job.seeds64 = indices_dtype == SHMT_I64;
    job.n = h == 0 ? n_seeds : 0;
    job.n_dev = h == 0 ? nullptr : words + (h - 1) * 8 + 3;
    job.k = fanouts[h];
    job.replace = replace != 0;
    job.rng_seed = rng_seed;
    job.off_lo = (uint32_t)(rng_offset + h);
    job.off_hi = (uint32_t)((rng_offset + h) >> 32);
    job.sub_indptr = out_sub_indptr[h];
    job.sub_indices = out_sub_indices[h];
    job.seeds_per_tile = spt[h];
    job.out_eids = out_edge_ids ? out_edge_ids[h] : nullptr;
    job.gpu_edge_base = gpu_edge_base;
    job.weights = weights;
    job.gpu_weights = gpu_weights;
    job.st = carve_tile_states(base + off_hop[h], hop_tiles[h]);
    job.ticket = w + 0;
    job.status = status;
    job.result = w + 1;
    const bool fuse_insert = true;  // every sampler claims the relabel slots of what it emits
    if (fuse_insert) {
      RelTable t;
      if (int rc = relabel_table(ctx, cap[h + 1], &t, s)) return rc;
      job.rel_slots = t.slots;
      job.rel_mask = t.mask;
      job.rel_out = out_relabel[h];
    }
    SHMT_CUDA_TRY(indices_dtype == SHMT_I64 ? launch_hop<long long>(job, hop_tiles[h], s, /*pdl=*/h > 0)
                                            : launch_hop<int>(job, hop_tiles[h], s, /*pdl=*/h > 0));
    SHMT_CUDA_TRY(cudaGetLastError());

    Parts ps{};
    ps.n = 2;
    ps.is64 = indices_dtype == SHMT_I64;
    ps.ptr[0] = cur_seeds;
    ps.ptr[1] = out_sub_indices[h];
    ps.start[1] = n_seeds;  // used for hop 0 only, whose seed count the host knows
    ps.dev_n0 = h == 0 ? nullptr : words + (h - 1) * 8 + 3;
    ps.dev_n1 = w + 1;
    // every size and the status word are final once the last hop's ids are counted: that kernel
    // hands them to the host, which returns while the last remap kernel is still running
    if (h == n_hops - 1) post = ctx_begin_post(ctx, words, n_hops * 8 + 8, w + 4);
    if (int rc = launch_relabel(ctx, ps, cap[h + 1], out_frontier[h], out_relabel[h],
                                carve_tile_states(base + off_rel[h], rel_tiles[h]), w + 2, status,
                                w + 3, s, fuse_insert, /*pdl=*/true, h == n_hops - 1 ? &post : nullptr))
      return rc;
    cur_seeds = out_frontier[h];
  }
  if (int rc = ctx_mark_tail(ctx, s)) return rc;
  if (int rc = ctx_await_post(ctx, post, s)) return rc;
  const int64_t st = ctx->h_words[n_hops * 8];
  if (st != DEV_OK) {
    ctx->table_dirty = true;
    set_error("shmt_sample_minibatch: device status %lld (%s)", (long long)st,
              st == DEV_TIMEOUT ? "a bounded look-back wait ran out" : "relabel table overflow");
    return st == DEV_TIMEOUT ? SHMT_ERR_TIMEOUT : SHMT_ERR_CAPACITY;
  }
  int64_t n_in = n_seeds;
  for (int h = 0; h < n_hops; ++h) {
    sizes_host[3 * h + 0] = n_in;
    sizes_host[3 * h + 1] = ctx->h_words[h * 8 + 1];
    sizes_host[3 * h + 2] = ctx->h_words[h * 8 + 3];
    n_in = sizes_host[3 * h + 2];
  }
  return SHMT_OK;
}

int shmt_sample_minibatch(shmt_ctx* ctx, const void* indptr, int indptr_dtype, const void* indices,
                          int indices_dtype, const void* gpu_indptr, const void* gpu_indices,
                          const shmt_map* map, const void* seeds, int64_t n_seeds,
                          const int64_t* fanouts, int n_hops, int replace, uint64_t rng_seed,
                          uint64_t rng_offset, void* const* out_sub_indptr,
                          void* const* out_sub_indices, void* const* out_relabel,
                          void* const* out_frontier, int64_t* sizes_host, void* stream) {
  return sample_minibatch_impl(ctx, indptr, indptr_dtype, indices, indices_dtype, gpu_indptr, gpu_indices, map,
                               seeds, n_seeds, fanouts, n_hops, replace, rng_seed, rng_offset, out_sub_indptr,
                               out_sub_indices, out_relabel, out_frontier, sizes_host, stream, nullptr, nullptr);
}

int shmt_sample_minibatch_eids(shmt_ctx* ctx, const void* indptr, int indptr_dtype, const void* indices,
                               int indices_dtype, const void* gpu_indptr, const void* gpu_indices,
                               const void* gpu_edge_base, const shmt_map* map, const void* seeds,
                               int64_t n_seeds, const int64_t* fanouts, int n_hops, int replace,
                               uint64_t rng_seed, uint64_t rng_offset, void* const* out_sub_indptr,
                               void* const* out_sub_indices, void* const* out_edge_ids,
                               void* const* out_relabel, void* const* out_frontier,
                               int64_t* sizes_host, void* stream) {
  SHMT_REQUIRE(out_edge_ids != nullptr, "shmt_sample_minibatch_eids: out_edge_ids is null");
  SHMT_REQUIRE(map == nullptr || gpu_edge_base != nullptr,
               "shmt_sample_minibatch_eids: a cached graph needs gpu_edge_base (shmt_subcsr_edge_base)");
  for (int h = 0; h < n_hops && h < 8; ++h)
    SHMT_REQUIRE(out_edge_ids[h] != nullptr, "shmt_sample_minibatch_eids: edge-id buffer of hop %d is null", h);
  return sample_minibatch_impl(ctx, indptr, indptr_dtype, indices, indices_dtype, gpu_indptr, gpu_indices, map,
                               seeds, n_seeds, fanouts, n_hops, replace, rng_seed, rng_offset, out_sub_indptr,
                               out_sub_indices, out_relabel, out_frontier, sizes_host, stream, gpu_edge_base,
                               out_edge_ids);
}

int shmt_sample_minibatch_weighted(shmt_ctx* ctx, const void* indptr, int indptr_dtype, const void* indices,
                                   int indices_dtype, const float* weights, const void* gpu_indptr,
                                   const void* gpu_indices, const float* gpu_weights, const shmt_map* map,
                                   const void* seeds, int64_t n_seeds, const int64_t* fanouts, int n_hops,
                                   int replace, uint64_t rng_seed, uint64_t rng_offset,
                                   void* const* out_sub_indptr, void* const* out_sub_indices,
                                   void* const* out_relabel, void* const* out_frontier, int64_t* sizes_host,
                                   void* stream) {
  SHMT_REQUIRE(weights != nullptr, "shmt_sample_minibatch_weighted: weights are null");
  SHMT_REQUIRE(map == nullptr || gpu_weights != nullptr,
               "shmt_sample_minibatch_weighted: a cached graph needs gpu_weights");
  for (int h = 0; fanouts && h < n_hops && h < 8; ++h)
    SHMT_REQUIRE(replace || fanouts[h] <= 32,
                 "shmt_sample_minibatch_weighted: without replacement the fan-out is at most 32 (hop %d has %lld)", h,
                 (long long)fanouts[h]);
  return sample_minibatch_impl(ctx, indptr, indptr_dtype, indices, indices_dtype, gpu_indptr, gpu_indices, map,
                               seeds, n_seeds, fanouts, n_hops, replace, rng_seed, rng_offset, out_sub_indptr,
                               out_sub_indices, out_relabel, out_frontier, sizes_host, stream, nullptr, nullptr,
                               weights, gpu_weights);
}

int shmt_subcsr_count(shmt_ctx* ctx, const void* indptr, int indptr_dtype, const void* seeds,
                      int seeds_dtype, int64_t n, void* out_gpu_indptr, int64_t* nnz_host,
                      void* stream) {
  SHMT_REQUIRE(ctx != nullptr, "shmt_subcsr_count: ctx is null");
  SHMT_REQUIRE(valid_int_dtype(indptr_dtype) && valid_int_dtype(seeds_dtype),
               "shmt_subcsr_count: ID can only be int32 or int64");
  SHMT_REQUIRE(n >= 0, "shmt_subcsr_count: negative count");
  SHMT_REQUIRE(indptr && out_gpu_indptr && (n == 0 || seeds), "shmt_subcsr_count: null argument");
  DeviceGuard guard(ctx->device);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (int rc = ctx_reserve(ctx, scan_scratch_bytes(n + 1))) return rc;
  int64_t blocks = (n + 1 + 255) / 256;
  const int64_t cap = (int64_t)sm_count() * 16;
  subcsr_degree_kernel<<<(unsigned)(blocks < cap ? blocks : cap), 256, 0, s>>>(
      indptr, indptr_dtype == SHMT_I64, seeds, seeds_dtype == SHMT_I64, n, out_gpu_indptr);
  SHMT_CUDA_TRY(cudaGetLastError());
  if (int rc = launch_scan(ctx, out_gpu_indptr, indptr_dtype, n + 1, /*exclusive=*/1, 0, s))
    return rc;
  if (nnz_host) {
    int64_t last = 0;
    const int sz = int_itemsize(indptr_dtype);
    SHMT_CUDA_TRY(cudaMemcpyAsync(&last, static_cast<char*>(out_gpu_indptr) + (size_t)n * sz, sz,
                                  cudaMemcpyDeviceToHost, s));
    if (int rc = ctx_fetch_words(ctx, s, "shmt_subcsr_count")) return rc;
    *nnz_host = indptr_dtype == SHMT_I64 ? last : (int64_t)(int32_t)last;
  }
  return SHMT_OK;
}

int shmt_subcsr_edge_base(const void* indptr, int indptr_dtype, const void* seeds, int seeds_dtype,
                          int64_t n, void* out_edge_base, void* stream) {
  SHMT_REQUIRE(valid_int_dtype(indptr_dtype) && valid_int_dtype(seeds_dtype),
               "shmt_subcsr_edge_base: ID can only be int32 or int64");
  SHMT_REQUIRE(n >= 0, "shmt_subcsr_edge_base: negative count");
  if (n == 0) return SHMT_OK;
  SHMT_REQUIRE(indptr && seeds && out_edge_base, "shmt_subcsr_edge_base: null argument");
  int64_t blocks = (n + 255) / 256;
  const int64_t cap = (int64_t)sm_count() * 16;
  subcsr_edge_base_kernel<<<(unsigned)(blocks < cap ? blocks : cap), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      indptr, indptr_dtype == SHMT_I64, seeds, seeds_dtype == SHMT_I64, n, out_edge_base);
  SHMT_CUDA_TRY(cudaGetLastError());
  return SHMT_OK;
}

int shmt_subcsr_fill(const void* indptr, int indptr_dtype, const void* indices, int indices_dtype,
                     const void* seeds, int seeds_dtype, int64_t n, const void* gpu_indptr,
                     void* out_gpu_indices, void* stream) {
  SHMT_REQUIRE(valid_int_dtype(indptr_dtype) && valid_int_dtype(indices_dtype) &&
                   valid_int_dtype(seeds_dtype),
               "shmt_subcsr_fill: ID can only be int32 or int64");
  SHMT_REQUIRE(n >= 0, "shmt_subcsr_fill: negative count");
  if (n == 0) return SHMT_OK;
  SHMT_REQUIRE(indptr && indices && seeds && gpu_indptr, "shmt_subcsr_fill: null argument");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  int64_t blocks = (n + 7) / 8;
  const int64_t cap = (int64_t)sm_count() * 32;
  const unsigned grid = (unsigned)(blocks < cap ? blocks : cap);
  if (indices_dtype == SHMT_I64)
    subcsr_fill_kernel<long long><<<grid, 256, 0, s>>>(
        indptr, indptr_dtype == SHMT_I64, static_cast<const long long*>(indices), seeds,
        seeds_dtype == SHMT_I64, n, gpu_indptr, static_cast<long long*>(out_gpu_indices));
  else
    subcsr_fill_kernel<int><<<grid, 256, 0, s>>>(
        indptr, indptr_dtype == SHMT_I64, static_cast<const int*>(indices), seeds,
        seeds_dtype == SHMT_I64, n, gpu_indptr, static_cast<int*>(out_gpu_indices));
  SHMT_CUDA_TRY(cudaGetLastError());
  return SHMT_OK;
}

}  // extern "C"
