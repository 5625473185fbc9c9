// In-place prefix sum in one pass with decoupled look-back: a ticketed kernel over 64 KB tiles
// for small inputs, a persistent thread-block-cluster kernel with early sums for large ones.
// Semantics follow cub_exclusiveSum (reference src/cache_graph_sampling.cu:30-45)
// and the intended meaning of thrust_scan (reference src/thrust_scan.cu:9-18,
// whose own lambda races); integer arithmetic wraps.
#include <stdlib.h>

#include "bulk.cuh"
#include "ctx.cuh"
#include "lookback.cuh"

namespace shmt {

constexpr int kScanThreads = 512;
constexpr int kScanWarps = kScanThreads / 32;
constexpr int kScanVecs = 8;                                     // 16-byte vectors per thread
constexpr int kScanTileBytes = kScanThreads * kScanVecs * 16;    // 64 KB per tile
constexpr int kScanTile = kScanTileBytes / 8;                    // items per tile of the widest type
constexpr int kScanPartials = kScanVecs * kScanWarps;            // one per (row, warp)
static_assert(kScanPartials % 32 == 0, "warp 0 scans the per-warp partials, the same number per lane");

template <typename T>
struct ScanWord;
template <>
struct ScanWord<int> { using type = unsigned; };
template <>
struct ScanWord<long long> { using type = unsigned long long; };

// A tile is 8 rows of 512 16-byte vectors (64 KB); thread t owns vector t of every row, so each
// load and store instruction of a warp covers 512 contiguous bytes.  Sums are taken in the unsigned
// type of the data (wrap-around is defined and the low bits are all the result keeps): inside a
// vector, across the warp with shuffles, across the 128 (row, warp) partials by warp 0, which
// also does the look-back; every thread then adds its three offsets and stores.  Large tiles
// matter: the look-back hands a prefix over at most 32 tiles per round trip through L2, so the
// bytes per tile bound the rate of the whole scan.
template <typename T>
__global__ void __launch_bounds__(kScanThreads, 2)
scan_kernel(T* __restrict__ data, int64_t n, int exclusive, int vec_ok, TileStates st, int64_t* words,
            const TileDesc* carry) {
  using U = typename ScanWord<T>::type;
  constexpr int VEC = 16 / (int)sizeof(T);
  constexpr int TILE = kScanTileBytes / (int)sizeof(T);
  constexpr int PER_LANE = kScanPartials / 32;
  __shared__ U partial[kScanPartials];  // [row][warp]
  __shared__ int64_t s_prefix;
  __shared__ int s_tile;
  const unsigned full = 0xffffffffu;
  const unsigned tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int tile = take_tile(words + W_TICKET, &s_tile);
  const int64_t tile_base = (int64_t)tile * TILE;
  union Pack {
    uint4 q;
    U a[VEC];
  };

  U v[kScanVecs][VEC], vsum[kScanVecs], inc[kScanVecs];
#pragma unroll
  for (int k = 0; k < kScanVecs; ++k) {
    const int64_t at = tile_base + ((int64_t)k * kScanThreads + tid) * VEC;
    if (vec_ok && at + VEC <= n) {
      Pack p;
      p.q = *reinterpret_cast<const uint4*>(data + at);
#pragma unroll
      for (int j = 0; j < VEC; ++j) v[k][j] = p.a[j];
    } else {
#pragma unroll
      for (int j = 0; j < VEC; ++j) v[k][j] = at + j < n ? (U)data[at + j] : U(0);
    }
  }
#pragma unroll
  for (int k = 0; k < kScanVecs; ++k) {
#pragma unroll
    for (int j = 1; j < VEC; ++j) v[k][j] += v[k][j - 1];
    vsum[k] = v[k][VEC - 1];
    inc[k] = vsum[k];
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const U up = __shfl_up_sync(full, inc[k], o);
      if (lane >= (unsigned)o) inc[k] += up;
    }
    if (lane == 31) partial[k * kScanWarps + warp] = inc[k];
  }
  __syncthreads();
  if (warp == 0) {
    // the partials in tile order, PER_LANE consecutive ones per lane
    U a[PER_LANE], lsum = 0;
#pragma unroll
    for (int q = 0; q < PER_LANE; ++q) {
      a[q] = partial[lane * PER_LANE + q];
      lsum += a[q];
    }
    U linc = lsum;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const U up = __shfl_up_sync(full, linc, o);
      if (lane >= (unsigned)o) linc += up;
    }
    U run = linc - lsum;
#pragma unroll
    for (int q = 0; q < PER_LANE; ++q) {
      partial[lane * PER_LANE + q] = run;  // everything ahead of this (row, warp)
      run += a[q];
    }
    const U total = __shfl_sync(full, linc, 31);
    // zero-extended aggregate: tile sums add up in 64 bits, of which the low bits are used
    const int64_t p = lookback_exclusive_prefix(st, tile, (int64_t)(uint64_t)total, words + W_STATUS);
    // `carry`: this launch continues a scan whose first part another kernel did (its last
    // descriptor holds the sum of everything before `data`)
    if (lane == 0) s_prefix = p + (carry ? carry->value : 0);
  }
  __syncthreads();
  const U prefix = (U)(uint64_t)s_prefix;
#pragma unroll
  for (int k = 0; k < kScanVecs; ++k) {
    const int64_t at = tile_base + ((int64_t)k * kScanThreads + tid) * VEC;
    const U before = prefix + partial[k * kScanWarps + warp] + (inc[k] - vsum[k]);
    Pack p;
#pragma unroll
    for (int j = 0; j < VEC; ++j)
      p.a[j] = before + (exclusive ? (j ? v[k][j - 1] : U(0)) : v[k][j]);
    if (vec_ok && at + VEC <= n) {
      *reinterpret_cast<uint4*>(data + at) = p.q;
    } else {
#pragma unroll
      for (int j = 0; j < VEC; ++j)
        if (at + j < n) data[at + j] = (T)p.a[j];
    }
  }
}


// ---- large inputs: persistent clusters ------------------------------------------------------
// What bounds the kernel above is not bytes but the time a tile sits in registers: ticket,
// load latency, local sums, look-back, store.  A tile cannot leave before EVERY earlier tile has
// published its sum, so each tile waits for the slowest load among the hundreds in flight;
// timed on B200, that wait was 4.0 us of a 7.0 us iteration.  This kernel takes the waits off
// that path:
// (1) The grid is persistent (every cluster resident at once, super-tiles dealt round-robin), so
//     there is no ticket: a tile's predecessors belong to clusters that are running and only
//     ever wait for still earlier tiles.
// (2) A CTA keeps two landing buffers: the tiles of its next two iterations are brought into
//     shared memory by bulk copies while the current one is scanned and stored from registers.
// (3) The sum of the NEXT tile is taken from its landing buffer and published one iteration
//     early, by the warps that would otherwise idle while warp 0 looks back for the current
//     tile.  When a tile's own look-back starts, the sums of everything in flight before it have
//     been out for a whole iteration: the look-back reads them, it does not wait for them.
// (4) The four CTAs of a cluster add their sums up through distributed shared memory and publish
//     one descriptor per 128 KB super-tile.  The sums travel as asynchronous remote stores that
//     complete a transaction on the receiver's mbarrier, so no cluster-wide barrier (and no
//     memory fence behind the previous tile's global stores) sits in the loop.
#ifndef SHMT_SCAN_CLUSTER
#define SHMT_SCAN_CLUSTER 4
#endif
#ifndef SHMT_SCAN_CL_THREADS
#define SHMT_SCAN_CL_THREADS 256
#endif
#ifndef SHMT_SCAN_CL_CTAS
#define SHMT_SCAN_CL_CTAS 3  // per SM: two 32 KB landing buffers each
#endif
#ifndef SHMT_SCAN_CL_WINDOWS
#define SHMT_SCAN_CL_WINDOWS 1
#endif
#ifndef SHMT_SCAN_CL_VECS
#define SHMT_SCAN_CL_VECS 8
#endif
constexpr int kScanCluster = SHMT_SCAN_CLUSTER;
constexpr int kClThreads = SHMT_SCAN_CL_THREADS;
constexpr int kClWarps = kClThreads / 32;
constexpr int kClVecs = SHMT_SCAN_CL_VECS;
constexpr int kClTileBytes = kClThreads * kClVecs * 16;
constexpr int kClTileVecs = kClThreads * kClVecs;
constexpr int kClPartials = kClVecs * kClWarps;
constexpr int kClCtasPerSm = SHMT_SCAN_CL_CTAS;
constexpr int kClWindows = SHMT_SCAN_CL_WINDOWS;  // x 32 predecessors read per look-back step
constexpr int kClSmemBytes = 2 * kClTileBytes;
static_assert(kClPartials % 32 == 0, "warp 0 scans the per-warp partials, the same number per lane");
static_assert(kClWarps >= 2 && kClWarps <= 32, "warp 0 looks back, the others sum the next tile");
constexpr int64_t kScanSuperBytes = (int64_t)kScanCluster * kClTileBytes;
constexpr int64_t kScanClusterMinBytes = (int64_t)32 << 20;  // below this the ticketed kernel spreads better

__device__ __forceinline__ unsigned cluster_ctarank() {
  unsigned r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ unsigned cluster_id_x() {
  unsigned r;
  asm volatile("mov.u32 %0, %%clusterid.x;" : "=r"(r));
  return r;
}
__device__ __forceinline__ unsigned cluster_count_x() {
  unsigned r;
  asm volatile("mov.u32 %0, %%nclusterid.x;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// barrier among the warps 1 .. kClWarps-1 of a CTA (warp 0 is looking back meanwhile)
__device__ __forceinline__ void helpers_sync() {
  asm volatile("bar.sync 1, %0;" ::"n"(kClThreads - 32) : "memory");
}
// 8 bytes into the shared memory of CTA `rank` of this cluster, at the address `local` has in the
// calling CTA (same kernel, same layout), counted as 8 bytes of transaction on the receiver's
// mbarrier `local_bar`: whoever waits on that barrier sees the data.
__device__ __forceinline__ void st_async_cluster_u64(void* local, void* local_bar, unsigned rank,
                                                     unsigned long long v) {
  uint32_t remote, remote_bar;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(smem_addr(local)), "r"(rank));
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote_bar) : "r"(smem_addr(local_bar)), "r"(rank));
  asm volatile("st.async.weak.shared::cluster.mbarrier::complete_tx::bytes.u64 [%0], %1, [%2];" ::"r"(remote),
               "l"(v), "r"(remote_bar)
               : "memory");
}

template <typename T>
__global__ void __launch_bounds__(kClThreads, kClCtasPerSm)
scan_cluster_kernel(T* __restrict__ data, int64_t n_super, int exclusive, TileStates st, int64_t* words) {
  using U = typename ScanWord<T>::type;
  constexpr int VEC = 16 / (int)sizeof(T);
  constexpr int PER_LANE = kClPartials / 32;
  extern __shared__ __align__(128) unsigned char landing[];  // two tiles, filled by bulk copies
  __shared__ U partial[kClPartials];
  __shared__ U s_help[32];                                            // per-warp sums of the next tile
  __shared__ __align__(8) unsigned long long s_sum[2][kScanCluster];  // CTA sums of the cluster, by tile parity
  __shared__ __align__(8) uint64_t s_sumbar[2];                       // their arrival, by tile parity
  __shared__ unsigned long long s_whole[2], s_before[2];              // cluster sum / sum of lower ranks, by tile parity
  __shared__ int64_t s_prefix;
  __shared__ __align__(8) uint64_t s_bar[2];                          // landing buffers, by tile parity
  const unsigned full = 0xffffffffu;
  const unsigned tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const unsigned rank = cluster_ctarank();
  const int64_t n_clusters = cluster_count_x();
  int64_t* status = words + W_STATUS;
  char* bytes = reinterpret_cast<char*>(data);
  union Pack {
    uint4 q;
    U a[VEC];
  };
  auto flag_timeout = [&]() {
    atomicMax(reinterpret_cast<unsigned long long*>(status), (unsigned long long)DEV_TIMEOUT);
  };
  // bulk copy of this CTA's part of super-tile `sup` into landing buffer j & 1 (one thread)
  auto issue_load = [&](int64_t sup, int j) {
    mbar_arrive_expect_tx(&s_bar[j & 1], kClTileBytes);
    bulk_load(landing + (size_t)(j & 1) * kClTileBytes, bytes + (sup * kScanCluster + rank) * kClTileBytes,
              kClTileBytes, &s_bar[j & 1]);
  };
  // The sum of tile j (of super-tile `sup`), taken from its landing buffer by the calling
  // threads -- `n_threads` of them, numbered `t`, whole warps, synchronised by `sync` -- and
  // handed round the cluster; the first warp of them waits for the cluster's sums, leaves the
  // totals for the look-back in s_whole / s_before and, on rank 0, publishes the aggregate.
  auto publish_sum = [&](int64_t sup, int j, unsigned t, unsigned n_threads, unsigned first_warp, auto sync) {
    const int b = j & 1;
    if (!mbar_wait_bounded(&s_bar[b], (uint32_t)(j >> 1) & 1u)) flag_timeout();
    const uint4* src = reinterpret_cast<const uint4*>(landing + (size_t)b * kClTileBytes);
    U acc = 0;
    for (unsigned q = t; q < (unsigned)kClTileVecs; q += n_threads) {
      Pack p;
      p.q = src[q];
#pragma unroll
      for (int e = 0; e < VEC; ++e) acc += p.a[e];
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(full, acc, o);
    if (lane == 0) s_help[warp] = acc;
    sync();
    if (warp == first_warp) {
      U total = 0;
      for (unsigned w = first_warp; w < first_warp + n_threads / 32; ++w) total += s_help[w];
      if (lane == 0) mbar_arrive_expect_tx(&s_sumbar[b], 8 * kScanCluster);
      if (lane < kScanCluster) st_async_cluster_u64(&s_sum[b][rank], &s_sumbar[b], lane, (unsigned long long)total);
      if (!mbar_wait_bounded(&s_sumbar[b], (uint32_t)(j >> 1) & 1u)) flag_timeout();
      unsigned long long before = 0, whole = 0;
#pragma unroll
      for (int r = 0; r < kScanCluster; ++r) {
        const unsigned long long x = s_sum[b][r];
        whole += x;
        if ((unsigned)r < rank) before += x;
      }
      if (lane == 0) {
        s_whole[b] = whole;
        s_before[b] = before;
        if (rank == 0) st_desc(st.d + sup, (long long)whole, sup == 0 ? kTileInclusive : kTileAggregate);
      }
    }
  };

  if (tid == 0) {
    mbar_init(&s_bar[0], 1);
    mbar_init(&s_bar[1], 1);
    mbar_init(&s_sumbar[0], 1);
    mbar_init(&s_sumbar[1], 1);
  }
  mbar_init_fence();
  __syncthreads();
  cluster_sync_all();  // every CTA of the cluster runs and has its barriers before anyone sends to it

  int64_t super = cluster_id_x();
  if (tid == 0) {
    if (super < n_super) issue_load(super, 0);
    if (super + n_clusters < n_super) issue_load(super + n_clusters, 1);
  }
  if (super < n_super) publish_sum(super, 0, tid, kClThreads, 0, [] { __syncthreads(); });
  __syncthreads();

  for (int it = 0; super < n_super; super += n_clusters, ++it) {
    const int b = it & 1;
    // ---- the tile into registers, sums inside vectors and warps.  It landed before its sum was
    // taken an iteration ago, so this wait returns at once; it is what entitles every thread (not
    // only those that summed) to read what the bulk copy wrote.
    if (!mbar_wait_bounded(&s_bar[b], (uint32_t)(it >> 1) & 1u)) flag_timeout();
    U v[kClVecs][VEC], inc[kClVecs];  // a vector's own sum stays in its last element
    const uint4* src = reinterpret_cast<const uint4*>(landing + (size_t)b * kClTileBytes);
#pragma unroll
    for (int k = 0; k < kClVecs; ++k) {
      Pack p;
      p.q = src[k * kClThreads + tid];
#pragma unroll
      for (int j = 0; j < VEC; ++j) v[k][j] = p.a[j];
    }
#pragma unroll
    for (int k = 0; k < kClVecs; ++k) {
#pragma unroll
      for (int j = 1; j < VEC; ++j) v[k][j] += v[k][j - 1];
      inc[k] = v[k][VEC - 1];
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const U up = __shfl_up_sync(full, inc[k], o);
        if (lane >= (unsigned)o) inc[k] += up;
      }
      if (lane == 31) partial[k * kClWarps + warp] = inc[k];
    }
    __syncthreads();  // the tile is in registers: its landing buffer is free
    const int64_t next = super + n_clusters, after_next = next + n_clusters;
    if (tid == 0 && after_next < n_super) issue_load(after_next, it + 2);
    if (warp == 0) {
      // ---- warp 0: offsets of the (row, warp) partials, then the look-back (every sum it needs
      // was published an iteration ago)
      U a[PER_LANE], lsum = 0;
#pragma unroll
      for (int q = 0; q < PER_LANE; ++q) {
        a[q] = partial[lane * PER_LANE + q];
        lsum += a[q];
      }
      U linc = lsum;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const U up = __shfl_up_sync(full, linc, o);
        if (lane >= (unsigned)o) linc += up;
      }
      U run = linc - lsum;
#pragma unroll
      for (int q = 0; q < PER_LANE; ++q) {
        partial[lane * PER_LANE + q] = run;
        run += a[q];
      }
      const int64_t p = lookback_published<kClWindows>(st, (int)super, (int64_t)s_whole[b], rank == 0, status);
      if (lane == 0) s_prefix = p + (int64_t)s_before[b];
    } else if (next < n_super) {
      // ---- the other warps: the next tile's sum, out to the cluster and (rank 0) to its descriptor
      publish_sum(next, it + 1, tid - 32, kClThreads - 32, 1, [] { helpers_sync(); });
    }
    __syncthreads();
    const U prefix = (U)(uint64_t)s_prefix;
    T* out = data + (super * kScanCluster + rank) * (kClTileBytes / (int64_t)sizeof(T));
#pragma unroll
    for (int k = 0; k < kClVecs; ++k) {
      const U ahead = prefix + partial[k * kClWarps + warp] + (inc[k] - v[k][VEC - 1]);
      Pack p;
#pragma unroll
      for (int j = 0; j < VEC; ++j)
        p.a[j] = ahead + (exclusive ? (j ? v[k][j - 1] : U(0)) : v[k][j]);
      reinterpret_cast<uint4*>(out)[k * kClThreads + tid] = p.q;
    }
  }
  // nobody leaves while a CTA of the cluster may still be sending to it or reading its barriers
  cluster_sync_all();
}

// Clusters of the persistent grid: as many as are resident at once (asked of the runtime once
// per device and element type), never more than there are super-tiles.
template <typename T>
static int scan_cluster_grid(int64_t n_super, unsigned* grid) {
  static int resident[64] = {0};
  int dev = 0;
  SHMT_CUDA_TRY(cudaGetDevice(&dev));
  SHMT_REQUIRE(dev >= 0 && dev < 64, "scan: device index %d not supported", dev);
  if (resident[dev] == 0) {
    SHMT_CUDA_TRY(cudaFuncSetAttribute(scan_cluster_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       kClSmemBytes));
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(kScanCluster * 64);
    cfg.blockDim = dim3(kClThreads);
    cfg.dynamicSmemBytes = kClSmemBytes;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = kScanCluster;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    int n = 0;
    SHMT_CUDA_TRY(cudaOccupancyMaxActiveClusters(&n, scan_cluster_kernel<T>, &cfg));
    SHMT_REQUIRE(n >= 1, "scan: no cluster of %d CTAs fits on this device", kScanCluster);
    resident[dev] = n;
  }
  const int64_t c = n_super < resident[dev] ? n_super : resident[dev];
  *grid = (unsigned)(c * kScanCluster);
  return SHMT_OK;
}

template <typename T>
static int run_scan_clusters(void* data, int64_t n_super, int exclusive, TileStates st, int64_t* words,
                             cudaStream_t s) {
  unsigned grid = 0;
  if (int rc = scan_cluster_grid<T>(n_super, &grid)) return rc;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(grid);
  cfg.blockDim = dim3(kClThreads);
  cfg.dynamicSmemBytes = kClSmemBytes;
  cfg.stream = s;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = kScanCluster;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  SHMT_CUDA_TRY(cudaLaunchKernelEx(&cfg, scan_cluster_kernel<T>, static_cast<T*>(data), n_super, exclusive, st, words));
  return SHMT_OK;
}

template <typename T>
static int64_t scan_tiles(int64_t n) {
  const int64_t tile = kScanTileBytes / (int64_t)sizeof(T);
  return (n + tile - 1) / tile;
}

template <typename T>
static void run_scan(void* data, int64_t n, int exclusive, TileStates st, int64_t* words, cudaStream_t s,
                     const TileDesc* carry = nullptr) {
  const int vec_ok = ((uintptr_t)data & 15) == 0;
  scan_kernel<T><<<(unsigned)scan_tiles<T>(n), kScanThreads, 0, s>>>(static_cast<T*>(data), n, exclusive,
                                                                      vec_ok, st, words, carry);
}

// Large, 16-byte aligned inputs: whole 256 KB super-tiles by the persistent cluster kernel, what
// is left (less than one super-tile) by the ticketed kernel, which starts from the sum the
// last super-tile's descriptor holds.
template <typename T>
static int run_scan_large(void* data, int64_t n, int exclusive, char* state_base, int64_t* words, cudaStream_t s) {
  const int64_t per_super = kScanSuperBytes / (int64_t)sizeof(T);
  const int64_t n_super = n / per_super;
  TileStates st = carve_tile_states(state_base, n_super);
  if (int rc = run_scan_clusters<T>(data, n_super, exclusive, st, words, s)) return rc;
  const int64_t rest = n - n_super * per_super;
  if (rest > 0) {
    TileStates tail = carve_tile_states(state_base + tile_state_bytes(n_super), scan_tiles<T>(rest));
    run_scan<T>(static_cast<T*>(data) + n_super * per_super, rest, exclusive, tail, words, s, st.d + (n_super - 1));
  }
  return SHMT_OK;
}

// Exercises the give-up path of the look-back on purpose, harmlessly: one warp plays tile 1
// of a scan whose tile 0 never runs, with a short spin limit.  It must record DEV_TIMEOUT and
// return; nothing else is touched.
__global__ void lookback_timeout_probe_kernel(TileStates st, int64_t* words, int spin_limit) {
  lookback_exclusive_prefix(st, /*tile=*/1, /*aggregate=*/1, words + W_STATUS, spin_limit);
}

// Launch helper shared with relabel / sub-CSR: scans `n` items in place using
// ctx scratch at byte offset `scratch_off` for the tile states.
int launch_scan(shmt_ctx* ctx, void* data, int dtype, int64_t n, int exclusive,
                size_t scratch_off, cudaStream_t stream) {
  if (n <= 0) return SHMT_OK;
  const int64_t n_tiles = (n + kScanTile - 1) / kScanTile;
  SHMT_REQUIRE(n_tiles < (int64_t)1 << 30, "scan: %lld items is too many", (long long)n);
  TileStates st = carve_tile_states(ctx->region() + scratch_off, n_tiles);
  // status / result / ticket words and the tile descriptors start at zero (one memset when the
  // descriptors sit right behind the words, as they do for a plain scan)
  if (scratch_off == 0) {
    SHMT_CUDA_TRY(cudaMemsetAsync(ctx->scratch, 0, 256 + tile_state_bytes(n_tiles), stream));
  } else {
    SHMT_CUDA_TRY(cudaMemsetAsync(ctx->d_words(), 0, 256, stream));
    SHMT_CUDA_TRY(cudaMemsetAsync(st.d, 0, tile_state_bytes(n_tiles), stream));
  }
  static const bool no_clusters = getenv("SHMT_SCAN_NO_CLUSTERS") != nullptr;
  if (!no_clusters && ((uintptr_t)data & 15) == 0 && n * int_itemsize(dtype) >= kScanClusterMinBytes) {
    // the ticketed kernel's descriptor block is larger than what both kernels need here
    char* base = reinterpret_cast<char*>(st.d);
    if (int rc = dtype == SHMT_I64 ? run_scan_large<long long>(data, n, exclusive, base, ctx->d_words(), stream)
                                   : run_scan_large<int>(data, n, exclusive, base, ctx->d_words(), stream))
      return rc;
  } else if (dtype == SHMT_I64) {
    run_scan<long long>(data, n, exclusive, st, ctx->d_words(), stream);
  } else {
    run_scan<int>(data, n, exclusive, st, ctx->d_words(), stream);
  }
  SHMT_CUDA_TRY(cudaGetLastError());
  return SHMT_OK;
}

size_t scan_scratch_bytes(int64_t n) {
  const int64_t n_tiles = (n + kScanTile - 1) / kScanTile;
  return (tile_state_bytes(n_tiles > 0 ? n_tiles : 1) + 255) & ~(size_t)255;
}

// ---- scan without any allocation ----------------------------------------------------
// Look-back state for shmt_scan_static lives in this fixed array instead of context
// scratch.  Every GPU that loads the library carries it (about 33 KB) until exit.
constexpr int64_t kStaticScanMaxItems = (int64_t)1 << 24;
constexpr int64_t kStaticScanMaxTiles = kStaticScanMaxItems / kScanTile;
constexpr size_t kStaticScanBytes = 256 + ((tile_state_bytes(kStaticScanMaxTiles) + 255) & ~(size_t)255);
static __device__ __align__(256) unsigned char g_static_scan_scratch[kStaticScanBytes];

// Device address of the array on the current device.  In host code the array's name is
// only a handle for the runtime, never an address a kernel may be given, so it is resolved
// once per device with cudaGetSymbolAddress and the result is what kernels receive.
static int static_scan_scratch(unsigned char** out) {
  static unsigned char* resolved[64] = {nullptr};
  int dev = 0;
  SHMT_CUDA_TRY(cudaGetDevice(&dev));
  SHMT_REQUIRE(dev >= 0 && dev < 64, "shmt_scan_static: device index %d not supported", dev);
  if (!resolved[dev]) {
    unsigned char* p = nullptr;
    SHMT_CUDA_TRY(cudaGetSymbolAddress((void**)&p, g_static_scan_scratch));
    SHMT_REQUIRE(p != nullptr, "shmt_scan_static: the scratch array has no device address");
    resolved[dev] = p;
  }
  *out = resolved[dev];
  return SHMT_OK;
}

}  // namespace shmt

using namespace shmt;

extern "C" int shmt_scan_static(void* data, int dtype, int64_t n, int exclusive, void* stream) {
  SHMT_REQUIRE(valid_int_dtype(dtype), "shmt_scan_static: dtype code %d is not SHMT_I32/SHMT_I64",
               dtype);
  SHMT_REQUIRE(n >= 0, "shmt_scan_static: negative length");
  SHMT_REQUIRE(n <= kStaticScanMaxItems,
               "shmt_scan_static: %lld items exceed the fixed scratch (limit %lld); use shmt_scan",
               (long long)n, (long long)kStaticScanMaxItems);
  if (n == 0) return SHMT_OK;
  SHMT_REQUIRE(data != nullptr, "shmt_scan_static: data is null");
  unsigned char* base = nullptr;
  if (int rc = static_scan_scratch(&base)) return rc;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int64_t n_tiles = (n + kScanTile - 1) / kScanTile;
  int64_t* words = reinterpret_cast<int64_t*>(base);
  TileStates st = carve_tile_states(reinterpret_cast<char*>(base) + 256, n_tiles);
  // the array still holds the previous call's ticket, status and tile descriptors: zero the
  // words and the descriptors this call will use (they sit right behind the 256-byte header)
  SHMT_CUDA_TRY(cudaMemsetAsync(base, 0, 256 + tile_state_bytes(n_tiles), s));
  if (dtype == SHMT_I64)
    run_scan<long long>(data, n, exclusive, st, words, s);
  else
    run_scan<int>(data, n, exclusive, st, words, s);
  SHMT_CUDA_TRY(cudaGetLastError());
  return SHMT_OK;
}

// What the last shmt_scan_static call on the current device left in its status word.  The word
// lives in the fixed array, which no context covers, so it has a check of its own; like the
// scan itself it allocates nothing (one 8-byte copy and a wait for `stream`).
extern "C" int shmt_scan_static_check(void* stream) {
  unsigned char* base = nullptr;
  if (int rc = static_scan_scratch(&base)) return rc;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  int64_t status = 0;
  SHMT_CUDA_TRY(cudaMemcpyAsync(&status, reinterpret_cast<int64_t*>(base) + W_STATUS, sizeof(status),
                                cudaMemcpyDeviceToHost, s));
  SHMT_CUDA_TRY(cudaStreamSynchronize(s));
  if (status == DEV_TIMEOUT) {
    set_error("shmt_scan_static: a bounded look-back wait ran out; the result is not a prefix sum");
    return SHMT_ERR_TIMEOUT;
  }
  return SHMT_OK;
}

extern "C" int shmt_debug_lookback_timeout(shmt_ctx* ctx, void* stream) {
  SHMT_REQUIRE(ctx != nullptr, "shmt_debug_lookback_timeout: ctx is null");
  DeviceGuard guard(ctx->device);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (int rc = ctx_reserve(ctx, tile_state_bytes(2))) return rc;
  TileStates st = carve_tile_states(ctx->region(), 2);
  SHMT_CUDA_TRY(cudaMemsetAsync(ctx->scratch, 0, 256 + tile_state_bytes(2), s));
  lookback_timeout_probe_kernel<<<1, 32, 0, s>>>(st, ctx->d_words(), 1 << 10);
  SHMT_CUDA_TRY(cudaGetLastError());
  return ctx_fetch_words(ctx, s, "shmt_debug_lookback_timeout");
}

extern "C" int shmt_scan(shmt_ctx* ctx, void* data, int dtype, int64_t n, int exclusive,
                         void* stream) {
  SHMT_REQUIRE(ctx != nullptr, "shmt_scan: ctx is null");
  SHMT_REQUIRE(valid_int_dtype(dtype), "shmt_scan: dtype code %d is not SHMT_I32/SHMT_I64", dtype);
  SHMT_REQUIRE(n >= 0, "shmt_scan: negative length");
  if (n == 0) return SHMT_OK;
  SHMT_REQUIRE(data != nullptr, "shmt_scan: data is null");
  DeviceGuard guard(ctx->device);
  if (int rc = ctx_reserve(ctx, scan_scratch_bytes(n))) return rc;
  return launch_scan(ctx, data, dtype, n, exclusive, 0, static_cast<cudaStream_t>(stream));
}
