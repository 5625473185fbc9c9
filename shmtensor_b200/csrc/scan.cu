// In-place prefix sum: one kernel, decoupled look-back between 64 KB tiles.
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
// load latency, local sums, look-back (a prefix crosses 32 tiles per round trip through L2 and
// ~100 tiles per microsecond are started), store.  This kernel takes the three longest waits off
// that path.  (1) The grid is persistent (every cluster resident at once, super-tiles dealt
// round-robin), so there is no ticket: a tile's predecessors belong to clusters that are
// running and only ever wait for still earlier tiles.  (2) A CTA's next tile is brought into
// shared memory by one bulk copy while the current one is summed, looked back and stored from
// registers, so load latency overlaps the rest.  (3) Four CTAs form a cluster, add their sums
// up through distributed shared memory and look back once for a 256 KB super-tile: a quarter of
// the descriptors per microsecond, so the nearest known prefix is one round trip away, not three.
#ifndef SHMT_SCAN_CLUSTER
#define SHMT_SCAN_CLUSTER 4
#endif
constexpr int kScanCluster = SHMT_SCAN_CLUSTER;
constexpr int64_t kScanSuperBytes = (int64_t)kScanCluster * kScanTileBytes;
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
// 8-byte store into the shared memory of CTA `rank` of this cluster, at the address `local`
// has in the calling CTA (same kernel, same layout).
__device__ __forceinline__ void st_cluster_u64(void* local, unsigned rank, unsigned long long v) {
  uint32_t remote;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(smem_addr(local)), "r"(rank));
  asm volatile("st.shared::cluster.u64 [%0], %1;" ::"r"(remote), "l"(v) : "memory");
}

template <typename T>
__global__ void __launch_bounds__(kScanThreads, 2)
scan_cluster_kernel(T* __restrict__ data, int64_t n_super, int exclusive, TileStates st, int64_t* words) {
  using U = typename ScanWord<T>::type;
  constexpr int VEC = 16 / (int)sizeof(T);
  constexpr int PER_LANE = kScanPartials / 32;
  extern __shared__ __align__(128) unsigned char landing[];  // one tile, filled by the bulk copy
  __shared__ U partial[kScanPartials];
  __shared__ unsigned long long s_sum[2][kScanCluster];  // CTA sums of the cluster, by iteration parity
  __shared__ int64_t s_prefix;
  __shared__ __align__(8) uint64_t s_bar;
  const unsigned full = 0xffffffffu;
  const unsigned tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const unsigned rank = cluster_ctarank();
  const int64_t n_clusters = cluster_count_x();
  char* bytes = reinterpret_cast<char*>(data);
  union Pack {
    uint4 q;
    U a[VEC];
  };

  if (tid == 0) mbar_init(&s_bar, 1);
  mbar_init_fence();
  __syncthreads();
  cluster_sync_all();  // every CTA of the cluster is running before anyone writes into its memory

  int64_t super = cluster_id_x();
  if (tid == 0 && super < n_super) {
    mbar_arrive_expect_tx(&s_bar, kScanTileBytes);
    bulk_load(landing, bytes + (super * kScanCluster + rank) * kScanTileBytes, kScanTileBytes, &s_bar);
  }
  uint32_t phase = 0;
  for (int it = 0; super < n_super; super += n_clusters, ++it) {
    if (!mbar_wait_bounded(&s_bar, phase))
      atomicMax(reinterpret_cast<unsigned long long*>(words + W_STATUS), (unsigned long long)DEV_TIMEOUT);
    phase ^= 1u;
    U v[kScanVecs][VEC], vsum[kScanVecs], inc[kScanVecs];
#pragma unroll
    for (int k = 0; k < kScanVecs; ++k) {
      Pack p;
      p.q = reinterpret_cast<const uint4*>(landing)[k * kScanThreads + tid];
#pragma unroll
      for (int j = 0; j < VEC; ++j) v[k][j] = p.a[j];
    }
    __syncthreads();  // the tile is in registers: the landing buffer is free, `partial` too
    const int64_t next = super + n_clusters;
    if (tid == 0 && next < n_super) {
      mbar_arrive_expect_tx(&s_bar, kScanTileBytes);
      bulk_load(landing, bytes + (next * kScanCluster + rank) * kScanTileBytes, kScanTileBytes, &s_bar);
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
      const U total = __shfl_sync(full, linc, 31);
      // this CTA's sum to every CTA of the cluster (its own copy included)
      if (lane < kScanCluster) st_cluster_u64(&s_sum[it & 1][rank], lane, (unsigned long long)total);
    }
#ifdef SHMT_DBG_NO_CLUSTER_BARRIER
    __syncthreads();
#else
    cluster_sync_all();  // sums delivered; also the CTA-wide barrier behind `partial`
#endif
    if (warp == 0) {
      unsigned long long before = 0, whole = 0;
#pragma unroll
      for (int r = 0; r < kScanCluster; ++r) {
        const unsigned long long t = s_sum[it & 1][r];
        whole += t;
        if ((unsigned)r < rank) before += t;
      }
#ifdef SHMT_DBG_NO_LOOKBACK
      const int64_t p = 0;
#else
      const int64_t p = rank == 0
          ? lookback_exclusive_prefix_shared<true>(st, (int)super, (int64_t)whole, words + W_STATUS)
          : lookback_exclusive_prefix_shared<false>(st, (int)super, (int64_t)whole, words + W_STATUS);
#endif
      if (lane == 0) s_prefix = p + (int64_t)before;
    }
    __syncthreads();
    const U prefix = (U)(uint64_t)s_prefix;
    T* out = data + (super * kScanCluster + rank) * (kScanTileBytes / (int64_t)sizeof(T));
#pragma unroll
    for (int k = 0; k < kScanVecs; ++k) {
      const U ahead = prefix + partial[k * kScanWarps + warp] + (inc[k] - vsum[k]);
      Pack p;
#pragma unroll
      for (int j = 0; j < VEC; ++j)
        p.a[j] = ahead + (exclusive ? (j ? v[k][j - 1] : U(0)) : v[k][j]);
#ifdef SHMT_DBG_NO_STORE
      if (p.a[0] == (U)0x12345678) reinterpret_cast<uint4*>(out)[k * kScanThreads + tid] = p.q;
#else
      reinterpret_cast<uint4*>(out)[k * kScanThreads + tid] = p.q;
#endif
    }
  }
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
                                       kScanTileBytes));
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(kScanCluster * 64);
    cfg.blockDim = dim3(kScanThreads);
    cfg.dynamicSmemBytes = kScanTileBytes;
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
  cfg.blockDim = dim3(kScanThreads);
  cfg.dynamicSmemBytes = kScanTileBytes;
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
  // status / result / ticket words and the tile descriptors start at zero
  SHMT_CUDA_TRY(cudaMemsetAsync(ctx->d_words(), 0, 256, stream));
  SHMT_CUDA_TRY(cudaMemsetAsync(st.d, 0, tile_state_bytes(n_tiles), stream));
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
