// In-place prefix sum: one kernel, decoupled look-back between 2048-item tiles.
// Semantics follow cub_exclusiveSum (reference src/cache_graph_sampling.cu:30-45)
// and the intended meaning of thrust_scan (reference src/thrust_scan.cu:9-18,
// whose own lambda races); integer arithmetic wraps.
#include "ctx.cuh"
#include "lookback.cuh"

namespace shmt {

constexpr int kScanThreads = 256;
constexpr int kScanItems = 8;
constexpr int kScanTile = kScanThreads * kScanItems;

template <typename T>
__global__ void __launch_bounds__(kScanThreads)
scan_kernel(T* __restrict__ data, int64_t n, int exclusive, TileStates st, int64_t* words) {
  __shared__ int64_t warp_sums[32];
  __shared__ int64_t s_total;
  __shared__ int64_t s_prefix;
  __shared__ int s_tile;
  const int tile = take_tile(words + W_TICKET, &s_tile);
  const int64_t base = (int64_t)tile * kScanTile + (int64_t)threadIdx.x * kScanItems;

  T v[kScanItems];
  int64_t sum = 0;
#pragma unroll
  for (int j = 0; j < kScanItems; ++j) {
    v[j] = base + j < n ? data[base + j] : T(0);
    sum += (int64_t)v[j];
  }
  const int64_t local = block_exclusive_scan(sum, warp_sums, &s_total);
  if (threadIdx.x < 32) {
    const int64_t p = lookback_exclusive_prefix(st, tile, s_total, words + W_STATUS);
    if (threadIdx.x == 0) s_prefix = p;
  }
  __syncthreads();
  // unsigned accumulation: wrap-around is defined, and narrowing to T keeps the low bits
  uint64_t run = (uint64_t)(s_prefix + local);
#pragma unroll
  for (int j = 0; j < kScanItems; ++j) {
    if (base + j < n) {
      if (exclusive) {
        data[base + j] = (T)run;
        run += (uint64_t)(int64_t)v[j];
      } else {
        run += (uint64_t)(int64_t)v[j];
        data[base + j] = (T)run;
      }
    }
  }
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
  // status / result / ticket words and the tile flags start at zero
  SHMT_CUDA_TRY(cudaMemsetAsync(ctx->d_words(), 0, 256, stream));
  SHMT_CUDA_TRY(cudaMemsetAsync(st.flag, 0, (size_t)n_tiles * 4, stream));
  if (dtype == SHMT_I64)
    scan_kernel<long long><<<(unsigned)n_tiles, kScanThreads, 0, stream>>>(
        static_cast<long long*>(data), n, exclusive, st, ctx->d_words());
  else
    scan_kernel<int><<<(unsigned)n_tiles, kScanThreads, 0, stream>>>(
        static_cast<int*>(data), n, exclusive, st, ctx->d_words());
  SHMT_CUDA_TRY(cudaGetLastError());
  return SHMT_OK;
}

size_t scan_scratch_bytes(int64_t n) {
  const int64_t n_tiles = (n + kScanTile - 1) / kScanTile;
  return (tile_state_bytes(n_tiles > 0 ? n_tiles : 1) + 255) & ~(size_t)255;
}

// ---- scan without any allocation ----------------------------------------------------
// Look-back state for shmt_scan_static lives in this fixed array instead of context
// scratch.  Every GPU that loads the library carries it (about 160 KB) until exit.
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
  // the array still holds the previous call's ticket, status and tile flags: zero the
  // words and the flags this call will use (flags sit right behind the 256-byte header)
  SHMT_CUDA_TRY(cudaMemsetAsync(base, 0, 256 + (size_t)n_tiles * 4, s));
  if (dtype == SHMT_I64)
    scan_kernel<long long><<<(unsigned)n_tiles, kScanThreads, 0, s>>>(
        static_cast<long long*>(data), n, exclusive, st, words);
  else
    scan_kernel<int><<<(unsigned)n_tiles, kScanThreads, 0, s>>>(static_cast<int*>(data), n,
                                                                exclusive, st, words);
  SHMT_CUDA_TRY(cudaGetLastError());
  return SHMT_OK;
}

extern "C" int shmt_debug_lookback_timeout(shmt_ctx* ctx, void* stream) {
  SHMT_REQUIRE(ctx != nullptr, "shmt_debug_lookback_timeout: ctx is null");
  DeviceGuard guard(ctx->device);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (int rc = ctx_reserve(ctx, tile_state_bytes(2))) return rc;
  TileStates st = carve_tile_states(ctx->region(), 2);
  SHMT_CUDA_TRY(cudaMemsetAsync(ctx->scratch, 0, 256 + 2 * 4, s));
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
