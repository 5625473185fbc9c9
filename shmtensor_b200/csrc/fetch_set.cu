// Fused probe + row gather (fetch) and probe + row scatter (set / insert-set).
//
// One warp owns a tile of R consecutive requests.  Phase A: one request per
// lane -- load the id, resolve its row address (cooperative map probe, caller's
// mask, or plain host row) and park the address in shared memory.  Phase B: the
// tile's rows are treated as one flat list of VEC-byte chunks that the 32 lanes
// stride through, U chunks per lane in flight before the first is used.  The
// request side of the copy (the output of a fetch, the update of a set) is
// contiguous over the whole tile; the table side jumps from row to row.  All
// lanes stay busy whatever the row size (400-byte rows are 25 chunks, not a
// multiple of 32), and loads that cross the host link or NVLink overlap with
// HBM loads of the same batch.
//
// Replaces the reference's six fetch and six set kernels
// (src/cache_feature_fetch.cu:15-45,89-129,188-224;
//  src/cache_feature_set.cu:6-37,77-116,167-207), which walk 32 rows per warp one
// after another with 4-byte accesses and probe the map redundantly on 32 lanes.
#include <stdlib.h>

#include "bulk.cuh"
#include "ctx.cuh"
#include "map.cuh"

namespace shmt {

constexpr int kRowThreads = 256;
constexpr int kRowWarps = kRowThreads / 32;
constexpr int kMaxBases = 16;

enum : int { MODE_HOST = 0, MODE_MAP = 1, MODE_MASK = 2 };

struct RowJob {
  MapView map;
  const void* mask;
  int mask64;
  int mode;
  char* host;             // host table (UVA) or nullptr
  char* bases[kMaxBases]; // cached-row buffers: [0] local; more for a partitioned cache
  int owner_shift;        // value = (owner << owner_shift) | slot
  const void* idx;
  int idx64;
  int64_t n;
  int64_t row_bytes;
  char* flat;             // fetch: output; set: update rows (request order)
  int rows_per_tile;      // R, 1..32
};

template <int VEC> struct VecT;
template <> struct VecT<16> { using type = uint4; };
template <> struct VecT<8> { using type = uint2; };
template <> struct VecT<4> { using type = uint32_t; };
template <> struct VecT<2> { using type = uint16_t; };
template <> struct VecT<1> { using type = uint8_t; };

template <int VEC>
__device__ __forceinline__ typename VecT<VEC>::type load_chunk(const char* p) {
  return __ldg(reinterpret_cast<const typename VecT<VEC>::type*>(p));
}
template <>
__device__ __forceinline__ uint4 load_chunk<16>(const char* p) {
  return ld_stream16(p);
}
template <int VEC>
__device__ __forceinline__ void store_chunk(char* p, typename VecT<VEC>::type v) {
  *reinterpret_cast<typename VecT<VEC>::type*>(p) = v;
}
template <>
__device__ __forceinline__ void store_chunk<16>(char* p, uint4 v) {
  st_stream16(p, v);
}

// Row address of request `first + lane` of a tile (nullptr: nothing to copy).
// All 32 lanes must call: the map probe is cooperative.
__device__ __forceinline__ int64_t load_id(const RowJob& job, int64_t first, int rows,
                                            unsigned lane) {
  return (int)lane < rows ? load_int(job.idx, job.idx64, first + lane) : kEmptyKey;
}

__device__ __forceinline__ char* resolve_row(const RowJob& job, int64_t first, int rows,
                                             unsigned lane, int64_t slot_mask, int64_t id) {
  const bool valid = (int)lane < rows;
  int64_t v = -1;
  if (job.mode == MODE_MAP)
    v = warp_find(job.map, id, valid);
  else if (job.mode == MODE_MASK)
    v = valid ? load_int(job.mask, job.mask64, first + lane) : -1;
  char* p = nullptr;
  if (valid) {
    if (v >= 0) {
      char* base = job.bases[v >> job.owner_shift];
      if (base) p = base + (v & slot_mask) * job.row_bytes;
    } else if (job.host) {
      p = job.host + id * job.row_bytes;
    }
  }
  return p;
}

// Set by a kernel whose bounded wait ran out; read (and cleared) by shmt_device_fault().
__device__ int g_device_fault = 0;

// Fetch through the TMA unit: rows never pass through registers.  Per warp, a ring
// of STAGES shared-memory buffers of R rows each (about 2 KB): every lane of a tile
// issues one bulk copy (row -> its slot of the buffer) that completes on the stage's
// mbarrier; the whole buffer then leaves with ONE bulk store, because the tile's
// rows are contiguous in the output.  While a stage's loads are in flight the warp
// already probes the map for the tile after it and issues those loads.  Tiles are
// dealt round-robin over a persistent grid, so neighbouring warps write
// neighbouring pieces of the output at about the same time.
template <int STAGES>
__global__ void __launch_bounds__(kRowThreads)
row_gather_bulk_kernel(const RowJob job) {
  extern __shared__ __align__(128) unsigned char smem_raw[];
  __shared__ __align__(8) uint64_t s_bar[kRowWarps][STAGES];
  const unsigned lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int R = job.rows_per_tile;
  const uint32_t rb = (uint32_t)job.row_bytes;
  const uint32_t stage_bytes = (uint32_t)R * rb;
  unsigned char* wbase = smem_raw + (size_t)warp * STAGES * stage_bytes;
  const int64_t n_tiles = (job.n + R - 1) / R;
  const int64_t stride = (int64_t)gridDim.x * kRowWarps;
  const int64_t slot_mask = ((int64_t)1 << job.owner_shift) - 1;

  if (lane == 0)
    for (int s = 0; s < STAGES; ++s) mbar_init(&s_bar[warp][s], 1);
  mbar_init_fence();
  __syncwarp();

  unsigned vmask[STAGES];  // lanes whose row is being loaded into the stage
  int nrows[STAGES];
  uint32_t parity = 0;     // bit s: phase of stage s to wait for next

  auto issue = [&](int64_t tile, int s) {
    const int64_t first = tile * R;
    const int rows = (int)min((int64_t)R, job.n - first);
    const int64_t id = load_id(job, first, rows, lane);
    char* p = resolve_row(job, first, rows, lane, slot_mask, id);
    const unsigned vm = __ballot_sync(0xffffffffu, p != nullptr);
    if (lane == 0) mbar_arrive_expect_tx(&s_bar[warp][s], (uint32_t)__popc(vm) * rb);
    if (p) bulk_load(wbase + (size_t)s * stage_bytes + (size_t)lane * rb, p, rb, &s_bar[warp][s]);
    vmask[s] = vm;
    nrows[s] = rows;
  };

  // D = STAGES - 1 tiles of loads are in flight while the oldest stage drains its store
  constexpr int D = STAGES - 1;
  int64_t tile = (int64_t)blockIdx.x * kRowWarps + warp;
  bool ok = true;
#pragma unroll
  for (int j = 0; j < D; ++j)
    if (tile + j * stride < n_tiles) issue(tile + j * stride, j);
  while (tile < n_tiles && ok) {
#pragma unroll
    for (int s = 0; s < STAGES; ++s) {
      if (tile >= n_tiles || !ok) break;
      const int64_t ahead = tile + D * stride;
      if (ahead < n_tiles) {
        bulk_wait_read<0>();  // the store that last used that stage no longer reads it
        __syncwarp();
        issue(ahead, (s + D) % STAGES);
      }
      // every lane polls: measured faster than one polling lane plus a vote, and fetching
      // the ids a tile ahead of their probe measured slower than loading them here
      if (!mbar_wait_bounded(&s_bar[warp][s], (parity >> s) & 1u)) {
        atomicExch(&g_device_fault, 1);
        ok = false;
      }
      ok = __all_sync(0xffffffffu, ok);
      parity ^= 1u << s;
      if (ok) {
        unsigned char* buf = wbase + (size_t)s * stage_bytes;
        char* dst = job.flat + tile * R * job.row_bytes;
        const unsigned vm = vmask[s];
        async_proxy_fence();
        if (__popc(vm) == nrows[s]) {
          if (lane == 0 && vm) bulk_store(dst, buf, (uint32_t)nrows[s] * rb);
        } else if ((vm >> lane) & 1u) {
          bulk_store(dst + (size_t)lane * rb, buf + (size_t)lane * rb, rb);
        }
        bulk_commit();
      }
      tile += stride;
    }
  }
  bulk_wait_read<0>();  // shared memory must outlive the stores that read it
}

// The mirror image for set: the tile's update rows are contiguous, so ONE bulk load brings
// them into the stage buffer; each lane then stores its row to where the probe sent it (the
// cached copy on a hit, the host table on a miss) with its own bulk store.
template <int STAGES>
__global__ void __launch_bounds__(kRowThreads)
row_scatter_bulk_kernel(const RowJob job) {
  extern __shared__ __align__(128) unsigned char smem_raw[];
  __shared__ __align__(8) uint64_t s_bar[kRowWarps][STAGES];
  const unsigned lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int R = job.rows_per_tile;
  const uint32_t rb = (uint32_t)job.row_bytes;
  const uint32_t stage_bytes = (uint32_t)R * rb;
  unsigned char* wbase = smem_raw + (size_t)warp * STAGES * stage_bytes;
  const int64_t n_tiles = (job.n + R - 1) / R;
  const int64_t stride = (int64_t)gridDim.x * kRowWarps;
  const int64_t slot_mask = ((int64_t)1 << job.owner_shift) - 1;

  if (lane == 0)
    for (int s = 0; s < STAGES; ++s) mbar_init(&s_bar[warp][s], 1);
  mbar_init_fence();
  __syncwarp();

  char* dst_row[STAGES];  // where this lane's row of the stage goes (nullptr: nowhere)
  uint32_t parity = 0;

  auto issue = [&](int64_t tile, int s) {
    const int64_t first = tile * R;
    const int rows = (int)min((int64_t)R, job.n - first);
    dst_row[s] = resolve_row(job, first, rows, lane, slot_mask, load_id(job, first, rows, lane));
    if (lane == 0) {
      mbar_arrive_expect_tx(&s_bar[warp][s], (uint32_t)rows * rb);
      bulk_load(wbase + (size_t)s * stage_bytes, job.flat + first * job.row_bytes, (uint32_t)rows * rb,
                &s_bar[warp][s]);
    }
  };

  constexpr int D = STAGES - 1;
  int64_t tile = (int64_t)blockIdx.x * kRowWarps + warp;
  bool ok = true;
#pragma unroll
  for (int j = 0; j < D; ++j)
    if (tile + j * stride < n_tiles) issue(tile + j * stride, j);
  while (tile < n_tiles && ok) {
#pragma unroll
    for (int s = 0; s < STAGES; ++s) {
      if (tile >= n_tiles || !ok) break;
      const int64_t ahead = tile + D * stride;
      if (ahead < n_tiles) {
        bulk_wait_read<0>();  // every lane's store out of that stage has read it
        __syncwarp();
        issue(ahead, (s + D) % STAGES);
      }
      if (!mbar_wait_bounded(&s_bar[warp][s], (parity >> s) & 1u)) {
        atomicExch(&g_device_fault, 1);
        ok = false;
      }
      ok = __all_sync(0xffffffffu, ok);
      parity ^= 1u << s;
      if (ok) {
        async_proxy_fence();
        if (dst_row[s])
          bulk_store(dst_row[s], wbase + (size_t)s * stage_bytes + (size_t)lane * rb, rb);
        bulk_commit();
      }
      tile += stride;
    }
  }
  bulk_wait_read<0>();
}

// SET == false: table row -> flat (fetch).  SET == true: flat -> table row.
template <int VEC, bool SET, int U>
__global__ void __launch_bounds__(kRowThreads) row_copy_kernel(const RowJob job) {
  using V = typename VecT<VEC>::type;
  __shared__ char* s_row[kRowWarps][32];
  const unsigned lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int R = job.rows_per_tile;
  const int64_t n_tiles = (job.n + R - 1) / R;
  const uint32_t cpr = (uint32_t)(job.row_bytes / VEC);  // chunks per row
  const uint32_t step_row = 32u / cpr, step_off = 32u % cpr;
  const int64_t slot_mask = ((int64_t)1 << job.owner_shift) - 1;

  for (int64_t tile = (int64_t)blockIdx.x * kRowWarps + warp; tile < n_tiles;
       tile += (int64_t)gridDim.x * kRowWarps) {
    const int64_t first = tile * R;
    const int rows = (int)min((int64_t)R, job.n - first);

    // ---- phase A: one request per lane -> row address
    {
      char* p = resolve_row(job, first, rows, lane, slot_mask, load_id(job, first, rows, lane));
      __syncwarp();  // previous tile's readers are done with s_row
      s_row[warp][lane] = p;
      __syncwarp();
    }

    // ---- phase B: flat chunk copy
    const uint32_t total = (uint32_t)rows * cpr;
    char* flat = job.flat + first * job.row_bytes;
    uint32_t row = lane / cpr, off = lane % cpr;
    for (uint32_t c0 = 0; c0 < total; c0 += 32u * U) {
      V v[U];
      char* tp[U];
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const uint32_t c = c0 + u * 32u + lane;
        tp[u] = nullptr;
        if (c < total) {
          char* base = s_row[warp][row];
          if (base) tp[u] = base + (size_t)off * VEC;
        }
        if (tp[u]) v[u] = load_chunk<VEC>(SET ? flat + (size_t)c * VEC : tp[u]);
        off += step_off;
        row += step_row;
        if (off >= cpr) {
          off -= cpr;
          ++row;
        }
      }
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const uint32_t c = c0 + u * 32u + lane;
        if (tp[u]) store_chunk<VEC>(SET ? tp[u] : flat + (size_t)c * VEC, v[u]);
      }
    }
  }
}

// Fused insert/overwrite: probe-or-claim the key, then write the row to the
// slot the map now holds for it.  (80 registers, 3 CTAs per SM: forcing 4 CTAs with 64
// registers measured 4 % slower on 4,000,000 keys x 512 bytes.)
template <int VEC, int U>
__global__ void __launch_bounds__(kRowThreads)
insert_set_kernel(MapView map, char* gpu_base, const void* keys, int keys64, const void* slots,
                  int slots64, int64_t n, int64_t row_bytes, const char* update, int R,
                  int64_t* meta) {
  using V = typename VecT<VEC>::type;
  __shared__ char* s_row[kRowWarps][32];
  const unsigned lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int64_t n_tiles = (n + R - 1) / R;
  const uint32_t cpr = (uint32_t)(row_bytes / VEC);
  const uint32_t step_row = 32u / cpr, step_off = 32u % cpr;
  int64_t total_new = 0;

  for (int64_t tile = (int64_t)blockIdx.x * kRowWarps + warp; tile < n_tiles;
       tile += (int64_t)gridDim.x * kRowWarps) {
    const int64_t first = tile * R;
    const int rows = (int)min((int64_t)R, n - first);
    {
      const bool valid = (int)lane < rows;
      const int64_t k = valid ? load_int(keys, keys64, first + lane) : kEmptyKey;
      const int64_t want = valid ? load_int(slots, slots64, first + lane) : -1;
      int n_new = 0;
      const int64_t got = warp_insert(map, k, want, valid, /*assign=*/false, meta, &n_new);
      total_new += n_new;
      __syncwarp();
      s_row[warp][lane] = (valid && got >= 0) ? gpu_base + got * row_bytes : nullptr;
      __syncwarp();
    }
    const uint32_t total = (uint32_t)rows * cpr;
    const char* flat = update + first * row_bytes;
    uint32_t row = lane / cpr, off = lane % cpr;
    for (uint32_t c0 = 0; c0 < total; c0 += 32u * U) {
      V v[U];
      char* tp[U];
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const uint32_t c = c0 + u * 32u + lane;
        tp[u] = nullptr;
        if (c < total) {
          char* base = s_row[warp][row];
          if (base) tp[u] = base + (size_t)off * VEC;
        }
        if (tp[u]) v[u] = load_chunk<VEC>(flat + (size_t)c * VEC);
        off += step_off;
        row += step_row;
        if (off >= cpr) {
          off -= cpr;
          ++row;
        }
      }
#pragma unroll
      for (int u = 0; u < U; ++u)
        if (tp[u]) store_chunk<VEC>(tp[u], v[u]);
    }
  }
  if (lane == 0 && total_new)
    atomicAdd(reinterpret_cast<unsigned long long*>(meta + 1), (unsigned long long)total_new);
}

// ---- host side ---------------------------------------------------------------

static int pick_vec(int64_t row_bytes, std::initializer_list<const void*> ptrs) {
  uintptr_t bits = (uintptr_t)row_bytes;
  for (const void* p : ptrs) bits |= (uintptr_t)p;
  if ((bits & 15) == 0) return 16;
  if ((bits & 7) == 0) return 8;
  if ((bits & 3) == 0) return 4;
  if ((bits & 1) == 0) return 2;
  return 1;
}

// Rows per warp tile: 32 when there is enough work to fill the GPU, fewer for
// small batches so that they still spread over all SMs.
static int pick_rows_per_tile(int64_t n) {
  const int64_t warps_wanted = (int64_t)sm_count() * 32;
  int r = 32;
  while (r > 1 && (n + r - 1) / r < warps_wanted) r >>= 1;
  return r;
}

// Persistent grid: never more CTAs than are resident at once (tiles are dealt round-robin
// inside the kernels), so there is no partly filled last wave.
template <typename Kernel>
static unsigned grid_for_tiles(Kernel kernel, int64_t n, int R, size_t smem = 0) {
  const int64_t tiles = (n + R - 1) / R;
  int64_t blocks = (tiles + kRowWarps - 1) / kRowWarps;
  int occ = 1;
  if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&occ, kernel, kRowThreads, smem) != cudaSuccess ||
      occ < 1)
    occ = 1;
  const int64_t resident = (int64_t)sm_count() * occ;
  if (blocks > resident) blocks = resident;
  return (unsigned)(blocks < 1 ? 1 : blocks);
}

template <int VEC, bool SET>
static int launch_lsu(const RowJob& job, cudaStream_t s) {
  const unsigned grid = grid_for_tiles(row_copy_kernel<VEC, SET, 8>, job.n, job.rows_per_tile);
  row_copy_kernel<VEC, SET, 8><<<grid, kRowThreads, 0, s>>>(job);
  SHMT_CUDA_TRY(cudaGetLastError());
  return SHMT_OK;
}

// Ring geometry of the bulk path: two buffers per warp of about 2 KB each (5 rows of
// 400 bytes, 4 of 512): measured best on B200 among 0.5 .. 12 KB buffers and 2 .. 4 stages.
constexpr int kBulkStages = 2;
constexpr int64_t kBulkStageBytes = 2048;
constexpr size_t kBulkSmemMax = 200 * 1024;

// Rows per ring buffer, 0 if the rows are not 16-byte units or do not fit.
static int bulk_rows_per_stage(int64_t row_bytes, int vec, int R_small) {
  if (vec != 16) return 0;
  static const int forced = [] {
    const char* e = getenv("SHMT_BULK_ROWS");
    return e ? atoi(e) : 0;
  }();
  int64_t r = forced > 0 ? forced : kBulkStageBytes / row_bytes;
  if (r < 1) r = 1;
  if (r > 32) r = 32;
  if (r > R_small) r = R_small;
  if ((size_t)kRowWarps * kBulkStages * r * row_bytes > kBulkSmemMax) return 0;
  return (int)r;
}

template <bool SET>
static int launch_bulk(RowJob job, int R, cudaStream_t s) {
  auto kernel = SET ? row_scatter_bulk_kernel<kBulkStages> : row_gather_bulk_kernel<kBulkStages>;
  static bool configured[64] = {false};
  int dev = 0;
  SHMT_CUDA_TRY(cudaGetDevice(&dev));
  if (dev < 64 && !configured[dev]) {
    SHMT_CUDA_TRY(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       (int)kBulkSmemMax));
    configured[dev] = true;
  }
  job.rows_per_tile = R;
  const size_t smem = (size_t)kRowWarps * kBulkStages * R * job.row_bytes;
  const unsigned blocks = grid_for_tiles(kernel, job.n, R, smem);
  kernel<<<blocks, kRowThreads, smem, s>>>(job);
  SHMT_CUDA_TRY(cudaGetLastError());
  return SHMT_OK;
}

template <bool SET>
static int launch_row_copy(const RowJob& job, int vec, cudaStream_t s) {
  {
    static const bool no_bulk = getenv("SHMT_NO_BULK") != nullptr;
    const int R = no_bulk ? 0 : bulk_rows_per_stage(job.row_bytes, vec, job.rows_per_tile);
    if (R >= 1) return launch_bulk<SET>(job, R, s);
  }
  switch (vec) {
    case 16: return launch_lsu<16, SET>(job, s);
    case 8: return launch_lsu<8, SET>(job, s);
    case 4: return launch_lsu<4, SET>(job, s);
    case 2: return launch_lsu<2, SET>(job, s);
    default: return launch_lsu<1, SET>(job, s);
  }
}

static int check_common(const char* who, const void* idx, int idx_dtype, int64_t n,
                        int64_t row_bytes) {
  SHMT_REQUIRE(valid_int_dtype(idx_dtype), "%s: indices can only be int32 or int64", who);
  SHMT_REQUIRE(n >= 0, "%s: negative count", who);
  SHMT_REQUIRE(row_bytes > 0 && row_bytes < ((int64_t)1 << 26),
               "%s: row_bytes %lld out of range (1 .. 64 MiB)", who, (long long)row_bytes);
  SHMT_REQUIRE(n == 0 || idx != nullptr, "%s: indices are null", who);
  return SHMT_OK;
}

static int fill_mode(const char* who, RowJob& job, const shmt_map* map, const void* mask,
                     int mask_dtype) {
  job.map = view_of(map);
  job.mask = mask;
  job.mask64 = mask_dtype == SHMT_I64;
  if (map) {
    SHMT_REQUIRE(mask == nullptr, "%s: give a map or a mask, not both", who);
    job.mode = MODE_MAP;
  } else if (mask) {
    SHMT_REQUIRE(valid_int_dtype(mask_dtype), "%s: mask can only be int32 or int64", who);
    job.mode = MODE_MASK;
  } else {
    job.mode = MODE_HOST;
  }
  return SHMT_OK;
}

}  // namespace shmt

using namespace shmt;

extern "C" {

int shmt_device_fault(int* out_code) {
  SHMT_REQUIRE(out_code != nullptr, "shmt_device_fault: out_code is null");
  int code = 0, zero = 0;
  SHMT_CUDA_TRY(cudaMemcpyFromSymbol(&code, g_device_fault, sizeof(int)));
  if (code) SHMT_CUDA_TRY(cudaMemcpyToSymbol(g_device_fault, &zero, sizeof(int)));
  *out_code = code;
  return SHMT_OK;
}

int shmt_fetch(const shmt_map* map, const void* mask, int mask_dtype, const void* host_base,
               const void* gpu_base, const void* idx, int idx_dtype, int64_t n, int64_t row_bytes,
               void* out, void* stream) {
  if (int rc = check_common("shmt_fetch", idx, idx_dtype, n, row_bytes)) return rc;
  if (n == 0) return SHMT_OK;
  SHMT_REQUIRE(out != nullptr, "shmt_fetch: out is null");
  DeviceGuard guard(map ? map->device : device_of_pointer(out));
  RowJob job{};
  if (int rc = fill_mode("shmt_fetch", job, map, mask, mask_dtype)) return rc;
  SHMT_REQUIRE(job.mode == MODE_HOST ? host_base != nullptr : (gpu_base || host_base),
               "shmt_fetch: the table pointer this mode reads is null");
  job.host = static_cast<char*>(const_cast<void*>(host_base));
  job.bases[0] = static_cast<char*>(const_cast<void*>(gpu_base));
  job.owner_shift = 62;
  job.idx = idx;
  job.idx64 = idx_dtype == SHMT_I64;
  job.n = n;
  job.row_bytes = row_bytes;
  job.flat = static_cast<char*>(out);
  job.rows_per_tile = pick_rows_per_tile(n);
  const int vec = pick_vec(row_bytes, {host_base, gpu_base, out});
  return launch_row_copy<false>(job, vec, static_cast<cudaStream_t>(stream));
}

int shmt_fetch_partitioned(const shmt_map* map, const void* const* bases, int n_bases,
                           int owner_shift, const void* host_base, const void* idx, int idx_dtype,
                           int64_t n, int64_t row_bytes, void* out, void* stream) {
  if (int rc = check_common("shmt_fetch_partitioned", idx, idx_dtype, n, row_bytes)) return rc;
  SHMT_REQUIRE(map != nullptr, "shmt_fetch_partitioned: map is null");
  SHMT_REQUIRE(bases != nullptr && n_bases >= 1 && n_bases <= kMaxBases,
               "shmt_fetch_partitioned: 1..%d row buffers", kMaxBases);
  SHMT_REQUIRE(owner_shift >= 1 && owner_shift <= 62, "shmt_fetch_partitioned: owner_shift 1..62");
  if (n == 0) return SHMT_OK;
  SHMT_REQUIRE(out != nullptr, "shmt_fetch_partitioned: out is null");
  DeviceGuard guard(map->device);
  RowJob job{};
  job.map = view_of(map);
  job.mode = MODE_MAP;
  job.host = static_cast<char*>(const_cast<void*>(host_base));
  uintptr_t align = 0;
  for (int g = 0; g < n_bases; ++g) {
    SHMT_REQUIRE(bases[g] != nullptr, "shmt_fetch_partitioned: row buffer %d is null", g);
    job.bases[g] = static_cast<char*>(const_cast<void*>(bases[g]));
    align |= (uintptr_t)bases[g];
  }
  // a value naming an owner beyond n_bases reads bases[0]; owners are the caller's contract
  for (int g = n_bases; g < kMaxBases; ++g) job.bases[g] = job.bases[0];
  job.owner_shift = owner_shift;
  job.idx = idx;
  job.idx64 = idx_dtype == SHMT_I64;
  job.n = n;
  job.row_bytes = row_bytes;
  job.flat = static_cast<char*>(out);
  job.rows_per_tile = pick_rows_per_tile(n);
  const int vec = pick_vec(row_bytes, {host_base, (const void*)align, out});
  return launch_row_copy<false>(job, vec, static_cast<cudaStream_t>(stream));
}

int shmt_set(const shmt_map* map, const void* mask, int mask_dtype, void* host_base,
             void* gpu_base, const void* idx, int idx_dtype, int64_t n, int64_t row_bytes,
             const void* update, void* stream) {
  if (int rc = check_common("shmt_set", idx, idx_dtype, n, row_bytes)) return rc;
  if (n == 0) return SHMT_OK;
  SHMT_REQUIRE(update != nullptr, "shmt_set: update is null");
  DeviceGuard guard(map ? map->device : device_of_pointer(update));
  RowJob job{};
  if (int rc = fill_mode("shmt_set", job, map, mask, mask_dtype)) return rc;
  SHMT_REQUIRE(job.mode == MODE_HOST ? host_base != nullptr : (gpu_base || host_base),
               "shmt_set: the table pointer this mode writes is null");
  job.host = static_cast<char*>(host_base);
  job.bases[0] = static_cast<char*>(gpu_base);
  job.owner_shift = 62;
  job.idx = idx;
  job.idx64 = idx_dtype == SHMT_I64;
  job.n = n;
  job.row_bytes = row_bytes;
  job.flat = static_cast<char*>(const_cast<void*>(update));
  job.rows_per_tile = pick_rows_per_tile(n);
  const int vec = pick_vec(row_bytes, {host_base, gpu_base, update});
  return launch_row_copy<true>(job, vec, static_cast<cudaStream_t>(stream));
}

int shmt_insert_set(shmt_map* map, void* gpu_base, const void* keys, int key_dtype,
                    const void* slots, int slots_dtype, int64_t n, int64_t row_bytes,
                    const void* update, void* stream) {
  if (int rc = check_common("shmt_insert_set", keys, key_dtype, n, row_bytes)) return rc;
  SHMT_REQUIRE(map != nullptr, "shmt_insert_set: map is null");
  SHMT_REQUIRE(valid_int_dtype(slots_dtype), "shmt_insert_set: slots can only be int32 or int64");
  if (n == 0) return SHMT_OK;
  SHMT_REQUIRE(gpu_base && slots && update, "shmt_insert_set: gpu_base/slots/update are null");
  DeviceGuard guard(map->device);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int R = pick_rows_per_tile(n);
  const unsigned grid = grid_for_tiles(insert_set_kernel<16, 8>, n, R);
  const int vec = pick_vec(row_bytes, {gpu_base, update});
  char* g = static_cast<char*>(gpu_base);
  const char* u = static_cast<const char*>(update);
  const int k64 = key_dtype == SHMT_I64, s64 = slots_dtype == SHMT_I64;
  // the status word reports on this call only (see shmt_map_insert)
  SHMT_CUDA_TRY(cudaMemsetAsync(map->d_meta, 0, sizeof(int64_t), s));
  switch (vec) {
    case 16: insert_set_kernel<16, 8><<<grid, kRowThreads, 0, s>>>(map->view, g, keys, k64, slots, s64, n, row_bytes, u, R, map->d_meta); break;
    case 8: insert_set_kernel<8, 8><<<grid, kRowThreads, 0, s>>>(map->view, g, keys, k64, slots, s64, n, row_bytes, u, R, map->d_meta); break;
    case 4: insert_set_kernel<4, 8><<<grid, kRowThreads, 0, s>>>(map->view, g, keys, k64, slots, s64, n, row_bytes, u, R, map->d_meta); break;
    case 2: insert_set_kernel<2, 8><<<grid, kRowThreads, 0, s>>>(map->view, g, keys, k64, slots, s64, n, row_bytes, u, R, map->d_meta); break;
    default: insert_set_kernel<1, 8><<<grid, kRowThreads, 0, s>>>(map->view, g, keys, k64, slots, s64, n, row_bytes, u, R, map->d_meta); break;
  }
  SHMT_CUDA_TRY(cudaGetLastError());
  int64_t meta[2] = {0, 0};
  SHMT_CUDA_TRY(cudaMemcpyAsync(meta, map->d_meta, sizeof(meta), cudaMemcpyDeviceToHost, s));
  SHMT_CUDA_TRY(cudaStreamSynchronize(s));
  map->size = meta[1];
  if (meta[0] == DEV_OVERFLOW) {
    set_error("shmt_insert_set: table overflow (%lld keys stored, capacity %lld)",
              (long long)meta[1], (long long)map->capacity);
    return SHMT_ERR_CAPACITY;
  }
  return SHMT_OK;
}

}  // extern "C"
