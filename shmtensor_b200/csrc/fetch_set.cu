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
      const bool valid = (int)lane < rows;
      const int64_t id = valid ? load_int(job.idx, job.idx64, first + lane) : kEmptyKey;
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
        } else if (job.host)
          p = job.host + id * job.row_bytes;
      }
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
// slot the map now holds for it.
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

static unsigned grid_for_tiles(int64_t n, int R) {
  const int64_t tiles = (n + R - 1) / R;
  int64_t blocks = (tiles + kRowWarps - 1) / kRowWarps;
  const int64_t cap = (int64_t)sm_count() * 256;
  if (blocks > cap) blocks = cap;
  return (unsigned)(blocks < 1 ? 1 : blocks);
}

template <bool SET>
static int launch_row_copy(const RowJob& job, int vec, cudaStream_t s) {
  const unsigned grid = grid_for_tiles(job.n, job.rows_per_tile);
  switch (vec) {
    case 16: row_copy_kernel<16, SET, 8><<<grid, kRowThreads, 0, s>>>(job); break;
    case 8: row_copy_kernel<8, SET, 8><<<grid, kRowThreads, 0, s>>>(job); break;
    case 4: row_copy_kernel<4, SET, 8><<<grid, kRowThreads, 0, s>>>(job); break;
    case 2: row_copy_kernel<2, SET, 8><<<grid, kRowThreads, 0, s>>>(job); break;
    default: row_copy_kernel<1, SET, 8><<<grid, kRowThreads, 0, s>>>(job); break;
  }
  SHMT_CUDA_TRY(cudaGetLastError());
  return SHMT_OK;
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

int shmt_fetch(const shmt_map* map, const void* mask, int mask_dtype, const void* host_base,
               const void* gpu_base, const void* idx, int idx_dtype, int64_t n, int64_t row_bytes,
               void* out, void* stream) {
  if (int rc = check_common("shmt_fetch", idx, idx_dtype, n, row_bytes)) return rc;
  if (n == 0) return SHMT_OK;
  SHMT_REQUIRE(out != nullptr, "shmt_fetch: out is null");
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
  const unsigned grid = grid_for_tiles(n, R);
  const int vec = pick_vec(row_bytes, {gpu_base, update});
  char* g = static_cast<char*>(gpu_base);
  const char* u = static_cast<const char*>(update);
  const int k64 = key_dtype == SHMT_I64, s64 = slots_dtype == SHMT_I64;
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
