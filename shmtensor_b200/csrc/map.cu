// Static hashmap: creation, bulk insert_or_assign, bulk query, bulk erase.
// Replaces pycuco::CUCOHashmap / CUCOHashmapWrapper of the reference
// (include/cuco_hashmap.cuh:49-93, src/cuco_hashmap.cu:10-41).
#include "ctx.cuh"
#include "map.cuh"

namespace shmt {

constexpr int kMapThreads = 256;

__global__ void __launch_bounds__(kMapThreads)
map_insert_kernel(MapView m, const void* __restrict__ keys, int keys64,
                  const void* __restrict__ vals, int vals64, int64_t n, int64_t* meta) {
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  int added = 0;
  bool overflow = false;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride)
    added += thread_insert(m, load_int(keys, keys64, i), load_int(vals, vals64, i), /*assign=*/true,
                           &overflow);
  // one atomic per warp for the key count
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) added += __shfl_xor_sync(0xffffffffu, added, o);
  if ((threadIdx.x & 31) == 0 && added)
    atomicAdd(reinterpret_cast<unsigned long long*>(meta + 1), (unsigned long long)added);
  if (overflow)
    atomicMax(reinterpret_cast<unsigned long long*>(meta), (unsigned long long)DEV_OVERFLOW);
}

__global__ void __launch_bounds__(kMapThreads)
map_erase_kernel(MapView m, const void* __restrict__ keys, int keys64, int64_t n,
                 void* __restrict__ out, int out64, int64_t* meta) {
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  int removed = 0;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
    const int64_t v = thread_erase(m, load_int(keys, keys64, i));
    removed += v >= 0;
    if (out) store_int(out, out64, i, v);
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) removed += __shfl_xor_sync(0xffffffffu, removed, o);
  if ((threadIdx.x & 31) == 0 && removed)
    atomicAdd(reinterpret_cast<unsigned long long*>(meta + 1), 0ULL - (unsigned long long)removed);
}

// Lookups are a chain of dependent reads (id, home window, now and then a further window), so
// what counts is how many warps are resident: 8 CTAs per SM (32 registers, a few spilled words)
// gave 8 % more lookups/s at 1,000,000 keys and 17 % more at 4,000,000 than the 4 the compiler picks.
#ifndef SHMT_QUERY_CTAS
#define SHMT_QUERY_CTAS 8
#endif
__global__ void __launch_bounds__(kMapThreads, SHMT_QUERY_CTAS)
map_query_kernel(MapView m, const void* __restrict__ req, int req64, int64_t n,
                 void* __restrict__ out, int out64) {
  const int64_t warp = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int64_t n_warps = ((int64_t)gridDim.x * blockDim.x) >> 5;
  const unsigned lane = threadIdx.x & 31;
  const int64_t n_batches = (n + 31) >> 5;
  for (int64_t b = warp; b < n_batches; b += n_warps) {
    const int64_t i = b * 32 + lane;
    const bool valid = i < n;
    const int64_t k = valid ? load_int(req, req64, i) : kEmptyKey;
    const int64_t v = warp_find(m, k, valid);
    if (valid) store_int(out, out64, i, v);
  }
}

inline unsigned grid_for_warps(int64_t n_items_per_warp32) {
  const int64_t batches = (n_items_per_warp32 + 31) / 32;
  int64_t blocks = (batches + kMapThreads / 32 - 1) / (kMapThreads / 32);
  const int64_t cap = (int64_t)sm_count() * 32;
  if (blocks > cap) blocks = cap;
  if (blocks < 1) blocks = 1;
  return (unsigned)blocks;
}

inline uint64_t windows_for(int64_t capacity, int64_t expected_keys) {
  // Probe length, not memory, is what the kernels pay for: provision at least two slots
  // per expected key (load <= 0.5: a lookup ends in its home window almost always, whatever
  // load factor the caller asked for), and never less than the requested capacity + 1/16.
  uint64_t slots = (uint64_t)capacity + (uint64_t)capacity / 16;
  if (expected_keys > 0 && (uint64_t)expected_keys * 2 > slots) slots = (uint64_t)expected_keys * 2;
  slots += kWindow;
  return (slots + kWindow - 1) / kWindow;
}

}  // namespace shmt

using namespace shmt;

extern "C" {

int64_t shmt_map_table_bytes(int64_t capacity, int64_t expected_keys) {
  if (capacity < 0) return 0;
  return (int64_t)(windows_for(capacity, expected_keys) * kWindow * sizeof(Slot) + 256);
}

int shmt_map_create(int device, int64_t capacity, int64_t expected_keys, int key_dtype,
                    int val_dtype, void* table_buf,
                    void* stream, shmt_map** out) {
  SHMT_REQUIRE(out != nullptr, "shmt_map_create: out is null");
  SHMT_REQUIRE(capacity >= 0, "shmt_map_create: negative capacity");
  SHMT_REQUIRE(valid_int_dtype(key_dtype) && valid_int_dtype(val_dtype),
               "shmt_map_create: keys and values can only be int32 or int64");
  SHMT_REQUIRE(((uintptr_t)table_buf & 15) == 0, "shmt_map_create: table buffer must be 16-byte aligned");
  DeviceGuard guard(device);
  shmt_map* m = new shmt_map();
  m->device = device;
  m->capacity = capacity;
  m->key_dtype = key_dtype;
  m->val_dtype = val_dtype;
  m->table_bytes = (size_t)shmt_map_table_bytes(capacity, expected_keys);
  void* buf = table_buf;
  if (!buf) {
    cudaError_t e = cudaMalloc(&buf, m->table_bytes);
    if (e != cudaSuccess) {
      set_error("shmt_map_create: cudaMalloc of %zu bytes failed: %s", m->table_bytes,
                cudaGetErrorString(e));
      delete m;
      return SHMT_ERR_CUDA;
    }
    m->owns_table = true;
  }
  m->view.slots = static_cast<Slot*>(buf);
  m->view.n_windows = windows_for(capacity, expected_keys);
  m->view.key32 = key_dtype == SHMT_I32;
  m->d_meta = reinterpret_cast<int64_t*>(static_cast<char*>(buf) + m->table_bytes - 256);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  // every slot {-1, -1}; then the trailing status / size words to zero
  cudaError_t e = cudaMemsetAsync(buf, 0xFF, m->table_bytes - 256, s);
  if (e == cudaSuccess) e = cudaMemsetAsync(m->d_meta, 0, 256, s);
  if (e != cudaSuccess) {
    set_error("shmt_map_create: memset failed: %s", cudaGetErrorString(e));
    if (m->owns_table) cudaFree(buf);
    delete m;
    return SHMT_ERR_CUDA;
  }
  *out = m;
  return SHMT_OK;
}

int shmt_map_insert(shmt_map* map, const void* keys, const void* values, int64_t n, void* stream) {
  SHMT_REQUIRE(map != nullptr, "shmt_map_insert: map is null");
  SHMT_REQUIRE(n >= 0, "shmt_map_insert: negative count");
  if (n == 0) return SHMT_OK;
  SHMT_REQUIRE(keys != nullptr && values != nullptr, "shmt_map_insert: keys/values are null");
  DeviceGuard guard(map->device);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  int64_t ins_blocks = (n + kMapThreads - 1) / kMapThreads;
  const int64_t ins_cap = (int64_t)sm_count() * 16;
  // the status word reports on this call only: an overflow of an earlier call must not make
  // every later insert fail once room has been freed again (the key count behind it stays)
  SHMT_CUDA_TRY(cudaMemsetAsync(map->d_meta, 0, sizeof(int64_t), s));
  map_insert_kernel<<<(unsigned)(ins_blocks < ins_cap ? ins_blocks : ins_cap), kMapThreads, 0, s>>>(
      map->view, keys, map->key_dtype == SHMT_I64, values, map->val_dtype == SHMT_I64, n,
      map->d_meta);
  SHMT_CUDA_TRY(cudaGetLastError());
  int64_t meta[2] = {0, 0};
  SHMT_CUDA_TRY(cudaMemcpyAsync(meta, map->d_meta, sizeof(meta), cudaMemcpyDeviceToHost, s));
  SHMT_CUDA_TRY(cudaStreamSynchronize(s));
  map->size = meta[1];
  if (meta[0] == DEV_OVERFLOW) {
    set_error("shmt_map_insert: table overflow (%lld keys stored, capacity %lld)",
              (long long)meta[1], (long long)map->capacity);
    return SHMT_ERR_CAPACITY;
  }
  return SHMT_OK;
}

int shmt_map_erase(shmt_map* map, const void* keys, int64_t n, void* out_values, void* stream) {
  SHMT_REQUIRE(map != nullptr, "shmt_map_erase: map is null");
  SHMT_REQUIRE(n >= 0, "shmt_map_erase: negative count");
  if (n == 0) return SHMT_OK;
  SHMT_REQUIRE(keys != nullptr, "shmt_map_erase: keys are null");
  DeviceGuard guard(map->device);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  int64_t blocks = (n + kMapThreads - 1) / kMapThreads;
  const int64_t cap = (int64_t)sm_count() * 16;
  map_erase_kernel<<<(unsigned)(blocks < cap ? blocks : cap), kMapThreads, 0, s>>>(
      map->view, keys, map->key_dtype == SHMT_I64, n, out_values, map->val_dtype == SHMT_I64,
      map->d_meta);
  SHMT_CUDA_TRY(cudaGetLastError());
  int64_t meta[2] = {0, 0};
  SHMT_CUDA_TRY(cudaMemcpyAsync(meta, map->d_meta, sizeof(meta), cudaMemcpyDeviceToHost, s));
  SHMT_CUDA_TRY(cudaStreamSynchronize(s));
  map->size = meta[1];
  return SHMT_OK;
}

int shmt_map_query(const shmt_map* map, const void* requests, int req_dtype, int64_t n, void* out,
                   void* stream) {
  SHMT_REQUIRE(map != nullptr, "shmt_map_query: map is null");
  SHMT_REQUIRE(valid_int_dtype(req_dtype), "shmt_map_query: requests can only be int32 or int64");
  SHMT_REQUIRE(n >= 0, "shmt_map_query: negative count");
  if (n == 0) return SHMT_OK;
  SHMT_REQUIRE(requests != nullptr && out != nullptr, "shmt_map_query: requests/out are null");
  DeviceGuard guard(map->device);
  map_query_kernel<<<grid_for_warps(n), kMapThreads, 0, static_cast<cudaStream_t>(stream)>>>(
      map->view, requests, req_dtype == SHMT_I64, n, out, map->val_dtype == SHMT_I64);
  SHMT_CUDA_TRY(cudaGetLastError());
  return SHMT_OK;
}

int64_t shmt_map_capacity(const shmt_map* map) { return map ? map->capacity : 0; }
int64_t shmt_map_memory_usage(const shmt_map* map) { return map ? (int64_t)map->table_bytes : 0; }
int64_t shmt_map_size(const shmt_map* map) { return map ? map->size : 0; }
int shmt_map_key_dtype(const shmt_map* map) { return map ? map->key_dtype : -1; }
int shmt_map_val_dtype(const shmt_map* map) { return map ? map->val_dtype : -1; }

int shmt_map_destroy(shmt_map* map) {
  if (!map) return SHMT_OK;
  if (map->owns_table) {
    DeviceGuard guard(map->device);
    cudaFree(map->view.slots);
  }
  delete map;
  return SHMT_OK;
}

}  // extern "C"
