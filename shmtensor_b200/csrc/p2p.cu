// Device buffers shared between ranks of a partitioned cache (CUDA IPC) and the
// streaming-read probe used to measure HBM / host-link / peer-link ceilings.
// The reference is single-GPU and has no counterpart for any of this.
#include <string.h>

#include "common.cuh"

namespace shmt {

// Every thread folds 16-byte loads into a checksum; a few threads publish it so
// the loads cannot be optimised away.  Plain per-thread loads only, so the
// source may be local HBM, pinned host memory or a peer GPU's buffer.
__global__ void __launch_bounds__(256)
stream_read_kernel(const uint4* __restrict__ src, int64_t n_vec, unsigned long long* sink) {
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  uint32_t acc = 0;
  for (; i + 3 * stride < n_vec; i += 4 * stride) {
    const uint4 a = ld_stream16(src + i), b = ld_stream16(src + i + stride),
                c = ld_stream16(src + i + 2 * stride), d = ld_stream16(src + i + 3 * stride);
    acc ^= a.x ^ a.y ^ a.z ^ a.w ^ b.x ^ b.y ^ b.z ^ b.w ^ c.x ^ c.y ^ c.z ^ c.w ^ d.x ^ d.y ^
           d.z ^ d.w;
  }
  for (; i < n_vec; i += stride) {
    const uint4 a = ld_stream16(src + i);
    acc ^= a.x ^ a.y ^ a.z ^ a.w;
  }
  if (acc == 0x9E3779B9u) atomicAdd(sink, 1ULL);  // practically never; keeps the loads alive
}

// Independent reads of UNIT bytes at pseudo-random UNIT-aligned offsets: the access pattern of
// a hash probe (16-byte slot), of a row-offset pair or of a short adjacency list.  What it
// measures is a rate of reads, not bytes: random sectors from HBM, small requests over the
// host link or NVLink.  Four reads per thread are in flight before the first is used.
template <int UNIT>
__global__ void __launch_bounds__(256)
random_read_kernel(const char* __restrict__ src, uint64_t n_units, int64_t n_reads, uint64_t seed,
                   unsigned long long* sink) {
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  uint32_t acc = 0;
  auto one = [&](int64_t i) {
    const uint64_t u = __umul64hi(mix64((uint64_t)i * 0x9E3779B97F4A7C15ULL + seed), n_units);
    const uint4* p = reinterpret_cast<const uint4*>(src + u * UNIT);
    uint32_t x = 0;
#pragma unroll
    for (int q = 0; q < UNIT / 16; ++q) {
      const uint4 v = ld_stream16(p + q);
      x ^= v.x ^ v.y ^ v.z ^ v.w;
    }
    return x;
  };
  int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  for (; i + 3 * stride < n_reads; i += 4 * stride) {
    const uint32_t a = one(i), b = one(i + stride), c = one(i + 2 * stride), d = one(i + 3 * stride);
    acc ^= a ^ b ^ c ^ d;
  }
  for (; i < n_reads; i += stride) acc ^= one(i);
  if (acc == 0x9E3779B9u) atomicAdd(sink, 1ULL);
}

}  // namespace shmt

using namespace shmt;

extern "C" {

int shmt_dev_alloc(int64_t bytes, void** out) {
  SHMT_REQUIRE(out != nullptr && bytes > 0, "shmt_dev_alloc: bad argument");
  // Whole 2 MB pages: a peer that opens the buffer through CUDA IPC maps an allocation whose
  // size is not a multiple of 2 MB with small pages, and random row reads from it then miss the
  // TLB on every row once the buffer outgrows its reach (measured on B200: 63,000 rows of 512
  // bytes from an 11.4 GB peer buffer in 1.04 ms, against 0.058 ms when the size is rounded up).
  const size_t page = (size_t)2 << 20;
  const size_t padded = ((size_t)bytes + page - 1) & ~(page - 1);
  SHMT_CUDA_TRY(cudaMalloc(out, padded));
  return SHMT_OK;
}

int shmt_dev_free(void* ptr) {
  if (ptr) SHMT_CUDA_TRY(cudaFree(ptr));
  return SHMT_OK;
}

int shmt_ipc_get_handle(void* dev_ptr, void* handle_64_bytes) {
  SHMT_REQUIRE(dev_ptr && handle_64_bytes, "shmt_ipc_get_handle: null argument");
  static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handle is 64 bytes");
  cudaIpcMemHandle_t h;
  SHMT_CUDA_TRY(cudaIpcGetMemHandle(&h, dev_ptr));
  memcpy(handle_64_bytes, &h, sizeof(h));
  return SHMT_OK;
}

int shmt_ipc_open_handle(const void* handle_64_bytes, void** out) {
  SHMT_REQUIRE(handle_64_bytes && out, "shmt_ipc_open_handle: null argument");
  cudaIpcMemHandle_t h;
  memcpy(&h, handle_64_bytes, sizeof(h));
  SHMT_CUDA_TRY(cudaIpcOpenMemHandle(out, h, cudaIpcMemLazyEnablePeerAccess));
  return SHMT_OK;
}

int shmt_ipc_close_handle(void* mapped_ptr) {
  if (mapped_ptr) SHMT_CUDA_TRY(cudaIpcCloseMemHandle(mapped_ptr));
  return SHMT_OK;
}

int shmt_random_read(const void* src, int64_t bytes, int64_t n_reads, int read_bytes,
                     uint64_t seed, void* sink_8_bytes, void* stream) {
  SHMT_REQUIRE(src && sink_8_bytes && n_reads >= 0, "shmt_random_read: bad argument");
  SHMT_REQUIRE(read_bytes == 16 || read_bytes == 32 || read_bytes == 64 || read_bytes == 128,
               "shmt_random_read: read_bytes must be 16, 32, 64 or 128");
  SHMT_REQUIRE(bytes >= read_bytes && ((uintptr_t)src & 15) == 0,
               "shmt_random_read: src must be 16-byte aligned and hold at least one read");
  if (n_reads == 0) return SHMT_OK;
  const uint64_t n_units = (uint64_t)bytes / (uint64_t)read_bytes;
  int64_t blocks = (n_reads + 255) / 256 / 4 + 1;
  const int64_t cap = (int64_t)sm_count() * 8;
  const unsigned grid = (unsigned)(blocks < cap ? blocks : cap);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const char* p = static_cast<const char*>(src);
  unsigned long long* sink = static_cast<unsigned long long*>(sink_8_bytes);
  switch (read_bytes) {
    case 16: random_read_kernel<16><<<grid, 256, 0, s>>>(p, n_units, n_reads, seed, sink); break;
    case 32: random_read_kernel<32><<<grid, 256, 0, s>>>(p, n_units, n_reads, seed, sink); break;
    case 64: random_read_kernel<64><<<grid, 256, 0, s>>>(p, n_units, n_reads, seed, sink); break;
    default: random_read_kernel<128><<<grid, 256, 0, s>>>(p, n_units, n_reads, seed, sink); break;
  }
  SHMT_CUDA_TRY(cudaGetLastError());
  return SHMT_OK;
}

int shmt_stream_read(const void* src, int64_t bytes, void* sink_8_bytes, void* stream) {
  SHMT_REQUIRE(src && sink_8_bytes && bytes >= 16, "shmt_stream_read: bad argument");
  SHMT_REQUIRE(((uintptr_t)src & 15) == 0, "shmt_stream_read: src must be 16-byte aligned");
  const int64_t n_vec = bytes / 16;
  int64_t blocks = (n_vec + 255) / 256 / 4 + 1;
  const int64_t cap = (int64_t)sm_count() * 8;
  stream_read_kernel<<<(unsigned)(blocks < cap ? blocks : cap), 256, 0,
                       static_cast<cudaStream_t>(stream)>>>(
      static_cast<const uint4*>(src), n_vec, static_cast<unsigned long long*>(sink_8_bytes));
  SHMT_CUDA_TRY(cudaGetLastError());
  return SHMT_OK;
}

}  // extern "C"
