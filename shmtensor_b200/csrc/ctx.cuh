// Per-device context: reusable scratch + result words (host side).
#pragma once

#include "common.cuh"

struct shmt_ctx {
  int device = 0;
  char* scratch = nullptr;      // device scratch, grown geometrically; the first
  size_t scratch_bytes = 0;     // 256 bytes are the result words (status, result, ticket ...)
  int64_t* h_words = nullptr;   // pinned host mirror of the result words
  // Relabel table (keys i64 | first-index u32 | new-id u32 per slot).  Kept all-ones between
  // calls: the remap kernel restores every slot it leaves, so no per-call memset is needed.
  char* table = nullptr;
  size_t table_bytes = 0;
  bool table_dirty = false;     // a failed call may have left entries behind
  int64_t* d_words() const { return reinterpret_cast<int64_t*>(scratch); }
  char* region() const { return scratch + 256; }
};

namespace shmt {

constexpr int kCtxWords = 128;
enum : int { W_STATUS = 0, W_RESULT = 1, W_TICKET = 2, W_DONE = 3 };

// Make sure ctx->region() holds at least `bytes` (256-byte aligned base).
int ctx_reserve(shmt_ctx* ctx, size_t bytes);

// Make sure ctx->table holds at least `bytes`, all ones.
int ctx_reserve_table(shmt_ctx* ctx, size_t bytes, cudaStream_t stream);

// Copy the first `n_words` result words to the host and wait for `stream`.
// Returns SHMT_ERR_TIMEOUT / SHMT_ERR_CAPACITY if the kernel flagged either.
int ctx_fetch_words(shmt_ctx* ctx, cudaStream_t stream, const char* what);

// Device that owns a device pointer (the current device if the runtime cannot tell).
int device_of_pointer(const void* p);

// RAII device guard for entry points that are handed a context or a map.
struct DeviceGuard {
  int prev = -1;
  bool switched = false;
  explicit DeviceGuard(int device) {
    if (cudaGetDevice(&prev) == cudaSuccess && prev != device) {
      switched = cudaSetDevice(device) == cudaSuccess;
    }
  }
  ~DeviceGuard() {
    if (switched) cudaSetDevice(prev);
  }
};

}  // namespace shmt
