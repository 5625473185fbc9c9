// Per-device context: reusable scratch + result words (host side).
#pragma once

#include "common.cuh"

struct shmt_ctx {
  int device = 0;
  char* scratch = nullptr;      // device scratch, grown geometrically; the first
  size_t scratch_bytes = 0;     // 256 bytes are the result words (status, result, ticket ...)
  int64_t* h_words = nullptr;   // pinned host mirror of the result words
  // Relabel table (16-byte slots: key i64, first-index u32, new-id u32).  Keys and first-index words all ones between
  // calls: the remap kernel restores every slot it leaves, so no per-call memset is needed.
  char* table = nullptr;
  size_t table_bytes = 0;
  bool table_dirty = false;     // a failed call may have left entries behind
  // Early hand-over of result words (see HostPost): sequence number of the last post, and an
  // event behind the kernels that were still running when the call returned.
  int64_t post_seq = 0;
  cudaEvent_t tail_event = nullptr;
  bool tail_pending = false;
  int64_t* d_words() const { return reinterpret_cast<int64_t*>(scratch); }
  char* region() const { return scratch + 256; }
};

namespace shmt {

constexpr int kCtxWords = 128;
enum : int { W_STATUS = 0, W_RESULT = 1, W_TICKET = 2, W_DONE = 3, W_RANGE = 4 };

// Make sure ctx->region() holds at least `bytes` (256-byte aligned base).
int ctx_reserve(shmt_ctx* ctx, size_t bytes);

// Make sure ctx->table holds at least `bytes`, all ones.
int ctx_reserve_table(shmt_ctx* ctx, size_t bytes, cudaStream_t stream);

// Copy the first `n_words` result words to the host and wait for `stream`.
// Returns SHMT_ERR_TIMEOUT / SHMT_ERR_CAPACITY if the kernel flagged either.
int ctx_fetch_words(shmt_ctx* ctx, cudaStream_t stream, const char* what);
// The same check on words that are already in ctx->h_words.
int ctx_status_of_words(shmt_ctx* ctx, const char* what);

// Result words handed to the host without a copy and before the stream drains: the thread that
// completes them stores them into the context's pinned host words and then a sequence number,
// which the host polls for.  Whatever the stream still runs behind that point must not produce
// results or errors the host needs.
struct HostPost {
  int64_t* host;         // pinned host words as the device sees them; nullptr = no post
  const int64_t* words;  // device words to mirror
  int n_words;
  int flag_at;           // index of the sequence word (the last pinned word)
  int64_t seq;           // stored to host[flag_at] after the words
  int64_t* done;         // zeroed device word counting the CTAs that have finished
};

#ifdef __CUDACC__
__device__ __forceinline__ void post_to_host(const HostPost& p) {
  if (!p.host) return;
  for (int i = 0; i < p.n_words; ++i)
    *reinterpret_cast<volatile int64_t*>(p.host + i) = ld_relaxed64(p.words + i);
  __threadfence_system();
  *reinterpret_cast<volatile int64_t*>(p.host + p.flag_at) = p.seq;
}

// Called by one thread of each of the `n_ctas` CTAs that produce results, after a CTA-wide
// barrier behind its last result or status write: the CTA that finishes last posts, so the host
// sees every CTA's words.
__device__ __forceinline__ void post_when_last(const HostPost& p, int64_t n_ctas) {
  if (!p.host) return;
  __threadfence();
  const unsigned long long before = atomicAdd(reinterpret_cast<unsigned long long*>(p.done), 1ULL);
  if ((int64_t)before + 1 == n_ctas) {
    __threadfence();
    post_to_host(p);
  }
}
#endif

// Host side of HostPost: a post for the next call on `stream` (mirroring `n_words` words from
// `dev_words`; `done_word` is a device word the call zeroes), and the wait for it.  ctx_await_post polls the pinned word, looks at the stream
// now and then (an error ends the wait; a drained stream without a post falls back to a copy),
// and leaves the words in ctx->h_words.  ctx_mark_tail records that kernels of this call may
// still be running; the next user of the context's scratch waits for them first.
HostPost ctx_begin_post(shmt_ctx* ctx, const int64_t* dev_words, int n_words, int64_t* done_word);
int ctx_await_post(shmt_ctx* ctx, const HostPost& post, cudaStream_t stream);
int ctx_mark_tail(shmt_ctx* ctx, cudaStream_t stream);
int ctx_join_tail(shmt_ctx* ctx);

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
