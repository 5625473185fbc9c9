// Context, error text and small device utilities of libshmt.
#include <stdarg.h>
#include <string.h>

#include "ctx.cuh"

namespace shmt {

static thread_local char g_error[1024] = "";

void set_error(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_error, sizeof(g_error), fmt, ap);
  va_end(ap);
}

int sm_count() {
  static int cached[64] = {0};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
  if (cached[dev] == 0) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0)
      n = 148;
    cached[dev] = n;
  }
  return cached[dev];
}

int device_of_pointer(const void* p) {
  int cur = 0;
  cudaGetDevice(&cur);
  cudaPointerAttributes a;
  if (p && cudaPointerGetAttributes(&a, p) == cudaSuccess && a.type == cudaMemoryTypeDevice)
    return a.device;
  cudaGetLastError();  // a failed query must not poison the next launch check
  return cur;
}

HostPost ctx_begin_post(shmt_ctx* ctx, const int64_t* dev_words, int n_words, int64_t* done_word) {
  HostPost p{};
  p.words = dev_words;
  p.n_words = n_words;
  p.done = done_word;
  if (n_words > kCtxWords - 1) return p;  // no room: ctx_await_post copies instead
  void* dev_view = nullptr;
  if (cudaHostGetDevicePointer(&dev_view, ctx->h_words, 0) != cudaSuccess) {
    cudaGetLastError();
    return p;
  }
  p.host = static_cast<int64_t*>(dev_view);
  p.flag_at = kCtxWords - 1;
  p.seq = ++ctx->post_seq;
  return p;
}

static inline void cpu_relax() {
#if defined(__x86_64__) || defined(__i386__)
  __builtin_ia32_pause();
#else
  asm volatile("" ::: "memory");
#endif
}

int ctx_await_post(shmt_ctx* ctx, const HostPost& post, cudaStream_t stream) {
  if (post.host) {
    const int64_t* flag = ctx->h_words + post.flag_at;
    for (uint64_t it = 1;; ++it) {
      if (__atomic_load_n(flag, __ATOMIC_ACQUIRE) == post.seq) return SHMT_OK;
      if ((it & 0xFFF) == 0) {
        const cudaError_t q = cudaStreamQuery(stream);
        if (q == cudaSuccess) {
          if (__atomic_load_n(flag, __ATOMIC_ACQUIRE) == post.seq) return SHMT_OK;
          break;  // drained without a post: read the words the ordinary way
        }
        if (q != cudaErrorNotReady) {
          set_error("waiting for posted results: %s", cudaGetErrorString(q));
          return SHMT_ERR_CUDA;
        }
      }
      cpu_relax();
    }
  }
  SHMT_CUDA_TRY(cudaMemcpyAsync(ctx->h_words, post.words, (size_t)post.n_words * sizeof(int64_t),
                                cudaMemcpyDeviceToHost, stream));
  SHMT_CUDA_TRY(cudaStreamSynchronize(stream));
  return SHMT_OK;
}

int ctx_mark_tail(shmt_ctx* ctx, cudaStream_t stream) {
  if (!ctx->tail_event)
    SHMT_CUDA_TRY(cudaEventCreateWithFlags(&ctx->tail_event, cudaEventDisableTiming));
  SHMT_CUDA_TRY(cudaEventRecord(ctx->tail_event, stream));
  ctx->tail_pending = true;
  return SHMT_OK;
}

int ctx_join_tail(shmt_ctx* ctx) {
  if (!ctx->tail_pending) return SHMT_OK;
  ctx->tail_pending = false;
  SHMT_CUDA_TRY(cudaEventSynchronize(ctx->tail_event));
  return SHMT_OK;
}

int ctx_reserve(shmt_ctx* ctx, size_t bytes) {
  if (int rc = ctx_join_tail(ctx)) return rc;
  bytes += 256;  // result words live in front of the region
  if (bytes <= ctx->scratch_bytes) return SHMT_OK;
  // cudaFree waits for work that may still read the old block.
  if (ctx->scratch) SHMT_CUDA_TRY(cudaFree(ctx->scratch));
  ctx->scratch = nullptr;
  ctx->scratch_bytes = 0;
  size_t want = bytes + bytes / 2;
  if (want < ((size_t)1 << 20)) want = (size_t)1 << 20;
  want = (want + 255) & ~(size_t)255;
  void* p = nullptr;
  SHMT_CUDA_TRY(cudaMalloc(&p, want));
  ctx->scratch = static_cast<char*>(p);
  ctx->scratch_bytes = want;
  return SHMT_OK;
}

int ctx_reserve_table(shmt_ctx* ctx, size_t bytes, cudaStream_t stream) {
  if (int rc = ctx_join_tail(ctx)) return rc;
  if (bytes > ctx->table_bytes) {
    if (ctx->table) SHMT_CUDA_TRY(cudaFree(ctx->table));
    ctx->table = nullptr;
    ctx->table_bytes = 0;
    size_t want = bytes + bytes / 2;
    if (want < ((size_t)4 << 20)) want = (size_t)4 << 20;
    want = (want + 255) & ~(size_t)255;
    void* p = nullptr;
    SHMT_CUDA_TRY(cudaMalloc(&p, want));
    ctx->table = static_cast<char*>(p);
    ctx->table_bytes = want;
    ctx->table_dirty = true;
  }
  if (ctx->table_dirty) {
    SHMT_CUDA_TRY(cudaMemsetAsync(ctx->table, 0xFF, ctx->table_bytes, stream));
    ctx->table_dirty = false;
  }
  return SHMT_OK;
}

int ctx_fetch_words(shmt_ctx* ctx, cudaStream_t stream, const char* what) {
  SHMT_CUDA_TRY(cudaMemcpyAsync(ctx->h_words, ctx->d_words(), 4 * sizeof(int64_t),
                                cudaMemcpyDeviceToHost, stream));
  SHMT_CUDA_TRY(cudaStreamSynchronize(stream));
  return ctx_status_of_words(ctx, what);
}

int ctx_status_of_words(shmt_ctx* ctx, const char* what) {
  const int64_t st = ctx->h_words[W_STATUS];
  if (st != DEV_OK) ctx->table_dirty = true;
  if (st == DEV_TIMEOUT) {
    set_error("%s: a bounded look-back wait ran out (device status %lld)", what, (long long)st);
    return SHMT_ERR_TIMEOUT;
  }
  if (st == DEV_OVERFLOW) {
    set_error("%s: table overflow (device status %lld)", what, (long long)st);
    return SHMT_ERR_CAPACITY;
  }
  return SHMT_OK;
}

}  // namespace shmt

using namespace shmt;

extern "C" {

const char* shmt_last_error(void) { return g_error; }

int shmt_version(void) { return 100; }

int shmt_ctx_create(int device, shmt_ctx** out) {
  SHMT_REQUIRE(out != nullptr, "shmt_ctx_create: out is null");
  int ndev = 0;
  SHMT_CUDA_TRY(cudaGetDeviceCount(&ndev));
  SHMT_REQUIRE(device >= 0 && device < ndev, "shmt_ctx_create: device %d out of range (%d devices)",
               device, ndev);
  DeviceGuard guard(device);
  shmt_ctx* ctx = new shmt_ctx();
  ctx->device = device;
  void* h = nullptr;
  cudaError_t e = cudaHostAlloc(&h, kCtxWords * sizeof(int64_t),
                                cudaHostAllocMapped | cudaHostAllocPortable);
  if (e != cudaSuccess) {
    set_error("shmt_ctx_create: %s", cudaGetErrorString(e));
    delete ctx;
    return SHMT_ERR_CUDA;
  }
  if (int rc = ctx_reserve(ctx, 0)) {
    cudaFreeHost(h);
    delete ctx;
    return rc;
  }
  ctx->h_words = static_cast<int64_t*>(h);
  memset(ctx->h_words, 0, kCtxWords * sizeof(int64_t));
  *out = ctx;
  return SHMT_OK;
}

int shmt_ctx_destroy(shmt_ctx* ctx) {
  if (!ctx) return SHMT_OK;
  DeviceGuard guard(ctx->device);
  if (ctx->scratch) cudaFree(ctx->scratch);
  if (ctx->table) cudaFree(ctx->table);
  if (ctx->h_words) cudaFreeHost(ctx->h_words);
  if (ctx->tail_event) cudaEventDestroy(ctx->tail_event);
  delete ctx;
  return SHMT_OK;
}

int shmt_ctx_check(shmt_ctx* ctx, void* stream) {
  SHMT_REQUIRE(ctx != nullptr, "shmt_ctx_check: ctx is null");
  DeviceGuard guard(ctx->device);
  return ctx_fetch_words(ctx, static_cast<cudaStream_t>(stream), "shmt_ctx_check");
}

int shmt_ctx_reserve(shmt_ctx* ctx, int64_t scratch_bytes, int64_t relabel_ids, void* stream) {
  SHMT_REQUIRE(ctx != nullptr, "shmt_ctx_reserve: ctx is null");
  SHMT_REQUIRE(scratch_bytes >= 0 && relabel_ids >= 0 && relabel_ids < ((int64_t)1 << 30),
               "shmt_ctx_reserve: sizes out of range");
  DeviceGuard guard(ctx->device);
  if (int rc = ctx_reserve(ctx, (size_t)scratch_bytes)) return rc;
  if (relabel_ids > 0) {
    uint64_t cap = 64;
    while (cap < (uint64_t)relabel_ids * 2) cap <<= 1;
    if (int rc = ctx_reserve_table(ctx, cap * 16, static_cast<cudaStream_t>(stream))) return rc;
  }
  return SHMT_OK;
}

int64_t shmt_ctx_scratch_bytes(const shmt_ctx* ctx) {
  return ctx ? (int64_t)(ctx->scratch_bytes + ctx->table_bytes) : 0;
}

}  // extern "C"
