// Shared host/device helpers of libshmt (sm_100a only).
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>

#include "shmt.h"

namespace shmt {

// ---- host side: error text + CUDA call wrapper --------------------------------
void set_error(const char* fmt, ...);

#define SHMT_CUDA_TRY(call)                                                    \
  do {                                                                         \
    cudaError_t e__ = (call);                                                  \
    if (e__ != cudaSuccess) {                                                  \
      ::shmt::set_error("%s:%d CUDA call `%s` failed: %s (%d)", __FILE__,      \
                        __LINE__, #call, cudaGetErrorString(e__), (int)e__);   \
      return SHMT_ERR_CUDA;                                                    \
    }                                                                          \
  } while (0)

#define SHMT_REQUIRE(cond, ...)          \
  do {                                   \
    if (!(cond)) {                       \
      ::shmt::set_error(__VA_ARGS__);    \
      return SHMT_ERR_INVALID;           \
    }                                    \
  } while (0)

inline bool valid_int_dtype(int d) { return d == SHMT_I32 || d == SHMT_I64; }
inline int int_itemsize(int d) { return d == SHMT_I64 ? 8 : 4; }

// Number of SMs of the current device (148 on B200); cached per device.
int sm_count();

// Device-side status word layout shared by every kernel that can give up.
enum : int { DEV_OK = 0, DEV_OVERFLOW = 1, DEV_TIMEOUT = 2 };

// Launch `kernel` allowing it to overlap its scheduling with the tail of the previous kernel
// in `stream` (see pdl_prologue); plain launch when `pdl` is false.
#ifdef __CUDACC__
template <typename... KArgs, typename... Args>
inline cudaError_t launch_kernel(bool pdl, void (*kernel)(KArgs...), unsigned grid, unsigned block,
                                 size_t smem, cudaStream_t stream, Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(grid);
  cfg.blockDim = dim3(block);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
}
#endif

// ---- device side -----------------------------------------------------------------
#ifdef __CUDACC__

constexpr int64_t kEmptyKey = -1;

__device__ __forceinline__ int64_t load_int(const void* p, int is64, int64_t i) {
  return is64 ? __ldg(reinterpret_cast<const long long*>(p) + i)
              : (int64_t)__ldg(reinterpret_cast<const int*>(p) + i);
}

__device__ __forceinline__ void store_int(void* p, int is64, int64_t i, int64_t v) {
  if (is64)
    reinterpret_cast<long long*>(p)[i] = v;
  else
    reinterpret_cast<int*>(p)[i] = (int)v;
}

// 64-bit finaliser (splitmix64 / murmur3 fmix style): full avalanche, so the
// slot index can be taken with a multiply-high instead of a modulo.
__device__ __forceinline__ uint64_t mix64(uint64_t x) {
  x ^= x >> 33;
  x *= 0xff51afd7ed558ccdULL;
  x ^= x >> 33;
  x *= 0xc4ceb9fe1a85ec53ULL;
  x ^= x >> 33;
  return x;
}

// acquire / release accesses at GPU scope for cross-CTA hand-offs.
__device__ __forceinline__ uint32_t ld_acquire(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_release(uint32_t* p, uint32_t v) {
  asm volatile("st.release.gpu.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ int64_t ld_relaxed64(const int64_t* p) {
  long long v;
  asm volatile("ld.relaxed.gpu.global.s64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_relaxed64(int64_t* p, int64_t v) {
  asm volatile("st.relaxed.gpu.global.s64 [%0], %1;" ::"l"(p), "l"((long long)v) : "memory");
}

// 16-byte streaming accesses: rows are touched once per call, so keep them out
// of L1 and mark them evict-first in L2 on the store side.
__device__ __forceinline__ uint4 ld_stream16(const void* p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p));
  return v;
}
__device__ __forceinline__ void st_stream16(void* p, uint4 v) {
  asm volatile("st.global.cs.v4.u32 [%0], {%1,%2,%3,%4};" ::"l"(p), "r"(v.x), "r"(v.y),
               "r"(v.z), "r"(v.w)
               : "memory");
}

// Programmatic dependent launch (sm_90+): a kernel that starts with pdl_prologue() lets the
// next kernel of the stream be scheduled as soon as all of its own CTAs are resident, and
// itself waits until the kernel before it has completed and flushed its writes.  Without the
// launch attribute both instructions do nothing.  Hides the launch latency between the short
// dependent kernels of a multi-hop mini-batch.
__device__ __forceinline__ void pdl_prologue() {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  asm volatile("griddepcontrol.wait;" ::: "memory");
}

// Philox4x32-10 (Salmon et al., SC'11): counter-based, so every (call, seed row,
// lane) gets an independent stream with no state carried between launches.
struct Philox {
  uint32_t k0, k1;
  __device__ __forceinline__ Philox(uint64_t seed) : k0((uint32_t)seed), k1((uint32_t)(seed >> 32)) {}
  __device__ __forceinline__ uint4 operator()(uint32_t c0, uint32_t c1, uint32_t c2,
                                              uint32_t c3) const {
    uint32_t a = k0, b = k1;
#pragma unroll
    for (int r = 0; r < 10; ++r) {
      const uint32_t hi0 = __umulhi(0xD2511F53u, c0), lo0 = 0xD2511F53u * c0;
      const uint32_t hi1 = __umulhi(0xCD9E8D57u, c2), lo1 = 0xCD9E8D57u * c2;
      const uint32_t n0 = hi1 ^ c1 ^ a, n2 = hi0 ^ c3 ^ b;
      c0 = n0;
      c1 = lo1;
      c2 = n2;
      c3 = lo0;
      a += 0x9E3779B9u;
      b += 0xBB67AE85u;
    }
    return make_uint4(c0, c1, c2, c3);
  }
};

// Uniform integer in [0, range) from 64 random bits (multiply-high; the bias is
// below range / 2^64).
__device__ __forceinline__ uint64_t bounded(uint32_t lo, uint32_t hi, uint64_t range) {
  return __umul64hi(((uint64_t)hi << 32) | lo, range);
}

#endif  // __CUDACC__

}  // namespace shmt
