// Stand-in for <cuco/static_map.cuh>, for compiling the reference's own sources as a
// GPU-side oracle / baseline.  TEST AND BENCH INFRASTRUCTURE, NOT PRODUCT CODE.
//
// The reference wraps NVIDIA/cuCollections (branch `dev`, fetched by its build, not part of
// its tree and not on this machine).  This header supplies exactly the part of that API the
// reference touches -- include/cuco_hashmap.cuh:52-55,66-70,84-85 and the device calls
// ref(cuco::find) / .find(k) / .end() / ->second in src/cache_feature_fetch.cu,
// src/cache_feature_set.cu and src/cache_graph_sampling.cu -- with the configuration the
// reference selects: linear probing with step 1, one thread per key, one slot per window,
// array-of-pairs storage, sentinel key/value.  It is written from that interface, not from
// cuCollections' sources; timings taken with it are labelled "reference kernels + stand-in map".
#pragma once

#include <cuda/atomic>
#include <cub/cub.cuh>
#include <cuda_runtime.h>
#include <thrust/device_ptr.h>
#include <thrust/functional.h>
#include <thrust/tuple.h>

#include <cstddef>
#include <cstdint>

namespace cuco {

template <typename First, typename Second>
struct alignas(sizeof(First) + sizeof(Second) <= 8 ? 8 : 16) pair {
  First first;
  Second second;
};

template <typename T>
struct empty_key {
  T value;
  __host__ __device__ explicit constexpr empty_key(T v) : value(v) {}
};
template <typename T>
struct empty_value {
  T value;
  __host__ __device__ explicit constexpr empty_value(T v) : value(v) {}
};

template <typename Key>
struct default_hash_function {
  __host__ __device__ std::uint64_t operator()(Key k) const {
    std::uint64_t x = static_cast<std::uint64_t>(static_cast<std::int64_t>(k));
    x ^= x >> 33;
    x *= 0xff51afd7ed558ccdULL;
    x ^= x >> 33;
    x *= 0xc4ceb9fe1a85ec53ULL;
    x ^= x >> 33;
    return x;
  }
};

template <int CGSize, typename Hash>
struct linear_probing {};
template <int WindowSize>
struct storage {};

namespace op {
struct find_tag {};
}  // namespace op
inline constexpr op::find_tag find{};

namespace detail {

template <typename Key>
__device__ inline Key cas_key(Key* addr, Key expected, Key desired) {
  if constexpr (sizeof(Key) == 4) {
    return static_cast<Key>(atomicCAS(reinterpret_cast<unsigned int*>(addr),
                                      static_cast<unsigned int>(expected),
                                      static_cast<unsigned int>(desired)));
  } else {
    return static_cast<Key>(atomicCAS(reinterpret_cast<unsigned long long*>(addr),
                                      static_cast<unsigned long long>(expected),
                                      static_cast<unsigned long long>(desired)));
  }
}

template <typename Key, typename Value>
struct find_ref {
  using value_type = pair<Key, Value>;
  const value_type* slots;
  std::size_t capacity;
  Key empty;

  __device__ const value_type* end() const { return nullptr; }
  __device__ const value_type* find(Key key) const {
    std::size_t pos = default_hash_function<Key>{}(key) % capacity;
    for (std::size_t step = 0; step < capacity; ++step) {
      const Key k = slots[pos].first;
      if (k == key) return slots + pos;
      if (k == empty) return nullptr;
      pos = pos + 1 == capacity ? 0 : pos + 1;
    }
    return nullptr;
  }
};

template <typename Key, typename Value>
__global__ void fill_kernel(pair<Key, Value>* slots, std::size_t n, Key k, Value v) {
  for (std::size_t i = blockIdx.x * (std::size_t)blockDim.x + threadIdx.x; i < n;
       i += (std::size_t)gridDim.x * blockDim.x) {
    slots[i].first = k;
    slots[i].second = v;
  }
}

template <typename Key, typename Value, typename InputIt>
__global__ void insert_kernel(pair<Key, Value>* slots, std::size_t capacity, Key empty,
                              InputIt first, std::size_t n) {
  for (std::size_t i = blockIdx.x * (std::size_t)blockDim.x + threadIdx.x; i < n;
       i += (std::size_t)gridDim.x * blockDim.x) {
    auto item = *(first + i);
    const Key key = thrust::get<0>(item);
    const Value val = thrust::get<1>(item);
    std::size_t pos = default_hash_function<Key>{}(key) % capacity;
    for (std::size_t step = 0; step < capacity; ++step) {
      const Key prev = cas_key(&slots[pos].first, empty, key);
      if (prev == empty || prev == key) {
        slots[pos].second = val;
        break;
      }
      pos = pos + 1 == capacity ? 0 : pos + 1;
    }
  }
}

template <typename Key, typename Value, typename InputIt, typename OutputIt>
__global__ void find_kernel(find_ref<Key, Value> ref, InputIt first, std::size_t n, OutputIt out,
                            Value missing) {
  for (std::size_t i = blockIdx.x * (std::size_t)blockDim.x + threadIdx.x; i < n;
       i += (std::size_t)gridDim.x * blockDim.x) {
    const auto* hit = ref.find(static_cast<Key>(*(first + i)));
    *(out + i) = hit ? hit->second : missing;
  }
}

inline unsigned blocks_for(std::size_t n) {
  std::size_t b = (n + 255) / 256;
  if (b < 1) b = 1;
  if (b > 65535) b = 65535;
  return static_cast<unsigned>(b);
}

}  // namespace detail

template <typename Key, typename T, typename Extent, cuda::thread_scope Scope, typename KeyEqual,
          typename ProbingScheme, typename Allocator, typename Storage>
class static_map {
 public:
  using value_type = pair<Key, T>;

  static_map(std::size_t capacity, empty_key<Key> ek, empty_value<T> ev)
      : capacity_(capacity < 1 ? 1 : capacity), empty_key_(ek.value), empty_value_(ev.value) {
    slots_ = alloc_.allocate(capacity_);
    detail::fill_kernel<<<detail::blocks_for(capacity_), 256>>>(slots_, capacity_, empty_key_,
                                                                empty_value_);
  }
  ~static_map() {
    if (slots_) alloc_.deallocate(slots_, capacity_);
  }
  static_map(const static_map&) = delete;
  static_map& operator=(const static_map&) = delete;

  template <typename InputIt>
  void insert(InputIt first, InputIt last) {
    const std::size_t n = static_cast<std::size_t>(last - first);
    if (n == 0) return;
    detail::insert_kernel<<<detail::blocks_for(n), 256>>>(slots_, capacity_, empty_key_, first, n);
    cudaStreamSynchronize(0);
  }

  template <typename InputIt, typename OutputIt>
  void find(InputIt first, InputIt last, OutputIt out) const {
    const std::size_t n = static_cast<std::size_t>(last - first);
    if (n == 0) return;
    detail::find_kernel<<<detail::blocks_for(n), 256>>>(ref(cuco::find), first, n, out, empty_value_);
  }

  detail::find_ref<Key, T> ref(op::find_tag) const {
    return detail::find_ref<Key, T>{slots_, capacity_, empty_key_};
  }

  std::size_t capacity() const { return capacity_; }

 private:
  Allocator alloc_{};
  value_type* slots_ = nullptr;
  std::size_t capacity_;
  Key empty_key_;
  T empty_value_;
};

}  // namespace cuco
