// Threaded CPU restatement of the hot path, for the timed CPU baseline.
// TEST / BENCH INFRASTRUCTURE, NOT PRODUCT CODE: nothing under shmtensor_b200/
// links or loads this file.
//
// The reference has no CPU sampler or CPU relabel (its scripts compare against
// DGL), so these follow the reference's CUDA algorithms on host threads:
//   oracle_gather       src/cache_feature_fetch.cu:27-45   out[i] = table[idx[i]]
//   oracle_sample_hop   src/cache_graph_sampling.cu:70-83 (picks + exclusive scan)
//                       and :109-145 / :163-176 (copy if deg <= k, else reservoir
//                       over positions; with replacement k draws rand % deg)
//   oracle_relabel      src/tensor_relabel.cu:147-203 (first-occurrence unique + remap)
// Build: g++ -O3 -fopenmp -shared -fPIC (oracle/build_oracle.py).
#include <omp.h>
#include <stdint.h>
#include <string.h>

#include <vector>

namespace {

inline uint64_t splitmix(uint64_t& s) {
  uint64_t z = (s += 0x9E3779B97F4A7C15ULL);
  z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ULL;
  z = (z ^ (z >> 27)) * 0x94D049BB133111EBULL;
  return z ^ (z >> 31);
}

inline uint64_t mix(uint64_t x) {
  x ^= x >> 33;
  x *= 0xff51afd7ed558ccdULL;
  x ^= x >> 33;
  x *= 0xc4ceb9fe1a85ec53ULL;
  x ^= x >> 33;
  return x;
}

template <typename IxT>
void sample_rows(const int64_t* indptr, const IxT* indices, const int64_t* seeds, int64_t n,
                 int64_t k, int replace, uint64_t seed, const int64_t* sub_indptr, IxT* out) {
#pragma omp parallel
  {
    std::vector<int64_t> res((size_t)k);
#pragma omp for schedule(dynamic, 64)
    for (int64_t i = 0; i < n; ++i) {
      const int64_t b = indptr[seeds[i]], deg = indptr[seeds[i] + 1] - b;
      IxT* o = out + sub_indptr[i];
      const IxT* in = indices + b;
      uint64_t s = seed ^ mix((uint64_t)i);
      if (replace) {
        if (deg > 0)
          for (int64_t p = 0; p < k; ++p) o[p] = in[splitmix(s) % (uint64_t)deg];
      } else if (deg <= k) {
        for (int64_t p = 0; p < deg; ++p) o[p] = in[p];
      } else {
        for (int64_t p = 0; p < k; ++p) res[p] = p;
        for (int64_t q = k; q < deg; ++q) {
          const uint64_t r = splitmix(s) % (uint64_t)(q + 1);
          if (r < (uint64_t)k) res[r] = q;
        }
        for (int64_t p = 0; p < k; ++p) o[p] = in[res[p]];
      }
    }
  }
}

}  // namespace

extern "C" {

int oracle_num_threads(void) { return omp_get_max_threads(); }

// The launcher of a multi-process job may export OMP_NUM_THREADS=1; the CPU baseline is meant to
// use every core the process may run on, so the caller says how many.
void oracle_set_threads(int n) {
  if (n > 0) omp_set_num_threads(n);
}

void oracle_gather(const char* table, const int64_t* idx, int64_t n, int64_t row_bytes, char* out) {
#pragma omp parallel for schedule(static)
  for (int64_t i = 0; i < n; ++i)
    memcpy(out + i * row_bytes, table + idx[i] * row_bytes, (size_t)row_bytes);
}

// indices_is64: element type of `indices` / `out`.  Returns nnz.
int64_t oracle_sample_hop(const int64_t* indptr, const void* indices, int indices_is64,
                          const int64_t* seeds, int64_t n, int64_t k, int replace, uint64_t seed,
                          int64_t* sub_indptr, void* out) {
  sub_indptr[0] = 0;
  for (int64_t i = 0; i < n; ++i) {
    const int64_t deg = indptr[seeds[i] + 1] - indptr[seeds[i]];
    const int64_t c = replace ? (deg == 0 ? 0 : k) : (deg < k ? deg : k);
    sub_indptr[i + 1] = sub_indptr[i] + c;
  }
  if (indices_is64)
    sample_rows<int64_t>(indptr, (const int64_t*)indices, seeds, n, k, replace, seed, sub_indptr,
                         (int64_t*)out);
  else
    sample_rows<int32_t>(indptr, (const int32_t*)indices, seeds, n, k, replace, seed, sub_indptr,
                         (int32_t*)out);
  return sub_indptr[n];
}

// Open-addressing build + lookup of int64 keys -> int32 slots on all cores: the CPU stand-in
// for the map half of the update path (cuco insert / find, include/cuco_hashmap.cuh:66-87).
// table: 2 * cap int64 words, {key, value} pairs, cap a power of two.  Returns hits.
int64_t oracle_map_build_query(const int64_t* keys, int64_t n, int64_t* table, int64_t cap,
                               const int64_t* req, int64_t n_req, int32_t* out) {
  const uint64_t mask = (uint64_t)cap - 1;
#pragma omp parallel for schedule(static)
  for (int64_t i = 0; i < 2 * cap; ++i) table[i] = -1;
#pragma omp parallel for schedule(static)
  for (int64_t i = 0; i < n; ++i) {
    uint64_t pos = mix((uint64_t)keys[i]) & mask;
    while (true) {
      int64_t expected = -1;
      if (__atomic_compare_exchange_n(&table[2 * pos], &expected, keys[i], false, __ATOMIC_RELAXED,
                                      __ATOMIC_RELAXED) ||
          expected == keys[i]) {
        table[2 * pos + 1] = i;
        break;
      }
      pos = (pos + 1) & mask;
    }
  }
  int64_t hits = 0;
#pragma omp parallel for schedule(static) reduction(+ : hits)
  for (int64_t i = 0; i < n_req; ++i) {
    uint64_t pos = mix((uint64_t)req[i]) & mask;
    int32_t v = -1;
    while (table[2 * pos] != -1) {
      if (table[2 * pos] == req[i]) {
        v = (int32_t)table[2 * pos + 1];
        break;
      }
      pos = (pos + 1) & mask;
    }
    out[i] = v;
    hits += v >= 0;
  }
  return hits;
}

// out[idx[i]] = rows[i]: the row-write half of the update path (data[ids] = upd,
// example/test_cache_set.py:183-184).
void oracle_scatter(char* table, const int64_t* idx, int64_t n, int64_t row_bytes, const char* rows) {
#pragma omp parallel for schedule(static)
  for (int64_t i = 0; i < n; ++i)
    memcpy(table + idx[i] * row_bytes, rows + i * row_bytes, (size_t)row_bytes);
}

// First-occurrence unique + remap of int64 ids (ids != -1).  Returns n_unique.
int64_t oracle_relabel(const int64_t* in, int64_t n, int64_t* unique, int64_t* relabel) {
  if (n == 0) return 0;
  uint64_t cap = 16;
  while (cap < (uint64_t)n * 2) cap <<= 1;
  std::vector<int64_t> keys(cap, -1), ids(cap, 0);
  int64_t n_unique = 0;
  for (int64_t i = 0; i < n; ++i) {
    uint64_t pos = mix((uint64_t)in[i]) & (cap - 1);
    while (keys[pos] != -1 && keys[pos] != in[i]) pos = (pos + 1) & (cap - 1);
    if (keys[pos] == -1) {
      keys[pos] = in[i];
      ids[pos] = n_unique;
      unique[n_unique++] = in[i];
    }
    relabel[i] = ids[pos];
  }
  return n_unique;
}

}  // extern "C"
