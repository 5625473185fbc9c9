// Unique (first-occurrence order) + dense remap of concatenated id arrays.
// Same result as the reference's TensorRelabel (src/tensor_relabel.cu:125-209):
// unique[j] is the j-th distinct id in order of first appearance and
// relabel[i] is the position of input[i] in unique.
//
// Three kernels instead of the reference's cat + 2 fills + 4 thrust passes + CUB
// scan: (1) claim a table slot per distinct id and take the minimum input
// index per slot, remembering each element's slot in the output array;
// (2) flag first occurrences, scan the flags with a decoupled look-back inside
// the same kernel, emit unique ids and the slot -> new id table; (3) remap, and
// put every slot that was used back to "empty", so the table needs no memset
// between calls.  Every element probes the table once (the reference four times).
// The element counts may live on the device (written by an earlier kernel), so a
// chain of hops can be queued without the host knowing any size.
#include "relabel.cuh"

namespace shmt {

constexpr uint64_t kRelDirectMinTableBytes = 32ull << 20;

__device__ __forceinline__ void resolve_sizes(Parts& ps, int64_t* numel) {
  if (ps.dev_n1) {  // |part 0| from the device if given there, else the host's start[1]
    const int64_t a = ps.dev_n0 ? *ps.dev_n0 : ps.start[1], b = *ps.dev_n1;
    ps.start[0] = 0;
#pragma unroll
    for (int q = 1; q <= kMaxParts; ++q) ps.start[q] = q == 1 ? a : a + b;
  }
  *numel = ps.start[kMaxParts];
}

__device__ __forceinline__ int64_t part_elem(const Parts& ps, int64_t i) {
  int p = 0;
#pragma unroll
  for (int q = 1; q < kMaxParts; ++q)
    if (q < ps.n && i >= ps.start[q]) p = q;
  return load_int(ps.ptr[p], ps.is64, i - ps.start[p]);
}

// Largest id of the input, read as an unsigned number (so that a negative id counts as huge).
__global__ void __launch_bounds__(kRelThreads)
relabel_range_kernel(Parts ps, unsigned long long* range) {
  pdl_prologue();
  int64_t numel;
  resolve_sizes(ps, &numel);
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  const int64_t gtid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  unsigned long long m = 0;
  int64_t done = 0;  // elements covered by the 16-byte loads below
  if (ps.n == 1 && (reinterpret_cast<uintptr_t>(ps.ptr[0]) & 15) == 0) {
    // one aligned array: 16-byte loads, four per thread in flight
    const int per = ps.is64 ? 2 : 4;
    const int64_t n_vec = numel / per;
    const uint4* src = static_cast<const uint4*>(ps.ptr[0]);
    for (int64_t v = gtid; v < n_vec; v += 4 * stride) {
      uint4 x[4];
#pragma unroll
      for (int u = 0; u < 4; ++u)
        x[u] = v + u * stride < n_vec ? __ldg(src + v + u * stride) : make_uint4(0, 0, 0, 0);
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        if (ps.is64) {
          m = max(m, ((unsigned long long)x[u].y << 32) | x[u].x);
          m = max(m, ((unsigned long long)x[u].w << 32) | x[u].z);
        } else {
          m = max(m, (unsigned long long)(long long)(int)x[u].x);
          m = max(m, (unsigned long long)(long long)(int)x[u].y);
          m = max(m, (unsigned long long)(long long)(int)x[u].z);
          m = max(m, (unsigned long long)(long long)(int)x[u].w);
        }
      }
    }
    done = n_vec * per;
  }
  for (int64_t i = done + gtid; i < numel; i += 4 * stride) {
    long long v[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) v[u] = i + u * stride < numel ? part_elem(ps, i + u * stride) : 0;
#pragma unroll
    for (int u = 0; u < 4; ++u) m = max(m, (unsigned long long)v[u]);
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) m = max(m, __shfl_xor_sync(0xffffffffu, m, o));
  if ((threadIdx.x & 31) == 0 && m) atomicMax(range, m);
}

__global__ void __launch_bounds__(kRelThreads)
relabel_insert_kernel(Parts ps, RelTable t, void* __restrict__ out, int64_t* status,
                      const unsigned long long* __restrict__ range) {
  pdl_prologue();
  int64_t numel;
  resolve_sizes(ps, &numel);
  // The table is provisioned for the largest input the caller allows; hash into only as
  // much of it as this input needs (load <= 0.5), so a small input stays in a small,
  // cache-resident part.  Only the inserting code hashes; the rest follows recorded slots.
  const uint32_t mask = relabel_mask_for(numel, t.mask);
  // ids that all fit the table are their own slots: a frontier of densely numbered nodes then
  // touches a compact, cache-resident part of the table instead of one line per distinct id
  const bool direct = range != nullptr && *range <= (unsigned long long)mask;
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < numel; i += stride) {
    bool maybe_first;
    const uint32_t pos = relabel_insert_one(t.slots, mask, part_elem(ps, i), (unsigned)i, status, &maybe_first,
                                            direct);
    store_int(out, ps.is64, i, relabel_pack(pos, maybe_first, ps.is64, t.mask));
  }
}

template <int ITEMS>
__global__ void __launch_bounds__(kRelThreads)
relabel_compact_kernel(Parts ps, RelTable t, const void* __restrict__ slot_of,
                       void* __restrict__ unique, TileStates st, int64_t* ticket, int64_t* status,
                       int64_t* result, HostPost post) {
  __shared__ int64_t warp_sums[32];
  __shared__ int64_t s_total;
  __shared__ int64_t s_prefix;
  __shared__ int s_tile;
  pdl_prologue();
  int64_t numel;
  resolve_sizes(ps, &numel);
  constexpr int kTile = kRelThreads * ITEMS;
  const int64_t n_tiles = (numel + kTile - 1) / kTile;
  const int tile = take_tile(ticket, &s_tile);
  if (tile >= n_tiles) {  // the grid is sized for the largest input the caller allows
    if (numel == 0 && tile == 0 && threadIdx.x == 0) {
      *result = 0;
      post_to_host(post);
    }
    return;
  }
  const int64_t base = (int64_t)tile * kTile + (int64_t)threadIdx.x * ITEMS;
  uint32_t pos[ITEMS];
  unsigned maybe = 0, is_first = 0;  // one bit per element of this thread
  // the thread's ITEMS slot numbers: 16-byte loads when the whole run lies inside the input
  // and the array is aligned, else one by one
  if (base + ITEMS <= numel && (reinterpret_cast<uintptr_t>(slot_of) & 15) == 0) {
    if (ps.is64) {
      const ulonglong2* src = reinterpret_cast<const ulonglong2*>(slot_of) + base / 2;
#pragma unroll
      for (int q = 0; q < ITEMS / 2; ++q) {
        const ulonglong2 v = __ldg(src + q);
        bool m0, m1;
        pos[2 * q] = relabel_unpack64(v.x, &m0);
        pos[2 * q + 1] = relabel_unpack64(v.y, &m1);
        maybe |= ((unsigned)m0 << (2 * q)) | ((unsigned)m1 << (2 * q + 1));
      }
    } else {
      const uint4* src = reinterpret_cast<const uint4*>(slot_of) + base / 4;
#pragma unroll
      for (int q = 0; q < ITEMS / 4; ++q) {
        const uint4 v = __ldg(src + q);
        const uint32_t raw[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          bool m;
          pos[4 * q + e] = relabel_unpack32(raw[e], t.mask, &m);
          maybe |= (unsigned)m << (4 * q + e);
        }
      }
    }
  } else {
#pragma unroll
    for (int j = 0; j < ITEMS; ++j) {
      pos[j] = 0;
      if (base + j < numel) {
        bool m;
        pos[j] = relabel_unpack(slot_of, ps.is64, base + j, t.mask, &m);
        maybe |= (unsigned)m << j;
      }
    }
  }
  // only an element the inserting pass did not rule out has to look at its slot
#pragma unroll
  for (int j = 0; j < ITEMS; ++j)
    if ((maybe >> j & 1u) && __ldcg(&t.slots[pos[j]].first) == (unsigned)(base + j)) is_first |= 1u << j;
  const int64_t cnt = __popc(is_first);
  const int64_t local = block_exclusive_scan(cnt, warp_sums, &s_total);
  if (threadIdx.x < 32) {
    const int64_t p = lookback_exclusive_prefix(st, tile, s_total, status);
    if (threadIdx.x == 0) {
      s_prefix = p;
      if (tile == n_tiles - 1) st_relaxed64(result, p + s_total);
    }
  }
  __syncthreads();
  if (threadIdx.x == 0) post_when_last(post, n_tiles);
  int64_t uid = s_prefix + local;
#pragma unroll
  for (int j = 0; j < ITEMS; ++j) {
    if (is_first >> j & 1u) {
      store_int(unique, ps.is64, uid, part_elem(ps, base + j));
      t.slots[pos[j]].newid = (unsigned)uid;
      ++uid;
    }
  }
}

__global__ void __launch_bounds__(kRelThreads)
relabel_remap_kernel(Parts ps, RelTable t, void* out) {
  pdl_prologue();
  int64_t numel;
  resolve_sizes(ps, &numel);
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < numel; i += stride) {
    bool maybe_first;
    const uint32_t pos = relabel_unpack(out, ps.is64, i, t.mask, &maybe_first);
    const uint4 slot = __ldcg(reinterpret_cast<const uint4*>(t.slots + pos));  // key lo, key hi, first, newid
    store_int(out, ps.is64, i, (int64_t)slot.w);
    // leave the slot empty for the next call: the id's first occurrence does it, once (the new id
    // stays, because another element of the same id may not have read it yet)
    if (maybe_first && slot.z == (unsigned)i)
      *reinterpret_cast<uint4*>(t.slots + pos) = make_uint4(0xFFFFFFFFu, 0xFFFFFFFFu, 0xFFFFFFFFu, slot.w);
  }
}

// Table for up to `numel_bound` ids at load <= 0.5, in the context's block whose keys and
// first-index words are all ones between calls (whatever the capacity, so regions of different
// capacities may overlap freely); the new-id words need no initial value.
uint64_t relabel_capacity(int64_t numel_bound) {
  uint64_t cap = 64;
  while (cap < (uint64_t)numel_bound * 2) cap <<= 1;
  return cap;
}

int relabel_table(shmt_ctx* ctx, int64_t numel_bound, RelTable* t, cudaStream_t s) {
  const uint64_t cap = relabel_capacity(numel_bound);
  if (int rc = ctx_reserve_table(ctx, cap * sizeof(RelSlot), s)) return rc;
  t->slots = reinterpret_cast<RelSlot*>(ctx->table);
  t->mask = (uint32_t)(cap - 1);
  return SHMT_OK;
}

int launch_relabel(shmt_ctx* ctx, const Parts& ps, int64_t numel_bound, void* out_unique, void* out_relabel, TileStates st, int64_t* ticket,
                   int64_t* status, int64_t* result, cudaStream_t s, bool inserted, bool pdl,
                   const HostPost* post, int64_t* range) {
  RelTable t;
  if (int rc = relabel_table(ctx, numel_bound, &t, s)) return rc;
  const int64_t n_tiles = (numel_bound + kRelTile - 1) / kRelTile;
  int64_t blocks = (numel_bound + kRelThreads - 1) / kRelThreads;
  const int64_t cap_blocks = (int64_t)sm_count() * 16;
  const unsigned grid = (unsigned)(blocks < cap_blocks ? blocks : cap_blocks);
  if (!inserted) {
    unsigned long long* r = reinterpret_cast<unsigned long long*>(range);
    if (r) SHMT_CUDA_TRY(launch_kernel(pdl, relabel_range_kernel, grid, kRelThreads, 0, s, ps, r));
    SHMT_CUDA_TRY(launch_kernel(pdl, relabel_insert_kernel, grid, kRelThreads, 0, s, ps, t, out_relabel, status,
                                (const unsigned long long*)r));
  }
  if (numel_bound >= kRelLargeInput) {
    const int64_t big_tiles = (numel_bound + kRelThreads * kRelItemsLarge - 1) / (kRelThreads * kRelItemsLarge);
    SHMT_CUDA_TRY(launch_kernel(pdl, relabel_compact_kernel<kRelItemsLarge>, (unsigned)big_tiles, kRelThreads, 0, s,
                                ps, t, (const void*)out_relabel, out_unique, st, ticket, status, result,
                                post ? *post : HostPost{}));
  } else {
    SHMT_CUDA_TRY(launch_kernel(pdl, relabel_compact_kernel<kRelItems>, (unsigned)n_tiles, kRelThreads, 0, s, ps, t,
                                (const void*)out_relabel, out_unique, st, ticket, status, result,
                                post ? *post : HostPost{}));
  }
  SHMT_CUDA_TRY(launch_kernel(pdl, relabel_remap_kernel, grid, kRelThreads, 0, s, ps, t, out_relabel));
  SHMT_CUDA_TRY(cudaGetLastError());
  return SHMT_OK;
}

}  // namespace shmt

using namespace shmt;

extern "C" int shmt_relabel(shmt_ctx* ctx, const void* const* parts, const int64_t* part_sizes,
                            int n_parts, int dtype, void* out_unique, void* out_relabel,
                            int64_t* n_unique_host, void* stream) {
  SHMT_REQUIRE(ctx != nullptr, "shmt_relabel: ctx is null");
  SHMT_REQUIRE(valid_int_dtype(dtype), "shmt_relabel: ids can only be int32 or int64");
  SHMT_REQUIRE(n_parts >= 0 && n_parts <= kMaxParts, "shmt_relabel: 0..%d parts", kMaxParts);
  SHMT_REQUIRE(n_parts == 0 || (parts && part_sizes), "shmt_relabel: parts/part_sizes are null");
  Parts ps{};
  ps.n = n_parts;
  ps.is64 = dtype == SHMT_I64;
  int64_t numel = 0;
  for (int p = 0; p < n_parts; ++p) {
    SHMT_REQUIRE(part_sizes[p] >= 0, "shmt_relabel: part %d has negative size", p);
    SHMT_REQUIRE(part_sizes[p] == 0 || parts[p] != nullptr, "shmt_relabel: part %d is null", p);
    ps.ptr[p] = parts[p];
    ps.start[p] = numel;
    numel += part_sizes[p];
  }
  for (int p = n_parts; p <= kMaxParts; ++p) ps.start[p] = numel;
  SHMT_REQUIRE(numel < ((int64_t)1 << 30), "shmt_relabel: %lld ids is too many (limit 2^30)",
               (long long)numel);
  if (numel == 0) {
    if (n_unique_host) *n_unique_host = 0;
    return SHMT_OK;
  }
  SHMT_REQUIRE(out_unique && out_relabel, "shmt_relabel: outputs are null");
  DeviceGuard guard(ctx->device);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int64_t n_tiles = (numel + kRelTile - 1) / kRelTile;
  const size_t states = (tile_state_bytes(n_tiles) + 255) & ~(size_t)255;
  if (int rc = ctx_reserve(ctx, states)) return rc;
  TileStates st = carve_tile_states(ctx->region(), n_tiles);
  // result words + tile descriptors to zero
  SHMT_CUDA_TRY(cudaMemsetAsync(ctx->scratch, 0, 256 + tile_state_bytes(n_tiles), s));
  int64_t* w = ctx->d_words();
  // with a count to return, the compact kernel posts it and the call returns while the remap
  // kernel runs; the next user of the context waits for that kernel first
  HostPost post{};
  if (n_unique_host) post = ctx_begin_post(ctx, w, 4, w + W_DONE);
  // a table that fits the L2 cache gains nothing from compact slots; a larger one may
  int64_t* range = relabel_capacity(numel) * sizeof(RelSlot) > kRelDirectMinTableBytes ? w + W_RANGE : nullptr;
  if (int rc = launch_relabel(ctx, ps, numel, out_unique, out_relabel, st, w + W_TICKET,
                              w + W_STATUS, w + W_RESULT, s, false, false,
                              n_unique_host ? &post : nullptr, range))
    return rc;
  if (n_unique_host) {
    if (int rc = ctx_mark_tail(ctx, s)) return rc;
    if (int rc = ctx_await_post(ctx, post, s)) return rc;
    if (int rc = ctx_status_of_words(ctx, "shmt_relabel")) return rc;
    *n_unique_host = ctx->h_words[W_RESULT];
  }
  return SHMT_OK;
}
