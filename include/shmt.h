/*
 * libshmt — C-ABI of the B200 (sm_100a) GPU-cache hot path.
 *
 * Every entry point is plain C: raw pointers, sizes, dtype codes and an opaque
 * cudaStream_t passed as void*.  No torch / pybind types cross this boundary.
 * Each function returns an int status (SHMT_OK == 0); shmt_last_error() gives
 * the text of the last failure on the calling thread.  Nothing here ever calls
 * exit(): the reference's CUDA_CALL (include/common.h:15-27) kills the process,
 * this library reports.
 *
 * Each declaration cites the reference interface it replaces, as
 * <file>:<line> inside the gpzlx1/ShmTensor source tree.
 */
#ifndef SHMT_H_
#define SHMT_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ---- status codes -------------------------------------------------------- */
#define SHMT_OK 0
#define SHMT_ERR_INVALID 1  /* bad argument (null, dtype code, alignment, size)   */
#define SHMT_ERR_CUDA 2     /* a CUDA runtime call failed                         */
#define SHMT_ERR_CAPACITY 3 /* hashmap full: a probe ran the whole table          */
#define SHMT_ERR_TIMEOUT 4  /* a bounded device-side wait (look-back) gave up     */
#define SHMT_ERR_OS 5       /* shm_open / mmap / file error (errno in the text)   */

/* ---- integer dtype codes (ids, keys, slots, indptr, indices) -------------- */
#define SHMT_I32 0
#define SHMT_I64 1

const char* shmt_last_error(void);
int shmt_version(void);

/* ---- context --------------------------------------------------------------
 * Owns the per-device scratch every op needs (look-back tile states, relabel
 * table, device/pinned result words).  Scratch grows on demand and is reused,
 * so steady-state calls allocate nothing.  One context serves one stream at a
 * time: two ops on the same context must not overlap on the GPU; callers that
 * use several streams keep one context per stream.
 * Replaces the reference's per-call torch::empty / raw_allocate temporaries
 * (src/cache_graph_sampling.cu:30-45,50-56; src/tensor_relabel.cu:141-177).   */
typedef struct shmt_ctx shmt_ctx;
int shmt_ctx_create(int device, shmt_ctx** out);
int shmt_ctx_destroy(shmt_ctx* ctx);
int64_t shmt_ctx_scratch_bytes(const shmt_ctx* ctx);
/* Size the context before the first call of a new shape, so that no hot call has to free and
 * allocate device memory (which stalls the device): at least scratch_bytes of look-back state
 * (16 bytes per tile; a scan of n items of 8 bytes needs n / 512 bytes) and a relabel table for
 * relabel_ids ids.  shmt_ctx_reserve_minibatch sizes both for shmt_sample_minibatch calls of up
 * to n_seeds seeds with these fan-outs.  No counterpart in the reference, which allocates
 * temporaries on every call (src/cache_graph_sampling.cu:50-56).                          */
int shmt_ctx_reserve(shmt_ctx* ctx, int64_t scratch_bytes, int64_t relabel_ids, void* stream);
int shmt_ctx_reserve_minibatch(shmt_ctx* ctx, int64_t n_seeds, const int64_t* fanouts,
                               int n_hops, void* stream);
/* Wait for `stream` and report what the last asynchronous op on this context (a scan,
 * or a hop / relabel called without a host result pointer) left in its status word:
 * SHMT_OK, SHMT_ERR_TIMEOUT or SHMT_ERR_CAPACITY.  No counterpart in the reference.  */
int shmt_ctx_check(shmt_ctx* ctx, void* stream);

/* ---- static hashmap --------------------------------------------------------
 * Open addressing, linear probing over 16-byte {int64 key, int64 value} slots,
 * probed by 4-lane tiles (one 64-byte window per step).  Empty key = -1.
 * Replaces pycuco::CUCOHashmapWrapper / CUCOHashmap
 * (include/cuco_hashmap.h:12-25, include/cuco_hashmap.cuh:49-93,
 *  src/cuco_hashmap.cu:10-41).                                                */
typedef struct shmt_map shmt_map;

/* bytes of table storage for a map of `capacity` requested slots that will hold
 * about `expected_keys` keys (0 = unknown).  The table is provisioned for load
 * <= 0.5 on the expected keys, and never below capacity + 1/16: short probes matter
 * more to the kernels than table bytes.                                           */
int64_t shmt_map_table_bytes(int64_t capacity, int64_t expected_keys);

/* Create an empty map.  `capacity` is what shmt_map_capacity() reports
 * (the reference reports ceil(n / load_factor), include/cuco_hashmap.cuh:62,75).
 * table_buf: device buffer of shmt_map_table_bytes(capacity, expected_keys)
 * bytes, 16-byte aligned, that must outlive the map; NULL lets the map cudaMalloc
 * its own.                                                                      */
int shmt_map_create(int device, int64_t capacity, int64_t expected_keys,
                    int key_dtype, int val_dtype, void* table_buf, void* stream,
                    shmt_map** out);

/* insert_or_assign of n (key, value) pairs; keys -1 and -2 are reserved and
 * skipped.  Synchronises `stream` and returns SHMT_ERR_CAPACITY if the table
 * overflowed.  Bulk-insert half of include/cuco_hashmap.cuh:68-70; inserting
 * into an existing map is new.  Slots freed by shmt_map_erase are taken again. */
int shmt_map_insert(shmt_map* map, const void* keys, const void* values,
                    int64_t n, void* stream);

/* Remove n keys (key dtype of the map).  out_values, if not NULL, receives per
 * key the value it had (value dtype of the map) or -1 if it was absent; a key
 * listed twice reports its value once.  Synchronises `stream` (the key count
 * is read back).  Must not overlap an insert into the same map.  No counterpart
 * in the reference, whose map is built once (include/cuco_hashmap.cuh:49-93):
 * it is what lets a cache evict rows and hand their slots to new ids.          */
int shmt_map_erase(shmt_map* map, const void* keys, int64_t n, void* out_values,
                   void* stream);

/* out[i] = value of requests[i] or -1 (include/cuco_hashmap.cuh:81-87).
 * Requests are first narrowed to the key dtype, as the reference's
 * requests.to(key_type_) does (src/cuco_hashmap.cu:29).  out has the value
 * dtype.  Asynchronous on `stream`.                                           */
int shmt_map_query(const shmt_map* map, const void* requests, int req_dtype,
                   int64_t n, void* out, void* stream);

int64_t shmt_map_capacity(const shmt_map* map);     /* include/cuco_hashmap.h:20 */
int64_t shmt_map_memory_usage(const shmt_map* map); /* include/cuco_hashmap.h:21 */
int64_t shmt_map_size(const shmt_map* map);         /* distinct keys stored       */
int shmt_map_key_dtype(const shmt_map* map);
int shmt_map_val_dtype(const shmt_map* map);
int shmt_map_destroy(shmt_map* map);

/* ---- feature fetch ---------------------------------------------------------
 * out[i] = hit(i) ? gpu_base[slot(i)] : host_base[idx[i]], rows of row_bytes.
 *   map  != NULL : slot from a fused probe   -> CacheTensorFetch
 *                                               (src/cache_feature_fetch.cu:131-185)
 *   mask != NULL : slot = mask[i] (>= 0 hit) -> CacheTensorFetchWithMask (:226-272)
 *   both NULL    : every row from host_base  -> UVATensorFetch (:47-87)
 * host_base is pinned/registered host memory read through UVA (or any device-
 * visible pointer).  Asynchronous on `stream`.                                */
int shmt_fetch(const shmt_map* map, const void* mask, int mask_dtype,
               const void* host_base, const void* gpu_base, const void* idx,
               int idx_dtype, int64_t n, int64_t row_bytes, void* out,
               void* stream);

/* Fetch kernels bound every device-side wait; one that gives up records a code
 * here instead of hanging.  Synchronises the device, returns the code of the
 * current device (0 = none) and clears it.  No counterpart in the reference.   */
int shmt_device_fault(int* out_code);

/* Partitioned cache: value = (owner << owner_shift) | slot; the row is read
 * from bases[owner] (this GPU's buffer or a peer's, by plain NVLink loads).
 * No counterpart in the reference (it is single-GPU).                         */
int shmt_fetch_partitioned(const shmt_map* map, const void* const* bases,
                           int n_bases, int owner_shift, const void* host_base,
                           const void* idx, int idx_dtype, int64_t n,
                           int64_t row_bytes, void* out, void* stream);

/* ---- feature set -----------------------------------------------------------
 * hit(i) ? gpu_base[slot(i)] = update[i] : host_base[idx[i]] = update[i].
 * Same three modes: CacheTensorSet (src/cache_feature_set.cu:118-165),
 * CacheTensorSetWithMask (:209-248), UVATensorSet (:39-75).  Duplicate ids
 * have no defined winner, as in the reference.                                */
int shmt_set(const shmt_map* map, const void* mask, int mask_dtype,
             void* host_base, void* gpu_base, const void* idx, int idx_dtype,
             int64_t n, int64_t row_bytes, const void* update, void* stream);

/* Fused insert/overwrite: key[i] is inserted with value slots[i] unless it is
 * already present (then its stored slot is kept); update[i] is written to
 * gpu_base[slot].  Synchronises and reports SHMT_ERR_CAPACITY like
 * shmt_map_insert.  New entry point (the reference never inserts into a live
 * map; src/cache_feature_set.cu:93-116 only overwrites).                      */
int shmt_insert_set(shmt_map* map, void* gpu_base, const void* keys,
                    int key_dtype, const void* slots, int slots_dtype,
                    int64_t n, int64_t row_bytes, const void* update,
                    void* stream);

/* ---- scan ------------------------------------------------------------------
 * In-place prefix sum by a single-pass decoupled look-back kernel, wrapping
 * integer arithmetic.  exclusive=0: the intended semantics of thrust_scan
 * (src/thrust_scan.cu:9-18); exclusive=1: cub_exclusiveSum
 * (src/cache_graph_sampling.cu:30-45, src/tensor_relabel.cu:11-26).           */
int shmt_scan(shmt_ctx* ctx, void* data, int dtype, int64_t n, int exclusive,
              void* stream);

/* The same scan for callers that must not allocate device memory at the point of
 * the call: a plugin inside a host application that owns and pre-plans every byte of
 * device memory, a serving loop with a hard latency bound (cudaMalloc and cudaFree
 * stall the whole device, and a context's scratch may have to grow), or any code
 * that runs where the CUDA allocator may not be entered.  The look-back state lives
 * in a fixed array inside the library (about 33 KB per GPU, held from library load
 * to process exit), so the call needs no context and never calls cudaMalloc or
 * cudaFree: it is one memset of that state plus one kernel on `stream`.
 * Limit: n <= 16,777,216 items; larger inputs are refused with SHMT_ERR_INVALID.
 * Run it with the device that owns `data` current.  The first call on a device also
 * looks up the array's device address (a runtime query, not an allocation); let
 * that first call happen before any stream capture is started.  All calls on a
 * device share the one array, which keeps what the last call left in it (each call
 * clears the part it uses first): two calls that overlap on the GPU — different
 * streams with no dependency between them — corrupt each other, calls ordered on
 * one stream do not.  This entry point has no counterpart in the reference.        */
int shmt_scan_static(void* data, int dtype, int64_t n, int exclusive, void* stream);
/* Wait for `stream` and report whether the last shmt_scan_static call on the current device
 * ran into its bounded look-back wait (SHMT_ERR_TIMEOUT) or not (SHMT_OK).  Allocates nothing
 * either.  This entry point has no counterpart in the reference.                          */
int shmt_scan_static_check(void* stream);

/* Test hook for the failure path of every look-back scan: runs one warp whose predecessor
 * tile never publishes, with a short spin limit, and returns what the host sees --
 * SHMT_ERR_TIMEOUT -- leaving the context usable.  Nothing faults, traps or hangs.
 * No counterpart in the reference.                                                    */
int shmt_debug_lookback_timeout(shmt_ctx* ctx, void* stream);

/* ---- relabel ---------------------------------------------------------------
 * Concatenation of `n_parts` id arrays -> distinct ids in first-occurrence
 * order (out_unique, capacity = total) and, for every input element, the index
 * of its id in out_unique (out_relabel, total elements, same dtype).  Ids must
 * not be -1.  If n_unique_host != NULL the call waits for the number of distinct
 * ids and stores it there; it returns as soon as that number is known, while the
 * last kernel may still be writing out_relabel (consume the outputs in `stream`
 * order, or synchronise).  TensorRelabel (src/tensor_relabel.cu:125-209).        */
int shmt_relabel(shmt_ctx* ctx, const void* const* parts,
                 const int64_t* part_sizes, int n_parts, int dtype,
                 void* out_unique, void* out_relabel, int64_t* n_unique_host,
                 void* stream);

/* ---- neighbour sampling ----------------------------------------------------
 * One fan-out hop over a CSR, fused into one kernel (probe, degree, look-back
 * scan, sample).  For seed i: row = seeds[i]; if a map is given and holds row,
 * the adjacency is gpu_indices[gpu_indptr[slot] .. gpu_indptr[slot+1]), else
 * indices[indptr[row] .. indptr[row+1]) (UVA).  Picks per seed:
 * replace ? (deg ? k : 0) : min(deg, k); deg <= k copies the row in CSR order,
 * otherwise k distinct uniform positions (without replacement) or k iid
 * uniform positions (with).  out_sub_indptr: n+1 entries of indptr dtype;
 * out_sub_indices: capacity n*k entries of indices dtype.  If nnz_host != NULL
 * the call waits for out_sub_indptr[n] and stores it there; it returns as soon as
 * that number is known, while the kernel may still be writing rows (consume the
 * outputs in `stream` order, or synchronise).
 * CSRWiseSampling / CSRWiseCacheSampling
 * (src/cache_graph_sampling.cu:179-220, :382-426; kernels :91-177, :291-380;
 *  GetSubIndptr(:47-89) / GetSubIndptrWithCache(:222-289)).
 * gpu_indptr / gpu_indices / map may all be NULL (uncached).  Randomness is
 * Philox4x32-10 keyed by rng_seed, countered by (rng_offset, seed index, lane). */
int shmt_sample_hop(shmt_ctx* ctx, const void* indptr, int indptr_dtype,
                    const void* indices, int indices_dtype,
                    const void* gpu_indptr, const void* gpu_indices,
                    const shmt_map* map, const void* seeds, int seeds_dtype,
                    int64_t n, int64_t k, int replace, uint64_t rng_seed,
                    uint64_t rng_offset, void* out_sub_indptr,
                    void* out_sub_indices, int64_t* nnz_host, void* stream);

/* The same hop that also reports, for every sampled neighbour, its edge id: its position in
 * the full `indices` array, in the dtype of indptr (out_edge_ids, capacity n*k, parallel to
 * out_sub_indices).  For a cached graph gpu_edge_base[slot] must hold where the cached row starts
 * in the full array (shmt_subcsr_edge_base).  The reference hands an empty edge-id tensor to its
 * block builder (python/shmtensor/sampling.py:9-20,137-142); this is what would fill it.      */
int shmt_sample_hop_eids(shmt_ctx* ctx, const void* indptr, int indptr_dtype,
                         const void* indices, int indices_dtype,
                         const void* gpu_indptr, const void* gpu_indices,
                         const void* gpu_edge_base, const shmt_map* map,
                         const void* seeds, int seeds_dtype, int64_t n, int64_t k,
                         int replace, uint64_t rng_seed, uint64_t rng_offset,
                         void* out_sub_indptr, void* out_sub_indices,
                         void* out_edge_ids, int64_t* nnz_host, void* stream);

/* Weighted hop: neighbours are picked with probabilities proportional to `weights` (one positive
 * float per edge, parallel to `indices`; gpu_weights parallel to gpu_indices for a cached graph;
 * a weight that is not positive counts as the smallest positive one).  Without replacement
 * (fan-out <= 32) by exponential keys -log(u)/w of which the k smallest win (Efraimidis and
 * Spirakis), i.e. sequential weighted draws without replacement; with replacement k independent
 * draws.  Rows with deg <= k are copied whole, as in the uniform hop.  out_edge_ids may be NULL.
 * Not in the reference, whose sampler is uniform only (src/cache_graph_sampling.cu:91-177).    */
int shmt_sample_hop_weighted(shmt_ctx* ctx, const void* indptr, int indptr_dtype,
                             const void* indices, int indices_dtype, const float* weights,
                             const void* gpu_indptr, const void* gpu_indices,
                             const float* gpu_weights, const void* gpu_edge_base,
                             const shmt_map* map, const void* seeds, int seeds_dtype,
                             int64_t n, int64_t k, int replace, uint64_t rng_seed,
                             uint64_t rng_offset, void* out_sub_indptr,
                             void* out_sub_indices, void* out_edge_ids, int64_t* nnz_host,
                             void* stream);

/* A whole multi-hop mini-batch in one call: for hop h (fan-out fanouts[h]) sample the
 * current frontier, relabel [frontier, sampled neighbours] and make the distinct ids the
 * next frontier -- the loop of GPUSamplingDataloader.__next__
 * (python/shmtensor/sampling.py:124-143) with csr_(cache_)sampling + tensor_relabel inside.
 * Nothing returns to the host between hops: every kernel reads its input size from the
 * device word the stage before it wrote, with grids sized for the largest frontier the
 * fan-outs allow, and the host waits once, for the sizes: the call returns as soon as
 * they are known, while the last hop's final kernel may still be running (consume the
 * outputs in `stream` order, or synchronise).  `seeds` and every id output have
 * the indices dtype.  With c_0 = n_seeds and c_{h+1} = c_h * (1 + fanouts[h]) the caller
 * provides per hop: out_sub_indptr[h] (c_h + 1 entries, indptr dtype), out_sub_indices[h]
 * (c_h * fanouts[h]), out_relabel[h] (c_{h+1}: relabelled seeds, then relabelled
 * neighbours, contiguous over the real sizes) and out_frontier[h] (c_{h+1}).
 * sizes_host receives 3 numbers per hop: seeds in, edges sampled, distinct ids out.
 * Draws equal those of n_hops successive shmt_sample_hop calls with rng_offset,
 * rng_offset + 1, ...                                                              */
int shmt_sample_minibatch(shmt_ctx* ctx, const void* indptr, int indptr_dtype,
                          const void* indices, int indices_dtype,
                          const void* gpu_indptr, const void* gpu_indices,
                          const shmt_map* map, const void* seeds, int64_t n_seeds,
                          const int64_t* fanouts, int n_hops, int replace,
                          uint64_t rng_seed, uint64_t rng_offset,
                          void* const* out_sub_indptr, void* const* out_sub_indices,
                          void* const* out_relabel, void* const* out_frontier,
                          int64_t* sizes_host, void* stream);

/* The same mini-batch with every hop picking in proportion to per-edge weights, as
 * shmt_sample_hop_weighted does (same draws as successive calls of it with rng_offset,
 * rng_offset + 1, ...; without replacement every fan-out is at most 32).  No counterpart in the
 * reference.                                                                                    */
int shmt_sample_minibatch_weighted(shmt_ctx* ctx, const void* indptr, int indptr_dtype,
                                   const void* indices, int indices_dtype, const float* weights,
                                   const void* gpu_indptr, const void* gpu_indices,
                                   const float* gpu_weights, const shmt_map* map,
                                   const void* seeds, int64_t n_seeds, const int64_t* fanouts,
                                   int n_hops, int replace, uint64_t rng_seed, uint64_t rng_offset,
                                   void* const* out_sub_indptr, void* const* out_sub_indices,
                                   void* const* out_relabel, void* const* out_frontier,
                                   int64_t* sizes_host, void* stream);

/* The same mini-batch that also reports the edge id of every sampled neighbour, per hop, in
 * out_edge_ids[h] (c_h * fanouts[h] entries of indptr dtype, parallel to out_sub_indices[h]);
 * see shmt_sample_hop_eids.  No counterpart in the reference.                              */
int shmt_sample_minibatch_eids(shmt_ctx* ctx, const void* indptr, int indptr_dtype,
                               const void* indices, int indices_dtype,
                               const void* gpu_indptr, const void* gpu_indices,
                               const void* gpu_edge_base, const shmt_map* map,
                               const void* seeds, int64_t n_seeds, const int64_t* fanouts,
                               int n_hops, int replace, uint64_t rng_seed, uint64_t rng_offset,
                               void* const* out_sub_indptr, void* const* out_sub_indices,
                               void* const* out_edge_ids, void* const* out_relabel,
                               void* const* out_frontier, int64_t* sizes_host, void* stream);

/* Compact CSR of the selected rows, in the given order: CreateCacheCSR
 * (src/cache_graph_sampling.cu:455-492).  _count writes the n+1 offsets and
 * (synchronising) the total; _fill copies the adjacency lists.               */
int shmt_subcsr_count(shmt_ctx* ctx, const void* indptr, int indptr_dtype,
                      const void* seeds, int seeds_dtype, int64_t n,
                      void* out_gpu_indptr, int64_t* nnz_host, void* stream);
/* out_edge_base[i] = indptr[seeds[i]] (indptr dtype): the start of each selected row in the
 * full edge array, kept beside a cached sub-CSR so that sampled edges of cached rows can be
 * named by their global edge ids.  No counterpart in the reference.                        */
int shmt_subcsr_edge_base(const void* indptr, int indptr_dtype, const void* seeds,
                          int seeds_dtype, int64_t n, void* out_edge_base, void* stream);
int shmt_subcsr_fill(const void* indptr, int indptr_dtype, const void* indices,
                     int indices_dtype, const void* seeds, int seeds_dtype,
                     int64_t n, const void* gpu_indptr, void* out_gpu_indices,
                     void* stream);

/* ---- host memory substrate -------------------------------------------------
 * POSIX shared memory (include/shm_memory.h:6-49), existence test
 * (include/utils.h:5-13), mmap'ed .npy (src/mmap_tensor.cc:10-55,
 * src/cnpy.cc:18-86) and host registration (src/cache_feature_fetch.cu:6-13). */
int shmt_shm_create(const char* name, int64_t size, int pin_memory,
                    int64_t* out_ptr, int64_t* out_fd);
int shmt_shm_open(const char* name, int64_t size, int pin_memory,
                  int64_t* out_ptr, int64_t* out_fd);
/* Create, failing with SHMT_ERR_OS if a segment of that name exists: one atomic step where
 * python/shmtensor/shm_tensor.py:38-53 tests file_exist() and creates afterwards (two
 * processes can both pass the test).  shmt_shm_unlink removes a name, e.g. the segment a
 * killed run left behind; a name that does not exist is not an error.                     */
int shmt_shm_create_excl(const char* name, int64_t size, int pin_memory,
                         int64_t* out_ptr, int64_t* out_fd);
int shmt_shm_unlink(const char* name);
int shmt_shm_release(const char* name, int64_t size, int64_t ptr, int64_t fd,
                     int pin_memory);
int shmt_shm_exists(const char* name); /* 1 / 0 */

typedef struct shmt_npy_info {
  char descr[8];     /* numpy dtype string, e.g. "<f4"                        */
  int32_t ndim;
  int32_t fortran_order;
  int64_t shape[8];
  int64_t data_offset; /* bytes from the start of the file to element 0       */
  int64_t file_size;   /* size of the mapping                                 */
  int64_t ptr;         /* base address of the mapping                         */
  int64_t fd;
} shmt_npy_info;
/* flags: SHMT_NPY_PIN registers the mapping with CUDA (the reference's pin_memory argument,
 * src/mmap_tensor.cc:10); SHMT_NPY_READONLY opens and maps the file without write permission
 * (the reference maps read/write only, src/mmap_tensor.cc:32) and registers it read-only.  */
#define SHMT_NPY_PIN 1
#define SHMT_NPY_READONLY 2
int shmt_npy_open(const char* path, int flags, shmt_npy_info* out);
int shmt_npy_close(int64_t size, int64_t ptr, int64_t fd, int pin_memory);

int shmt_host_register(void* ptr, int64_t nbytes);
int shmt_host_unregister(void* ptr);

/* Where the pages of a host table live decides which memory controllers, and which
 * inter-socket links, the GPUs' reads of it load.  SHMT_NUMA_INTERLEAVE spreads the range
 * over all memory nodes; SHMT_NUMA_BIND puts it on `node` (one copy of a read-mostly table per
 * socket).  Call it on a fresh mapping, before the data is written and before the range is
 * registered: mbind() where the kernel allows it (pages already present are moved), else
 * first touch from threads running on the wanted node.  The range must start on a page
 * boundary.  No counterpart in the reference, which leaves placement to whoever writes first
 * (include/shm_memory.h:6-23).                                                            */
#define SHMT_NUMA_INTERLEAVE 1
#define SHMT_NUMA_BIND 2
/* Make the pages of a FRESH mapping present by writing one zero byte into each from n_threads
 * threads (a new shared segment is all zeros, so nothing is lost).  Registering 64 GB whose
 * pages one thread has to fault in takes 25 s; with the pages present it takes a quarter of
 * that.  No counterpart in the reference.                                                  */
int shmt_host_prefault(void* ptr, int64_t nbytes, int n_threads);
int shmt_host_numa_nodes(void); /* memory nodes of this machine (>= 1) */
int shmt_host_numa_place(void* ptr, int64_t nbytes, int policy, int node);

/* ---- device buffers shared between ranks (partitioned cache) ---------------
 * cudaMalloc'ed so that a CUDA IPC handle maps the buffer itself; the size is
 * rounded up to whole 2 MB pages, without which a peer maps it with small pages
 * and random reads from a buffer of several GB slow down 10-20x.  No
 * counterpart in the reference.                                              */
int shmt_dev_alloc(int64_t bytes, void** out);
int shmt_dev_free(void* ptr);
int shmt_ipc_get_handle(void* dev_ptr, void* handle_64_bytes);
int shmt_ipc_open_handle(const void* handle_64_bytes, void** out);
int shmt_ipc_close_handle(void* mapped_ptr);

/* Streaming-read probe used to measure the host-link / peer-link / HBM
 * ceilings: sums `bytes` of memory at `src` (16-byte loads) into *sink.       */
int shmt_stream_read(const void* src, int64_t bytes, void* sink_8_bytes,
                     void* stream);
/* Random-read probe for the kernels that are bound by a rate of small reads rather than by
 * bytes (hash probes, row-offset pairs, short adjacency lists): n_reads independent reads of
 * read_bytes (16, 32, 64 or 128) at pseudo-random aligned offsets inside [src, src+bytes),
 * which may be HBM, pinned host memory or a peer's buffer.  No counterpart in the reference. */
int shmt_random_read(const void* src, int64_t bytes, int64_t n_reads, int read_bytes,
                     uint64_t seed, void* sink_8_bytes, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* SHMT_H_ */
