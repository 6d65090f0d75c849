/*
 * ugache_b200 -- C ABI of the B200-native embedding-extraction path.
 *
 * Plain C: pointers, sizes and integer status codes only; no exception crosses this
 * boundary and no function aborts the process.  Every call returns UGC_OK (0) or an
 * error code; ugc_last_error() gives the message of the calling thread's last failure.
 *
 * Each entry point cites the interface of the reference (SJTU-IPADS/ugache, paths
 * relative to its project root) that it replaces.
 *
 * Vocabulary (the reference's): a *replica* is one GPU worker; a *location* is a source
 * of rows -- replicas 0..G-1 are the GPUs' cache slices, location G is the host table;
 * the *placement* is the host-side input (4 arrays) saying which GPUs store which rows
 * and where each reader fetches each row from.
 */
#ifndef UGACHE_B200_H_
#define UGACHE_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define UGC_MAX_DEVICE 8 /* placement bitmask is one byte: optimal_solver_class.cc:1381 */

typedef enum {
  UGC_OK = 0,
  UGC_ERR_INVALID = 1,     /* bad argument or configuration                         */
  UGC_ERR_CUDA = 2,        /* a CUDA runtime call failed (message has the details)  */
  UGC_ERR_NOMEM = 3,       /* allocator returned NULL                               */
  UGC_ERR_CAPACITY = 4,    /* placement needs more cache rows than the slice holds  */
  UGC_ERR_STATE = 5,       /* call out of order (e.g. lookup before build)          */
  UGC_ERR_KEY_RANGE = 6,   /* a key outside [0, num_total_item) was seen            */
  UGC_ERR_TIMEOUT = 7,     /* a bounded host-side wait ran out                      */
  UGC_ERR_UNSUPPORTED = 8, /* row size / key space outside what the kernels handle  */
  UGC_ERR_TABLE = 9        /* table inconsistency found on the device (dup / miss)  */
} ugc_status;

/* Placement heuristics of the reference that need no MILP licence
 * (python/collcache/common/__init__.py:46-64 numbering). */
typedef enum {
  UGC_POLICY_INTUITIVE = 9, /* coll_intuitive: replicate hottest, partition next      */
  UGC_POLICY_REP = 12,      /* rep: replicate hottest on every GPU                    */
  UGC_POLICY_CLIQUE_PART = 14, /* clique_part: partition hottest round-robin          */
  UGC_POLICY_SPLIT_SEARCH = 100 /* no reference number: stands in for the reference's MILP
                                   policies (coll_cache_asymm_link and relatives,
                                   coll_cache_lib/coll_cache/optimal_solver_class.cc:957-1112) on a
                                   switch-connected box, where the optimum is a replicate /
                                   partition / host split: every split is costed against the
                                   recorded hotness with max((local + served + 1) * t_local,
                                   peers * t_remote, host * t_cpu), where "served" is what the
                                   peers read from this GPU, and the cheapest kept; among equals
                                   the most replicated                                     */
} ugc_policy;

typedef enum { UGC_TABLE_AUTO = 0, UGC_TABLE_FLAT = 1, UGC_TABLE_HASHED = 2 } ugc_table_kind;

/* How a lookup extracts its rows.  The reference offers both shapes among its extraction
 * implementations (coll_cache_lib/common.h:85-101): grouped by source with a per-source share
 * of the SMs (its default, coll_cache_lib/cache_context.cu:1405-1465), and ungrouped, one copy
 * kernel that resolves the source row by row (kDirectNoGroup, cache_context.cu:1295-1329).
 *   GROUPED  lookup kernel writes one index list per source group (local / peers / host),
 *            gather kernel splits its CTAs over the groups: best when many rows of a batch
 *            come from the host table;
 *   DIRECT   one kernel probes the table and copies each row from wherever it is, with no
 *            index lists: best when nearly all rows come from GPU memory;
 *   AUTO     DIRECT while the last finished lookup of the replica took no more than
 *            ugc_tuning.direct_max_host_rows rows from the host table, or more rows from
 *            peers than from the host; else GROUPED
 *            (the library reads those counts from a pinned mirror the kernels write; no
 *            synchronisation). */
typedef enum { UGC_EXTRACT_AUTO = 0, UGC_EXTRACT_GROUPED = 1, UGC_EXTRACT_DIRECT = 2 } ugc_extract_mode;

/* Device-memory allocator supplied by the caller, the C form of the reference's
 * std::function<MemHandle(size_t)> gpu_mem_allocator (coll_cache_lib/facade.h:57-60,
 * coll_cache_lib/common.h:140-149).  Called with the replica's device current.
 * NULL callbacks select cudaMalloc / cudaFree. */
typedef void* (*ugc_alloc_fn)(size_t nbytes, void* user);
typedef void (*ugc_free_fn)(void* ptr, void* user);

/* Replaces the static RunConfig + config map of the reference
 * (coll_cache_lib/run_config.h:30-111, python/collcache/common/operation.cc:68-104). */
typedef struct {
  uint32_t struct_size;     /* sizeof(ugc_config), for forward compatibility          */
  int32_t num_device;       /* G: replicas in the job, 1..8                            */
  uint64_t num_total_item;  /* N: rows of the table, < 2^31-1                          */
  uint32_t row_bytes;       /* bytes per row (dim * element size), multiple of 4       */
  double cache_percentage;  /* per-GPU cache size as a FRACTION of N, 0..1             */
  int32_t empty_feat;       /* k>0: host rows wrap to key mod 2^k (SAMGRAPH_EMPTY_FEAT,
                               coll_cache_lib/cache_context.h:346-352); 0 = off        */
  int32_t table_kind;       /* ugc_table_kind; AUTO follows cache_context.cu:2489-2497 */
  uint32_t max_batch;       /* largest key batch one lookup may carry (scratch size)   */
  int32_t register_host;    /* 1: cudaHostRegister the host table if it is not already
                               GPU-visible (coll_cache_lib/facade.cc:476)              */
  /* Link bandwidths (GB/s) used to share the gather's CTAs out over the source groups in
   * proportion to bytes / bandwidth (the B200 counterpart of
   * coll_cache_lib/coll_cache/asymm_link_desc.cc:247-289).  0 = ugc_link_desc's figure. */
  double bw_local_gbs, bw_remote_gbs, bw_host_gbs;
  int32_t gather_ctas_per_sm; /* CTAs of the gather kernel per SM; 0 = default          */
  int32_t host_ctas;          /* most CTAs the host-row group may take; 0 = what keeps the
                                 host link full by ugc_link_desc                         */
  int32_t remote_ctas;        /* most CTAs the peer-row group may take; 0 = what keeps the
                                 NVLink port full by ugc_link_desc                       */
  int32_t gather_vec_bytes;   /* 16 or 32 bytes per lane per load in the gather (host rows
                                 always use 16); 0 = 32 with 8 GPUs, else 16            */
  ugc_alloc_fn alloc;
  ugc_free_fn free;
  void* alloc_user;
} ugc_config;

typedef struct ugc_ctx ugc_ctx; /* one per process; holds the replicas built in it */

/* What one replica publishes so that peers can read its slice and its table, and the C
 * form of DevicePointerExchanger's page of pointers / IPC handles
 * (coll_cache_lib/cache_context.cu:2648-2680). */
typedef struct {
  int32_t replica_id;
  int32_t device_id;
  int64_t pid;
  uint64_t slice_ptr;        /* device address in the owner's process                  */
  uint64_t table_ptr;
  uint64_t table_lines;      /* hashed: number of 32-byte lines; flat: N               */
  int32_t table_kind;
  int32_t has_ipc;             /* 0: pointers only (same process); 1: cudaIpcMemHandle_t in
                                  the two blobs; 2: {int64 file descriptor in the owner's
                                  process, int64 mapped size, int64 token of the owner's
                                  descriptor socket} in the two blobs -- blocks from
                                  the CUDA virtual-memory API, which the importer maps with
                                  the owner's 2 MiB pages                               */
  unsigned char slice_ipc[64];
  unsigned char table_ipc[64];
} ugc_peer_handle;

typedef struct {
  uint64_t num_local_rows;     /* rows this replica stores                             */
  uint64_t num_remote_keys;    /* keys it reads from peers                             */
  uint64_t num_host_keys;      /* keys it reads from the host table                    */
  uint64_t capacity_rows;
  uint64_t free_rows;
  int32_t table_kind;
  uint64_t table_bytes;
  uint64_t slice_bytes;
  /* last completed lookup (valid after the stream it ran on is synchronised) */
  uint64_t last_keys;
  uint64_t last_local, last_remote, last_host;
  /* sticky device-side error counters */
  uint64_t err_key_range;
  uint64_t err_table;
  uint64_t lookups;            /* lookups issued on this replica                       */
  /* device-clock time (ns) from the start of the last gather kernel until the last CTA of
     each source group was done; 0 for an empty group */
  uint64_t last_local_ns, last_remote_ns, last_host_ns;
  uint64_t last_index_ns;      /* grouped extraction: device-clock time from the start of
                                  the lookup kernel to the start of the gather kernel (the
                                  index-building phase); 0 for a direct extraction        */
  /* device memory this context (all its replicas in this process) holds now: obtained through
     the caller's allocator callbacks / by the library itself (cudaMalloc, or virtual-memory
     blocks that other processes can map), i.e. outside the caller's pool */
  uint64_t device_bytes_from_allocator, device_bytes_own;
  uint64_t lookups_host_ordered; /* grouped lookups whose host list was put in address order */
  uint64_t lookups_direct;     /* lookups that took the direct (one-kernel) extraction  */
  uint64_t kernel_launches;    /* kernels launched by lookups: 2 per grouped, 1 per direct */
  uint64_t lookups_pooled;     /* ugc_lookup_pool calls                                   */
  uint64_t pool_rows[3];       /* rows they summed so far: local / peers / host           */
} ugc_stats_t;

/* sizeof of the structs of this header, in the order ugc_config, ugc_peer_handle,
 * ugc_stats_t, ugc_tuning, ugc_link_desc_t: lets a binding in another language check its own
 * declarations against the library it loaded.  No reference counterpart. */
int ugc_abi_sizes(uint32_t sizes[5]);

const char* ugc_version(void);
const char* ugc_last_error(void);
const char* ugc_status_string(int status);

/* Fills *cfg with defaults (struct_size set, everything else zero / default). */
int ugc_config_default(ugc_config* cfg);

/* -- context ------------------------------------------------------------------------ */
/* CollCache constructor + coll_cache_config (coll_cache_lib/facade.h:39,
 * python/collcache/common/operation.cc:160-173). */
int ugc_create(const ugc_config* cfg, ugc_ctx** out);
int ugc_destroy(ugc_ctx* ctx);

/* -- placement (host side; no GPU needed) -------------------------------------------- */
/* The reference's non-MILP solvers: IntuitiveSolver / RepSolver / CliquePartSolver
 * (coll_cache_lib/coll_cache/optimal_solver_class.cc:1251-1404, :1869-1924, :1926-2058).
 * cache_percent is in PERCENT (0..100) as the solvers take it.  Output arrays are caller
 * allocated: nid_to_block[N], block_placement[G+2], block_access_from[G*(G+2)],
 * block_density[G+2]; *num_block receives the number of blocks actually used (row stride
 * of block_access_from). */
int ugc_solve_placement(int policy, int num_device, uint64_t num_total_item,
                        const uint32_t* rank_ids, const uint32_t* rank_freqs,
                        double cache_percent, double t_local, double t_remote, double t_cpu,
                        uint32_t* nid_to_block, uint8_t* block_placement,
                        uint8_t* block_access_from, double* block_density, int* num_block);

/* Default B200 time-per-byte ratios (local : remote : host) for the solvers, the
 * counterpart of coll_cache_lib/coll_cache/asymm_link_desc.cc:247-289. */
int ugc_link_model(int num_device, double* t_local, double* t_remote, double* t_cpu);

/* The B200 link description behind that model, for a job of num_device GPUs and rows of
 * row_bytes (0: bandwidth figures only): what one GPU can pull from local HBM, from all its
 * peers together (one NVLink port through the switch) and from the host table while every GPU
 * of the job does the same (its own PCIe link, its share of what the host side sustains for
 * all GPUs, and the rate at which scattered pinned rows arrive), the load-to-use latencies, and
 * from bandwidth x latency the number of gather CTAs that keeps each far link full.  The
 * reference holds such a table per platform with SM counts per link
 * (coll_cache_lib/coll_cache/asymm_link_desc.cc:242-392).  struct_size must be set. */
typedef struct {
  uint32_t struct_size;
  int32_t num_device;
  double bw_local_gbs, bw_remote_gbs, bw_host_gbs;
  double lat_local_us, lat_remote_us, lat_host_us;
  double host_rows_per_s;
  double host_total_gbs;
  double t_local, t_remote, t_cpu; /* time-per-byte ratios with the row-rate host term */
  int32_t host_ctas, remote_ctas, per_peer_ctas;
} ugc_link_desc_t;
int ugc_link_desc(int num_device, uint32_t row_bytes, ugc_link_desc_t* out);

/* Modelled cost per reader of a placement under the concurrent-source model above (shares of
 * the recorded hotness served from the local slice, from peers and from the host).  No
 * reference counterpart; lets a caller compare policies before building.  cost has num_device
 * entries. */
int ugc_placement_cost(int num_device, uint64_t num_total_item, const uint32_t* rank_ids,
                       const uint32_t* rank_freqs, const uint32_t* nid_to_block,
                       const uint8_t* block_access_from, int num_block, double t_local,
                       double t_remote, double t_cpu, double* cost);

/* Hands the placement to the context (arrays are copied).  Corresponds to the four shm
 * tensors the reference publishes (coll_cache_lib/facade.cc:238-261). */
int ugc_set_placement(ugc_ctx* ctx, const uint32_t* nid_to_block, const uint8_t* block_placement,
                      const uint8_t* block_access_from, const double* block_density,
                      int num_block);

/* Host-side key classification for one reader: which source serves each key.
 * Replaces CacheEntryManager::DetectKeysForAllSource
 * (coll_cache_lib/cuda/cache_hashtable.cuh:741-835); lists come out in ascending key
 * order.  counts[G+1] receives the per-location key counts (index G = host).  If
 * keys_out is non-NULL it must hold N entries and receives the GPU-served keys grouped by
 * source (source s starts at the sum of counts[0..s)).  Needs ugc_set_placement. */
int ugc_classify_keys(ugc_ctx* ctx, int replica_id, uint64_t* counts, uint32_t* keys_out);

/* -- build ---------------------------------------------------------------------------- */
/* Per-replica cache build: allocate the slice, fill it from the host table, build the
 * table for the rows stored here.  Replaces CollCache::build_v2 -> CacheContext::build
 * (coll_cache_lib/facade.cc:430-511, coll_cache_lib/cache_context.cu:2414-2520).
 * host_table: N rows (or 2^empty_feat rows) of row_bytes, caller owned, must stay valid.
 * stream: a cudaStream_t (NULL = default stream).  Returns after the stream is idle. */
int ugc_build(ugc_ctx* ctx, int replica_id, int device_id, const void* host_table,
              void* stream);

/* Publishes / receives peer pointers (DevicePointerExchanger signin / extract,
 * coll_cache_lib/cache_context.cu:2519-2526, :2658-2680).  ugc_connect_local wires every
 * replica built in THIS process to every other one (peer access is enabled when they sit
 * on different devices); ugc_import_peer takes a handle from another process. */
int ugc_export(ugc_ctx* ctx, int replica_id, ugc_peer_handle* out);
int ugc_import_peer(ugc_ctx* ctx, int replica_id, const ugc_peer_handle* peer);
int ugc_connect_local(ugc_ctx* ctx);

/* Resolves the slice offsets of the keys this replica reads from peers by probing the
 * peers' tables over P2P, and inserts them into its own table.  Replaces the per-peer
 * loop of coll_cache_lib/cache_context.cu:2531-2570.  Every peer named by the placement
 * must have been imported and must have finished ugc_build. */
int ugc_attach_peers(ugc_ctx* ctx, int replica_id, void* stream);

/* -- lookup (the hot path) ------------------------------------------------------------ */
/* out[i, :] = row of keys[i], for i in [0, n).  keys and out are DEVICE pointers on the
 * replica's GPU; out holds n * row_bytes bytes.  Work is enqueued on `stream` and the
 * call returns without synchronising (the reference's call returns after its internal
 * streams are idle; its shim adds the synchronise).  Replaces CollCache::lookup ->
 * ExtractSession::ExtractFeat (coll_cache_lib/facade.cc:74-88,
 * coll_cache_lib/cache_context.cu:1199) and coll_cache_lookup
 * (python/collcache/common/operation.cc:232-236), whose keys are 32-bit. */
int ugc_lookup_u32(ugc_ctx* ctx, int replica_id, const uint32_t* keys, size_t n, void* out,
                   void* stream);
/* Same with 64-bit ids (results identical for ids below 2^31-1). */
int ugc_lookup_i64(ugc_ctx* ctx, int replica_id, const int64_t* keys, size_t n, void* out,
                   void* stream);

/* ugc_lookup_i64 without any device memory of its own: the index lists and counters of the
 * lookup live in a fixed array compiled into the library (about 6.3 MB on every GPU that loads
 * it, held until the process exits) instead of the scratch that ugc_build / ugc_reserve_batch
 * obtain from the allocator.  Meant for callers that cannot get device memory at the point
 * where they look keys up: a caller-supplied allocator that is a fixed arena with nothing left
 * once the cache slice is in it, or a serving thread that must not take the device-wide
 * synchronisation ugc_reserve_batch does when a batch outgrows max_batch.  The call itself
 * performs no allocation of any kind.
 *   - at most 262,144 keys per call (UGC_ERR_INVALID beyond that);
 *   - the first call on a GPU asks the runtime for the array's device address; make that
 *     first call before any stream capture starts;
 *   - all replicas on one GPU, and all calls, share the one array: two such lookups that
 *     overlap on the GPU (different streams, different replicas on the same device) race;
 *     keep them ordered on one stream;
 *   - out-of-range keys are skipped as usual but are not added to ugc_stats' counters.
 * Same results as ugc_lookup_i64.  This entry point has no counterpart in the reference. */
int ugc_lookup_i64_static(ugc_ctx* ctx, int replica_id, const int64_t* keys, size_t n, void* out,
                          void* stream);

/* Deduplicated lookup, all on the GPU: finds the distinct keys of the batch, extracts each of
 * their rows once and returns the index that reassembles the batch.  A recommendation batch
 * under a skewed distribution repeats its hottest ids thousands of times; a consumer that
 * pools or scatters by index anyway (embedding-bag forward, sparse-gradient backward) then
 * needs every distinct row once, which also spares most of the output write.
 *   unique_keys[0 .. *n_unique)  the distinct keys (same width as keys), in order of discovery;
 *   out_rows[j, :]               row of unique_keys[j];
 *   inverse[i]                   index of keys[i] in unique_keys (-1 for an id outside the key
 *                                space, which is counted in err_key_range);
 *   *n_unique                    their number -- device memory like the rest, so nothing here
 *                                synchronises; capacity of out_rows / unique_keys: n entries.
 * keys: key_bytes 4 or 8.  Uses one 32-bit stamp per id of the key space (allocated on the
 * first call); at most 2^24-2 keys per call.  After the call ugc_stats' last_local/remote/host
 * add up to the number of distinct keys.  The reference has no such call; its applications
 * deduplicate before they look up (example/dlr and the GNN samplers hand over unique ids). */
int ugc_lookup_unique(ugc_ctx* ctx, int replica_id, const void* keys, int key_bytes, size_t n,
                      void* out_rows, void* unique_keys, int32_t* inverse, uint32_t* n_unique,
                      void* stream);

/* Pooled lookup (embedding bag): out[b, :] = the sum, or the mean, of the rows of the keys of
 * bag b, as fp32 -- lookup, row fetch and reduction in one kernel, so the looked-up rows never
 * reach memory and the output is n_bags x dim x 4 bytes instead of n_keys x row_bytes.
 *   keys      n_keys ids (key_bytes 4 or 8), device memory;
 *   offsets   n_bags + 1 ascending positions into keys (device memory): bag b is
 *             keys[offsets[b] .. offsets[b+1]); or NULL: bag b is keys[b*bag_size .. (b+1)*bag_size);
 *   elem_type what a row holds (the library otherwise treats rows as bytes);
 *   out       n_bags x dim fp32, dim = row_bytes / element size, 16-byte aligned.
 * Defined bit for bit: every output element starts at +0 and takes its bag's rows in key order,
 * one IEEE fp32 addition each (fp16 elements are widened first, which is exact); the mean
 * divides that sum once by the bag's length (as fp32); an empty bag gives zeros.  Ids outside
 * the key space are counted in err_key_range and add nothing.  Rows must be a multiple of 16
 * bytes and the tables 16-byte aligned (UGC_ERR_UNSUPPORTED otherwise).  Ordered against a
 * refresh like every lookup.  The reference has no such call: its applications hand the rows
 * to the model, which pools them (example/dlr/main.py: `combiner`). */
typedef enum { UGC_ELEM_F32 = 0, UGC_ELEM_F16 = 1 } ugc_elem_type;
typedef enum { UGC_POOL_SUM = 0, UGC_POOL_MEAN = 1 } ugc_pool_mode;
int ugc_lookup_pool(ugc_ctx* ctx, int replica_id, const void* keys, int key_bytes, size_t n_keys,
                    const int64_t* offsets, size_t n_bags, size_t bag_size, int elem_type, int mode,
                    float* out, void* stream);

/* Grows the per-replica lookup scratch so that batches of up to max_batch keys are accepted
 * (the reference re-allocates its output buffer when a larger batch shows up,
 * python/collcache/torch/adapter.cc:213-224).  Must not run while a lookup of that replica
 * is in flight. */
int ugc_reserve_batch(ugc_ctx* ctx, int replica_id, uint32_t max_batch);

/* Host-buffer form: keys and out are HOST pointers.  Returns after the rows have landed in
 * `out`.  key_bytes is 4 or 8.  A buffer that is pinned and mapped for the GPU (cudaHostAlloc /
 * cudaHostRegister with the mapped flag, or ugc_host_alloc) can be used in place, as
 * ugc_tuning.host_zero_copy says: by default the kernel reads the keys across PCIe itself,
 * while the rows are staged in device memory and leave through the copy engine (measured
 * faster than stores from the SMs: 56 against 51 GB/s), in four pieces for batches of 65,536
 * keys or more so that one piece crosses PCIe while the next is being extracted.  After such
 * a call ugc_stats' last_* fields describe the last piece only.  Pageable buffers always go
 * through staging copies. */
int ugc_lookup_host(ugc_ctx* ctx, int replica_id, const void* keys, int key_bytes, size_t n,
                    void* out, void* stream);

/* -- refresh --------------------------------------------------------------------------- */
/* Moves a replica from the current placement to a new one while lookups keep running.
 * Replaces CollCache::refresh -> RefreshSession::refresh_after_solve_new
 * (coll_cache_lib/facade.cc:513-557, coll_cache_lib/cache_context.cu:3944-4107) in three
 * phases; the caller puts a barrier over all replicas between them, as the reference
 * does (cache_context.cu:4047, :4077, :4099):
 *   ugc_refresh_set_placement  once per process: the new placement (old one is kept)
 *   ugc_refresh_evict          steps 1-4: classify, evict local and re-pointed remote keys
 *   ugc_refresh_fill           step 6: scatter new rows into freed slots, insert them
 *   ugc_refresh_attach         step 7: resolve and insert the new remote keys
 *   ugc_refresh_commit         once per process: new placement becomes current
 * Lookups of the same replica may be issued from another thread (on another stream) during all
 * of it, as the reference's background refresh allows: an evicted key is served from the host
 * table until it is cached again, a slot is reused only after every lookup that could still
 * name it has drained (ugc_refresh_evict waits, on the host, until the replica's count of
 * finished lookups has reached the number enqueued; no stream of the device is stalled; the
 * reference waits on its step counter, cache_context.cu:4045-4052), and a new entry becomes
 * visible only after its row has been written (same stream, one 64-bit publish).  The phase
 * calls of one replica must come from one thread at a time.
 */
int ugc_refresh_set_placement(ugc_ctx* ctx, const uint32_t* nid_to_block,
                              const uint8_t* block_placement, const uint8_t* block_access_from,
                              const double* block_density, int num_block);
int ugc_refresh_evict(ugc_ctx* ctx, int replica_id, void* stream);
int ugc_refresh_fill(ugc_ctx* ctx, int replica_id, void* stream);
int ugc_refresh_attach(ugc_ctx* ctx, int replica_id, void* stream);
int ugc_refresh_commit(ugc_ctx* ctx);

/* -- hotness recording --------------------------------------------------------------------- */
/* Counts key accesses on the GPU: counts[key] += 1 for every key of a device-resident batch
 * (key_bytes 4 or 8).  The counter array (4 bytes per id of the key space) is allocated on
 * the first call.  Replaces FreqRecorder::Record on host copies of the keys
 * (coll_cache_lib/freq_recorder.cc, fed by python_tf2/.../lookup_manager.cc:290-312).
 * ugc_hotness_read copies the counters to host memory (num_total_item uint32) after
 * synchronising `stream`, and zeroes them on the device if `reset` is non-zero; ranking them
 * (ids by descending count) gives the rank_ids / rank_freqs input of ugc_solve_placement. */
int ugc_record(ugc_ctx* ctx, int replica_id, const void* keys, int key_bytes, size_t n, void* stream);
int ugc_hotness_read(ugc_ctx* ctx, int replica_id, uint32_t* counts_out, int reset, void* stream);

/* -- introspection --------------------------------------------------------------------- */
int ugc_stats(ugc_ctx* ctx, int replica_id, ugc_stats_t* out);

/* Launch shape of one replica's lookups.  The reference fixes the corresponding numbers per
 * platform in its link tables (SMs for the host and peer streams,
 * coll_cache_lib/coll_cache/asymm_link_desc.cc:247-289) and in constant.h:74-75 (block and
 * tile size).  ugc_get_tuning fills the struct with the current values; ugc_set_tuning
 * applies it (struct_size must be set). */
typedef struct {
  uint32_t struct_size;
  int32_t gather_ctas_per_sm;     /* CTAs of the gather kernel per SM                       */
  int32_t gather_block_threads;   /* 256, 512 or 1024                                       */
  int32_t gather_vec_bytes;       /* 16 or 32 bytes per lane per load                       */
  int32_t host_ctas;              /* most CTAs the host-row group may take                       */
  int32_t remote_ctas;            /* most CTAs the peer-row group may take                       */
  int32_t bulk_mask;              /* far sources staged through shared memory by the
                                     bulk-async copy engine: bit 0 host rows, bit 1 peer rows */
  int32_t lookup_keys_per_thread; /* 1, 2 or 4                                              */
  int32_t programmatic_launch;    /* programmatic stream serialization: bit 0 for the lookup
                                     kernel (its key loads and probes overlap the tail of
                                     the previous gather), bit 1 for the gather kernel (it is
                                     scheduled while the lookup kernel drains)              */
  int32_t extract_mode;           /* ugc_extract_mode                                       */
  int32_t direct_ctas_per_sm;     /* CTAs of the direct extraction kernel per SM, 1..16     */
  int32_t direct_max_host_rows;   /* auto mode: direct while the last finished lookup took at
                                     most this many rows from the host table                */
  int32_t direct_block_threads;   /* threads per CTA of the direct kernel: 128 or 256       */
  int32_t direct_tile_keys;       /* keys one warp of the direct kernel probes at a time: 8,
                                     16 or 32; 0 = the largest that balances the warps      */
  int32_t direct_deep;            /* direct kernel: 1 = twice the rows in flight per warp at
                                     3 instead of 4 CTAs per SM                             */
  int32_t direct_early_host;      /* direct kernel: the first host row of every warp's first tile
                                     is fetched before the kernel waits for the launch ahead of
                                     it, so that the host link's queue stays filled from one
                                     lookup to the next: 0 = when the last finished lookup took
                                     at least 1024 host rows, 1 = always, 2 = never          */
  int32_t host_order_min_rows;    /* grouped extraction: order the host list by address (two
                                     small kernels between lookup and gather) when the last
                                     finished lookup took at least this many rows from the
                                     host table; 0 = never                                  */
  int32_t refresh_fill_ctas;      /* refresh-time fill: CTAs per launch (20, as the reference,
                                     coll_cache_lib/cache_context.cu:4067), rows per launch    */
  int32_t refresh_fill_batch_rows; /* (131,072) and a host-side pause between launches in us    */
  int32_t refresh_fill_pause_us;  /* (0).  The reference sleeps 3 ms between 4092-row batches
                                     (:4061-4070) to keep the fill out of the lookups' way; on
                                     the B200 machines measured neither a pause nor a smaller
                                     grid changed the lookup times during a refresh          */
  int32_t refresh_early_repoint;  /* refresh: 1 (default) = a key whose new source is a peer that
                                     holds the row already is re-pointed to it in place in the
                                     evict phase; 0 = removed there and attached in the attach
                                     phase, served by the host in between (the reference's order) */
  int32_t pool_vec_bytes;         /* ugc_lookup_pool: bytes of a row one lane adds up, 16 or 4;
                                     0 (default) = 16 unless the batch has so few bags (fewer
                                     than two warps' worth per SM) that 4, with four times the
                                     lane groups per bag, fills the GPU better                */
  int32_t gather_dynamic;         /* grouped gather: 1 = lists are handed out in chunks and a
                                     CTA whose own list is drained takes chunks of the other
                                     groups' lists; 0 = fixed striding inside each group     */
  int32_t split_fixed;            /* 1 = host_ctas and remote_ctas are the CTA counts of their
                                     groups instead of caps on the derived split (sweeps)     */
  int32_t host_zero_copy;         /* ugc_lookup_host with GPU-mapped pinned buffers: bit 0 the
                                     kernel reads the keys in place, bit 1 it writes the rows
                                     in place; a cleared bit selects a staging copy          */
} ugc_tuning;
int ugc_get_tuning(ugc_ctx* ctx, int replica_id, ugc_tuning* out);
int ugc_set_tuning(ugc_ctx* ctx, int replica_id, const ugc_tuning* in);

/* Per-kernel device timing of the lookups issued between begin and end: CUDA events are
 * recorded on the lookup's stream around the lookup_group kernel and around the gather
 * kernel.  Replaces the host-timer phase breakdown the reference logs per step
 * (kLogL3CacheGetIndexTime / kLogL3CacheCombine*Time, coll_cache_lib/cache_context.cu:1662-1679).
 * ugc_profile_end synchronises the device and returns the summed kernel times (ms). */
int ugc_profile_begin(ugc_ctx* ctx, int replica_id, int max_lookups);
int ugc_profile_end(ugc_ctx* ctx, int replica_id, double* lookup_group_ms, double* gather_ms,
                    uint64_t* lookups);

/* Debug / test aid: the packed (location << 28 | offset) word the replica's table holds
 * for each of n keys (0xffffffff = not in the table, i.e. served by the host).  keys and
 * words are DEVICE pointers.  The word format is the reference's EmbCacheOff
 * (coll_cache_lib/cuda/cache_hashtable.h:20-28). */
int ugc_table_words(ugc_ctx* ctx, int replica_id, const uint32_t* keys, size_t n,
                    uint32_t* words, void* stream);

/* Pins caller-owned host memory and maps it for every GPU; *dev_ptr receives the address
 * kernels use for it.  The library does this itself inside ugc_build when register_host is
 * set (as the reference does, coll_cache_lib/facade.cc:476); the explicit form lets a
 * harness fill the table from the GPU before the build. */
int ugc_host_register(void* host_ptr, size_t nbytes, void** dev_ptr);
int ugc_host_unregister(void* host_ptr);                       /* regions up to 1 GiB */
int ugc_host_unregister_sized(void* host_ptr, size_t nbytes);  /* any size */
/* Pinned, GPU-mapped host memory for callers that let the library own the host table's
 * storage, as the reference's binding does for its embedding table
 * (python/collcache/torch/adapter.cc:239-270, coll_cache_lib/cpu/cpu_device.cc:36-112).
 * The memory is taken through the CUDA virtual-memory API at the GPU's host NUMA node when
 * the driver offers that (2 MiB chunks, mapped by the GPU with large pages, which keeps
 * random row reads over tens of GB from missing in address translation); cudaHostAlloc
 * otherwise.  *host_ptr is valid on the CPU, *dev_ptr in kernels. */
int ugc_host_alloc(size_t nbytes, void** host_ptr, void** dev_ptr);
int ugc_host_free(void* host_ptr);
/* 1 if host_ptr came from ugc_host_alloc through the virtual-memory route, else 0. */
int ugc_host_is_large_page(const void* host_ptr);

/* Synthetic-input helper for benchmarks: writes rows [row_begin, row_begin+n_rows) of the
 * seeded uniform[-1,1) table into dst (device memory, or GPU-visible pinned host memory).
 * elem_bytes 4 = fp32, 2 = fp16.  No counterpart in the reference (its tables are loaded
 * from datasets, python/collcache/torch/adapter.cc:239-270). */
int ugc_gen_table(void* dst, uint64_t seed, uint64_t row_begin, uint64_t n_rows, uint64_t dim,
                  int elem_bytes, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* UGACHE_B200_H_ */
