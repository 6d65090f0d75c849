/*
 * The reference's own extern "C" entry points for the extraction path, served by the
 * B200-native library.  Names, argument order and argument meaning are those of
 * python/collcache/common/operation.h:29-59 (paths relative to the reference's project root),
 * so a binding written for the reference (its ctypes table,
 * python/collcache/common/__init__.py:164-260) loads this library instead of libcoll_cache.so.
 *
 * Differences: functions that return void in the reference return an int status here (0 =
 * ok; a caller that ignores it behaves as before), and a failure is reported, not abort()ed.
 * Process model: one process per replica (fork after loading the library, as the reference
 * requires, coll_cache_lib/common.cc:677-689; or unrelated processes that share the
 * environment variable UGC_SESSION), or one process with one thread per replica.
 */
#ifndef COLL_CACHE_API_H_
#define COLL_CACHE_API_H_

#include <stddef.h>
#include <stdint.h>

#include "ugache_b200.h"

#ifdef __cplusplus
extern "C" {
#endif

/* operation.h:34-35, operation.cc:160-173.  Keys: cache_percentage, _cache_policy, num_device,
 * num_global_step_per_epoch, num_epoch, num_total_item, omp_thread_num (operation.cc:72-78).
 * Policies that need the MILP solver (8, 13, 18) are served by the library's split search
 * (UGC_POLICY_SPLIT_SEARCH in ugache_b200.h), which costs every replicate/partition split. */
int coll_cache_config(const char** config_keys, const char** config_values, size_t num_config_items);

size_t coll_cache_num_epoch(void); /* operation.h:37 */

/* operation.h:41-45: per-step profile values (item ids of profiler.h:58-120). */
int coll_cache_log_step_by_key(uint64_t key, int item, double val);
int coll_cache_report_step_by_key(uint64_t key);
int coll_cache_report_step_average_by_key(uint64_t key);

int coll_cache_train_barrier(void);        /* operation.h:48; bounded wait, UGC_ERR_TIMEOUT */
int coll_cache_wait_one_child(void);       /* operation.h:52, operation.cc:219-230 */
int coll_cache_print_memory_usage(void);   /* operation.h:54 */

/* operation.h:56, operation.cc:232-236: keys and output are device pointers of the
 * replica's GPU; returns after the rows have landed (stream synchronised). */
int coll_cache_lookup(int replica_id, uint32_t* key, size_t num_keys, void* output, void* stream);

/* Hotness recording: operation.cc:209-213 (init) and :241-244 (record; keys are HOST memory,
 * as the reference's callers pass them, example/gnn/dgl_sample.py:242). */
int coll_cache_record_init(int replica_id);
int coll_cache_record(int replica_id, uint32_t* key, size_t num_keys);

/* C form of the C++ coll_cache_init (operation.h:29, operation.cc:129-150): combines the
 * recorded hotness, solves the placement on replica 0, builds this replica's cache and
 * connects it to the others.  dtype uses the reference's DataType numbering
 * (coll_cache_lib/common.h:39-49: 0 f32, 1 f64, 2 f16, 3 u8, 4 i32, 5 i8, 6 i64).
 * alloc/free may be NULL (cudaMalloc/cudaFree).  Every replica must call it. */
int coll_cache_init_c(int replica_id, size_t key_space_size, ugc_alloc_fn alloc, ugc_free_fn free_fn,
                      void* alloc_user, void* cpu_data, int dtype, size_t dim,
                      double cache_percentage, void* stream);

/* CollCache::refresh (coll_cache_lib/facade.cc:513-557) for the hotness recorded since the
 * last placement; the reference reaches it only from its TF2 binding.  Every replica must
 * call it; lookups on other threads keep running. */
int coll_cache_refresh(int replica_id, void* stream);

/* Device a replica runs on.  The reference fixes replica i -> device i
 * (python/collcache/common/operation.cc:84-86); its torch binding takes a dev_id per replica
 * (python/collcache/torch/adapter.cc:151).  Call before coll_cache_init_c. */
int coll_cache_set_device(int replica_id, int device_id);

/* The underlying context of this process (for ugc_stats and friends), or NULL. */
ugc_ctx* coll_cache_context(void);

/* Tears the process-wide state down (the reference never does). */
int coll_cache_shutdown(void);

#ifdef __cplusplus
}
#endif
#endif /* COLL_CACHE_API_H_ */
