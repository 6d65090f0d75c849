// sm_100a kernels of the extraction path and their launchers.
//
//   lookup_group   keys -> (location, offset) through the replica's table, grouped by
//                  source into three record lists (local / peers / host) with the counts
//                  left in device memory: no sort, nothing goes through the host.
//   gather_roles   one launch whose CTAs split into per-source groups sized from those
//                  counts and the per-link CTA caps; each group copies its rows with vector
//                  loads (local HBM, peer HBM over NVLink P2P, zero-copy host over PCIe).
//   extract_direct lookup and row copy fused: each warp probes 32 keys and copies their rows
//                  from whatever source holds them; no lists, one launch.
//   fill_scatter   host rows -> cache slots (build and refresh).
//   table_*        insert / evict / word lookup / peer-table resolve.
//   gen_table      seeded synthetic table rows (benchmark input helper).
#pragma once
#include <cuda_runtime.h>

#include "device_types.h"

namespace ugc {

// All launchers enqueue on `stream` and return the launch status; none synchronises.

cudaError_t launch_lookup_group(const void* keys, int key_bytes, uint32_t n, const TableView& table,
                                uint32_t local_loc, uint32_t host_loc, int empty_feat,
                                uint64_t* list_local, uint64_t* list_remote, uint64_t* list_host,
                                Counters* counters, int keys_per_thread, bool pdl,
                                cudaStream_t stream);

cudaError_t launch_gather_roles(const GatherParams& p, int grid, int block, int vec_bytes,
                                cudaStream_t stream);

// Distinct keys of a batch: unique_keys[0 .. *n_unique) (order of discovery), inverse[i] = index
// of keys[i] among them (-1 for an id outside [0, num_keys)).  `stamp` is one uint32 per id of
// the key space, zeroed once; `epoch` (1..255) must differ from the one of the previous call on
// the same stamp array and the array be zeroed again before an epoch value comes round.
cudaError_t launch_unique(const void* keys, int key_bytes, uint32_t n, uint64_t num_keys, uint32_t epoch,
                          uint32_t* stamp, void* unique_keys, int32_t* inverse, uint32_t* n_unique,
                          Counters* counters, cudaStream_t stream);

// Pooled lookup: out[b] = sum (or mean) over the keys of bag b of their rows, fp32, added in key
// order.  Rows must be a multiple of 16 bytes and every source and `out` 16-byte aligned.
// vec_bytes: 16 or 4 forces the size of the pieces a lane adds up, anything else lets the
// launcher choose by how many warps the batch fills.
cudaError_t launch_lookup_pool(const void* keys, int key_bytes, const PoolParams& p, bool f16,
                               int max_ctas, int vec_bytes, cudaStream_t stream);

// Orders the host list of the lookup just enqueued by address range (counting sort into 256
// buckets over `host_rows` rows) into `sorted`; `hist` is host_order_scratch_bytes() of scratch.
// Enqueue between launch_lookup_group and launch_gather_roles and hand `sorted` to the gather.
size_t host_order_scratch_bytes();
cudaError_t launch_host_order(const uint64_t* list_host, uint64_t* sorted, const Counters* counters,
                              uint32_t* hist, uint64_t host_rows, int sm_count, cudaStream_t stream);

// Lookup and row copy in one kernel (no index lists): out[i] = row of keys[i].  `grid` is
// the most CTAs to use (a multiple of the SM count); fewer are launched for small batches.
// `deep`: twice the rows in flight per warp at 3 instead of 4 CTAs per SM.  p.tile_shift 3..5
// forces tiles of 8 / 16 / 32 keys; anything else lets the launcher choose.
// `early_host` (ignored with `deep`): the first host row of every warp's first tile is fetched
// before the kernel waits for the launch ahead of it.
cudaError_t launch_extract_direct(const void* keys, int key_bytes, const DirectParams& p, int grid,
                                  int block, int vec_bytes, bool deep, bool early_host, bool pdl,
                                  cudaStream_t stream);

// Widest of 32 / 16 / 4 bytes, not above `want`, that divides row_bytes and the address of
// `out` and of every non-null source base: rows then start on a multiple of it on both sides.
int usable_vec_bytes(uint32_t row_bytes, int want, const void* out, const void* const* src_base,
                     int n_src);

// slice[slot(j)] = host[key(j) & mask]; slot(j) as SlotView describes.
cudaError_t launch_fill_scatter(const void* host_table, void* slice, const uint32_t* keys,
                                const SlotView& slots, uint32_t n, uint32_t row_bytes,
                                int empty_feat, int grid, cudaStream_t stream);
// dst[i] = start + i
cudaError_t launch_iota(uint32_t* dst, uint32_t start, uint32_t n, cudaStream_t stream);

cudaError_t launch_table_clear(const TableView& t, cudaStream_t stream);
// word(j) = pack(loc, slot(j)), slot(j) as SlotView describes
// allow_same: a key that is live already with exactly this word is not an error
cudaError_t launch_table_insert(const TableView& t, const uint32_t* keys, const SlotView& offs,
                                uint32_t loc, uint32_t n, Counters* counters, cudaStream_t stream,
                                bool allow_same = false);
// Refresh: the keys leave their present source; entries whose new source is a peer that holds
// the row already are re-pointed in place, the others removed.
cudaError_t launch_table_repoint(const RepointParams& p, const uint32_t* keys, uint32_t n,
                                 Counters* counters, cudaStream_t stream);
cudaError_t launch_table_evict(const TableView& t, const uint32_t* keys, uint32_t n,
                               Counters* counters, cudaStream_t stream);
cudaError_t launch_table_words(const TableView& t, const uint32_t* keys, uint32_t n,
                               uint32_t* words, cudaStream_t stream);
// Entry j of `offs` (a plain array or a window of the free-slot ring) = offset the peer's
// table holds for keys[j] (must be stored on `expect_loc`).
cudaError_t launch_table_resolve(const TableView& peer, const uint32_t* keys, uint32_t n,
                                 uint32_t expect_loc, const SlotView& offs, Counters* counters,
                                 cudaStream_t stream);

// Whole-id-space classification into ascending key lists (see ClassifyParams).  Pass 1+2
// (launch_classify_count) leave per-tile offsets and per-list totals in `scratch`
// (classify_scratch_bytes(N) bytes); after reading the totals (classify_totals) the caller
// fills p.list_base and runs the scatter pass into `out`.
size_t classify_scratch_bytes(uint64_t num_keys);
cudaError_t launch_classify_count(const ClassifyParams& p, void* scratch, cudaStream_t stream);
const unsigned long long* classify_totals(void* scratch, uint64_t num_keys);
cudaError_t launch_classify_scatter(const ClassifyParams& p, const void* scratch, uint32_t* out,
                                    cudaStream_t stream);

// counts[key] += 1 for every key of the batch (keys outside [0, num_keys) are ignored)
cudaError_t launch_record(const void* keys, int key_bytes, uint32_t n, uint32_t* counts,
                          uint64_t num_keys, cudaStream_t stream);

cudaError_t launch_gen_table(void* dst, uint64_t seed, uint64_t row_begin, uint64_t n_rows,
                             uint64_t dim, int elem_bytes, cudaStream_t stream);

}  // namespace ugc
