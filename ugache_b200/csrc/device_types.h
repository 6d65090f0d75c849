// Types shared by the host runtime and the sm_100a kernels.
#pragma once
#include <cstddef>
#include <cstdint>

namespace ugc {

constexpr int kMaxDevice = 8;
constexpr int kMaxLocation = kMaxDevice + 1;     // GPUs + host
constexpr uint32_t kEmptyWord = 0xffffffffu;     // "not in the table" / never-used slot key
constexpr uint32_t kTombstone = 0x80000000u;     // top bit of a slot key: evicted entry
constexpr int kSlotsPerLine = 4;                 // one 32-byte line = 4 x {key, word}

// Packed (location, row offset) word: the reference's EmbCacheOff
// (coll_cache_lib/cuda/cache_hashtable.h:20-28): 4-bit location above a 28-bit offset.
constexpr uint32_t kOffBits = 28;
constexpr uint32_t kOffMask = (1u << kOffBits) - 1;
__host__ __device__ inline uint32_t pack_word(uint32_t loc, uint32_t off) {
  return (loc << kOffBits) + off;
}
__host__ __device__ inline uint32_t word_loc(uint32_t w) { return (w >> kOffBits) & 0xfu; }
__host__ __device__ inline uint32_t word_off(uint32_t w) { return w & kOffMask; }

// Index record emitted by the lookup for one output row:
//   bits  0..31  source row offset (slice row, or host row)
//   bits 32..35  source location
//   bits 36..63  destination row in the output (28 bits)
// The reference's 8-byte SrcKeyDstVal (coll_cache_lib/cache_context.h:47-52) keeps only 28
// offset bits, which cannot address host rows beyond 2^28.
constexpr uint32_t kMaxBatch = 1u << 28;
__host__ __device__ inline uint64_t make_record(uint32_t dst, uint32_t loc, uint32_t off) {
  return ((uint64_t)dst << 36) | ((uint64_t)loc << 32) | off;
}
__host__ __device__ inline uint32_t rec_off(uint64_t r) { return (uint32_t)r; }
__host__ __device__ inline uint32_t rec_loc(uint64_t r) { return (uint32_t)(r >> 32) & 0xfu; }
__host__ __device__ inline uint32_t rec_dst(uint64_t r) { return (uint32_t)(r >> 36); }

enum TableKind : int { kTableNone = 0, kTableFlat = 1, kTableHashed = 2 };

// Device view of one replica's key -> word table.
//  flat:   words[key], kEmptyWord = absent                       (4 B / key of the id space)
//  hashed: open addressing over 32-byte lines of 4 slots {key, word}; line index =
//          murmur3(key) & line_mask, linear probing over lines; a slot key of kEmptyWord
//          has never been used (search stops), top bit set = evicted (search goes on).
struct TableView {
  int kind;
  uint32_t* flat;
  uint2* slots;
  uint32_t line_mask;
  uint64_t num_keys;  // N, for range checks
};

// Source groups of the factored extraction.
enum Group : int { kGroupLocal = 0, kGroupRemote = 1, kGroupHost = 2, kNumGroup = 3 };

// Device-resident counters of one replica (zeroed at build; the gather's last CTA
// re-zeroes the per-lookup part).
struct Counters {
  uint32_t count[kNumGroup];     // records emitted per group by the current lookup
  uint32_t done_ctas;            // gather CTAs that have finished
  uint32_t last_count[kNumGroup];// copy of count[] of the last finished lookup
  uint32_t last_keys;
  unsigned long long err_key_range;  // sticky
  unsigned long long err_table;      // sticky
  // device clock (ns) of the last gather: earliest CTA start and, per group, latest CTA end
  unsigned long long t_start;
  unsigned long long t_end[kNumGroup];
  uint32_t reserved0[2];
  // grouped gather: rows of each list handed out so far beyond every CTA's first chunk
  // (zeroed by the last CTA of the gather)
  uint32_t cursor[kNumGroup];
  uint32_t reserved2;
  unsigned long long t_index;    // device clock (ns) when the lookup kernel started; 0 = direct
  // direct extraction: per-source counts of the launches that own slot 0 / slot 1 in turn; a
  // launch adds to its slot and clears the other one (whose launch is complete by then)
  uint32_t dcount[2][kNumGroup];
  uint32_t reserved3[2];
  // pooled lookups: rows summed so far, per source group (cumulative)
  unsigned long long pool_rows[kNumGroup];
};

// Written by the last CTA of every extraction into pinned host memory: the host reads it
// without synchronising to pick the extraction mode of the lookups it enqueues next.
struct Feedback {
  uint32_t keys;
  uint32_t count[kNumGroup];
  uint32_t seq;  // ordinal of the lookup these counts belong to (written last; 0 = none yet)
};

// Everything the role-partitioned gather needs.
struct GatherParams {
  const void* src_base[kMaxLocation];  // per location: slice base / peer slice / host table
  void* out;
  const uint64_t* list[kNumGroup];
  Counters* counters;
  Feedback* feedback;   // pinned host mirror of the last lookup's counts, or nullptr
  uint32_t row_bytes;
  uint32_t n_keys;
  int remote_cta_cap;   // most CTAs of the peer group: what keeps the NVLink port full
  int host_cta_cap;     // most CTAs of the host group: what keeps the host link full
  int rows_per_cta_min; // do not give a group more CTAs than count / this
  int fixed_split;      // 1: the two caps ARE the CTA counts of their groups (for sweeps)
  // Seconds per byte over each group's link, scaled by any common factor (local counts twice:
  // row read and row write both use HBM).  The CTAs of a launch are shared out in proportion
  // to rows * row_bytes * t_byte of the groups, within the caps above.
  float t_byte[kNumGroup];
  uint32_t seq;         // ordinal of this lookup among the replica's lookups (for the mirror)
  int dynamic;          // 1: lists are handed out in chunks; a CTA whose own list is drained
                        //    takes chunks of the other groups' lists.  0: fixed striding.
  int pdl;              // launched with programmatic stream serialization
  int bulk_mask;        // bit 0: host rows, bit 1: peer rows go through bulk-async staging
};

// Everything the pooled lookup (table probe, row fetch and per-bag sum in one kernel) needs.
struct PoolParams {
  const void* src_base[kMaxLocation];
  float* out;                // [n_bags, dim] fp32
  TableView table;
  Counters* counters;
  const long long* offsets;  // n_bags + 1 entries (device), or nullptr: bags of bag_size keys
  uint32_t n_keys;
  uint32_t n_bags;
  uint32_t bag_size;
  uint32_t row_bytes;
  uint32_t dim;              // elements per row
  uint32_t local_loc;
  uint32_t host_loc;
  uint32_t host_mask;
  uint32_t lpr_shift;        // log2 of the lanes that share one bag
  uint32_t bags_per_tile;    // consecutive bags one lane group walks through
  uint32_t mean;             // 1: the sum is divided by the bag's length
};

// Everything the direct extraction (lookup and row copy in one kernel, no index lists) needs.
struct DirectParams {
  const void* src_base[kMaxLocation];
  void* out;
  TableView table;
  Counters* counters;
  Feedback* feedback;   // pinned host mirror of the last lookup's counts, or nullptr
  const uint32_t* n_dev;  // if set: the number of keys, in device memory (never above n_keys)
  const void* host_base;  // src_base[host_loc], for the kernel's prologue
  uint32_t n_keys;
  uint32_t row_bytes;
  uint32_t local_loc;
  uint32_t host_loc;
  uint32_t host_mask;
  uint32_t lpr_shift;   // log2 of the lanes that share one row
  uint32_t tile_shift;  // log2 of the keys one warp probes at a time (3..5)
  uint32_t slot;        // which of Counters::dcount this launch adds to (launches alternate)
  uint32_t publish_prev;  // 1: the launch before this one was a direct one; hand its counts on
  uint32_t prev_keys;     // its batch size
  uint32_t prev_seq;      // its ordinal among the replica's lookups
};

// Slot (row offset) numbers for entries j = 0..n-1 of a build / refresh step:
//   data == nullptr          slot(j) = base + j
//   data != nullptr, size 0  slot(j) = data[j]
//   data != nullptr, size>0  slot(j) = data[(base + j) % size]   (a window of the free-slot ring)
struct SlotView {
  uint32_t* data;
  uint32_t base;
  uint32_t size;
};
__host__ __device__ inline uint32_t slot_pos(const SlotView& v, uint32_t j) {
  return v.size ? (uint32_t)(((uint64_t)v.base + j) % v.size) : j;
}

// Classification of the whole id space into ascending key lists.
//  build   (n2b_old == nullptr): list s = keys this reader fetches from GPU s, s in [0, G)
//  refresh (n2b_old != nullptr): kListEvict  = stored here before, not now
//                                kListInsert = stored here now, not before
//                                kListDropRemote = read from a peer before, source changed
//                                kListAttach0+s  = read from peer s now, not before
constexpr int kListEvict = 0, kListInsert = 1, kListDropRemote = 2, kListAttach0 = 3;
constexpr int kMaxClassLists = kListAttach0 + kMaxDevice;  // 11
// Refresh: keys leaving their present source.  A key whose new source is a peer that holds the
// row already gets its entry re-pointed to that peer in place (no interval in which lookups
// would fetch it from the host); every other key's entry is removed.
struct RepointParams {
  TableView own;
  TableView peer[kMaxDevice];  // num_keys == 0: that peer's table is not known here
  const uint32_t* n2b_new;     // device, N entries
  const uint8_t* acc_new;      // device: this reader's source per block (new placement)
  uint32_t me;
  uint32_t num_device;
};

struct ClassifyParams {
  const uint32_t* n2b_old;   // device, N entries, or nullptr
  const uint32_t* n2b_new;   // device, N entries
  const uint8_t* acc_old;    // device: this reader's source per block (old placement)
  const uint8_t* acc_new;    // device: same for the new placement
  uint64_t num_keys;
  uint32_t me;
  uint32_t num_device;
  int num_lists;
  uint64_t list_base[kMaxClassLists];  // start of each list in the output buffer (scatter pass)
};

}  // namespace ugc
