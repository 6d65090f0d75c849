/*
 * CPU ORACLE for the UGache embedding-extraction path.  TEST INFRASTRUCTURE ONLY.
 *
 * This file restates, in plain C, the algorithm of the reference's lookup -> group ->
 * gather path and of its cache build / refresh bookkeeping, so that the CUDA product
 * can be checked against it.  Nothing in the shipped library links, loads or calls it:
 * only the test-suite, the smoke check and the CPU-baseline leg of the benchmark do.
 *
 * Parity status: the reference holds no tests, golden vectors or known-answer fixtures
 * for this path, and it has no CPU extraction routine.  The oracle is pinned against the
 * reference's OWN code instead, compiled in place from the reference tree into oracle/_ref/:
 *   - integer helpers (murmur3 hash, packed location/offset word, table sizing): values
 *     printed by the reference's headers (ref_pin.cu, tests/golden/ref_pin.json);
 *   - both key tables (insert, evict, re-insert, lookup with the host fallback): the words the
 *     reference's SimpleHashTable / FlatHashTable kernels returned on a B200 (ref_pin.cu --gpu,
 *     tests/golden/ref_tables.npz, tests/test_gpu_refpin.py);
 *   - lookup records, grouping, group boundaries, the per-location row copy, the build fill and
 *     the refresh scatter: the reference's LookupHelper, radix-sort dispatcher, find_boundary
 *     and extract_data device code run on a B200 (ref_extract_pin.cu,
 *     tests/golden/ref_extract.json, tests/test_gpu_refpin.py).
 *   - the placement heuristics (Intuitive, Rep, CliquePart): the four placement arrays the
 *     reference's solver classes produce on 13 seeded rankings, run on the CPU
 *     (ref_solver_pin.cc, tests/golden/ref_solver.json, tests/test_oracle_golden.py).
 * Still pinned only by reading ("parity unpinned"): the host-side slot bookkeeping of a refresh.
 *
 * Every function cites the reference file:line it follows (paths relative to the
 * reference project root).
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

#define ORC_EMPTY_KEY 0xffffffffu /* coll_cache_lib/constant.h:83  kEmptyKey  */
#define ORC_EMPTY_POS 0xffffffffu /* coll_cache_lib/cuda/cache_hashtable.h:17 kEmptyPos */

/* ------------------------------------------------------------------------------------
 * Integer helpers (pinned against the reference headers)
 * ---------------------------------------------------------------------------------- */

static inline uint32_t rotl32(uint32_t x, int r) { return (x << r) | (x >> (32 - r)); }

/* MurmurHash3_32 of one 32-bit key.
 * coll_cache_lib/cuda/cache_hashtable.cuh:56-135 (len = 4: one body block, no tail). */
uint32_t orc_murmur3_32(uint32_t key, uint32_t seed) {
  uint32_t h1 = seed;
  uint32_t k1 = key;
  k1 *= 0xcc9e2d51u;
  k1 = rotl32(k1, 15);
  k1 *= 0x1b873593u;
  h1 ^= k1;
  h1 = rotl32(h1, 13);
  h1 = h1 * 5u + 0xe6546b64u;
  h1 ^= 4u; /* len */
  h1 ^= h1 >> 16;
  h1 *= 0x85ebca6bu;
  h1 ^= h1 >> 13;
  h1 *= 0xc2b2ae35u;
  h1 ^= h1 >> 16;
  return h1;
}

/* Packed (location, offset) word: 4-bit location above a 28-bit row offset.
 * coll_cache_lib/cuda/cache_hashtable.h:20-28 (EmbCacheOff). */
uint32_t orc_pack_loc_off(uint32_t loc, uint32_t off) { return (loc << 28) + off; }
uint32_t orc_word_loc(uint32_t w) { return (w >> 28) & 0x0fu; }
uint32_t orc_word_off(uint32_t w) { return w & 0x0fffffffu; }

/* Bucket count of the probing table for `num` entries.
 * coll_cache_lib/cuda/cache_hashtable.cu:222-225 (TableSize, default scale 2). */
uint64_t orc_table_size(uint64_t num, uint64_t scale) {
  uint64_t e = (uint64_t)(1.0 + log2((double)(num >> 1)));
  return ((uint64_t)1 << e) << scale;
}

/* Table choice at build: direct-index table iff the probing table would need more than
 * N/2 buckets.  coll_cache_lib/cache_context.cu:2489-2497. */
int orc_use_flat_table(uint64_t cached_plus_remote, uint64_t num_total) {
  return orc_table_size(cached_plus_remote, 2) > num_total / 2;
}

/* Cache slice capacity in rows.  coll_cache_lib/cache_context.cu:2473. */
uint64_t orc_cache_capacity(uint64_t num_total, double cache_percentage) {
  return (uint64_t)((double)num_total * (cache_percentage + 0.001));
}

/* ------------------------------------------------------------------------------------
 * The reference's probing table ("SimpleHashTable"), restated on the CPU.
 * Buckets are {state_key, val} pairs; state_key == 0xffffffff is "never used"; the top
 * bit set on any other value marks an evicted entry that searches must walk past.
 * ---------------------------------------------------------------------------------- */
typedef struct {
  uint32_t state_key;
  uint32_t val;
} orc_bucket;

/* coll_cache_lib/cuda/cache_hashtable.cuh:207-213 (HashO2N). */
static inline uint32_t hash_o2n(uint32_t id, uint64_t size) {
  return (uint32_t)(orc_murmur3_32(id, 0) % size);
}

void orc_simple_init(orc_bucket* t, uint64_t size) {
  for (uint64_t i = 0; i < size; i++) {
    t[i].state_key = ORC_EMPTY_KEY;
    t[i].val = ORC_EMPTY_POS;
  }
}

/* Insert of a key known to be absent.  Probe order: pos = H(id); on conflict
 * pos = H(pos + delta), delta = 1,2,...  A bucket is free if its top bit is set (never
 * used, or evicted).  coll_cache_lib/cuda/cache_hashtable.cu:75-109, :113-131.
 * Returns the bucket position. */
uint32_t orc_simple_insert(orc_bucket* t, uint64_t size, uint32_t id, uint32_t val) {
  uint32_t pos = hash_o2n(id, size);
  uint32_t delta = 1;
  while ((t[pos].state_key & 0x80000000u) == 0) {
    pos = hash_o2n(pos + delta, size);
    delta += 1;
  }
  t[pos].state_key = id;
  t[pos].val = val;
  return pos;
}

/* Search.  Returns the bucket position or ORC_EMPTY_POS.
 * coll_cache_lib/cuda/cache_hashtable.cuh:175-190 (SearchO2N). */
uint32_t orc_simple_search(const orc_bucket* t, uint64_t size, uint32_t id) {
  uint32_t pos = hash_o2n(id, size);
  uint32_t delta = 1;
  while ((t[pos].state_key & 0x7fffffffu) != id) {
    if (t[pos].state_key == ORC_EMPTY_KEY) return ORC_EMPTY_POS;
    pos = hash_o2n(pos + delta, size);
    delta += 1;
  }
  if (t[pos].state_key & 0x80000000u) return ORC_EMPTY_POS;
  return pos;
}

/* Evict: set the top bit of the key word.
 * coll_cache_lib/cuda/cache_hashtable.cu:269-288. */
void orc_simple_evict(orc_bucket* t, uint64_t size, uint32_t id) {
  uint32_t pos = orc_simple_search(t, size, id);
  if (pos != ORC_EMPTY_POS) t[pos].state_key |= 0x80000000u;
}

/* ------------------------------------------------------------------------------------
 * Lookup -> index records -> gather
 * ---------------------------------------------------------------------------------- */

/* One index record of the lookup: where row i of the output comes from.
 * coll_cache_lib/cache_context.h:47-52 (SrcKeyDstVal) widened to 64-bit offsets so that
 * host fall-back rows beyond 2^28 stay addressable. */
typedef struct {
  uint32_t dst;
  uint32_t loc;
  uint64_t off;
} orc_record;

/* Direct-index table ("FlatHashTable"): word[key], 0xffffffff = absent.
 * Lookup rule: hit -> (loc, off) of the word; miss -> (fallback_loc, key), or
 * (fallback_loc, key mod 2^empty_feat) when the mock-host option is on.
 * coll_cache_lib/cuda/cache_hashtable.cuh:233-237 and :480-503 (LookupHelper). */
void orc_lookup_flat(const uint32_t* flat, const int64_t* keys, uint64_t n, int fallback_loc,
                     int empty_feat, orc_record* rec) {
  for (uint64_t i = 0; i < n; i++) {
    uint64_t key = (uint64_t)keys[i];
    uint32_t w = flat[key];
    rec[i].dst = (uint32_t)i;
    if (w != ORC_EMPTY_POS) {
      rec[i].loc = orc_word_loc(w);
      rec[i].off = orc_word_off(w);
    } else {
      rec[i].loc = (uint32_t)fallback_loc;
      rec[i].off = empty_feat ? (key % ((uint64_t)1 << empty_feat)) : key;
    }
  }
}

/* Same rule through the probing table. */
void orc_lookup_simple(const orc_bucket* t, uint64_t size, const int64_t* keys, uint64_t n,
                       int fallback_loc, int empty_feat, orc_record* rec) {
  for (uint64_t i = 0; i < n; i++) {
    uint64_t key = (uint64_t)keys[i];
    uint32_t pos = orc_simple_search(t, size, (uint32_t)key);
    rec[i].dst = (uint32_t)i;
    if (pos != ORC_EMPTY_POS) {
      rec[i].loc = orc_word_loc(t[pos].val);
      rec[i].off = orc_word_off(t[pos].val);
    } else {
      rec[i].loc = (uint32_t)fallback_loc;
      rec[i].off = empty_feat ? (key % ((uint64_t)1 << empty_feat)) : key;
    }
  }
}

/* The gather over index records: out[rec.dst] = src[rec.loc][rec.off], whole rows.
 * coll_cache_lib/cache_context.cu:214-231 (extract_data) with the per-row pointer-table
 * addressing of :137-159 (DataIterMixLoc). */
void orc_extract_records(const orc_record* rec, uint64_t n, const void* const* src_base,
                         uint64_t row_bytes, void* out) {
  for (uint64_t i = 0; i < n; i++) {
    const char* s = (const char*)src_base[rec[i].loc] + rec[i].off * row_bytes;
    memcpy((char*)out + (uint64_t)rec[i].dst * row_bytes, s, row_bytes);
  }
}

/* What the whole path collapses to for any correct placement: out[i] = table[keys[i]].
 * One memcpy per key, OpenMP static schedule over keys; this is the routine the CPU
 * baseline times.  coll_cache_lib/cache_context.cu:214-231 with the host-only source of
 * :195-212 (DataIterPerLoc over IdxStoreDirect, cache_context.h:340-355). */
void orc_gather(const void* table, const int64_t* keys, uint64_t n, uint64_t row_bytes,
                int empty_feat, void* out, int num_threads) {
  const uint64_t mask = empty_feat ? (((uint64_t)1 << empty_feat) - 1) : ~(uint64_t)0;
#ifdef _OPENMP
  if (num_threads <= 0) num_threads = omp_get_max_threads();
#pragma omp parallel for schedule(static) num_threads(num_threads)
#endif
  for (int64_t i = 0; i < (int64_t)n; i++) {
    uint64_t row = (uint64_t)keys[i] & mask;
    memcpy((char*)out + (uint64_t)i * row_bytes, (const char*)table + row * row_bytes, row_bytes);
  }
}

int orc_max_threads(void) {
#ifdef _OPENMP
  return omp_get_max_threads();
#else
  return 1;
#endif
}

/* Fill / refresh scatter: slice[slot[j]] = host[key[j]] (slot == NULL means slot[j] = j).
 * coll_cache_lib/cache_context.cu:2480-2484 (build) and :4061-4070 with the destination
 * list of cache_context.h:356-361 (refresh). */
void orc_fill(const void* host_table, const uint32_t* keys, const uint32_t* slots, uint64_t n,
              uint64_t row_bytes, int empty_feat, void* slice) {
  const uint64_t mask = empty_feat ? (((uint64_t)1 << empty_feat) - 1) : ~(uint64_t)0;
  for (uint64_t j = 0; j < n; j++) {
    uint64_t row = (uint64_t)keys[j] & mask;
    uint64_t slot = slots ? slots[j] : j;
    memcpy((char*)slice + slot * row_bytes, (const char*)host_table + row * row_bytes, row_bytes);
  }
}

/* ------------------------------------------------------------------------------------
 * Placement heuristics (host-side input of the path).  Output arrays:
 *   nid_to_block[N], block_placement[B] (bit g = stored on GPU g),
 *   block_access_from[G*B] (row g = source per block for reader g; G = host),
 *   block_density[B] (percent of N).
 * rank_ids: ids by descending frequency; rank_freqs: the frequencies.
 * ---------------------------------------------------------------------------------- */

/* coll_cache_lib/coll_cache/optimal_solver_class.cc:1251-1404 (IntuitiveSolver::Solve).
 * cache_percent is in percent (0..100) as in the reference.  Returns the block count. */
int orc_solve_intuitive(int num_device, uint32_t num_node, const uint32_t* rank_ids,
                        const uint32_t* rank_freqs, double cache_percent, double T_local,
                        double T_remote, double T_cpu, double min_freq, uint32_t* nid_to_block,
                        uint8_t* block_placement, uint8_t* block_access_from,
                        double* block_density) {
  const int num_block = num_device + 2;
  const uint32_t num_cached = (uint32_t)(num_node * (cache_percent / (double)100));
  uint32_t part_min = 0;
  uint32_t part_max = 0;
  if (num_device > 1) {
    uint32_t a = num_cached, b = (num_node - num_cached) / (uint32_t)(num_device - 1);
    part_max = a < b ? a : b;
  }
#define ORC_LB(p) (num_cached - (p))
#define ORC_RB(p)                                                                            \
  ((((num_cached + (p) * (uint32_t)(num_device - 1)) > 1u)                                  \
        ? (num_cached + (p) * (uint32_t)(num_device - 1))                                    \
        : 1u) -                                                                              \
   1u)
#define ORC_FMAX(x) (min_freq > (double)(x) ? min_freq : (double)(x))
  const double mu = 1 + (T_cpu - T_remote) / (T_remote - T_local) * num_device;
  uint32_t part = part_min;
  if (mu < 1) {
    part = part_min;
  } else if ((double)rank_freqs[ORC_LB(part_max)] < ORC_FMAX(rank_freqs[ORC_RB(part_max)]) * mu) {
    part = part_max;
  } else {
    while (part_max - part_min > 1) {
      part = (part_min + part_max) / 2;
      if ((double)rank_freqs[ORC_LB(part)] < ORC_FMAX(rank_freqs[ORC_RB(part)]) * mu) {
        part_min = part;
      } else {
        part_max = part;
      }
    }
    part = part_max;
  }
  const uint32_t lb = ORC_LB(part), rb = ORC_RB(part);
  for (uint32_t rank = 0; rank < num_node; rank++) {
    uint32_t id = rank_ids[rank];
    if (rank < lb) {
      nid_to_block[id] = 0;
    } else if (rank <= rb) {
      nid_to_block[id] = (rank % (uint32_t)num_device) + 1;
    } else {
      nid_to_block[id] = (uint32_t)num_device + 1;
    }
  }
  block_placement[0] = (uint8_t)((1 << num_device) - 1);
  for (int i = 0; i < num_device; i++) block_placement[i + 1] = (uint8_t)(1 << i);
  block_placement[num_device + 1] = 0;
  for (int dev = 0; dev < num_device; dev++) {
    uint8_t* row = block_access_from + (size_t)dev * num_block;
    row[0] = (uint8_t)dev;
    for (int b = 1; b <= num_device; b++) row[b] = (uint8_t)(b - 1);
    row[num_device + 1] = (uint8_t)num_device;
  }
  block_density[0] = (double)lb * 100 / (double)num_node;
  for (int b = 1; b <= num_device; b++) block_density[b] = part * (double)100 / (double)num_node;
  block_density[num_device + 1] = 100 - (rb / (double)num_node) * 100;
#undef ORC_LB
#undef ORC_RB
#undef ORC_FMAX
  return num_block;
}

/* coll_cache_lib/coll_cache/optimal_solver_class.cc:1869-1924 (RepSolver::Solve). */
int orc_solve_rep(int num_device, uint32_t num_node, const uint32_t* rank_ids,
                  double cache_percent, uint32_t* nid_to_block, uint8_t* block_placement,
                  uint8_t* block_access_from, double* block_density) {
  const int num_block = 2;
  const uint32_t rep = (uint32_t)(num_node * (cache_percent / (double)100));
  for (uint32_t rank = 0; rank < num_node; rank++) nid_to_block[rank_ids[rank]] = rank < rep ? 0 : 1;
  block_placement[0] = (uint8_t)((1 << num_device) - 1);
  block_placement[1] = 0;
  for (int dev = 0; dev < num_device; dev++) {
    block_access_from[dev * num_block + 0] = (uint8_t)dev;
    block_access_from[dev * num_block + 1] = (uint8_t)num_device;
  }
  block_density[0] = (double)rep * 100 / (double)num_node;
  block_density[1] = (double)(num_node - rep) * 100 / (double)num_node;
  return num_block;
}

/* coll_cache_lib/coll_cache/optimal_solver_class.cc:1926-2058 (CliquePartSolver::Solve,
 * default hash: block = rank % clique_size); clique_size == num_device on a switch
 * (coll_cache_lib/coll_cache/asymm_link_desc.cc:420-424). */
int orc_solve_clique_part(int num_device, int clique_size, uint32_t num_node,
                          const uint32_t* rank_ids, double cache_percent, uint32_t* nid_to_block,
                          uint8_t* block_placement, uint8_t* block_access_from,
                          double* block_density) {
  const int num_clique = (num_device + clique_size - 1) / clique_size;
  const int num_block = clique_size + 1;
  const uint32_t num_cached = (uint32_t)ceil(num_node * (cache_percent / (double)100));
  const uint32_t per = (num_node + (uint32_t)clique_size - 1) / (uint32_t)clique_size;
  const uint32_t part = num_cached < per ? num_cached : per;
  for (uint32_t rank = 0; rank < num_node; rank++) {
    uint32_t b = (uint32_t)clique_size;
    if ((uint64_t)rank < (uint64_t)part * clique_size) b = rank % (uint32_t)clique_size;
    nid_to_block[rank_ids[rank]] = b;
  }
  for (int b = 0; b < clique_size; b++) {
    uint8_t storage = 0;
    for (int c = 0; c < num_clique; c++) storage |= (uint8_t)(1 << (c * clique_size + b));
    block_placement[b] = storage;
    for (int dev = 0; dev < num_device; dev++)
      block_access_from[dev * num_block + b] = (uint8_t)((dev / clique_size) * clique_size + b);
    block_density[b] = (double)part * 100 / (double)num_node;
  }
  block_placement[clique_size] = 0;
  for (int dev = 0; dev < num_device; dev++)
    block_access_from[dev * num_block + clique_size] = (uint8_t)num_device;
  block_density[clique_size] =
      ((double)num_node - (double)part * clique_size) * 100 / (double)num_node;
  return num_block;
}

/* ------------------------------------------------------------------------------------
 * Cache model: for reader `rank`, the (location, offset) word of every key.
 *
 * Keys are bucketed by block_access_from[rank][nid_to_block[key]]
 * (coll_cache_lib/cuda/cache_hashtable.cuh:741-835, DetectKeysForAllSource); a GPU's
 * slot for a key it stores is the key's position in that GPU's own list
 * (cache_hashtable.cuh:516-522, :605-608, InsertSeqOffWithLoc); a reader learns a peer's
 * slot from the peer's table (coll_cache_lib/cache_context.cu:2531-2570).  The reference
 * builds those lists with an OpenMP scan whose chunk order varies run to run, so only
 * the SET per GPU is defined there; this model fixes the order to ascending key, which
 * the product follows.
 *
 * words[key] = pack(loc, off) for keys served from a GPU, 0xffffffff for host keys.
 * slot_of[g*N + key] (caller scratch, G*N u32) receives each GPU's own slot numbering.
 * Returns 0, or -1 if some GPU's list exceeds `capacity`.
 * ---------------------------------------------------------------------------------- */
int orc_model_build(int num_device, uint32_t num_node, const uint32_t* nid_to_block,
                    const uint8_t* block_access_from, int num_block, int rank, uint64_t capacity,
                    uint32_t* slot_of, uint32_t* words, uint64_t* per_src_count) {
  for (int g = 0; g < num_device; g++) {
    const uint8_t* acc = block_access_from + (size_t)g * num_block;
    uint32_t next = 0;
    uint32_t* slots = slot_of + (size_t)g * num_node;
    for (uint32_t k = 0; k < num_node; k++) {
      if (acc[nid_to_block[k]] == g) {
        slots[k] = next++;
      } else {
        slots[k] = ORC_EMPTY_POS;
      }
    }
    if ((uint64_t)next > capacity) return -1;
  }
  const uint8_t* acc = block_access_from + (size_t)rank * num_block;
  for (int s = 0; s <= num_device; s++) per_src_count[s] = 0;
  for (uint32_t k = 0; k < num_node; k++) {
    uint32_t s = acc[nid_to_block[k]];
    per_src_count[s]++;
    if (s == (uint32_t)num_device) {
      words[k] = ORC_EMPTY_POS;
    } else {
      words[k] = orc_pack_loc_off(s, slot_of[(size_t)s * num_node + k]);
    }
  }
  return 0;
}

/* Refresh bookkeeping for ONE GPU's own slots, old placement -> new placement.
 * coll_cache_lib/cache_context.cu:3944-4107:
 *   evicted  = stored under the old placement, not under the new  (:3980-3990)
 *   inserted = stored under the new placement, not under the old  (:3962-3972)
 *   freed slots are appended to the free list (cache_hashtable.cuh:625-630), new rows
 *   take slots from its FRONT (:637-645), preserved rows keep their slot.
 * Both lists are walked in ascending key order (see orc_model_build on ordering).
 * free_list holds *n_free entries on entry (capacity of the array: cap_free).
 * slots[key] is updated in place.  Returns 0, -1 if the free list runs dry. */
int orc_model_refresh_slots(uint32_t num_node, int gpu, const uint32_t* old_nid_to_block,
                            const uint8_t* old_placement, const uint32_t* new_nid_to_block,
                            const uint8_t* new_placement, uint32_t* slots, uint32_t* free_list,
                            uint64_t* n_free, uint64_t cap_free, uint64_t* n_evicted,
                            uint64_t* n_inserted) {
  const uint8_t bit = (uint8_t)(1 << gpu);
  uint64_t nf = *n_free, ev = 0, ins = 0;
  for (uint32_t k = 0; k < num_node; k++) {
    int was = (old_placement[old_nid_to_block[k]] & bit) != 0;
    int is = (new_placement[new_nid_to_block[k]] & bit) != 0;
    if (was && !is) {
      if (nf >= cap_free) return -1;
      free_list[nf++] = slots[k];
      slots[k] = ORC_EMPTY_POS;
      ev++;
    }
  }
  uint64_t head = 0;
  for (uint32_t k = 0; k < num_node; k++) {
    int was = (old_placement[old_nid_to_block[k]] & bit) != 0;
    int is = (new_placement[new_nid_to_block[k]] & bit) != 0;
    if (is && !was) {
      if (head >= nf) return -1;
      slots[k] = free_list[head++];
      ins++;
    }
  }
  memmove(free_list, free_list + head, (nf - head) * sizeof(uint32_t));
  *n_free = nf - head;
  *n_evicted = ev;
  *n_inserted = ins;
  return 0;
}

/* ------------------------------------------------------------------------------------
 * Synthetic inputs (stand-ins for the reference's datasets; same shapes and skew).
 * ---------------------------------------------------------------------------------- */

static inline uint64_t splitmix64(uint64_t x) {
  x += 0x9e3779b97f4a7c15ull;
  x = (x ^ (x >> 30)) * 0xbf58476d1ce4e5b9ull;
  x = (x ^ (x >> 27)) * 0x94d049bb133111ebull;
  return x ^ (x >> 31);
}

/* Table generator: element e = row*dim + col of the table gets a value uniform in [-1,1)
 * that depends only on (seed, e), so any row can be regenerated on demand.
 * fp32: 24 random bits -> bits*2^-23 - 1 (exact).  fp16 bit pattern: 11 random bits ->
 * bits*2^-10 - 1 (exact in binary16). */
static inline float gen_f32(uint64_t seed, uint64_t e) {
  uint64_t x = splitmix64(seed ^ splitmix64(e));
  return (float)(x >> 40) * (1.0f / 8388608.0f) - 1.0f;
}
static inline uint16_t gen_f16_bits(uint64_t seed, uint64_t e) {
  uint64_t x = splitmix64(seed ^ splitmix64(e));
  int v = (int)(x >> 53) - 1024; /* value = v * 2^-10, v in [-1024, 1023] */
  if (v == 0) return 0;
  uint16_t sign = 0;
  if (v < 0) {
    sign = 0x8000;
    v = -v;
  }
  int msb = 31 - __builtin_clz((unsigned)v);              /* 0..10 */
  int exp = msb - 10 + 15;                                /* biased exponent */
  uint16_t man = (uint16_t)(((unsigned)v << (10 - msb)) & 0x3ff);
  return (uint16_t)(sign | (exp << 10) | man);
}

void orc_gen_rows_f32(uint64_t seed, uint64_t row_begin, uint64_t n_rows, uint64_t dim, float* out) {
#ifdef _OPENMP
#pragma omp parallel for schedule(static)
#endif
  for (int64_t r = 0; r < (int64_t)n_rows; r++)
    for (uint64_t c = 0; c < dim; c++)
      out[(uint64_t)r * dim + c] = gen_f32(seed, (row_begin + (uint64_t)r) * dim + c);
}

void orc_gen_rows_f16(uint64_t seed, uint64_t row_begin, uint64_t n_rows, uint64_t dim,
                      uint16_t* out) {
#ifdef _OPENMP
#pragma omp parallel for schedule(static)
#endif
  for (int64_t r = 0; r < (int64_t)n_rows; r++)
    for (uint64_t c = 0; c < dim; c++)
      out[(uint64_t)r * dim + c] = gen_f16_bits(seed, (row_begin + (uint64_t)r) * dim + c);
}

/* Rows for an arbitrary key list (what a gather of those keys must return). */
void orc_gen_rows_for_keys_f32(uint64_t seed, const int64_t* keys, uint64_t n, uint64_t dim,
                               float* out) {
#ifdef _OPENMP
#pragma omp parallel for schedule(static)
#endif
  for (int64_t i = 0; i < (int64_t)n; i++)
    for (uint64_t c = 0; c < dim; c++)
      out[(uint64_t)i * dim + c] = gen_f32(seed, (uint64_t)keys[i] * dim + c);
}
void orc_gen_rows_for_keys_f16(uint64_t seed, const int64_t* keys, uint64_t n, uint64_t dim,
                               uint16_t* out) {
#ifdef _OPENMP
#pragma omp parallel for schedule(static)
#endif
  for (int64_t i = 0; i < (int64_t)n; i++)
    for (uint64_t c = 0; c < dim; c++)
      out[(uint64_t)i * dim + c] = gen_f16_bits(seed, (uint64_t)keys[i] * dim + c);
}

/* Zipf ranks by the reference generator's bounded-Pareto inverse CDF
 * (eval/dlr/common/ds_generator.py:11-15 with datagen/dlr/syn.py:43 passing alpha-1):
 *   x = ((-H^a L^a) / (u (H^a - L^a) - H^a))^(1/a),  a = alpha-1, L = 1, H = N,
 *   rank0 = floor(x) - 1  in [0, N-1];   a == 0 uses the limit x = H^u.
 * u[i] in [0,1) are supplied by the caller (seeded generator on the harness side). */
void orc_zipf_ranks(const double* u, uint64_t n, uint64_t N, double alpha, int64_t* rank0) {
  const double a = alpha - 1.0;
  const double H = (double)N;
  const double Ha = pow(H, a);
  for (uint64_t i = 0; i < n; i++) {
    double x;
    if (fabs(a) < 1e-12) {
      x = pow(H, u[i]);
    } else {
      x = pow((-Ha) / (u[i] * (Ha - 1.0) - Ha), 1.0 / a);
    }
    int64_t r = (int64_t)x - 1;
    if (r < 0) r = 0;
    if (r >= (int64_t)N) r = (int64_t)N - 1;
    rank0[i] = r;
  }
}

/* rank -> id bijection on [0, N): id = (A*rank + B) mod N, gcd(A, N) = 1. */
void orc_rank_to_id(const int64_t* rank0, uint64_t n, uint64_t N, uint64_t A, uint64_t B,
                    int64_t* ids) {
  for (uint64_t i = 0; i < n; i++) {
    __uint128_t t = (__uint128_t)A * (uint64_t)rank0[i] + B;
    ids[i] = (int64_t)(uint64_t)(t % N);
  }
}
