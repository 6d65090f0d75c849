// sm_100a kernels of the extraction path.  Everything here is integer index arithmetic
// and raw byte copies; rows move as 16- or 32-byte vectors (4-byte words when a row size
// is not a multiple of 16).
#include "kernels.cuh"

#include <cuda_fp16.h>

#include <algorithm>
#include <cstring>

namespace ugc {

namespace {

constexpr int kBlock = 256;          // threads per CTA everywhere
constexpr int kWarpsPerBlock = kBlock / 32;
constexpr unsigned kFull = 0xffffffffu;

// ------------------------------------------------------------------------------------
// memory access helpers
// ------------------------------------------------------------------------------------

template <int BYTES>
struct Vec;
template <>
struct Vec<4> {
  uint32_t v[1];
};
template <>
struct __align__(16) Vec<16> {
  uint32_t v[4];
};
template <>
struct __align__(32) Vec<32> {
  uint32_t v[8];
};

// Row payload loads: read-only path, allocating in L1.  Under a Zipf key distribution a few
// rows make up a large share of every batch (the hottest row alone is 18 % of the keys at
// alpha 1.2, 32 % at 1.4); without L1 allocation all of those reads queue at the few L2 slices
// that hold the row, which cost 20-25 % of the step (42 -> 31 us at alpha 1.4, measured).
#define UGC_LD_ROW "ld.global.nc"
__device__ __forceinline__ void ld_row(Vec<4>& r, const void* p) {
  asm volatile(UGC_LD_ROW ".b32 %0, [%1];" : "=r"(r.v[0]) : "l"(p));
}
__device__ __forceinline__ void ld_row(Vec<16>& r, const void* p) {
  asm volatile(UGC_LD_ROW ".v4.b32 {%0,%1,%2,%3}, [%4];"
               : "=r"(r.v[0]), "=r"(r.v[1]), "=r"(r.v[2]), "=r"(r.v[3])
               : "l"(p));
}
__device__ __forceinline__ void ld_row(Vec<32>& r, const void* p) {
  asm volatile(UGC_LD_ROW ".v8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
               : "=r"(r.v[0]), "=r"(r.v[1]), "=r"(r.v[2]), "=r"(r.v[3]), "=r"(r.v[4]),
                 "=r"(r.v[5]), "=r"(r.v[6]), "=r"(r.v[7])
               : "l"(p));
}
// Output stores: streaming (evict-first) so the written rows do not push hot cache rows
// out of L2.
__device__ __forceinline__ void st_row(void* p, const Vec<4>& r) {
  asm volatile("st.global.cs.b32 [%0], %1;" ::"l"(p), "r"(r.v[0]) : "memory");
}
__device__ __forceinline__ void st_row(void* p, const Vec<16>& r) {
  asm volatile("st.global.cs.v4.b32 [%0], {%1,%2,%3,%4};" ::"l"(p), "r"(r.v[0]), "r"(r.v[1]),
               "r"(r.v[2]), "r"(r.v[3])
               : "memory");
}
__device__ __forceinline__ void st_row(void* p, const Vec<32>& r) {
  asm volatile("st.global.cs.v8.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};" ::"l"(p), "r"(r.v[0]),
               "r"(r.v[1]), "r"(r.v[2]), "r"(r.v[3]), "r"(r.v[4]), "r"(r.v[5]), "r"(r.v[6]),
               "r"(r.v[7])
               : "memory");
}
// Plain (write-back) store used when the destination is the cache slice itself.
__device__ __forceinline__ void st_keep(void* p, const Vec<4>& r) {
  *reinterpret_cast<uint32_t*>(p) = r.v[0];
}
__device__ __forceinline__ void st_keep(void* p, const Vec<16>& r) {
  *reinterpret_cast<uint4*>(p) = make_uint4(r.v[0], r.v[1], r.v[2], r.v[3]);
}
__device__ __forceinline__ void st_keep(void* p, const Vec<32>& r) {
  asm volatile("st.global.v8.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};" ::"l"(p), "r"(r.v[0]),
               "r"(r.v[1]), "r"(r.v[2]), "r"(r.v[3]), "r"(r.v[4]), "r"(r.v[5]), "r"(r.v[6]),
               "r"(r.v[7])
               : "memory");
}

// One 32-byte table line = 4 slots {key, word}.  Coherent load (a refresh may be
// inserting or evicting while lookups run), L2 only.
struct Line {
  uint32_t key[kSlotsPerLine];
  uint32_t word[kSlotsPerLine];
};
__device__ __forceinline__ Line ld_line(const uint2* slots, uint32_t line) {
  Line l;
  const uint2* p = slots + (size_t)line * kSlotsPerLine;
  asm volatile("ld.global.cg.v8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
               : "=r"(l.key[0]), "=r"(l.word[0]), "=r"(l.key[1]), "=r"(l.word[1]),
                 "=r"(l.key[2]), "=r"(l.word[2]), "=r"(l.key[3]), "=r"(l.word[3])
               : "l"(p));
  return l;
}

// MurmurHash3_32 of one 32-bit key, seed 0: the hash of the reference's probing table
// (coll_cache_lib/cuda/cache_hashtable.cuh:56-135); here it picks the first line.
__host__ __device__ __forceinline__ uint32_t murmur3_32(uint32_t key) {
  uint32_t k1 = key * 0xcc9e2d51u;
  k1 = (k1 << 15) | (k1 >> 17);
  k1 *= 0x1b873593u;
  uint32_t h1 = k1;
  h1 = (h1 << 13) | (h1 >> 19);
  h1 = h1 * 5u + 0xe6546b64u;
  h1 ^= 4u;
  h1 ^= h1 >> 16;
  h1 *= 0x85ebca6bu;
  h1 ^= h1 >> 13;
  h1 *= 0xc2b2ae35u;
  h1 ^= h1 >> 16;
  return h1;
}

// Result of inspecting one line for `key`: the word if a live slot matches, else whether
// the search may stop (a never-used slot was seen).
__device__ __forceinline__ bool line_find(const Line& l, uint32_t key, uint32_t& word, bool& stop) {
  stop = false;
#pragma unroll
  for (int s = 0; s < kSlotsPerLine; s++) {
    if (l.key[s] == key) {  // live slots carry the key with the top bit clear
      word = l.word[s];
      return true;
    }
  }
#pragma unroll
  for (int s = 0; s < kSlotsPerLine; s++) stop |= (l.key[s] == kEmptyWord);
  return false;
}

// Probes after the first line (already loaded by the caller).  Bounded by the table size.
__device__ __forceinline__ uint32_t probe_rest(const uint2* slots, uint32_t line_mask, uint32_t key,
                                            uint32_t line) {
  for (uint32_t step = 0; step < line_mask; step++) {
    line = (line + 1) & line_mask;
    Line l = ld_line(slots, line);
    uint32_t w;
    bool stop;
    if (line_find(l, key, w, stop)) return w;
    if (stop) return kEmptyWord;
  }
  return kEmptyWord;
}

__device__ __forceinline__ uint32_t table_lookup(const TableView& t, uint32_t key) {
  if (t.kind == kTableFlat) {
    uint32_t w;
    asm volatile("ld.global.cg.b32 %0, [%1];" : "=r"(w) : "l"(t.flat + key));
    return w;
  }
  uint32_t line = murmur3_32(key) & t.line_mask;
  Line l = ld_line(t.slots, line);
  uint32_t w;
  bool stop;
  if (line_find(l, key, w, stop)) return w;
  if (stop) return kEmptyWord;
  return probe_rest(t.slots, t.line_mask, key, line);
}

// ------------------------------------------------------------------------------------
// lookup + group by source
// ------------------------------------------------------------------------------------
template <typename KeyT, int kKeysPerThread>
__global__ void __launch_bounds__(kBlock)
    lookup_group_kernel(const KeyT* __restrict__ keys, uint32_t n, TableView t, uint32_t local_loc,
                        uint32_t host_loc, uint32_t host_mask, uint64_t* __restrict__ list_local,
                        uint64_t* __restrict__ list_remote, uint64_t* __restrict__ list_host,
                        Counters* counters) {
  __shared__ uint32_t s_cnt[kWarpsPerBlock][kKeysPerThread][kNumGroup];
  __shared__ uint32_t s_base[kNumGroup];

  const uint32_t tid = threadIdx.x;
  const uint32_t warp = tid >> 5, lane = tid & 31;
  const uint32_t tile_base = blockIdx.x * (kBlock * kKeysPerThread);
  unsigned long long t_begin = 0;
  if (blockIdx.x == 0 && tid == 0) asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t_begin));

  uint32_t key[kKeysPerThread];
  bool valid[kKeysPerThread];
  uint32_t bad = 0;
#pragma unroll
  for (int j = 0; j < kKeysPerThread; j++) {
    uint32_t idx = tile_base + j * kBlock + tid;
    valid[j] = idx < n;
    uint64_t k = valid[j] ? (uint64_t)keys[idx] : 0;
    if (k >= t.num_keys) {  // also catches negative int64 ids
      valid[j] = false;
      bad++;
      k = 0;
    }
    key[j] = (uint32_t)k;
  }
  // Let the gather that follows in the stream be scheduled as soon as SM resources allow
  // (it waits for this grid's completion before it reads the lists).
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

  // First probe of every key is issued before any is consumed.
  uint32_t word[kKeysPerThread];
  if (t.kind == kTableFlat) {
#pragma unroll
    for (int j = 0; j < kKeysPerThread; j++) {
      word[j] = kEmptyWord;
      if (valid[j]) asm volatile("ld.global.cg.b32 %0, [%1];" : "=r"(word[j]) : "l"(t.flat + key[j]));
    }
  } else {
    Line first[kKeysPerThread];
    uint32_t line[kKeysPerThread];
#pragma unroll
    for (int j = 0; j < kKeysPerThread; j++) {
      line[j] = murmur3_32(key[j]) & t.line_mask;
      first[j] = ld_line(t.slots, line[j]);
    }
#pragma unroll
    for (int j = 0; j < kKeysPerThread; j++) {
      uint32_t w;
      bool stop;
      if (line_find(first[j], key[j], w, stop)) {
        word[j] = w;
      } else if (stop) {
        word[j] = kEmptyWord;
      } else {
        word[j] = probe_rest(t.slots, t.line_mask, key[j], line[j]);
      }
    }
  }

  // Keys and table have been read; everything below touches the lists and counters that
  // the previous lookup's gather may still be using: wait for it (no-op unless this kernel
  // was launched with programmatic stream serialization).
  asm volatile("griddepcontrol.wait;" ::: "memory");
  if (bad) atomicAdd(&counters->err_key_range, (unsigned long long)bad);
  if (blockIdx.x == 0 && tid < kNumGroup) counters->t_end[tid] = 0;  // re-armed for the gather's timestamps
  if (blockIdx.x == 0 && tid == 0) counters->t_index = t_begin;

  // Group, count per warp with ballots.
  uint32_t group[kKeysPerThread], rank_in_warp[kKeysPerThread];
  uint64_t rec[kKeysPerThread];
#pragma unroll
  for (int j = 0; j < kKeysPerThread; j++) {
    uint32_t idx = tile_base + j * kBlock + tid;
    uint32_t loc, off;
    if (word[j] == kEmptyWord) {
      loc = host_loc;
      off = key[j] & host_mask;
      group[j] = kGroupHost;
    } else {
      loc = word_loc(word[j]);
      off = word_off(word[j]);
      group[j] = (loc == local_loc) ? kGroupLocal : kGroupRemote;
    }
    if (!valid[j]) group[j] = kNumGroup;
    rec[j] = make_record(idx, loc, off);
    rank_in_warp[j] = 0;
#pragma unroll
    for (int g = 0; g < kNumGroup; g++) {
      unsigned m = __ballot_sync(kFull, group[j] == (uint32_t)g);
      if (group[j] == (uint32_t)g) rank_in_warp[j] = __popc(m & ((1u << lane) - 1));
      if (lane == 0) s_cnt[warp][j][g] = __popc(m);
    }
  }
  __syncthreads();
  // Exclusive scan of the 8x4 per-warp counts of each group (one thread per group), then
  // one global atomic per (CTA, group).
  if (tid < kNumGroup) {
    uint32_t run = 0;
    for (int j = 0; j < kKeysPerThread; j++)
      for (int w = 0; w < kWarpsPerBlock; w++) {
        uint32_t c = s_cnt[w][j][tid];
        s_cnt[w][j][tid] = run;
        run += c;
      }
    s_base[tid] = run ? atomicAdd(&counters->count[tid], run) : 0;
  }
  __syncthreads();
#pragma unroll
  for (int j = 0; j < kKeysPerThread; j++) {
    if (group[j] == kNumGroup) continue;
    uint32_t pos = s_base[group[j]] + s_cnt[warp][j][group[j]] + rank_in_warp[j];
    uint64_t* dst = group[j] == kGroupLocal ? list_local
                                             : (group[j] == kGroupRemote ? list_remote : list_host);
    dst[pos] = rec[j];
  }
}

// ------------------------------------------------------------------------------------
// row copy core: a "worker" is a group of LPR lanes that copies one row at a time,
// UNROLL rows in flight per worker.
// ------------------------------------------------------------------------------------
struct RecordIndex {  // rows described by 64-bit records
  const uint64_t* list;
  const void* const* src_base;  // per location
  char* out;
  uint32_t row_bytes;
  __device__ __forceinline__ void get(uint32_t i, const char*& src, char*& dst) const {
    uint64_t r = list[i];
    src = static_cast<const char*>(src_base[rec_loc(r)]) + (size_t)rec_off(r) * row_bytes;
    dst = out + (size_t)rec_dst(r) * row_bytes;
  }
};
struct KeySlotIndex {  // fill: host row of a key -> cache slot
  const uint32_t* keys;
  SlotView slots;
  uint32_t host_mask;
  const char* host;
  char* slice;
  uint32_t row_bytes;
  __device__ __forceinline__ void get(uint32_t i, const char*& src, char*& dst) const {
    uint32_t k = keys[i] & host_mask;
    uint32_t s = slots.data ? slots.data[slot_pos(slots, i)] : slots.base + i;
    src = host + (size_t)k * row_bytes;
    dst = slice + (size_t)s * row_bytes;
  }
};

template <int VEC, int LPR, int UNROLL, bool STREAM_OUT, typename Index>
__device__ __forceinline__ void copy_rows(const Index& ix, uint32_t count, uint32_t worker,
                                          uint32_t n_workers, uint32_t sublane,
                                          uint32_t vecs_per_row) {
  for (uint32_t base = worker; base < count; base += n_workers * UNROLL) {
    const char* src[UNROLL];
    char* dst[UNROLL];
    bool ok[UNROLL];
#pragma unroll
    for (int u = 0; u < UNROLL; u++) {
      uint32_t i = base + u * n_workers;
      ok[u] = i < count;
      src[u] = nullptr;
      dst[u] = nullptr;
      if (ok[u]) ix.get(i, src[u], dst[u]);
    }
    for (uint32_t c = sublane; c < vecs_per_row; c += LPR) {
      Vec<VEC> v[UNROLL];
#pragma unroll
      for (int u = 0; u < UNROLL; u++)
        if (ok[u]) ld_row(v[u], src[u] + (size_t)c * VEC);
#pragma unroll
      for (int u = 0; u < UNROLL; u++)
        if (ok[u]) {
          if (STREAM_OUT) {
            st_row(dst[u] + (size_t)c * VEC, v[u]);
          } else {
            st_keep(dst[u] + (size_t)c * VEC, v[u]);
          }
        }
    }
  }
}

// ------------------------------------------------------------------------------------
// role-partitioned gather
// ------------------------------------------------------------------------------------
__device__ __forceinline__ int ceil_div_i(uint32_t a, uint32_t b) { return (int)((a + b - 1) / b); }

// Splits the grid (>= 3 CTAs) into host / remote / local groups from the device-resident
// counts.  CTAs [0, n_host) serve host rows, [n_host, n_host+n_remote) peer rows, the rest
// local rows: the long-latency sources get the lowest block indices, which start first.
// A group's share of the CTAs follows the time its bytes need on its link (bytes / bandwidth,
// the rule the reference's link tables encode as SM counts per link,
// coll_cache_lib/coll_cache/asymm_link_desc.cc:247-289), limited by what keeps that link full
// (the caps) and by the rows there are.  A non-empty group always gets at least one CTA.
__device__ __forceinline__ void split_roles(const GatherParams& p, const uint32_t cnt[kNumGroup],
                                            int grid, int& n_host, int& n_remote) {
  const uint32_t rmin = (uint32_t)p.rows_per_cta_min;
  const float t_loc = (float)cnt[kGroupLocal] * 2.0f * p.t_byte[kGroupLocal];
  const float t_rem = (float)cnt[kGroupRemote] * p.t_byte[kGroupRemote];
  const float t_host = (float)cnt[kGroupHost] * p.t_byte[kGroupHost];
  const float t_all = t_loc + t_rem + t_host;
  auto share = [&](float t, uint32_t c, int cap) -> int {
    if (c == 0) return 0;
    int n = t_all > 0.f ? (int)ceilf((float)grid * t / t_all) : cap;
    n = min(n, min(cap, ceil_div_i(c, rmin)));
    return max(n, 1);
  };
  n_host = share(t_host, cnt[kGroupHost], p.host_cta_cap);
  n_remote = share(t_rem, cnt[kGroupRemote], p.remote_cta_cap);
  if (p.fixed_split) {
    n_host = cnt[kGroupHost] ? max(p.host_cta_cap, 1) : 0;
    n_remote = cnt[kGroupRemote] ? max(p.remote_cta_cap, 1) : 0;
  }
  const int avail = grid - (cnt[kGroupLocal] ? 1 : 0);
  while (n_host + n_remote > avail) {  // small grids only
    if (n_remote >= n_host && n_remote > 1) {
      n_remote--;
    } else if (n_host > 1) {
      n_host--;
    } else {
      n_remote--;
    }
  }
  if (cnt[kGroupLocal] == 0) {  // nothing local: the spare CTAs help the other groups
    if (cnt[kGroupRemote]) {
      n_remote = grid - n_host;
    } else if (cnt[kGroupHost]) {
      n_host = grid;
    }
  }
}

// ---- bulk-async (TMA engine) staging of rows whose source is far away -------------------
// One elected lane per warp moves whole rows: cp.async.bulk global -> shared with an mbarrier
// counting the bytes, then cp.async.bulk shared -> global.  The copy engine keeps many rows
// in flight without holding registers or load-queue slots of the SM.  No cluster, no
// multicast; source may be pinned host memory or a peer GPU's memory.
constexpr int kBulkSlots = 8;          // rows in flight per warp
constexpr uint32_t kBulkSpinLimit = 1u << 22;

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return (uint32_t)__cvta_generic_to_shared(p);
}
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}
__device__ __forceinline__ void bulk_g2s(uint32_t dst_smem, const void* src, uint32_t bytes,
                                         uint32_t bar) {
  asm volatile(
      "cp.async.bulk.shared::cta.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
          dst_smem),
      "l"(src), "r"(bytes), "r"(bar)
      : "memory");
}
__device__ __forceinline__ void bulk_s2g(void* dst, uint32_t src_smem, uint32_t bytes) {
  asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(dst),
               "r"(src_smem), "r"(bytes)
               : "memory");
}

// Rows [worker, worker + n_workers, ...) of the list, one warp per worker, lane 0 drives.
// Returns false if a wait ran out (the caller records it; the kernel still terminates).
__device__ __forceinline__ bool copy_rows_bulk(const RecordIndex& ix, uint32_t count,
                                               uint32_t worker, uint32_t n_workers,
                                               unsigned char* stage, uint64_t* bars) {
  const uint32_t lane = threadIdx.x & 31;
  bool ok_all = true;
  if (lane == 0) {
    uint32_t parity = 0;
    for (int u = 0; u < kBulkSlots; u++) mbar_init(smem_u32(&bars[u]), 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    for (uint32_t base = worker; base < count; base += n_workers * kBulkSlots) {
      char* dst[kBulkSlots];
      bool ok[kBulkSlots];
#pragma unroll
      for (int u = 0; u < kBulkSlots; u++) {
        uint32_t i = base + u * n_workers;
        ok[u] = i < count;
        dst[u] = nullptr;
        if (ok[u]) {
          const char* src;
          ix.get(i, src, dst[u]);
          uint32_t bar = smem_u32(&bars[u]);
          mbar_expect_tx(bar, ix.row_bytes);
          bulk_g2s(smem_u32(stage + (size_t)u * ix.row_bytes), src, ix.row_bytes, bar);
        }
      }
#pragma unroll
      for (int u = 0; u < kBulkSlots; u++) {
        if (!ok[u]) continue;
        uint32_t bar = smem_u32(&bars[u]);
        uint32_t spins = 0;
        while (!mbar_try_wait(bar, parity)) {
          if (++spins > kBulkSpinLimit) {
            ok_all = false;
            break;
          }
        }
        if (!ok_all) break;
        bulk_s2g(dst[u], smem_u32(stage + (size_t)u * ix.row_bytes), ix.row_bytes);
      }
      asm volatile("cp.async.bulk.commit_group;" ::: "memory");
      // the slots are reused by the next pass: wait until the stores have read them
      asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
      if (!ok_all) break;
      parity ^= 1;
    }
    asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
  }
  __syncwarp();
  return ok_all;
}

// Counts of the lookup that just finished, into the pinned host mirror (plain stores that
// cross PCIe; the sequence number goes last).
__device__ __forceinline__ void publish_feedback(Feedback* f, uint32_t n_keys,
                                                 const uint32_t cnt[kNumGroup], uint32_t seq) {
  if (f == nullptr) return;
  volatile Feedback* vf = f;
  vf->keys = n_keys;
#pragma unroll
  for (int g = 0; g < kNumGroup; g++) vf->count[g] = cnt[g];
  __threadfence_system();
  vf->seq = seq;
}

template <int VEC, int LPR, int UNROLL>
__global__ void __launch_bounds__(1024) gather_roles_kernel(GatherParams p) {
  extern __shared__ __align__(128) unsigned char dyn_smem[];
  const int grid = (int)gridDim.x;
  const int b = (int)blockIdx.x;
  // The lookup kernel ahead of this one in the stream must have finished writing the lists.
  asm volatile("griddepcontrol.wait;" ::: "memory");
  // The next lookup's key loads and table probes may start while this grid drains.
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  unsigned long long t0 = 0;
  if (threadIdx.x == 0) asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t0));
  uint32_t cnt[kNumGroup];
#pragma unroll
  for (int g = 0; g < kNumGroup; g++) cnt[g] = p.counters->count[g];

  int n_host, n_remote;
  split_roles(p, cnt, grid, n_host, n_remote);

  const uint32_t vecs_per_row = p.row_bytes / VEC;
  const uint32_t workers_per_cta = blockDim.x / LPR;
  const uint32_t worker_in_cta = threadIdx.x / LPR;
  const uint32_t sublane = threadIdx.x % LPR;

  int g, first, num;
  if (b < n_host) {
    g = kGroupHost;
    first = 0;
    num = n_host;
  } else if (b < n_host + n_remote) {
    g = kGroupRemote;
    first = n_host;
    num = n_remote;
  } else {
    g = kGroupLocal;
    first = n_host + n_remote;
    num = grid - first;
  }
  RecordIndex ix;
  ix.src_base = p.src_base;
  ix.out = static_cast<char*>(p.out);
  ix.row_bytes = p.row_bytes;
  // rows [lo, lo + len) of list `gg`, shared among `n_ctas` CTAs of which this one is `cta`
  auto copy_span = [&](int gg, uint32_t lo, uint32_t len, uint32_t cta, uint32_t n_ctas) {
    ix.list = (gg == kGroupLocal ? p.list[kGroupLocal]
                                 : (gg == kGroupRemote ? p.list[kGroupRemote] : p.list[kGroupHost])) + lo;
    if (VEC == 32 && gg == kGroupHost) {
      // host rows always move as 16-byte vectors, 4 rows in flight per lane group: 32-byte
      // loads from pinned host memory were slower on every machine measured
      constexpr int kHostLpr = LPR * 2 > 32 ? 32 : LPR * 2;
      const uint32_t wpc = blockDim.x / kHostLpr;
      copy_rows<16, kHostLpr, 4, true>(ix, len, cta * wpc + threadIdx.x / kHostLpr, n_ctas * wpc,
                                       threadIdx.x % kHostLpr, p.row_bytes / 16);
    } else {
      copy_rows<VEC, LPR, UNROLL, true>(ix, len, cta * workers_per_cta + worker_in_cta,
                                        n_ctas * workers_per_cta, sublane, vecs_per_row);
    }
  };
  if (!p.dynamic || p.bulk_mask != 0) {
    // fixed striding: every CTA of a group takes rows b-first, b-first+num, ... of its list
    if (cnt[g] != 0) {
      const bool bulk = (g == kGroupHost && (p.bulk_mask & 1)) || (g == kGroupRemote && (p.bulk_mask & 2));
      if (bulk) {
        ix.list = p.list[g];
        const uint32_t warps_per_cta = blockDim.x >> 5;
        const uint32_t warp = threadIdx.x >> 5;
        uint64_t* bars = reinterpret_cast<uint64_t*>(dyn_smem) + (size_t)warp * kBulkSlots;
        unsigned char* stage = dyn_smem + (size_t)warps_per_cta * kBulkSlots * sizeof(uint64_t) +
                               (size_t)warp * kBulkSlots * p.row_bytes;
        bool ok = copy_rows_bulk(ix, cnt[g], (uint32_t)(b - first) * warps_per_cta + warp,
                                 (uint32_t)num * warps_per_cta, stage, bars);
        if (!ok && (threadIdx.x & 31) == 0) atomicAdd(&p.counters->err_table, 1ull);
      } else {
        copy_span(g, 0, cnt[g], (uint32_t)(b - first), (uint32_t)num);
      }
    }
  } else {
    // Chunked hand-out.  Chunk i < (CTAs of the group) of a list belongs to the group's i-th
    // CTA without any atomic; further chunks come from the list's cursor, fetched one chunk
    // ahead so that the atomic's latency overlaps the copy.  A CTA that finds its own list
    // drained moves on to the other lists (far sources first), so no CTA idles while rows
    // are left anywhere.
    __shared__ uint32_t s_next;
    const uint32_t chunk = workers_per_cta * UNROLL * 2;
    const int o1 = g == kGroupRemote ? kGroupHost : kGroupRemote;
    const int o2 = g == kGroupLocal ? kGroupHost : kGroupLocal;
#pragma unroll
    for (int k = 0; k < kNumGroup; k++) {
      const int gg = k == 0 ? g : (k == 1 ? o1 : o2);
      const uint32_t total =
          gg == kGroupLocal ? cnt[kGroupLocal] : (gg == kGroupRemote ? cnt[kGroupRemote] : cnt[kGroupHost]);
      if (total == 0) continue;
      const int ctas_gg = gg == kGroupLocal ? grid - n_host - n_remote : (gg == kGroupRemote ? n_remote : n_host);
      const uint32_t owned = (uint32_t)ctas_gg * chunk;  // rows covered by the first chunks
      if (k > 0 && owned >= total) continue;             // nothing beyond them to take
      uint32_t* cursor = &p.counters->cursor[0] + gg;
      uint32_t base, fetched = 0;
      if (k == 0) {
        base = (uint32_t)(b - first) * chunk;
        if (threadIdx.x == 0 && owned < total) fetched = atomicAdd(cursor, chunk);
      } else {
        if (threadIdx.x == 0) s_next = atomicAdd(cursor, chunk);
        __syncthreads();
        base = owned + s_next;
        __syncthreads();
        if (threadIdx.x == 0 && base < total) fetched = atomicAdd(cursor, chunk);
      }
      bool did = false;
      while (base < total) {
        copy_span(gg, base, min(chunk, total - base), 0u, 1u);
        did = true;
        if (threadIdx.x == 0) s_next = fetched;
        __syncthreads();
        base = owned + s_next;
        __syncthreads();
        if (threadIdx.x == 0 && base < total) fetched = atomicAdd(cursor, chunk);
      }
      if (did && k > 0 && threadIdx.x == 0) {  // finish time of a group this CTA helped
        unsigned long long th;
        asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(th));
        atomicMax(&p.counters->t_end[0] + gg, th);
      }
    }
  }

  // The last CTA to finish publishes the counts of this lookup and re-arms the counters.
  __syncthreads();
  if (threadIdx.x == 0) {
    // when each source group was done, for ugc_stats (one atomic per CTA)
    unsigned long long t1;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t1));
    if (b == 0) p.counters->t_start = t0;
    if (cnt[g] != 0) atomicMax(&p.counters->t_end[g], t1);
    __threadfence();
    uint32_t done = atomicAdd(&p.counters->done_ctas, 1u);
    if (done == (uint32_t)grid - 1) {
#pragma unroll
      for (int g2 = 0; g2 < kNumGroup; g2++) {
        p.counters->last_count[g2] = cnt[g2];
        p.counters->count[g2] = 0;
      }
      p.counters->last_keys = p.n_keys;
      p.counters->done_ctas = 0;
#pragma unroll
      for (int g2 = 0; g2 < kNumGroup; g2++) p.counters->cursor[g2] = 0;
      publish_feedback(p.feedback, p.n_keys, cnt, p.seq);
      __threadfence();
    }
  }
}

// ------------------------------------------------------------------------------------
// distinct keys of a batch
// ------------------------------------------------------------------------------------
// One 32-bit stamp per id of the key space: {epoch : 8 | index : 24}.  A key is new in this
// batch when its stamp carries another epoch; the thread that swings the stamp to the current
// epoch takes the next index and records the key.  A second pass reads the index of every key
// (the owner may not have stored it yet when another thread of the first pass looks).  No sort,
// no hashing: the key space is dense and its table already costs 4 bytes per id.
constexpr uint32_t kStampPending = 0x00ffffffu;

template <typename KeyT>
__global__ void __launch_bounds__(kBlock)
    unique_claim_kernel(const KeyT* __restrict__ keys, uint32_t n, uint64_t num_keys, uint32_t epoch,
                        uint32_t* stamp, KeyT* __restrict__ unique_keys, uint32_t* n_unique,
                        Counters* counters) {
  const uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
  const uint32_t lane = threadIdx.x & 31;
  bool winner = false;
  uint64_t k = 0;
  if (i < n) {
    k = (uint64_t)keys[i];
    if (k >= num_keys) {
      atomicAdd(&counters->err_key_range, 1ull);
    } else {
      const uint32_t mine = (epoch << 24) | kStampPending;
      uint32_t cur = *reinterpret_cast<volatile uint32_t*>(stamp + k);
      while ((cur >> 24) != epoch) {
        const uint32_t old = atomicCAS(stamp + k, cur, mine);
        if (old == cur) {
          winner = true;
          break;
        }
        cur = old;
      }
    }
  }
  // one atomic per warp for the indices of its winners
  const unsigned m = __ballot_sync(kFull, winner);
  uint32_t base = 0;
  if (m != 0 && lane == (uint32_t)(__ffs(m) - 1)) base = atomicAdd(n_unique, (uint32_t)__popc(m));
  base = __shfl_sync(kFull, base, m ? __ffs(m) - 1 : 0);
  if (winner) {
    const uint32_t idx = base + __popc(m & ((1u << lane) - 1));
    unique_keys[idx] = (KeyT)k;
    atomicExch(stamp + k, (epoch << 24) | idx);
  }
}

template <typename KeyT>
__global__ void __launch_bounds__(kBlock)
    unique_inverse_kernel(const KeyT* __restrict__ keys, uint32_t n, uint64_t num_keys,
                          const uint32_t* __restrict__ stamp, int32_t* __restrict__ inverse) {
  const uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const uint64_t k = (uint64_t)keys[i];
  inverse[i] = k < num_keys ? (int32_t)(stamp[k] & kStampPending) : -1;
}

// ------------------------------------------------------------------------------------
// host list in address order
// ------------------------------------------------------------------------------------
// Scattered rows of pinned host memory arrive about 15 % faster when the reads in flight move
// through the table in ascending address order (63-68 M against 55-60 M rows per second,
// measured with nothing else running), which is what the reference gets from sorting its
// whole index (coll_cache_lib/cache_context.cu:702-761).  Here only the host list is ordered,
// and only coarsely: a counting sort into kHostBuckets address ranges.  Two small kernels
// between the lookup and the gather; `hist` holds kHostBuckets counts followed by
// kHostBuckets cursors, all zero on entry.
constexpr int kHostBuckets = 256;

__device__ __forceinline__ uint32_t host_bucket(uint64_t rec, uint32_t shift) {
  const uint32_t b = rec_off(rec) >> shift;
  return b < (uint32_t)kHostBuckets ? b : (uint32_t)kHostBuckets - 1;
}

__global__ void __launch_bounds__(kBlock)
    host_hist_kernel(const uint64_t* __restrict__ list, const Counters* counters, uint32_t* hist,
                     uint32_t shift) {
  __shared__ uint32_t s_hist[kHostBuckets];
  for (int i = threadIdx.x; i < kHostBuckets; i += kBlock) s_hist[i] = 0;
  __syncthreads();
  const uint32_t n = counters->count[kGroupHost];
  for (uint32_t i = blockIdx.x * kBlock + threadIdx.x; i < n; i += gridDim.x * kBlock)
    atomicAdd(&s_hist[host_bucket(list[i], shift)], 1u);
  __syncthreads();
  for (int i = threadIdx.x; i < kHostBuckets; i += kBlock)
    if (s_hist[i]) atomicAdd(&hist[i], s_hist[i]);
}

__global__ void __launch_bounds__(kBlock)
    host_scatter_kernel(const uint64_t* __restrict__ list, uint64_t* __restrict__ sorted,
                        const Counters* counters, uint32_t* hist, uint32_t shift) {
  __shared__ uint32_t s_start[kHostBuckets];
  if (threadIdx.x == 0) {  // exclusive prefix of the bucket counts (256 adds, same in every CTA)
    uint32_t run = 0;
    for (int i = 0; i < kHostBuckets; i++) {
      s_start[i] = run;
      run += hist[i];
    }
  }
  __syncthreads();
  uint32_t* cursor = hist + kHostBuckets;
  const uint32_t n = counters->count[kGroupHost];
  for (uint32_t i = blockIdx.x * kBlock + threadIdx.x; i < n; i += gridDim.x * kBlock) {
    const uint64_t rec = list[i];
    const uint32_t b = host_bucket(rec, shift);
    sorted[s_start[b] + atomicAdd(&cursor[b], 1u)] = rec;
  }
}

// ------------------------------------------------------------------------------------
// direct extraction: table probe and row copy in ONE kernel, no index lists
// ------------------------------------------------------------------------------------
// A warp owns tiles of 32 (or 16, or 8) consecutive keys -- the launcher picks the largest
// size that leaves every warp nearly the same number of tiles; with 32-key tiles a batch of
// 212,992 keys is 1.4 tiles per warp, so 40 % of the warps would carry twice the work of the
// rest.  Lane l probes the table for key l of the tile;
// the row addresses then travel by shuffle to the lane groups that copy the rows, so the
// destination of a tile is one contiguous piece of the output.  Rows of every source (local
// slice, peer slice over NVLink, pinned host memory) are copied where they come up, which
// spreads the few far rows of a batch evenly over the SMs and over the kernel's duration.
// Keys are loaded two tiles ahead and probed one tile ahead of the tile being copied.
// Tiles are dealt to warps so that consecutive tiles land on different CTAs: every SM gets
// the same number of rows to within one tile.
//
// This is the counterpart of the reference's ungrouped extraction (one extract_data over
// DataIterMixLoc, coll_cache_lib/cache_context.cu:1295-1329, :137-159) with the table
// lookup folded in; the grouped path above stays the better shape when many rows of a batch
// come from the host.
struct Probe {  // a table read in flight: one 4-slot line (probing table) or one word (flat)
  uint32_t k0, k1, k2, k3, w0, w1, w2, w3;
};

__device__ __forceinline__ void probe_issue(const TableView& t, uint32_t key, bool valid, Probe& pr) {
  pr.k0 = pr.k1 = pr.k2 = pr.k3 = kEmptyWord;
  pr.w0 = pr.w1 = pr.w2 = pr.w3 = kEmptyWord;
  if (valid) {
    if (t.kind == kTableFlat) {
      asm volatile("ld.global.cg.b32 %0, [%1];" : "=r"(pr.w0) : "l"(t.flat + key));
    } else {
      const uint2* a = t.slots + (size_t)(murmur3_32(key) & t.line_mask) * kSlotsPerLine;
      asm volatile("ld.global.cg.v8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
                   : "=r"(pr.k0), "=r"(pr.w0), "=r"(pr.k1), "=r"(pr.w1), "=r"(pr.k2), "=r"(pr.w2),
                     "=r"(pr.k3), "=r"(pr.w3)
                   : "l"(a));
    }
  }
}

__device__ __forceinline__ uint32_t probe_resolve(const TableView& t, const Probe& pr, uint32_t key,
                                                  bool valid) {
  if (!valid || t.kind == kTableFlat) return pr.w0;
  if (pr.k0 == key) return pr.w0;  // live slots carry the key with the top bit clear
  if (pr.k1 == key) return pr.w1;
  if (pr.k2 == key) return pr.w2;
  if (pr.k3 == key) return pr.w3;
  if (pr.k0 == kEmptyWord || pr.k1 == kEmptyWord || pr.k2 == kEmptyWord || pr.k3 == kEmptyWord)
    return kEmptyWord;  // a never-used slot ends the search
  return probe_rest(t.slots, t.line_mask, key, murmur3_32(key) & t.line_mask);
}

// Key `lane` of tile `tl` (tiles of 1 << shift keys; lanes beyond the tile hold no key); ids
// outside [0, num_keys) are counted and dropped.
template <typename KeyT>
__device__ __forceinline__ void fetch_key(const KeyT* __restrict__ keys, uint32_t tl, uint32_t n_tiles,
                                          uint32_t shift, uint32_t n_keys, uint64_t num_keys,
                                          uint32_t lane, uint32_t& key, bool& valid, uint32_t& bad) {
  const uint32_t idx = (tl << shift) + lane;
  valid = tl < n_tiles && (lane >> shift) == 0 && idx < n_keys;
  uint64_t k = valid ? (uint64_t)keys[idx] : 0;
  if (k >= num_keys) {  // also catches negative int64 ids
    valid = false;
    bad++;
    k = 0;
  }
  key = (uint32_t)k;
}

template <typename KeyT, int VEC, bool DEEP, bool EARLY>
__global__ void __launch_bounds__(kBlock, DEEP ? 3 : 4)
    extract_direct_kernel(const KeyT* __restrict__ keys, DirectParams p) {
  // rows in flight per lane group: 4 (2 with 32-byte vectors) at 4 CTAs per SM, or twice that
  // at 3 CTAs per SM
  constexpr int UNROLL = (VEC == 32 ? 2 : 4) * (DEEP ? 2 : 1);
  __shared__ uint32_t s_cnt[kNumGroup];
  __shared__ const char* s_src[kMaxLocation];
  if (threadIdx.x == 0) {
#pragma unroll
    for (int i = 0; i < kMaxLocation; i++) s_src[i] = static_cast<const char*>(p.src_base[i]);
  }
  const uint32_t lane = threadIdx.x & 31;
  const uint32_t n_warps = gridDim.x * (blockDim.x >> 5);
  const uint32_t tshift = p.tile_shift;
  const uint32_t tile_keys = 1u << tshift;
  // the number of keys may live in device memory (distinct keys of a batch, counted on the GPU)
  const uint32_t n_keys = p.n_dev ? min(*p.n_dev, p.n_keys) : p.n_keys;
  const uint32_t n_tiles = (n_keys + tile_keys - 1) >> tshift;
  uint32_t tile = (threadIdx.x >> 5) * gridDim.x + blockIdx.x;
  if (threadIdx.x < kNumGroup) s_cnt[threadIdx.x] = 0;

  unsigned long long t0 = 0;
  if ((threadIdx.x & 31) == 0) asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t0));

  uint32_t bad = 0;

  // Keys and table are not written by the extraction ahead of this one in the stream: the
  // first two key loads and the first probe run before the dependency wait.
  uint32_t key_cur, key_nxt;
  bool ok_cur, ok_nxt;
  fetch_key(keys, tile, n_tiles, tshift, n_keys, p.table.num_keys, lane, key_cur, ok_cur, bad);
  fetch_key(keys, tile + n_warps, n_tiles, tshift, n_keys, p.table.num_keys, lane, key_nxt, ok_nxt, bad);
  Probe pr;
  probe_issue(p.table, key_cur, ok_cur, pr);
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  uint32_t word = probe_resolve(p.table, pr, key_cur, ok_cur);
  // EARLY: the first host row of this warp's first tile is fetched before the dependency wait
  // (the host table is never written by a lookup) and held in registers, one piece per lane.
  // CTAs of this launch become resident while the launch ahead is still waiting for ITS last
  // host rows; their requests keep the host link's queue filled across the boundary between
  // two launches, where it would otherwise run empty and fill up again.
  Vec<VEC> early;
  uint32_t early_lane = 32;  // lane whose key the held row belongs to; 32 = none
  if (EARLY) {
    const bool is_host = ok_cur && word == kEmptyWord;
    const unsigned hmask = __ballot_sync(kFull, is_host);
    if (hmask && p.row_bytes / VEC <= 32) {
      early_lane = __ffs(hmask) - 1;
      const uint32_t k = __shfl_sync(kFull, key_cur, early_lane);
      if (lane < p.row_bytes / VEC)
        ld_row(early, static_cast<const char*>(p.host_base) + (size_t)(k & p.host_mask) * p.row_bytes +
                          (size_t)lane * VEC);
    }
  }
  asm volatile("griddepcontrol.wait;" ::: "memory");
  if (EARLY && early_lane < 32) {
    if (lane < p.row_bytes / VEC)
      st_row(static_cast<char*>(p.out) + (((size_t)tile << tshift) + early_lane) * p.row_bytes + (size_t)lane * VEC,
             early);
  }
  // The extraction ahead of this one is complete now.  One thread hands ITS counts on (they
  // sit in the other slot, final) -- to the pinned host mirror the library reads to choose
  // the mode of later lookups -- and clears that slot for the launch after this one.
  // (the thread chosen for this belongs to the warp that is dealt the fewest tiles -- the last
  // warp of the last CTA -- so that the writes across PCIe delay no warp the launch waits for)
  if (blockIdx.x == gridDim.x - 1 && threadIdx.x == blockDim.x - 32) {
    uint32_t* other = p.counters->dcount[p.slot ^ 1u];
    uint32_t prev[kNumGroup];
#pragma unroll
    for (int g = 0; g < kNumGroup; g++) prev[g] = other[g];
    if (p.publish_prev) publish_feedback(p.feedback, p.prev_keys, prev, p.prev_seq);
#pragma unroll
    for (int g = 0; g < kNumGroup; g++) other[g] = 0;
    p.counters->t_start = t0;
    p.counters->t_index = 0;
    p.counters->last_keys = p.n_keys;
  }

  const uint32_t lpr = 1u << p.lpr_shift;
  const uint32_t rpi = 32u >> p.lpr_shift;       // rows per warp-wide load
  const uint32_t sub = lane & (lpr - 1);
  const uint32_t rsel = lane >> p.lpr_shift;
  const uint32_t vecs_per_row = p.row_bytes / VEC;
  uint32_t n_local = 0, n_remote = 0, n_host = 0;
  __syncthreads();  // s_src, s_cnt

  while (tile < n_tiles) {
    // next tile's probe and the key load two tiles ahead go out before this tile's rows
    probe_issue(p.table, key_nxt, ok_nxt, pr);
    uint32_t key_nn;
    bool ok_nn;
    fetch_key(keys, tile + 2 * n_warps, n_tiles, tshift, n_keys, p.table.num_keys, lane, key_nn, ok_nn, bad);

    // this lane's key: source address and group
    const char* src = nullptr;
    uint32_t group = kNumGroup;
    if (ok_cur) {
      uint32_t loc, off;
      if (word == kEmptyWord) {
        loc = p.host_loc;
        off = key_cur & p.host_mask;
        group = kGroupHost;
      } else {
        loc = word_loc(word);
        off = word_off(word);
        group = loc == p.local_loc ? kGroupLocal : kGroupRemote;
      }
      src = s_src[loc] + (size_t)off * p.row_bytes;
    }
    if (EARLY && lane == early_lane) src = nullptr;  // copied already (still counted below)
    early_lane = 32;
    n_local += __popc(__ballot_sync(kFull, group == (uint32_t)kGroupLocal));
    n_remote += __popc(__ballot_sync(kFull, group == (uint32_t)kGroupRemote));
    n_host += __popc(__ballot_sync(kFull, group == (uint32_t)kGroupHost));

    char* out_tile = static_cast<char*>(p.out) + ((size_t)tile << tshift) * p.row_bytes;
    const unsigned long long src_bits = reinterpret_cast<unsigned long long>(src);
    const size_t row_step = (size_t)rpi * p.row_bytes;  // between the rows of one lane group
    for (uint32_t rb = 0; rb < tile_keys; rb += UNROLL * rpi) {
      const char* s[UNROLL];
#pragma unroll
      for (int u = 0; u < UNROLL; u++) {
        const uint32_t r = rb + u * rpi + rsel;
        const unsigned long long a = __shfl_sync(kFull, src_bits, r & 31);
        s[u] = r < tile_keys ? reinterpret_cast<const char*>(a) : nullptr;
      }
      char* d0 = out_tile + (size_t)(rb + rsel) * p.row_bytes;
      for (uint32_t c = sub; c < vecs_per_row; c += lpr) {
        Vec<VEC> v[UNROLL];
#pragma unroll
        for (int u = 0; u < UNROLL; u++)
          if (s[u]) ld_row(v[u], s[u] + (size_t)c * VEC);
#pragma unroll
        for (int u = 0; u < UNROLL; u++)
          if (s[u]) st_row(d0 + u * row_step + (size_t)c * VEC, v[u]);
      }
    }

    word = probe_resolve(p.table, pr, key_nxt, ok_nxt);
    key_cur = key_nxt;
    ok_cur = ok_nxt;
    key_nxt = key_nn;
    ok_nxt = ok_nn;
    tile += n_warps;
  }

  // Per-source counts of this lookup: fire-and-forget adds into the slot this launch owns.
  // Nothing here waits on memory, so the kernel ends with its last row store: no count of
  // finished CTAs, no fence, no single CTA that tidies up after the others.
  if (bad) atomicAdd(&p.counters->err_key_range, (unsigned long long)bad);
  if (lane == 0) {
    if (n_local) atomicAdd(&s_cnt[kGroupLocal], n_local);
    if (n_remote) atomicAdd(&s_cnt[kGroupRemote], n_remote);
    if (n_host) atomicAdd(&s_cnt[kGroupHost], n_host);
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    uint32_t* mine = p.counters->dcount[p.slot];
#pragma unroll
    for (int g = 0; g < kNumGroup; g++)
      if (s_cnt[g]) atomicAdd(mine + g, s_cnt[g]);
    unsigned long long t1;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t1));
    atomicMax(&p.counters->t_end[kGroupLocal], t1);  // one span for the whole kernel
  }
}

// ------------------------------------------------------------------------------------
// pooled lookup: table probe, row fetch and per-bag sum in ONE kernel
// ------------------------------------------------------------------------------------
// A bag is a run of consecutive keys; its result is the sum (or mean) of its rows, one fp32
// vector of `dim` elements.  The looked-up rows never reach memory: a group of lanes (as many
// as a row has 16-byte pieces, at most 32) owns a bag, each lane probes the table for one key of
// the bag, the row addresses travel by shuffle inside the group, and every lane adds up its
// own 16-byte column of the rows.  The additions of one output element happen in key order,
// in fp32, starting from +0, one rounding each (no fused multiply-add is involved), so the
// result is bit-for-bit what a sequential fp32 loop over the bag gives on any machine.
// Keys outside [0, num_keys) are counted and contribute nothing.  The reference leaves pooling
// to the model that consumes the rows; this is the fused form of lookup + segment sum.
template <bool F16, int VEC>
__device__ __forceinline__ void pool_add(float* acc, const Vec<VEC>& v) {
  if (F16) {
    const __half2* h = reinterpret_cast<const __half2*>(&v);
#pragma unroll
    for (int i = 0; i < VEC / 4; i++) {
      const float2 f = __half22float2(h[i]);
      acc[2 * i] = __fadd_rn(acc[2 * i], f.x);
      acc[2 * i + 1] = __fadd_rn(acc[2 * i + 1], f.y);
    }
  } else {
    const float* f = reinterpret_cast<const float*>(&v);
#pragma unroll
    for (int i = 0; i < VEC / 4; i++) acc[i] = __fadd_rn(acc[i], f[i]);
  }
}

// Position in `keys` where bag b starts (b == n_bags: where the last one ends), inside [0, n_keys].
__device__ __forceinline__ uint32_t pool_bag_start(const PoolParams& p, uint32_t b) {
  const long long o = p.offsets ? p.offsets[b] : (long long)b * p.bag_size;
  return (uint32_t)min(max(o, 0ll), (long long)p.n_keys);
}

template <typename KeyT, bool F16, int VEC>
__global__ void __launch_bounds__(kBlock, 3) lookup_pool_kernel(const KeyT* __restrict__ keys, PoolParams p) {
  constexpr int NF = VEC / (F16 ? 2 : 4);  // elements per piece of a row (VEC bytes)
  constexpr int UNROLL = VEC == 16 ? 8 : 16;  // rows in flight per lane
  __shared__ const char* s_src[kMaxLocation];
  if (threadIdx.x < kMaxLocation) s_src[threadIdx.x] = static_cast<const char*>(p.src_base[threadIdx.x]);
  __syncthreads();
  const uint32_t lane = threadIdx.x & 31;
  const uint32_t lpr = 1u << p.lpr_shift;
  const uint32_t sub = lane & (lpr - 1);
  const uint32_t gbase = lane & ~(lpr - 1);
  const unsigned gmask = lpr == 32 ? kFull : (((1u << lpr) - 1u) << gbase);
  const uint32_t workers_per_cta = blockDim.x >> p.lpr_shift;
  const uint32_t n_workers = gridDim.x * workers_per_cta;
  const uint32_t vecs = p.row_bytes / VEC;
  const uint32_t n_tiles = (p.n_bags + p.bags_per_tile - 1) / p.bags_per_tile;
  // rows wider than one lane group (32 pieces) are cut into column passes; a pass over a tile
  // is the unit of work, so that wide rows (or, with 4-byte pieces, every row) spread a bag
  // over several lane groups
  const uint32_t n_pass = (vecs + lpr - 1) >> p.lpr_shift;
  const uint32_t n_items = n_tiles * n_pass;
  uint32_t bad = 0, n_local = 0, n_remote = 0, n_host = 0;

  // A lane group owns a tile of consecutive bags (several when bags are shorter than the group
  // is wide, so that every lane has a key to probe) and walks the tile's keys in order: probe
  // `lpr` keys, fetch their rows UNROLL at a time, add them up in key order, and write a bag out
  // whenever the walk crosses into the next one.
  for (uint32_t item = blockIdx.x * workers_per_cta + (threadIdx.x >> p.lpr_shift); item < n_items;
       item += n_workers) {
    const uint32_t tile = item / n_pass;
    const uint32_t c0 = (item - tile * n_pass) << p.lpr_shift;
    const uint32_t bag_lo = tile * p.bags_per_tile;
    const uint32_t bag_hi = min(bag_lo + p.bags_per_tile, p.n_bags);
    const uint32_t k_lo = pool_bag_start(p, bag_lo);
    const uint32_t k_hi = max(k_lo, pool_bag_start(p, bag_hi));
    {
      const uint32_t c = c0 + sub;
      const bool has = c < vecs;
      float acc[NF];
#pragma unroll
      for (int i = 0; i < NF; i++) acc[i] = 0.f;
      uint32_t bag = bag_lo;
      uint32_t bag_begin = k_lo;
      uint32_t bag_end = max(bag_begin, min(pool_bag_start(p, bag + 1), k_hi));
      // writes bag `bag` out and moves on to the next one of the tile
      auto flush = [&]() {
        if (has) {
          const uint32_t len = bag_end - bag_begin;
          if (p.mean && len > 0) {
            const float d = (float)len;
#pragma unroll
            for (int i = 0; i < NF; i++) acc[i] = __fdiv_rn(acc[i], d);
          }
          float* dst = p.out + (size_t)bag * p.dim + (size_t)c * NF;
          if (NF >= 4) {
#pragma unroll
            for (int i = 0; i + 3 < NF; i += 4)
              reinterpret_cast<float4*>(dst)[i / 4] = make_float4(acc[i], acc[i + 1], acc[i + 2], acc[i + 3]);
          } else if (NF == 2) {
            *reinterpret_cast<float2*>(dst) = make_float2(acc[0], acc[NF - 1]);
          } else {
            dst[0] = acc[0];
          }
        }
#pragma unroll
        for (int i = 0; i < NF; i++) acc[i] = 0.f;
        bag++;
        bag_begin = bag_end;
        if (bag < bag_hi) bag_end = max(bag_begin, min(pool_bag_start(p, bag + 1), k_hi));
      };
      for (uint32_t k0 = k_lo; k0 < k_hi; k0 += lpr) {
        // this lane's key: source address of its row
        const uint32_t idx = k0 + sub;
        bool valid = idx < k_hi;
        unsigned long long k = valid ? (unsigned long long)keys[idx] : 0ull;
        if (k >= p.table.num_keys) {  // also catches negative int64 ids
          if (valid && c0 == 0) bad++;
          valid = false;
        }
        const char* src = nullptr;
        if (valid) {
          const uint32_t w = table_lookup(p.table, (uint32_t)k);
          uint32_t loc, off;
          if (w == kEmptyWord) {
            loc = p.host_loc;
            off = (uint32_t)k & p.host_mask;
            if (c0 == 0) n_host++;
          } else {
            loc = word_loc(w);
            off = word_off(w);
            if (c0 == 0) {
              if (loc == p.local_loc) {
                n_local++;
              } else {
                n_remote++;
              }
            }
          }
          src = s_src[loc] + (size_t)off * p.row_bytes;
        }
        const unsigned long long src_bits = reinterpret_cast<unsigned long long>(src);
        const uint32_t cnt = min(lpr, k_hi - k0);
        for (uint32_t j = 0; j < cnt; j += UNROLL) {
          Vec<VEC> v[UNROLL];
          bool ok[UNROLL];
#pragma unroll
          for (int u = 0; u < UNROLL; u++) {
            const unsigned long long a = __shfl_sync(gmask, src_bits, gbase + ((j + u) & (lpr - 1)));
            ok[u] = has && j + u < cnt && a != 0ull;
            if (ok[u]) ld_row(v[u], reinterpret_cast<const char*>(a) + (size_t)c * VEC);
          }
#pragma unroll
          for (int u = 0; u < UNROLL; u++) {
            if (j + u < cnt) {
              while (k0 + j + u >= bag_end && bag < bag_hi) flush();  // also passes empty bags
              if (ok[u]) pool_add<F16, VEC>(acc, v[u]);
            }
          }
        }
      }
      while (bag < bag_hi) flush();  // the last bag of the tile, and empty ones after it
    }
  }
  // counts: one global atomic per CTA and counter (an atomic per thread on one address would
  // take longer than the kernel's memory traffic)
  __shared__ uint32_t s_cnt[kNumGroup + 1];
  if (threadIdx.x <= kNumGroup) s_cnt[threadIdx.x] = 0;
  __syncthreads();
  n_local = __reduce_add_sync(kFull, n_local);
  n_remote = __reduce_add_sync(kFull, n_remote);
  n_host = __reduce_add_sync(kFull, n_host);
  bad = __reduce_add_sync(kFull, bad);
  if (lane == 0) {
    if (n_local) atomicAdd(&s_cnt[kGroupLocal], n_local);
    if (n_remote) atomicAdd(&s_cnt[kGroupRemote], n_remote);
    if (n_host) atomicAdd(&s_cnt[kGroupHost], n_host);
    if (bad) atomicAdd(&s_cnt[kNumGroup], bad);
  }
  __syncthreads();
  if (threadIdx.x < kNumGroup && s_cnt[threadIdx.x])
    atomicAdd(&p.counters->pool_rows[threadIdx.x], (unsigned long long)s_cnt[threadIdx.x]);
  if (threadIdx.x == kNumGroup && s_cnt[kNumGroup])
    atomicAdd(&p.counters->err_key_range, (unsigned long long)s_cnt[kNumGroup]);
}

template <int VEC, int LPR, int UNROLL>
__global__ void __launch_bounds__(kBlock) fill_scatter_kernel(KeySlotIndex ix, uint32_t n) {
  const uint32_t vecs_per_row = ix.row_bytes / VEC;
  constexpr uint32_t kWorkersPerCta = kBlock / LPR;
  const uint32_t worker = blockIdx.x * kWorkersPerCta + threadIdx.x / LPR;
  copy_rows<VEC, LPR, UNROLL, false>(ix, n, worker, gridDim.x * kWorkersPerCta, threadIdx.x % LPR,
                                     vecs_per_row);
}

// ------------------------------------------------------------------------------------
// table maintenance
// ------------------------------------------------------------------------------------
__global__ void table_clear_kernel(uint4* p, size_t n16) {
  size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  for (; i < n16; i += stride) p[i] = make_uint4(kEmptyWord, kEmptyWord, kEmptyWord, kEmptyWord);
}

// Inserts a key that is not live in the table.  A slot is free when its key has the top
// bit set (never used, or evicted).  Key and word are published by one 64-bit
// compare-and-swap, so a concurrent lookup sees the slot either free or complete.
__device__ __forceinline__ bool insert_hashed(const TableView& t, uint32_t key, uint32_t word) {
  uint32_t line = murmur3_32(key) & t.line_mask;
  for (uint32_t step = 0; step <= t.line_mask; step++) {
    Line l = ld_line(t.slots, line);
#pragma unroll
    for (int s = 0; s < kSlotsPerLine; s++) {
      if (l.key[s] == key) return false;  // already live: caller counts it as an error
      if (l.key[s] & kTombstone) {
        unsigned long long* slot =
            reinterpret_cast<unsigned long long*>(t.slots + (size_t)line * kSlotsPerLine + s);
        unsigned long long expect = ((unsigned long long)l.word[s] << 32) | l.key[s];
        unsigned long long want = ((unsigned long long)word << 32) | key;
        if (atomicCAS(slot, expect, want) == expect) return true;
        // lost the race for this slot: keep scanning (the winner holds a different key)
      }
    }
    line = (line + 1) & t.line_mask;
  }
  return false;
}

__global__ void __launch_bounds__(kBlock)
    table_insert_kernel(TableView t, const uint32_t* __restrict__ keys, SlotView offs, uint32_t loc,
                        uint32_t n, Counters* counters, bool allow_same) {
  uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  uint32_t key = keys[i];
  uint32_t word = pack_word(loc, offs.data ? offs.data[slot_pos(offs, i)] : offs.base + i);
  bool ok;
  if (key >= t.num_keys) {
    ok = false;
  } else if (t.kind == kTableFlat) {
    const uint32_t old = atomicExch(t.flat + key, word);
    ok = old == kEmptyWord || (allow_same && old == word);
  } else if (allow_same) {
    // The key may be live further along its probe sequence than the first free slot: look
    // for it before a slot is claimed, or it would end up in the table twice.
    const uint32_t w = table_lookup(t, key);
    ok = w == word || (w == kEmptyWord && insert_hashed(t, key, word));
  } else {
    ok = insert_hashed(t, key, word);
  }
  if (!ok) atomicAdd(&counters->err_table, 1ull);
}

// Refresh: every key of the list leaves its present source.  If its new source is a peer whose
// table shows the row there already, the entry's word is replaced in place by (peer, slot) --
// one 32-bit store, so a concurrent lookup sees the old or the new source, both valid until the
// grace period ends; otherwise the entry is removed (the key is served by the host until a later
// phase of the refresh inserts it again).
__global__ void __launch_bounds__(kBlock)
    table_repoint_kernel(RepointParams p, const uint32_t* __restrict__ keys, uint32_t n, Counters* counters) {
  uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const uint32_t key = keys[i];
  const TableView& t = p.own;
  bool ok = false;
  if (key < t.num_keys) {
    uint32_t word_new = kEmptyWord;
    const uint32_t src_new = p.acc_new[p.n2b_new[key]];
    if (src_new < p.num_device && src_new != p.me && p.peer[src_new].num_keys) {
      const uint32_t w = table_lookup(p.peer[src_new], key);
      if (w != kEmptyWord && word_loc(w) == src_new) word_new = w;
    }
    if (t.kind == kTableFlat) {
      ok = atomicExch(t.flat + key, word_new) != kEmptyWord;
    } else {
      uint32_t line = murmur3_32(key) & t.line_mask;
      for (uint32_t step = 0; step <= t.line_mask && !ok; step++) {
        Line l = ld_line(t.slots, line);
        bool stop = false;
#pragma unroll
        for (int s = 0; s < kSlotsPerLine; s++) {
          if (l.key[s] == key && !ok) {
            uint2* slot = &t.slots[(size_t)line * kSlotsPerLine + s];
            if (word_new == kEmptyWord) {
              atomicOr(&slot->x, kTombstone);
            } else {
              atomicExch(&slot->y, word_new);
            }
            ok = true;
          }
          stop |= (l.key[s] == kEmptyWord);
        }
        if (stop) break;
        line = (line + 1) & t.line_mask;
      }
    }
  }
  if (!ok) atomicAdd(&counters->err_table, 1ull);
}

__global__ void __launch_bounds__(kBlock)
    table_evict_kernel(TableView t, const uint32_t* __restrict__ keys, uint32_t n,
                       Counters* counters) {
  uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  uint32_t key = keys[i];
  bool ok = false;
  if (key < t.num_keys) {
    if (t.kind == kTableFlat) {
      ok = atomicExch(t.flat + key, kEmptyWord) != kEmptyWord;
    } else {
      uint32_t line = murmur3_32(key) & t.line_mask;
      for (uint32_t step = 0; step <= t.line_mask && !ok; step++) {
        Line l = ld_line(t.slots, line);
        bool stop = false;
#pragma unroll
        for (int s = 0; s < kSlotsPerLine; s++) {
          if (l.key[s] == key && !ok) {
            atomicOr(&t.slots[(size_t)line * kSlotsPerLine + s].x, kTombstone);
            ok = true;
          }
          stop |= (l.key[s] == kEmptyWord);
        }
        if (stop) break;
        line = (line + 1) & t.line_mask;
      }
    }
  }
  if (!ok) atomicAdd(&counters->err_table, 1ull);
}

__global__ void __launch_bounds__(kBlock)
    table_words_kernel(TableView t, const uint32_t* __restrict__ keys, uint32_t n,
                       uint32_t* __restrict__ words) {
  uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  uint32_t key = keys[i];
  words[i] = key < t.num_keys ? table_lookup(t, key) : kEmptyWord;
}

__global__ void __launch_bounds__(kBlock)
    table_resolve_kernel(TableView peer, const uint32_t* __restrict__ keys, uint32_t n,
                         uint32_t expect_loc, SlotView offs, Counters* counters) {
  uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  uint32_t key = keys[i];
  uint32_t w = key < peer.num_keys ? table_lookup(peer, key) : kEmptyWord;
  uint32_t* dst = offs.data + slot_pos(offs, i);
  if (w == kEmptyWord || word_loc(w) != expect_loc) {
    atomicAdd(&counters->err_table, 1ull);
    *dst = 0;
  } else {
    *dst = word_off(w);
  }
}

__global__ void iota_kernel(uint32_t* dst, uint32_t start, uint32_t n) {
  uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
  const uint32_t stride = gridDim.x * blockDim.x;
  for (; i < n; i += stride) dst[i] = start + i;
}

// ------------------------------------------------------------------------------------
// key classification over the whole id space (build and refresh), ordered compaction
// ------------------------------------------------------------------------------------
// For every key the placement gives the source that serves this reader.  Build wants one
// ascending key list per GPU source; a refresh wants the ascending lists of keys whose
// source changed (evict here, bring in here, drop a peer entry, point to a peer).  Three
// passes over tiles of kClassTile keys: per-tile counts, a scan over tiles, a stable scatter.
constexpr int kClassTile = 2048;
constexpr int kClassRounds = kClassTile / kBlock;

// Bit mask of the lists key k belongs to (see ClassifyParams in device_types.h).
__device__ __forceinline__ uint32_t class_mask(const ClassifyParams& p, uint64_t k) {
  const uint32_t src_new = p.acc_new[p.n2b_new[k]];
  if (p.n2b_old == nullptr) return src_new < p.num_device ? (1u << src_new) : 0u;  // build
  const uint32_t src_old = p.acc_old[p.n2b_old[k]];
  if (src_old == src_new) return 0u;
  uint32_t m = 0;
  if (src_old == p.me) m |= 1u << kListEvict;
  if (src_new == p.me) m |= 1u << kListInsert;
  if (src_old < p.num_device && src_old != p.me) m |= 1u << kListDropRemote;
  if (src_new < p.num_device && src_new != p.me) m |= 1u << (kListAttach0 + src_new);
  return m;
}

__global__ void __launch_bounds__(kBlock) classify_count_kernel(ClassifyParams p, uint32_t* tile_counts) {
  __shared__ uint32_t s_cnt[kMaxClassLists];
  if (threadIdx.x < kMaxClassLists) s_cnt[threadIdx.x] = 0;
  __syncthreads();
  const uint64_t base = (uint64_t)blockIdx.x * kClassTile;
  uint32_t masks[kClassRounds];
#pragma unroll
  for (int j = 0; j < kClassRounds; j++) {
    uint64_t k = base + (uint64_t)j * kBlock + threadIdx.x;
    masks[j] = k < p.num_keys ? class_mask(p, k) : 0u;
  }
  for (int l = 0; l < p.num_lists; l++) {
    uint32_t c = 0;
#pragma unroll
    for (int j = 0; j < kClassRounds; j++) c += (masks[j] >> l) & 1u;
    c = __reduce_add_sync(kFull, c);
    if ((threadIdx.x & 31) == 0 && c) atomicAdd(&s_cnt[l], c);
  }
  __syncthreads();
  if (threadIdx.x < kMaxClassLists)
    tile_counts[(size_t)threadIdx.x * gridDim.x + blockIdx.x] = s_cnt[threadIdx.x];
}

// One CTA per list: exclusive scan of that list's per-tile counts, total to totals[list].
__global__ void __launch_bounds__(1024) classify_scan_kernel(uint32_t* tile_counts, uint32_t n_tiles,
                                                             unsigned long long* totals) {
  __shared__ uint32_t s_warp[32];
  __shared__ uint32_t s_carry;
  uint32_t* row = tile_counts + (size_t)blockIdx.x * n_tiles;
  const uint32_t lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (threadIdx.x == 0) s_carry = 0;
  __syncthreads();
  unsigned long long total = 0;
  for (uint32_t start = 0; start < n_tiles; start += 1024) {
    const uint32_t i = start + threadIdx.x;
    const uint32_t v = i < n_tiles ? row[i] : 0;
    uint32_t x = v;
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
      uint32_t y = __shfl_up_sync(kFull, x, d);
      if (lane >= (uint32_t)d) x += y;
    }
    if (lane == 31) s_warp[warp] = x;
    __syncthreads();
    if (warp == 0) {
      uint32_t w = s_warp[lane];
#pragma unroll
      for (int d = 1; d < 32; d <<= 1) {
        uint32_t y = __shfl_up_sync(kFull, w, d);
        if (lane >= (uint32_t)d) w += y;
      }
      s_warp[lane] = w;  // inclusive over warps
    }
    __syncthreads();
    const uint32_t carry = s_carry;
    const uint32_t before = carry + (warp ? s_warp[warp - 1] : 0) + x - v;  // exclusive prefix
    if (i < n_tiles) row[i] = before;
    __syncthreads();
    if (threadIdx.x == 1023) {
      s_carry = carry + s_warp[31];
    }
    __syncthreads();
    total = s_carry;
  }
  // per-tile offsets are 32-bit: a list holds fewer than 2^32 keys (the id space is < 2^31)
  if (threadIdx.x == 0) totals[blockIdx.x] = total;
}

__global__ void __launch_bounds__(kBlock)
    classify_scatter_kernel(ClassifyParams p, const uint32_t* __restrict__ tile_offsets,
                            uint32_t* __restrict__ out) {
  __shared__ uint32_t s_warp_cnt[kWarpsPerBlock][kMaxClassLists];
  __shared__ uint32_t s_running[kMaxClassLists];
  const uint32_t lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (threadIdx.x < kMaxClassLists)
    s_running[threadIdx.x] = tile_offsets[(size_t)threadIdx.x * gridDim.x + blockIdx.x];
  __syncthreads();
  const uint64_t base = (uint64_t)blockIdx.x * kClassTile;
  for (int j = 0; j < kClassRounds; j++) {
    const uint64_t k = base + (uint64_t)j * kBlock + threadIdx.x;
    const uint32_t m = k < p.num_keys ? class_mask(p, k) : 0u;
    uint32_t rank[kMaxClassLists];
    for (int l = 0; l < p.num_lists; l++) {
      const unsigned b = __ballot_sync(kFull, (m >> l) & 1u);
      rank[l] = __popc(b & ((1u << lane) - 1));
      if (lane == 0) s_warp_cnt[warp][l] = __popc(b);
    }
    __syncthreads();
    for (int l = 0; l < p.num_lists; l++) {
      if ((m >> l) & 1u) {
        uint32_t pos = s_running[l] + rank[l];
        for (uint32_t w = 0; w < warp; w++) pos += s_warp_cnt[w][l];
        out[p.list_base[l] + pos] = (uint32_t)k;
      }
    }
    __syncthreads();
    if (threadIdx.x < (uint32_t)p.num_lists) {
      uint32_t add = 0;
      for (int w = 0; w < kWarpsPerBlock; w++) add += s_warp_cnt[w][threadIdx.x];
      s_running[threadIdx.x] += add;
    }
    __syncthreads();
  }
}

// ------------------------------------------------------------------------------------
// hotness recording: per-key access counts of a batch, kept on the device
// ------------------------------------------------------------------------------------
template <typename KeyT>
__global__ void __launch_bounds__(kBlock)
    record_kernel(const KeyT* __restrict__ keys, uint32_t n, uint32_t* __restrict__ counts,
                  uint64_t num_keys) {
  uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  uint64_t k = (uint64_t)keys[i];
  if (k < num_keys) atomicAdd(counts + k, 1u);  // fire-and-forget reduction in L2
}

// ------------------------------------------------------------------------------------
// synthetic table rows
// ------------------------------------------------------------------------------------
__device__ __forceinline__ uint64_t splitmix64(uint64_t x) {
  x += 0x9e3779b97f4a7c15ull;
  x = (x ^ (x >> 30)) * 0xbf58476d1ce4e5b9ull;
  x = (x ^ (x >> 27)) * 0x94d049bb133111ebull;
  return x ^ (x >> 31);
}
__device__ __forceinline__ uint32_t gen_f32_bits(uint64_t seed, uint64_t e) {
  uint64_t x = splitmix64(seed ^ splitmix64(e));
  return __float_as_uint((float)(x >> 40) * (1.0f / 8388608.0f) - 1.0f);
}
__device__ __forceinline__ uint32_t gen_f16_bits(uint64_t seed, uint64_t e) {
  uint64_t x = splitmix64(seed ^ splitmix64(e));
  int v = (int)(x >> 53) - 1024;  // value = v * 2^-10
  if (v == 0) return 0;
  uint32_t sign = 0;
  if (v < 0) {
    sign = 0x8000u;
    v = -v;
  }
  int msb = 31 - __clz(v);
  uint32_t exp = (uint32_t)(msb - 10 + 15);
  uint32_t man = ((uint32_t)v << (10 - msb)) & 0x3ffu;
  return sign | (exp << 10) | man;
}

// One thread writes 4 bytes: one fp32 element or two fp16 elements.
__global__ void gen_table_kernel(uint32_t* dst, uint64_t seed, uint64_t elem_begin, uint64_t n_words,
                                 int elem_bytes) {
  uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const uint64_t stride = (uint64_t)gridDim.x * blockDim.x;
  for (; i < n_words; i += stride) {
    uint32_t w;
    if (elem_bytes == 4) {
      w = gen_f32_bits(seed, elem_begin + i);
    } else {
      uint64_t e = elem_begin + 2 * i;
      w = gen_f16_bits(seed, e) | (gen_f16_bits(seed, e + 1) << 16);
    }
    dst[i] = w;
  }
}

// ------------------------------------------------------------------------------------
// dispatch helpers
// ------------------------------------------------------------------------------------
inline int grid_for(uint32_t n) { return (int)((n + kBlock - 1) / kBlock); }

// Lanes per row: the smallest power of two >= vectors per row, at most a warp.
inline int lanes_per_row(uint32_t row_bytes, int vec) {
  uint32_t vecs = row_bytes / (uint32_t)vec;
  int l = 1;
  while ((uint32_t)l < vecs && l < 32) l <<= 1;
  return l;
}

// Launch with programmatic stream serialization: the kernel may be scheduled while its
// predecessor in the stream is still running and orders itself with griddepcontrol.wait.
template <typename... KArgs, typename... Args>
cudaError_t launch_pdl(void (*kern)(KArgs...), int grid, int block, size_t smem, cudaStream_t s,
                       bool pdl, Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)grid);
  cfg.blockDim = dim3((unsigned)block);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = s;
  cudaLaunchAttribute attr = {};
  attr.id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr.val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = &attr;
  cfg.numAttrs = pdl ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kern, args...);
}

template <int VEC, int LPR, int UNROLL>
cudaError_t gather_launch(const GatherParams& p, int grid, int block, size_t smem, cudaStream_t s) {
  auto kern = gather_roles_kernel<VEC, LPR, UNROLL>;
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return e;
  }
  return launch_pdl(kern, grid, block, smem, s, p.pdl != 0, p);
}

template <int VEC, int UNROLL>
cudaError_t gather_dispatch_lpr(const GatherParams& p, int grid, int block, size_t smem, cudaStream_t s) {
  switch (lanes_per_row(p.row_bytes, VEC)) {
    case 1: return gather_launch<VEC, 1, UNROLL>(p, grid, block, smem, s);
    case 2: return gather_launch<VEC, 2, UNROLL>(p, grid, block, smem, s);
    case 4: return gather_launch<VEC, 4, UNROLL>(p, grid, block, smem, s);
    case 8: return gather_launch<VEC, 8, UNROLL>(p, grid, block, smem, s);
    case 16: return gather_launch<VEC, 16, UNROLL>(p, grid, block, smem, s);
    default: return gather_launch<VEC, 32, UNROLL>(p, grid, block, smem, s);
  }
}

template <int VEC, int UNROLL>
cudaError_t fill_dispatch_lpr(const KeySlotIndex& ix, uint32_t n, int grid, cudaStream_t s) {
  switch (lanes_per_row(ix.row_bytes, VEC)) {
    case 1: fill_scatter_kernel<VEC, 1, UNROLL><<<grid, kBlock, 0, s>>>(ix, n); break;
    case 2: fill_scatter_kernel<VEC, 2, UNROLL><<<grid, kBlock, 0, s>>>(ix, n); break;
    case 4: fill_scatter_kernel<VEC, 4, UNROLL><<<grid, kBlock, 0, s>>>(ix, n); break;
    case 8: fill_scatter_kernel<VEC, 8, UNROLL><<<grid, kBlock, 0, s>>>(ix, n); break;
    case 16: fill_scatter_kernel<VEC, 16, UNROLL><<<grid, kBlock, 0, s>>>(ix, n); break;
    default: fill_scatter_kernel<VEC, 32, UNROLL><<<grid, kBlock, 0, s>>>(ix, n); break;
  }
  return cudaGetLastError();
}

inline uint32_t host_mask_of(int empty_feat) {
  return empty_feat > 0 && empty_feat < 32 ? ((1u << empty_feat) - 1u) : 0xffffffffu;
}

}  // namespace

// ------------------------------------------------------------------------------------
// launchers
// ------------------------------------------------------------------------------------
cudaError_t launch_lookup_group(const void* keys, int key_bytes, uint32_t n, const TableView& table,
                                uint32_t local_loc, uint32_t host_loc, int empty_feat,
                                uint64_t* list_local, uint64_t* list_remote, uint64_t* list_host,
                                Counters* counters, int keys_per_thread, bool pdl,
                                cudaStream_t stream) {
  if (n == 0) return cudaSuccess;
  const uint32_t mask = host_mask_of(empty_feat);
#define UGC_LAUNCH_LOOKUP(KEYT, KPT)                                                             \
  return launch_pdl(lookup_group_kernel<KEYT, KPT>, (int)((n + kBlock * KPT - 1) / (kBlock * KPT)), \
                    kBlock, 0, stream, pdl, static_cast<const KEYT*>(keys), n, table, local_loc,   \
                    host_loc, mask, list_local, list_remote, list_host, counters)
  if (key_bytes == 8) {
    if (keys_per_thread == 1) UGC_LAUNCH_LOOKUP(long long, 1);
    if (keys_per_thread == 2) UGC_LAUNCH_LOOKUP(long long, 2);
    UGC_LAUNCH_LOOKUP(long long, 4);
  } else {
    if (keys_per_thread == 1) UGC_LAUNCH_LOOKUP(uint32_t, 1);
    if (keys_per_thread == 2) UGC_LAUNCH_LOOKUP(uint32_t, 2);
    UGC_LAUNCH_LOOKUP(uint32_t, 4);
  }
#undef UGC_LAUNCH_LOOKUP
}

int usable_vec_bytes(uint32_t row_bytes, int want, const void* out, const void* const* src_base,
                     int n_src) {
  uintptr_t bits = reinterpret_cast<uintptr_t>(out) | row_bytes;
  for (int i = 0; i < n_src; i++) bits |= reinterpret_cast<uintptr_t>(src_base[i]);
  if (want >= 32 && (bits & 31) == 0) return 32;
  if (want >= 16 && (bits & 15) == 0) return 16;
  return 4;
}

cudaError_t launch_extract_direct(const void* keys, int key_bytes, const DirectParams& p_in, int grid,
                                  int block, int vec_bytes, bool deep, bool early_host, bool pdl,
                                  cudaStream_t stream) {
  if (block != 128 && block != 256) block = kBlock;
  const int warps_per_block = block / 32;
  if (p_in.n_keys == 0) return cudaSuccess;
  DirectParams p = p_in;
  const int vec = usable_vec_bytes(p.row_bytes, vec_bytes, p.out, p.src_base, kMaxLocation);
  const int lpr = lanes_per_row(p.row_bytes, vec);
  p.lpr_shift = 0;
  while ((1 << p.lpr_shift) < lpr) p.lpr_shift++;
  // Tile size: the largest of 32 / 16 / 8 keys (never less than the rows one pass of a warp
  // copies) with which the warps' tile counts differ by less than a tenth; forced by
  // p.tile_shift when that is set.
  const int unroll = (vec == 32 ? 2 : 4) * (deep ? 2 : 1);
  const int rows_per_pass = std::min(32, unroll * (32 / lpr));
  const long long n_warps = (long long)grid * warps_per_block;
  uint32_t shift = p_in.tile_shift;
  if (shift < 3 || shift > 5) {
    shift = 5;
    while (shift > 3 && (1 << (shift - 1)) >= rows_per_pass) {
      const long long tiles = ((long long)p.n_keys + (1ll << shift) - 1) >> shift;
      const long long rounds = (tiles + n_warps - 1) / n_warps;
      if (tiles <= n_warps || (double)tiles / (double)(rounds * n_warps) >= 0.9) break;
      shift--;
    }
  }
  p.tile_shift = shift;
  const int tiles = (int)(((long long)p.n_keys + (1ll << shift) - 1) >> shift);
  grid = std::max(1, std::min(grid, (tiles + warps_per_block - 1) / warps_per_block));
#define UGC_LAUNCH_DIRECT(KEYT, VEC)                                                              \
  do {                                                                                            \
    if (deep)                                                                                     \
      return launch_pdl(extract_direct_kernel<KEYT, VEC, true, false>, grid, block, 0, stream, pdl, \
                        static_cast<const KEYT*>(keys), p);                                       \
    if (early_host)                                                                               \
      return launch_pdl(extract_direct_kernel<KEYT, VEC, false, true>, grid, block, 0, stream, pdl, \
                        static_cast<const KEYT*>(keys), p);                                       \
    return launch_pdl(extract_direct_kernel<KEYT, VEC, false, false>, grid, block, 0, stream, pdl, \
                      static_cast<const KEYT*>(keys), p);                                         \
  } while (0)
  if (key_bytes == 8) {
    if (vec == 32) UGC_LAUNCH_DIRECT(long long, 32);
    if (vec == 16) UGC_LAUNCH_DIRECT(long long, 16);
    UGC_LAUNCH_DIRECT(long long, 4);
  } else {
    if (vec == 32) UGC_LAUNCH_DIRECT(uint32_t, 32);
    if (vec == 16) UGC_LAUNCH_DIRECT(uint32_t, 16);
    UGC_LAUNCH_DIRECT(uint32_t, 4);
  }
#undef UGC_LAUNCH_DIRECT
}

namespace {
// Launch shape of the pooled lookup for pieces of `vec` bytes: lanes per group, bags per tile,
// and the number of warps the batch fills.
struct PoolShape {
  uint32_t lpr_shift, bags_per_tile, warps;
};
PoolShape pool_shape(const PoolParams& p, int vec) {
  PoolShape sh{};
  const int lpr = lanes_per_row(p.row_bytes, vec);
  while ((1 << sh.lpr_shift) < lpr) sh.lpr_shift++;
  // bags per lane group: as many as it takes to give every lane of the group a key to probe
  const uint64_t avg_bag = std::max<uint64_t>(1, p.offsets ? (uint64_t)p.n_keys / p.n_bags : p.bag_size);
  sh.bags_per_tile = (uint32_t)std::max<uint64_t>(1, (uint64_t)lpr / avg_bag);
  const uint64_t n_tiles = ((uint64_t)p.n_bags + sh.bags_per_tile - 1) / sh.bags_per_tile;
  const uint64_t n_pass = (p.row_bytes / (uint32_t)vec + lpr - 1) / lpr;
  sh.warps = (uint32_t)std::min<uint64_t>((n_tiles * n_pass * lpr + 31) / 32, 0xffffffffu);
  return sh;
}
}  // namespace

cudaError_t launch_lookup_pool(const void* keys, int key_bytes, const PoolParams& p_in, bool f16,
                               int max_ctas, int vec_bytes, cudaStream_t stream) {
  if (p_in.n_bags == 0) return cudaSuccess;
  PoolParams p = p_in;
  // 16-byte pieces unless the batch then fills fewer than two warps per SM (few, very long
  // bags): 4-byte pieces put four times as many lane groups on a bag and keep twice as many
  // rows in flight per lane, at four times the probes and load instructions (measured on
  // 212,992 keys of 512-byte rows: bags of 1024 keys 152 against 200 us, bags of 128 keys 51
  // against 33 us)
  PoolShape sh = pool_shape(p, 16);
  int vec = 16;
  if (vec_bytes == 4 || (vec_bytes != 16 && sh.warps < (uint32_t)max_ctas * (kBlock / 32) / 32)) {
    vec = 4;
    sh = pool_shape(p, 4);
  }
  p.lpr_shift = sh.lpr_shift;
  p.bags_per_tile = sh.bags_per_tile;
  const int grid = (int)std::max<uint32_t>(1, std::min<uint32_t>((uint32_t)max_ctas,
                                                                 (sh.warps + kBlock / 32 - 1) / (kBlock / 32)));
#define UGC_LAUNCH_POOL(KEYT, F16, VEC) \
  lookup_pool_kernel<KEYT, F16, VEC><<<grid, kBlock, 0, stream>>>(static_cast<const KEYT*>(keys), p)
  if (key_bytes == 8) {
    if (f16) {
      if (vec == 16) UGC_LAUNCH_POOL(long long, true, 16); else UGC_LAUNCH_POOL(long long, true, 4);
    } else {
      if (vec == 16) UGC_LAUNCH_POOL(long long, false, 16); else UGC_LAUNCH_POOL(long long, false, 4);
    }
  } else {
    if (f16) {
      if (vec == 16) UGC_LAUNCH_POOL(uint32_t, true, 16); else UGC_LAUNCH_POOL(uint32_t, true, 4);
    } else {
      if (vec == 16) UGC_LAUNCH_POOL(uint32_t, false, 16); else UGC_LAUNCH_POOL(uint32_t, false, 4);
    }
  }
#undef UGC_LAUNCH_POOL
  return cudaGetLastError();
}

cudaError_t launch_unique(const void* keys, int key_bytes, uint32_t n, uint64_t num_keys, uint32_t epoch,
                          uint32_t* stamp, void* unique_keys, int32_t* inverse, uint32_t* n_unique,
                          Counters* counters, cudaStream_t stream) {
  if (n == 0) return cudaMemsetAsync(n_unique, 0, sizeof(uint32_t), stream);
  cudaError_t e = cudaMemsetAsync(n_unique, 0, sizeof(uint32_t), stream);
  if (e != cudaSuccess) return e;
  if (key_bytes == 8) {
    unique_claim_kernel<long long><<<grid_for(n), kBlock, 0, stream>>>(
        static_cast<const long long*>(keys), n, num_keys, epoch, stamp, static_cast<long long*>(unique_keys),
        n_unique, counters);
    unique_inverse_kernel<long long><<<grid_for(n), kBlock, 0, stream>>>(static_cast<const long long*>(keys), n,
                                                                         num_keys, stamp, inverse);
  } else {
    unique_claim_kernel<uint32_t><<<grid_for(n), kBlock, 0, stream>>>(
        static_cast<const uint32_t*>(keys), n, num_keys, epoch, stamp, static_cast<uint32_t*>(unique_keys),
        n_unique, counters);
    unique_inverse_kernel<uint32_t><<<grid_for(n), kBlock, 0, stream>>>(static_cast<const uint32_t*>(keys), n,
                                                                        num_keys, stamp, inverse);
  }
  return cudaGetLastError();
}

size_t host_order_scratch_bytes() { return 2 * kHostBuckets * sizeof(uint32_t); }

cudaError_t launch_host_order(const uint64_t* list_host, uint64_t* sorted, const Counters* counters,
                              uint32_t* hist, uint64_t host_rows, int sm_count, cudaStream_t stream) {
  cudaError_t e = cudaMemsetAsync(hist, 0, host_order_scratch_bytes(), stream);
  if (e != cudaSuccess) return e;
  uint32_t shift = 0;  // bucket = row offset >> shift, kHostBuckets buckets over the host table
  while (shift < 32 && (host_rows >> shift) > (uint64_t)kHostBuckets) shift++;
  host_hist_kernel<<<sm_count, kBlock, 0, stream>>>(list_host, counters, hist, shift);
  host_scatter_kernel<<<sm_count, kBlock, 0, stream>>>(list_host, sorted, counters, hist, shift);
  return cudaGetLastError();
}

cudaError_t launch_gather_roles(const GatherParams& p_in, int grid, int block, int vec_bytes,
                                cudaStream_t stream) {
  GatherParams p = p_in;
  vec_bytes = usable_vec_bytes(p.row_bytes, vec_bytes, p.out, p.src_base, kMaxLocation);
  if (grid < 3) grid = 3;  // one CTA per source group at least
  if (block != 256 && block != 512 && block != 1024) block = 256;
  // bulk staging needs 16-byte aligned rows on both sides
  if (p.row_bytes % 16 != 0 || (reinterpret_cast<uintptr_t>(p.out) & 15)) p.bulk_mask = 0;
  size_t smem = 0;
  if (p.bulk_mask) {
    smem = (size_t)(block / 32) * kBulkSlots * (sizeof(uint64_t) + p.row_bytes);
    if (smem > 200 * 1024) {
      p.bulk_mask = 0;
      smem = 0;
    }
  }
  if (vec_bytes == 32) return gather_dispatch_lpr<32, 2>(p, grid, block, smem, stream);
  if (vec_bytes == 16) return gather_dispatch_lpr<16, 4>(p, grid, block, smem, stream);
  return gather_dispatch_lpr<4, 4>(p, grid, block, smem, stream);
}

cudaError_t launch_fill_scatter(const void* host_table, void* slice, const uint32_t* keys,
                                const SlotView& slots, uint32_t n, uint32_t row_bytes,
                                int empty_feat, int grid, cudaStream_t stream) {
  if (n == 0) return cudaSuccess;
  KeySlotIndex ix;
  ix.keys = keys;
  ix.slots = slots;
  ix.host_mask = host_mask_of(empty_feat);
  ix.host = static_cast<const char*>(host_table);
  ix.slice = static_cast<char*>(slice);
  ix.row_bytes = row_bytes;
  if (grid < 1) grid = 1;
  const void* bases[1] = {host_table};
  if (usable_vec_bytes(row_bytes, 16, slice, bases, 1) == 16) return fill_dispatch_lpr<16, 8>(ix, n, grid, stream);
  return fill_dispatch_lpr<4, 8>(ix, n, grid, stream);
}

cudaError_t launch_table_clear(const TableView& t, cudaStream_t stream) {
  size_t bytes = t.kind == kTableFlat ? (size_t)t.num_keys * 4
                                      : ((size_t)t.line_mask + 1) * kSlotsPerLine * sizeof(uint2);
  // flat tables are allocated rounded up to 16 bytes by the runtime
  size_t n16 = (bytes + 15) / 16;
  void* base = t.kind == kTableFlat ? static_cast<void*>(t.flat) : static_cast<void*>(t.slots);
  table_clear_kernel<<<1184, kBlock, 0, stream>>>(static_cast<uint4*>(base), n16);
  return cudaGetLastError();
}

cudaError_t launch_table_insert(const TableView& t, const uint32_t* keys, const SlotView& offs,
                                uint32_t loc, uint32_t n, Counters* counters, cudaStream_t stream,
                                bool allow_same) {
  if (n == 0) return cudaSuccess;
  table_insert_kernel<<<grid_for(n), kBlock, 0, stream>>>(t, keys, offs, loc, n, counters, allow_same);
  return cudaGetLastError();
}

cudaError_t launch_table_repoint(const RepointParams& p, const uint32_t* keys, uint32_t n,
                                 Counters* counters, cudaStream_t stream) {
  if (n == 0) return cudaSuccess;
  table_repoint_kernel<<<grid_for(n), kBlock, 0, stream>>>(p, keys, n, counters);
  return cudaGetLastError();
}

cudaError_t launch_iota(uint32_t* dst, uint32_t start, uint32_t n, cudaStream_t stream) {
  if (n == 0) return cudaSuccess;
  iota_kernel<<<std::min(grid_for(n), 148 * 8), kBlock, 0, stream>>>(dst, start, n);
  return cudaGetLastError();
}

cudaError_t launch_table_evict(const TableView& t, const uint32_t* keys, uint32_t n,
                               Counters* counters, cudaStream_t stream) {
  if (n == 0) return cudaSuccess;
  table_evict_kernel<<<grid_for(n), kBlock, 0, stream>>>(t, keys, n, counters);
  return cudaGetLastError();
}

cudaError_t launch_table_words(const TableView& t, const uint32_t* keys, uint32_t n,
                               uint32_t* words, cudaStream_t stream) {
  if (n == 0) return cudaSuccess;
  table_words_kernel<<<grid_for(n), kBlock, 0, stream>>>(t, keys, n, words);
  return cudaGetLastError();
}

cudaError_t launch_table_resolve(const TableView& peer, const uint32_t* keys, uint32_t n,
                                 uint32_t expect_loc, const SlotView& offs, Counters* counters,
                                 cudaStream_t stream) {
  if (n == 0) return cudaSuccess;
  table_resolve_kernel<<<grid_for(n), kBlock, 0, stream>>>(peer, keys, n, expect_loc, offs, counters);
  return cudaGetLastError();
}

size_t classify_scratch_bytes(uint64_t num_keys) {
  const size_t n_tiles = (size_t)((num_keys + kClassTile - 1) / kClassTile);
  return n_tiles * kMaxClassLists * sizeof(uint32_t) + kMaxClassLists * sizeof(unsigned long long) + 256;
}

// scratch layout: tile counts [kMaxClassLists][n_tiles] u32, then totals [kMaxClassLists] u64
cudaError_t launch_classify_count(const ClassifyParams& p, void* scratch, cudaStream_t stream) {
  const uint32_t n_tiles = (uint32_t)((p.num_keys + kClassTile - 1) / kClassTile);
  uint32_t* tile_counts = static_cast<uint32_t*>(scratch);
  size_t off = ((size_t)n_tiles * kMaxClassLists * sizeof(uint32_t) + 255) / 256 * 256;
  unsigned long long* totals = reinterpret_cast<unsigned long long*>(static_cast<char*>(scratch) + off);
  classify_count_kernel<<<n_tiles, kBlock, 0, stream>>>(p, tile_counts);
  classify_scan_kernel<<<kMaxClassLists, 1024, 0, stream>>>(tile_counts, n_tiles, totals);
  return cudaGetLastError();
}

const unsigned long long* classify_totals(void* scratch, uint64_t num_keys) {
  const size_t n_tiles = (size_t)((num_keys + kClassTile - 1) / kClassTile);
  size_t off = (n_tiles * kMaxClassLists * sizeof(uint32_t) + 255) / 256 * 256;
  return reinterpret_cast<const unsigned long long*>(static_cast<char*>(scratch) + off);
}

cudaError_t launch_classify_scatter(const ClassifyParams& p, const void* scratch, uint32_t* out,
                                    cudaStream_t stream) {
  const uint32_t n_tiles = (uint32_t)((p.num_keys + kClassTile - 1) / kClassTile);
  classify_scatter_kernel<<<n_tiles, kBlock, 0, stream>>>(p, static_cast<const uint32_t*>(scratch), out);
  return cudaGetLastError();
}

cudaError_t launch_record(const void* keys, int key_bytes, uint32_t n, uint32_t* counts,
                          uint64_t num_keys, cudaStream_t stream) {
  if (n == 0) return cudaSuccess;
  if (key_bytes == 8) {
    record_kernel<long long><<<grid_for(n), kBlock, 0, stream>>>(static_cast<const long long*>(keys), n,
                                                                counts, num_keys);
  } else {
    record_kernel<uint32_t><<<grid_for(n), kBlock, 0, stream>>>(static_cast<const uint32_t*>(keys), n,
                                                               counts, num_keys);
  }
  return cudaGetLastError();
}

cudaError_t launch_gen_table(void* dst, uint64_t seed, uint64_t row_begin, uint64_t n_rows,
                             uint64_t dim, int elem_bytes, cudaStream_t stream) {
  uint64_t n_words = n_rows * dim * (uint64_t)elem_bytes / 4;
  if (n_words == 0) return cudaSuccess;
  uint64_t blocks = (n_words + kBlock - 1) / kBlock;
  int grid = (int)(blocks < 148ull * 16 ? blocks : 148ull * 16);
  gen_table_kernel<<<grid, kBlock, 0, stream>>>(static_cast<uint32_t*>(dst), seed, row_begin * dim,
                                                n_words, elem_bytes);
  return cudaGetLastError();
}

}  // namespace ugc
