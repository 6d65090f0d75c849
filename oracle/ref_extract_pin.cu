/*
 * Runs the REFERENCE's own extraction device code on a file-described case.  TEST
 * INFRASTRUCTURE ONLY — built into oracle/_ref/ (never shipped, never loaded by the product).
 *
 * The reference's extraction source file (coll_cache_lib/cache_context.cu) is compiled in place
 * by including it here, which makes its file-local kernels callable.  The steps below are the
 * ones ExtractSession performs for one lookup, each done by the reference's code:
 *   1. key table: SimpleHashTable / FlatHashTable, InsertUnique<SingleLoc> per location
 *      (cuda/cache_hashtable.cuh);
 *   2. records: LookupValCustom with LookupHelper<false, IdxStoreCompact>
 *      (what CacheEntryManager::LookupSrcDst launches, cuda/cache_hashtable.cuh:583-594);
 *   3. grouping: CubSortDispatcher over the 64-bit records, as
 *      ExtractSession::GetMissCacheIndex does (cache_context.cu:702-761);
 *   4. boundaries: find_boundary + the host fix-up of ExtractSession::SplitGroup
 *      (cache_context.cu:825-847);
 *   5. row copy: Combine(DataIterPerLoc<IdxStoreCompact>) per location -> extract_data
 *      (cache_context.cu:1076-1100, :214-231), with the element type the facade picks
 *      (16-byte elements when the row size allows, facade.cc:459-463).
 * Only this sequencing and the file I/O are written here.
 *
 * Input  <dir>/extract.bin : u32 header {N, n_entries, n_keys, n_loc, row_bytes, use_flat},
 *        entry keys / locs / offs (u32 x n_entries each), rows_per_loc (u32 x n_loc),
 *        batch keys (u32 x n_keys), then the source arrays (rows_per_loc[l] x row_bytes bytes)
 *        for l = 0..n_loc-1.  The last location is the host: its array is placed in pinned
 *        host memory, the others in device memory.
 * Output <dir>/out.bin (n_keys x row_bytes), records.bin (sorted 8-byte records),
 *        groups.bin (u32 x (n_loc + 1)).
 *
 * With "--fill <dir>" it runs the reference's two ways of writing rows INTO a cache slice:
 *   build:   Combine(DataIterPerLoc<IdxStoreDirect<false>>): slice[j] = host[keys[j]]
 *            (cache_context.cu:2480-2484);
 *   refresh: Combine(DataIterPerLoc<IdxStoreDst<false>>) in batches of 4092 rows on 20 blocks:
 *            slice[dst[j]] = host[keys[j]] (cache_context.cu:4061-4070; the pauses between
 *            batches are left out).
 * Input  <dir>/fill.bin : u32 header {N, n_build, row_bytes, slice_rows, n_scatter}, build keys,
 *        scatter keys, scatter destinations, then the host table (N x row_bytes bytes).
 * Output <dir>/slice.bin (slice_rows x row_bytes; rows nothing wrote stay zero).
 *
 * With "--time <dir>" it TIMES the same device code on a one-GPU cache (local slice + host
 * table), as the baseline a recompiled reference would give on this GPU:
 *   per lookup: records (+ sync), radix sort (+ sync), find_boundary (+ sync, host fix-up), then
 *   the host group and the local group copied by extract_data on two streams, then both synced
 *   - the order and the synchronisations of ExtractSession::GetMissCacheIndex / SplitGroup /
 *   ExtractFeat (cache_context.cu:702-761, :825-847, :1330-1440).  Left out, all in the
 *   reference's favour: its per-source host threads and their semaphore hand-off, the 60 us
 *   sleep, and the SM-mask / MPS partitioning of the copy kernels (the mask interface addresses
 *   the SM count of older GPUs only).  Device memory comes from a size-keyed pool, standing in
 *   for the caching allocator of the framework the reference runs under.
 * Input  <dir>/time.bin : u32 header {N, n_cached, n_keys, n_steps, warmup, row_bytes, k}, the
 *        cached keys in slot order, then (warmup + n_steps) key batches of n_keys u32 each.
 *        k != 0 selects the reference's mock host table of 2^k rows (host row = key mod 2^k,
 *        RunConfig::option_empty_feat); the reference packs a host row index into 28 bits, so
 *        without it N may not exceed 2^28 and the program refuses such a case.
 *        Host row r is filled with the 32-bit value r, so the output can be checked from the keys.
 * Output one JSON line on stdout.
 */
#include "coll_cache_lib/cache_context.cu"

#include <chrono>
#include <cstdio>
#include <map>
#include <string>
#include <vector>

using namespace coll_cache_lib;
using namespace coll_cache_lib::common;

#define PIN_CUDA(call)                                                                     \
  do {                                                                                     \
    cudaError_t e_ = (call);                                                               \
    if (e_ != cudaSuccess) {                                                               \
      fprintf(stderr, "%s:%d %s\n", __FILE__, __LINE__, cudaGetErrorString(e_));           \
      exit(2);                                                                             \
    }                                                                                      \
  } while (0)

namespace {

// freed blocks are kept by size and handed out again (time mode only)
bool g_pool_blocks = false;
std::multimap<size_t, void*> g_pool;

class PinDeviceBlock : public ExternelGPUMemoryHandler {
 public:
  explicit PinDeviceBlock(size_t n) : n_(n ? n : 1) {
    auto it = g_pool.find(n_);
    if (it != g_pool.end()) { p_ = it->second; g_pool.erase(it); return; }
    PIN_CUDA(cudaMalloc(&p_, n_));
  }
  ~PinDeviceBlock() override {
    if (g_pool_blocks) g_pool.emplace(n_, p_);
    else cudaFree(p_);
  }
  void* ptr() override { return p_; }
  size_t nbytes() override { return n_; }

 private:
  void* p_ = nullptr;
  size_t n_;
};

// The reference packs (location, row index) into 4 + 28 bits (cuda/cache_hashtable.h:22-25): a
// host row index of 2^28 or more would spill into the location bits and send find_boundary past
// the end of the boundary array.  Such a case is refused before anything runs.
bool offsets_overflow(unsigned long long host_rows) {
  if (host_rows <= (1ull << 28)) return false;
  fprintf(stderr, "refused: %llu host rows do not fit the reference's 28-bit row index\n", host_rows);
  return true;
}

std::vector<uint32_t> read_u32(FILE* f, size_t n) {
  std::vector<uint32_t> v(n);
  if (n && fread(v.data(), 4, n, f) != n) { fprintf(stderr, "short read\n"); exit(3); }
  return v;
}

template <typename T>
T* to_dev(const std::vector<T>& v) {
  T* d = nullptr;
  PIN_CUDA(cudaMalloc(&d, v.size() * sizeof(T) + 16));
  PIN_CUDA(cudaMemcpy(d, v.data(), v.size() * sizeof(T), cudaMemcpyHostToDevice));
  return d;
}

void dump(const std::string& path, const void* p, size_t bytes) {
  FILE* f = fopen(path.c_str(), "wb");
  fwrite(p, 1, bytes, f);
  fclose(f);
}

template <typename Table>
void insert_entries(Table& t, uint32_t n_loc, const std::vector<uint32_t>& keys,
                    const std::vector<uint32_t>& locs, const std::vector<uint32_t>& offs,
                    cudaStream_t s) {
  for (uint32_t loc = 0; loc < n_loc; loc++) {
    std::vector<uint32_t> k, o;
    for (size_t i = 0; i < keys.size(); i++)
      if (locs[i] == loc) { k.push_back(keys[i]); o.push_back(offs[i]); }
    if (k.empty()) continue;
    uint32_t* dk = to_dev(k);
    uint32_t* dof = to_dev(o);
    t.template InsertUnique<HashTableInsertHelper::SingleLoc>(
        dk, HashTableInsertHelper::SingleLoc(dof, (int)loc), k.size(), s);
    PIN_CUDA(cudaStreamSynchronize(s));
    cudaFree(dk);
    cudaFree(dof);
  }
}

}  // namespace

static int fill_mode(const std::string& dir) {
  FILE* f = fopen((dir + "/fill.bin").c_str(), "rb");
  if (!f) { fprintf(stderr, "no fill.bin in %s\n", dir.c_str()); return 3; }
  auto hdr = read_u32(f, 5);
  const uint32_t N = hdr[0], n_build = hdr[1], row_bytes = hdr[2], slice_rows = hdr[3], n_sc = hdr[4];
  auto bkeys = read_u32(f, n_build), skeys = read_u32(f, n_sc), sdst = read_u32(f, n_sc);
  if (n_build > slice_rows) { fprintf(stderr, "build list longer than the slice\n"); return 5; }
  for (uint32_t k : bkeys) if (k >= N) { fprintf(stderr, "build key out of range\n"); return 5; }
  for (size_t i = 0; i < n_sc; i++)
    if (skeys[i] >= N || sdst[i] >= slice_rows) { fprintf(stderr, "scatter %zu out of range\n", i); return 5; }
  PIN_CUDA(cudaSetDevice(0));
  RunConfig::option_empty_feat = 0;
  Context gpu = GPU(0);
  cudaStream_t s = nullptr;
  PIN_CUDA(cudaStreamCreate(&s));
  const size_t tbytes = (size_t)N * row_bytes;
  void* host = nullptr;
  PIN_CUDA(cudaHostAlloc(&host, tbytes, cudaHostAllocMapped));
  if (fread(host, 1, tbytes, f) != tbytes) { fprintf(stderr, "short read\n"); return 3; }
  fclose(f);
  void* slice = nullptr;
  const size_t sbytes = (size_t)slice_rows * row_bytes;
  PIN_CUDA(cudaMalloc(&slice, sbytes + 16));
  PIN_CUDA(cudaMemset(slice, 0, sbytes));
  DataType dtype = kF32;
  IdType dim = row_bytes / 4;
  if (row_bytes % 16 == 0) { dtype = kF64_2; dim = row_bytes / 16; }
  uint32_t* d_bkeys = to_dev(bkeys);
  if (n_build) {
    IdxStoreDirect<false> idx_store(d_bkeys);
    DataIterPerLoc<decltype(idx_store)> it(idx_store, host, slice, dim);
    Combine(it, n_build, gpu, dtype, dim, s);
  }
  uint32_t* d_skeys = to_dev(skeys);
  uint32_t* d_sdst = to_dev(sdst);
  const size_t batch = 4092;
  for (size_t b = 0; b < n_sc; b += batch) {
    const size_t cur = (b + batch < n_sc) ? batch : (n_sc - b);
    IdxStoreDst<false> idx_store(d_skeys + b, d_sdst + b);
    DataIterPerLoc<decltype(idx_store)> it(idx_store, host, slice, dim);
    Combine(it, cur, gpu, dtype, dim, s, 20);
  }
  PIN_CUDA(cudaStreamSynchronize(s));
  std::vector<char> h(sbytes);
  PIN_CUDA(cudaMemcpy(h.data(), slice, sbytes, cudaMemcpyDeviceToHost));
  dump(dir + "/slice.bin", h.data(), sbytes);
  printf("ref fill ok\n");
  return 0;
}

static int time_mode(const std::string& dir) {
  FILE* f = fopen((dir + "/time.bin").c_str(), "rb");
  if (!f) { fprintf(stderr, "no time.bin in %s\n", dir.c_str()); return 3; }
  auto hdr = read_u32(f, 7);
  const uint32_t N = hdr[0], n_cached = hdr[1], n_keys = hdr[2], n_steps = hdr[3], warmup = hdr[4];
  const uint32_t row_bytes = hdr[5], mock_bits = hdr[6];
  if (offsets_overflow(mock_bits ? (1ull << mock_bits) : N) || mock_bits > 28) { fclose(f); return 5; }
  const size_t host_rows = mock_bits ? ((size_t)1 << mock_bits) : N;
  auto cached = read_u32(f, n_cached);
  auto batches = read_u32(f, (size_t)(n_steps + warmup) * n_keys);
  fclose(f);
  for (uint32_t k : cached) if (k >= N) { fprintf(stderr, "cached key out of range\n"); return 5; }
  for (uint32_t k : batches) if (k >= N) { fprintf(stderr, "key out of range\n"); return 5; }
  PIN_CUDA(cudaSetDevice(0));
  RunConfig::option_empty_feat = mock_bits;
  g_pool_blocks = true;
  Context gpu = GPU(0);
  cudaStream_t s = nullptr, s_host = nullptr, s_local = nullptr;
  PIN_CUDA(cudaStreamCreate(&s));
  PIN_CUDA(cudaStreamCreate(&s_host));
  PIN_CUDA(cudaStreamCreate(&s_local));
  std::function<MemHandle(size_t)> alloc = [](size_t n) -> MemHandle {
    return std::make_shared<PinDeviceBlock>(n);
  };
  const size_t words_per_row = row_bytes / 4;
  uint32_t* host = nullptr;
  PIN_CUDA(cudaHostAlloc(&host, host_rows * row_bytes, cudaHostAllocMapped));
#pragma omp parallel for schedule(static)
  for (long long r = 0; r < (long long)host_rows; r++)
    for (size_t w = 0; w < words_per_row; w++) host[(size_t)r * words_per_row + w] = (uint32_t)r;
  DataType dtype = kF32;
  IdType dim = row_bytes / 4;
  if (row_bytes % 16 == 0) { dtype = kF64_2; dim = row_bytes / 16; }

  // build: slice[j] = host[cached[j]], table entry cached[j] -> (location 0, j)
  void* slice = nullptr;
  PIN_CUDA(cudaMalloc(&slice, (size_t)n_cached * row_bytes + 16));
  uint32_t* d_cached = to_dev(cached);
  if (mock_bits) {
    IdxStoreDirect<true> idx_store(d_cached);
    DataIterPerLoc<decltype(idx_store)> it(idx_store, host, slice, dim);
    Combine(it, n_cached, gpu, dtype, dim, s);
  } else {
    IdxStoreDirect<false> idx_store(d_cached);
    DataIterPerLoc<decltype(idx_store)> it(idx_store, host, slice, dim);
    Combine(it, n_cached, gpu, dtype, dim, s);
  }
  FlatHashTable table(alloc, (size_t)N, gpu, s);
  {
    std::vector<uint32_t> offs(n_cached);
    for (uint32_t j = 0; j < n_cached; j++) offs[j] = j;
    uint32_t* d_offs = to_dev(offs);
    table.InsertUnique<HashTableInsertHelper::SingleLoc>(d_cached, HashTableInsertHelper::SingleLoc(d_offs, 0),
                                                        n_cached, s);
    PIN_CUDA(cudaStreamSynchronize(s));
    cudaFree(d_offs);
  }
  uint32_t* d_batches = to_dev(batches);
  void* out = nullptr;
  PIN_CUDA(cudaMalloc(&out, (size_t)n_keys * row_bytes + 16));
  const int host_loc = 1, n_loc = 2;
  void* src[2] = {slice, host};
  IdType* group_offset = nullptr;
  PIN_CUDA(cudaHostAlloc(&group_offset, sizeof(IdType) * (n_loc + 1), cudaHostAllocMapped));
  MemHandle idx_mem, alter_mem;
  cudaEvent_t e0, e1, e_idx, e_host, e_local;
  PIN_CUDA(cudaEventCreate(&e0));
  PIN_CUDA(cudaEventCreate(&e1));
  PIN_CUDA(cudaEventCreate(&e_idx));
  PIN_CUDA(cudaEventCreateWithFlags(&e_host, cudaEventDisableTiming));
  PIN_CUDA(cudaEventCreateWithFlags(&e_local, cudaEventDisableTiming));
  double sum_dev = 0, sum_idx = 0, sum_wall = 0;
  uint64_t n_host_rows = 0, n_local_rows = 0;
  for (uint32_t step = 0; step < n_steps + warmup; step++) {
    const uint32_t* d_keys = d_batches + (size_t)step * n_keys;
    PIN_CUDA(cudaDeviceSynchronize());
    auto w0 = std::chrono::steady_clock::now();
    PIN_CUDA(cudaEventRecord(e0, s));
    IdxStoreCompact idx, idx_alter;
    if (idx_mem == nullptr || idx_mem->nbytes() < idx.required_mem(n_keys)) {
      idx_mem = alloc(idx.required_mem(n_keys));
      alter_mem = alloc(idx.required_mem(n_keys));
    }
    idx.prepare_mem(idx_mem->ptr<uint8_t>(), n_keys);
    if (mock_bits) {
      auto helper = HashTableLookupHelper::LookupHelper<true, IdxStoreCompact>(host_loc);
      helper.idx_store = idx;
      table.LookupValCustom(d_keys, n_keys, helper, s);
      PIN_CUDA(cudaStreamSynchronize(s));
    } else {
      auto helper = HashTableLookupHelper::LookupHelper<false, IdxStoreCompact>(host_loc);
      helper.idx_store = idx;
      table.LookupValCustom(d_keys, n_keys, helper, s);
      PIN_CUDA(cudaStreamSynchronize(s));
    }
    idx_alter.prepare_mem(alter_mem->ptr<uint8_t>(), n_keys);
    common::cuda::CubSortDispatcher(idx.keys_for_sort(), idx_alter.keys_for_sort(), idx.vals_for_sort(),
                                    idx_alter.vals_for_sort(), n_keys, gpu, alloc, false, s);
    memset(group_offset, 0, sizeof(IdType) * (n_loc + 1));
    PIN_CUDA(cudaStreamSynchronize(s));
    group_offset[n_loc] = n_keys;
    {
      const dim3 grid(RoundUpDiv((size_t)n_keys, Constant::kCudaTileSize));
      const dim3 block(Constant::kCudaBlockSize);
      find_boundary<><<<grid, block, 0, s>>>(idx, n_keys, group_offset);
      PIN_CUDA(cudaEventRecord(e_idx, s));
      PIN_CUDA(cudaStreamSynchronize(s));
      for (int i = 1; i < n_loc; i++)
        if (group_offset[i + 1] == 0) group_offset[i + 1] = group_offset[i];
    }
    // host group first, then the local group, each on its own stream
    PIN_CUDA(cudaStreamWaitEvent(s_host, e_idx, 0));
    PIN_CUDA(cudaStreamWaitEvent(s_local, e_idx, 0));
    for (int l = n_loc - 1; l >= 0; l--) {
      const size_t cnt = group_offset[l + 1] - group_offset[l];
      DataIterPerLoc<IdxStoreCompact> it(idx.sub_array(group_offset[l]), src[l], out, dim);
      Combine(it, cnt, gpu, dtype, dim, l == host_loc ? s_host : s_local, 0, true);
    }
    PIN_CUDA(cudaEventRecord(e_host, s_host));
    PIN_CUDA(cudaEventRecord(e_local, s_local));
    PIN_CUDA(cudaStreamWaitEvent(s, e_host, 0));
    PIN_CUDA(cudaStreamWaitEvent(s, e_local, 0));
    PIN_CUDA(cudaEventRecord(e1, s));
    PIN_CUDA(cudaStreamSynchronize(s_host));
    PIN_CUDA(cudaStreamSynchronize(s_local));
    PIN_CUDA(cudaStreamSynchronize(s));
    auto w1 = std::chrono::steady_clock::now();
    // the swap of the sort's double buffer moved the records: keep the handles in step
    if (idx.src_dst_idx != (SrcKeyDstVal*)idx_mem->ptr()) std::swap(idx_mem, alter_mem);
    if (step >= warmup) {
      float ms = 0, ms_idx = 0;
      PIN_CUDA(cudaEventElapsedTime(&ms, e0, e1));
      PIN_CUDA(cudaEventElapsedTime(&ms_idx, e0, e_idx));
      sum_dev += ms * 1e3;
      sum_idx += ms_idx * 1e3;
      sum_wall += std::chrono::duration<double, std::micro>(w1 - w0).count();
      n_local_rows += group_offset[1];
      n_host_rows += group_offset[2] - group_offset[1];
    }
  }
  // check the last batch: every word of output row i is the key of that row
  std::vector<uint32_t> h_out((size_t)n_keys * words_per_row);
  PIN_CUDA(cudaMemcpy(h_out.data(), out, h_out.size() * 4, cudaMemcpyDeviceToHost));
  const uint32_t* last = batches.data() + (size_t)(n_steps + warmup - 1) * n_keys;
  size_t bad = 0;
  for (size_t i = 0; i < n_keys; i++)
    for (size_t w = 0; w < words_per_row; w++)
      bad += h_out[i * words_per_row + w] != (mock_bits ? last[i] % (1u << mock_bits) : last[i]);
  printf("{\"steps\": %u, \"keys\": %u, \"row_bytes\": %u, \"device_us\": %.2f, \"index_us\": %.2f, "
         "\"wall_us\": %.2f, \"local_rows\": %.1f, \"host_rows\": %.1f, \"mismatched_words\": %zu}\n",
         n_steps, n_keys, row_bytes, sum_dev / n_steps, sum_idx / n_steps, sum_wall / n_steps,
         (double)n_local_rows / n_steps, (double)n_host_rows / n_steps, bad);
  return bad ? 4 : 0;
}

int main(int argc, char** argv) {
  if (argc < 2) { fprintf(stderr, "usage: %s [--fill|--time] <dir>\n", argv[0]); return 1; }
  if (argc >= 3 && std::string(argv[1]) == "--fill") return fill_mode(argv[2]);
  if (argc >= 3 && std::string(argv[1]) == "--time") return time_mode(argv[2]);
  const std::string dir = argv[1];
  FILE* f = fopen((dir + "/extract.bin").c_str(), "rb");
  if (!f) { fprintf(stderr, "no extract.bin in %s\n", dir.c_str()); return 3; }
  auto hdr = read_u32(f, 6);
  const uint32_t N = hdr[0], n_ent = hdr[1], n_keys = hdr[2], n_loc = hdr[3], row_bytes = hdr[4];
  const bool use_flat = hdr[5] != 0;
  if (offsets_overflow(N) || n_loc > 9) { fclose(f); return 5; }
  const int host_loc = (int)n_loc - 1;
  auto ekeys = read_u32(f, n_ent), elocs = read_u32(f, n_ent), eoffs = read_u32(f, n_ent);
  auto rows = read_u32(f, n_loc);
  auto batch = read_u32(f, n_keys);
  // every index the kernels will dereference is checked here, on the host
  if (rows[host_loc] < N) { fprintf(stderr, "host source shorter than the id space\n"); return 5; }
  for (size_t i = 0; i < n_ent; i++)
    if (ekeys[i] >= N || elocs[i] >= n_loc || eoffs[i] >= rows[elocs[i]]) {
      fprintf(stderr, "entry %zu out of range\n", i);
      return 5;
    }
  for (size_t i = 0; i < n_keys; i++)
    if (batch[i] >= N) { fprintf(stderr, "key %zu out of range\n", i); return 5; }

  PIN_CUDA(cudaSetDevice(0));
  RunConfig::option_empty_feat = 0;
  Context gpu = GPU(0);
  cudaStream_t s = nullptr;
  PIN_CUDA(cudaStreamCreate(&s));
  std::function<MemHandle(size_t)> alloc = [](size_t n) -> MemHandle {
    return std::make_shared<PinDeviceBlock>(n);
  };

  // the sources: device arrays for the GPU locations, pinned host memory for the last one
  std::vector<void*> src(n_loc, nullptr);
  for (uint32_t l = 0; l < n_loc; l++) {
    const size_t bytes = (size_t)rows[l] * row_bytes;
    std::vector<char> h(bytes);
    if (bytes && fread(h.data(), 1, bytes, f) != bytes) { fprintf(stderr, "short read\n"); return 3; }
    if ((int)l == host_loc) {
      PIN_CUDA(cudaHostAlloc(&src[l], bytes ? bytes : 16, cudaHostAllocMapped));
      memcpy(src[l], h.data(), bytes);
    } else {
      PIN_CUDA(cudaMalloc(&src[l], bytes ? bytes : 16));
      PIN_CUDA(cudaMemcpy(src[l], h.data(), bytes, cudaMemcpyHostToDevice));
    }
  }
  fclose(f);

  // 1. key table
  std::shared_ptr<SimpleHashTable> simple;
  std::shared_ptr<FlatHashTable> flat;
  if (use_flat) {
    flat = std::make_shared<FlatHashTable>(alloc, (size_t)N, gpu, s);
    insert_entries(*flat, n_loc, ekeys, elocs, eoffs, s);
  } else {
    simple = std::make_shared<SimpleHashTable>(alloc, (size_t)n_ent, gpu, s);
    insert_entries(*simple, n_loc, ekeys, elocs, eoffs, s);
  }

  // 2. records
  uint32_t* d_keys = to_dev(batch);
  IdxStoreCompact idx, idx_alter;
  MemHandle idx_mem = alloc(idx.required_mem(n_keys)), alter_mem = alloc(idx.required_mem(n_keys));
  idx.prepare_mem(idx_mem->ptr<uint8_t>(), n_keys);
  idx_alter.prepare_mem(alter_mem->ptr<uint8_t>(), n_keys);
  {
    auto helper = HashTableLookupHelper::LookupHelper<false, IdxStoreCompact>(host_loc);
    helper.idx_store = idx;
    if (use_flat) flat->LookupValCustom(d_keys, n_keys, helper, s);
    else simple->LookupValCustom(d_keys, n_keys, helper, s);
    PIN_CUDA(cudaStreamSynchronize(s));
  }

  // 3. grouping
  common::cuda::CubSortDispatcher(idx.keys_for_sort(), idx_alter.keys_for_sort(), idx.vals_for_sort(),
                                  idx_alter.vals_for_sort(), n_keys, gpu, alloc, false, s);
  PIN_CUDA(cudaStreamSynchronize(s));

  // 4. boundaries
  IdType* group_offset = nullptr;
  PIN_CUDA(cudaHostAlloc(&group_offset, sizeof(IdType) * (n_loc + 1), cudaHostAllocMapped));
  memset(group_offset, 0, sizeof(IdType) * (n_loc + 1));
  group_offset[n_loc] = n_keys;
  if (n_keys) {
    const dim3 grid(RoundUpDiv((size_t)n_keys, Constant::kCudaTileSize));
    const dim3 block(Constant::kCudaBlockSize);
    find_boundary<><<<grid, block, 0, s>>>(idx, n_keys, group_offset);
    PIN_CUDA(cudaStreamSynchronize(s));
    for (int i = 1; i < (int)n_loc; i++)
      if (group_offset[i + 1] == 0) group_offset[i + 1] = group_offset[i];
  }

  // 5. row copy, one launch per location
  void* out = nullptr;
  PIN_CUDA(cudaMalloc(&out, (size_t)n_keys * row_bytes + 16));
  PIN_CUDA(cudaMemset(out, 0xA5, (size_t)n_keys * row_bytes));
  DataType dtype = kF32;
  IdType dim = row_bytes / 4;
  if (row_bytes % 16 == 0) { dtype = kF64_2; dim = row_bytes / 16; }
  for (uint32_t l = 0; l < n_loc; l++) {
    const size_t cnt = group_offset[l + 1] - group_offset[l];
    DataIterPerLoc<IdxStoreCompact> it(idx.sub_array(group_offset[l]), src[l], out, dim);
    Combine(it, cnt, gpu, dtype, dim, s, 0, false);
  }
  PIN_CUDA(cudaStreamSynchronize(s));

  std::vector<char> h_out((size_t)n_keys * row_bytes);
  PIN_CUDA(cudaMemcpy(h_out.data(), out, h_out.size(), cudaMemcpyDeviceToHost));
  dump(dir + "/out.bin", h_out.data(), h_out.size());
  std::vector<uint64_t> h_rec(n_keys);
  PIN_CUDA(cudaMemcpy(h_rec.data(), idx.src_dst_idx, (size_t)n_keys * 8, cudaMemcpyDeviceToHost));
  dump(dir + "/records.bin", h_rec.data(), (size_t)n_keys * 8);
  dump(dir + "/groups.bin", group_offset, sizeof(IdType) * (n_loc + 1));
  printf("ref extract ok\n");
  return 0;
}
