// Reference pin: prints known-answer values computed BY THE REFERENCE'S OWN CODE (its
// headers and sources are compiled in place from the reference tree; none are copied).
// Test infrastructure only.  Output is JSON on stdout; tests/golden/make_golden.py stores
// it as tests/golden/ref_pin.json, which pins the CPU oracle's integer helpers.
//
// Host-side values (no GPU needed): MurmurHash3_32<uint32>, EmbCacheOff packing,
// TableSize.  With `--gpu` and a visible device it additionally builds the reference's
// SimpleHashTable / FlatHashTable with the reference's kernels, looks keys up through
// them and prints a digest of the answers.
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <string>
#include <vector>

#include "coll_cache_lib/cuda/cache_hashtable.cuh"

using namespace coll_cache_lib::common;

static uint64_t mix(uint64_t x) {
  x += 0x9e3779b97f4a7c15ull;
  x = (x ^ (x >> 30)) * 0xbf58476d1ce4e5b9ull;
  x = (x ^ (x >> 27)) * 0x94d049bb133111ebull;
  return x ^ (x >> 31);
}

// ---- GPU mode: the reference's own table kernels on a scenario read from files --------------
//   ref_pin --gpu <dir>
// <dir>/scenario.bin : u32 header {N, n_ins, n_evict, n_reins, fallback_loc}, then
//   keys[n_ins], locs[n_ins], offs[n_ins], evict[n_evict], reins_keys[n_reins], reins_offs[n_reins]
//   (re-inserted keys get location 1).  Every evicted key is present; every inserted key absent.
// Writes <dir>/words_simple.bin and <dir>/words_flat.bin: the packed word the reference's
// lookup (lookup_hashmap_with_helper + its EmbedVal helper) returns for every key in [0, N).
#define PIN_CUDA(expr)                                                                   \
  do {                                                                                   \
    cudaError_t e__ = (expr);                                                            \
    if (e__ != cudaSuccess) {                                                            \
      fprintf(stderr, "%s failed: %s\n", #expr, cudaGetErrorString(e__));                \
      exit(4);                                                                           \
    }                                                                                    \
  } while (0)

static std::vector<uint32_t> read_u32(FILE* f, size_t n) {
  std::vector<uint32_t> v(n);
  if (n && fread(v.data(), 4, n, f) != n) { fprintf(stderr, "short scenario file\n"); exit(3); }
  return v;
}

template <typename Table>
static void run_table(Table& t, uint32_t N, const std::vector<uint32_t>& keys, const std::vector<uint32_t>& locs,
                      const std::vector<uint32_t>& offs, const std::vector<uint32_t>& evict,
                      const std::vector<uint32_t>& rk, const std::vector<uint32_t>& ro, int fallback_loc,
                      const std::string& out_path) {
  cudaStream_t s;
  PIN_CUDA(cudaStreamCreate(&s));
  auto to_dev = [&](const std::vector<uint32_t>& h) {
    uint32_t* d = nullptr;
    PIN_CUDA(cudaMalloc(&d, std::max<size_t>(h.size(), 1) * 4));
    if (!h.empty()) PIN_CUDA(cudaMemcpy(d, h.data(), h.size() * 4, cudaMemcpyHostToDevice));
    return d;
  };
  // one insert launch per location (as the build does: local rows, then each peer's rows)
  for (uint32_t loc = 0; loc < 8; loc++) {
    std::vector<uint32_t> k, o;
    for (size_t i = 0; i < keys.size(); i++) if (locs[i] == loc) { k.push_back(keys[i]); o.push_back(offs[i]); }
    if (k.empty()) continue;
    uint32_t* dk = to_dev(k); uint32_t* dof = to_dev(o);
    t.template InsertUnique<HashTableInsertHelper::SingleLoc>(dk, HashTableInsertHelper::SingleLoc(dof, (int)loc), k.size(), s);
    PIN_CUDA(cudaStreamSynchronize(s));
    cudaFree(dk); cudaFree(dof);
  }
  if (!evict.empty()) {
    uint32_t* de = to_dev(evict);
    t.EvictWithUnique(de, evict.size(), s);
    PIN_CUDA(cudaStreamSynchronize(s));
    cudaFree(de);
  }
  if (!rk.empty()) {
    uint32_t* dk = to_dev(rk); uint32_t* dof = to_dev(ro);
    t.template InsertUnique<HashTableInsertHelper::SingleLoc>(dk, HashTableInsertHelper::SingleLoc(dof, 1), rk.size(), s);
    PIN_CUDA(cudaStreamSynchronize(s));
    cudaFree(dk); cudaFree(dof);
  }
  std::vector<uint32_t> all(N);
  for (uint32_t i = 0; i < N; i++) all[i] = i;
  uint32_t* dall = to_dev(all);
  ValType* dvals = nullptr;
  PIN_CUDA(cudaMalloc(&dvals, (size_t)N * sizeof(ValType)));
  t.LookupValCustom(dall, N, HashTableLookupHelper::EmbedVal(dvals, nullptr, fallback_loc), s);
  PIN_CUDA(cudaStreamSynchronize(s));
  std::vector<uint32_t> words(N);
  PIN_CUDA(cudaMemcpy(words.data(), dvals, (size_t)N * 4, cudaMemcpyDeviceToHost));
  FILE* f = fopen(out_path.c_str(), "wb");
  fwrite(words.data(), 4, N, f);
  fclose(f);
  cudaFree(dall); cudaFree(dvals);
  cudaStreamDestroy(s);
}

// The reference's tables take their memory from a caller-supplied allocator (its cache manager
// passes the framework's); this is the pin program's own cudaMalloc-backed one.
class PinDeviceBlock : public ExternelGPUMemoryHandler {
 public:
  explicit PinDeviceBlock(size_t n) : n_(n) { PIN_CUDA(cudaMalloc(&p_, n)); }
  ~PinDeviceBlock() override { cudaFree(p_); }
  void* ptr() override { return p_; }
  size_t nbytes() override { return n_; }
 private:
  void* p_ = nullptr;
  size_t n_;
};

static int gpu_mode(const std::string& dir) {
  FILE* f = fopen((dir + "/scenario.bin").c_str(), "rb");
  if (!f) { fprintf(stderr, "no scenario.bin in %s\n", dir.c_str()); return 3; }
  auto hdr = read_u32(f, 5);
  const uint32_t N = hdr[0], n_ins = hdr[1], n_ev = hdr[2], n_re = hdr[3];
  const int fallback = (int)hdr[4];
  auto keys = read_u32(f, n_ins), locs = read_u32(f, n_ins), offs = read_u32(f, n_ins);
  auto evict = read_u32(f, n_ev), rk = read_u32(f, n_re), ro = read_u32(f, n_re);
  fclose(f);
  PIN_CUDA(cudaSetDevice(0));
  cudaStream_t s0 = nullptr;
  std::function<MemHandle(size_t)> alloc = [](size_t n) -> MemHandle { return std::make_shared<PinDeviceBlock>(n); };
  {
    SimpleHashTable t(alloc, n_ins, GPU(0), s0);
    run_table(t, N, keys, locs, offs, evict, rk, ro, fallback, dir + "/words_simple.bin");
  }
  {
    FlatHashTable t(alloc, N, GPU(0), s0);
    run_table(t, N, keys, locs, offs, evict, rk, ro, fallback, dir + "/words_flat.bin");
  }
  printf("ref tables ok\n");
  return 0;
}

int main(int argc, char** argv) {
  if (argc >= 3 && std::string(argv[1]) == "--gpu") return gpu_mode(argv[2]);
  MurmurHash3_32<IdType> hasher;
  printf("{\n  \"murmur3_32\": [");
  // fixed keys + 4096 pseudo-random keys below 2^31
  std::vector<uint32_t> keys = {0u, 1u, 2u, 3u, 255u, 256u, 65535u, 65536u, 12345u, 1000000u,
                                99999999u, 0x7ffffffeu, 0x7fffffffu};
  for (uint64_t i = 0; i < 4096; i++) keys.push_back((uint32_t)(mix(i) & 0x7fffffffu));
  for (size_t i = 0; i < keys.size(); i++)
    printf("%s[%u, %u]", i ? ", " : "", keys[i], hasher(keys[i]));
  printf("],\n  \"emb_cache_off\": [");
  const uint32_t locs[] = {0, 1, 7, 8, 15};
  const uint32_t offs[] = {0, 1, 12345, 0x0ffffffeu, 0x0fffffffu};
  bool first = true;
  for (uint32_t l : locs) for (uint32_t o : offs) {
    EmbCacheOff e(l, o);
    printf("%s[%u, %u, %u, %u, %u]", first ? "" : ", ", l, o, e.data, e.loc(), e.off());
    first = false;
  }
  printf("],\n  \"table_size\": [");
  const size_t nums[] = {2, 3, 4, 5, 100, 1000, 1024, 1025, 65536, 1000000, 2000000, 10000000,
                         16777215, 16777216, 16777217, 40000000, 80000000, 100000000};
  for (size_t i = 0; i < sizeof(nums) / sizeof(nums[0]); i++)
    printf("%s[%zu, %zu]", i ? ", " : "", nums[i], TableSize(nums[i]));
  printf("],\n  \"constants\": {\"kEmptyKey\": %u, \"kEmptyPos\": %u}\n}\n",
         (unsigned)Constant::kEmptyKey, (unsigned)kEmptyPos);
  return 0;
}
