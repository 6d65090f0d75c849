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
#include <vector>

#include "coll_cache_lib/cuda/cache_hashtable.cuh"

using namespace coll_cache_lib::common;

static uint64_t mix(uint64_t x) {
  x += 0x9e3779b97f4a7c15ull;
  x = (x ^ (x >> 30)) * 0xbf58476d1ce4e5b9ull;
  x = (x ^ (x >> 27)) * 0x94d049bb133111ebull;
  return x ^ (x >> 31);
}

int main(int argc, char** argv) {
  (void)argc; (void)argv;
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
