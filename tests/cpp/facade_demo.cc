// Exercises the C++ facade (include/coll_cache_lib/facade.h) the way a program written for
// the reference uses CollCache: one thread per replica, build_v2 -> lookup -> refresh ->
// lookup, results compared with a plain CPU gather.  Prints "facade ok" on success.
#include <cuda_runtime.h>

#include <atomic>
#include <condition_variable>
#include <cstdio>
#include <cstring>
#include <mutex>
#include <numeric>
#include <thread>
#include <vector>

#include "coll_cache_lib/facade.h"

using namespace coll_cache_lib;

struct CudaMem : common::ExternelGPUMemoryHandler {
  void* p = nullptr;
  size_t n = 0;
  ~CudaMem() override { cudaFree(p); }
  void* ptr() override { return p; }
  size_t nbytes() override { return n; }
};

struct ThreadBarrier : common::ExternalBarrierHandler {
  std::mutex m;
  std::condition_variable cv;
  int count = 0, gen = 0, n;
  explicit ThreadBarrier(int n) : n(n) {}
  void Wait() override {
    std::unique_lock<std::mutex> l(m);
    int g = gen;
    if (++count == n) {
      count = 0;
      gen++;
      cv.notify_all();
    } else {
      cv.wait(l, [&] { return gen != g; });
    }
  }
};

static uint64_t mix(uint64_t x) {
  x += 0x9e3779b97f4a7c15ull;
  x = (x ^ (x >> 30)) * 0xbf58476d1ce4e5b9ull;
  x = (x ^ (x >> 27)) * 0x94d049bb133111ebull;
  return x ^ (x >> 31);
}

int main() {
  const int G = 2;
  const common::IdType N = 30000;
  const size_t dim = 32;
  int ndev = 0;
  if (cudaGetDeviceCount(&ndev) != cudaSuccess || ndev < 1) {
    printf("no GPU\n");
    return 2;
  }
  common::RunConfig::num_device() = G;
  common::RunConfig::cache_policy() = UGC_POLICY_INTUITIVE;
  common::RunConfig::device_id_list() = {0, ndev > 1 ? 1 : 0};
  common::RunConfig::max_batch() = 1 << 14;

  float* table = nullptr;
  cudaHostAlloc(&table, (size_t)N * dim * sizeof(float), cudaHostAllocPortable | cudaHostAllocMapped);
  for (size_t i = 0; i < (size_t)N * dim; i++) table[i] = (float)(mix(i) >> 40) / 8388608.0f - 1.0f;

  std::vector<common::IdType> rank_ids(N), rank_freqs(N);
  std::iota(rank_ids.begin(), rank_ids.end(), 0u);
  for (common::IdType r = 0; r < N; r++) rank_freqs[r] = 4000000000u / (r + 1);
  std::vector<common::IdType> rank_ids2(rank_ids);
  for (common::IdType r = 0; r < N; r++) rank_ids2[r] = (rank_ids[r] + 7000) % N;  // hot set moves

  auto barrier = std::make_shared<ThreadBarrier>(G);
  auto cache = std::make_shared<CollCache>(nullptr, barrier);
  std::atomic<int> failures{0};

  auto worker = [&](int r) {
    try {
      const int dev = common::RunConfig::device_id_list()[r];
      cudaSetDevice(dev);
      cudaStream_t stream;
      cudaStreamCreate(&stream);
      auto alloc = [dev](size_t nbytes) -> common::MemHandle {
        auto h = std::make_shared<CudaMem>();
        cudaSetDevice(dev);
        if (cudaMalloc(&h->p, nbytes) != cudaSuccess) return nullptr;
        h->n = nbytes;
        return h;
      };
      cache->build_v2(r, rank_ids.data(), rank_freqs.data(), N, alloc, table, common::kF32, dim, 0.10, stream);
      const size_t n = 5000;
      std::vector<common::IdType> keys(n);
      for (size_t i = 0; i < n; i++) keys[i] = (common::IdType)(mix(1000 * r + i) % (i % 3 ? 3000 : N));
      common::IdType* dkeys;
      float* dout;
      cudaMalloc(&dkeys, n * sizeof(common::IdType));
      cudaMalloc(&dout, n * dim * sizeof(float));
      cudaMemcpy(dkeys, keys.data(), n * sizeof(common::IdType), cudaMemcpyHostToDevice);
      std::vector<float> got(n * dim);
      for (int round = 0; round < 2; round++) {
        cache->lookup(r, dkeys, n, dout, stream, (uint64_t)(round * G + r));
        cudaMemcpy(got.data(), dout, got.size() * sizeof(float), cudaMemcpyDeviceToHost);
        for (size_t i = 0; i < n; i++)
          if (memcmp(&got[i * dim], &table[(size_t)keys[i] * dim], dim * sizeof(float)) != 0) {
            failures++;
            break;
          }
        if (round == 0) cache->refresh(r, rank_ids2.data(), rank_freqs.data(), stream, true);
      }
      cudaFree(dkeys);
      cudaFree(dout);
      cudaStreamDestroy(stream);
    } catch (const std::exception& e) {
      fprintf(stderr, "replica %d: %s\n", r, e.what());
      failures++;
    }
  };
  std::vector<std::thread> ts;
  for (int r = 0; r < G; r++) ts.emplace_back(worker, r);
  for (auto& t : ts) t.join();

  // profile surface of the facade: the lookups above logged their time, phase times and byte
  // counts per step key; the application adds values of its own under the reference's item names
  cache->set_step_profile_value(0, common::kLogL1TrainTime, 0.125);
  cache->add_epoch_profile_value(0, common::kLogEpochTrainTime, 1.5);
  cache->add_epoch_profile_value(0, common::kLogEpochTrainTime, 2.5);
  double v = 0;
  if (cache->_profiler->NumSteps() != (size_t)(2 * G)) failures++;
  if (!cache->_profiler->Get(0, common::kLogL2CacheCopyTime, &v) || v <= 0) failures++;
  if (!cache->_profiler->Get(1, common::kLogL1FeatureBytes, &v) || v != 5000.0 * dim * sizeof(float)) failures++;
  if (!cache->_profiler->Get(0, common::kLogL1TrainTime, &v) || v != 0.125) failures++;
  cache->report(0);
  cache->report_last_epoch(0);
  cache->report_avg();
  cache.reset();

  // the two-call form: solve() fixes the placement, build() builds every replica in threads of
  // its own with the allocator the builder returns per replica
  {
    auto cache2 = std::make_shared<CollCache>(nullptr, barrier);
    cache2->solve(rank_ids.data(), rank_freqs.data(), N);
    cache2->build(
        [&](int r) -> std::function<common::MemHandle(size_t)> {
          const int dev = common::RunConfig::device_id_list()[r];
          return [dev](size_t nbytes) -> common::MemHandle {
            auto h = std::make_shared<CudaMem>();
            cudaSetDevice(dev);
            if (cudaMalloc(&h->p, nbytes) != cudaSuccess) return nullptr;
            h->n = nbytes;
            return h;
          };
        },
        table, common::kF32, dim, 0.10, nullptr);
    const size_t n = 3000;
    std::vector<common::IdType> keys(n);
    for (size_t i = 0; i < n; i++) keys[i] = (common::IdType)(mix(77 + i) % N);
    for (int r = 0; r < G; r++) {
      cudaSetDevice(common::RunConfig::device_id_list()[r]);
      common::IdType* dkeys;
      float* dout;
      cudaMalloc(&dkeys, n * sizeof(common::IdType));
      cudaMalloc(&dout, n * dim * sizeof(float));
      cudaMemcpy(dkeys, keys.data(), n * sizeof(common::IdType), cudaMemcpyHostToDevice);
      cache2->lookup(r, dkeys, n, dout, nullptr, (uint64_t)r);
      std::vector<float> got(n * dim);
      cudaMemcpy(got.data(), dout, got.size() * sizeof(float), cudaMemcpyDeviceToHost);
      for (size_t i = 0; i < n; i++)
        if (memcmp(&got[i * dim], &table[(size_t)keys[i] * dim], dim * sizeof(float)) != 0) {
          failures++;
          break;
        }
      cudaFree(dkeys);
      cudaFree(dout);
    }
  }
  cudaFreeHost(table);
  if (failures.load()) {
    printf("facade FAILED (%d)\n", failures.load());
    return 1;
  }
  printf("facade ok\n");
  return 0;
}
