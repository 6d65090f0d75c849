// C++ facade with the reference's signatures (coll_cache_lib/facade.h:16-81 of the reference,
// paths relative to its project root), implemented header-only on top of the ugc_* C ABI.
//
// A program written against the reference's `coll_cache_lib::CollCache` compiles against
// this header and links libugache_b200.so instead of libcoll_cache.so.  Scope: the lookup /
// build / refresh path with all replicas as threads of ONE process (the reference's
// `cross_process = false` mode); one process per replica goes through the C entry points of
// coll_cache_api.h.  Differences: failures throw std::runtime_error instead of abort()ing;
// MILP policies fall back to the intuitive heuristic.
#pragma once

#include <cuda_runtime.h>

#include <algorithm>
#include <chrono>
#include <condition_variable>
#include <cstdint>
#include <cstdio>
#include <functional>
#include <map>
#include <memory>
#include <mutex>
#include <stdexcept>
#include <string>
#include <thread>
#include <vector>

#include "../ugache_b200.h"

namespace coll_cache_lib {
namespace common {

using IdType = unsigned int;       // coll_cache_lib/constant.h:28
using StreamHandle = void*;        // coll_cache_lib/common.h
enum DataType { kF32 = 0, kF64 = 1, kF16 = 2, kU8 = 3, kI32 = 4, kI8 = 5, kI64 = 6, kF64_2 = 7, kF64_4 = 8 };

inline size_t GetDataTypeBytes(DataType t) {
  static const size_t b[] = {4, 8, 2, 1, 4, 1, 8, 16, 32};
  return b[(int)t];
}

// coll_cache_lib/common.h:140-149
class ExternelGPUMemoryHandler {
 public:
  virtual ~ExternelGPUMemoryHandler() {}
  virtual void* ptr() = 0;
  virtual size_t nbytes() { return 0; }
  template <typename T>
  T* ptr() { return static_cast<T*>(ptr()); }
};
using MemHandle = std::shared_ptr<ExternelGPUMemoryHandler>;

// coll_cache_lib/common.h:162-187
class ExternalBarrierHandler {
 public:
  virtual ~ExternalBarrierHandler() {}
  virtual void Wait() = 0;
};
using BarHandle = std::shared_ptr<ExternalBarrierHandler>;

// coll_cache_lib/freq_recorder.h: ids by descending frequency with their counts
struct ContFreqBuf {
  std::vector<IdType> rank_vec;
  std::vector<IdType> freq_vec;
};

// Step and epoch profile items, numbered as in the reference (coll_cache_lib/profiler.h:61-138)
// so that values logged by an application against those names land in the same slots.
enum LogStepItem {
  kLogL1NumSample = 0, kLogL1NumNode, kLogL1SampleTotalTime, kLogL1SampleTime, kLogL1SendTime,
  kLogL1RecvTime, kLogL1CopyTime, kLogL1ConvertTime, kLogL1TrainTime, kLogL1FeatureBytes,
  kLogL1LabelBytes, kLogL1IdBytes, kLogL1GraphBytes, kLogL1MissBytes, kLogL1RemoteBytes,
  kLogL1PrefetchAdvanced, kLogL1GetNeighbourTime, kLogL1SamplerId,
  kLogL2ShuffleTime, kLogL2LastLayerTime, kLogL2LastLayerSize, kLogL2CoreSampleTime,
  kLogL2IdRemapTime, kLogL2GraphCopyTime, kLogL2IdCopyTime, kLogL2ExtractTime, kLogL2FeatCopyTime,
  kLogL2CacheCopyTime,
  kLogL3KHopSampleCooTime, kLogL3KHopSampleKernelTime, kLogL3KHopSampleSortCooTime,
  kLogL3KHopSampleCountEdgeTime, kLogL3KHopSampleCompactEdgesTime, kLogL3RandomWalkSampleCooTime,
  kLogL3RandomWalkTopKTime, kLogL3RandomWalkTopKStep1Time, kLogL3RandomWalkTopKStep2Time,
  kLogL3RandomWalkTopKStep3Time, kLogL3RandomWalkTopKStep4Time, kLogL3RandomWalkTopKStep5Time,
  kLogL3RandomWalkTopKStep6Time, kLogL3RandomWalkTopKStep7Time, kLogL3RemapFillUniqueTime,
  kLogL3RemapPopulateTime, kLogL3RemapMapNodeTime, kLogL3RemapMapEdgeTime,
  kLogL3CacheGetIndexTime, KLogL3CacheCopyIndexTime, kLogL3CacheExtractMissTime,
  kLogL3CacheCopyMissTime, kLogL3CacheCombineMissTime, kLogL3CacheCombineCacheTime,
  kLogL3CacheCombineRemoteTime, kLogL3LabelExtractTime,
  kNumLogStepItems
};
enum LogEpochItem {
  kLogEpochSampleTime = 0, KLogEpochSampleGetCacheMissIndexTime, kLogEpochSampleSendTime,
  kLogEpochSampleTotalTime, kLogEpochCoreSampleTime, kLogEpochSampleCooTime, kLogEpochIdRemapTime,
  kLogEpochShuffleTime, kLogEpochSampleKernelTime, kLogEpochCopyTime, kLogEpochConvertTime,
  kLogEpochTrainTime, kLogEpochTotalTime, kLogEpochFeatureBytes, kLogEpochMissBytes,
  kNumLogEpochItems
};

// In-process stand-in for the reference's Profiler (coll_cache_lib/profiler.h/.cc; its
// shared-memory report backend is not rebuilt): values per step key and per epoch, averages,
// and the percentiles of the lookup time the reference prints in report_avg
// (coll_cache_lib/facade.cc:570-584).
class Profiler {
 public:
  void LogStep(uint64_t key, LogStepItem item, double val) {
    if (item < 0 || item >= kNumLogStepItems) return;
    std::lock_guard<std::mutex> lock(_mu);
    Row& r = _steps[key];
    r.val[item] = val;
    r.set[item] = true;
  }
  void LogEpochAdd(uint64_t epoch, LogEpochItem item, double val) {
    if (item < 0 || item >= kNumLogEpochItems) return;
    std::lock_guard<std::mutex> lock(_mu);
    _epochs[epoch].val[item] += val;
    _epochs[epoch].set[item] = true;
  }
  bool Get(uint64_t key, LogStepItem item, double* out) {
    std::lock_guard<std::mutex> lock(_mu);
    auto it = _steps.find(key);
    if (it == _steps.end() || !it->second.set[item]) return false;
    *out = it->second.val[item];
    return true;
  }
  void ReportStep(uint64_t key) {
    std::lock_guard<std::mutex> lock(_mu);
    auto it = _steps.find(key);
    if (it == _steps.end()) return;
    std::printf("[Step %llu]", (unsigned long long)key);
    for (int i = 0; i < kNumLogStepItems; i++)
      if (it->second.set[i]) std::printf(" item%d=%.6g", i, it->second.val[i]);
    std::printf("\n");
    std::fflush(stdout);
  }
  // Averages over the steps whose key is >= first_key, then percentiles of the lookup time.
  void ReportStepAverage(uint64_t first_key = 0) {
    std::lock_guard<std::mutex> lock(_mu);
    double sum[kNumLogStepItems] = {0};
    size_t cnt[kNumLogStepItems] = {0};
    std::vector<double> copy;
    for (auto& kv : _steps) {
      if (kv.first < first_key) continue;
      for (int i = 0; i < kNumLogStepItems; i++)
        if (kv.second.set[i]) {
          sum[i] += kv.second.val[i];
          cnt[i]++;
          if (i == kLogL2CacheCopyTime) copy.push_back(kv.second.val[i]);
        }
    }
    std::printf("[Step(average)]");
    for (int i = 0; i < kNumLogStepItems; i++)
      if (cnt[i]) std::printf(" item%d=%.6g", i, sum[i] / cnt[i]);
    std::printf("\n");
    if (!copy.empty()) {
      std::sort(copy.begin(), copy.end());
      const double ps[] = {50, 90, 95, 99, 99.9};
      std::printf("tail_logl2featcopy");
      for (double p : ps)
        std::printf(" p%g=%.6g", p, copy[std::min(copy.size() - 1, (size_t)(p / 100.0 * copy.size()))]);
      std::printf("\n");
    }
    for (auto& kv : _epochs) {
      std::printf("[Epoch %llu]", (unsigned long long)kv.first);
      for (int i = 0; i < kNumLogEpochItems; i++)
        if (kv.second.set[i]) std::printf(" item%d=%.6g", i, kv.second.val[i]);
      std::printf("\n");
    }
    std::fflush(stdout);
  }
  size_t NumSteps() {
    std::lock_guard<std::mutex> lock(_mu);
    return _steps.size();
  }

 private:
  static constexpr int kRowItems =
      (int)kNumLogStepItems > (int)kNumLogEpochItems ? (int)kNumLogStepItems : (int)kNumLogEpochItems;
  struct Row {
    double val[kRowItems] = {0};
    bool set[kRowItems] = {false};
  };
  std::mutex _mu;
  std::map<uint64_t, Row> _steps, _epochs;
};

// The few static settings of the reference's RunConfig this path reads
// (coll_cache_lib/run_config.h:30-111).
struct RunConfig {
  static int& num_device() { static int v = 1; return v; }
  static int& cache_policy() { static int v = UGC_POLICY_INTUITIVE; return v; }
  static std::vector<int>& device_id_list() { static std::vector<int> v; return v; }
  static uint32_t& max_batch() { static uint32_t v = 1u << 21; return v; }
  // step keys are epoch * steps_per_epoch + step (coll_cache_lib/run_config.h)
  static uint64_t& num_global_step_per_epoch() { static uint64_t v = 1; return v; }
  static uint64_t& num_epoch() { static uint64_t v = 1; return v; }
};

}  // namespace common

using namespace common;

class CollCache : public std::enable_shared_from_this<CollCache> {
 public:
  CollCache(BarHandle process_barrier, BarHandle replica_barrier)
      : _process_barrier(process_barrier), _replica_barrier(replica_barrier),
        _profiler(std::make_shared<Profiler>()) {}
  ~CollCache() {
    if (_ctx) ugc_destroy(_ctx);
  }

  // The two-call form of the reference (coll_cache_lib/facade.h:47-53, facade.cc:38-72): `solve`
  // fixes the placement from a hotness ranking, `build` then builds every replica of this
  // process, one thread per replica, each with the allocator `allocator_builder` returns for it.
  void solve(IdType* ranking_nodes_list_ptr, IdType* ranking_nodes_freq_list_ptr, IdType num_node) {
    _solve_ids.assign(ranking_nodes_list_ptr, ranking_nodes_list_ptr + num_node);
    if (ranking_nodes_freq_list_ptr)
      _solve_freqs.assign(ranking_nodes_freq_list_ptr, ranking_nodes_freq_list_ptr + num_node);
    else
      _solve_freqs.clear();
  }
  void build(std::function<std::function<MemHandle(size_t)>(int)> allocator_builder, void* cpu_data,
             DataType dtype, size_t dim, double cache_percentage, StreamHandle stream = nullptr) {
    if (_solve_ids.empty()) throw std::runtime_error("CollCache::build: call solve() first");
    const int G = RunConfig::num_device();
    // the replica barrier handed to the constructor belongs to the caller's own threads; the
    // builder threads of this call meet at a barrier of their own
    struct LocalBarrier : ExternalBarrierHandler {
      explicit LocalBarrier(int n) : n(n) {}
      void Wait() override {
        std::unique_lock<std::mutex> lock(mu);
        const uint64_t gen = generation;
        if (++waiting == n) {
          waiting = 0;
          generation++;
          cv.notify_all();
        } else {
          cv.wait(lock, [&] { return generation != gen; });
        }
      }
      int n, waiting = 0;
      uint64_t generation = 0;
      std::mutex mu;
      std::condition_variable cv;
    };
    BarHandle saved = _replica_barrier;
    _replica_barrier = std::make_shared<LocalBarrier>(G);
    std::vector<std::thread> builders;
    std::vector<std::string> errors(G);
    for (int r = 0; r < G; r++)
      builders.emplace_back([&, r] {
        try {
          build_v2(r, _solve_ids.data(), _solve_freqs.empty() ? nullptr : _solve_freqs.data(),
                   (IdType)_solve_ids.size(), allocator_builder(r), cpu_data, dtype, dim,
                   cache_percentage, stream);
        } catch (const std::exception& e) {
          errors[r] = e.what();
        }
      });
    for (auto& t : builders) t.join();
    _replica_barrier = saved;
    for (auto& e : errors)
      if (!e.empty()) throw std::runtime_error("CollCache::build: " + e);
  }

  void build_v2(int replica_id, IdType* ranking_nodes_list_ptr, IdType* ranking_nodes_freq_list_ptr,
                IdType num_node, std::function<MemHandle(size_t)> gpu_mem_allocator, void* cpu_data,
                DataType dtype, size_t dim, double cache_percentage, StreamHandle stream = nullptr) {
    const int G = RunConfig::num_device();
    if (replica_id == 0) {
      ugc_config cfg;
      ugc_config_default(&cfg);
      cfg.num_device = G;
      cfg.num_total_item = num_node;
      cfg.row_bytes = (uint32_t)(dim * GetDataTypeBytes(dtype));
      _row_bytes = cfg.row_bytes;
      cfg.cache_percentage = cache_percentage;
      cfg.max_batch = RunConfig::max_batch();
      cfg.alloc = &CollCache::alloc_tramp;
      cfg.free = &CollCache::free_tramp;
      cfg.alloc_user = this;
      check(ugc_create(&cfg, &_ctx), "ugc_create");
      _allocators.assign(G, nullptr);
      solve(ranking_nodes_list_ptr, ranking_nodes_freq_list_ptr, num_node, cache_percentage, false);
    }
    wait();
    {
      std::lock_guard<std::mutex> lock(_mu);
      _allocators[replica_id] = gpu_mem_allocator;
    }
    const auto& ids = RunConfig::device_id_list();
    const int dev = replica_id < (int)ids.size() ? ids[replica_id] : replica_id;
    _tls_replica() = replica_id;
    check(ugc_build(_ctx, replica_id, dev, cpu_data, stream), "ugc_build");
    wait();
    if (replica_id == 0) check(ugc_connect_local(_ctx), "ugc_connect_local");
    wait();
    check(ugc_attach_peers(_ctx, replica_id, stream), "ugc_attach_peers");
    wait();
  }

  void build_v2(int replica_id, ContFreqBuf* freq_rank, IdType num_node,
                std::function<MemHandle(size_t)> gpu_mem_allocator, void* cpu_data, DataType dtype,
                size_t dim, double cache_percentage, StreamHandle stream = nullptr) {
    build_v2(replica_id, freq_rank ? freq_rank->rank_vec.data() : nullptr,
             freq_rank ? freq_rank->freq_vec.data() : nullptr, num_node, gpu_mem_allocator, cpu_data,
             dtype, dim, cache_percentage, stream);
  }

  // Returns after the rows are in `output` (the reference synchronises its internal streams).
  // The time of the call goes to the step log under kLogL2CacheCopyTime as in the reference
  // (coll_cache_lib/facade.cc:85-87); the phase times the reference logs inside its extraction
  // (index building, then the copy from each kind of source, cache_context.cu:1662-1679) come
  // from the device clock of the kernels, and the byte counts from the per-source row counts.
  void lookup(int replica_id, const IdType* nodes, const size_t num_nodes, void* output,
              StreamHandle stream, uint64_t step_key) {
    const auto t0 = std::chrono::steady_clock::now();
    check(ugc_lookup_u32(_ctx, replica_id, nodes, num_nodes, output, stream), "ugc_lookup_u32");
    if (cudaStreamSynchronize(static_cast<cudaStream_t>(stream)) != cudaSuccess)
      throw std::runtime_error("CollCache::lookup: stream synchronise failed");
    const double dt = std::chrono::duration<double>(std::chrono::steady_clock::now() - t0).count();
    _profiler->LogStep(step_key, kLogL2CacheCopyTime, dt);
    ugc_stats_t st;
    if (ugc_stats(_ctx, replica_id, &st) == UGC_OK) {
      _profiler->LogStep(step_key, kLogL3CacheGetIndexTime, st.last_index_ns * 1e-9);
      _profiler->LogStep(step_key, kLogL3CacheCombineMissTime, st.last_host_ns * 1e-9);
      _profiler->LogStep(step_key, kLogL3CacheCombineRemoteTime, st.last_remote_ns * 1e-9);
      _profiler->LogStep(step_key, kLogL3CacheCombineCacheTime, st.last_local_ns * 1e-9);
      _profiler->LogStep(step_key, kLogL1FeatureBytes, (double)num_nodes * _row_bytes);
      _profiler->LogStep(step_key, kLogL1MissBytes, (double)st.last_host * _row_bytes);
      _profiler->LogStep(step_key, kLogL1RemoteBytes, (double)st.last_remote * _row_bytes);
    }
  }

  void refresh(int replica_id, IdType* ranking_nodes_list_ptr, IdType* ranking_nodes_freq_list_ptr,
               StreamHandle stream = nullptr, bool foreground = false) {
    (void)foreground;
    if (replica_id == 0)
      solve(ranking_nodes_list_ptr, ranking_nodes_freq_list_ptr, (IdType)_num_node, _pct, true);
    wait();
    check(ugc_refresh_evict(_ctx, replica_id, stream), "ugc_refresh_evict");
    wait();
    check(ugc_refresh_fill(_ctx, replica_id, stream), "ugc_refresh_fill");
    wait();
    check(ugc_refresh_attach(_ctx, replica_id, stream), "ugc_refresh_attach");
    wait();
    if (replica_id == 0) check(ugc_refresh_commit(_ctx), "ugc_refresh_commit");
    wait();
  }
  void refresh(int replica_id, ContFreqBuf* freq_rank, StreamHandle stream = nullptr, bool foreground = false) {
    refresh(replica_id, freq_rank ? freq_rank->rank_vec.data() : nullptr,
            freq_rank ? freq_rank->freq_vec.data() : nullptr, stream, foreground);
  }

  // coll_cache_lib/facade.cc:559-588
  void report_avg() { _profiler->ReportStepAverage(0); }
  void report_last_epoch(uint64_t epoch) {
    _profiler->ReportStepAverage(epoch * RunConfig::num_global_step_per_epoch());
  }
  void report(uint64_t key) { _profiler->ReportStep(key); }
  std::shared_ptr<Profiler> _profiler;

  // for profile (coll_cache_lib/facade.h:75-81)
  inline void set_step_profile_value(uint64_t key, LogStepItem item, double val) {
    _profiler->LogStep(key, item, val);
  }
  inline void add_epoch_profile_value(uint64_t key, LogEpochItem item, double val) {
    _profiler->LogEpochAdd(key, item, val);
  }

  ugc_ctx* context() { return _ctx; }

 private:
  static int& _tls_replica() {
    thread_local int r = 0;
    return r;
  }
  void wait() {
    if (_replica_barrier) _replica_barrier->Wait();
  }
  void check(int rc, const char* what) {
    if (rc != UGC_OK) throw std::runtime_error(std::string(what) + ": " + ugc_last_error());
  }
  void solve(IdType* ids, IdType* freqs, IdType num_node, double pct, bool is_refresh) {
    const int G = RunConfig::num_device();
    int policy = RunConfig::cache_policy();
    if (policy != UGC_POLICY_REP && policy != UGC_POLICY_CLIQUE_PART) policy = UGC_POLICY_INTUITIVE;
    std::vector<uint32_t> n2b(num_node);
    std::vector<uint8_t> bp(G + 2), ba((size_t)G * (G + 2));
    std::vector<double> bd(G + 2);
    double tl, tr, tc;
    ugc_link_model(G, &tl, &tr, &tc);
    int nb = 0;
    check(ugc_solve_placement(policy, G, num_node, ids, freqs, pct * 100.0, tl, tr, tc, n2b.data(),
                              bp.data(), ba.data(), bd.data(), &nb),
          "ugc_solve_placement");
    if (is_refresh) {
      check(ugc_refresh_set_placement(_ctx, n2b.data(), bp.data(), ba.data(), bd.data(), nb),
            "ugc_refresh_set_placement");
    } else {
      check(ugc_set_placement(_ctx, n2b.data(), bp.data(), ba.data(), bd.data(), nb), "ugc_set_placement");
    }
    _num_node = num_node;
    _pct = pct;
  }
  std::vector<IdType> _solve_ids, _solve_freqs;
  uint32_t _row_bytes = 0;
  // the caller's allocator returns ref-counted handles; keep them until the library frees
  static void* alloc_tramp(size_t nbytes, void* user) {
    CollCache* self = static_cast<CollCache*>(user);
    std::lock_guard<std::mutex> lock(self->_mu);
    auto& fn = self->_allocators[_tls_replica()];
    if (!fn) return nullptr;
    MemHandle h = fn(nbytes);
    if (!h) return nullptr;
    void* p = h->ptr();
    self->_held[p] = h;
    return p;
  }
  static void free_tramp(void* p, void* user) {
    CollCache* self = static_cast<CollCache*>(user);
    std::lock_guard<std::mutex> lock(self->_mu);
    self->_held.erase(p);
  }

  BarHandle _process_barrier, _replica_barrier;
  ugc_ctx* _ctx = nullptr;
  std::mutex _mu;
  std::vector<std::function<MemHandle(size_t)>> _allocators;
  std::map<void*, MemHandle> _held;
  size_t _num_node = 0;
  double _pct = 0;
};

}  // namespace coll_cache_lib
