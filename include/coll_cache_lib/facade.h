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

#include <cstdint>
#include <functional>
#include <map>
#include <memory>
#include <mutex>
#include <stdexcept>
#include <string>
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

// The few static settings of the reference's RunConfig this path reads
// (coll_cache_lib/run_config.h:30-111).
struct RunConfig {
  static int& num_device() { static int v = 1; return v; }
  static int& cache_policy() { static int v = UGC_POLICY_INTUITIVE; return v; }
  static std::vector<int>& device_id_list() { static std::vector<int> v; return v; }
  static uint32_t& max_batch() { static uint32_t v = 1u << 21; return v; }
};

}  // namespace common

using namespace common;

class CollCache : public std::enable_shared_from_this<CollCache> {
 public:
  CollCache(BarHandle process_barrier, BarHandle replica_barrier)
      : _process_barrier(process_barrier), _replica_barrier(replica_barrier) {}
  ~CollCache() {
    if (_ctx) ugc_destroy(_ctx);
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
  void lookup(int replica_id, const IdType* nodes, const size_t num_nodes, void* output,
              StreamHandle stream, uint64_t step_key) {
    (void)step_key;
    check(ugc_lookup_u32(_ctx, replica_id, nodes, num_nodes, output, stream), "ugc_lookup_u32");
    if (cudaStreamSynchronize(static_cast<cudaStream_t>(stream)) != cudaSuccess)
      throw std::runtime_error("CollCache::lookup: stream synchronise failed");
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

  void report_avg() {}
  void report_last_epoch(uint64_t) {}
  void report(uint64_t) {}

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
