// Host-side (no CUDA) parts of the runtime: the placement arrays, the reference's non-MILP
// placement heuristics, the B200 link model and the per-reader key classification.
#pragma once
#include <cstdint>
#include <memory>
#include <string>
#include <utility>
#include <vector>

namespace ugc {

// Allocator whose resize() leaves new elements uninitialised: the per-key array of a placement
// is 4 bytes per id (1.6 GB at 4*10^8 ids) and is always overwritten in full right after it is
// sized, by several threads; value-initialising it first would touch every page from one thread.
template <class T>
struct NoInitAlloc : std::allocator<T> {
  template <class U>
  struct rebind {
    using other = NoInitAlloc<U>;
  };
  NoInitAlloc() = default;
  template <class U>
  NoInitAlloc(const NoInitAlloc<U>&) {}
  template <class U, class... Args>
  void construct(U* p, Args&&... args) {
    if constexpr (sizeof...(Args) == 0) {
      ::new (static_cast<void*>(p)) U;
    } else {
      ::new (static_cast<void*>(p)) U(std::forward<Args>(args)...);
    }
  }
};

// The four arrays the policy hands to the cache runtime
// (coll_cache_lib/facade.cc:238-261, coll_cache_lib/coll_cache/optimal_solver_class.h:34-70).
struct Placement {
  std::vector<uint32_t, NoInitAlloc<uint32_t>> nid_to_block;  // [N]
  std::vector<uint8_t> block_placement;     // [B] bit g: rows of the block are stored on GPU g
  std::vector<uint8_t> block_access_from;   // [G][B] source location per reader (G = host)
  std::vector<double> block_density;        // [B] percent of N
  int num_block = 0;
  int num_device = 0;
  bool valid = false;

  uint8_t access(int reader, uint32_t block) const {
    return block_access_from[(size_t)reader * num_block + block];
  }
  bool stored_on(int gpu, uint32_t key) const {
    return (block_placement[nid_to_block[key]] >> gpu) & 1;
  }
};

// Checks that the arrays describe a placement the runtime can serve: every reader's
// source for a block stores that block, and a GPU that stores a block reads its own copy.
// Returns an empty string or the reason.
// `check_block_ids` = false skips the pass over nid_to_block (for callers that range-checked
// the ids while copying them).
std::string validate_placement(const Placement& p, int num_device, uint64_t num_total_item,
                               bool check_block_ids = true);

// Time-per-byte ratios local : peer : host on an NVSwitch-connected B200 box (HBM3e ~8 TB/s,
// NVLink 5 900 GB/s per direction, PCIe Gen5 ~64 GB/s).  With G-1 peers read concurrently the
// aggregated peer time is t_remote (the reference divides by the link count,
// coll_cache_lib/coll_cache/asymm_link_desc.cc:412-419; on NVSwitch every peer shares the one
// 900 GB/s port, so no division applies here).
void b200_link_model(int num_device, double* t_local, double* t_remote, double* t_cpu);

// What one GPU of an NVSwitch-connected B200 box can pull from each kind of source while all
// `num_device` GPUs of the job do the same, and what it takes to keep each link busy: the
// B200 counterpart of the reference's per-platform link table with its SM counts per link
// (AsymmLinkDesc::AutoBuild, coll_cache_lib/coll_cache/asymm_link_desc.cc:242-392).
struct LinkDesc {
  int num_device;
  double bw_local_gbs;     // HBM3e, read or write
  double bw_remote_gbs;    // all peers together into this GPU: one NVLink port; 0 with one GPU
  double bw_host_gbs;      // host rows into this GPU (link, shared host side, scattered-row rate)
  double lat_local_us, lat_remote_us, lat_host_us;  // load-to-use latencies, for Little's law
  double host_rows_per_s;  // scattered rows of pinned host memory per second per GPU
  double host_total_gbs;   // what the host side sustains for all GPUs together
  double t_local, t_remote, t_cpu;  // time-per-byte ratios for the placement solvers
  int host_ctas, remote_ctas, per_peer_ctas;  // 256-thread CTAs that keep each far link full
};
// row_bytes == 0: bandwidth figures only (no scattered-row term).  Zero / negative overrides
// are ignored.
LinkDesc b200_link_desc(int num_device, uint32_t row_bytes, double bw_local_override = 0,
                        double bw_remote_override = 0, double bw_host_override = 0);

// IntuitiveSolver / RepSolver / CliquePartSolver of the reference
// (coll_cache_lib/coll_cache/optimal_solver_class.cc:1251-1404, :1869-1924, :1926-2058).
// plus UGC_POLICY_SPLIT_SEARCH, which has no counterpart among them: it stands in for the
// reference's MILP (optimal_solver_class.cc:957-1112) on a switch-connected box by costing every
// replicate/partition split against the recorded hotness.
// cache_percent in percent.  Returns an empty string or the reason for failure.
std::string solve_placement(int policy, int num_device, uint64_t num_total_item,
                            const uint32_t* rank_ids, const uint32_t* rank_freqs,
                            double cache_percent, double t_local, double t_remote, double t_cpu,
                            Placement* out);

// Modelled cost of a placement per reader under the concurrent-source model the split-search
// policy minimises: max((local + served to peers + 1) * t_local, peers * t_remote, host * t_cpu),
// the fractions being shares of the recorded hotness.  Lets callers compare policies before building.
// `nid_to_block_in_place`, if given, is read instead of p.nid_to_block (spares the caller a copy
// of the per-key array).
std::string placement_cost(const Placement& p, uint64_t num_total_item, const uint32_t* rank_ids,
                           const uint32_t* rank_freqs, double t_local, double t_remote, double t_cpu,
                           double* cost_per_reader, const uint32_t* nid_to_block_in_place = nullptr);

// Keys served to `reader` by each GPU source, ascending key order
// (replaces coll_cache_lib/cuda/cache_hashtable.cuh:741-835).  counts has G+1 entries
// (index G = host keys, which are not listed).
void classify_keys(const Placement& p, int reader, uint64_t num_total_item,
                   std::vector<uint32_t> keys_by_src[], uint64_t* counts);

// Rule of the reference for choosing the direct-index table over the probing one
// (coll_cache_lib/cache_context.cu:2489-2497 with cuda/cache_hashtable.cu:222-225).
bool reference_prefers_flat_table(uint64_t cached_plus_remote, uint64_t num_total_item);

// Rows of one GPU's cache slice (coll_cache_lib/cache_context.cu:2473).
uint64_t cache_capacity_rows(uint64_t num_total_item, double cache_fraction);

}  // namespace ugc
