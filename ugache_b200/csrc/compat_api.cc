// The reference's extern "C" entry points (python/collcache/common/operation.h:29-59) on top
// of the ugc_* C ABI.  Host code only: process-wide configuration, the fork-shared control
// block (barrier, peer handles), hotness counters and placement exchange through POSIX shared
// memory, and the per-step profile log.  No kernel is launched from this file.
#include <cuda_runtime.h>
#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <sys/wait.h>
#include <unistd.h>

#include <algorithm>
#include <atomic>
#include <chrono>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <map>
#include <mutex>
#include <numeric>
#include <parallel/algorithm>
#include <string>
#include <thread>
#include <vector>

#include "../../include/coll_cache_api.h"

namespace {

constexpr int kMaxReplica = UGC_MAX_DEVICE;
constexpr int kNumLogItems = 64;  // the reference has 54 step items (profiler.h:58-120)
constexpr int kLogL1FeatureBytes = 9, kLogL1MissBytes = 13, kLogL1RemoteBytes = 14;
constexpr int kLogL2CacheCopyTime = 27;
// per-phase times of one extraction (profiler.h:111-117; logged by the reference at
// coll_cache_lib/cache_context.cu:1662-1679)
constexpr int kLogL3CacheGetIndexTime = 46, kLogL3CacheCombineMissTime = 50,
              kLogL3CacheCombineCacheTime = 51, kLogL3CacheCombineRemoteTime = 52;

// ---- state shared by all replicas' processes ----------------------------------------------
struct Barrier {
  std::atomic<uint32_t> count;
  std::atomic<uint32_t> gen;
};
struct Control {
  std::atomic<uint32_t> ready;
  std::atomic<uint32_t> failed;  // some replica gave up: waits return at once
  Barrier bar, refresh_bar;
  int64_t owner_pid;
  int32_t num_worker;
  int32_t placement_blocks;
  uint32_t placement_epoch;
  uint32_t max_num_keys[kMaxReplica];
  uint32_t recorded[kMaxReplica];
  ugc_peer_handle handles[kMaxReplica];
};

Control* g_ctl = nullptr;
std::string g_session;  // shm name prefix

double barrier_timeout_s() {
  const char* e = getenv("UGC_BARRIER_TIMEOUT_S");
  return e ? atof(e) : 600.0;
}

// Sense-reversing barrier with a deadline (the reference's spin barrier has none,
// coll_cache_lib/atomic_barrier.h:15-24): a missing replica becomes UGC_ERR_TIMEOUT.
int barrier_wait(Barrier* b) {
  const uint32_t n = (uint32_t)g_ctl->num_worker;
  if (n <= 1) return UGC_OK;
  const uint32_t gen = b->gen.load(std::memory_order_acquire);
  if (b->count.fetch_add(1, std::memory_order_acq_rel) + 1 == n) {
    b->count.store(0, std::memory_order_relaxed);
    b->gen.fetch_add(1, std::memory_order_acq_rel);
    return UGC_OK;
  }
  const auto t0 = std::chrono::steady_clock::now();
  const double limit = barrier_timeout_s();
  while (b->gen.load(std::memory_order_acquire) == gen) {
    if (g_ctl->failed.load(std::memory_order_acquire)) return UGC_ERR_STATE;
    std::this_thread::sleep_for(std::chrono::microseconds(50));
    if (std::chrono::duration<double>(std::chrono::steady_clock::now() - t0).count() > limit) {
      g_ctl->failed.store(1, std::memory_order_release);
      return UGC_ERR_TIMEOUT;
    }
  }
  return UGC_OK;
}

void* shm_map(const std::string& name, size_t bytes, bool create, bool* created = nullptr) {
  int fd = -1;
  if (create) {
    fd = shm_open(name.c_str(), O_CREAT | O_EXCL | O_RDWR, 0600);
    if (created) *created = fd >= 0;
    if (fd < 0) fd = shm_open(name.c_str(), O_RDWR, 0600);
    if (fd >= 0 && ftruncate(fd, (off_t)bytes) != 0) {
      close(fd);
      return nullptr;
    }
  } else {
    fd = shm_open(name.c_str(), O_RDWR, 0600);
  }
  if (fd < 0) return nullptr;
  void* p = mmap(nullptr, bytes, PROT_READ | PROT_WRITE, MAP_SHARED, fd, 0);
  close(fd);
  return p == MAP_FAILED ? nullptr : p;
}

// Created when the library is loaded, so that processes forked afterwards share it.
struct ControlInit {
  ControlInit() {
    const char* session = getenv("UGC_SESSION");
    char buf[128];
    if (session && *session) {
      snprintf(buf, sizeof(buf), "/ugc_%d_%s", (int)getuid(), session);
      g_session = buf;
      bool created = false;
      g_ctl = static_cast<Control*>(shm_map(g_session + "_ctl", sizeof(Control), true, &created));
      if (g_ctl && created) {
        g_ctl->owner_pid = getpid();
        g_ctl->ready.store(1, std::memory_order_release);
      }
    } else {
      snprintf(buf, sizeof(buf), "/ugc_%d_%d", (int)getuid(), (int)getpid());
      g_session = buf;
      void* p = mmap(nullptr, sizeof(Control), PROT_READ | PROT_WRITE, MAP_SHARED | MAP_ANONYMOUS, -1, 0);
      g_ctl = p == MAP_FAILED ? nullptr : static_cast<Control*>(p);
      if (g_ctl) {
        g_ctl->owner_pid = getpid();
        g_ctl->ready.store(1, std::memory_order_release);
      }
    }
  }
};
ControlInit g_control_init;

// ---- per-process state --------------------------------------------------------------------
struct Config {
  bool configured = false;
  double cache_percentage = 0;
  int policy = UGC_POLICY_INTUITIVE;
  int num_device = 1;
  size_t num_global_step_per_epoch = 1, num_epoch = 1, num_total_item = 0;
  int omp_thread_num = 0;
};
Config g_cfg;
std::mutex g_mu;
ugc_ctx* g_ctx = nullptr;
bool g_placement_set = false;
uint32_t g_row_bytes = 0;
void* g_cpu_data = nullptr;
uint32_t* g_freq[kMaxReplica] = {nullptr};
uint64_t g_steps[kMaxReplica] = {0};
std::vector<std::string> g_shm_names;

struct StepLog {
  double val[kNumLogItems];
  bool set[kNumLogItems];
};
std::map<uint64_t, StepLog> g_log;
std::mutex g_log_mu;

thread_local std::string g_err;
int fail(int code, const std::string& msg) {
  g_err = msg;
  fprintf(stderr, "[coll_cache] error: %s\n", msg.c_str());
  if (g_ctl && code != UGC_ERR_INVALID) g_ctl->failed.store(1, std::memory_order_release);
  return code;
}
int pass(int rc, const char* what) {
  if (rc == UGC_OK) return rc;
  return fail(rc, std::string(what) + ": " + ugc_last_error());
}

// An error return out of a call that every replica makes together (init, refresh): the other
// replicas are, or soon will be, waiting at a barrier for this one, so whatever the error
// code, they are told at once instead of waiting for the barrier's time limit.
int collective(int rc) {
  if (rc != UGC_OK && g_ctl) g_ctl->failed.store(1, std::memory_order_release);
  return rc;
}

int g_device_map[kMaxReplica] = {-1, -1, -1, -1, -1, -1, -1, -1};

int device_of(int replica) {
  if (replica >= 0 && replica < kMaxReplica && g_device_map[replica] >= 0) return g_device_map[replica];
  // The reference maps replica i to device i (operation.cc:84-86); UGC_DEVICE_MAP="a,b,..."
  // overrides it (several replicas may share a device, e.g. on a one-GPU test box).
  const char* e = getenv("UGC_DEVICE_MAP");
  if (e && *e) {
    std::vector<int> v;
    const char* p = e;
    while (*p) {
      v.push_back(atoi(p));
      const char* c = strchr(p, ',');
      if (!c) break;
      p = c + 1;
    }
    if (replica < (int)v.size()) return v[replica];
  }
  return replica;
}

size_t elem_bytes(int dtype) {
  switch (dtype) {
    case 0: return 4;
    case 1: return 8;
    case 2: return 2;
    case 3: return 1;
    case 4: return 4;
    case 5: return 1;
    case 6: return 8;
    case 7: return 16;
    case 8: return 32;
    default: return 0;
  }
}

std::string freq_name(int r) { return g_session + "_freq_" + std::to_string(r); }
std::string place_name(uint32_t epoch) { return g_session + "_place_" + std::to_string(epoch); }

size_t place_bytes(size_t N, int G) {
  const int B = G + 2;
  return 64 + N * 4 + (size_t)B + (size_t)G * B + (size_t)B * 8 + 64;
}
struct PlaceView {
  int32_t* num_block;
  uint32_t* nid_to_block;
  uint8_t* block_placement;
  uint8_t* access;
  double* density;
};
PlaceView place_view(void* base, size_t N, int G) {
  const int B = G + 2;
  char* p = static_cast<char*>(base);
  PlaceView v;
  v.num_block = reinterpret_cast<int32_t*>(p);
  v.nid_to_block = reinterpret_cast<uint32_t*>(p + 64);
  char* q = p + 64 + N * 4;
  v.density = reinterpret_cast<double*>(q + ((8 - ((uintptr_t)q & 7)) & 7));
  char* r = reinterpret_cast<char*>(v.density + B);
  v.block_placement = reinterpret_cast<uint8_t*>(r);
  v.access = reinterpret_cast<uint8_t*>(r + B);
  return v;
}

// Replica 0: hotness of all replicas -> ids by descending frequency -> placement arrays in
// shared memory.  Replaces FreqRecorder::GlobalCombine/Sort (coll_cache_lib/freq_recorder.cc:207-274)
// and CollCache::solve_impl_master (coll_cache_lib/facade.cc:93-236) for the non-MILP policies.
int solve_to_shm(uint32_t epoch) {
  const size_t N = g_cfg.num_total_item;
  const int G = g_cfg.num_device;
  std::vector<uint32_t> total(N, 0);
  bool any = false;
  for (int r = 0; r < G; r++) {
    if (!g_ctl->recorded[r]) continue;
    uint32_t* f = g_freq[r];
    bool mapped_here = false;
    if (!f) {
      f = static_cast<uint32_t*>(shm_map(freq_name(r), N * 4, false));
      mapped_here = true;
    }
    if (!f) continue;
    any = true;
#pragma omp parallel for
    for (int64_t k = 0; k < (int64_t)N; k++) total[k] += f[k];
    if (mapped_here) munmap(f, N * 4);
  }
  std::vector<uint32_t> ids(N);
  std::iota(ids.begin(), ids.end(), 0u);
  if (any) {
    __gnu_parallel::stable_sort(ids.begin(), ids.end(),
                                [&](uint32_t a, uint32_t b) { return total[a] > total[b]; });
  }
  std::vector<uint32_t> freqs(N);
#pragma omp parallel for
  for (int64_t i = 0; i < (int64_t)N; i++) freqs[i] = total[ids[i]];
  void* base = shm_map(place_name(epoch), place_bytes(N, G), true);
  if (!base) return fail(UGC_ERR_NOMEM, "cannot create the placement segment in shared memory");
  PlaceView v = place_view(base, N, G);
  double tl, tr, tc;
  ugc_link_model(G, &tl, &tr, &tc);
  int nb = 0;
  int rc = ugc_solve_placement(g_cfg.policy, G, N, ids.data(), freqs.data(), g_cfg.cache_percentage * 100.0,
                               tl, tr, tc, v.nid_to_block, v.block_placement, v.access, v.density, &nb);
  if (rc != UGC_OK) return pass(rc, "ugc_solve_placement");
  // ugc_solve_placement packs block_access_from with stride nb; keep that stride.
  *v.num_block = nb;
  g_ctl->placement_blocks = nb;
  munmap(base, place_bytes(N, G));
  std::lock_guard<std::mutex> lock(g_mu);
  g_shm_names.push_back(place_name(epoch));
  return UGC_OK;
}

int open_placement(uint32_t epoch, void** base_out, PlaceView* v) {
  const size_t N = g_cfg.num_total_item;
  void* base = shm_map(place_name(epoch), place_bytes(N, g_cfg.num_device), false);
  if (!base) return fail(UGC_ERR_STATE, "cannot open the placement segment");
  *v = place_view(base, N, g_cfg.num_device);
  *base_out = base;
  return UGC_OK;
}

}  // namespace

extern "C" {

int coll_cache_config(const char** keys, const char** values, size_t n) {
  if (!g_ctl) return fail(UGC_ERR_STATE, "shared control block could not be created");
  std::map<std::string, std::string> m;
  for (size_t i = 0; i < n; i++) m[keys[i]] = values[i];
  for (const char* need : {"cache_percentage", "_cache_policy", "num_device", "num_global_step_per_epoch",
                           "num_epoch", "num_total_item", "omp_thread_num"})
    if (!m.count(need)) return fail(UGC_ERR_INVALID, std::string("config key missing: ") + need);
  std::lock_guard<std::mutex> lock(g_mu);
  g_cfg.cache_percentage = atof(m["cache_percentage"].c_str());
  int pol = atoi(m["_cache_policy"].c_str());
  // the MILP policies have no solver here: the split search stands in for them
  if (pol == 8 || pol == 13 || pol == 18) pol = UGC_POLICY_SPLIT_SEARCH;
  if (pol != UGC_POLICY_INTUITIVE && pol != UGC_POLICY_REP && pol != UGC_POLICY_CLIQUE_PART &&
      pol != UGC_POLICY_SPLIT_SEARCH)
    return fail(UGC_ERR_UNSUPPORTED, "cache policy " + m["_cache_policy"] + " is not supported");
  g_cfg.policy = pol;
  g_cfg.num_device = atoi(m["num_device"].c_str());
  g_cfg.num_global_step_per_epoch = strtoull(m["num_global_step_per_epoch"].c_str(), nullptr, 10);
  g_cfg.num_epoch = strtoull(m["num_epoch"].c_str(), nullptr, 10);
  g_cfg.num_total_item = strtoull(m["num_total_item"].c_str(), nullptr, 10);
  g_cfg.omp_thread_num = atoi(m["omp_thread_num"].c_str());
  if (g_cfg.num_device < 1 || g_cfg.num_device > kMaxReplica) return fail(UGC_ERR_INVALID, "num_device must be 1..8");
  if (g_cfg.num_total_item == 0) return fail(UGC_ERR_INVALID, "num_total_item must be positive");
  g_cfg.configured = true;
  g_ctl->num_worker = g_cfg.num_device;
  return UGC_OK;
}

size_t coll_cache_num_epoch(void) { return g_cfg.num_epoch; }

int coll_cache_log_step_by_key(uint64_t key, int item, double val) {
  if (item < 0 || item >= kNumLogItems) return fail(UGC_ERR_INVALID, "log item out of range");
  std::lock_guard<std::mutex> lock(g_log_mu);
  StepLog& s = g_log[key];
  s.val[item] = val;
  s.set[item] = true;
  return UGC_OK;
}

int coll_cache_report_step_by_key(uint64_t key) {
  std::lock_guard<std::mutex> lock(g_log_mu);
  auto it = g_log.find(key);
  if (it == g_log.end()) return UGC_OK;
  printf("[Step %llu]", (unsigned long long)key);
  for (int i = 0; i < kNumLogItems; i++)
    if (it->second.set[i]) printf(" item%d=%.6g", i, it->second.val[i]);
  printf("\n");
  fflush(stdout);
  return UGC_OK;
}

int coll_cache_report_step_average_by_key(uint64_t) {
  std::lock_guard<std::mutex> lock(g_log_mu);
  double sum[kNumLogItems] = {0};
  size_t cnt[kNumLogItems] = {0};
  std::vector<double> copy_times;
  for (auto& kv : g_log)
    for (int i = 0; i < kNumLogItems; i++)
      if (kv.second.set[i]) {
        sum[i] += kv.second.val[i];
        cnt[i]++;
        if (i == kLogL2CacheCopyTime) copy_times.push_back(kv.second.val[i]);
      }
  printf("[Step(average)]");
  for (int i = 0; i < kNumLogItems; i++)
    if (cnt[i]) printf(" item%d=%.6g", i, sum[i] / cnt[i]);
  printf("\n");
  if (!copy_times.empty()) {
    std::sort(copy_times.begin(), copy_times.end());
    auto pct = [&](double p) { return copy_times[std::min(copy_times.size() - 1, (size_t)(p * copy_times.size()))]; };
    printf("    tail_logl2featcopy p50=%.6g p90=%.6g p99=%.6g\n", pct(0.5), pct(0.9), pct(0.99));
  }
  fflush(stdout);
  return UGC_OK;
}

int coll_cache_train_barrier(void) {
  if (!g_ctl) return fail(UGC_ERR_STATE, "not configured");
  int rc = barrier_wait(&g_ctl->bar);
  return rc == UGC_OK ? rc : fail(rc, "barrier did not complete");
}

int coll_cache_wait_one_child(void) {
  int st = 0;
  pid_t pid = waitpid(-1, &st, 0);
  if (pid < 0) return 1;
  if (WIFSIGNALED(st) || (WIFEXITED(st) && WEXITSTATUS(st) != 0)) {
    fprintf(stderr, "[coll_cache] child %d ended abnormally\n", (int)pid);
    if (g_ctl) g_ctl->failed.store(1, std::memory_order_release);
    return 1;
  }
  return 0;
}

int coll_cache_print_memory_usage(void) {
  size_t free_b = 0, total_b = 0;
  if (cudaMemGetInfo(&free_b, &total_b) != cudaSuccess) {
    cudaGetLastError();
    return fail(UGC_ERR_CUDA, "cudaMemGetInfo failed");
  }
  printf("[CUDA] cuda: usage: %.2f GB\n", (double)(total_b - free_b) / (1024.0 * 1024.0 * 1024.0));
  fflush(stdout);
  return UGC_OK;
}

int coll_cache_record_init(int replica_id) {
  if (!g_cfg.configured) return fail(UGC_ERR_STATE, "coll_cache_config has not been called");
  if (replica_id < 0 || replica_id >= g_cfg.num_device) return fail(UGC_ERR_INVALID, "bad replica id");
  const size_t N = g_cfg.num_total_item;
  bool created = false;
  void* p = shm_map(freq_name(replica_id), N * 4, true, &created);
  if (!p) return fail(UGC_ERR_NOMEM, "cannot create the hotness segment in shared memory");
  if (created) memset(p, 0, N * 4);
  std::lock_guard<std::mutex> lock(g_mu);
  g_freq[replica_id] = static_cast<uint32_t*>(p);
  g_shm_names.push_back(freq_name(replica_id));
  g_ctl->recorded[replica_id] = 1;
  return UGC_OK;
}

int coll_cache_record(int replica_id, uint32_t* key, size_t n) {
  if (replica_id < 0 || replica_id >= kMaxReplica || !g_freq[replica_id])
    return fail(UGC_ERR_STATE, "coll_cache_record_init has not been called for this replica");
  uint32_t* f = g_freq[replica_id];
  const size_t N = g_cfg.num_total_item;
  for (size_t i = 0; i < n; i++)
    if (key[i] < N) f[key[i]]++;
  if (n > g_ctl->max_num_keys[replica_id]) g_ctl->max_num_keys[replica_id] = (uint32_t)n;
  return UGC_OK;
}

int coll_cache_init_c(int replica_id, size_t key_space_size, ugc_alloc_fn alloc, ugc_free_fn free_fn,
                      void* alloc_user, void* cpu_data, int dtype, size_t dim, double cache_percentage,
                      void* stream) {
  if (!g_cfg.configured) return collective(fail(UGC_ERR_STATE, "coll_cache_config has not been called"));
  if (replica_id < 0 || replica_id >= g_cfg.num_device) return collective(fail(UGC_ERR_INVALID, "bad replica id"));
  if (key_space_size != g_cfg.num_total_item)
    return collective(fail(UGC_ERR_INVALID, "key_space_size differs from the configured num_total_item"));
  const size_t eb = elem_bytes(dtype);
  if (!eb || !dim) return collective(fail(UGC_ERR_INVALID, "bad dtype / dim"));
  const int G = g_cfg.num_device;
  int rc;
  if ((rc = barrier_wait(&g_ctl->bar)) != UGC_OK) return collective(fail(rc, "replicas did not all reach init"));
  if (replica_id == 0) {
    g_ctl->placement_epoch = 1;
    if ((rc = solve_to_shm(1)) != UGC_OK) return collective(rc);
  }
  if ((rc = barrier_wait(&g_ctl->bar)) != UGC_OK) return collective(fail(rc, "placement was not published"));
  {
    std::lock_guard<std::mutex> lock(g_mu);
    if (!g_ctx) {
      ugc_config cfg;
      ugc_config_default(&cfg);
      cfg.num_device = G;
      cfg.num_total_item = key_space_size;
      cfg.row_bytes = (uint32_t)(dim * eb);
      cfg.cache_percentage = cache_percentage;
      uint32_t mb = 0;
      for (int r = 0; r < G; r++) mb = std::max(mb, g_ctl->max_num_keys[r]);
      cfg.max_batch = std::max<uint32_t>((uint32_t)(mb * 1.05), 1u << 16);
      const char* ef = getenv("SAMGRAPH_EMPTY_FEAT");
      cfg.empty_feat = ef ? atoi(ef) : 0;
      cfg.alloc = alloc;
      cfg.free = free_fn;
      cfg.alloc_user = alloc_user;
      if ((rc = ugc_create(&cfg, &g_ctx)) != UGC_OK) return collective(pass(rc, "ugc_create"));
      g_row_bytes = cfg.row_bytes;
      g_cpu_data = cpu_data;
    }
    if (!g_placement_set) {
      void* base;
      PlaceView v;
      if ((rc = open_placement(1, &base, &v)) != UGC_OK) return collective(rc);
      rc = ugc_set_placement(g_ctx, v.nid_to_block, v.block_placement, v.access, v.density, *v.num_block);
      munmap(base, place_bytes(key_space_size, G));
      if (rc != UGC_OK) return collective(pass(rc, "ugc_set_placement"));
      g_placement_set = true;
    }
  }
  if ((rc = ugc_build(g_ctx, replica_id, device_of(replica_id), cpu_data, stream)) != UGC_OK)
    return collective(pass(rc, "ugc_build"));
  if ((rc = ugc_export(g_ctx, replica_id, &g_ctl->handles[replica_id])) != UGC_OK) return collective(pass(rc, "ugc_export"));
  if ((rc = barrier_wait(&g_ctl->bar)) != UGC_OK) return collective(fail(rc, "peers did not publish their handles"));
  for (int r = 0; r < G; r++) {
    if (r == replica_id) continue;
    ugc_peer_handle h = g_ctl->handles[r];
    if ((rc = ugc_import_peer(g_ctx, replica_id, &h)) != UGC_OK) return collective(pass(rc, "ugc_import_peer"));
  }
  if ((rc = ugc_attach_peers(g_ctx, replica_id, stream)) != UGC_OK) return collective(pass(rc, "ugc_attach_peers"));
  if ((rc = barrier_wait(&g_ctl->bar)) != UGC_OK) return collective(fail(rc, "peers did not finish attaching"));
  return UGC_OK;
}

int coll_cache_lookup(int replica_id, uint32_t* key, size_t num_keys, void* output, void* stream) {
  if (!g_ctx) return fail(UGC_ERR_STATE, "coll_cache_init has not run");
  const auto t0 = std::chrono::steady_clock::now();
  ugc_stats_t st;
  int rc = ugc_lookup_u32(g_ctx, replica_id, key, num_keys, output, stream);
  if (rc == UGC_ERR_INVALID && num_keys) {  // a larger batch than any seen while recording
    if ((rc = ugc_reserve_batch(g_ctx, replica_id, (uint32_t)(num_keys * 1.05) + 8)) != UGC_OK)
      return pass(rc, "ugc_reserve_batch");
    rc = ugc_lookup_u32(g_ctx, replica_id, key, num_keys, output, stream);
  }
  if (rc != UGC_OK) return pass(rc, "ugc_lookup_u32");
  if (cudaStreamSynchronize(static_cast<cudaStream_t>(stream)) != cudaSuccess)
    return fail(UGC_ERR_CUDA, std::string("stream synchronise failed: ") + cudaGetErrorString(cudaGetLastError()));
  const double dt = std::chrono::duration<double>(std::chrono::steady_clock::now() - t0).count();
  // step key as the reference forms it (operation.cc:233-234)
  const uint64_t step_key = g_steps[replica_id] * (uint64_t)g_cfg.num_device + (uint64_t)replica_id;
  g_steps[replica_id]++;
  coll_cache_log_step_by_key(step_key, kLogL2CacheCopyTime, dt);
  if (ugc_stats(g_ctx, replica_id, &st) == UGC_OK) {
    coll_cache_log_step_by_key(step_key, kLogL1FeatureBytes, (double)num_keys * g_row_bytes);
    coll_cache_log_step_by_key(step_key, kLogL1MissBytes, (double)st.last_host * g_row_bytes);
    coll_cache_log_step_by_key(step_key, kLogL1RemoteBytes, (double)st.last_remote * g_row_bytes);
    coll_cache_log_step_by_key(step_key, kLogL3CacheGetIndexTime, st.last_index_ns * 1e-9);
    coll_cache_log_step_by_key(step_key, kLogL3CacheCombineMissTime, st.last_host_ns * 1e-9);
    coll_cache_log_step_by_key(step_key, kLogL3CacheCombineRemoteTime, st.last_remote_ns * 1e-9);
    coll_cache_log_step_by_key(step_key, kLogL3CacheCombineCacheTime, st.last_local_ns * 1e-9);
  }
  return UGC_OK;
}

int coll_cache_refresh(int replica_id, void* stream) {
  if (!g_ctx) return collective(fail(UGC_ERR_STATE, "coll_cache_init has not run"));
  const int G = g_cfg.num_device;
  int rc;
  Barrier* b = &g_ctl->refresh_bar;
  if ((rc = barrier_wait(b)) != UGC_OK) return collective(fail(rc, "replicas did not all reach refresh"));
  if (replica_id == 0) {
    g_ctl->placement_epoch++;
    if ((rc = solve_to_shm(g_ctl->placement_epoch)) != UGC_OK) return collective(rc);
  }
  if ((rc = barrier_wait(b)) != UGC_OK) return collective(fail(rc, "new placement was not published"));
  static std::mutex once_mu;
  static uint32_t loaded_epoch = 1, committed_epoch = 1;
  const uint32_t epoch = g_ctl->placement_epoch;
  {
    std::lock_guard<std::mutex> lock(once_mu);
    if (loaded_epoch != epoch) {
      void* base;
      PlaceView v;
      if ((rc = open_placement(epoch, &base, &v)) != UGC_OK) return collective(rc);
      rc = ugc_refresh_set_placement(g_ctx, v.nid_to_block, v.block_placement, v.access, v.density, *v.num_block);
      munmap(base, place_bytes(g_cfg.num_total_item, G));
      if (rc != UGC_OK) return collective(pass(rc, "ugc_refresh_set_placement"));
      loaded_epoch = epoch;
    }
  }
  if ((rc = ugc_refresh_evict(g_ctx, replica_id, stream)) != UGC_OK) return collective(pass(rc, "ugc_refresh_evict"));
  if ((rc = barrier_wait(b)) != UGC_OK) return collective(fail(rc, "refresh: evict phase incomplete"));
  if ((rc = ugc_refresh_fill(g_ctx, replica_id, stream)) != UGC_OK) return collective(pass(rc, "ugc_refresh_fill"));
  if ((rc = barrier_wait(b)) != UGC_OK) return collective(fail(rc, "refresh: fill phase incomplete"));
  if ((rc = ugc_refresh_attach(g_ctx, replica_id, stream)) != UGC_OK) return collective(pass(rc, "ugc_refresh_attach"));
  if ((rc = barrier_wait(b)) != UGC_OK) return collective(fail(rc, "refresh: attach phase incomplete"));
  {
    // every replica of every process has finished its phases: the first caller in this
    // process makes the new placement current
    std::lock_guard<std::mutex> lock(once_mu);
    if (committed_epoch != epoch) {
      if ((rc = ugc_refresh_commit(g_ctx)) != UGC_OK) return collective(pass(rc, "ugc_refresh_commit"));
      committed_epoch = epoch;
    }
  }
  if ((rc = barrier_wait(b)) != UGC_OK) return collective(fail(rc, "refresh: commit incomplete"));
  return UGC_OK;
}

int coll_cache_set_device(int replica_id, int device_id) {
  if (replica_id < 0 || replica_id >= kMaxReplica || device_id < 0) return fail(UGC_ERR_INVALID, "bad replica / device id");
  g_device_map[replica_id] = device_id;
  return UGC_OK;
}

ugc_ctx* coll_cache_context(void) { return g_ctx; }

int coll_cache_shutdown(void) {
  std::lock_guard<std::mutex> lock(g_mu);
  if (g_ctx) {
    ugc_destroy(g_ctx);
    g_ctx = nullptr;
  }
  const size_t N = g_cfg.num_total_item;
  for (int r = 0; r < kMaxReplica; r++)
    if (g_freq[r]) {
      munmap(g_freq[r], N * 4);
      g_freq[r] = nullptr;
    }
  for (auto& n : g_shm_names) shm_unlink(n.c_str());
  g_shm_names.clear();
  g_placement_set = false;
  g_cfg = Config{};
  for (auto& s : g_steps) s = 0;
  {
    std::lock_guard<std::mutex> l2(g_log_mu);
    g_log.clear();
  }
  if (g_ctl) {
    // keep the mapping (forked children may still hold it); reset what a new session reads
    g_ctl->failed.store(0);
    g_ctl->bar.count.store(0);
    g_ctl->refresh_bar.count.store(0);
    memset(g_ctl->max_num_keys, 0, sizeof(g_ctl->max_num_keys));
    memset(g_ctl->recorded, 0, sizeof(g_ctl->recorded));
  }
  return UGC_OK;
}

}  // extern "C"
