// C ABI of the extraction path: context, build, peer exchange, lookup, refresh, stats.
// Host runtime in C++; device work in kernels.cu.  Nothing here throws across the ABI or
// aborts: every entry point returns a ugc_status and records a per-thread message.
#include <cuda.h>
#include <cuda_runtime.h>
#include <omp.h>
#include <sys/socket.h>
#include <sys/time.h>
#include <sys/un.h>
#include <sys/syscall.h>
#include <unistd.h>

#include <algorithm>
#include <cerrno>
#include <cstdarg>
#include <cstddef>
#include <cstdio>
#include <cstring>
#include <map>
#include <mutex>
#include <new>
#include <set>
#include <string>
#include <thread>
#include <vector>

#include "../../include/ugache_b200.h"
#include "device_types.h"
#include "kernels.cuh"
#include "placement.h"

using namespace ugc;

namespace {

thread_local std::string g_last_error;

int fail(int code, const char* fmt, ...) {
  char buf[1024];
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(buf, sizeof(buf), fmt, ap);
  va_end(ap);
  g_last_error = buf;
  return code;
}

#define UGC_CUDA(expr)                                                                        \
  do {                                                                                        \
    cudaError_t e__ = (expr);                                                                 \
    if (e__ != cudaSuccess)                                                                   \
      return fail(UGC_ERR_CUDA, "%s failed: %s (%s:%d)", #expr, cudaGetErrorString(e__),     \
                  __FILE__, __LINE__);                                                        \
  } while (0)

#define UGC_TRY(expr)              \
  do {                             \
    int rc__ = (expr);             \
    if (rc__ != UGC_OK) return rc__; \
  } while (0)

size_t round_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

uint64_t pow2_ceil(uint64_t v) {
  uint64_t p = 1;
  while (p < v) p <<= 1;
  return p;
}

}  // namespace

// Host tables allocated through the virtual-memory API at a host NUMA location come in
// 2 MiB physical chunks, which the GPU can map with large pages, so random row reads over a
// table of tens of GB need far fewer GPU-side translations than 4 KiB mappings of registered
// memory.  (On the machines measured so far the host-row rate came out the same either way:
// the limit sat on the far side of PCIe.)  The driver entry points are resolved at run time
// so that the library still loads on a machine without a driver.
namespace {
struct VmmApi {
  CUresult (*create)(CUmemGenericAllocationHandle*, size_t, const CUmemAllocationProp*, unsigned long long) = nullptr;
  CUresult (*release)(CUmemGenericAllocationHandle) = nullptr;
  CUresult (*reserve)(CUdeviceptr*, size_t, size_t, CUdeviceptr, unsigned long long) = nullptr;
  CUresult (*addr_free)(CUdeviceptr, size_t) = nullptr;
  CUresult (*map)(CUdeviceptr, size_t, size_t, CUmemGenericAllocationHandle, unsigned long long) = nullptr;
  CUresult (*unmap)(CUdeviceptr, size_t) = nullptr;
  CUresult (*set_access)(CUdeviceptr, size_t, const CUmemAccessDesc*, size_t) = nullptr;
  CUresult (*granularity)(size_t*, const CUmemAllocationProp*, CUmemAllocationGranularity_flags) = nullptr;
  CUresult (*export_handle)(void*, CUmemGenericAllocationHandle, CUmemAllocationHandleType, unsigned long long) = nullptr;
  CUresult (*import_handle)(CUmemGenericAllocationHandle*, void*, CUmemAllocationHandleType) = nullptr;
  bool ok = false;
};
struct VmmBlock {
  CUmemGenericAllocationHandle handle;
  size_t size;
};
std::mutex g_vmm_mu;
std::map<void*, VmmBlock> g_vmm_blocks;

template <typename F>
bool resolve(const char* name, F* out) {
  void* fn = nullptr;
  cudaDriverEntryPointQueryResult st;
  if (cudaGetDriverEntryPoint(name, &fn, cudaEnableDefault, &st) != cudaSuccess || !fn ||
      st != cudaDriverEntryPointSuccess) {
    cudaGetLastError();
    return false;
  }
  *out = reinterpret_cast<F>(fn);
  return true;
}

const VmmApi& vmm_api() {
  static VmmApi api = [] {
    VmmApi a;
    a.ok = resolve("cuMemCreate", &a.create) && resolve("cuMemRelease", &a.release) &&
           resolve("cuMemAddressReserve", &a.reserve) && resolve("cuMemAddressFree", &a.addr_free) &&
           resolve("cuMemMap", &a.map) && resolve("cuMemUnmap", &a.unmap) &&
           resolve("cuMemSetAccess", &a.set_access) &&
           resolve("cuMemGetAllocationGranularity", &a.granularity) &&
           resolve("cuMemExportToShareableHandle", &a.export_handle) &&
           resolve("cuMemImportFromShareableHandle", &a.import_handle);
    return a;
  }();
  return api;
}

// Returns nullptr if this route is not available; the caller falls back to cudaHostAlloc.
void* vmm_host_alloc(size_t nbytes, size_t* mapped) {
  const VmmApi& a = vmm_api();
  if (!a.ok) return nullptr;
  int dev = 0, supported = 0, n_dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || cudaGetDeviceCount(&n_dev) != cudaSuccess) return nullptr;
  if (cudaDeviceGetAttribute(&supported, static_cast<cudaDeviceAttr>(141) /* host-NUMA virtual memory management supported */, dev) != cudaSuccess ||
      !supported) {
    cudaGetLastError();
    return nullptr;
  }
  int numa = 0;
  if (cudaDeviceGetAttribute(&numa, cudaDevAttrHostNumaId, dev) != cudaSuccess || numa < 0) {
    cudaGetLastError();
    numa = 0;
  }
  CUmemAllocationProp prop;
  memset(&prop, 0, sizeof(prop));
  prop.type = CU_MEM_ALLOCATION_TYPE_PINNED;
  prop.location.type = CU_MEM_LOCATION_TYPE_HOST_NUMA;
  prop.location.id = numa;
  size_t gran = 0;
  if (a.granularity(&gran, &prop, CU_MEM_ALLOC_GRANULARITY_RECOMMENDED) != CUDA_SUCCESS || !gran) return nullptr;
  const size_t size = (nbytes + gran - 1) / gran * gran;
  CUmemGenericAllocationHandle h;
  if (a.create(&h, size, &prop, 0) != CUDA_SUCCESS) return nullptr;
  CUdeviceptr va = 0;
  if (a.reserve(&va, size, gran, 0, 0) != CUDA_SUCCESS) {
    a.release(h);
    return nullptr;
  }
  if (a.map(va, size, 0, h, 0) != CUDA_SUCCESS) {
    a.addr_free(va, size);
    a.release(h);
    return nullptr;
  }
  std::vector<CUmemAccessDesc> acc;
  for (int d = 0; d < n_dev; d++) {  // every GPU of this process may read the table
    CUmemAccessDesc x;
    memset(&x, 0, sizeof(x));
    x.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
    x.location.id = d;
    x.flags = CU_MEM_ACCESS_FLAGS_PROT_READWRITE;
    acc.push_back(x);
  }
  CUmemAccessDesc hostacc;
  memset(&hostacc, 0, sizeof(hostacc));
  hostacc.location.type = CU_MEM_LOCATION_TYPE_HOST_NUMA;
  hostacc.location.id = numa;
  hostacc.flags = CU_MEM_ACCESS_FLAGS_PROT_READWRITE;
  acc.push_back(hostacc);
  if (a.set_access(va, size, acc.data(), acc.size()) != CUDA_SUCCESS) {
    a.unmap(va, size);
    a.addr_free(va, size);
    a.release(h);
    return nullptr;
  }
  void* p = reinterpret_cast<void*>(va);
  std::lock_guard<std::mutex> lock(g_vmm_mu);
  g_vmm_blocks[p] = VmmBlock{h, size};
  *mapped = size;
  return p;
}

bool vmm_host_free(void* p) {
  VmmBlock b;
  {
    std::lock_guard<std::mutex> lock(g_vmm_mu);
    auto it = g_vmm_blocks.find(p);
    if (it == g_vmm_blocks.end()) return false;
    b = it->second;
    g_vmm_blocks.erase(it);
  }
  const VmmApi& a = vmm_api();
  CUdeviceptr va = reinterpret_cast<CUdeviceptr>(p);
  a.unmap(va, b.size);
  a.addr_free(va, b.size);
  a.release(b.handle);
  return true;
}

// ---- device memory that other processes can map with large pages ---------------------------
// The cache slice and the table are what peers read.  Memory from cudaMalloc can be shared
// with cudaIpc* handles, but the importing process then reads it through a mapping whose
// random-access behaviour was several times slower on the test machines (2000 peer rows cost
// +55 us against +2 us in one process).  Allocations made through the virtual-memory API are
// exported as POSIX file descriptors and mapped by the importer with the same 2 MiB
// granularity as the owner.
struct DevBlock {
  CUmemGenericAllocationHandle handle;
  size_t size;
  int device;
  int fd;         // exported descriptor, -1 until first export
  bool imported;  // mapping of another process' allocation
};
std::map<void*, DevBlock> g_dev_blocks;

bool dev_granularity(int device, size_t* gran, CUmemAllocationProp* prop) {
  memset(prop, 0, sizeof(*prop));
  prop->type = CU_MEM_ALLOCATION_TYPE_PINNED;
  prop->location.type = CU_MEM_LOCATION_TYPE_DEVICE;
  prop->location.id = device;
  prop->requestedHandleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
  return vmm_api().granularity(gran, prop, CU_MEM_ALLOC_GRANULARITY_RECOMMENDED) == CUDA_SUCCESS && *gran;
}

bool dev_set_access(void* p, size_t size, int device) {
  CUmemAccessDesc acc;
  memset(&acc, 0, sizeof(acc));
  acc.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
  acc.location.id = device;
  acc.flags = CU_MEM_ACCESS_FLAGS_PROT_READWRITE;
  return vmm_api().set_access(reinterpret_cast<CUdeviceptr>(p), size, &acc, 1) == CUDA_SUCCESS;
}

// Maps `handle` (size bytes) for `device`; registers the block.  nullptr on failure.
void* dev_map(CUmemGenericAllocationHandle handle, size_t size, size_t gran, int device, bool imported) {
  const VmmApi& a = vmm_api();
  CUdeviceptr va = 0;
  if (a.reserve(&va, size, gran, 0, 0) != CUDA_SUCCESS) return nullptr;
  if (a.map(va, size, 0, handle, 0) != CUDA_SUCCESS) {
    a.addr_free(va, size);
    return nullptr;
  }
  void* p = reinterpret_cast<void*>(va);
  if (!dev_set_access(p, size, device)) {
    a.unmap(va, size);
    a.addr_free(va, size);
    return nullptr;
  }
  std::lock_guard<std::mutex> lock(g_vmm_mu);
  g_dev_blocks[p] = DevBlock{handle, size, device, -1, imported};
  return p;
}

// Shareable device memory on the current device; nullptr if this route is unavailable.
void* dev_shareable_alloc(size_t nbytes) {
  const VmmApi& a = vmm_api();
  if (!a.ok) return nullptr;
  int device = 0;
  if (cudaGetDevice(&device) != cudaSuccess) return nullptr;
  CUmemAllocationProp prop;
  size_t gran = 0;
  if (!dev_granularity(device, &gran, &prop)) return nullptr;
  const size_t size = (nbytes + gran - 1) / gran * gran;
  CUmemGenericAllocationHandle h;
  if (a.create(&h, size, &prop, 0) != CUDA_SUCCESS) return nullptr;
  void* p = dev_map(h, size, gran, device, false);
  if (!p) a.release(h);
  return p;
}

bool dev_block_free(void* p) {
  DevBlock b;
  {
    std::lock_guard<std::mutex> lock(g_vmm_mu);
    auto it = g_dev_blocks.find(p);
    if (it == g_dev_blocks.end()) return false;
    b = it->second;
    g_dev_blocks.erase(it);
  }
  const VmmApi& a = vmm_api();
  CUdeviceptr va = reinterpret_cast<CUdeviceptr>(p);
  a.unmap(va, b.size);
  a.addr_free(va, b.size);
  a.release(b.handle);
  if (b.fd >= 0) close(b.fd);
  return true;
}

bool dev_block_find(void* p, DevBlock* out) {
  std::lock_guard<std::mutex> lock(g_vmm_mu);
  auto it = g_dev_blocks.find(p);
  if (it == g_dev_blocks.end()) return false;
  *out = it->second;
  return true;
}

// File descriptor under which other processes can import the block (created once).
int dev_block_export_fd(void* p) {
  std::lock_guard<std::mutex> lock(g_vmm_mu);
  auto it = g_dev_blocks.find(p);
  if (it == g_dev_blocks.end()) return -1;
  if (it->second.fd < 0) {
    int fd = -1;
    if (vmm_api().export_handle(&fd, it->second.handle, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR, 0) != CUDA_SUCCESS)
      return -1;
    it->second.fd = fd;
  }
  return it->second.fd;
}

// ---- handing exported descriptors to other processes ----------------------------------------
// First choice: the importer duplicates the descriptor straight out of the owner
// (pidfd_open + pidfd_getfd).  Where the kernel's ptrace policy forbids that, the owner serves
// its exported descriptors over an abstract-namespace Unix socket (SCM_RIGHTS), to processes of
// the same user only.
std::set<int> g_served_fds;
bool g_fd_server_running = false;

uint64_t g_fd_token = 0;   // random per process; part of the socket name, carried in the handle
std::string g_fd_server_error;

// Abstract-namespace name: uid, pid and a random token, so that processes in different pid
// namespaces that share a network namespace do not collide and the name cannot be guessed.
void fd_socket_name(int64_t pid, uint64_t token, sockaddr_un* addr, socklen_t* len) {
  memset(addr, 0, sizeof(*addr));
  addr->sun_family = AF_UNIX;
  int n = snprintf(addr->sun_path + 1, sizeof(addr->sun_path) - 1, "ugc_fd_%u_%lld_%016llx",
                   (unsigned)geteuid(), (long long)pid, (unsigned long long)token);
  *len = (socklen_t)(offsetof(sockaddr_un, sun_path) + 1 + n);
}

void set_socket_timeouts(int fd, int seconds) {
  timeval tv;
  tv.tv_sec = seconds;
  tv.tv_usec = 0;
  setsockopt(fd, SOL_SOCKET, SO_RCVTIMEO, &tv, sizeof(tv));
  setsockopt(fd, SOL_SOCKET, SO_SNDTIMEO, &tv, sizeof(tv));
}

void fd_server_loop(int listen_fd) {
  for (;;) {
    int c = accept(listen_fd, nullptr, nullptr);
    if (c < 0) {
      if (errno == EINTR) continue;
      return;
    }
    // only processes of the same user are served (the descriptors give access to the cache memory)
    ucred peer;
    socklen_t peer_len = sizeof(peer);
    if (getsockopt(c, SOL_SOCKET, SO_PEERCRED, &peer, &peer_len) != 0 || peer.uid != geteuid()) {
      close(c);
      continue;
    }
    set_socket_timeouts(c, 2);  // a client that stalls must not block the importers behind it
    int wanted = -1;
    if (read(c, &wanted, sizeof(wanted)) == (ssize_t)sizeof(wanted)) {
      bool ok;
      {
        std::lock_guard<std::mutex> lock(g_vmm_mu);
        ok = g_served_fds.count(wanted) != 0;
      }
      char byte = ok ? 1 : 0;
      msghdr msg;
      memset(&msg, 0, sizeof(msg));
      iovec iov = {&byte, 1};
      msg.msg_iov = &iov;
      msg.msg_iovlen = 1;
      char ctrl[CMSG_SPACE(sizeof(int))];
      if (ok) {
        memset(ctrl, 0, sizeof(ctrl));
        msg.msg_control = ctrl;
        msg.msg_controllen = sizeof(ctrl);
        cmsghdr* cm = CMSG_FIRSTHDR(&msg);
        cm->cmsg_level = SOL_SOCKET;
        cm->cmsg_type = SCM_RIGHTS;
        cm->cmsg_len = CMSG_LEN(sizeof(int));
        memcpy(CMSG_DATA(cm), &wanted, sizeof(int));
      }
      sendmsg(c, &msg, MSG_NOSIGNAL);  // a client that left must not raise SIGPIPE here
    }
    close(c);
  }
}

// Called by the owner when it exports descriptor `fd`.  Returns false (and keeps a message)
// if the descriptor socket could not be set up; the pidfd route may still work then.
bool fd_server_publish(int fd) {
  std::lock_guard<std::mutex> lock(g_vmm_mu);
  g_served_fds.insert(fd);
  if (g_fd_server_running) return true;
  if (g_fd_token == 0) {
    uint64_t t = 0;
    FILE* f = fopen("/dev/urandom", "rb");
    if (f) {
      if (fread(&t, sizeof(t), 1, f) != 1) t = 0;
      fclose(f);
    }
    if (t == 0) t = ((uint64_t)getpid() << 32) ^ (uint64_t)reinterpret_cast<uintptr_t>(&t) ^ 0x9e3779b97f4a7c15ull;
    g_fd_token = t;
  }
  int s = socket(AF_UNIX, SOCK_STREAM | SOCK_CLOEXEC, 0);
  if (s < 0) {
    g_fd_server_error = std::string("descriptor socket: socket() failed: ") + strerror(errno);
    return false;
  }
  sockaddr_un addr;
  socklen_t len;
  fd_socket_name((int64_t)getpid(), g_fd_token, &addr, &len);
  if (bind(s, reinterpret_cast<sockaddr*>(&addr), len) != 0 || listen(s, 16) != 0) {
    g_fd_server_error = std::string("descriptor socket: bind/listen failed: ") + strerror(errno);
    close(s);
    return false;
  }
  g_fd_server_running = true;
  std::thread(fd_server_loop, s).detach();
  return true;
}

int fd_from_socket(int64_t pid, uint64_t token, int fd) {
  int s = socket(AF_UNIX, SOCK_STREAM | SOCK_CLOEXEC, 0);
  if (s < 0) return -1;
  set_socket_timeouts(s, 5);
  sockaddr_un addr;
  socklen_t len;
  fd_socket_name(pid, token, &addr, &len);
  int got = -1;
  if (connect(s, reinterpret_cast<sockaddr*>(&addr), len) == 0 &&
      write(s, &fd, sizeof(fd)) == (ssize_t)sizeof(fd)) {
    char byte = 0;
    msghdr msg;
    memset(&msg, 0, sizeof(msg));
    iovec iov = {&byte, 1};
    msg.msg_iov = &iov;
    msg.msg_iovlen = 1;
    char ctrl[CMSG_SPACE(sizeof(int))];
    memset(ctrl, 0, sizeof(ctrl));
    msg.msg_control = ctrl;
    msg.msg_controllen = sizeof(ctrl);
    if (recvmsg(s, &msg, 0) == 1 && byte == 1) {
      cmsghdr* cm = CMSG_FIRSTHDR(&msg);
      if (cm && cm->cmsg_level == SOL_SOCKET && cm->cmsg_type == SCM_RIGHTS) memcpy(&got, CMSG_DATA(cm), sizeof(int));
    }
  }
  close(s);
  return got;
}

// A duplicate, in this process, of descriptor `fd` of process `pid`: straight out of the owner
// where the kernel's ptrace policy lets this process do that (same user and an unrestricted
// ptrace scope, or a privileged importer), else over the owner's descriptor socket.
int steal_fd(int64_t pid, uint64_t token, int fd) {
  if (!getenv("UGC_NO_PIDFD")) {
#if defined(SYS_pidfd_open) && defined(SYS_pidfd_getfd)
    int pidfd = (int)syscall(SYS_pidfd_open, (pid_t)pid, 0);
    if (pidfd >= 0) {
      int local = (int)syscall(SYS_pidfd_getfd, pidfd, fd, 0);
      close(pidfd);
      if (local >= 0) return local;
    }
#endif
  }
  return fd_from_socket(pid, token, fd);
}

// Maps another process' exported block for `device`.
void* dev_import(int64_t pid, uint64_t token, int fd, size_t size, int device) {
  const VmmApi& a = vmm_api();
  if (!a.ok) return nullptr;
  int local = steal_fd(pid, token, fd);
  if (local < 0) return nullptr;
  CUmemGenericAllocationHandle h;
  CUresult rc = a.import_handle(&h, reinterpret_cast<void*>(static_cast<uintptr_t>(local)),
                                CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR);
  close(local);
  if (rc != CUDA_SUCCESS) return nullptr;
  CUmemAllocationProp prop;
  size_t gran = 0;
  if (!dev_granularity(device, &gran, &prop)) {
    a.release(h);
    return nullptr;
  }
  void* p = dev_map(h, size, gran, device, true);
  if (!p) a.release(h);
  return p;
}
}  // namespace



namespace {

// A device buffer that grows on demand through the context's allocator.
struct DevBuf {
  void* ptr = nullptr;
  size_t bytes = 0;
};

struct Replica {
  bool built = false;
  bool attached = false;
  int id = -1;
  int device = -1;
  int sm_count = 148;
  // cache slice
  void* slice = nullptr;
  uint64_t capacity = 0;
  size_t slice_bytes = 0;
  // table
  TableView table{};
  void* table_mem = nullptr;
  size_t table_bytes = 0;
  uint64_t table_entry_cap = 0;  // hashed: entries the table is sized for
  // sources, as seen from this replica's device
  const void* src_base[kMaxLocation] = {nullptr};
  TableView peer_table[kMaxDevice] = {};
  bool peer_known[kMaxDevice] = {false};
  void* ipc_opened[2 * kMaxDevice] = {nullptr};
  int n_ipc_opened = 0;
  // lookup scratch
  uint64_t* list[kNumGroup] = {nullptr, nullptr, nullptr};
  Counters* counters = nullptr;
  uint32_t max_batch = 0;
  // host-buffer lookups
  DevBuf stage_keys, stage_out;
  // hotness counters (one uint32 per id), allocated on first use
  uint32_t* hot_counts = nullptr;
  // build / refresh staging
  DevBuf stage_a, stage_b;
  // bookkeeping mirrored from the reference's CacheEntryManager
  // (coll_cache_lib/cuda/cache_hashtable.cuh:548-557): keys per source, free slots
  // free cache rows: a ring of slot numbers in device memory, `capacity` entries; evicted rows
  // are appended at the tail, new rows take slots from the head
  // (coll_cache_lib/cuda/cache_hashtable.cuh:637-645 keeps the same order on the host)
  uint32_t* free_ring = nullptr;
  uint64_t free_head = 0, free_count = 0;
  bool static_used = false;                // lookups through the fixed scratch array were issued
  int refresh_fill_ctas = 20;              // grid of the refresh-time fill kernel
  int refresh_fill_batch_rows = 131072;    // rows per launch of it
  int refresh_fill_pause_us = 0;           // host-side pause between two launches
  cudaStream_t fill_stream = nullptr;      // lowest-priority stream the refresh-time fill runs on
  cudaEvent_t fill_ev[2] = {nullptr, nullptr};
  float t_byte[kNumGroup] = {0, 0, 0};     // seconds per byte (any common scale) per source group
  int gather_dynamic = 1;
  int split_fixed = 0;                     // host_ctas / remote_ctas are counts, not caps
  int early_repoint = 1;                   // refresh: re-point keys to a peer that holds them, in place
  int pool_vec_bytes = 0;                  // pooled lookup: 0 = chosen per launch, 16 or 4 forced
  cudaStream_t copy_stream = nullptr;      // host-buffer lookups: rows leave on this stream
  std::vector<cudaEvent_t> copy_events;
  uint32_t* stamp = nullptr;               // deduplicated lookups: one stamp per id (first use)
  uint32_t stamp_epoch = 0;
  uint64_t* host_sorted = nullptr;         // host list in address order (allocated on first use)
  uint32_t* host_hist = nullptr;
  int host_order_min_rows = 8192;
  uint64_t lookups_host_ordered = 0;
  uint32_t direct_slot = 0, last_slot = 0; // count slot of the next / the last direct launch
  bool last_was_direct = false;
  uint32_t last_n = 0, last_seq = 0;
  cudaStream_t recent_streams[4] = {nullptr, nullptr, nullptr, nullptr};  // streams lookups ran on
  bool recent_valid[4] = {false, false, false, false};
  int direct_block = 256;
  int direct_max_host_rows = 8192;
  int direct_tile_shift = 0;               // 0: chosen per launch
  int direct_deep = 0;
  int direct_early_host = 0;               // 0 auto, 1 always, 2 never
  uint64_t n_local = 0;                    // rows stored here
  uint64_t n_remote = 0;                   // keys read from peers
  // Device-resident placement view of this reader and the key lists of the last
  // classification (build: one list per source; refresh: evict / insert / drop / attach).
  uint32_t* n2b_dev = nullptr;             // nid_to_block of the current placement
  uint32_t* n2b_next = nullptr;            // same for the placement a refresh is moving to
  DevBuf acc_dev;                          // [old row | new row] of block_access_from
  DevBuf class_scratch;
  DevBuf lists;                            // all lists back to back
  uint64_t list_count[kMaxClassLists] = {0};
  uint64_t list_base[kMaxClassLists] = {0};
  uint64_t next_n_local = 0;
  bool refresh_open = false;
  uint64_t counts[kMaxLocation] = {0};
  uint64_t lookups = 0;
  int gather_grid = 0;
  int host_ctas = 0, remote_ctas = 0;
  int vec_bytes = 32;
  int block_threads = 256;
  int bulk_mask = 0;
  int lookup_kpt = 1;
  int pdl = 3;  // bit 0: lookup kernel, bit 1: gather kernel launched with programmatic serialization
  // extraction mode: UGC_EXTRACT_AUTO / _GROUPED / _DIRECT; in auto mode the choice follows
  // the host-row share of the last finished lookup, read from the pinned mirror below
  int extract_mode = UGC_EXTRACT_AUTO;
  int direct_grid = 0;
  Feedback* feedback = nullptr;      // pinned host memory, written by the kernels
  Feedback* feedback_dev = nullptr;  // the same memory as the device addresses it
  uint64_t lookups_direct = 0;
  uint64_t kernel_launches = 0;
  uint64_t lookups_pooled = 0;
  int host_zero_copy = 1;  // keys read in place; rows staged (the copy engine beats SM stores over PCIe)
  // per-kernel profiling (three events per lookup)
  std::vector<cudaEvent_t> prof_events;
  size_t prof_used = 0;
  bool prof_on = false;
};

}  // namespace

struct ugc_ctx {
  ugc_config cfg;
  Placement cur, next;
  std::vector<Replica> reps;
  const void* host_table = nullptr;
  const void* host_dev = nullptr;
  bool host_registered_here = false;
  size_t host_registered_bytes = 0;
  std::mutex mu;
  // device memory held now: through the caller's allocator / obtained by the library itself
  // (cudaMalloc or virtual-memory blocks), for ugc_stats
  std::mutex acct_mu;
  std::map<void*, size_t> acct;
  uint64_t bytes_from_allocator = 0, bytes_own = 0;
};

namespace {

void account(ugc_ctx* c, void* p, size_t bytes, bool own) {
  std::lock_guard<std::mutex> lock(c->acct_mu);
  c->acct[p] = bytes;
  (own ? c->bytes_own : c->bytes_from_allocator) += bytes;
}
void unaccount(ugc_ctx* c, void* p, bool own) {
  std::lock_guard<std::mutex> lock(c->acct_mu);
  auto it = c->acct.find(p);
  if (it == c->acct.end()) return;
  (own ? c->bytes_own : c->bytes_from_allocator) -= it->second;
  c->acct.erase(it);
}

void* ctx_alloc(ugc_ctx* c, size_t bytes) {
  bytes = round_up(std::max<size_t>(bytes, 256), 256);
  if (c->cfg.alloc) {
    void* q = c->cfg.alloc(bytes, c->cfg.alloc_user);
    if (q) account(c, q, bytes, false);
    return q;
  }
  void* p = nullptr;
  if (cudaMalloc(&p, bytes) != cudaSuccess) {
    cudaGetLastError();
    return nullptr;
  }
  account(c, p, bytes, true);
  return p;
}
void ctx_free(ugc_ctx* c, void* p) {
  if (!p) return;
  if (c->cfg.free) {
    unaccount(c, p, false);
    c->cfg.free(p, c->cfg.alloc_user);
  } else if (!c->cfg.alloc) {
    unaccount(c, p, true);
    cudaFree(p);
  }
}

// Memory that peers will read (slice, table): shareable large-page blocks when the built-in
// allocator is in use and the driver offers them, the ordinary route otherwise.
void* ctx_alloc_shared(ugc_ctx* c, size_t bytes) {
  if (!c->cfg.alloc && !getenv("UGC_NO_VMM")) {
    void* p = dev_shareable_alloc(std::max<size_t>(bytes, 256));
    if (p) {
      DevBlock b;
      account(c, p, dev_block_find(p, &b) ? b.size : bytes, true);
      return p;
    }
  }
  return ctx_alloc(c, bytes);
}
void ctx_free_shared(ugc_ctx* c, void* p) {
  if (!p) return;
  DevBlock b;
  if (dev_block_find(p, &b)) unaccount(c, p, true);
  if (dev_block_free(p)) return;
  ctx_free(c, p);
}

int ensure(ugc_ctx* c, DevBuf& b, size_t bytes) {
  if (b.bytes >= bytes) return UGC_OK;
  ctx_free(c, b.ptr);
  b.ptr = ctx_alloc(c, bytes);
  b.bytes = b.ptr ? round_up(std::max<size_t>(bytes, 256), 256) : 0;
  if (!b.ptr) return fail(UGC_ERR_NOMEM, "device allocation of %zu bytes failed", bytes);
  return UGC_OK;
}

int get_replica(ugc_ctx* c, int id, bool need_built, Replica** out) {
  if (!c) return fail(UGC_ERR_INVALID, "null context");
  if (id < 0 || id >= c->cfg.num_device)
    return fail(UGC_ERR_INVALID, "replica_id %d outside [0, %d)", id, c->cfg.num_device);
  Replica* r = &c->reps[id];
  if (need_built && !r->built) return fail(UGC_ERR_STATE, "replica %d has not been built", id);
  *out = r;
  return UGC_OK;
}

// Device-visible address of the caller's host table.
int map_host_table(ugc_ctx* c, const void* host_table) {
  if (c->host_table == host_table && c->host_dev) return UGC_OK;
  const uint64_t rows = c->cfg.empty_feat > 0 ? ((uint64_t)1 << c->cfg.empty_feat)
                                               : c->cfg.num_total_item;
  const size_t bytes = (size_t)rows * c->cfg.row_bytes;
  void* dptr = nullptr;
  cudaPointerAttributes attr;
  if (cudaPointerGetAttributes(&attr, host_table) == cudaSuccess && attr.devicePointer &&
      (attr.type == cudaMemoryTypeHost || attr.type == cudaMemoryTypeManaged ||
       attr.type == cudaMemoryTypeDevice)) {
    // already GPU-visible (pinned, registered, or mapped through the virtual-memory API)
    c->host_table = host_table;
    c->host_dev = attr.devicePointer;
    return UGC_OK;
  }
  cudaGetLastError();
  cudaError_t e = cudaHostGetDevicePointer(&dptr, const_cast<void*>(host_table), 0);
  if (e != cudaSuccess) {
    cudaGetLastError();
    if (!c->cfg.register_host)
      return fail(UGC_ERR_INVALID,
                  "host table is not GPU-visible (pin it, or set register_host): %s",
                  cudaGetErrorString(e));
    // The reference registers the table here as well (coll_cache_lib/facade.cc:476).
    UGC_TRY(ugc_host_register(const_cast<void*>(host_table), bytes, &dptr));
    c->host_registered_here = true;
    c->host_registered_bytes = bytes;
  }
  c->host_table = host_table;
  c->host_dev = dptr;
  return UGC_OK;
}

int read_counters(Replica* r, Counters* out) {
  UGC_CUDA(cudaMemcpy(out, r->counters, sizeof(Counters), cudaMemcpyDeviceToHost));
  return UGC_OK;
}

// Synchronises the stream and turns device-side table errors into a status.
int check_table_errors(Replica* r, cudaStream_t s, const char* what) {
  UGC_CUDA(cudaStreamSynchronize(s));
  Counters h;
  UGC_TRY(read_counters(r, &h));
  if (h.err_table)
    return fail(UGC_ERR_TABLE, "%s: %llu table operations failed on replica %d", what,
                (unsigned long long)h.err_table, r->id);
  return UGC_OK;
}

// `entries`: rows the placement maps to GPUs now (drives the reference's flat-vs-probing
// rule); `reserve`: entries the table must be able to hold over its lifetime.
int alloc_table(ugc_ctx* c, Replica* r, uint64_t entries, uint64_t reserve, cudaStream_t s) {
  const uint64_t N = c->cfg.num_total_item;
  int kind = c->cfg.table_kind;
  if (kind == UGC_TABLE_AUTO)
    kind = reference_prefers_flat_table(std::max<uint64_t>(entries, 2), N) ? UGC_TABLE_FLAT
                                                                           : UGC_TABLE_HASHED;
  // a probing table as large as the direct-index one buys nothing
  if (kind == UGC_TABLE_HASHED && c->cfg.table_kind == UGC_TABLE_AUTO &&
      pow2_ceil(std::max<uint64_t>(reserve, 1)) * 16 > N * 4)
    kind = UGC_TABLE_FLAT;
  entries = reserve;
  r->table = TableView{};
  r->table.num_keys = N;
  if (kind == UGC_TABLE_FLAT) {
    r->table.kind = kTableFlat;
    r->table_bytes = round_up((size_t)N * 4, 256);
    r->table_entry_cap = N;
  } else {
    // 4-slot lines; slots = 2 * pow2_ceil(entries): load factor 25..50 %.
    uint64_t lines = std::max<uint64_t>(pow2_ceil(std::max<uint64_t>(entries, 1)) / 2, 64);
    if (lines > (1ull << 31)) return fail(UGC_ERR_UNSUPPORTED, "hashed table too large");
    r->table.kind = kTableHashed;
    r->table.line_mask = (uint32_t)(lines - 1);
    r->table_bytes = (size_t)lines * kSlotsPerLine * sizeof(uint2);
    r->table_entry_cap = lines * 2;
  }
  r->table_mem = ctx_alloc_shared(c, r->table_bytes);
  if (!r->table_mem) return fail(UGC_ERR_NOMEM, "table allocation of %zu bytes failed", r->table_bytes);
  if (r->table.kind == kTableFlat) {
    r->table.flat = static_cast<uint32_t*>(r->table_mem);
  } else {
    r->table.slots = static_cast<uint2*>(r->table_mem);
  }
  UGC_CUDA(launch_table_clear(r->table, s));
  return UGC_OK;
}

// Classifies the whole id space on the GPU (replaces the host OpenMP passes of the reference,
// coll_cache_lib/cuda/cache_hashtable.cuh:693-835).  `old_p` == nullptr: build lists (one per
// GPU source).  Otherwise the refresh lists.  Leaves counts / bases in the replica and the
// keys in r->lists; returns after the stream is idle.
int gpu_classify(ugc_ctx* c, Replica* r, const Placement* old_p, const Placement& new_p,
                 const uint32_t* n2b_old_dev, const uint32_t* n2b_new_dev, cudaStream_t s) {
  const uint64_t N = c->cfg.num_total_item;
  const int G = c->cfg.num_device;
  const size_t row_old = old_p ? (size_t)old_p->num_block : 0, row_new = (size_t)new_p.num_block;
  UGC_TRY(ensure(c, r->acc_dev, row_old + row_new + 16));
  uint8_t* acc = static_cast<uint8_t*>(r->acc_dev.ptr);
  if (old_p)
    UGC_CUDA(cudaMemcpyAsync(acc, &old_p->block_access_from[(size_t)r->id * row_old], row_old,
                             cudaMemcpyHostToDevice, s));
  UGC_CUDA(cudaMemcpyAsync(acc + row_old, &new_p.block_access_from[(size_t)r->id * row_new], row_new,
                           cudaMemcpyHostToDevice, s));
  ClassifyParams p;
  memset(&p, 0, sizeof(p));
  p.n2b_old = old_p ? n2b_old_dev : nullptr;
  p.n2b_new = n2b_new_dev;
  p.acc_old = acc;
  p.acc_new = acc + row_old;
  p.num_keys = N;
  p.me = (uint32_t)r->id;
  p.num_device = (uint32_t)G;
  p.num_lists = old_p ? kListAttach0 + G : G;
  UGC_TRY(ensure(c, r->class_scratch, classify_scratch_bytes(N)));
  UGC_CUDA(launch_classify_count(p, r->class_scratch.ptr, s));
  unsigned long long totals[kMaxClassLists];
  UGC_CUDA(cudaMemcpyAsync(totals, classify_totals(r->class_scratch.ptr, N), sizeof(totals),
                           cudaMemcpyDeviceToHost, s));
  UGC_CUDA(cudaStreamSynchronize(s));
  uint64_t sum = 0;
  for (int l = 0; l < kMaxClassLists; l++) {
    r->list_count[l] = l < p.num_lists ? totals[l] : 0;
    r->list_base[l] = sum;
    p.list_base[l] = sum;
    sum += r->list_count[l];
  }
  UGC_TRY(ensure(c, r->lists, std::max<uint64_t>(sum, 1) * sizeof(uint32_t)));
  UGC_CUDA(launch_classify_scatter(p, r->class_scratch.ptr, static_cast<uint32_t*>(r->lists.ptr), s));
  UGC_CUDA(cudaStreamSynchronize(s));
  return UGC_OK;
}

uint32_t* list_ptr(Replica* r, int l) { return static_cast<uint32_t*>(r->lists.ptr) + r->list_base[l]; }

int upload_n2b(ugc_ctx* c, const Placement& p, uint32_t** dst, cudaStream_t s) {
  const size_t bytes = (size_t)c->cfg.num_total_item * sizeof(uint32_t);
  if (!*dst) {
    *dst = static_cast<uint32_t*>(ctx_alloc(c, bytes));
    if (!*dst) return fail(UGC_ERR_NOMEM, "placement copy (%zu bytes) could not be allocated", bytes);
  }
  UGC_CUDA(cudaMemcpyAsync(*dst, p.nid_to_block.data(), bytes, cudaMemcpyHostToDevice, s));
  return UGC_OK;
}

void release_replica(ugc_ctx* c, Replica* r) {
  if (r->device >= 0) cudaSetDevice(r->device);
  for (cudaEvent_t e : r->prof_events) cudaEventDestroy(e);
  for (cudaEvent_t e : r->copy_events) cudaEventDestroy(e);
  if (r->copy_stream) cudaStreamDestroy(r->copy_stream);
  if (r->fill_stream) {
    cudaStreamDestroy(r->fill_stream);
    cudaEventDestroy(r->fill_ev[0]);
    cudaEventDestroy(r->fill_ev[1]);
  }
  for (int i = 0; i < r->n_ipc_opened; i++)
    if (!dev_block_free(r->ipc_opened[i])) cudaIpcCloseMemHandle(r->ipc_opened[i]);
  ctx_free_shared(c, r->slice);
  ctx_free_shared(c, r->table_mem);
  for (auto& l : r->list) ctx_free(c, l);
  ctx_free(c, r->counters);
  ctx_free(c, r->free_ring);
  ctx_free(c, r->host_sorted);
  ctx_free(c, r->host_hist);
  ctx_free(c, r->stamp);
  ctx_free(c, r->hot_counts);
  ctx_free(c, r->n2b_dev);
  ctx_free(c, r->n2b_next);
  ctx_free(c, r->acc_dev.ptr);
  ctx_free(c, r->class_scratch.ptr);
  ctx_free(c, r->lists.ptr);
  ctx_free(c, r->stage_keys.ptr);
  ctx_free(c, r->stage_out.ptr);
  ctx_free(c, r->stage_a.ptr);
  ctx_free(c, r->stage_b.ptr);
  if (r->feedback) cudaFreeHost(r->feedback);
  *r = Replica{};
}

GatherParams gather_params(ugc_ctx* c, Replica* r, void* out, uint32_t n) {
  GatherParams p{};
  for (int i = 0; i < kMaxLocation; i++) p.src_base[i] = r->src_base[i];
  p.out = out;
  for (int g = 0; g < kNumGroup; g++) p.list[g] = r->list[g];
  p.counters = r->counters;
  p.feedback = r->feedback_dev;
  p.row_bytes = c->cfg.row_bytes;
  p.n_keys = n;
  p.remote_cta_cap = r->remote_ctas;
  p.host_cta_cap = r->host_ctas;
  p.rows_per_cta_min = 32;
  for (int g = 0; g < kNumGroup; g++) p.t_byte[g] = r->t_byte[g];
  p.seq = (uint32_t)r->lookups;
  p.dynamic = r->gather_dynamic;
  p.fixed_split = r->split_fixed;
  p.bulk_mask = r->bulk_mask;
  p.pdl = (r->pdl & 2) ? 1 : 0;
  return p;
}

// Device-side address of pinned host memory that the GPU has mapped, else nullptr.
void* mapped_device_pointer(const void* host) {
  cudaPointerAttributes attr;
  if (cudaPointerGetAttributes(&attr, host) != cudaSuccess) {
    cudaGetLastError();
    return nullptr;
  }
  if (attr.type != cudaMemoryTypeHost || !attr.devicePointer) return nullptr;
  return attr.devicePointer;
}

// The last few streams lookups of this replica were enqueued on (most callers use one).
void remember_stream(Replica* r, cudaStream_t s) {
  for (int i = 0; i < 4; i++)
    if (r->recent_valid[i] && r->recent_streams[i] == s) return;
  for (int i = 3; i > 0; i--) {
    r->recent_streams[i] = r->recent_streams[i - 1];
    r->recent_valid[i] = r->recent_valid[i - 1];
  }
  r->recent_streams[0] = s;
  r->recent_valid[0] = true;
}

// Waits until every lookup of this replica enqueued so far has finished on the GPU: the
// streams those lookups ran on are synchronised, which blocks this host thread only and
// stalls no other stream (the reference waits for the trainer's step counter in the same
// spirit, coll_cache_lib/cache_context.cu:4045-4052).  Falls back to a device-wide wait when
// a stream cannot be waited on (destroyed meanwhile) or lookups went through the fixed scratch
// array, whose streams are not recorded.
int drain_lookups(Replica* r) {
  bool ok = !r->static_used;
  for (int i = 0; ok && i < 4; i++)
    if (r->recent_valid[i] && cudaStreamSynchronize(r->recent_streams[i]) != cudaSuccess) {
      cudaGetLastError();
      r->recent_valid[i] = false;
      ok = false;
    }
  if (!ok) UGC_CUDA(cudaDeviceSynchronize());
  return UGC_OK;
}

uint32_t host_mask_value(int empty_feat) {
  return empty_feat > 0 && empty_feat < 32 ? ((1u << empty_feat) - 1u) : 0xffffffffu;
}

// Grouped mode: order the host list by address when the last finished lookup took at least
// host_order_min_rows rows from the host (0 = never).  Read from the pinned mirror like the
// mode choice.
bool want_host_order(const Replica* r) {
  if (r->host_order_min_rows <= 0 || !r->feedback) return false;
  const volatile Feedback* f = r->feedback;
  return f->seq != 0 && f->count[kGroupHost] >= (uint32_t)r->host_order_min_rows;
}

// Direct (one fused kernel) or grouped (index lists + per-source CTA groups) for the lookup
// about to be enqueued.  In auto mode the last finished lookup decides: few host rows ->
// direct.  The mirror is read without synchronising, so the answer may lag a few lookups.
bool choose_direct(const Replica* r) {
  if (r->extract_mode == UGC_EXTRACT_DIRECT) return true;
  if (r->extract_mode == UGC_EXTRACT_GROUPED || !r->feedback) return false;
  const volatile Feedback* f = r->feedback;
  if (f->seq == 0) return false;
  // Grouped pays off when a batch takes many rows from the host (ordered host list, all CTAs
  // helping) and few from peers; with peer rows in the mix the direct kernel was faster at
  // every point measured (2 GPUs: 1078 against 1207 us with 49 k host / 93 k peer rows,
  // 2376 against 2514 us with 128 k host / 317 k peer rows).
  const uint32_t host = f->count[kGroupHost], remote = f->count[kGroupRemote];
  return host <= (uint32_t)r->direct_max_host_rows || remote > host;
}

// `n_dev` != nullptr: the key count is read on the device from there (at most n); such a lookup
// always takes the direct extraction and is launched without programmatic overlap, because its
// keys were produced by the kernels just ahead of it in the stream.
int do_lookup(ugc_ctx* c, Replica* r, const void* keys, int key_bytes, size_t n, void* out,
              cudaStream_t s, const uint32_t* n_dev = nullptr) {
  if (n == 0) return UGC_OK;
  if (!keys || !out) return fail(UGC_ERR_INVALID, "keys and out must be non-null");
  if (n > r->max_batch)
    return fail(UGC_ERR_INVALID, "batch of %zu keys exceeds max_batch %u", n, r->max_batch);
  if (c->cfg.num_device > 1 && !r->attached)
    return fail(UGC_ERR_STATE, "replica %d reads from peers: call ugc_attach_peers first", r->id);
  const bool prof = r->prof_on && r->prof_used + 3 <= r->prof_events.size();
  if (prof) UGC_CUDA(cudaEventRecord(r->prof_events[r->prof_used], s));
  // counted before the launch: drain_lookups() must never miss a lookup that could be running
  __atomic_fetch_add(&r->lookups, 1, __ATOMIC_SEQ_CST);
  if (n_dev != nullptr || choose_direct(r)) {
    if (prof) UGC_CUDA(cudaEventRecord(r->prof_events[r->prof_used + 1], s));
    DirectParams d{};
    d.n_dev = n_dev;
    for (int i = 0; i < kMaxLocation; i++) d.src_base[i] = r->src_base[i];
    d.out = out;
    d.table = r->table;
    d.counters = r->counters;
    d.feedback = r->feedback_dev;
    d.n_keys = (uint32_t)n;
    d.row_bytes = c->cfg.row_bytes;
    d.local_loc = (uint32_t)r->id;
    d.host_loc = (uint32_t)c->cfg.num_device;
    d.host_mask = host_mask_value(c->cfg.empty_feat);
    d.tile_shift = (uint32_t)r->direct_tile_shift;
    // count slots alternate from one direct launch to the next; a launch also hands on the
    // counts of the direct launch before it
    d.slot = r->direct_slot;
    d.publish_prev = r->last_was_direct ? 1u : 0u;
    d.prev_keys = r->last_n;
    d.prev_seq = r->last_seq;
    r->direct_slot ^= 1u;
    r->last_slot = d.slot;
    d.host_base = r->src_base[c->cfg.num_device];
    // host rows fetched ahead of the dependency wait: worth its prologue when a lookup takes
    // enough rows from the host for the link's queue to matter
    bool early = r->direct_early_host == 1;
    if (r->direct_early_host == 0 && r->feedback) {
      const volatile Feedback* f = r->feedback;
      early = f->seq != 0 && f->count[kGroupHost] >= 1024u;
    }
    UGC_CUDA(launch_extract_direct(keys, key_bytes, d, r->direct_grid, r->direct_block, r->vec_bytes, r->direct_deep != 0,
                                   early && d.host_base != nullptr, (r->pdl & 1) != 0 && n_dev == nullptr, s));
    if (prof) {
      UGC_CUDA(cudaEventRecord(r->prof_events[r->prof_used + 2], s));
      r->prof_used += 3;
    }
    r->lookups_direct++;
    r->kernel_launches += 1;
    r->last_was_direct = true;
    r->last_n = (uint32_t)n;
    r->last_seq = (uint32_t)r->lookups;
    remember_stream(r, s);
    return UGC_OK;
  }
  UGC_CUDA(launch_lookup_group(keys, key_bytes, (uint32_t)n, r->table, (uint32_t)r->id,
                               (uint32_t)c->cfg.num_device, c->cfg.empty_feat, r->list[kGroupLocal],
                               r->list[kGroupRemote], r->list[kGroupHost], r->counters, r->lookup_kpt, (r->pdl & 1) != 0, s));
  if (prof) UGC_CUDA(cudaEventRecord(r->prof_events[r->prof_used + 1], s));
  GatherParams p = gather_params(c, r, out, (uint32_t)n);
  if (want_host_order(r)) {
    // many host rows last time: order this lookup's host list by address before the gather
    if (!r->host_sorted) {
      r->host_sorted = static_cast<uint64_t*>(ctx_alloc(c, (size_t)r->max_batch * sizeof(uint64_t)));
      r->host_hist = static_cast<uint32_t*>(ctx_alloc(c, host_order_scratch_bytes()));
    }
    if (r->host_sorted && r->host_hist) {
      const uint64_t host_rows = c->cfg.empty_feat > 0 ? ((uint64_t)1 << c->cfg.empty_feat) : c->cfg.num_total_item;
      UGC_CUDA(launch_host_order(r->list[kGroupHost], r->host_sorted, r->counters, r->host_hist, host_rows,
                                 r->sm_count, s));
      p.list[kGroupHost] = r->host_sorted;
      r->kernel_launches += 2;
      r->lookups_host_ordered++;
    }
  }
  UGC_CUDA(launch_gather_roles(p, r->gather_grid, r->block_threads, r->vec_bytes, s));
  if (prof) {
    UGC_CUDA(cudaEventRecord(r->prof_events[r->prof_used + 2], s));
    r->prof_used += 3;
  }
  r->kernel_launches += 2;
  r->last_was_direct = false;
  r->last_n = (uint32_t)n;
  r->last_seq = (uint32_t)r->lookups;
  remember_stream(r, s);
  return UGC_OK;
}

}  // namespace

// ---- lookup scratch that needs no allocation ------------------------------------------------
// ugc_lookup_i64_static keeps its index lists and counters in this fixed device array instead
// of memory obtained at build time.  Every GPU that loads the library carries the array
// (about 6.3 MB) until the process exits.  Layout: Counters (padded to 256 bytes), then the
// three record lists of kStaticMaxKeys entries each.
constexpr uint32_t kStaticMaxKeys = 1u << 18;  // 262,144 keys per call
constexpr size_t kStaticHeader = 256;
constexpr size_t kStaticBytes = kStaticHeader + (size_t)kNumGroup * kStaticMaxKeys * sizeof(uint64_t);
static_assert(sizeof(Counters) <= kStaticHeader, "counters must fit the header");
static __device__ __align__(256) unsigned char g_static_scratch[kStaticBytes];

namespace {
constexpr int kStaticMaxDevices = 64;
std::mutex g_static_mu;
void* g_static_addr[kStaticMaxDevices] = {nullptr};

// Device address of g_static_scratch on the CURRENT device.  In host code the array's name is
// only a handle for the runtime, not an address a kernel could use, hence the symbol query;
// it is made once per device and cached.
int static_scratch_address(int device, void** out) {
  if (device < 0 || device >= kStaticMaxDevices) return fail(UGC_ERR_UNSUPPORTED, "device ordinal %d too large", device);
  std::lock_guard<std::mutex> lock(g_static_mu);
  if (!g_static_addr[device]) {
    // the symbol query answers for whichever device is current: make sure it is `device`
    int cur = -1;
    if (cudaGetDevice(&cur) != cudaSuccess || cur != device) {
      cudaGetLastError();
      return fail(UGC_ERR_STATE, "static scratch set-up needs device %d current, found %d", device, cur);
    }
    void* p = nullptr;
    cudaError_t e = cudaGetSymbolAddress(&p, g_static_scratch);
    if (e != cudaSuccess || !p) {
      cudaGetLastError();
      return fail(UGC_ERR_CUDA, "cudaGetSymbolAddress(static scratch) failed on device %d: %s", device,
                  cudaGetErrorString(e));
    }
    g_static_addr[device] = p;
  }
  *out = g_static_addr[device];
  return UGC_OK;
}
}  // namespace

// --------------------------------------------------------------------------------------
extern "C" {

const char* ugc_version(void) { return "ugache_b200 0.2 (sm_100a)"; }

int ugc_abi_sizes(uint32_t sizes[5]) {
  if (!sizes) return fail(UGC_ERR_INVALID, "null output");
  sizes[0] = sizeof(ugc_config);
  sizes[1] = sizeof(ugc_peer_handle);
  sizes[2] = sizeof(ugc_stats_t);
  sizes[3] = sizeof(ugc_tuning);
  sizes[4] = sizeof(ugc_link_desc_t);
  return UGC_OK;
}
const char* ugc_last_error(void) { return g_last_error.c_str(); }

const char* ugc_status_string(int s) {
  switch (s) {
    case UGC_OK: return "ok";
    case UGC_ERR_INVALID: return "invalid argument";
    case UGC_ERR_CUDA: return "CUDA error";
    case UGC_ERR_NOMEM: return "out of device memory";
    case UGC_ERR_CAPACITY: return "cache capacity exceeded";
    case UGC_ERR_STATE: return "call out of order";
    case UGC_ERR_KEY_RANGE: return "key out of range";
    case UGC_ERR_TIMEOUT: return "timed out";
    case UGC_ERR_UNSUPPORTED: return "unsupported configuration";
    case UGC_ERR_TABLE: return "table inconsistency";
    default: return "unknown status";
  }
}

int ugc_config_default(ugc_config* cfg) {
  if (!cfg) return fail(UGC_ERR_INVALID, "null config");
  memset(cfg, 0, sizeof(*cfg));
  cfg->struct_size = sizeof(*cfg);
  cfg->num_device = 1;
  cfg->max_batch = 1u << 20;
  cfg->register_host = 1;
  return UGC_OK;
}

int ugc_create(const ugc_config* cfg, ugc_ctx** out) {
  if (!cfg || !out) return fail(UGC_ERR_INVALID, "null argument");
  if (cfg->struct_size != sizeof(ugc_config))
    return fail(UGC_ERR_INVALID, "ugc_config.struct_size %u != %zu", cfg->struct_size, sizeof(ugc_config));
  if (cfg->num_device < 1 || cfg->num_device > UGC_MAX_DEVICE)
    return fail(UGC_ERR_INVALID, "num_device must be 1..%d", UGC_MAX_DEVICE);
  if (cfg->num_total_item == 0 || cfg->num_total_item >= 0x7fffffffull)
    return fail(UGC_ERR_UNSUPPORTED, "num_total_item must be in [1, 2^31-1)");
  if (cfg->row_bytes == 0 || cfg->row_bytes % 4 != 0)
    return fail(UGC_ERR_UNSUPPORTED, "row_bytes must be a positive multiple of 4");
  if (cfg->cache_percentage < 0 || cfg->cache_percentage > 1)
    return fail(UGC_ERR_INVALID, "cache_percentage is a fraction in [0, 1]");
  if (cfg->empty_feat < 0 || cfg->empty_feat > 31)
    return fail(UGC_ERR_INVALID, "empty_feat must be in [0, 31]");
  if (cfg->max_batch == 0 || cfg->max_batch > kMaxBatch)
    return fail(UGC_ERR_INVALID, "max_batch must be in [1, 2^28]");
  if ((cfg->alloc == nullptr) != (cfg->free == nullptr) && cfg->free != nullptr)
    return fail(UGC_ERR_INVALID, "a free callback needs an alloc callback");
  if (cache_capacity_rows(cfg->num_total_item, cfg->cache_percentage) > (uint64_t)kOffMask)
    return fail(UGC_ERR_UNSUPPORTED, "a cache slice holds at most 2^28-1 rows");
  ugc_ctx* c = new (std::nothrow) ugc_ctx();
  if (!c) return fail(UGC_ERR_NOMEM, "out of host memory");
  c->cfg = *cfg;
  c->reps.resize(cfg->num_device);
  *out = c;
  return UGC_OK;
}

int ugc_destroy(ugc_ctx* c) {
  if (!c) return UGC_OK;
  for (auto& r : c->reps)
    if (r.built) release_replica(c, &r);
  if (c->host_registered_here && c->host_table)
    ugc_host_unregister_sized(const_cast<void*>(c->host_table), c->host_registered_bytes);
  delete c;
  return UGC_OK;
}

int ugc_solve_placement(int policy, int num_device, uint64_t N, const uint32_t* rank_ids,
                        const uint32_t* rank_freqs, double cache_percent, double t_local,
                        double t_remote, double t_cpu, uint32_t* nid_to_block,
                        uint8_t* block_placement, uint8_t* block_access_from, double* block_density,
                        int* num_block) {
  if (!nid_to_block || !block_placement || !block_access_from || !block_density || !num_block)
    return fail(UGC_ERR_INVALID, "null output array");
  Placement p;
  std::string err = solve_placement(policy, num_device, N, rank_ids, rank_freqs, cache_percent,
                                    t_local, t_remote, t_cpu, &p);
  if (!err.empty()) return fail(UGC_ERR_INVALID, "%s", err.c_str());
  memcpy(nid_to_block, p.nid_to_block.data(), N * sizeof(uint32_t));
  memcpy(block_placement, p.block_placement.data(), p.num_block);
  memcpy(block_access_from, p.block_access_from.data(), (size_t)num_device * p.num_block);
  memcpy(block_density, p.block_density.data(), p.num_block * sizeof(double));
  *num_block = p.num_block;
  return UGC_OK;
}

int ugc_placement_cost(int num_device, uint64_t N, const uint32_t* rank_ids, const uint32_t* rank_freqs,
                       const uint32_t* nid_to_block, const uint8_t* block_access_from, int num_block,
                       double t_local, double t_remote, double t_cpu, double* cost) {
  if (num_device < 1 || num_device > UGC_MAX_DEVICE || num_block < 1 || !nid_to_block || !block_access_from)
    return fail(UGC_ERR_INVALID, "bad placement arguments");
  Placement p;
  p.num_device = num_device;
  p.num_block = num_block;
  p.block_access_from.assign(block_access_from, block_access_from + (size_t)num_device * num_block);
  int bad = 0;  // the per-key array is read in place (4 bytes per id: no copy per call)
#pragma omp parallel for schedule(static) reduction(| : bad)
  for (int64_t k = 0; k < (int64_t)N; k++) bad |= (nid_to_block[k] >= (uint32_t)num_block);
  if (bad) return fail(UGC_ERR_INVALID, "block id out of range");
  for (uint8_t a : p.block_access_from)
    if (a > num_device) return fail(UGC_ERR_INVALID, "source location out of range");
  std::string err = placement_cost(p, N, rank_ids, rank_freqs, t_local, t_remote, t_cpu, cost, nid_to_block);
  if (!err.empty()) return fail(UGC_ERR_INVALID, "%s", err.c_str());
  return UGC_OK;
}

int ugc_link_desc(int num_device, uint32_t row_bytes, ugc_link_desc_t* out) {
  if (!out || out->struct_size != sizeof(ugc_link_desc_t)) return fail(UGC_ERR_INVALID, "bad ugc_link_desc_t");
  if (num_device < 1 || num_device > UGC_MAX_DEVICE) return fail(UGC_ERR_INVALID, "num_device must be 1..%d", UGC_MAX_DEVICE);
  const LinkDesc d = b200_link_desc(num_device, row_bytes);
  out->num_device = d.num_device;
  out->bw_local_gbs = d.bw_local_gbs;
  out->bw_remote_gbs = d.bw_remote_gbs;
  out->bw_host_gbs = d.bw_host_gbs;
  out->lat_local_us = d.lat_local_us;
  out->lat_remote_us = d.lat_remote_us;
  out->lat_host_us = d.lat_host_us;
  out->host_rows_per_s = d.host_rows_per_s;
  out->host_total_gbs = d.host_total_gbs;
  out->t_local = d.t_local;
  out->t_remote = d.t_remote;
  out->t_cpu = d.t_cpu;
  out->host_ctas = d.host_ctas;
  out->remote_ctas = d.remote_ctas;
  out->per_peer_ctas = d.per_peer_ctas;
  return UGC_OK;
}

int ugc_link_model(int num_device, double* t_local, double* t_remote, double* t_cpu) {
  if (!t_local || !t_remote || !t_cpu) return fail(UGC_ERR_INVALID, "null output");
  b200_link_model(num_device, t_local, t_remote, t_cpu);
  return UGC_OK;
}

static int load_placement(ugc_ctx* c, Placement* dst, const uint32_t* n2b, const uint8_t* bp,
                          const uint8_t* ba, const double* bd, int B) {
  if (!c) return fail(UGC_ERR_INVALID, "null context");
  if (!n2b || !bp || !ba || B <= 0) return fail(UGC_ERR_INVALID, "null placement array");
  const int G = c->cfg.num_device;
  const uint64_t N = c->cfg.num_total_item;
  // The per-key array is the large one (4 bytes per id: 1.6 GB at 4*10^8 ids).  It is copied
  // into storage that is kept from one refresh to the next (no fresh pages to fault in), by
  // several threads, and its block ids are range-checked in the same pass.
  Placement& p = *dst;
  p.valid = false;
  p.num_block = B;
  p.num_device = G;
  if (p.nid_to_block.size() != N) p.nid_to_block.resize(N);
  uint32_t* copy = p.nid_to_block.data();
  const uint32_t nb = (uint32_t)B;
  int bad = 0;
  const int threads = std::max(1, std::min(16, omp_get_num_procs()));
#pragma omp parallel for schedule(static) num_threads(threads) reduction(| : bad)
  for (int64_t i = 0; i < (int64_t)N; i++) {
    const uint32_t b = n2b[i];
    copy[i] = b;
    bad |= (b >= nb);
  }
  if (bad) return fail(UGC_ERR_INVALID, "placement rejected: nid_to_block holds a block id >= num_block");
  p.block_placement.assign(bp, bp + B);
  p.block_access_from.assign(ba, ba + (size_t)G * B);
  if (bd) {
    p.block_density.assign(bd, bd + B);
  } else {
    p.block_density.clear();
  }
  std::string err = validate_placement(p, G, N, false);
  if (!err.empty()) return fail(UGC_ERR_INVALID, "placement rejected: %s", err.c_str());
  p.valid = true;
  return UGC_OK;
}

int ugc_set_placement(ugc_ctx* c, const uint32_t* n2b, const uint8_t* bp, const uint8_t* ba,
                      const double* bd, int B) {
  if (c)
    for (auto& r : c->reps)
      if (r.built) return fail(UGC_ERR_STATE, "replicas are built: use the refresh calls");
  return load_placement(c, c ? &c->cur : nullptr, n2b, bp, ba, bd, B);
}

int ugc_classify_keys(ugc_ctx* c, int replica_id, uint64_t* counts, uint32_t* keys_out) {
  Replica* r;
  UGC_TRY(get_replica(c, replica_id, false, &r));
  if (!c->cur.valid) return fail(UGC_ERR_STATE, "no placement set");
  if (!counts) return fail(UGC_ERR_INVALID, "null counts");
  std::vector<uint32_t> lists[kMaxDevice];
  classify_keys(c->cur, replica_id, c->cfg.num_total_item, lists, counts);
  if (keys_out) {
    size_t pos = 0;
    for (int s = 0; s < c->cfg.num_device; s++) {
      memcpy(keys_out + pos, lists[s].data(), lists[s].size() * sizeof(uint32_t));
      pos += lists[s].size();
    }
  }
  return UGC_OK;
}

int ugc_build(ugc_ctx* c, int replica_id, int device_id, const void* host_table, void* stream) {
  Replica* r;
  UGC_TRY(get_replica(c, replica_id, false, &r));
  if (r->built) return fail(UGC_ERR_STATE, "replica %d is already built", replica_id);
  if (!c->cur.valid) return fail(UGC_ERR_STATE, "no placement set");
  if (!host_table) return fail(UGC_ERR_INVALID, "null host table");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int G = c->cfg.num_device;
  const uint64_t N = c->cfg.num_total_item;
  UGC_CUDA(cudaSetDevice(device_id));
  {
    std::lock_guard<std::mutex> lock(c->mu);
    UGC_TRY(map_host_table(c, host_table));
  }
  r->id = replica_id;
  r->device = device_id;
  cudaDeviceProp prop;
  UGC_CUDA(cudaGetDeviceProperties(&prop, device_id));
  r->sm_count = prop.multiProcessorCount;
  const int per_sm = c->cfg.gather_ctas_per_sm > 0 ? c->cfg.gather_ctas_per_sm : 8;
  r->gather_grid = r->sm_count * per_sm;
  r->direct_grid = r->sm_count * 4;
  if (const char* m = getenv("UGC_EXTRACT_MODE")) {  // initial ugc_tuning.extract_mode
    if (!strcmp(m, "grouped")) r->extract_mode = UGC_EXTRACT_GROUPED;
    if (!strcmp(m, "direct")) r->extract_mode = UGC_EXTRACT_DIRECT;
    if (!strcmp(m, "auto")) r->extract_mode = UGC_EXTRACT_AUTO;
    if (!strcmp(m, "grouped_static")) {  // grouped with fixed striding instead of chunk hand-out
      r->extract_mode = UGC_EXTRACT_GROUPED;
      r->gather_dynamic = 0;
    }
    if (!strcmp(m, "direct_early")) {  // direct, host rows always fetched ahead of the wait
      r->extract_mode = UGC_EXTRACT_DIRECT;
      r->direct_early_host = 1;
    }
  }
  // Far-source CTA budgets and the per-group time-per-byte come from the link description:
  // bandwidth x latency gives the CTAs that keep a link full, bytes / bandwidth the share of
  // the launch each group gets.
  {
    const LinkDesc ld = b200_link_desc(G, c->cfg.row_bytes, c->cfg.bw_local_gbs, c->cfg.bw_remote_gbs,
                                       c->cfg.bw_host_gbs);
    r->host_ctas = c->cfg.host_ctas > 0 ? c->cfg.host_ctas : ld.host_ctas;
    r->remote_ctas = c->cfg.remote_ctas > 0 ? c->cfg.remote_ctas : ld.remote_ctas;
    r->t_byte[kGroupLocal] = (float)(1.0 / ld.bw_local_gbs);
    r->t_byte[kGroupRemote] = ld.bw_remote_gbs > 0 ? (float)(1.0 / ld.bw_remote_gbs) : 0.0f;
    r->t_byte[kGroupHost] = (float)(1.0 / ld.bw_host_gbs);
  }
  // 32-byte loads win when almost every row comes from HBM (8 GPUs, 458 host rows per batch:
  // 36.5 us per step against 45); with more host rows per batch 16-byte loads were faster
  // (1 GPU: 113 vs 133 us, 2 GPUs: 84 vs 110 us, 4 GPUs: 54 vs 61 us).
  r->vec_bytes = c->cfg.gather_vec_bytes ? (c->cfg.gather_vec_bytes == 32 ? 32 : 16) : (G >= 8 ? 32 : 16);

  // 1. which source serves each key: ascending key lists per GPU source, made on the GPU
  {
    int rc0 = upload_n2b(c, c->cur, &r->n2b_dev, s);
    if (rc0 == UGC_OK) rc0 = gpu_classify(c, r, nullptr, c->cur, nullptr, r->n2b_dev, s);
    if (rc0 != UGC_OK) {
      std::string keep = g_last_error;
      release_replica(c, r);
      g_last_error = keep;
      return rc0;
    }
  }
  const uint64_t n_local = r->list_count[replica_id];
  uint64_t n_remote = 0;
  for (int s2 = 0; s2 < G; s2++)
    if (s2 != replica_id) n_remote += r->list_count[s2];
  r->n_local = n_local;
  r->n_remote = n_remote;

  // 2. the slice
  r->capacity = cache_capacity_rows(N, c->cfg.cache_percentage);
  if (n_local > r->capacity) {
    int rc = fail(UGC_ERR_CAPACITY, "placement stores %llu rows on replica %d, slice holds %llu",
                  (unsigned long long)n_local, replica_id, (unsigned long long)r->capacity);
    release_replica(c, r);
    return rc;
  }
  r->slice_bytes = std::max<size_t>((size_t)r->capacity * c->cfg.row_bytes, 256);
  r->slice = ctx_alloc_shared(c, r->slice_bytes);
  if (!r->slice) {
    int rc = fail(UGC_ERR_NOMEM, "slice allocation of %zu bytes failed", r->slice_bytes);
    release_replica(c, r);
    return rc;
  }
  auto bail = [&](int rc) {
    std::string keep = g_last_error;
    release_replica(c, r);
    g_last_error = keep;
    return rc;
  };
  int rc;
  // 3. lookup scratch and counters
  r->max_batch = c->cfg.max_batch;
  for (int g = 0; g < kNumGroup; g++) {
    r->list[g] = static_cast<uint64_t*>(ctx_alloc(c, (size_t)r->max_batch * sizeof(uint64_t)));
    if (!r->list[g]) return bail(fail(UGC_ERR_NOMEM, "scratch allocation failed"));
  }
  r->counters = static_cast<Counters*>(ctx_alloc(c, sizeof(Counters)));
  if (!r->counters) return bail(fail(UGC_ERR_NOMEM, "counter allocation failed"));
  // pinned mirror of the last lookup's counts (16 bytes written across PCIe per lookup)
  {
    void* fb = nullptr;
    void* fb_dev = nullptr;
    if (cudaHostAlloc(&fb, sizeof(Feedback), cudaHostAllocMapped) == cudaSuccess &&
        cudaHostGetDevicePointer(&fb_dev, fb, 0) == cudaSuccess) {
      memset(fb, 0, sizeof(Feedback));
      r->feedback = static_cast<Feedback*>(fb);
      r->feedback_dev = static_cast<Feedback*>(fb_dev);
    } else {  // without the mirror the auto mode stays on the grouped path
      cudaGetLastError();
      if (fb) cudaFreeHost(fb);
    }
  }
  if (cudaMemsetAsync(r->counters, 0, sizeof(Counters), s) != cudaSuccess)
    return bail(fail(UGC_ERR_CUDA, "cudaMemsetAsync failed: %s", cudaGetErrorString(cudaGetLastError())));

  // 4. fill: slice[j] = host[local_keys[j]]
  if (launch_fill_scatter(c->host_dev, r->slice, list_ptr(r, replica_id), SlotView{nullptr, 0, 0},
                          (uint32_t)n_local, c->cfg.row_bytes, c->cfg.empty_feat, r->sm_count * 2,
                          s) != cudaSuccess)
    return bail(fail(UGC_ERR_CUDA, "fill launch failed: %s", cudaGetErrorString(cudaGetLastError())));

  // 5. table with the local entries (slot = position in the list)
  // Size the table for every row the GPUs can hold together, so that a later refresh to a
  // placement with more partitioned rows still fits (the reference sizes its table once, for
  // the build-time entry count, coll_cache_lib/cache_context.cu:2489-2497).
  const uint64_t max_entries = std::min<uint64_t>(N, (uint64_t)G * r->capacity);
  if ((rc = alloc_table(c, r, n_local + n_remote, std::max(n_local + n_remote, max_entries), s)) != UGC_OK)
    return bail(rc);
  if (launch_table_insert(r->table, list_ptr(r, replica_id), SlotView{nullptr, 0, 0},
                          (uint32_t)replica_id, (uint32_t)n_local, r->counters, s) != cudaSuccess)
    return bail(fail(UGC_ERR_CUDA, "insert launch failed: %s", cudaGetErrorString(cudaGetLastError())));
  if ((rc = check_table_errors(r, s, "build insert")) != UGC_OK) return bail(rc);

  // 6. free slots: [n_local, capacity)  (coll_cache_lib/cache_context.cu:2577-2585)
  r->free_ring = static_cast<uint32_t*>(ctx_alloc(c, std::max<size_t>(r->capacity, 1) * sizeof(uint32_t)));
  if (!r->free_ring) return bail(fail(UGC_ERR_NOMEM, "free-slot ring allocation failed"));
  r->free_head = 0;
  r->free_count = r->capacity - n_local;
  if (launch_iota(r->free_ring, (uint32_t)n_local, (uint32_t)r->free_count, s) != cudaSuccess ||
      cudaStreamSynchronize(s) != cudaSuccess)
    return bail(fail(UGC_ERR_CUDA, "free-slot ring set-up failed: %s", cudaGetErrorString(cudaGetLastError())));

  r->src_base[replica_id] = r->slice;
  r->src_base[G] = c->host_dev;
  r->attached = (n_remote == 0);
  if (r->attached) {  // no peer lists to resolve later: the build lists can go now
    ctx_free(c, r->lists.ptr);
    r->lists = DevBuf{};
  }
  r->built = true;
  return UGC_OK;
}

int ugc_export(ugc_ctx* c, int replica_id, ugc_peer_handle* out) {
  Replica* r;
  UGC_TRY(get_replica(c, replica_id, true, &r));
  if (!out) return fail(UGC_ERR_INVALID, "null handle");
  memset(out, 0, sizeof(*out));
  out->replica_id = r->id;
  out->device_id = r->device;
  out->pid = (int64_t)getpid();
  out->slice_ptr = (uint64_t)(uintptr_t)r->slice;
  out->table_ptr = (uint64_t)(uintptr_t)r->table_mem;
  out->table_kind = r->table.kind;
  out->table_lines = r->table.kind == kTableFlat ? r->table.num_keys : (uint64_t)r->table.line_mask + 1;
  // Cross-process export needs the built-in allocator (IPC handles describe whole
  // allocations; a caller's allocator may hand out pieces of a larger block).
  DevBlock sb, tb;
  if (!c->cfg.alloc && dev_block_find(r->slice, &sb) && dev_block_find(r->table_mem, &tb)) {
    const int sfd = dev_block_export_fd(r->slice), tfd = dev_block_export_fd(r->table_mem);
    if (sfd >= 0 && tfd >= 0) {
      // Importers duplicate the two descriptors out of this process where the kernel lets
      // them, else ask for them over the descriptor socket (same user only).  Nothing is done
      // here to widen who may attach to this process.
      const bool served = fd_server_publish(sfd) && fd_server_publish(tfd);
      if (!served) g_last_error = g_fd_server_error;  // not fatal: read with ugc_last_error()
      out->has_ipc = 2;
      int64_t v[3] = {sfd, (int64_t)sb.size, (int64_t)g_fd_token};
      memcpy(out->slice_ipc, v, sizeof(v));
      int64_t w[3] = {tfd, (int64_t)tb.size, (int64_t)g_fd_token};
      memcpy(out->table_ipc, w, sizeof(w));
      return UGC_OK;
    }
  }
  if (!c->cfg.alloc && !dev_block_find(r->slice, &sb)) {
    UGC_CUDA(cudaSetDevice(r->device));
    cudaIpcMemHandle_t h;
    static_assert(sizeof(h) == 64, "cudaIpcMemHandle_t is 64 bytes");
    UGC_CUDA(cudaIpcGetMemHandle(&h, r->slice));
    memcpy(out->slice_ipc, &h, 64);
    UGC_CUDA(cudaIpcGetMemHandle(&h, r->table_mem));
    memcpy(out->table_ipc, &h, 64);
    out->has_ipc = 1;
  }
  return UGC_OK;
}

static TableView view_from_handle(const ugc_peer_handle* h, void* table_ptr, uint64_t N) {
  TableView t{};
  t.kind = h->table_kind;
  t.num_keys = N;
  if (t.kind == kTableFlat) {
    t.flat = static_cast<uint32_t*>(table_ptr);
  } else {
    t.slots = static_cast<uint2*>(table_ptr);
    t.line_mask = (uint32_t)(h->table_lines - 1);
  }
  return t;
}

static int enable_peer(int from_dev, int to_dev) {
  if (from_dev == to_dev) return UGC_OK;
  UGC_CUDA(cudaSetDevice(from_dev));
  int can = 0;
  UGC_CUDA(cudaDeviceCanAccessPeer(&can, from_dev, to_dev));
  if (!can) return fail(UGC_ERR_UNSUPPORTED, "device %d cannot access device %d", from_dev, to_dev);
  cudaError_t e = cudaDeviceEnablePeerAccess(to_dev, 0);
  if (e != cudaSuccess && e != cudaErrorPeerAccessAlreadyEnabled)
    return fail(UGC_ERR_CUDA, "cudaDeviceEnablePeerAccess(%d) failed: %s", to_dev, cudaGetErrorString(e));
  cudaGetLastError();
  return UGC_OK;
}

int ugc_import_peer(ugc_ctx* c, int replica_id, const ugc_peer_handle* peer) {
  Replica* r;
  UGC_TRY(get_replica(c, replica_id, true, &r));
  if (!peer) return fail(UGC_ERR_INVALID, "null handle");
  const int p = peer->replica_id;
  if (p < 0 || p >= c->cfg.num_device || p == replica_id)
    return fail(UGC_ERR_INVALID, "bad peer replica id %d", p);
  void* slice = nullptr;
  void* table = nullptr;
  if (peer->pid == (int64_t)getpid()) {
    slice = (void*)(uintptr_t)peer->slice_ptr;
    table = (void*)(uintptr_t)peer->table_ptr;
    DevBlock sb, tb;
    if (dev_block_find(slice, &sb) && dev_block_find(table, &tb)) {
      // virtual-memory blocks: access is granted per device, peer-access enabling does not apply
      if (!dev_set_access(slice, sb.size, r->device) || !dev_set_access(table, tb.size, r->device))
        return fail(UGC_ERR_CUDA, "cannot grant device %d access to replica %d's memory", r->device, p);
      // keep the owner's own access
      dev_set_access(slice, sb.size, sb.device);
      dev_set_access(table, tb.size, tb.device);
    } else {
      UGC_TRY(enable_peer(r->device, peer->device_id));
    }
  } else if (peer->has_ipc == 2) {
    UGC_CUDA(cudaSetDevice(r->device));
    int64_t v[3], w[3];
    memcpy(v, peer->slice_ipc, sizeof(v));
    memcpy(w, peer->table_ipc, sizeof(w));
    slice = dev_import(peer->pid, (uint64_t)v[2], (int)v[0], (size_t)v[1], r->device);
    if (!slice)
      return fail(UGC_ERR_CUDA, "cannot import replica %d's slice (descriptor %d of process %lld)", p,
                  (int)v[0], (long long)peer->pid);
    r->ipc_opened[r->n_ipc_opened++] = slice;
    table = dev_import(peer->pid, (uint64_t)w[2], (int)w[0], (size_t)w[1], r->device);
    if (!table) return fail(UGC_ERR_CUDA, "cannot import replica %d's table", p);
    r->ipc_opened[r->n_ipc_opened++] = table;
  } else {
    if (!peer->has_ipc) return fail(UGC_ERR_INVALID, "peer handle from another process carries no IPC handles");
    UGC_CUDA(cudaSetDevice(r->device));
    cudaIpcMemHandle_t h;
    memcpy(&h, peer->slice_ipc, 64);
    UGC_CUDA(cudaIpcOpenMemHandle(&slice, h, cudaIpcMemLazyEnablePeerAccess));
    r->ipc_opened[r->n_ipc_opened++] = slice;
    memcpy(&h, peer->table_ipc, 64);
    UGC_CUDA(cudaIpcOpenMemHandle(&table, h, cudaIpcMemLazyEnablePeerAccess));
    r->ipc_opened[r->n_ipc_opened++] = table;
  }
  r->src_base[p] = slice;
  r->peer_table[p] = view_from_handle(peer, table, c->cfg.num_total_item);
  r->peer_known[p] = true;
  return UGC_OK;
}

int ugc_connect_local(ugc_ctx* c) {
  if (!c) return fail(UGC_ERR_INVALID, "null context");
  for (auto& a : c->reps) {
    if (!a.built) continue;
    for (auto& b : c->reps) {
      if (!b.built || a.id == b.id) continue;
      ugc_peer_handle h;
      memset(&h, 0, sizeof(h));
      h.replica_id = b.id;
      h.device_id = b.device;
      h.pid = (int64_t)getpid();
      h.slice_ptr = (uint64_t)(uintptr_t)b.slice;
      h.table_ptr = (uint64_t)(uintptr_t)b.table_mem;
      h.table_kind = b.table.kind;
      h.table_lines = b.table.kind == kTableFlat ? b.table.num_keys : (uint64_t)b.table.line_mask + 1;
      UGC_TRY(ugc_import_peer(c, a.id, &h));
    }
  }
  return UGC_OK;
}

// Resolve the slots of `keys` (all served by `src`) from src's table and insert them.
// Resolve the slots of `n` device-resident keys (all served by `src`) from src's table and
// insert them into this replica's table.
static int attach_keys(ugc_ctx* c, Replica* r, int src, const uint32_t* keys_dev, uint64_t n, cudaStream_t s) {
  if (n == 0) return UGC_OK;
  if (!r->peer_known[src] || !r->src_base[src])
    return fail(UGC_ERR_STATE, "replica %d reads from replica %d, which has not been imported", r->id, src);
  UGC_TRY(ensure(c, r->stage_b, n * sizeof(uint32_t)));
  const SlotView offs{static_cast<uint32_t*>(r->stage_b.ptr), 0, 0};
  UGC_CUDA(launch_table_resolve(r->peer_table[src], keys_dev, (uint32_t)n, (uint32_t)src, offs, r->counters, s));
  // (a refresh may have re-pointed some of these keys to `src` already, with the same word)
  UGC_CUDA(launch_table_insert(r->table, keys_dev, offs, (uint32_t)src, (uint32_t)n, r->counters, s, true));
  // the offset buffer is reused by the next source
  return check_table_errors(r, s, "peer attach");
}

int ugc_attach_peers(ugc_ctx* c, int replica_id, void* stream) {
  Replica* r;
  UGC_TRY(get_replica(c, replica_id, true, &r));
  if (r->attached) return UGC_OK;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  UGC_CUDA(cudaSetDevice(r->device));
  for (int src = 0; src < c->cfg.num_device; src++) {
    if (src == replica_id) continue;
    UGC_TRY(attach_keys(c, r, src, list_ptr(r, src), r->list_count[src], s));
  }
  r->attached = true;
  // the build lists are not needed any more
  ctx_free(c, r->lists.ptr);
  r->lists = DevBuf{};
  return UGC_OK;
}

int ugc_lookup_u32(ugc_ctx* c, int replica_id, const uint32_t* keys, size_t n, void* out, void* stream) {
  Replica* r;
  UGC_TRY(get_replica(c, replica_id, true, &r));
  UGC_CUDA(cudaSetDevice(r->device));
  return do_lookup(c, r, keys, 4, n, out, static_cast<cudaStream_t>(stream));
}

int ugc_lookup_i64(ugc_ctx* c, int replica_id, const int64_t* keys, size_t n, void* out, void* stream) {
  Replica* r;
  UGC_TRY(get_replica(c, replica_id, true, &r));
  UGC_CUDA(cudaSetDevice(r->device));
  return do_lookup(c, r, keys, 8, n, out, static_cast<cudaStream_t>(stream));
}

int ugc_lookup_i64_static(ugc_ctx* c, int replica_id, const int64_t* keys, size_t n, void* out,
                          void* stream) {
  Replica* r;
  UGC_TRY(get_replica(c, replica_id, true, &r));
  if (n == 0) return UGC_OK;
  if (!keys || !out) return fail(UGC_ERR_INVALID, "keys and out must be non-null");
  if (n > kStaticMaxKeys)
    return fail(UGC_ERR_INVALID, "ugc_lookup_i64_static takes at most %u keys per call, got %zu",
                kStaticMaxKeys, n);
  if (c->cfg.num_device > 1 && !r->attached)
    return fail(UGC_ERR_STATE, "replica %d reads from peers: call ugc_attach_peers first", r->id);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  UGC_CUDA(cudaSetDevice(r->device));
  r->static_used = true;  // a refresh then drains the device instead of counting lookups
  void* base = nullptr;
  UGC_TRY(static_scratch_address(r->device, &base));
  Counters* counters = static_cast<Counters*>(base);
  uint64_t* lists = reinterpret_cast<uint64_t*>(static_cast<unsigned char*>(base) + kStaticHeader);
  // The array still holds whatever the previous call (of any replica on this GPU) left:
  // the per-lookup counts must start from zero.
  UGC_CUDA(cudaMemsetAsync(counters, 0, sizeof(Counters), s));
  UGC_CUDA(launch_lookup_group(keys, 8, (uint32_t)n, r->table, (uint32_t)r->id, (uint32_t)c->cfg.num_device,
                               c->cfg.empty_feat, lists, lists + kStaticMaxKeys, lists + 2 * (size_t)kStaticMaxKeys,
                               counters, r->lookup_kpt, false, s));
  GatherParams p{};
  for (int i = 0; i < kMaxLocation; i++) p.src_base[i] = r->src_base[i];
  p.out = out;
  for (int g = 0; g < kNumGroup; g++) p.list[g] = lists + (size_t)g * kStaticMaxKeys;
  p.counters = counters;
  p.row_bytes = c->cfg.row_bytes;
  p.n_keys = (uint32_t)n;
  p.remote_cta_cap = r->remote_ctas;
  p.host_cta_cap = r->host_ctas;
  p.rows_per_cta_min = 32;
  for (int g = 0; g < kNumGroup; g++) p.t_byte[g] = r->t_byte[g];
  p.dynamic = 0;
  p.bulk_mask = 0;
  p.pdl = 0;
  UGC_CUDA(launch_gather_roles(p, r->gather_grid, r->block_threads, r->vec_bytes, s));
  return UGC_OK;
}

int ugc_lookup_unique(ugc_ctx* c, int replica_id, const void* keys, int key_bytes, size_t n, void* out_rows,
                      void* unique_keys, int32_t* inverse, uint32_t* n_unique, void* stream) {
  Replica* r;
  UGC_TRY(get_replica(c, replica_id, true, &r));
  if (key_bytes != 4 && key_bytes != 8) return fail(UGC_ERR_INVALID, "key_bytes must be 4 or 8");
  if (!n_unique) return fail(UGC_ERR_INVALID, "n_unique must be non-null");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  UGC_CUDA(cudaSetDevice(r->device));
  if (n == 0) {
    UGC_CUDA(cudaMemsetAsync(n_unique, 0, sizeof(uint32_t), s));
    return UGC_OK;
  }
  if (!keys || !out_rows || !unique_keys || !inverse) return fail(UGC_ERR_INVALID, "null argument");
  if (n > r->max_batch) return fail(UGC_ERR_INVALID, "batch of %zu keys exceeds max_batch %u", n, r->max_batch);
  if (n >= 0x00ffffffu) return fail(UGC_ERR_UNSUPPORTED, "at most 2^24-2 keys per deduplicated lookup");
  if (c->cfg.num_device > 1 && !r->attached)
    return fail(UGC_ERR_STATE, "replica %d reads from peers: call ugc_attach_peers first", r->id);
  const size_t stamp_bytes = (size_t)c->cfg.num_total_item * sizeof(uint32_t);
  if (!r->stamp) {
    r->stamp = static_cast<uint32_t*>(ctx_alloc(c, stamp_bytes));
    if (!r->stamp) return fail(UGC_ERR_NOMEM, "stamp array (%zu bytes) could not be allocated", stamp_bytes);
    r->stamp_epoch = 255;  // forces the clearing below
  }
  if (++r->stamp_epoch > 255) {  // all stamps back to epoch 0 before an epoch value is reused
    UGC_CUDA(cudaMemsetAsync(r->stamp, 0, stamp_bytes, s));
    r->stamp_epoch = 1;
  }
  UGC_CUDA(launch_unique(keys, key_bytes, (uint32_t)n, c->cfg.num_total_item, r->stamp_epoch, r->stamp,
                         unique_keys, inverse, n_unique, r->counters, s));
  r->kernel_launches += 2;
  return do_lookup(c, r, unique_keys, key_bytes, n, out_rows, s, n_unique);
}

int ugc_lookup_pool(ugc_ctx* c, int replica_id, const void* keys, int key_bytes, size_t n_keys,
                    const int64_t* offsets, size_t n_bags, size_t bag_size, int elem_type, int mode,
                    float* out, void* stream) {
  Replica* r;
  UGC_TRY(get_replica(c, replica_id, true, &r));
  if (key_bytes != 4 && key_bytes != 8) return fail(UGC_ERR_INVALID, "key_bytes must be 4 or 8");
  if (elem_type != UGC_ELEM_F32 && elem_type != UGC_ELEM_F16) return fail(UGC_ERR_INVALID, "unknown element type %d", elem_type);
  if (mode != UGC_POOL_SUM && mode != UGC_POOL_MEAN) return fail(UGC_ERR_INVALID, "unknown pooling mode %d", mode);
  if (n_bags == 0) return UGC_OK;
  if (!out || (n_keys && !keys)) return fail(UGC_ERR_INVALID, "keys and out must be non-null");
  if (!offsets && bag_size == 0) return fail(UGC_ERR_INVALID, "give offsets or a bag size");
  if (!offsets && bag_size > n_keys / n_bags)  // n_bags * bag_size > n_keys, without overflow
    return fail(UGC_ERR_INVALID, "%zu bags of %zu keys need more than the %zu keys given", n_bags, bag_size, n_keys);
  if (n_keys > kMaxBatch || n_bags > kMaxBatch) return fail(UGC_ERR_INVALID, "at most 2^28 keys and bags per call");
  const uint32_t row_bytes = c->cfg.row_bytes;
  const uint32_t elem = elem_type == UGC_ELEM_F16 ? 2u : 4u;
  if (row_bytes % 16 != 0) return fail(UGC_ERR_UNSUPPORTED, "pooled lookup needs rows of a multiple of 16 bytes");
  uintptr_t bits = reinterpret_cast<uintptr_t>(out);
  for (int i = 0; i < kMaxLocation; i++) bits |= reinterpret_cast<uintptr_t>(r->src_base[i]);
  if (bits & 15) return fail(UGC_ERR_UNSUPPORTED, "pooled lookup needs 16-byte aligned tables and output");
  if (c->cfg.num_device > 1 && !r->attached)
    return fail(UGC_ERR_STATE, "replica %d reads from peers: call ugc_attach_peers first", r->id);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  UGC_CUDA(cudaSetDevice(r->device));
  // counted before the launch, like every lookup: a refresh waits for it before it reuses slots
  __atomic_fetch_add(&r->lookups, 1, __ATOMIC_SEQ_CST);
  PoolParams p{};
  for (int i = 0; i < kMaxLocation; i++) p.src_base[i] = r->src_base[i];
  p.out = out;
  p.table = r->table;
  p.counters = r->counters;
  p.offsets = reinterpret_cast<const long long*>(offsets);
  p.n_keys = (uint32_t)n_keys;
  p.n_bags = (uint32_t)n_bags;
  p.bag_size = (uint32_t)bag_size;
  p.row_bytes = row_bytes;
  p.dim = row_bytes / elem;
  p.local_loc = (uint32_t)r->id;
  p.host_loc = (uint32_t)c->cfg.num_device;
  p.host_mask = host_mask_value(c->cfg.empty_feat);
  p.mean = mode == UGC_POOL_MEAN ? 1u : 0u;
  UGC_CUDA(launch_lookup_pool(keys, key_bytes, p, elem_type == UGC_ELEM_F16, r->sm_count * 8, r->pool_vec_bytes, s));
  r->kernel_launches += 1;
  r->lookups_pooled++;
  remember_stream(r, s);
  return UGC_OK;
}

int ugc_reserve_batch(ugc_ctx* c, int replica_id, uint32_t max_batch) {
  Replica* r;
  UGC_TRY(get_replica(c, replica_id, true, &r));
  if (max_batch == 0 || max_batch > kMaxBatch) return fail(UGC_ERR_INVALID, "max_batch must be in [1, 2^28]");
  if (max_batch <= r->max_batch) return UGC_OK;
  UGC_CUDA(cudaSetDevice(r->device));
  UGC_TRY(drain_lookups(r));  // the old lists may still be in use by lookups in flight
  uint64_t* fresh[kNumGroup] = {nullptr, nullptr, nullptr};
  for (int g = 0; g < kNumGroup; g++) {
    fresh[g] = static_cast<uint64_t*>(ctx_alloc(c, (size_t)max_batch * sizeof(uint64_t)));
    if (!fresh[g]) {
      for (int k = 0; k < g; k++) ctx_free(c, fresh[k]);
      return fail(UGC_ERR_NOMEM, "scratch allocation for %u keys failed", max_batch);
    }
  }
  for (int g = 0; g < kNumGroup; g++) {
    ctx_free(c, r->list[g]);
    r->list[g] = fresh[g];
  }
  ctx_free(c, r->host_sorted);  // sized by max_batch: re-made on the next ordered lookup
  r->host_sorted = nullptr;
  r->max_batch = max_batch;
  return UGC_OK;
}

int ugc_lookup_host(ugc_ctx* c, int replica_id, const void* keys, int key_bytes, size_t n, void* out,
                    void* stream) {
  Replica* r;
  UGC_TRY(get_replica(c, replica_id, true, &r));
  if (key_bytes != 4 && key_bytes != 8) return fail(UGC_ERR_INVALID, "key_bytes must be 4 or 8");
  if (n == 0) return UGC_OK;
  if (!keys || !out) return fail(UGC_ERR_INVALID, "keys and out must be non-null");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  UGC_CUDA(cudaSetDevice(r->device));
  // Pinned buffers that the GPU has mapped are used in place: the kernel reads the keys and
  // writes the rows across PCIe itself.
  const void* keys_dev = (r->host_zero_copy & 1) ? mapped_device_pointer(keys) : nullptr;
  void* out_dev = (r->host_zero_copy & 2) ? mapped_device_pointer(out) : nullptr;
  if (!keys_dev) {
    UGC_TRY(ensure(c, r->stage_keys, n * (size_t)key_bytes));
    UGC_CUDA(cudaMemcpyAsync(r->stage_keys.ptr, keys, n * (size_t)key_bytes, cudaMemcpyHostToDevice, s));
    keys_dev = r->stage_keys.ptr;
  }
  if (out_dev) {
    UGC_TRY(do_lookup(c, r, keys_dev, key_bytes, n, out_dev, s));
    UGC_CUDA(cudaStreamSynchronize(s));
    return UGC_OK;
  }
  // Rows are staged in device memory and leave through the copy engine, which moves them
  // faster than stores from the SMs do.  Large batches go in pieces: while piece i crosses
  // PCIe on a second stream, piece i+1 is being extracted.
  const size_t rb = c->cfg.row_bytes;
  UGC_TRY(ensure(c, r->stage_out, n * rb));
  // four pieces, the first half the size of the others: the copy engine starts early and then
  // runs few, large copies (each copy costs about 10 us of its own)
  const size_t pieces = n >= (1u << 16) ? 4 : 1;
  const size_t first = pieces > 1 ? (n / 7 + 31) / 32 * 32 : n;          // multiples of 32 keys keep
  const size_t piece = pieces > 1 ? ((n - first) / 3 + 31) / 32 * 32 : n;  // every piece aligned
  if (pieces > 1) {
    if (!r->copy_stream) UGC_CUDA(cudaStreamCreateWithFlags(&r->copy_stream, cudaStreamNonBlocking));
    while (r->copy_events.size() < pieces + 1) {
      cudaEvent_t e;
      UGC_CUDA(cudaEventCreateWithFlags(&e, cudaEventDisableTiming));
      r->copy_events.push_back(e);
    }
  }
  const char* kp = static_cast<const char*>(keys_dev);
  char* stage = static_cast<char*>(r->stage_out.ptr);
  size_t idx = 0;
  for (size_t off = 0; off < n; idx++) {
    const size_t m = std::min(idx == 0 ? first : piece, n - off);
    UGC_TRY(do_lookup(c, r, kp + off * (size_t)key_bytes, key_bytes, m, stage + off * rb, s));
    if (pieces > 1) {
      UGC_CUDA(cudaEventRecord(r->copy_events[idx], s));
      UGC_CUDA(cudaStreamWaitEvent(r->copy_stream, r->copy_events[idx], 0));
      UGC_CUDA(cudaMemcpyAsync(static_cast<char*>(out) + off * rb, stage + off * rb, m * rb,
                               cudaMemcpyDeviceToHost, r->copy_stream));
    } else {
      UGC_CUDA(cudaMemcpyAsync(out, stage, m * rb, cudaMemcpyDeviceToHost, s));
    }
    off += m;
  }
  if (pieces > 1) UGC_CUDA(cudaStreamSynchronize(r->copy_stream));
  UGC_CUDA(cudaStreamSynchronize(s));
  return UGC_OK;
}

// --------------------------------------------------------------------------------------
// refresh
// --------------------------------------------------------------------------------------
int ugc_refresh_set_placement(ugc_ctx* c, const uint32_t* n2b, const uint8_t* bp, const uint8_t* ba,
                              const double* bd, int B) {
  if (c && !c->cur.valid) return fail(UGC_ERR_STATE, "no current placement");
  return load_placement(c, c ? &c->next : nullptr, n2b, bp, ba, bd, B);
}

int ugc_refresh_evict(ugc_ctx* c, int replica_id, void* stream) {
  Replica* r;
  UGC_TRY(get_replica(c, replica_id, true, &r));
  if (!c->next.valid) return fail(UGC_ERR_STATE, "call ugc_refresh_set_placement first");
  if (r->refresh_open) return fail(UGC_ERR_STATE, "a refresh is already open on replica %d", replica_id);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int G = c->cfg.num_device;
  const int me = replica_id;
  UGC_CUDA(cudaSetDevice(r->device));

  // steps 1-4 of the reference's refresh in one pass over the id space on the GPU: keys whose
  // source changed, as ascending lists (evict here / bring in here / drop a peer entry /
  // point to a peer)
  UGC_TRY(upload_n2b(c, c->next, &r->n2b_next, s));
  UGC_TRY(gpu_classify(c, r, &c->cur, c->next, r->n2b_dev, r->n2b_next, s));
  const uint64_t n_evict = r->list_count[kListEvict], n_insert = r->list_count[kListInsert];
  const uint64_t n_drop = r->list_count[kListDropRemote];
  const uint64_t n_new_local = r->n_local - n_evict + n_insert;
  // a placement that does not fit is refused before anything changed: give back what the
  // classification allocated so that a later refresh starts clean
  auto refuse = [&](int rc) {
    std::string keep = g_last_error;
    ctx_free(c, r->n2b_next);
    r->n2b_next = nullptr;
    ctx_free(c, r->lists.ptr);
    r->lists = DevBuf{};
    g_last_error = keep;
    return rc;
  };
  if (n_new_local > r->capacity)
    return refuse(fail(UGC_ERR_CAPACITY, "new placement stores %llu rows on replica %d, slice holds %llu",
                (unsigned long long)n_new_local, me, (unsigned long long)r->capacity));
  uint64_t n_attach = 0;
  for (int s2 = 0; s2 < G; s2++)
    if (s2 != me) n_attach += r->list_count[kListAttach0 + s2];
  const uint64_t n_new_entries = r->n_local + r->n_remote - n_evict - n_drop + n_insert + n_attach;
  if (r->table.kind == kTableHashed && n_new_entries > r->table_entry_cap)
    return refuse(fail(UGC_ERR_CAPACITY, "new placement needs %llu table entries, table is sized for %llu",
                       (unsigned long long)n_new_entries, (unsigned long long)r->table_entry_cap));
  if (n_insert > r->free_count + n_evict)
    return refuse(fail(UGC_ERR_CAPACITY, "refresh needs %llu free slots, %llu available",
                       (unsigned long long)n_insert, (unsigned long long)(r->free_count + n_evict)));

  // Keys that leave their source for a peer that holds the row ALREADY (rows leaving the
  // replicated set, typically the hottest keys a refresh moves) are re-pointed to that peer
  // in place instead of being removed now and attached three phases later: between those two
  // moments every lookup of such a key would go to the host table (measured at 2 GPUs on the
  // 400 M x 64 configuration: 41 % of a batch, 5.2 ms per lookup against 1.1 ms).  The attach
  // phase finds these entries in place and leaves them.  The reference removes first and
  // inserts after its fill (coll_cache_lib/cache_context.cu:3103-3136, :4086-4100).
  RepointParams rp{};
  rp.own = r->table;
  for (int p2 = 0; p2 < G; p2++)
    if (p2 != me && r->peer_known[p2] && r->src_base[p2] && r->early_repoint) rp.peer[p2] = r->peer_table[p2];
  rp.n2b_new = r->n2b_next;
  rp.acc_new = static_cast<const uint8_t*>(r->acc_dev.ptr) + (size_t)c->cur.num_block;
  rp.me = (uint32_t)me;
  rp.num_device = (uint32_t)G;
  // step 3: evicted rows give their slots back (written by the resolve kernel straight to the
  // tail of the free ring; the slot numbers never visit the host), then leave the table
  if (n_evict) {
    const SlotView tail{r->free_ring, (uint32_t)((r->free_head + r->free_count) % r->capacity),
                        (uint32_t)r->capacity};
    UGC_CUDA(launch_table_resolve(r->table, list_ptr(r, kListEvict), (uint32_t)n_evict, (uint32_t)me, tail,
                                  r->counters, s));
    UGC_CUDA(launch_table_repoint(rp, list_ptr(r, kListEvict), (uint32_t)n_evict, r->counters, s));
    UGC_TRY(check_table_errors(r, s, "refresh evict"));
    r->free_count += n_evict;
  }
  // step 4: remote entries whose source changed (coll_cache_lib/cache_context.cu:3103-3136)
  if (n_drop) {
    UGC_CUDA(launch_table_repoint(rp, list_ptr(r, kListDropRemote), (uint32_t)n_drop, r->counters, s));
    UGC_TRY(check_table_errors(r, s, "refresh evict remote"));
  }
  // Grace period.  A lookup that was enqueued before the evictions above completed may hold a
  // record naming a slot that is about to be given to another key (here, or on a peer that this
  // replica just stopped reading from).  Every lookup of this replica enqueued so far is
  // drained before the call returns (by its finished-lookup counter, no stream is stalled);
  // the caller's barrier between the evict and fill phases then keeps every replica's fill
  // behind every replica's drain.  Lookups enqueued from now on see only the tables without
  // the evicted entries.
  UGC_TRY(drain_lookups(r));
  r->next_n_local = n_new_local;
  r->refresh_open = true;
  return UGC_OK;
}

int ugc_refresh_fill(ugc_ctx* c, int replica_id, void* stream) {
  Replica* r;
  UGC_TRY(get_replica(c, replica_id, true, &r));
  if (!r->refresh_open) return fail(UGC_ERR_STATE, "call ugc_refresh_evict first");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  UGC_CUDA(cudaSetDevice(r->device));
  const size_t n = (size_t)r->list_count[kListInsert];
  if (n) {
    // new rows take slots from the HEAD of the free ring
    // (coll_cache_lib/cuda/cache_hashtable.cuh:637-645)
    if (n > r->free_count) return fail(UGC_ERR_CAPACITY, "refresh fill: free slots ran out");
    const SlotView head{r->free_ring, (uint32_t)r->free_head, (uint32_t)r->capacity};
    // The refill must not stand in the way of running lookups: a small grid (the reference
    // limits it to 20 blocks, coll_cache_lib/cache_context.cu:4067), in batches of 131,072 rows
    // so that no fill CTA stays resident for long, on a stream of the lowest priority (the
    // reference's low_pri_stream, coll_cache_lib/facade.cc:376) tied to the caller's stream
    // by events.  An extraction kernel that needs every SM slot of the GPU for its one wave
    // then gets the slots between two batches.
    if (!r->fill_stream) {
      int lo = 0, hi = 0;
      UGC_CUDA(cudaDeviceGetStreamPriorityRange(&lo, &hi));
      UGC_CUDA(cudaStreamCreateWithPriority(&r->fill_stream, cudaStreamNonBlocking, lo));
      UGC_CUDA(cudaEventCreateWithFlags(&r->fill_ev[0], cudaEventDisableTiming));
      UGC_CUDA(cudaEventCreateWithFlags(&r->fill_ev[1], cudaEventDisableTiming));
    }
    UGC_CUDA(cudaEventRecord(r->fill_ev[0], s));
    UGC_CUDA(cudaStreamWaitEvent(r->fill_stream, r->fill_ev[0], 0));
    const size_t batch = (size_t)std::max(r->refresh_fill_batch_rows, 1024);
    for (size_t off = 0; off < n; off += batch) {
      const size_t m = std::min(batch, n - off);
      SlotView part = head;
      part.base = (uint32_t)((r->free_head + off) % r->capacity);
      UGC_CUDA(launch_fill_scatter(c->host_dev, r->slice, list_ptr(r, kListInsert) + off, part, (uint32_t)m,
                                   c->cfg.row_bytes, c->cfg.empty_feat, r->refresh_fill_ctas, r->fill_stream));
      if (r->refresh_fill_pause_us > 0 && off + batch < n) {
        // optional pacing, as the reference's 3 ms sleeps between its 4092-row batches
        // (coll_cache_lib/cache_context.cu:4061-4070); off by default
        UGC_CUDA(cudaStreamSynchronize(r->fill_stream));
        usleep((useconds_t)r->refresh_fill_pause_us);
      }
    }
    UGC_CUDA(cudaEventRecord(r->fill_ev[1], r->fill_stream));
    UGC_CUDA(cudaStreamWaitEvent(s, r->fill_ev[1], 0));
    UGC_CUDA(launch_table_insert(r->table, list_ptr(r, kListInsert), head, (uint32_t)replica_id, (uint32_t)n,
                                 r->counters, s));
    UGC_TRY(check_table_errors(r, s, "refresh insert"));
    r->free_head = (r->free_head + n) % r->capacity;
    r->free_count -= n;
  }
  return UGC_OK;
}

int ugc_refresh_attach(ugc_ctx* c, int replica_id, void* stream) {
  Replica* r;
  UGC_TRY(get_replica(c, replica_id, true, &r));
  if (!r->refresh_open) return fail(UGC_ERR_STATE, "call ugc_refresh_evict first");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  UGC_CUDA(cudaSetDevice(r->device));
  const int G = c->cfg.num_device;
  for (int src = 0; src < G; src++) {
    if (src == replica_id) continue;
    UGC_TRY(attach_keys(c, r, src, list_ptr(r, kListAttach0 + src), r->list_count[kListAttach0 + src], s));
  }
  uint64_t attach_total = 0;
  for (int src = 0; src < G; src++)
    if (src != replica_id) attach_total += r->list_count[kListAttach0 + src];
  r->n_remote = r->n_remote - r->list_count[kListDropRemote] + attach_total;
  r->n_local = r->next_n_local;
  std::swap(r->n2b_dev, r->n2b_next);
  ctx_free(c, r->n2b_next);
  r->n2b_next = nullptr;
  ctx_free(c, r->lists.ptr);
  r->lists = DevBuf{};
  r->refresh_open = false;
  return UGC_OK;
}

int ugc_refresh_commit(ugc_ctx* c) {
  if (!c) return fail(UGC_ERR_INVALID, "null context");
  if (!c->next.valid) return fail(UGC_ERR_STATE, "no new placement to commit");
  for (auto& r : c->reps)
    if (r.built && r.refresh_open)
      return fail(UGC_ERR_STATE, "replica %d has not finished its refresh", r.id);
  std::swap(c->cur, c->next);  // the old placement's storage serves the next refresh
  c->next.valid = false;
  return UGC_OK;
}

// --------------------------------------------------------------------------------------
int ugc_record(ugc_ctx* c, int replica_id, const void* keys, int key_bytes, size_t n, void* stream) {
  Replica* r;
  UGC_TRY(get_replica(c, replica_id, true, &r));
  if (key_bytes != 4 && key_bytes != 8) return fail(UGC_ERR_INVALID, "key_bytes must be 4 or 8");
  if (n == 0) return UGC_OK;
  if (!keys || n > 0xffffffffull) return fail(UGC_ERR_INVALID, "bad key batch");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  UGC_CUDA(cudaSetDevice(r->device));
  if (!r->hot_counts) {
    const size_t bytes = (size_t)c->cfg.num_total_item * sizeof(uint32_t);
    r->hot_counts = static_cast<uint32_t*>(ctx_alloc(c, bytes));
    if (!r->hot_counts) return fail(UGC_ERR_NOMEM, "hotness counters (%zu bytes) could not be allocated", bytes);
    UGC_CUDA(cudaMemsetAsync(r->hot_counts, 0, bytes, s));
  }
  UGC_CUDA(launch_record(keys, key_bytes, (uint32_t)n, r->hot_counts, c->cfg.num_total_item, s));
  return UGC_OK;
}

int ugc_hotness_read(ugc_ctx* c, int replica_id, uint32_t* counts_out, int reset, void* stream) {
  Replica* r;
  UGC_TRY(get_replica(c, replica_id, true, &r));
  if (!counts_out) return fail(UGC_ERR_INVALID, "null output");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  UGC_CUDA(cudaSetDevice(r->device));
  const size_t bytes = (size_t)c->cfg.num_total_item * sizeof(uint32_t);
  if (!r->hot_counts) {
    memset(counts_out, 0, bytes);
    return UGC_OK;
  }
  UGC_CUDA(cudaMemcpyAsync(counts_out, r->hot_counts, bytes, cudaMemcpyDeviceToHost, s));
  if (reset) UGC_CUDA(cudaMemsetAsync(r->hot_counts, 0, bytes, s));
  UGC_CUDA(cudaStreamSynchronize(s));
  return UGC_OK;
}

int ugc_stats(ugc_ctx* c, int replica_id, ugc_stats_t* out) {
  Replica* r;
  UGC_TRY(get_replica(c, replica_id, true, &r));
  if (!out) return fail(UGC_ERR_INVALID, "null output");
  UGC_CUDA(cudaSetDevice(r->device));
  Counters h;
  UGC_TRY(read_counters(r, &h));
  memset(out, 0, sizeof(*out));
  out->num_local_rows = r->n_local;
  out->num_remote_keys = r->n_remote;
  out->num_host_keys = c->cfg.num_total_item - out->num_local_rows - out->num_remote_keys;
  out->capacity_rows = r->capacity;
  out->free_rows = r->free_count;
  out->table_kind = r->table.kind;
  out->table_bytes = r->table_bytes;
  out->slice_bytes = r->slice_bytes;
  if (r->last_was_direct) {  // counts of a direct launch sit in the slot it owned
    out->last_keys = r->last_n;
    out->last_local = h.dcount[r->last_slot][kGroupLocal];
    out->last_remote = h.dcount[r->last_slot][kGroupRemote];
    out->last_host = h.dcount[r->last_slot][kGroupHost];
  } else {
    out->last_keys = h.last_keys;
    out->last_local = h.last_count[kGroupLocal];
    out->last_remote = h.last_count[kGroupRemote];
    out->last_host = h.last_count[kGroupHost];
  }
  out->err_key_range = h.err_key_range;
  out->err_table = h.err_table;
  out->lookups = r->lookups;
  auto span = [&](int g) -> uint64_t {
    return (h.t_end[g] > h.t_start && h.t_start) ? (uint64_t)(h.t_end[g] - h.t_start) : 0;
  };
  out->last_local_ns = span(kGroupLocal);
  out->last_remote_ns = span(kGroupRemote);
  out->last_host_ns = span(kGroupHost);
  out->last_index_ns = (h.t_index && h.t_start > h.t_index) ? (uint64_t)(h.t_start - h.t_index) : 0;
  {
    std::lock_guard<std::mutex> lock(c->acct_mu);
    out->device_bytes_from_allocator = c->bytes_from_allocator;
    out->device_bytes_own = c->bytes_own;
  }
  out->lookups_host_ordered = r->lookups_host_ordered;
  out->lookups_direct = r->lookups_direct;
  out->kernel_launches = r->kernel_launches;
  out->lookups_pooled = r->lookups_pooled;
  for (int g = 0; g < kNumGroup; g++) out->pool_rows[g] = h.pool_rows[g];
  return UGC_OK;
}

int ugc_get_tuning(ugc_ctx* c, int replica_id, ugc_tuning* out) {
  Replica* r;
  UGC_TRY(get_replica(c, replica_id, true, &r));
  if (!out) return fail(UGC_ERR_INVALID, "null output");
  memset(out, 0, sizeof(*out));
  out->struct_size = sizeof(*out);
  out->gather_ctas_per_sm = r->gather_grid / std::max(r->sm_count, 1);
  out->gather_block_threads = r->block_threads;
  out->gather_vec_bytes = r->vec_bytes;
  out->host_ctas = r->host_ctas;
  out->remote_ctas = r->remote_ctas;
  out->bulk_mask = r->bulk_mask;
  out->lookup_keys_per_thread = r->lookup_kpt;
  out->programmatic_launch = r->pdl;
  out->extract_mode = r->extract_mode;
  out->direct_ctas_per_sm = r->direct_grid / std::max(r->sm_count, 1);
  out->direct_max_host_rows = r->direct_max_host_rows;
  out->direct_block_threads = r->direct_block;
  out->host_zero_copy = r->host_zero_copy;
  out->gather_dynamic = r->gather_dynamic;
  out->split_fixed = r->split_fixed;
  out->direct_tile_keys = r->direct_tile_shift ? (1 << r->direct_tile_shift) : 0;
  out->direct_deep = r->direct_deep;
  out->direct_early_host = r->direct_early_host;
  out->host_order_min_rows = r->host_order_min_rows;
  out->refresh_fill_ctas = r->refresh_fill_ctas;
  out->refresh_fill_batch_rows = r->refresh_fill_batch_rows;
  out->refresh_fill_pause_us = r->refresh_fill_pause_us;
  out->refresh_early_repoint = r->early_repoint;
  out->pool_vec_bytes = r->pool_vec_bytes;
  return UGC_OK;
}

int ugc_set_tuning(ugc_ctx* c, int replica_id, const ugc_tuning* t) {
  Replica* r;
  UGC_TRY(get_replica(c, replica_id, true, &r));
  if (!t || t->struct_size != sizeof(ugc_tuning)) return fail(UGC_ERR_INVALID, "bad ugc_tuning");
  const int bt = t->gather_block_threads, kpt = t->lookup_keys_per_thread, vec = t->gather_vec_bytes;
  if (t->gather_ctas_per_sm < 1 || t->gather_ctas_per_sm > 32 || (bt != 256 && bt != 512 && bt != 1024) ||
      (vec != 16 && vec != 32) || t->host_ctas < 1 || t->remote_ctas < 1 || t->bulk_mask < 0 ||
      t->bulk_mask > 3 || (kpt != 1 && kpt != 2 && kpt != 4) || t->extract_mode < UGC_EXTRACT_AUTO ||
      t->extract_mode > UGC_EXTRACT_DIRECT || t->direct_ctas_per_sm < 1 || t->direct_ctas_per_sm > 16 ||
      t->direct_max_host_rows < 0 || (t->direct_block_threads != 128 && t->direct_block_threads != 256) ||
      t->host_zero_copy < 0 || t->host_zero_copy > 3)
    return fail(UGC_ERR_INVALID, "ugc_tuning holds a value outside its range");
  r->gather_grid = r->sm_count * t->gather_ctas_per_sm;
  r->block_threads = bt;
  r->vec_bytes = vec;
  r->host_ctas = t->host_ctas;
  r->remote_ctas = t->remote_ctas;
  r->bulk_mask = t->bulk_mask;
  r->lookup_kpt = kpt;
  r->pdl = t->programmatic_launch & 3;
  r->extract_mode = t->extract_mode;
  r->direct_grid = r->sm_count * t->direct_ctas_per_sm;
  r->direct_max_host_rows = t->direct_max_host_rows;
  r->direct_block = t->direct_block_threads;
  r->host_zero_copy = t->host_zero_copy;
  r->gather_dynamic = t->gather_dynamic ? 1 : 0;
  r->split_fixed = t->split_fixed ? 1 : 0;
  r->direct_tile_shift = t->direct_tile_keys == 8 ? 3 : t->direct_tile_keys == 16 ? 4 : t->direct_tile_keys == 32 ? 5 : 0;
  r->direct_deep = t->direct_deep ? 1 : 0;
  r->direct_early_host = (t->direct_early_host >= 0 && t->direct_early_host <= 2) ? t->direct_early_host : 0;
  r->host_order_min_rows = t->host_order_min_rows < 0 ? 0 : t->host_order_min_rows;
  if (t->refresh_fill_ctas > 0) r->refresh_fill_ctas = t->refresh_fill_ctas;
  if (t->refresh_fill_batch_rows > 0) r->refresh_fill_batch_rows = t->refresh_fill_batch_rows;
  r->refresh_fill_pause_us = t->refresh_fill_pause_us < 0 ? 0 : t->refresh_fill_pause_us;
  r->early_repoint = t->refresh_early_repoint ? 1 : 0;
  r->pool_vec_bytes = (t->pool_vec_bytes == 16 || t->pool_vec_bytes == 4) ? t->pool_vec_bytes : 0;
  return UGC_OK;
}

int ugc_profile_begin(ugc_ctx* c, int replica_id, int max_lookups) {
  Replica* r;
  UGC_TRY(get_replica(c, replica_id, true, &r));
  if (max_lookups < 1 || max_lookups > (1 << 20)) return fail(UGC_ERR_INVALID, "max_lookups out of range");
  UGC_CUDA(cudaSetDevice(r->device));
  while (r->prof_events.size() < (size_t)max_lookups * 3) {
    cudaEvent_t e;
    UGC_CUDA(cudaEventCreate(&e));
    r->prof_events.push_back(e);
  }
  r->prof_used = 0;
  r->prof_on = true;
  return UGC_OK;
}

int ugc_profile_end(ugc_ctx* c, int replica_id, double* lookup_ms, double* gather_ms, uint64_t* lookups) {
  Replica* r;
  UGC_TRY(get_replica(c, replica_id, true, &r));
  if (!lookup_ms || !gather_ms || !lookups) return fail(UGC_ERR_INVALID, "null output");
  if (!r->prof_on) return fail(UGC_ERR_STATE, "profiling is not on");
  UGC_CUDA(cudaSetDevice(r->device));
  UGC_CUDA(cudaDeviceSynchronize());
  double a = 0, b = 0;
  for (size_t i = 0; i + 3 <= r->prof_used; i += 3) {
    float ms = 0;
    UGC_CUDA(cudaEventElapsedTime(&ms, r->prof_events[i], r->prof_events[i + 1]));
    a += ms;
    UGC_CUDA(cudaEventElapsedTime(&ms, r->prof_events[i + 1], r->prof_events[i + 2]));
    b += ms;
  }
  *lookup_ms = a;
  *gather_ms = b;
  *lookups = r->prof_used / 3;
  r->prof_on = false;
  r->prof_used = 0;
  return UGC_OK;
}

int ugc_table_words(ugc_ctx* c, int replica_id, const uint32_t* keys, size_t n, uint32_t* words,
                    void* stream) {
  Replica* r;
  UGC_TRY(get_replica(c, replica_id, true, &r));
  UGC_CUDA(cudaSetDevice(r->device));
  UGC_CUDA(launch_table_words(r->table, keys, (uint32_t)n, words, static_cast<cudaStream_t>(stream)));
  return UGC_OK;
}

// Registration goes chunk by chunk: one call over tens of GB of a shared-memory mapping was
// refused by the OS on the test machines, 1 GiB pieces are accepted.
static const size_t kRegisterChunk = (size_t)1 << 30;

int ugc_host_unregister_sized(void* host_ptr, size_t nbytes) {
  if (!host_ptr) return fail(UGC_ERR_INVALID, "null argument");
  char* base = static_cast<char*>(host_ptr);
  int rc = UGC_OK;
  for (size_t off = 0; off < std::max<size_t>(nbytes, 1); off += kRegisterChunk) {
    cudaError_t e = cudaHostUnregister(base + off);
    if (e != cudaSuccess) {
      cudaGetLastError();
      rc = fail(UGC_ERR_CUDA, "cudaHostUnregister failed: %s", cudaGetErrorString(e));
    }
  }
  return rc;
}

int ugc_host_unregister(void* host_ptr) { return ugc_host_unregister_sized(host_ptr, 1); }

int ugc_host_register(void* host_ptr, size_t nbytes, void** dev_ptr) {
  if (!host_ptr || !nbytes || !dev_ptr) return fail(UGC_ERR_INVALID, "null argument");
  char* base = static_cast<char*>(host_ptr);
  size_t done = 0;
  while (done < nbytes) {
    size_t len = std::min(kRegisterChunk, nbytes - done);
    cudaError_t e = cudaHostRegister(base + done, len, cudaHostRegisterPortable | cudaHostRegisterMapped);
    if (e != cudaSuccess) {
      cudaGetLastError();
      for (size_t off = 0; off < done; off += kRegisterChunk) cudaHostUnregister(base + off);
      cudaGetLastError();
      return fail(UGC_ERR_CUDA, "cudaHostRegister of %zu bytes at offset %zu failed: %s", len, done,
                  cudaGetErrorString(e));
    }
    done += len;
  }
  void* d0 = nullptr;
  UGC_CUDA(cudaHostGetDevicePointer(&d0, host_ptr, 0));
  // the chunks must form one contiguous device range (true with unified addressing)
  for (size_t off = kRegisterChunk; off < nbytes; off += kRegisterChunk) {
    void* d = nullptr;
    UGC_CUDA(cudaHostGetDevicePointer(&d, base + off, 0));
    if (d != static_cast<char*>(d0) + off) {
      ugc_host_unregister_sized(host_ptr, nbytes);
      return fail(UGC_ERR_UNSUPPORTED, "registered chunks are not contiguous on the device");
    }
  }
  *dev_ptr = d0;
  return UGC_OK;
}

int ugc_host_alloc(size_t nbytes, void** host_ptr, void** dev_ptr) {
  if (!nbytes || !host_ptr || !dev_ptr) return fail(UGC_ERR_INVALID, "null argument");
  UGC_CUDA(cudaFree(0));  // make sure the primary context exists
  size_t mapped = 0;
  void* p = vmm_host_alloc(nbytes, &mapped);
  if (p) {
    *host_ptr = p;
    *dev_ptr = p;  // one address for CPU and GPU
    return UGC_OK;
  }
  cudaError_t e = cudaHostAlloc(host_ptr, nbytes, cudaHostAllocPortable | cudaHostAllocMapped);
  if (e != cudaSuccess) {
    cudaGetLastError();
    return fail(UGC_ERR_NOMEM, "cudaHostAlloc of %zu bytes failed: %s", nbytes, cudaGetErrorString(e));
  }
  UGC_CUDA(cudaHostGetDevicePointer(dev_ptr, *host_ptr, 0));
  return UGC_OK;
}

int ugc_host_is_large_page(const void* host_ptr) {
  std::lock_guard<std::mutex> lock(g_vmm_mu);
  return g_vmm_blocks.count(const_cast<void*>(host_ptr)) ? 1 : 0;
}

int ugc_host_free(void* host_ptr) {
  if (!host_ptr) return UGC_OK;
  if (vmm_host_free(host_ptr)) return UGC_OK;
  UGC_CUDA(cudaFreeHost(host_ptr));
  return UGC_OK;
}


int ugc_gen_table(void* dst, uint64_t seed, uint64_t row_begin, uint64_t n_rows, uint64_t dim,
                  int elem_bytes, void* stream) {
  if (!dst) return fail(UGC_ERR_INVALID, "null destination");
  if (elem_bytes != 4 && elem_bytes != 2) return fail(UGC_ERR_INVALID, "elem_bytes must be 4 or 2");
  if (elem_bytes == 2 && dim % 2) return fail(UGC_ERR_INVALID, "fp16 rows need an even dim");
  UGC_CUDA(launch_gen_table(dst, seed, row_begin, n_rows, dim, elem_bytes, static_cast<cudaStream_t>(stream)));
  return UGC_OK;
}

}  // extern "C"
