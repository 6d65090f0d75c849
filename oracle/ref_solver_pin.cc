// Reference pin for the placement heuristics: runs THE REFERENCE'S OWN solver classes
// (IntuitiveSolver, RepSolver, CliquePartSolver; their source is compiled in place from the
// reference tree, none of it is copied) on a hotness ranking read from a file and writes the
// placement they produce.  tests/golden/make_solver_pin.py stores digests of the per-key result
// in tests/golden/ref_solver.json, which pins the CPU oracle's (and through it the library's)
// solvers.  Test infrastructure only; no GPU is needed.
//
//   ref_solver_pin <dir>
// <dir>/solver_case.bin: u32 {G, N, policy (0 intuitive, 1 rep, 2 clique_part), clique_size},
//   f64 {cache_percent, T_local, T_remote, T_cpu}, u32 rank_ids[N], u32 rank_freqs[N]
// writes <dir>/ref_nid_to_block.bin (u32 [N]) and <dir>/ref_blocks.bin:
//   u32 num_block, u8 placement[num_block], u8 access_from[G * num_block], f64 density[num_block]
#include <sys/mman.h>
#include <unistd.h>

#include <cstdio>
#include <cstdlib>
#include <string>
#include <vector>

#include "coll_cache_lib/coll_cache/optimal_solver_class.cc"

using namespace coll_cache_lib::common;
using namespace coll_cache_lib::common::coll_cache;

static void die(const char* m) {
  fprintf(stderr, "ref_solver_pin: %s\n", m);
  exit(2);
}

int main(int argc, char** argv) {
  if (argc != 2) die("usage: ref_solver_pin <dir>");
  const std::string dir = argv[1];
  FILE* f = fopen((dir + "/solver_case.bin").c_str(), "rb");
  if (!f) die("cannot open solver_case.bin");
  uint32_t head[4];
  double par[4];
  if (fread(head, 4, 4, f) != 4 || fread(par, 8, 4, f) != 4) die("short header");
  const uint32_t G = head[0], N = head[1], policy = head[2], clique = head[3];
  std::vector<uint32_t> ids(N), freqs(N);
  if (fread(ids.data(), 4, N, f) != N || fread(freqs.data(), 4, N, f) != N) die("short ranking");
  fclose(f);

  RunConfig::num_device = G;
  RunConfig::omp_thread_num = 4;
  RunConfig::coll_cache_concurrent_link = false;
  RunConfig::coll_hash_impl = kDefault;
  RunConfig::coll_cache_hyperparam_T_local = par[1];
  RunConfig::coll_cache_hyperparam_T_remote = par[2];
  RunConfig::coll_cache_hyperparam_T_cpu = par[3];
  RunConfig::cache_policy = policy == 0 ? kCollCacheIntuitive : (policy == 1 ? kRepCache : kCliquePart);
  // link description as AsymmLinkDesc::AutoBuild(Context) would leave it on a switched 8-GPU
  // machine, without asking a GPU for its name (the SM numbers only enter a printed estimate)
  auto& desc = RunConfig::coll_cache_link_desc;
  desc.BuildSwitch(G);
  desc.cpu_sm.assign(G, 10);
  desc.total_sm_for_remote.assign(G, 56);
  desc.local_sm.assign(G, 98);
  desc.SMPercentToNum(56);

  const std::string tag = "ugc_solver_pin_" + std::to_string(getpid());
  CollCacheSolver::_shm_name_place = tag + "_place";
  CollCacheSolver::_shm_name_access = tag + "_access";
  CollCacheSolver::_shm_name_dens = tag + "_dens";
  CollCacheSolver::_shm_name_nid_to_block = tag + "_n2b";

  auto id_list = Tensor::FromBlob(ids.data(), kI32, {1, (size_t)N}, CPU(CPU_FOREIGN), "rank_ids");
  auto freq_list = Tensor::FromBlob(freqs.data(), kI32, {1, (size_t)N}, CPU(CPU_FOREIGN), "rank_freqs");
  std::vector<uint32_t> n2b(N, 0xffffffffu);
  auto n2b_tensor = Tensor::FromBlob(n2b.data(), kI32, {(size_t)N}, CPU(CPU_FOREIGN), "nid_to_block");

  std::vector<int> device_to_stream(G, 0);
  std::vector<PerT> percent(G, par[0]);
  CollCacheSolver* solver = nullptr;
  if (policy == 0) solver = new IntuitiveSolver();
  if (policy == 1) solver = new RepSolver();
  if (policy == 2) {
    auto* cp = new CliquePartSolver();  // its clique size comes from the link description: all G GPUs
    if (clique) cp->clique_size = (int)clique;
    solver = cp;
  }
  if (!solver) die("unknown policy");
  solver->Build(id_list, freq_list, device_to_stream, N, n2b_tensor);
  solver->Solve(device_to_stream, percent, "BIN", par[1], par[3]);

  const uint32_t num_block = (uint32_t)solver->block_placement->Shape()[0];
  f = fopen((dir + "/ref_nid_to_block.bin").c_str(), "wb");
  if (!f || fwrite(n2b.data(), 4, N, f) != N) die("cannot write nid_to_block");
  fclose(f);
  f = fopen((dir + "/ref_blocks.bin").c_str(), "wb");
  if (!f) die("cannot write blocks");
  fwrite(&num_block, 4, 1, f);
  fwrite(solver->block_placement->CPtr<uint8_t>(), 1, num_block, f);
  fwrite(solver->block_access_from->CPtr<uint8_t>(), 1, (size_t)G * num_block, f);
  fwrite(solver->block_density_tensor->CPtr<double>(), 8, num_block, f);
  fclose(f);
  shm_unlink(CollCacheSolver::_shm_name_place.c_str());
  shm_unlink(CollCacheSolver::_shm_name_access.c_str());
  shm_unlink(CollCacheSolver::_shm_name_dens.c_str());
  return 0;
}
