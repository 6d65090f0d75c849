#include "placement.h"

#include <algorithm>
#include <cmath>
#include <omp.h>
#include <cstring>

#include "../../include/ugache_b200.h"

namespace ugc {

std::string validate_placement(const Placement& p, int G, uint64_t N, bool check_block_ids) {
  if (p.num_block <= 0) return "placement has no blocks";
  if (p.nid_to_block.size() != N) return "nid_to_block must have num_total_item entries";
  if (p.block_placement.size() != (size_t)p.num_block) return "block_placement size mismatch";
  if (p.block_access_from.size() != (size_t)G * p.num_block) return "block_access_from size mismatch";
  for (int b = 0; b < p.num_block; b++) {
    if (G < 8 && (p.block_placement[b] >> G)) return "block_placement names a GPU >= num_device";
    for (int g = 0; g < G; g++) {
      int s = p.access(g, b);
      if (s > G) return "block_access_from names a location > num_device";
      bool stored_here = (p.block_placement[b] >> g) & 1;
      if (s < G && !((p.block_placement[b] >> s) & 1))
        return "a reader's source does not store the block";
      if (stored_here != (s == g)) return "a GPU that stores a block must read its own copy (and only then)";
    }
  }
  if (!check_block_ids) return "";
  bool bad = false;
  const uint32_t nb = (uint32_t)p.num_block;
#pragma omp parallel for reduction(|| : bad)
  for (int64_t k = 0; k < (int64_t)N; k++) bad = bad || (p.nid_to_block[k] >= nb);
  if (bad) return "nid_to_block holds a block id >= num_block";
  return "";
}

void b200_link_model(int num_device, double* t_local, double* t_remote, double* t_cpu) {
  (void)num_device;
  *t_local = 1.0;
  *t_remote = 8000.0 / 900.0;
  *t_cpu = 8000.0 / 64.0;
}

LinkDesc b200_link_desc(int num_device, uint32_t row_bytes, double bw_local_override,
                        double bw_remote_override, double bw_host_override) {
  LinkDesc d;
  const int G = num_device < 1 ? 1 : num_device;
  d.num_device = G;
  // Nominal link rates of the platform; the host side of the machines measured sustains about
  // 100 GB/s for all GPUs together (eight concurrent device-to-host copies: 94 GB/s), so with
  // more than one GPU reading host rows each gets its share of that, not its own 64 GB/s.
  d.bw_local_gbs = bw_local_override > 0 ? bw_local_override : 8000.0;
  d.bw_remote_gbs = G > 1 ? (bw_remote_override > 0 ? bw_remote_override : 900.0) : 0.0;
  d.host_total_gbs = 100.0;
  // scattered rows of pinned memory, per GPU, measured: 55-60 M rows/s alone whatever the row
  // size from 128 to 512 bytes (63-68 M in ascending address order), about 30-45 M while the
  // same kernel also saturates HBM
  d.host_rows_per_s = 45e6;
  double host = bw_host_override > 0 ? bw_host_override : 64.0;
  if (bw_host_override <= 0) {
    host = std::min(host, d.host_total_gbs / G);
    if (row_bytes) host = std::min(host, d.host_rows_per_s * row_bytes / 1e9);
  }
  d.bw_host_gbs = host;
  d.lat_local_us = 0.8;
  d.lat_remote_us = 2.0;
  // Scattered rows of pinned host memory come back slowly once many are in flight (address
  // translation on the far side of PCIe): the measured ceiling is a row RATE, reached only
  // with tens of microseconds' worth of requests outstanding.
  d.lat_host_us = 20.0;
  // placement ratios keep the nominal rates (what the reference's tables hold: local / link)
  d.t_local = 1.0;
  d.t_remote = G > 1 ? d.bw_local_gbs / d.bw_remote_gbs : 0.0;
  d.t_cpu = d.bw_local_gbs / d.bw_host_gbs;
  // Little's law: bytes in flight = bandwidth x latency; one 256-thread CTA of the gather keeps
  // 256 x 16 B x 4 rows = 16 KiB in flight.  Twice that many CTAs as a margin for uneven rows.
  const double inflight = 256.0 * 16.0 * 4.0;
  auto ctas = [&](double bw_gbs, double lat_us) {
    int n = (int)std::ceil(bw_gbs * 1e3 * lat_us / inflight) * 2;
    return n < 2 ? 2 : n;
  };
  d.host_ctas = ctas(std::min(64.0, d.bw_host_gbs > 0 ? 64.0 : 0.0), d.lat_host_us);
  d.remote_ctas = G > 1 ? ctas(d.bw_remote_gbs, d.lat_remote_us) : 2;
  d.per_peer_ctas = G > 1 ? std::max(1, d.remote_ctas / (G - 1)) : 0;
  return d;
}

bool reference_prefers_flat_table(uint64_t num, uint64_t N) {
  uint64_t e = (uint64_t)(1.0 + std::log2((double)(num >> 1)));
  uint64_t table_size = ((uint64_t)1 << e) << 2;
  return table_size > N / 2;
}

uint64_t cache_capacity_rows(uint64_t N, double frac) { return (uint64_t)((double)N * (frac + 0.001)); }

namespace {

void alloc_out(Placement* out, int G, uint64_t N, int B) {
  out->nid_to_block.assign(N, 0);
  out->block_placement.assign(B, 0);
  out->block_access_from.assign((size_t)G * B, 0);
  out->block_density.assign(B, 0.0);
  out->num_block = B;
  out->num_device = G;
}

// Blocks of a replicate / partition / host split: ranks < L on every GPU (block 0), ranks
// L..R dealt round-robin (block 1 + rank % G), ranks > R on the host (block G + 1).
void emit_split(int G, uint32_t N, const uint32_t* ids, uint32_t L, uint32_t R, uint32_t part,
                Placement* out) {
#pragma omp parallel for
  for (int64_t rank = 0; rank < (int64_t)N; rank++) {
    uint32_t b;
    if ((uint32_t)rank < L) b = 0;
    else if ((uint32_t)rank <= R) b = (uint32_t)rank % (uint32_t)G + 1;
    else b = (uint32_t)G + 1;
    out->nid_to_block[ids[rank]] = b;
  }
  const int B = G + 2;
  out->block_placement[0] = (uint8_t)((1 << G) - 1);
  for (int g = 0; g < G; g++) out->block_placement[g + 1] = (uint8_t)(1 << g);
  for (int g = 0; g < G; g++) {
    uint8_t* row = &out->block_access_from[(size_t)g * B];
    row[0] = (uint8_t)g;
    for (int b = 1; b <= G; b++) row[b] = (uint8_t)(b - 1);
    row[G + 1] = (uint8_t)G;
  }
  out->block_density[0] = (double)L * 100 / (double)N;
  for (int b = 1; b <= G; b++) out->block_density[b] = part * 100.0 / (double)N;
  out->block_density[G + 1] = 100 - (R / (double)N) * 100;
}

std::string solve_intuitive(int G, uint32_t N, const uint32_t* ids, const uint32_t* freq, double pct,
                            double T_local, double T_remote, double T_cpu, Placement* out) {
  if (!freq) return "the intuitive policy needs rank_freqs";
  alloc_out(out, G, N, G + 2);
  const uint32_t cached = (uint32_t)(N * (pct / 100.0));
  uint32_t lo = 0, hi = 0;
  if (G > 1) hi = std::min<uint32_t>(cached, (N - cached) / (uint32_t)(G - 1));
  auto lb = [&](uint32_t p) { return cached - p; };
  auto rb = [&](uint32_t p) { return std::max<uint32_t>(cached + p * (uint32_t)(G - 1), 1u) - 1u; };
  const double mu = 1 + (T_cpu - T_remote) / (T_remote - T_local) * G;
  auto colder = [&](uint32_t p) { return (double)freq[lb(p)] < (double)freq[rb(p)] * mu; };
  uint32_t part = lo;
  if (mu < 1) {
    part = lo;
  } else if (colder(hi)) {
    part = hi;
  } else {
    while (hi - lo > 1) {
      part = (lo + hi) / 2;
      if (colder(part)) lo = part; else hi = part;
    }
    part = hi;
  }
  emit_split(G, N, ids, lb(part), rb(part), part, out);
  return "";
}

// Hotness mass below a rank, from coarse prefix sums with linear interpolation inside a step.
struct HotnessPrefix {
  std::vector<double> sum;  // sum[j] = total frequency of ranks < j * step
  uint64_t step = 1, n = 0;
  void build(uint32_t N, const uint32_t* freq) {
    n = N;
    step = std::max<uint64_t>(1, N / 16384);
    const int64_t J = (int64_t)((N + step - 1) / step);
    std::vector<double> part((size_t)J, 0.0);
#pragma omp parallel for schedule(static)
    for (int64_t j = 0; j < J; j++) {
      const uint64_t end = std::min<uint64_t>(N, (uint64_t)(j + 1) * step);
      double a = 0;
      for (uint64_t r = (uint64_t)j * step; r < end; r++) a += (double)freq[r];
      part[(size_t)j] = a;
    }
    sum.assign((size_t)J + 1, 0.0);
    for (int64_t j = 0; j < J; j++) sum[(size_t)j + 1] = sum[(size_t)j] + part[(size_t)j];
  }
  double below(uint64_t rank) const {
    if (rank >= n) return sum.back();
    const uint64_t j = rank / step;
    const uint64_t width = std::min<uint64_t>(step, n - j * step);
    return sum[j] + (sum[j + 1] - sum[j]) * (double)(rank - j * step) / (double)width;
  }
};

// Modelled time of one GPU per unit of looked-up bytes when its sources are read concurrently
// (one launch, role-partitioned): the slowest of
//   HBM   : (bytes it reads from its own slice + bytes its peers read from its slice + every
//            output byte it writes) * t_local
//   links : bytes it reads from peers * t_remote
//   host  : bytes it reads from the host table * t_cpu
double concurrent_cost(double f_local, double f_remote, double f_host, double f_served,
                       double t_local, double t_remote, double t_cpu) {
  return std::max((f_local + f_served + 1.0) * t_local, std::max(f_remote * t_remote, f_host * t_cpu));
}

// Split search for a switch-connected box.  On a uniform topology the optimum of the reference's
// MILP (OptimalAsymmLinkSolver, coll_cache_lib/coll_cache/optimal_solver_class.cc:957-1112) has
// the shape the intuitive policy assumes: the hottest L ranks on every GPU, the next ranks dealt
// round-robin, the rest on the host, with L + part = capacity.  The only free variable is `part`,
// so every feasible value (in 4096 steps) is costed with the concurrent-source model against the
// recorded hotness and the cheapest kept; among equals the one with more replication wins
// (fewer rows cross the links).
std::string solve_split_search(int G, uint32_t N, const uint32_t* ids, const uint32_t* freq, double pct,
                               double T_local, double T_remote, double T_cpu, Placement* out) {
  if (!freq) return "the split-search policy needs rank_freqs";
  alloc_out(out, G, N, G + 2);
  const uint32_t cached = (uint32_t)(N * (pct / 100.0));
  uint32_t hi = 0;
  if (G > 1) hi = std::min<uint32_t>(cached, (N - cached) / (uint32_t)(G - 1));
  HotnessPrefix hp;
  hp.build(N, freq);
  const double total = std::max(hp.sum.back(), 1.0);
  uint32_t best_part = 0;
  double best = 0;
  const uint32_t kSteps = 4096;
  for (uint32_t i = 0; i <= kSteps; i++) {
    const uint32_t part = (uint32_t)((uint64_t)hi * i / kSteps);
    if (i && part == (uint32_t)((uint64_t)hi * (i - 1) / kSteps)) continue;
    const uint64_t L = cached - part, R = (uint64_t)cached + (uint64_t)part * (G - 1);
    const double f_rep = hp.below(L) / total, f_cov = hp.below(R) / total;
    const double f_part = f_cov - f_rep;
    // every GPU serves as much to its peers as it reads from them (same hotness on every reader)
    const double f_remote = f_part * (G - 1) / G;
    const double cost =
        concurrent_cost(f_rep + f_part / G, f_remote, 1.0 - f_cov, f_remote, T_local, T_remote, T_cpu);
    if (i == 0 || cost < best * (1 - 1e-9)) {
      best = cost;
      best_part = part;
    }
  }
  const uint32_t L = cached - best_part;
  const uint32_t R = std::max<uint32_t>(cached + best_part * (uint32_t)(G - 1), 1u) - 1u;
  emit_split(G, N, ids, L, R, best_part, out);
  return "";
}

std::string solve_rep(int G, uint32_t N, const uint32_t* ids, double pct, Placement* out) {
  alloc_out(out, G, N, 2);
  const uint32_t rep = (uint32_t)(N * (pct / 100.0));
#pragma omp parallel for
  for (int64_t rank = 0; rank < (int64_t)N; rank++) out->nid_to_block[ids[rank]] = (uint32_t)rank < rep ? 0 : 1;
  out->block_placement[0] = (uint8_t)((1 << G) - 1);
  for (int g = 0; g < G; g++) {
    out->block_access_from[(size_t)g * 2 + 0] = (uint8_t)g;
    out->block_access_from[(size_t)g * 2 + 1] = (uint8_t)G;
  }
  out->block_density[0] = (double)rep * 100 / (double)N;
  out->block_density[1] = (double)(N - rep) * 100 / (double)N;
  return "";
}

std::string solve_clique(int G, uint32_t N, const uint32_t* ids, double pct, Placement* out) {
  const int C = G;  // one NVSwitch domain: the clique is the whole box
  alloc_out(out, G, N, C + 1);
  const uint32_t cached = (uint32_t)std::ceil(N * (pct / 100.0));
  const uint32_t part = std::min<uint32_t>(cached, (N + (uint32_t)C - 1) / (uint32_t)C);
  const uint64_t covered = (uint64_t)part * C;
#pragma omp parallel for
  for (int64_t rank = 0; rank < (int64_t)N; rank++)
    out->nid_to_block[ids[rank]] = (uint64_t)rank < covered ? (uint32_t)rank % (uint32_t)C : (uint32_t)C;
  const int B = C + 1;
  for (int b = 0; b < C; b++) {
    out->block_placement[b] = (uint8_t)(1 << b);
    for (int g = 0; g < G; g++) out->block_access_from[(size_t)g * B + b] = (uint8_t)b;
    out->block_density[b] = (double)part * 100 / (double)N;
  }
  for (int g = 0; g < G; g++) out->block_access_from[(size_t)g * B + C] = (uint8_t)G;
  out->block_density[C] = ((double)N - (double)covered) * 100 / (double)N;
  return "";
}

}  // namespace

std::string solve_placement(int policy, int G, uint64_t N, const uint32_t* ids, const uint32_t* freq,
                            double pct, double T_local, double T_remote, double T_cpu, Placement* out) {
  if (G < 1 || G > UGC_MAX_DEVICE) return "num_device must be 1..8";
  if (N == 0 || N >= 0x7fffffffull) return "num_total_item must be in [1, 2^31-1)";
  if (!ids) return "rank_ids is required";
  if (pct < 0 || pct > 100) return "cache_percent must be in [0, 100]";
  std::string err;
  switch (policy) {
    case UGC_POLICY_INTUITIVE:
      err = solve_intuitive(G, (uint32_t)N, ids, freq, pct, T_local, T_remote, T_cpu, out);
      break;
    case UGC_POLICY_REP: err = solve_rep(G, (uint32_t)N, ids, pct, out); break;
    case UGC_POLICY_CLIQUE_PART: err = solve_clique(G, (uint32_t)N, ids, pct, out); break;
    case UGC_POLICY_SPLIT_SEARCH:
      err = solve_split_search(G, (uint32_t)N, ids, freq, pct, T_local, T_remote, T_cpu, out);
      break;
    default: return "unknown policy (supported: 9 intuitive, 12 rep, 14 clique_part, 100 split search)";
  }
  out->valid = err.empty();
  return err;
}

std::string placement_cost(const Placement& p, uint64_t N, const uint32_t* ids, const uint32_t* freq,
                           double T_local, double T_remote, double T_cpu, double* cost_per_reader,
                           const uint32_t* n2b_in_place) {
  const int G = p.num_device, B = p.num_block;
  if (!ids || !freq || !cost_per_reader) return "rank_ids, rank_freqs and the output are required";
  if (!n2b_in_place && p.nid_to_block.size() < N) return "placement is smaller than the id space";
  const uint32_t* n2b = n2b_in_place ? n2b_in_place : p.nid_to_block.data();
  std::vector<double> mass((size_t)B, 0.0);
  {
    const int T = omp_get_max_threads();
    std::vector<double> priv((size_t)T * B, 0.0);
#pragma omp parallel
    {
      double* mine = &priv[(size_t)omp_get_thread_num() * B];
#pragma omp for schedule(static)
      for (int64_t r = 0; r < (int64_t)N; r++) mine[n2b[ids[r]]] += (double)freq[r];
    }
    for (int t = 0; t < T; t++)
      for (int b = 0; b < B; b++) mass[(size_t)b] += priv[(size_t)t * B + b];
  }
  double total = 0;
  for (double m : mass) total += m;
  total = std::max(total, 1.0);
  for (int g = 0; g < G; g++) {
    double f[3] = {0, 0, 0};  // local, peers, host
    double served = 0;        // read from this GPU's slice by the other readers
    for (int b = 0; b < B; b++) {
      const double m = mass[(size_t)b] / total;
      const int src = p.access(g, (uint32_t)b);
      f[src == g ? 0 : (src == G ? 2 : 1)] += m;
      for (int r = 0; r < G; r++)
        if (r != g && p.access(r, (uint32_t)b) == g) served += m;
    }
    cost_per_reader[g] = concurrent_cost(f[0], f[1], f[2], served, T_local, T_remote, T_cpu);
  }
  return "";
}

void classify_keys(const Placement& p, int reader, uint64_t N, std::vector<uint32_t> keys_by_src[],
                   uint64_t* counts) {
  const int G = p.num_device;
  const uint8_t* acc = &p.block_access_from[(size_t)reader * p.num_block];
  const uint32_t* n2b = p.nid_to_block.data();
  // Two passes over fixed chunks keep the lists in ascending key order whatever the
  // thread count.
  const uint64_t kChunk = 1u << 20;
  const int64_t n_chunk = (int64_t)((N + kChunk - 1) / kChunk);
  std::vector<uint64_t> chunk_cnt((size_t)n_chunk * (G + 1), 0);
#pragma omp parallel for schedule(dynamic, 4)
  for (int64_t c = 0; c < n_chunk; c++) {
    uint64_t local[UGC_MAX_DEVICE + 1] = {0};
    const uint64_t end = std::min<uint64_t>(N, (uint64_t)(c + 1) * kChunk);
    for (uint64_t k = (uint64_t)c * kChunk; k < end; k++) local[acc[n2b[k]]]++;
    for (int s = 0; s <= G; s++) chunk_cnt[(size_t)c * (G + 1) + s] = local[s];
  }
  for (int s = 0; s <= G; s++) {
    uint64_t run = 0;
    for (int64_t c = 0; c < n_chunk; c++) {
      uint64_t v = chunk_cnt[(size_t)c * (G + 1) + s];
      chunk_cnt[(size_t)c * (G + 1) + s] = run;
      run += v;
    }
    counts[s] = run;
    if (s < G) keys_by_src[s].resize(run);
  }
#pragma omp parallel for schedule(dynamic, 4)
  for (int64_t c = 0; c < n_chunk; c++) {
    uint64_t pos[UGC_MAX_DEVICE + 1];
    for (int s = 0; s <= G; s++) pos[s] = chunk_cnt[(size_t)c * (G + 1) + s];
    const uint64_t end = std::min<uint64_t>(N, (uint64_t)(c + 1) * kChunk);
    for (uint64_t k = (uint64_t)c * kChunk; k < end; k++) {
      int s = acc[n2b[k]];
      if (s < G) keys_by_src[s][pos[s]++] = (uint32_t)k;
    }
  }
}

}  // namespace ugc
