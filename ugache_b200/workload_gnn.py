"""Synthetic GNN feature-extraction workload (stand-in for the reference's papers100M /
com-friendster runs, whose graphs are not available offline).

* graph: R-MAT edge list with (a, b, c, d) = (0.57, 0.19, 0.19, 0.05), stored as CSR;
* key batch of one iteration: the deduplicated union of all nodes touched by a 3-hop
  GraphSAGE-style neighbour sampling (fan-out 15/10/5, uniform with replacement) from a seeded
  set of seed nodes — what the reference's example feeds to the lookup
  (example/gnn/dgl_sample.py:259 looks up ``input_nodes`` of the sampled blocks);
* hotness for the placement: node degree (the reference's "cache by degree" ordering),
  passed as ``rank_ids`` / ``rank_freqs``.

Harness code: PyTorch tensor ops on whatever device the caller picks (CPU for tests, the GPU
for the 100 M-node benchmark).  The sampler is not part of the extraction path.
"""
import torch


def rmat_edges(num_nodes, num_edges, seed, device="cpu", a=0.57, b=0.19, c=0.19, chunk=1 << 26):
    """(src, dst) int64 tensors of an R-MAT graph; ids are taken modulo num_nodes."""
    g = torch.Generator(device=device)
    g.manual_seed(seed)
    scale = max(1, (num_nodes - 1).bit_length())
    src_parts, dst_parts = [], []
    done = 0
    while done < num_edges:
        n = min(chunk, num_edges - done)
        src = torch.zeros(n, dtype=torch.int64, device=device)
        dst = torch.zeros(n, dtype=torch.int64, device=device)
        for _ in range(scale):
            r = torch.rand(n, generator=g, device=device)
            # quadrant: a -> (0,0), b -> (0,1), c -> (1,0), d -> (1,1)
            sbit = (r >= a + b).to(torch.int64)
            dbit = (((r >= a) & (r < a + b)) | (r >= a + b + c)).to(torch.int64)
            src = (src << 1) | sbit
            dst = (dst << 1) | dbit
        src_parts.append(src % num_nodes)
        dst_parts.append(dst % num_nodes)
        done += n
    return torch.cat(src_parts), torch.cat(dst_parts)


def to_csr(src, dst, num_nodes):
    """(rowptr[int64, N+1], col[int32 or int64, E]) with the edges grouped by source."""
    order = torch.argsort(src)
    col = dst[order]
    deg = torch.bincount(src, minlength=num_nodes)
    rowptr = torch.zeros(num_nodes + 1, dtype=torch.int64, device=src.device)
    rowptr[1:] = torch.cumsum(deg, 0)
    total_deg = deg + torch.bincount(dst, minlength=num_nodes)
    return rowptr, col, deg, total_deg


def sample_batch(rowptr, col, seeds, fanouts, generator):
    """Deduplicated ids of every node reached from ``seeds`` by uniform neighbour sampling
    with the given fan-outs (nodes without neighbours contribute only themselves)."""
    frontier = seeds
    seen = [seeds]
    for f in fanouts:
        start = rowptr[frontier]
        deg = rowptr[frontier + 1] - start
        has = deg > 0
        start, deg = start[has], deg[has]
        r = torch.rand((start.numel(), f), generator=generator, device=rowptr.device)
        idx = start[:, None] + (r * deg[:, None].to(r.dtype)).to(torch.int64)
        idx = torch.minimum(idx, (start + deg - 1)[:, None])
        nbr = col[idx.reshape(-1)].to(torch.int64)
        frontier = torch.unique(nbr)
        seen.append(frontier)
    return torch.unique(torch.cat(seen))


def degree_hotness(deg):
    """(rank_ids uint32-valued int64 tensor, rank_freqs): nodes by descending degree."""
    freqs, ids = torch.sort(deg, descending=True, stable=True)
    return ids, freqs


class GnnWorkload:
    def __init__(self, num_nodes, avg_degree, seed, device="cpu"):
        self.N = num_nodes
        self.device = device
        src, dst = rmat_edges(num_nodes, num_nodes * avg_degree, seed, device)
        self.rowptr, self.col, self.deg, self.total_deg = to_csr(src, dst, num_nodes)
        del src, dst
        if num_nodes < (1 << 31):
            self.col = self.col.to(torch.int32)
        self.seed = seed
        self.train_nodes = torch.nonzero(self.deg > 0).reshape(-1)

    def hotness(self):
        ids, freqs = degree_hotness(self.total_deg)
        return ids.cpu().numpy().astype("uint32"), freqs.cpu().numpy().astype("uint32")

    def batch(self, rank, it, num_seeds=8000, fanouts=(15, 10, 5)):
        g = torch.Generator(device=self.device)
        g.manual_seed(self.seed * 1000003 + rank * 1009 + it)
        # seeds are drawn from the nodes that have neighbours (the "training set")
        pick = torch.randint(0, self.train_nodes.numel(), (num_seeds,), generator=g, device=self.device)
        return sample_batch(self.rowptr, self.col, torch.unique(self.train_nodes[pick]), fanouts, g)
