"""Multi-replica host logic on CPU ranks (gloo, world_size 2): placement solved on rank 0 and
broadcast, per-rank key classification, cross-rank consistency of who stores / who reads what,
and the bounded barrier of the reference-named layer (a missing replica is a timeout status,
not a hang)."""
import os
import subprocess
import sys
import textwrap

import numpy as np
import pytest

from tests.conftest import ROOT

WORKER = textwrap.dedent("""
    import os, sys
    sys.path.insert(0, %(root)r)
    import numpy as np
    import torch
    import torch.distributed as dist
    from ugache_b200 import runtime as rt, workload as wl
    from oracle import oracle as orc

    rank = int(os.environ["RANK"]); world = int(os.environ["WORLD_SIZE"])
    dist.init_process_group("gloo", rank=rank, world_size=world)
    N, G, pct = 30000, world, 0.10
    # replica 0 solves, the others receive the four arrays (the reference publishes them
    # through shared memory, coll_cache_lib/facade.cc:238-261)
    if rank == 0:
        ids, freqs = wl.analytic_hotness(N, 1.2)
        p = rt.solve_placement("intuitive", G, ids, freqs, pct * 100)
        meta = torch.tensor([p.num_block], dtype=torch.int64)
    else:
        meta = torch.zeros(1, dtype=torch.int64)
    dist.broadcast(meta, 0)
    B = int(meta[0])
    n2b = torch.from_numpy(p.nid_to_block.astype(np.int64)) if rank == 0 else torch.zeros(N, dtype=torch.int64)
    bp = torch.from_numpy(p.block_placement.astype(np.int64)) if rank == 0 else torch.zeros(B, dtype=torch.int64)
    ba = torch.from_numpy(p.block_access_from.astype(np.int64)) if rank == 0 else torch.zeros((G, B), dtype=torch.int64)
    bd = torch.from_numpy(p.block_density) if rank == 0 else torch.zeros(B, dtype=torch.float64)
    for t in (n2b, bp, ba, bd):
        dist.broadcast(t, 0)
    place = rt.PlacementArrays(n2b.numpy().astype(np.uint32), bp.numpy().astype(np.uint8),
                               ba.numpy().astype(np.uint8), bd.numpy())
    cache = rt.Cache(G, N, 512, pct, max_batch=4096)
    cache.set_placement(place)
    counts, lists = cache.classify_keys(rank, want_keys=True)
    # every rank's view of "rows stored on rank s" must be the same set: gather the list each
    # rank reads from source 0 and compare with what rank 0 stores
    mine = torch.zeros(N, dtype=torch.int64)
    mine[torch.from_numpy(lists[0].astype(np.int64))] = 1
    views = [torch.zeros(N, dtype=torch.int64) for _ in range(world)]
    dist.all_gather(views, mine)
    o = orc.Placement(place.nid_to_block, place.block_placement, place.block_access_from, place.block_density)
    words, cnt, slot_of = orc.model_build(o, rank, int(N * (pct + 0.001)))
    assert [int(x) for x in counts] == [int(x) for x in cnt], (counts, cnt)
    stored0 = (place.block_placement[place.nid_to_block] & 1).astype(np.int64)
    if rank == 0:
        assert np.array_equal(views[0].numpy(), stored0)          # rank 0 reads all it stores
    for r in range(world):                                          # nobody reads from 0 what 0 lacks
        assert not np.any(views[r].numpy() & (1 - stored0))
    # partitioned rows are read by everyone from their single owner
    part0 = (place.block_placement[place.nid_to_block] == 1).astype(np.int64)
    for r in range(world):
        assert np.all(views[r].numpy()[part0 == 1] == 1)
    tot = torch.tensor([int(counts[:G].sum()), int(counts[G])], dtype=torch.int64)
    dist.all_reduce(tot)
    assert int(tot.sum()) == N * world
    cache.close()
    dist.barrier()
    print("rank", rank, "ok")
""")


def test_two_rank_placement_exchange_and_classification(built_lib, tmp_path):
    script = tmp_path / "worker.py"
    script.write_text(WORKER % {"root": ROOT})
    procs = []
    for r in range(2):
        env = dict(os.environ, RANK=str(r), WORLD_SIZE="2", MASTER_ADDR="127.0.0.1",
                   MASTER_PORT="29621", OMP_NUM_THREADS="2")
        procs.append(subprocess.Popen([sys.executable, str(script)], env=env,
                                      stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True))
    outs = [p.communicate(timeout=240)[0] for p in procs]
    for r, (p, o) in enumerate(zip(procs, outs)):
        assert p.returncode == 0, "rank %d failed:\n%s" % (r, o)
        assert "rank %d ok" % r in o


BARRIER = textwrap.dedent("""
    import os, sys, ctypes
    sys.path.insert(0, %(root)r)
    from ugache_b200.collcache import common
    b = common._basics
    b.config({"cache_percentage": 0.1, "_cache_policy": 9, "num_device": 2,
              "num_global_step_per_epoch": 1, "num_epoch": 1, "num_total_item": 1000,
              "omp_thread_num": 2})
    rc = b.C_LIB_CTYPES.coll_cache_train_barrier()      # the second replica never arrives
    print("rc", rc)
    sys.exit(0 if rc == 7 else 1)                        # UGC_ERR_TIMEOUT
""")


def test_barrier_with_missing_replica_times_out(built_lib, tmp_path):
    script = tmp_path / "barrier.py"
    script.write_text(BARRIER % {"root": ROOT})
    env = dict(os.environ, UGC_BARRIER_TIMEOUT_S="0.3")
    p = subprocess.run([sys.executable, str(script)], env=env, capture_output=True, text=True,
                       timeout=120)
    assert p.returncode == 0, p.stdout + p.stderr


FORKED = textwrap.dedent("""
    import os, sys
    sys.path.insert(0, %(root)r)
    from ugache_b200.collcache import common     # library loaded BEFORE the fork: shared control block
    b = common._basics
    b.config({"cache_percentage": 0.1, "_cache_policy": 12, "num_device": 2,
              "num_global_step_per_epoch": 1, "num_epoch": 1, "num_total_item": 1000,
              "omp_thread_num": 2})
    pid = os.fork()
    rc = b.C_LIB_CTYPES.coll_cache_train_barrier()
    rc2 = b.C_LIB_CTYPES.coll_cache_train_barrier()
    if pid == 0:
        os._exit(0 if (rc == 0 and rc2 == 0) else 3)
    st = b.wait_one_child()
    sys.exit(0 if (rc == 0 and rc2 == 0 and st == 0) else 1)
""")


def test_fork_shared_barrier(built_lib, tmp_path):
    script = tmp_path / "forked.py"
    script.write_text(FORKED % {"root": ROOT})
    p = subprocess.run([sys.executable, str(script)], env=dict(os.environ, UGC_BARRIER_TIMEOUT_S="20"),
                       capture_output=True, text=True, timeout=120)
    assert p.returncode == 0, p.stdout + p.stderr


FAILING_PEER = textwrap.dedent("""
    import os, sys, time
    sys.path.insert(0, %(root)r)
    from ugache_b200.collcache import common     # loaded before the fork: shared control block
    b = common._basics
    b.config({"cache_percentage": 0.1, "_cache_policy": 12, "num_device": 2,
              "num_global_step_per_epoch": 1, "num_epoch": 1, "num_total_item": 1000,
              "omp_thread_num": 2})
    pid = os.fork()
    if pid == 0:
        # this replica fails inside a call all replicas make together (no cache was built)
        rc = b.C_LIB_CTYPES.coll_cache_refresh(1, None)
        os._exit(0 if rc != 0 else 3)
    t0 = time.time()
    rc = b.C_LIB_CTYPES.coll_cache_train_barrier()       # would wait 60 s for the failed peer
    dt = time.time() - t0
    st = b.wait_one_child()
    print("rc", rc, "dt", dt, "child", st)
    sys.exit(0 if (rc == 5 and dt < 20 and st == 0) else 1)   # UGC_ERR_STATE, promptly
""")


def test_failure_of_one_replica_releases_the_others_promptly(built_lib, tmp_path):
    """A replica that fails in a collective call flags the shared control block, so replicas
    waiting at a barrier return an error at once instead of sitting out the time limit."""
    script = tmp_path / "failing_peer.py"
    script.write_text(FAILING_PEER % {"root": ROOT})
    p = subprocess.run([sys.executable, str(script)], env=dict(os.environ, UGC_BARRIER_TIMEOUT_S="60"),
                       capture_output=True, text=True, timeout=120)
    assert p.returncode == 0, p.stdout + p.stderr
