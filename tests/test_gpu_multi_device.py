"""Replicas on DISTINCT GPUs: peer rows really cross NVLink, peer tables are probed over P2P,
and another process maps this process' slice onto a different device.  Skipped on a box with
one GPU (there every replica shares device 0 and only the hop itself is missing, see
test_gpu_parity.py).  Covers what the reference does in its peer attach
(coll_cache_lib/cache_context.cu:2531-2570) and pointer exchange (:2648-2680).
"""
import multiprocessing as mp
import os

import numpy as np
import pytest

from oracle import oracle as orc
from tests.helpers import case_workload, digest

pytestmark = pytest.mark.gpu
torch = pytest.importorskip("torch")


def _need(n):
    if not torch.cuda.is_available() or torch.cuda.device_count() < n:
        pytest.skip("needs %d GPUs" % n)


@pytest.mark.parametrize("mode", ["grouped", "direct"])
@pytest.mark.parametrize("case_index", [2, 4])        # g2_intuitive, g8_intuitive
def test_replicas_on_distinct_devices_in_one_process(built_lib, golden_cases, case_index, mode,
                                                     monkeypatch):
    case = golden_cases[case_index]
    _need(min(case["G"], 2))
    monkeypatch.setenv("UGC_EXTRACT_MODE", mode)
    from tests.test_gpu_parity import lookup_np, make_cache
    ndev = torch.cuda.device_count()
    w = case_workload(case)
    cache = make_cache(w)                      # replica r on device r % ndev
    devices = {r % ndev for r in range(w.G)}
    assert len(devices) == min(w.G, ndev) >= 2
    for r in range(w.G):
        keys = w.keys(rank=r)
        got = lookup_np(cache, r, keys)
        assert got.tobytes() == orc.gather(w.table, keys).tobytes(), (case["name"], r)
        assert digest(got) == case["ranks"][str(r)]["out"]
        st = cache.stats(r)
        assert st["err_table"] == 0 and st["err_key_range"] == 0
        assert st["last_remote"] > 0            # some rows did come from another replica
    cache.close()


def _worker(rank, world, case, route, q_in, q_out, mode):
    """One process per replica, each on its own GPU; handles travel through queues."""
    try:
        os.environ["UGC_EXTRACT_MODE"] = mode
        if route == "socket":
            os.environ["UGC_NO_PIDFD"] = "1"
        import torch as th
        from ugache_b200 import _lib, runtime as rt
        from tests.helpers import case_workload as cw
        th.cuda.set_device(rank)
        w = cw(case)
        cache = rt.Cache(w.G, w.N, w.row_bytes, w.pct, max_batch=1 << 16)
        cache.set_placement(w.placement)
        host = th.from_numpy(w.table.view(np.uint8).reshape(w.N, -1).copy()).pin_memory()
        cache.build(rank, rank, host.data_ptr())
        q_out.put((rank, bytes(cache.export(rank))))
        handles = q_in.get(timeout=120)
        for r, blob in handles:
            if r != rank:
                cache.import_peer(rank, _lib.PeerHandle.from_buffer_copy(blob))
        cache.attach_peers(rank)
        q_out.put((rank, "attached"))
        assert q_in.get(timeout=120) == "go"
        keys = w.keys(rank=rank)
        k = th.from_numpy(keys).cuda()
        out = cache.lookup(rank, k)
        th.cuda.synchronize()
        st = cache.stats(rank)
        ok = out.cpu().numpy().tobytes() == orc.gather(w.table, keys).tobytes()
        q_out.put((rank, ("ok" if ok else "mismatch", int(st["last_remote"]), int(st["err_table"]))))
        assert q_in.get(timeout=120) == "done"   # peers may still be reading this slice
        cache.close()
    except Exception as e:                       # reported to the parent, which fails the test
        q_out.put((rank, ("error", repr(e), 0)))


@pytest.mark.parametrize("route,mode", [("pidfd", "direct"), ("socket", "grouped")])
def test_replicas_in_separate_processes_on_distinct_devices(built_lib, golden_cases, route, mode):
    """The slice and the table of each replica are mapped by the OTHER process onto the other
    GPU (file-descriptor export of virtual-memory blocks, both hand-over routes)."""
    _need(2)
    case = golden_cases[2]                       # g2_intuitive
    ctx = mp.get_context("spawn")
    q_out = ctx.Queue()
    q_in = [ctx.Queue() for _ in range(2)]
    procs = [ctx.Process(target=_worker, args=(r, 2, case, route, q_in[r], q_out, mode)) for r in range(2)]
    for p in procs:
        p.start()
    try:
        handles = [q_out.get(timeout=300) for _ in range(2)]
        assert all(isinstance(h[1], bytes) for h in handles), handles
        for q in q_in:
            q.put(handles)
        att = [q_out.get(timeout=300) for _ in range(2)]
        assert all(a[1] == "attached" for a in att), att
        for q in q_in:
            q.put("go")
        res = [q_out.get(timeout=300) for _ in range(2)]
        for q in q_in:
            q.put("done")
        for rank, (status, n_remote, err_table) in res:
            assert status == "ok", (rank, status, n_remote)
            assert n_remote > 0 and err_table == 0
    finally:
        for p in procs:
            p.join(timeout=60)
            if p.is_alive():
                p.kill()
