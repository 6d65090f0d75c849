"""The reference-facing API on a GPU: the ``collcache.torch`` function names end to end
(config -> record -> create_emb_shm -> init -> lookup -> refresh), with the replicas as
threads of one process and as separate processes (CUDA IPC), checked against the oracle."""
import os
import subprocess
import sys
import textwrap
import threading

import numpy as np
import pytest

from oracle import oracle as orc
from tests.conftest import ROOT

pytestmark = pytest.mark.gpu
torch = pytest.importorskip("torch")


def test_collcache_torch_api_threads(built_lib):
    import ugache_b200.collcache.torch as co
    from ugache_b200 import workload as wl
    N, dim, G = 60000, 64, 2
    ndev = torch.cuda.device_count()
    os.environ["UGC_SESSION"] = "pytest_threads_%d" % os.getpid()
    co.config({"cache_percentage": 0.10, "_cache_policy": co.cache_policies["coll_intuitive"],
               "num_device": G, "num_global_step_per_epoch": 10, "num_epoch": 1,
               "num_total_item": N, "omp_thread_num": 4})
    emb = co.coll_torch_create_emb_shm(0, N, dim, torch.float32)
    emb.copy_(torch.from_numpy(wl.table(77, N, dim)))
    table = emb.numpy().copy()
    batches = {r: [wl.zipf_keys(500 + 10 * r + i, 5000, N, 1.2) for i in range(4)] for r in range(G)}
    errors = []

    def run(r):
        try:
            co.coll_cache_record_init(r)
            for k in batches[r][:2]:
                co.coll_torch_record(r, torch.from_numpy(k))
            co.coll_torch_init_t(r, r % ndev, emb, 0.10)
            dev = "cuda:%d" % (r % ndev)
            for k in batches[r]:
                for dt in (torch.int32, torch.int64):
                    out = co.coll_torch_lookup_key_t_val_ret(r, torch.from_numpy(k).to(dev).to(dt),
                                                             pad_to_8=True)
                    assert out.shape == ((len(k) + 7) // 8 * 8, dim) and out.dtype == torch.float32
                    got = out[:len(k)].cpu().numpy()
                    assert got.tobytes() == orc.gather(table, k).tobytes()
            # hotness drifts: record other keys, refresh, look up again
            for i in range(3):
                co.coll_torch_record(r, torch.from_numpy(wl.zipf_keys(900 + i, 20000, N, 0.9)))
            co.coll_torch_refresh(r)
            for k in batches[r]:
                out = co.coll_torch_lookup_key_t_val_ret(r, torch.from_numpy(k).to(dev).to(torch.int32),
                                                         pad_to_8=False)
                assert out.cpu().numpy().tobytes() == orc.gather(table, k).tobytes()
            # embedding-bag forward in one kernel: bit for bit the sequential fp32 sum of those rows
            k = batches[r][0]
            pooled = co.coll_torch_lookup_pool(r, torch.from_numpy(k).to(dev), bag_size=10, mode="sum")
            assert pooled.cpu().numpy().tobytes() == orc.pool(table, k, bag_size=10).tobytes()
            offs = torch.tensor([0, 3, 3, 1000, len(k)])
            pooled = co.coll_torch_lookup_pool(r, torch.from_numpy(k).to(dev).to(torch.int32), offsets=offs,
                                               mode="mean")
            assert pooled.cpu().numpy().tobytes() == orc.pool(table, k, offsets=offs.numpy(), mean=True).tobytes()
            # a second refresh in the background while this thread keeps looking up
            for i in range(3):
                co.coll_torch_record(r, torch.from_numpy(wl.zipf_keys(950 + i, 20000, N, 1.3)))
            job = co.coll_torch_refresh_async(r)
            rounds = 0
            while rounds < 3 or not job.done():
                for k in batches[r]:
                    out = co.coll_torch_lookup_key_t_val_ret(r, torch.from_numpy(k).to(dev).to(torch.int64),
                                                             pad_to_8=False)
                    assert out.cpu().numpy().tobytes() == orc.gather(table, k).tobytes()
                rounds += 1
            job.wait(timeout=120)
            # a batch larger than anything recorded grows the scratch
            big = wl.zipf_keys(7, 90000, N, 1.2)
            out = co.coll_torch_lookup_key_t_val_ret(r, torch.from_numpy(big).to(dev).to(torch.int32), False)
            assert out.cpu().numpy().tobytes() == orc.gather(table, big).tobytes()
        except Exception as e:  # surfaced in the main thread
            import traceback
            errors.append("replica %d: %s\n%s" % (r, e, traceback.format_exc()))

    ts = [threading.Thread(target=run, args=(r,)) for r in range(G)]
    for t in ts:
        t.start()
    for t in ts:
        t.join(timeout=300)
    co.report_step_average(0)
    co.coll_torch_shutdown()
    assert not errors, "\n".join(errors)


WORKER = textwrap.dedent("""
    import os, sys
    sys.path.insert(0, %(root)r)
    import numpy as np, torch
    import ugache_b200.collcache.torch as co
    from ugache_b200 import workload as wl
    from oracle import oracle as orc
    r = int(sys.argv[1]); G = int(sys.argv[2])
    N, dim = 50000, 128
    ndev = torch.cuda.device_count()
    co.config({"cache_percentage": 0.08, "_cache_policy": co.cache_policies["clique_part"],
               "num_device": G, "num_global_step_per_epoch": 10, "num_epoch": 1,
               "num_total_item": N, "omp_thread_num": 2})
    co.coll_cache_record_init(r)
    for i in range(2):
        co.coll_torch_record(r, torch.from_numpy(wl.zipf_keys(40 + i, 8000, N, 1.2)).to(torch.int32))
    emb = co.coll_torch_create_emb_shm(r, N, dim, torch.float16)
    if r == 0:
        emb.copy_(torch.from_numpy(wl.table(5, N, dim, np.float16)))
    co.train_barrier()
    co.coll_torch_init_t(r, r %% ndev, emb, 0.08)
    table = emb.numpy()
    dev = "cuda:%%d" %% (r %% ndev)
    for i in range(3):
        k = wl.zipf_keys(100 * r + i, 6000, N, 1.2)
        out = co.coll_torch_lookup_key_t_val_ret(r, torch.from_numpy(k).to(dev).to(torch.int32), False)
        assert out.dtype == torch.float16
        assert out.cpu().numpy().tobytes() == orc.gather(table, k).tobytes()
    pooled = co.coll_torch_lookup_pool(r, torch.from_numpy(k).to(dev), bag_size=6)
    assert pooled.dtype == torch.float32 and pooled.shape == (1000, dim)
    assert pooled.cpu().numpy().tobytes() == orc.pool(table, k, bag_size=6).tobytes()
    import ctypes
    from ugache_b200 import _lib
    st = _lib.Stats()
    _lib.check(_lib.lib().ugc_stats(ctypes.c_void_p(co._L().coll_cache_context()), r, ctypes.byref(st)))
    assert st.err_table == 0 and st.last_remote > 0, (st.err_table, st.last_remote)
    co.train_barrier()
    co.coll_torch_shutdown()
    print("replica", r, "ok")
""")


@pytest.mark.parametrize("route", ["pidfd", "socket", "cuda_ipc"])
def test_collcache_processes_with_ipc(built_lib, tmp_path, route):
    """One process per replica (both on GPU 0 when only one GPU is visible): peer slices and
    peer tables are mapped from another process -- as exported virtual-memory blocks whose
    descriptor is duplicated out of the owner (pidfd), or served over the descriptor socket,
    or through cudaIpc handles of cudaMalloc memory."""
    script = tmp_path / "worker.py"
    script.write_text(WORKER % {"root": ROOT})
    G = 2
    env = dict(os.environ, UGC_SESSION="pytest_ipc_%s_%d" % (route, os.getpid()),
               UGC_BARRIER_TIMEOUT_S="120")
    if route == "socket":
        env["UGC_NO_PIDFD"] = "1"
    if route == "cuda_ipc":
        env["UGC_NO_VMM"] = "1"
    procs = [subprocess.Popen([sys.executable, str(script), str(r), str(G)], env=env,
                              stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
             for r in range(G)]
    outs = []
    for p in procs:
        try:
            outs.append(p.communicate(timeout=400)[0])
        except subprocess.TimeoutExpired:
            p.kill()
            outs.append("timeout")
    for r, (p, o) in enumerate(zip(procs, outs)):
        assert p.returncode == 0, "replica %d failed:\n%s" % (r, o[-3000:])
    for name in os.listdir("/dev/shm"):
        if name.startswith("ugc_%d_pytest_ipc_%s_%d" % (os.getuid(), route, os.getpid())):
            os.unlink(os.path.join("/dev/shm", name))


def test_cpp_facade_program(built_lib, tmp_path):
    """A C++ program written against coll_cache_lib::CollCache (the reference's facade
    signatures) builds against include/coll_cache_lib/facade.h, links the library, and gets
    exact rows before and after a refresh."""
    import shutil
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    exe = tmp_path / "facade_demo"
    libdir = os.path.dirname(built_lib)
    cmd = [nvcc, "-std=c++17", "-O1", "-I", os.path.join(ROOT, "include"),
           os.path.join(ROOT, "tests", "cpp", "facade_demo.cc"), "-o", str(exe),
           "-L" + libdir, "-lugache_b200", "-Xlinker", "-rpath=" + libdir, "-Xcompiler", "-pthread",
           "-Wno-deprecated-gpu-targets"]
    c = subprocess.run(cmd, capture_output=True, text=True, timeout=300)
    assert c.returncode == 0, c.stderr
    p = subprocess.run([str(exe)], capture_output=True, text=True, timeout=300)
    assert p.returncode == 0 and "facade ok" in p.stdout, p.stdout + p.stderr
