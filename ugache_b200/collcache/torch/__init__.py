"""The reference's ``collcache.torch`` functions (python/collcache/torch/adapter.py:28-55 and
the pybind module behind it, python/collcache/torch/adapter.cc:124-281), implemented with
ctypes calls into libugache_b200.so.  PyTorch only owns tensors here.

Extensions beyond the reference: int64 key tensors are accepted, ``coll_torch_refresh`` /
``coll_torch_refresh_async`` expose the refresh path (the reference reaches it only from its
TF2 binding), ``coll_torch_lookup_unique`` looks every distinct key of a batch up once, and
``coll_torch_shutdown`` releases everything.
"""
import ctypes
import mmap
import os

import torch

from ..common import *            # noqa: F401,F403  (constants, as the reference re-exports)
from ..common import _basics
from ... import _lib

config = _basics.config
log_step_by_key = _basics.log_step_by_key
report_step = _basics.report_step
report_step_average = _basics.report_step_average
train_barrier = _basics.train_barrier
wait_one_child = _basics.wait_one_child
print_memory_usage = _basics.print_memory_usage
coll_cache_record_init = _basics.coll_cache_record_init

_DTYPE_CODE = {torch.float32: 0, torch.float64: 1, torch.float16: 2, torch.uint8: 3,
               torch.int32: 4, torch.int8: 5, torch.int64: 6}

_state = {"dim": 0, "dtype": torch.float32, "dev": {}, "out": {}, "max_keys": 0, "shm": []}


def _L():
    return _basics.C_LIB_CTYPES


def _num_total_item():
    return _state.get("num_total_item", 0)


_orig_config = config


def config(run_config: dict):  # noqa: F811
    _state["num_total_item"] = int(run_config["num_total_item"])
    _state["num_device"] = int(run_config["num_device"])
    _orig_config(run_config)


def coll_torch_record(local_id, keys):
    """keys: CPU integer tensor (the reference takes 32-bit ids; int64 is narrowed here)."""
    k = keys.detach().to("cpu")
    if k.dtype == torch.int64:
        k = k.to(torch.int32)
    k = k.contiguous()
    _state["max_keys"] = max(_state["max_keys"], k.numel())
    _basics._ok(_L().coll_cache_record(local_id, ctypes.c_void_p(k.data_ptr()), k.numel()),
                "coll_cache_record")


def coll_torch_create_emb_shm(replica_id, n_keys, dim, dtype, fname=""):
    """A CPU tensor [n_keys, dim] over POSIX shared memory that every replica process maps
    (the reference names it SAMG_FEAT_SHM, adapter.cc:246); filled from ``fname`` if given."""
    k = os.environ.get("SAMGRAPH_EMPTY_FEAT", "")
    if k:
        n_keys = 1 << int(k)
        fname = ""
    item = torch.empty(0, dtype=dtype).element_size()
    nbytes = n_keys * dim * item
    path = "/dev/shm/SAMG_FEAT_SHM_%d_%s" % (os.getuid(), os.environ.get("UGC_SESSION", str(os.getppid())))
    fd = os.open(path, os.O_CREAT | os.O_RDWR, 0o600)
    if os.fstat(fd).st_size != nbytes:
        os.ftruncate(fd, nbytes)
    mm = mmap.mmap(fd, nbytes, flags=mmap.MAP_SHARED)
    os.close(fd)
    t = torch.frombuffer(mm, dtype=dtype).reshape(n_keys, dim)
    _state["shm"].append((path, mm))
    if fname:
        if os.stat(fname).st_size != nbytes:
            raise RuntimeError("feat file on disk not equal with claimed shape")
        with open(fname, "rb") as f:
            f.readinto(mm)
    return t


def coll_torch_init_t(replica_id, dev_id, emb, cache_percentage):
    """emb: the CPU table [N, dim] (fp32 or fp16), kept alive by the caller."""
    if emb.dtype not in _DTYPE_CODE:
        raise TypeError("unsupported embedding dtype %s" % emb.dtype)
    torch.cuda.set_device(dev_id)
    _state["dim"], _state["dtype"] = emb.size(1), emb.dtype
    _state["dev"][replica_id] = dev_id
    _state["emb"] = emb
    _basics._ok(_L().coll_cache_set_device(replica_id, dev_id), "coll_cache_set_device")
    stream = torch.cuda.current_stream(dev_id).cuda_stream
    rc = _L().coll_cache_init_c(replica_id, emb.size(0) if not os.environ.get("SAMGRAPH_EMPTY_FEAT")
                                else _num_total_item(), None, None, None,
                                ctypes.c_void_p(emb.data_ptr()), _DTYPE_CODE[emb.dtype], emb.size(1),
                                float(cache_percentage), ctypes.c_void_p(stream))
    _basics._ok(rc, "coll_cache_init")


def coll_torch_test(local_id, keys):
    dev = _state["dev"].get(local_id, 0)
    return torch.empty((keys.size(0), _state["dim"]), dtype=torch.float32, device="cuda:%d" % dev)


def coll_torch_lookup_key_t_val_ret(local_id, keys, pad_to_8=True):
    """Rows of ``keys`` as a [len(keys) (padded to 8), dim] tensor on the replica's GPU.  As in
    the reference (adapter.cc:213-228) the tensor aliases a reusable buffer that the next
    lookup of this replica overwrites."""
    dev = _state["dev"][local_id]
    n = keys.size(0)
    padded = (n + 7) // 8 * 8 if pad_to_8 else n
    buf = _state["out"].get(local_id)
    if buf is None or buf.size(0) < padded:
        rows = int(max(padded, _state["max_keys"]) * 1.05) + 8
        buf = torch.empty((rows, _state["dim"]), dtype=_state["dtype"], device="cuda:%d" % dev)
        _state["out"][local_id] = buf
    out = buf[:padded]
    if n == 0:
        return out
    keys = keys.contiguous()
    stream = torch.cuda.current_stream(dev).cuda_stream
    if keys.dtype == torch.int64:
        ctx = _L().coll_cache_context()
        L = _lib.lib()
        rc = L.ugc_lookup_i64(ctx, local_id, ctypes.c_void_p(keys.data_ptr()), n,
                              ctypes.c_void_p(out.data_ptr()), ctypes.c_void_p(stream))
        if rc == 1:  # batch larger than the scratch: grow and retry
            _lib.check(L.ugc_reserve_batch(ctx, local_id, int(n * 1.05) + 8))
            rc = L.ugc_lookup_i64(ctx, local_id, ctypes.c_void_p(keys.data_ptr()), n,
                                  ctypes.c_void_p(out.data_ptr()), ctypes.c_void_p(stream))
        _lib.check(rc)
        torch.cuda.current_stream(dev).synchronize()
    else:
        rc = _L().coll_cache_lookup(local_id, ctypes.c_void_p(keys.data_ptr()), n,
                                    ctypes.c_void_p(out.data_ptr()), ctypes.c_void_p(stream))
        _basics._ok(rc, "coll_cache_lookup")
    return out


def coll_torch_refresh(local_id):
    """Re-solve the placement from the hotness recorded so far and move the caches to it."""
    dev = _state["dev"][local_id]
    stream = torch.cuda.current_stream(dev).cuda_stream
    _basics._ok(_L().coll_cache_refresh(local_id, ctypes.c_void_p(stream)), "coll_cache_refresh")


def lookup_unique(keys, lookup_fn):
    """Dedup-aware lookup: the distinct keys of a batch are looked up once.

    ``lookup_fn(unique_keys)`` returns the rows of ``unique_keys`` ([u, dim]); the result is
    ``(rows_unique, inverse)`` with ``rows_unique[inverse]`` equal to the rows of ``keys`` in
    batch order.  Returns views of whatever ``lookup_fn`` returns, so the aliasing rules of the
    underlying lookup apply.  The distinct keys come out ascending, which also makes the table
    probes of the lookup coalesce."""
    unique, inverse = torch.unique(keys.reshape(-1), sorted=True, return_inverse=True)
    rows = lookup_fn(unique)
    return rows[:unique.numel()], inverse


def coll_torch_lookup_unique(local_id, keys):
    """``(rows_unique, inverse)`` for a key batch with duplicates (a recommendation batch under a
    skewed distribution repeats its hottest ids thousands of times): consumers that pool or
    scatter by ``inverse`` anyway (embedding-bag forward, sparse-gradient backward) need every
    distinct row once.  ``rows_unique[inverse]`` is what ``coll_torch_lookup_key_t_val_ret``
    returns for the same keys.  The distinct keys are found on the GPU by the library
    (``ugc_lookup_unique``: stamps per id, no sort) in the same stream as the extraction; they
    come out in order of discovery, not ascending.  No counterpart in the reference."""
    dev = _state["dev"][local_id]
    keys = keys.reshape(-1).contiguous()
    n = keys.numel()
    if n == 0:
        return (torch.empty((0, _state["dim"]), dtype=_state["dtype"], device="cuda:%d" % dev),
                torch.empty(0, dtype=torch.int64, device="cuda:%d" % dev))
    if keys.dtype not in (torch.int64, torch.int32):
        keys = keys.to(torch.int64)
    kb = 8 if keys.dtype == torch.int64 else 4
    rows = torch.empty((n, _state["dim"]), dtype=_state["dtype"], device="cuda:%d" % dev)
    uniq = torch.empty_like(keys)
    inverse = torch.empty(n, dtype=torch.int32, device="cuda:%d" % dev)
    n_unique = torch.zeros(1, dtype=torch.int32, device="cuda:%d" % dev)
    stream = torch.cuda.current_stream(dev).cuda_stream
    ctx = _L().coll_cache_context()
    L = _lib.lib()

    def call():
        return L.ugc_lookup_unique(ctx, local_id, ctypes.c_void_p(keys.data_ptr()), kb, n,
                                   ctypes.c_void_p(rows.data_ptr()), ctypes.c_void_p(uniq.data_ptr()),
                                   ctypes.c_void_p(inverse.data_ptr()),
                                   ctypes.c_void_p(n_unique.data_ptr()), ctypes.c_void_p(stream))

    rc = call()
    if rc == 1:  # batch larger than the scratch: grow and retry
        _lib.check(L.ugc_reserve_batch(ctx, local_id, int(n * 1.05) + 8))
        rc = call()
    _lib.check(rc)
    return rows[:int(n_unique.item())], inverse.to(torch.int64)


def coll_torch_lookup_pool(local_id, keys, offsets=None, bag_size=0, mode="sum"):
    """Embedding-bag forward in one kernel (``ugc_lookup_pool``): ``out[b]`` = the sum or mean of
    the rows of bag ``b`` as fp32 ``[n_bags, dim]``; bags are ``keys[offsets[b]:offsets[b+1]]``
    (int64 ``offsets`` of ``n_bags + 1`` entries) or runs of ``bag_size`` keys.  Bit for bit the
    result of a sequential fp32 sum over ``coll_torch_lookup_key_t_val_ret``'s rows in key order.
    No counterpart in the reference, whose applications pool in the model."""
    dev = _state["dev"][local_id]
    device = "cuda:%d" % dev
    keys = keys.reshape(-1).contiguous()
    if keys.dtype not in (torch.int64, torch.int32):
        keys = keys.to(torch.int64)
    if _state["dtype"] not in (torch.float32, torch.float16):
        raise ValueError("pooled lookup needs an fp32 or fp16 table")
    kb = 8 if keys.dtype == torch.int64 else 4
    if offsets is not None:
        offsets = offsets.to(device=device, dtype=torch.int64).contiguous()
        n_bags = offsets.numel() - 1
    else:
        if bag_size <= 0:
            raise ValueError("give offsets or a bag size")
        n_bags = keys.numel() // bag_size
    out = torch.empty((max(n_bags, 0), _state["dim"]), dtype=torch.float32, device=device)
    stream = torch.cuda.current_stream(dev).cuda_stream
    _lib.check(_lib.lib().ugc_lookup_pool(
        _L().coll_cache_context(), local_id, ctypes.c_void_p(keys.data_ptr()), kb, keys.numel(),
        ctypes.c_void_p(offsets.data_ptr() if offsets is not None else None), max(n_bags, 0), bag_size,
        0 if _state["dtype"] == torch.float32 else 1, {"sum": 0, "mean": 1}[mode],
        ctypes.c_void_p(out.data_ptr()), ctypes.c_void_p(stream)))
    return out


class _RefreshJob:
    """Handle of a background refresh: ``wait()`` joins it and re-raises its failure."""

    def __init__(self, local_id, dev):
        import threading
        self.error = None

        def work():
            try:
                with torch.cuda.device(dev):
                    stream = torch.cuda.Stream(dev)
                    _basics._ok(_L().coll_cache_refresh(local_id, ctypes.c_void_p(stream.cuda_stream)),
                                "coll_cache_refresh")
                    stream.synchronize()
            except Exception as e:  # handed to wait()
                self.error = e

        self._t = threading.Thread(target=work, name="collcache-refresh-%d" % local_id, daemon=True)
        self._t.start()

    def done(self):
        return not self._t.is_alive()

    def wait(self, timeout=None):
        self._t.join(timeout)
        if self._t.is_alive():
            raise TimeoutError("background refresh still running")
        if self.error is not None:
            raise self.error


def coll_torch_refresh_async(local_id):
    """Starts ``coll_torch_refresh`` on a background thread with a stream of its own and returns
    a handle; lookups of the replica may go on meanwhile (the reference's TensorFlow binding
    refreshes this way, from a helper thread, ``CollCache::refresh(..., foreground=false)``).
    Every replica must start one, as with the blocking form."""
    return _RefreshJob(local_id, _state["dev"][local_id])


def coll_torch_shutdown():
    _basics.shutdown()
    _state["out"].clear()
    for path, mm in _state["shm"]:
        try:
            os.unlink(path)
        except OSError:
            pass
    _state["shm"].clear()
