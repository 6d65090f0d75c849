"""ugc_lookup_i64_static: the lookup whose scratch is a fixed array inside the library, for
callers that cannot obtain device memory where they look keys up (a fixed-arena allocator
that is already full, a serving thread that must not trigger the device-wide synchronisation
of a scratch re-allocation).

The check: through the C ABI, its output equals that of the ordinary entry point
(ugc_lookup_i64) byte for byte, on two calls in a row with different batches that share the
array; sizes beyond its limit are refused with a message.  Collected last on purpose.
"""
import ctypes as C

import numpy as np
import pytest

pytestmark = pytest.mark.gpu
torch = pytest.importorskip("torch")


def test_static_scratch_lookup_matches_regular_entry_point(built_lib):
    from ugache_b200 import _lib, runtime as rt, workload as wl
    L = _lib.lib()
    N, dim, G = 70000, 128, 2
    ndev = torch.cuda.device_count()
    table = wl.table(41, N, dim)
    ids, freqs = wl.analytic_hotness(N, 1.2)
    cache = rt.Cache(G, N, dim * 4, 0.10, max_batch=1 << 15)
    cache.set_placement(rt.solve_placement("intuitive", G, ids, freqs, 10.0))
    host = torch.from_numpy(table).pin_memory()
    for r in range(G):
        cache.build(r, r % ndev, host.data_ptr())
    cache.connect_local()
    for r in range(G):
        cache.attach_peers(r)

    def both(r, keys_np):
        dev = torch.device("cuda", r % ndev)
        with torch.cuda.device(dev):
            k = torch.from_numpy(keys_np).to(dev)
            s = torch.cuda.current_stream(dev).cuda_stream
            ref = torch.full((len(keys_np), dim * 4), 0xAB, dtype=torch.uint8, device=dev)
            new = torch.full((len(keys_np), dim * 4), 0xCD, dtype=torch.uint8, device=dev)
            _lib.check(L.ugc_lookup_i64(cache._h, r, C.c_void_p(k.data_ptr()), len(keys_np),
                                        C.c_void_p(ref.data_ptr()), C.c_void_p(s)))
            _lib.check(L.ugc_lookup_i64_static(cache._h, r, C.c_void_p(k.data_ptr()), len(keys_np),
                                               C.c_void_p(new.data_ptr()), C.c_void_p(s)))
            torch.cuda.synchronize(dev)
            return ref.cpu().numpy(), new.cpu().numpy()

    # two calls in a row on the same replica (the second finds the first one's leftovers in the
    # array), then one on the other replica
    for r, seed, n in ((0, 1, 20000), (0, 2, 7777), (1, 3, 30001)):
        keys = wl.zipf_keys(seed, n, N, 1.2)
        ref, new = both(r, keys)
        assert new.tobytes() == ref.tobytes(), (r, seed)
        assert ref.tobytes() == table[keys].tobytes()
    # the ordinary entry point is unaffected afterwards
    keys = wl.zipf_keys(9, 5000, N, 1.2)
    ref, new = both(0, keys)
    assert ref.tobytes() == new.tobytes() == table[keys].tobytes()

    # beyond the fixed limit: refused, with a message, nothing launched
    dev = torch.device("cuda", 0)
    big = torch.zeros((1 << 18) + 1, dtype=torch.int64, device=dev)
    out = torch.empty(16, dtype=torch.uint8, device=dev)
    rc = L.ugc_lookup_i64_static(cache._h, 0, C.c_void_p(big.data_ptr()), big.numel(),
                                 C.c_void_p(out.data_ptr()), None)
    assert rc == 1
    assert b"at most 262144 keys" in L.ugc_last_error()
    cache.close()
