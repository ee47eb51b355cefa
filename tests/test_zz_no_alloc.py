"""xs_moe_permute_noalloc: the permutation for callers that cannot allocate device memory (an engine whose KV
page pool already owns all free HBM; a serving thread that must not hit cudaMalloc's device-wide
synchronisation).  Its scratch is a fixed array inside the library, so this test checks, through the C ABI,
that it returns exactly what xs_moe_permute returns -- and what the CPU oracle's permutation gives -- on two calls in a row (the second smaller than the first,
so anything the first call left in the shared array would show), that device memory does not move, and that
oversized calls are refused with a clear message.  Collected last on purpose."""
import ctypes as C

import numpy as np
import pytest
import torch

from xstar_moe import capi

import gpu_util as gu

pytestmark = pytest.mark.gpu


def _ids(T, E, K, seed):
    rng = np.random.default_rng(seed)
    p = rng.random(E) ** 2 + 1e-3
    return np.stack([np.sort(rng.choice(E, K, replace=False, p=p / p.sum())) for _ in range(T)]).astype(np.int32)


def _noalloc(T, E, K, ids_dev):
    cfg = capi.make_config(T, 256, E, K, 128, 0)
    outs = [torch.full((n,), -7, dtype=torch.int32, device="cuda") for n in (E, E + 1, T * K, T * K)]
    capi.check(capi.lib().xs_moe_permute_noalloc(C.byref(cfg), capi.ptr(ids_dev), *[capi.ptr(o) for o in outs], gu.stream_ptr()))
    torch.cuda.synchronize()
    return [o.cpu().numpy() for o in outs]


def test_noalloc_permute_equals_workspace_permute_twice_in_a_row(oracle):
    if not torch.cuda.is_available():
        pytest.fail("needs a CUDA device")
    cases = [(3000, 256, 6, 1), (77, 64, 4, 2)]  # 12 chunks then 1 chunk: the second call reuses a dirtier array
    for T, E, K, seed in cases:
        ids = _ids(T, E, K, seed)
        ids_dev = torch.from_numpy(ids).cuda()
        got = _noalloc(T, E, K, ids_dev)
        dims = dict(T=T, H=256, E=E, K=K, I=128, S=0, fmt="bf16", bias=None)
        ref = [t.cpu().numpy() for t in gu.permute(dims, ids_dev)]
        for name, a, b, c in zip(("counts", "offsets", "perm", "inv"), got, ref, oracle.permute(ids, E)):
            assert np.array_equal(a, b), name  # integer outputs: bit-exact
            assert np.array_equal(a, c), name + " (against the CPU oracle)"
    # same inputs again after the small call: still identical
    T, E, K, seed = cases[0]
    ids_dev = torch.from_numpy(_ids(T, E, K, seed)).cuda()
    again = _noalloc(T, E, K, ids_dev)
    ref = [t.cpu().numpy() for t in gu.permute(dict(T=T, H=256, E=E, K=K, I=128, S=0, fmt="bf16", bias=None), ids_dev)]
    assert all(np.array_equal(a, b) for a, b in zip(again, ref))
    del ids_dev
    torch.cuda.synchronize()


def test_noalloc_permute_does_not_take_device_memory():
    L = capi.lib()
    T, E, K = 512, 32, 2
    ids_dev = torch.from_numpy(_ids(T, E, K, 3)).cuda()
    outs = [torch.empty((n,), dtype=torch.int32, device="cuda") for n in (E, E + 1, T * K, T * K)]
    cfg = capi.make_config(T, 256, E, K, 128, 0)
    capi.check(L.xs_moe_permute_noalloc(C.byref(cfg), capi.ptr(ids_dev), *[capi.ptr(o) for o in outs], gu.stream_ptr()))
    torch.cuda.synchronize()
    a, b = C.c_size_t(0), C.c_size_t(0)
    capi.check(L.xs_moe_device_free_bytes(C.byref(a)))
    for _ in range(20):
        capi.check(L.xs_moe_permute_noalloc(C.byref(cfg), capi.ptr(ids_dev), *[capi.ptr(o) for o in outs], gu.stream_ptr()))
    torch.cuda.synchronize()
    capi.check(L.xs_moe_device_free_bytes(C.byref(b)))
    assert a.value == b.value


def test_noalloc_permute_refuses_sizes_beyond_its_array():
    L = capi.lib()
    cfg = capi.make_config(16385, 256, 8, 2, 128, 0)
    dummy = torch.zeros(4, dtype=torch.int32, device="cuda")
    rc = L.xs_moe_permute_noalloc(C.byref(cfg), *[capi.ptr(dummy)] * 5, None)
    assert rc == -3
    msg = L.xs_moe_last_error()
    assert b"built-in scratch too small" in msg and b"16384" in msg
