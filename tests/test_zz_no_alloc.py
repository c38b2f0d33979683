"""The sort entry point that takes no workspace and allocates nothing: same bits as dsgx_sort_pack, call after call.

Collected last (file name), so that it also runs after every other GPU test has used the library."""
import ctypes as C

import numpy as np
import pytest
import torch

from dsgx10_b200 import _lib, moe

pytestmark = pytest.mark.gpu

KEYS = ("counts", "offsets", "perm_tok", "perm_slot", "pos_of", "row_order")


def _picks(T, E, topk, seed):
    rng = np.random.default_rng(seed)
    # distinct experts a row, skewed popularity, some experts never picked
    p = 1.0 / (1.0 + np.arange(E)) ** 1.1
    p[E // 2::7] = 0.0
    p /= p.sum()
    return np.stack([rng.choice(E, size=topk, replace=False, p=p) for _ in range(T)]).astype(np.int32)


@pytest.mark.parametrize("T,E,topk", [(1, 8, 2), (300, 64, 6), (4097, 256, 8), (8192, 512, 8)])
def test_static_scratch_matches_workspace_version_twice(T, E, topk):
    for call, seed in enumerate((11, 12)):  # two calls in a row: the second finds the first one's scratch contents
        idx = torch.from_numpy(_picks(T, E, topk, seed + T)).cuda()
        want = moe.sort_pack(idx, E)
        got = moe.sort_pack_static(idx, E)
        torch.cuda.synchronize()
        for k in KEYS:
            assert torch.equal(got[k], want[k]), (call, k)


def test_smaller_call_after_larger_one():
    big = torch.from_numpy(_picks(8192, 512, 8, 5)).cuda()
    moe.sort_pack_static(big, 512)
    small = torch.from_numpy(_picks(37, 16, 4, 6)).cuda()
    got, want = moe.sort_pack_static(small, 16), moe.sort_pack(small, 16)
    torch.cuda.synchronize()
    for k in KEYS:
        assert torch.equal(got[k], want[k]), k


def test_beyond_the_limit_is_refused_and_nothing_runs():
    T, E, topk = 16384, 512, 8
    assert _lib.lib().dsgx_sort_ws_bytes(T, topk, E) > 131328
    idx = torch.zeros(T, topk, dtype=torch.int32, device="cuda")
    sentinel = torch.full((E,), -7, dtype=torch.int32, device="cuda")
    out = [torch.empty(n, dtype=torch.int32, device="cuda") for n in (E + 1, T * topk, T * topk, T * topk, T * topk)]
    ptr = lambda t: C.c_void_p(t.data_ptr())
    rc = _lib.lib().dsgx_sort_pack_static(ptr(idx), T, topk, E, ptr(sentinel), *[ptr(t) for t in out], None)
    torch.cuda.synchronize()
    assert rc == _lib.ERR_LIMIT
    assert bool((sentinel == -7).all())
    with pytest.raises(_lib.DsgxError):
        moe.sort_pack_static(idx, E)


def test_the_call_takes_no_device_memory():
    """The point of the entry point: with the outputs in place and the first call on the device made (it looks the
    array's address up), a call leaves the driver's free-memory figure and torch's allocator counters where they were."""
    T, E, topk = 2048, 256, 8
    idx = torch.from_numpy(_picks(T, E, topk, 21)).cuda()
    out = [torch.empty(n, dtype=torch.int32, device="cuda") for n in (E, E + 1, T * topk, T * topk, T * topk, T * topk)]
    ptr = lambda t: C.c_void_p(t.data_ptr())
    call = lambda: _lib.lib().dsgx_sort_pack_static(ptr(idx), T, topk, E, *[ptr(t) for t in out], None)
    assert call() == 0
    torch.cuda.synchronize()
    free0, _ = torch.cuda.mem_get_info()
    stats0 = torch.cuda.memory_stats()["allocation.all.allocated"]
    for _ in range(3):
        assert call() == 0
    torch.cuda.synchronize()
    free1, _ = torch.cuda.mem_get_info()
    assert free1 == free0
    assert torch.cuda.memory_stats()["allocation.all.allocated"] == stats0
    want = moe.sort_pack(idx, E)
    for t, k in zip(out, KEYS):
        assert torch.equal(t, want[k].flatten()), k


def test_out_of_range_expert_ids_are_reported():
    """A pick outside [0, E) is left out of the order and recorded: dsgx_ws_status on the workspace of dsgx_sort_pack,
    dsgx_sort_static_status after the static form; the next clean sort clears the word."""
    T, E, topk = 64, 16, 4
    good = torch.from_numpy(_picks(T, E, topk, 31)).cuda()
    bad = good.clone()
    bad[5, 1], bad[40, 0] = E, -1
    L = _lib.lib()
    moe.sort_pack_static(bad, E)
    assert L.dsgx_sort_static_status() == _lib.ERR_ARG
    got = moe.sort_pack_static(good, E)
    assert L.dsgx_sort_static_status() == _lib.OK
    want = moe.sort_pack(good, E)
    for k in KEYS:
        assert torch.equal(got[k], want[k]), k
    # the workspace form: the word is the first of the workspace
    i32 = dict(dtype=torch.int32, device="cuda")
    outs = [torch.empty(n, **i32) for n in (E, E + 1, T * topk, T * topk, T * topk, T * topk)]
    ws = torch.empty(max(L.dsgx_sort_ws_bytes(T, topk, E), 256), dtype=torch.uint8, device="cuda")
    ptr = lambda t: C.c_void_p(t.data_ptr())
    assert L.dsgx_sort_pack(ptr(bad), T, topk, E, *[ptr(t) for t in outs], ptr(ws), None) == 0
    assert L.dsgx_ws_status(ptr(ws)) == _lib.ERR_ARG
    assert int(outs[0].sum()) == T * topk - 2       # the two bad picks are not counted
    assert L.dsgx_sort_pack(ptr(good), T, topk, E, *[ptr(t) for t in outs], ptr(ws), None) == 0
    assert L.dsgx_ws_status(ptr(ws)) == _lib.OK
