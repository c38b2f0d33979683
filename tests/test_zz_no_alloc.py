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
