"""Parity of merge / merge_by_key (through the C ABI) with the CPU oracle."""
import numpy as np
import pytest
import torch

from thrust_b200 import datagen as dg
from gpu_util import dev, host, rand_of

pytestmark = pytest.mark.gpu
KEY_TYPES = [np.int32, np.uint32, np.float32, np.int64, np.uint64, np.float64]


@pytest.mark.parametrize("n", [0, 1, 2, 33, 2815, 2816, 2817, 3839, 3841, 8193, 65536 + 17, (1 << 20) + 3])
def test_merge_by_key_u64_bit_exact_and_stable(tb, oracles, n):
    # testing/merge_by_key.cu:129-196 splits n unevenly, including an empty side
    for na, nb in [(n, n), (n, n // 3), (0, n), (n, 0), (n // 9, n)]:
        a = np.sort((dg.rand64(4, na) >> np.uint64(52)).astype(np.uint64))     # 12-bit keys: ties between A and B
        b = np.sort((dg.rand64(5, nb) >> np.uint64(52)).astype(np.uint64))
        va = np.arange(na, dtype=np.uint32)
        vb = np.arange(nb, dtype=np.uint32) + np.uint32(1 << 27)               # payload tells A from B
        ko, vo = tb.merge_by_key(dev(a), dev(b), dev(va), dev(vb))
        for o in oracles:
            rk, rv = o.merge_by_key(a, b, va, vb)
            assert np.array_equal(host(ko), rk) and np.array_equal(host(vo), rv), (na, nb)


def test_merge_types_orders_payloads(tb, port):
    n = 30011
    for dt in KEY_TYPES:
        for desc in (False, True):
            a, _ = port.sort_by_key(rand_of(dt, n, 71, small=True), None, desc)
            b, _ = port.sort_by_key(rand_of(dt, n // 2, 72, small=True), None, desc)
            rk, _ = port.merge_by_key(a, b, None, None, desc)
            assert np.array_equal(host(tb.merge(dev(a), dev(b), desc)), rk), (dt, desc)
            for vt in (np.uint32, np.uint64):
                va, vb = np.arange(a.size, dtype=vt), np.arange(b.size, dtype=vt) + vt(1 << 30)
                ko, vo = tb.merge_by_key(dev(a), dev(b), dev(va), dev(vb), desc)
                rk, rv = port.merge_by_key(a, b, va, vb, desc)
                assert np.array_equal(host(ko), rk) and np.array_equal(host(vo), rv), (dt, vt, desc)


def test_golden_merge(tb, golden):
    for n in (1, 777, 12345):
        a, b = golden[f"merge_a_{n}"], golden[f"merge_b_{n}"]
        va = np.arange(a.size, dtype=np.uint32)
        vb = np.arange(b.size, dtype=np.uint32) + np.uint32(1 << 27)
        ko, vo = tb.merge_by_key(dev(a), dev(b), dev(va), dev(vb))
        assert np.array_equal(host(ko), golden[f"merge_keys_out_{n}"]) and np.array_equal(host(vo), golden[f"merge_vals_out_{n}"])


def test_full_size_merge_properties(tb):
    """2 x 2^27 (u64 key, u32 payload): output sorted, each input a subsequence (payloads of A and of
    B each appear in increasing order), ties put A first."""
    n = 1 << 27
    a = dev(dg.merge_keys_u64(n, 4))
    b = dev(dg.merge_keys_u64(n, 5))
    va = torch.arange(n, dtype=torch.int32, device="cuda")
    vb = va + n
    ko, vo = tb.merge_by_key(a, b, va, vb)
    ki = ko.view(torch.int64)                                  # keys < 2^48: signed view keeps the order
    assert bool((ki[1:] >= ki[:-1]).all())
    from_a = vo < n
    assert torch.equal(vo[from_a], va) and torch.equal(vo[~from_a], vb)
    assert torch.equal(ki[from_a], a.view(torch.int64)) and torch.equal(ki[~from_a], b.view(torch.int64))
    ties = ki[1:] == ki[:-1]
    assert bool((~(from_a[1:] & ~from_a[:-1] & ties)).all())   # never B directly before an equal A


@pytest.mark.parametrize("num_runs", [1, 2, 3, 5, 8])
def test_merge_runs_tree(tb, port, num_runs):
    """tb200_merge_runs: many sorted runs in one call, equal to folding the oracle's two-way merge
    over them in order (ties keep the earlier run first)."""
    import ctypes as C
    from thrust_b200 import api
    lib = tb._lib.load()
    runs_k, runs_v, dk, dv = [], [], [], []
    for r in range(num_runs):
        n = [30011, 0, 4097, 1, 70001, 2816, 5, 12345][r]
        k = np.sort((dg.rand64(80 + r, n) >> np.uint64(54)).astype(np.uint32))       # 10-bit keys: ties across runs
        v = (np.arange(n, dtype=np.uint32) + np.uint32(r << 24))
        runs_k.append(k); runs_v.append(v); dk.append(dev(k)); dv.append(dev(v))
    total = sum(k.size for k in runs_k)
    wk, wv = runs_k[0], runs_v[0]
    for r in range(1, num_runs):
        wk, wv = port.merge_by_key(wk, runs_k[r], wv, runs_v[r])
    ko = torch.empty(total, dtype=torch.uint32, device="cuda"); kt = torch.empty_like(ko)
    vo = torch.empty(total, dtype=torch.uint32, device="cuda"); vt = torch.empty_like(vo)
    kp = (C.c_void_p * num_runs)(*[t.data_ptr() for t in dk])
    vp = (C.c_void_p * num_runs)(*[t.data_ptr() for t in dv])
    cn = (C.c_size_t * num_runs)(*[t.numel() for t in dk])
    ws = api._call_with_ws("merge", "tb200_merge_runs", kp, vp, cn, num_runs, api._ptr(ko), api._ptr(vo), api._ptr(kt), api._ptr(vt), 5, 4, 0)
    api._sync_and_check(ws, "merge_runs")
    assert np.array_equal(host(ko), wk) and np.array_equal(host(vo), wv)
