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
