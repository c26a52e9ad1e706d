"""Parity of the set operations on sorted ranges (through the C ABI) with the reference's multiset
semantics, restated here with numpy: an element occurring m times in A and n times in B appears
max(m, n) / min(m, n) / max(m - n, 0) / |m - n| times in the union / intersection / difference /
symmetric difference, A's copies first where both sides contribute
(thrust/system/cuda/detail/set_operations.h; testing/set_union.cu, set_intersection.cu,
set_difference.cu, set_symmetric_difference.cu and their _by_key and _descending siblings)."""
import numpy as np
import pytest

from thrust_b200 import datagen as dg
from gpu_util import dev, host

pytestmark = pytest.mark.gpu


def _expected(op, a, b, va, vb, descending):
    """Stable two-pointer walk over the two sorted ranges, one run of equal keys at a time."""
    keys, vals = [], []
    i = j = 0
    before = (lambda x, y: x > y) if descending else (lambda x, y: x < y)
    while i < a.size or j < b.size:
        if j >= b.size or (i < a.size and before(a[i], b[j])):
            x = a[i]
        elif i >= a.size or before(b[j], a[i]):
            x = b[j]
        else:
            x = a[i]
        i2 = i
        while i2 < a.size and a[i2] == x:
            i2 += 1
        j2 = j
        while j2 < b.size and b[j2] == x:
            j2 += 1
        m, n = i2 - i, j2 - j
        if op == "union":
            take_a, take_b = range(i, i2), range(j + m, j2) if n > m else range(0)
        elif op == "intersection":
            take_a, take_b = range(i, i + min(m, n)), range(0)
        elif op == "difference":
            take_a, take_b = range(i + n, i2) if m > n else range(0), range(0)
        else:
            take_a, take_b = (range(i + n, i2) if m > n else range(0)), (range(j + m, j2) if n > m else range(0))
        for t in take_a:
            keys.append(a[t]); vals.append(va[t])
        for t in take_b:
            keys.append(b[t]); vals.append(vb[t])
        i, j = i2, j2
    return np.array(keys, dtype=a.dtype), np.array(vals, dtype=va.dtype)


@pytest.mark.parametrize("op", ["union", "intersection", "difference", "symmetric_difference"])
@pytest.mark.parametrize("na,nb,bits", [(0, 0, 8), (0, 37, 8), (41, 0, 8), (1, 1, 2), (1000, 777, 6), (5000, 5003, 10), (20011, 30011, 40)])
def test_set_operations_match_the_multiset_definition(tb, op, na, nb, bits):
    for dt, desc in ((np.uint32, False), (np.int64, True), (np.float32, False)):
        a = (dg.rand64(71, na) >> np.uint64(64 - bits)).astype(np.int64)
        b = (dg.rand64(72, nb) >> np.uint64(64 - bits)).astype(np.int64)
        a, b = np.sort(a.astype(dt)), np.sort(b.astype(dt))      # cast first: the cast may wrap, the ranges must be sorted as dt
        if desc:
            a, b = a[::-1].copy(), b[::-1].copy()
        va, vb = np.arange(na, dtype=np.uint32), np.arange(nb, dtype=np.uint32) + np.uint32(1 << 30)
        wk, wv = _expected(op, a, b, va, vb, desc)
        gk, _ = tb.set_operation(op, dev(a), dev(b), descending=desc)
        assert np.array_equal(host(gk), wk), (op, dt, na, nb)
        gk, gv = tb.set_operation(op, dev(a), dev(b), dev(va), dev(vb), descending=desc)
        assert np.array_equal(host(gk), wk) and np.array_equal(host(gv), wv), (op, dt, na, nb)


def test_set_operations_large_sorted_inputs(tb):
    """2 x 2^22 keys with many ties between and inside the ranges, checked through numpy's own
    multiset arithmetic on the value counts."""
    n = 1 << 22
    a = np.sort((dg.rand64(73, n) >> np.uint64(44)).astype(np.uint32))
    b = np.sort((dg.rand64(74, n) >> np.uint64(44)).astype(np.uint32))
    top = 1 << 20
    ca, cb = np.bincount(a, minlength=top), np.bincount(b, minlength=top)
    want = {"union": np.maximum(ca, cb), "intersection": np.minimum(ca, cb), "difference": np.maximum(ca - cb, 0),
            "symmetric_difference": np.abs(ca - cb)}
    for op, counts in want.items():
        gk, _ = tb.set_operation(op, dev(a), dev(b))
        g = host(gk)
        assert g.size == int(counts.sum()) and bool((g[1:] >= g[:-1]).all()), op
        assert np.array_equal(np.bincount(g, minlength=top), counts), op
