"""Parity of scan_by_key and unique_by_key (the first "next" components) with the CPU oracle."""
import numpy as np
import pytest

from thrust_b200 import datagen as dg
from gpu_util import ALL, EDGE_SIZES, WIDE, dev, host, rand_of

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("n", EDGE_SIZES)
def test_scan_by_key_and_unique_by_key_bit_exact(tb, oracles, n):
    keys = dg.run_keys(n)
    vals = dg.scan_input_i32(n, 7)
    inc = host(tb.inclusive_scan_by_key(dev(keys), dev(vals)))
    exc = host(tb.exclusive_scan_by_key(dev(keys), dev(vals), 11))
    uk, uv = tb.unique_by_key_copy(dev(keys), dev(np.arange(n, dtype=np.uint32)))
    for o in oracles:
        assert np.array_equal(inc, o.scan_by_key(keys, vals))
        assert np.array_equal(exc, o.scan_by_key(keys, vals, "plus", True, 11))
        rk, rv = o.unique_by_key_copy(keys, np.arange(n, dtype=np.uint32))
        assert np.array_equal(host(uk), rk) and np.array_equal(host(uv), rv)


def test_by_key_types_ops_in_place(tb, port):
    n = 40009
    for kt in ALL:
        keys = rand_of(kt, n, 91, small=True)
        for vt in WIDE:
            vals = rand_of(vt, n, 92, small=True)
            for op in ("plus", "min", "max"):
                assert np.array_equal(host(tb.inclusive_scan_by_key(dev(keys), dev(vals), op=op)), port.scan_by_key(keys, vals, op)), (kt, vt, op)
                assert np.array_equal(host(tb.exclusive_scan_by_key(dev(keys), dev(vals), 2, op=op)), port.scan_by_key(keys, vals, op, True, 2)), (kt, vt, op)
        for vt in (np.uint32, np.uint64):
            v = np.arange(n, dtype=vt)
            gk, gv = tb.unique_by_key_copy(dev(keys), dev(v))
            rk, rv = port.unique_by_key_copy(keys, v)
            assert np.array_equal(host(gk), rk) and np.array_equal(host(gv), rv), (kt, vt)
    keys = dg.run_keys(100001)
    vals = dg.scan_input_i32(100001)
    d = dev(vals)
    tb.inclusive_scan_by_key(dev(keys), d, out=d)                                  # in place
    assert np.array_equal(host(d), port.scan_by_key(keys, vals))
    dk, dv = dev(keys), dev(np.arange(keys.size, dtype=np.uint32))
    gk, gv = tb.unique_by_key(dk, dv)                                               # in place
    rk, rv = port.unique_by_key_copy(keys, np.arange(keys.size, dtype=np.uint32))
    assert np.array_equal(host(gk), rk) and np.array_equal(host(gv), rv)
    # one run spanning many tiles; fp32 within tolerance of the exact partial sums
    f = dg.scan_input_f32(300000)
    got = host(tb.inclusive_scan_by_key(dev(np.zeros(300000, np.int32)), dev(f))).astype(np.float64)
    exact = np.cumsum(f.astype(np.float64))
    assert np.max(np.abs(got - exact) / np.maximum(exact, 1.0)) < 1e-5


@pytest.mark.parametrize("kt,vt", [(np.int32, np.int32), (np.uint32, np.float32), (np.int64, np.int64), (np.uint64, np.float64), (np.int32, np.int64)])
def test_scan_by_key_large_bit_exact(tb, oracles, kt, vt):
    """2^25 + 12345 items: keys and values of one size take the two-pass streaming kernels, mixed sizes
    the single-pass one; the last row of the input is partial.  Floating-point values are small
    integers here, so their sums are exact."""
    n = (1 << 25) + 12345
    keys = dg.run_keys(n).astype(kt)
    vals = (dg.scan_input_i32(n, 7) % 1000).astype(vt)
    init = np.asarray(11, dtype=vt)[()]
    inc = host(tb.inclusive_scan_by_key(dev(keys), dev(vals)))
    exc = host(tb.exclusive_scan_by_key(dev(keys), dev(vals), init))
    mx = host(tb.inclusive_scan_by_key(dev(keys), dev(vals), op="max"))
    d = dev(vals)
    tb.inclusive_scan_by_key(dev(keys), d, out=d)                              # in place
    for o in oracles:
        assert np.array_equal(inc, o.scan_by_key(keys, vals))
        assert np.array_equal(exc, o.scan_by_key(keys, vals, "plus", True, init))
        assert np.array_equal(mx, o.scan_by_key(keys, vals, "max"))
        assert np.array_equal(host(d), o.scan_by_key(keys, vals))
