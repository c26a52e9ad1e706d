"""Parity of the CUDA reduce and scan (through the C ABI) with the CPU oracle."""
import numpy as np
import pytest

from thrust_b200 import datagen as dg
from gpu_util import EDGE_SIZES, WIDE, dev, host, misaligned, rand_of

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("n", EDGE_SIZES)
def test_reduce_int_bit_exact(tb, oracles, n):
    x = dg.reduce_input(n)
    got = tb.reduce(dev(x), np.int64(7))
    for o in oracles:
        assert got == o.reduce(x, np.int64(7))


def test_reduce_types_and_ops(tb, port):
    n = 100003
    for dt, acc in [(np.int8, np.int32), (np.int8, np.int64), (np.int16, np.int32), (np.int16, np.int64), (np.int32, np.int32),
                    (np.int32, np.int64), (np.uint8, np.uint32), (np.uint8, np.uint64), (np.uint16, np.uint32), (np.uint16, np.uint64),
                    (np.uint32, np.uint32), (np.uint32, np.uint64), (np.int64, np.int64), (np.uint64, np.uint64)]:
        x = rand_of(dt, n, 41)
        for op in ("plus", "min", "max"):
            init = np.asarray(3, dtype=acc)[()]
            assert tb.reduce(dev(x), init, op) == port.reduce(x, init, op), (dt, acc, op)
    # floating point: reassociation is allowed, tolerance 1e-5 relative to the fp64 sum
    for dt, acc in [(np.float32, np.float32), (np.float32, np.float64), (np.float64, np.float64)]:
        x = dg.scan_input_f32(n).astype(dt)
        exact = float(np.sum(x.astype(np.float64))) + 1.0
        got = float(tb.reduce(dev(x), np.asarray(1.0, dtype=acc)[()]))
        assert abs(got - exact) <= 1e-5 * abs(exact), (dt, acc)
        assert tb.reduce(dev(x), np.asarray(0.5, dtype=acc)[()], "max") == port.reduce(x, np.asarray(0.5, dtype=acc)[()], "max")
        assert tb.reduce(dev(x), np.asarray(0.5, dtype=acc)[()], "min") == port.reduce(x, np.asarray(0.5, dtype=acc)[()], "min")


def test_reduce_misaligned_and_default_init(tb, port):
    x = dg.reduce_input(70001)
    for off in (1, 2, 3):
        assert tb.reduce(misaligned(x, off), np.int64(0)) == port.reduce(x, np.int64(0))
    assert tb.reduce(dev(x)) == port.reduce(x, np.int32(0))          # no init: value_type(0), reduce.h:1057-1067
    assert tb.reduce(dev(x[:0]), np.int64(-9)) == -9                 # empty range returns init, reduce.h:863-864


@pytest.mark.parametrize("n", EDGE_SIZES)
def test_scan_int_bit_exact(tb, oracles, n):
    x = dg.scan_input_i32(n)
    incl = host(tb.inclusive_scan(dev(x)))
    excl = host(tb.exclusive_scan(dev(x), 5))
    for o in oracles:
        assert np.array_equal(incl, o.inclusive_scan(x))
        assert np.array_equal(excl, o.exclusive_scan(x, 5))


@pytest.mark.parametrize("dt", [np.int32, np.int64, np.uint32, np.float64])
def test_scan_chunked_route_bit_exact(tb, oracles, dt):
    """Large inputs take the two-pass route (per-chunk totals, then chunk-wise scans); sizes chosen
    so that the last chunk is short and the last tile partial.  float64 holds integers here, so its
    sums are exact too."""
    n = (1 << 25) + 12345
    x = dg.scan_input_i32(n).astype(dt)
    init = np.asarray(5, dtype=dt)[()]
    incl = host(tb.inclusive_scan(dev(x)))
    excl = host(tb.exclusive_scan(dev(x), init))
    d = dev(x)
    tb.inclusive_scan(d, out=d)                                                # in place
    mx = host(tb.inclusive_scan(dev(x), op="max"))
    for o in oracles:
        assert np.array_equal(incl, o.inclusive_scan(x))
        assert np.array_equal(excl, o.exclusive_scan(x, init))
        assert np.array_equal(host(d), o.inclusive_scan(x))
        assert np.array_equal(mx, o.inclusive_scan(x, "max"))


def test_scan_in_place_and_misaligned(tb, port):
    x = dg.scan_input_i32(100001)
    d = dev(x)
    assert tb.inclusive_scan(d, out=d) is d and np.array_equal(host(d), port.inclusive_scan(x))   # testing/scan.cu:71-91
    d = dev(x)
    tb.exclusive_scan(d, 0, out=d)
    assert np.array_equal(host(d), port.exclusive_scan(x, 0))
    for off in (1, 3):
        assert np.array_equal(host(tb.inclusive_scan(misaligned(x, off))), port.inclusive_scan(x))
    assert np.array_equal(host(tb.inclusive_scan(dev(x), init=11)), port.inclusive_scan(x) + 11)


def test_scan_types_and_ops(tb, port):
    n = 50021
    for dt in WIDE:
        x = rand_of(dt, n, 43, small=True)           # small exact values: float sums are exact too
        for op in ("plus", "min", "max"):
            assert np.array_equal(host(tb.inclusive_scan(dev(x), op=op)), port.inclusive_scan(x, op)), (dt, op)
            assert np.array_equal(host(tb.exclusive_scan(dev(x), 3, op=op)), port.exclusive_scan(x, 3, op)), (dt, op)
    big = rand_of(np.int64, n, 44)                   # wrap-around arithmetic must match too
    assert np.array_equal(host(tb.inclusive_scan(dev(big))), port.inclusive_scan(big))


def test_scan_fp32_tolerance(tb, port):
    """fp32 plus-scan: within 1e-5 relative of the fp64-accumulated yardstick at every position.
    (The reference's own sequential fp32 scan is further from it than that at this length.)"""
    n = (1 << 22) + 77
    x = dg.scan_input_f32(n)
    yard = port.scan_f32_via_f64(x).astype(np.float64)
    got = host(tb.inclusive_scan(dev(x))).astype(np.float64)
    assert np.max(np.abs(got - yard) / np.maximum(yard, 1.0)) < 1e-5
    yard = port.scan_f32_via_f64(x, True, 2.5).astype(np.float64)
    got = host(tb.exclusive_scan(dev(x), 2.5)).astype(np.float64)
    assert np.max(np.abs(got - yard) / np.maximum(yard, 1.0)) < 1e-5


@pytest.mark.parametrize("n", [(1 << 25) + 12345, 1 << 28])
def test_scan_fp32_tolerance_on_the_large_input_route(tb, port, n):
    """The fp32 variant of the benchmark configuration at the sizes that take the large-input route
    (above a few million items): inclusive and exclusive plus-scan within 1e-5 relative of the
    fp64-accumulated yardstick at EVERY position, in place as well."""
    x = dg.scan_input_f32(n)
    d = dev(x)
    yard = port.scan_f32_via_f64(x).astype(np.float64)
    got = host(tb.inclusive_scan(d)).astype(np.float64)
    assert np.max(np.abs(got - yard) / np.maximum(yard, 1.0)) < 1e-5
    del got
    e = tb.exclusive_scan(d, 2.5)
    tb.inclusive_scan(d, out=d)                                               # in place, testing/scan.cu:71-91
    assert np.max(np.abs(host(d).astype(np.float64) - yard) / np.maximum(yard, 1.0)) < 1e-5
    yard = port.scan_f32_via_f64(x, True, 2.5).astype(np.float64)
    assert np.max(np.abs(host(e).astype(np.float64) - yard) / np.maximum(yard, 1.0)) < 1e-5


def test_golden_reduce_scan(tb, golden):
    for n in (1, 777, 12345):
        assert tb.reduce(dev(golden[f"reduce_in_{n}"]), np.int64(0)) == golden[f"reduce_out_{n}"]
        assert np.array_equal(host(tb.inclusive_scan(dev(golden[f"scan_in_{n}"]))), golden[f"scan_incl_{n}"])
        assert np.array_equal(host(tb.exclusive_scan(dev(golden[f"scan_in_{n}"]), 0)), golden[f"scan_excl_{n}"])


def test_full_size_reduce_and_scan(tb, oracles):
    """The benchmark sizes (2^28): reduce bit-exact against the oracle; scan checked through its
    defining property out[i] - out[i-1] == in[i] and its last element against the reduce."""
    import torch
    n = 1 << 28
    x = dg.reduce_input(n)
    got = tb.reduce(dev(x), np.int64(0))
    assert got == oracles[-1].reduce(x, np.int64(0)) == int(x.sum(dtype=np.int64))
    del x
    s = dev(dg.scan_input_i32(n))
    out = tb.inclusive_scan(s)
    assert torch.equal(out[1:] - out[:-1], s[1:]) and out[0] == s[0]
    assert int(out[-1]) == int(tb.reduce(s, np.int64(0)))
    ex = tb.exclusive_scan(s, 0)
    assert torch.equal(ex[1:], out[:-1]) and int(ex[0]) == 0
