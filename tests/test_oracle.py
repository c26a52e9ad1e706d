"""The CPU oracle is pinned three ways: against the small known-answer cases of the reference's
own unit tests, against the committed outputs of the reference (tests/golden), and -- restatement
versus reference build -- on random inputs of every supported type."""
import numpy as np
import pytest

from thrust_b200 import datagen as dg

INT_TYPES = [np.int8, np.uint8, np.int16, np.uint16, np.int32, np.uint32, np.int64, np.uint64]
ALL_TYPES = INT_TYPES + [np.float32, np.float64]
WIDE_TYPES = [np.int32, np.uint32, np.int64, np.uint64, np.float32, np.float64]
SIZES = [0, 1, 2, 17, 1000, 4099]


def rand_of(dtype, n, seed, small=False):
    u = dg.rand64(seed, n)
    if small:
        u = u % np.uint64(7)
    dt = np.dtype(dtype)
    if dt.kind == "f":
        x = ((u >> np.uint64(40)).astype(np.float64) / 2.0 ** 23 - 1.0)
        return (np.round(x * 8) / 8 if small else x).astype(dt)
    return u.astype(np.uint64).view(np.uint64).astype(dt)  # wraps modulo 2^bits


# ------------------------------------------------------------------ known answers (reference tests)
def test_known_answers(oracles):
    for o in oracles:
        # testing/reduce.cu:26-39
        v = np.array([1, -2, 3], np.int32)
        assert o.reduce(v, np.int32(0)) == 2 and o.reduce(v, np.int32(10)) == 12
        # testing/scan.cu:23-60
        x = np.array([1, 3, -2, 4, -5], np.int32)
        assert o.inclusive_scan(x).tolist() == [1, 4, 2, 6, 1]
        assert o.exclusive_scan(x, 0).tolist() == [0, 1, 4, 2, 6]
        assert o.exclusive_scan(x, 3).tolist() == [3, 4, 7, 5, 9]
        y = x.copy()
        o.inclusive_scan(y, out=y)                      # in place, testing/scan.cu:71-91
        assert y.tolist() == [1, 4, 2, 6, 1]
        # testing/sort_by_key.cu:46-69
        k, vv = o.sort_by_key(np.array([1, 3, 6, 5, 2, 0, 4], np.int32), np.arange(7, dtype=np.int32))
        assert k.tolist() == [0, 1, 2, 3, 4, 5, 6] and vv.tolist() == [5, 0, 4, 1, 6, 3, 2]
        # testing/copy.cu:252-269 (is_true)
        assert o.copy_if(np.arange(5, dtype=np.int32), "ne", 0).tolist() == [1, 2, 3, 4]
        # testing/partition.cu:19-42 (is_even): split point and both halves as multisets
        d, cnt = o.partition(np.array([1, 2, 1, 1, 2], np.int32), "mod_eq", 2, 0)
        assert cnt == 2 and d[:2].tolist() == [2, 2] and sorted(d[2:].tolist()) == [1, 1, 1]
        d, cnt = o.stable_partition(np.array([1, 2, 1, 1, 2], np.int32), "mod_eq", 2, 0)
        assert cnt == 2 and d.tolist() == [2, 2, 1, 1, 1]
        # testing/unique.cu:171-208
        u = o.unique_copy(np.array([11, 11, 12, 20, 29, 21, 21, 31, 31, 37], np.int32))
        assert u.tolist() == [11, 12, 20, 29, 21, 31, 37]
        # testing/reduce_by_key.cu:19-80
        ko, vo = o.reduce_by_key(np.array([11, 11, 21, 20, 21, 21, 21, 37, 37], np.int32), np.arange(9, dtype=np.int32))
        assert ko.tolist() == [11, 21, 20, 21, 37] and vo.tolist() == [1, 2, 3, 15, 15]
        # testing/merge.cu:11-37, testing/merge_by_key.cu:10-44 (ties: range A first)
        mk, mv = o.merge_by_key(np.array([0, 2, 4], np.int32), np.array([0, 3, 3, 4], np.int32),
                                np.array([13, 7, 42], np.int32), np.array([42, 42, 7, 13], np.int32))
        assert mk.tolist() == [0, 0, 2, 3, 3, 4, 4] and mv.tolist() == [13, 42, 7, 42, 7, 42, 13]


def test_known_answer_stable_sort(oracles):
    # testing/stable_sort_by_key.cu:43-78 orders by key / 10; a stable sort by the decade is the same
    keys = np.array([25, 14, 35, 16, 26, 34, 36, 24, 15], np.uint32)
    for o in oracles:
        k, v = o.stable_sort_zip_by_first(keys // 10, np.arange(9, dtype=np.uint32))
        assert v.tolist() == [1, 3, 8, 0, 4, 7, 2, 5, 6]
        assert keys[v].tolist() == [14, 16, 15, 25, 26, 24, 35, 34, 36]


# ------------------------------------------------------------------ committed reference outputs
@pytest.mark.parametrize("n", [1, 777, 12345])
def test_port_matches_golden(port, golden, n):
    g = golden
    assert port.reduce(g[f"reduce_in_{n}"], np.int64(0)) == g[f"reduce_out_{n}"]
    assert np.array_equal(port.inclusive_scan(g[f"scan_in_{n}"]), g[f"scan_incl_{n}"])
    assert np.array_equal(port.exclusive_scan(g[f"scan_in_{n}"], 0), g[f"scan_excl_{n}"])
    v = np.arange(n, dtype=np.uint32)
    k, vv = port.sort_by_key(g[f"sort_keys_in_{n}"], v)
    assert np.array_equal(k, g[f"sort_keys_out_{n}"]) and np.array_equal(vv, g[f"sort_vals_out_{n}"])
    k, vv = port.sort_by_key(g[f"sort64_keys_in_{n}"], v)
    assert np.array_equal(k, g[f"sort64_keys_out_{n}"]) and np.array_equal(vv, g[f"sort64_vals_out_{n}"])
    c = g[f"compact_in_{n}"]
    assert np.array_equal(port.copy_if(c, "mod_eq", 2, 0), g[f"copy_if_out_{n}"])
    d, cnt = port.stable_partition(c, "mod_eq", 2, 0)
    assert cnt == g[f"partition_count_{n}"] and np.array_equal(d, g[f"stable_partition_out_{n}"])
    d, cnt = port.partition(c, "mod_eq", 2, 0)
    assert cnt == g[f"partition_count_{n}"] and np.array_equal(d, g[f"partition_out_{n}"])
    assert np.array_equal(port.unique_copy(g[f"run_keys_{n}"]), g[f"unique_out_{n}"])
    ko, vo = port.reduce_by_key(g[f"run_keys_{n}"], g[f"run_vals_{n}"])
    assert np.array_equal(ko, g[f"rbk_keys_out_{n}"]) and np.array_equal(vo, g[f"rbk_vals_out_{n}"])
    a, b = g[f"merge_a_{n}"], g[f"merge_b_{n}"]
    mk, mv = port.merge_by_key(a, b, np.arange(a.size, dtype=np.uint32), np.arange(b.size, dtype=np.uint32) + np.uint32(1 << 27))
    assert np.array_equal(mk, g[f"merge_keys_out_{n}"]) and np.array_equal(mv, g[f"merge_vals_out_{n}"])
    k, vv = port.stable_sort_zip_by_first(g[f"zip_keys_in_{n}"], g[f"zip_vals_in_{n}"].view(np.uint32))
    assert np.array_equal(k, g[f"zip_keys_out_{n}"]) and np.array_equal(vv, g[f"zip_vals_out_{n}"])


# ------------------------------------------------------------------ restatement vs reference build
@pytest.mark.parametrize("n", SIZES)
def test_port_vs_ref_reduce_scan(port, ref, n):
    for dt, acc in [(np.int8, np.int32), (np.int16, np.int64), (np.int32, np.int64), (np.int32, np.int32), (np.uint8, np.uint32),
                    (np.uint16, np.uint64), (np.uint32, np.uint64), (np.int64, np.int64), (np.uint64, np.uint64)]:
        x = rand_of(dt, n, 11)
        for op in ("plus", "min", "max"):
            init = np.asarray(5, dtype=acc)[()]
            assert port.reduce(x, init, op) == ref.reduce(x, init, op), (dt, acc, op)
    xf = rand_of(np.float32, n, 12)
    assert np.isclose(port.reduce(xf, np.float64(1.0)), ref.reduce(xf, np.float64(1.0)), rtol=1e-12)
    assert port.reduce(xf, np.float32(0), "max") == ref.reduce(xf, np.float32(0), "max")
    for dt in WIDE_TYPES:
        x = rand_of(dt, n, 13, small=True)
        for op in ("plus", "min", "max"):
            assert np.array_equal(port.inclusive_scan(x, op), ref.inclusive_scan(x, op)), (dt, op)
            assert np.array_equal(port.exclusive_scan(x, 3, op), ref.exclusive_scan(x, 3, op)), (dt, op)


@pytest.mark.parametrize("n", SIZES)
def test_port_vs_ref_sort_merge(port, ref, n):
    for dt in ALL_TYPES:
        k = rand_of(dt, n, 21)
        if np.dtype(dt).kind == "f":
            k[k == 0] = 0.0   # avoid -0.0: the radix coding orders it before +0.0, operator< does not
        v = np.arange(n, dtype=np.uint32)
        for desc in (False, True):
            pk, pv = port.sort_by_key(k, v, desc)
            rk, rv = ref.sort_by_key(k, v, desc)
            assert np.array_equal(pk, rk) and np.array_equal(pv, rv), (dt, desc)
            pk, _ = port.sort_by_key(k, None, desc)
            assert np.array_equal(pk, rk)
            a, _ = port.sort_by_key(rand_of(dt, n, 22, small=True), None, desc)
            b, _ = port.sort_by_key(rand_of(dt, n // 2, 23, small=True), None, desc)
            va = np.arange(a.size, dtype=np.uint64)
            vb = np.arange(b.size, dtype=np.uint64) + np.uint64(1 << 40)
            pk, pv = port.merge_by_key(a, b, va, vb, desc)
            rk, rv = ref.merge_by_key(a, b, va, vb, desc)
            assert np.array_equal(pk, rk) and np.array_equal(pv, rv), (dt, desc)
    k = (rand_of(np.uint32, n, 24) % 100).astype(np.uint32)
    v = rand_of(np.uint32, n, 25)
    pk, pv = port.stable_sort_zip_by_first(k, v)
    rk, rv = ref.stable_sort_zip_by_first(k, v)
    assert np.array_equal(pk, rk) and np.array_equal(pv, rv)


@pytest.mark.parametrize("n", SIZES)
def test_port_vs_ref_compaction(port, ref, n):
    for dt in ALL_TYPES:
        x = rand_of(dt, n, 31, small=True)
        preds = [("ne", 3, 0), ("lt", 3, 0), ("ge", 2, 0)] + ([("mod_eq", 3, 1)] if np.dtype(dt).kind != "f" else [])
        for pred, a, b in preds:
            assert np.array_equal(port.copy_if(x, pred, a, b), ref.copy_if(x, pred, a, b)), (dt, pred)
            pt, pf = port.partition_copy(x, pred, a, b)
            rt, rf = ref.partition_copy(x, pred, a, b)
            assert np.array_equal(pt, rt) and np.array_equal(pf, rf), (dt, pred)
            pd, pc = port.stable_partition(x, pred, a, b)
            rd, rc = ref.stable_partition(x, pred, a, b)
            assert pc == rc and np.array_equal(pd, rd), (dt, pred)
            pd, pc = port.partition(x, pred, a, b)
            rd, rc = ref.partition(x, pred, a, b)
            assert pc == rc and np.array_equal(pd, rd), (dt, pred)
        st = rand_of(np.uint8, n, 32, small=True)
        assert np.array_equal(port.copy_if(x, "ne", 0, 0, stencil=st), ref.copy_if(x, "ne", 0, 0, stencil=st)), dt
        assert np.array_equal(port.unique_copy(x), ref.unique_copy(x)), dt
        for vt in WIDE_TYPES:
            vals = rand_of(vt, n, 33, small=True)
            for op in ("plus", "min", "max"):
                pk, pv = port.reduce_by_key(x, vals, op)
                rk, rv = ref.reduce_by_key(x, vals, op)
                assert np.array_equal(pk, rk) and np.array_equal(pv, rv), (dt, vt, op)


def test_f64_yardsticks(port, ref):
    x = dg.scan_input_f32(100000)
    assert np.array_equal(port.scan_f32_via_f64(x), ref.scan_f32_via_f64(x))
    assert np.array_equal(port.scan_f32_via_f64(x, True, 2.0), ref.scan_f32_via_f64(x, True, 2.0))
    exact = np.cumsum(x.astype(np.float64))
    assert np.allclose(port.scan_f32_via_f64(x), exact, rtol=1e-7)
    k = dg.run_keys(100000)
    pk, pv = port.reduce_by_key_f32_via_f64(k, x)
    rk, rv = ref.reduce_by_key_f32_via_f64(k, x)
    assert np.array_equal(pk, rk) and np.array_equal(pv, rv)


def test_reference_fp32_scan_drifts(port):
    # the sequential fp32 scan of the reference (sequential/scan.h:67-72) loses accuracy as the running
    # sum grows; this is why fp32 parity is judged against the fp64-accumulated yardstick instead
    x = dg.scan_input_f32(1 << 20)
    seq = port.inclusive_scan(x)
    yard = port.scan_f32_via_f64(x)
    rel = abs(float(seq[-1]) - float(yard[-1])) / float(yard[-1])
    assert 1e-7 < rel < 1e-3


@pytest.mark.parametrize("n", SIZES)
def test_port_vs_ref_by_key(port, ref, n):
    """scan_by_key and unique_by_key_copy (the first of the "next" components): restatement vs reference."""
    for kt in (np.int32, np.uint8, np.int64, np.float32):
        keys = rand_of(kt, n, 41, small=True)
        for vt in WIDE_TYPES:
            vals = rand_of(vt, n, 42, small=True)
            for op in ("plus", "min", "max"):
                assert np.array_equal(port.scan_by_key(keys, vals, op), ref.scan_by_key(keys, vals, op)), (kt, vt, op)
                assert np.array_equal(port.scan_by_key(keys, vals, op, True, 3), ref.scan_by_key(keys, vals, op, True, 3)), (kt, vt, op)
        for vt in (np.uint32, np.uint64):
            vals = np.arange(n, dtype=vt)
            pk, pv = port.unique_by_key_copy(keys, vals)
            rk, rv = ref.unique_by_key_copy(keys, vals)
            assert np.array_equal(pk, rk) and np.array_equal(pv, rv), (kt, vt)


def test_known_answers_by_key(oracles):
    # the worked example of the reference's documentation, thrust/scan.h (inclusive_scan_by_key / exclusive_scan_by_key)
    keys = np.array([0, 0, 0, 1, 1, 2, 3, 3, 3, 3], np.int32)
    ones = np.ones(10, np.int32)
    for o in oracles:
        assert o.scan_by_key(keys, ones).tolist() == [1, 2, 3, 1, 2, 1, 1, 2, 3, 4]
        assert o.scan_by_key(keys, ones, "plus", True, 5).tolist() == [5, 6, 7, 5, 6, 5, 5, 6, 7, 8]
        k, v = o.unique_by_key_copy(np.array([1, 3, 3, 3, 2, 2, 1], np.int32), np.array([9, 8, 7, 6, 5, 4, 3], np.uint32))
        assert k.tolist() == [1, 3, 2, 1] and v.tolist() == [9, 8, 5, 3]


def test_extrema_known_answers_and_port_vs_ref(oracles, port, ref):
    # testing/minmax_element.cu:8-20, testing/min_element.cu, testing/max_element.cu (the "Simple" cases)
    data = np.array([3, 5, 1, 2, 5, 1], np.int32)
    for o in oracles:
        assert o.minmax_element(data) == (2, 1)
        assert o.minmax_element(np.zeros(0, np.int32)) == (0, 0)
        assert o.minmax_element(np.array([7], np.uint8)) == (0, 0)
        assert o.minmax_element(np.full(1000, 4, np.int64)) == (0, 0)        # all equivalent: the first
    rng = np.random.default_rng(11)
    for dt in (np.int8, np.uint8, np.int16, np.uint16, np.int32, np.uint32, np.int64, np.uint64, np.float32, np.float64):
        for n in (1, 2, 33, 1000, 100003):
            x = rng.integers(0, 50, n).astype(dt) if n < 2000 else (rng.standard_normal(n) * 1000).astype(dt)
            assert port.minmax_element(x) == ref.minmax_element(x), (dt, n)
