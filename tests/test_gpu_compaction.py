"""Parity of copy_if, partition, unique and reduce_by_key (through the C ABI) with the CPU oracle."""
import numpy as np
import pytest
import torch

from thrust_b200 import datagen as dg
from gpu_util import ALL, EDGE_SIZES, WIDE, dev, host, misaligned, rand_of

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("n", EDGE_SIZES)
def test_copy_if_and_partition_bit_exact(tb, oracles, n):
    x = dg.compaction_input(n)
    got = host(tb.copy_if(dev(x), "mod_eq", 2, 0))
    gt, gf = tb.partition_copy(dev(x), "mod_eq", 2, 0)
    d = dev(x)
    split = tb.partition(d, "mod_eq", 2, 0)
    for o in oracles:
        assert np.array_equal(got, o.copy_if(x, "mod_eq", 2, 0))
        ot, of = o.partition_copy(x, "mod_eq", 2, 0)
        assert np.array_equal(host(gt), ot) and np.array_equal(host(gf), of)
        sd, sc = o.stable_partition(x, "mod_eq", 2, 0)
        assert split == sc and np.array_equal(host(d), sd)
        # thrust::partition contract: split point and selected half exact, rejected half as a multiset
        # (testing/partition.cu:309-312 sorts both halves before comparing)
        ud, uc = o.partition(x, "mod_eq", 2, 0)
        assert split == uc and np.array_equal(host(d)[:split], ud[:uc])
        assert np.array_equal(np.sort(host(d)[split:]), np.sort(ud[uc:]))


def test_copy_if_types_predicates_stencils(tb, port):
    n = 33333
    for dt in ALL:
        x = rand_of(dt, n, 61, small=True)
        preds = [("ne", 3, 0), ("lt", 3, 0), ("ge", 2, 0)] + ([("mod_eq", 3, 1)] if np.dtype(dt).kind != "f" else [])
        for pred, a, b in preds:
            assert np.array_equal(host(tb.copy_if(dev(x), pred, a, b)), port.copy_if(x, pred, a, b)), (dt, pred)
            gt, gf = tb.partition_copy(dev(x), pred, a, b)
            ot, of = port.partition_copy(x, pred, a, b)
            assert np.array_equal(host(gt), ot) and np.array_equal(host(gf), of), (dt, pred)
            d = dev(x)
            split = tb.stable_partition(d, pred, a, b)
            sd, sc = port.stable_partition(x, pred, a, b)
            assert split == sc and np.array_equal(host(d), sd), (dt, pred)
        for st_dt in (np.uint8, np.int32):
            st = rand_of(st_dt, n, 62, small=True)
            assert np.array_equal(host(tb.copy_if(dev(x), "ne", 0, 0, stencil=dev(st))), port.copy_if(x, "ne", 0, 0, stencil=st)), (dt, st_dt)
            gt, gf = tb.partition_copy(dev(x), "ge", 3, 0, stencil=dev(st))
            keep = st >= 3
            assert np.array_equal(host(gt), x[keep]) and np.array_equal(host(gf), x[~keep]), (dt, st_dt)


def test_copy_if_extremes_in_place_misaligned(tb, port):
    x = dg.compaction_input(100001)
    assert tb.copy_if(dev(x), "lt", 0, 0).numel() == 0                        # nothing selected
    assert np.array_equal(host(tb.copy_if(dev(x), "ge", 0, 0)), x)            # everything selected
    d = dev(x)
    out = tb.copy_if(d, "mod_eq", 2, 0, out=d)                                # result == first (remove_if, remove.h:38-65)
    assert np.array_equal(host(out), port.copy_if(x, "mod_eq", 2, 0))
    assert np.array_equal(host(tb.copy_if(misaligned(x, 3), "mod_eq", 2, 0)), port.copy_if(x, "mod_eq", 2, 0))


@pytest.mark.parametrize("dt", [np.int32, np.int64])
def test_compaction_large_bit_exact(tb, oracles, dt):
    """2^25 + 12345 items (thousands of tiles, a partial last one), out of place and in place."""
    n = (1 << 25) + 12345
    x = dg.compaction_input(n).astype(dt)
    keys = dg.run_keys(n).astype(dt)
    stencil = (dg.scan_input_i32(n, 9) & 3).astype(np.int32)
    got = host(tb.copy_if(dev(x), "mod_eq", 3, 1))
    got_st = host(tb.copy_if(dev(x), "ne", 0, 0, stencil=dev(stencil)))
    gt, gf = tb.partition_copy(dev(x), "lt", 1 << 20, 0)
    d = dev(x)
    split = tb.partition(d, "mod_eq", 2, 0)
    u = host(tb.unique_copy(dev(keys)))
    dk = dev(keys)
    ui = host(tb.unique(dk))
    for o in oracles:
        assert np.array_equal(got, o.copy_if(x, "mod_eq", 3, 1))
        assert np.array_equal(got_st, o.copy_if(x, "ne", 0, 0, stencil=stencil))
        ot, of = o.partition_copy(x, "lt", 1 << 20, 0)
        assert np.array_equal(host(gt), ot) and np.array_equal(host(gf), of)
        sd, sc = o.stable_partition(x, "mod_eq", 2, 0)
        assert split == sc and np.array_equal(host(d), sd)
        ref_u = o.unique_copy(keys)
        assert np.array_equal(u, ref_u) and np.array_equal(ui, ref_u)


@pytest.mark.parametrize("kt,vt", [(np.int32, np.int32), (np.uint32, np.float32), (np.int64, np.int64), (np.uint64, np.float64), (np.int32, np.int64)])
def test_reduce_by_key_large_bit_exact(tb, oracles, kt, vt):
    """2^25 + 12345 items: keys and values of one size take the two-pass streaming kernels, mixed
    sizes the single-pass one; the last row of the input is partial.  Integer sums, minima and the
    first-of-run selection of unique_by_key are exact; floating-point values are small integers here,
    so their sums are exact too."""
    n = (1 << 25) + 12345
    keys = dg.run_keys(n).astype(kt)
    vals = (dg.scan_input_i32(n, 7) % 1000).astype(vt)
    ko, vo = tb.reduce_by_key(dev(keys), dev(vals))
    km, vm = tb.reduce_by_key(dev(keys), dev(vals), op="min")
    uk, uv = (None, None)
    if np.dtype(vt).itemsize in (4, 8):
        uk, uv = tb.unique_by_key_copy(dev(keys), dev(vals))
    dk, dv = dev(keys), dev(vals)
    ik, iv = tb.unique_by_key(dk, dv)                                          # in place: single-pass kernel
    for o in oracles:
        rk, rv = o.reduce_by_key(keys, vals)
        assert np.array_equal(host(ko), rk) and np.array_equal(host(vo), rv)
        mk, mv = o.reduce_by_key(keys, vals, "min")
        assert np.array_equal(host(km), mk) and np.array_equal(host(vm), mv)
        fk, fv = o.unique_by_key_copy(keys, vals)
        assert np.array_equal(host(uk), fk) and np.array_equal(host(uv), fv)
        assert np.array_equal(host(ik), fk) and np.array_equal(host(iv), fv)


@pytest.mark.parametrize("n", EDGE_SIZES)
def test_unique_and_reduce_by_key(tb, oracles, n):
    keys = dg.run_keys(n)
    ivals = dg.scan_input_i32(n, 7)
    fvals = dg.run_values_f32(n)
    u = host(tb.unique_copy(dev(keys)))
    d = dev(keys)
    ui = host(tb.unique(d))                                                   # in place, unique.h:772
    ko, vo = tb.reduce_by_key(dev(keys), dev(ivals))
    kf, vf = tb.reduce_by_key(dev(keys), dev(fvals))
    for o in oracles:
        ref_u = o.unique_copy(keys)
        assert np.array_equal(u, ref_u) and np.array_equal(ui, ref_u)
        rk, rv = o.reduce_by_key(keys, ivals)
        assert np.array_equal(host(ko), rk) and np.array_equal(host(vo), rv)
        # fp32 values: keys and run count exact, sums within 1e-6 relative of the fp64 yardstick
        yk, yv = o.reduce_by_key_f32_via_f64(keys, fvals)
        assert np.array_equal(host(kf), yk)
        assert np.allclose(host(vf), yv, rtol=1e-6, atol=0)


def test_unique_rbk_types_and_shapes(tb, port):
    n = 40009
    for dt in ALL:
        x = rand_of(dt, n, 63, small=True)
        assert np.array_equal(host(tb.unique_copy(dev(x))), port.unique_copy(x)), dt
        for vt in WIDE:
            vals = rand_of(vt, n, 64, small=True)
            for op in ("plus", "min", "max"):
                gk, gv = tb.reduce_by_key(dev(x), dev(vals), op)
                rk, rv = port.reduce_by_key(x, vals, op)
                assert np.array_equal(host(gk), rk) and np.array_equal(host(gv), rv), (dt, vt, op)
    # one long run spanning many tiles, all-distinct keys, alternating keys
    for keys in (np.zeros(50000, np.int32), np.arange(50000, dtype=np.int32), (np.arange(50000) % 2).astype(np.int32)):
        vals = np.ones(keys.size, np.int64)
        gk, gv = tb.reduce_by_key(dev(keys), dev(vals))
        rk, rv = port.reduce_by_key(keys, vals)
        assert np.array_equal(host(gk), rk) and np.array_equal(host(gv), rv)
        assert np.array_equal(host(tb.unique_copy(dev(keys))), port.unique_copy(keys))
    f = np.array([0.0, -0.0, 1.0, np.nan, np.nan, 2.0, 2.0], np.float32)     # IEEE equality: -0 == 0, NaN != NaN
    assert host(tb.unique_copy(dev(f))).size == port.unique_copy(f).size == 5


def test_golden_compaction(tb, golden):
    for n in (1, 777, 12345):
        c = golden[f"compact_in_{n}"]
        assert np.array_equal(host(tb.copy_if(dev(c), "mod_eq", 2, 0)), golden[f"copy_if_out_{n}"])
        d = dev(c)
        assert tb.stable_partition(d, "mod_eq", 2, 0) == golden[f"partition_count_{n}"]
        assert np.array_equal(host(d), golden[f"stable_partition_out_{n}"])
        assert np.array_equal(host(tb.unique_copy(dev(golden[f"run_keys_{n}"]))), golden[f"unique_out_{n}"])
        gk, gv = tb.reduce_by_key(dev(golden[f"run_keys_{n}"]), dev(golden[f"run_vals_{n}"]))
        assert np.array_equal(host(gk), golden[f"rbk_keys_out_{n}"]) and np.array_equal(host(gv), golden[f"rbk_vals_out_{n}"])


def test_full_size_compaction_properties(tb):
    """2^28 elements: copy_if output equals a boolean-mask selection; partition halves concatenate to
    a stable split; unique of run keys is 0..runs-1; reduce_by_key of ones gives the run lengths."""
    n = 1 << 28
    x = dev(dg.compaction_input(n))
    sel = tb.copy_if(x, "mod_eq", 2, 0)
    mask = (x & 1) == 0
    assert sel.numel() == int(mask.sum()) and torch.equal(sel, x[mask])
    del sel
    d = x.clone()
    split = tb.partition(d, "mod_eq", 2, 0)
    assert split == int(mask.sum()) and torch.equal(d[:split], x[mask]) and torch.equal(d[split:], x[~mask])
    del d, x, mask
    keys = dev(dg.run_keys(n))
    runs = int(keys[-1]) + 1
    u = tb.unique_copy(keys)
    assert u.numel() == runs and torch.equal(u, torch.arange(runs, dtype=torch.int32, device="cuda"))
    del u
    ones = torch.ones(n, dtype=torch.int32, device="cuda")
    gk, gv = tb.reduce_by_key(keys, ones)
    assert gk.numel() == runs and int(gv.sum()) == n
    assert torch.equal(gv, torch.bincount(keys, minlength=runs).to(torch.int32))


def test_full_size_reduce_by_key_fp32(tb):
    """reduce_by_key at the benchmark size with its fp32 values in [0, 1): output keys and run count
    exact (against bincount), every segment sum within 1e-6 relative of an fp64 segment sum."""
    n = 1 << 28
    keys = dev(dg.run_keys(n))
    vals = dev(dg.run_values_f32(n))
    runs = int(keys[-1]) + 1
    gk, gv = tb.reduce_by_key(keys, vals)
    assert gk.numel() == runs and gv.numel() == runs
    assert torch.equal(gk, torch.arange(runs, dtype=torch.int32, device="cuda"))
    del gk
    yard = torch.zeros(runs, dtype=torch.float64, device="cuda")
    step = 1 << 26                                       # bounded temporaries
    for lo in range(0, n, step):
        yard.index_add_(0, keys[lo:lo + step].long(), vals[lo:lo + step].double())
    err = (gv.double() - yard).abs() / yard.clamp(min=1e-30)
    assert float(err.max()) < 1e-6, float(err.max())
