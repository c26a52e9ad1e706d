"""The seeded generators are counter based: any slice can be produced independently."""
import numpy as np

from thrust_b200 import datagen as dg


def test_streams_are_sliceable_and_distinct():
    a = dg.rand64(2, 1000)
    assert np.array_equal(a[100:200], dg.rand64(2, 100, start=100))
    assert not np.array_equal(a, dg.rand64(3, 1000))
    assert np.array_equal(dg.sort_keys_u32(64, start=64), dg.sort_keys_u32(128)[64:])


def test_value_ranges():
    n = 1 << 16
    x = dg.reduce_input(n)
    assert x.dtype == np.int32 and x.min() >= -(1 << 20) and x.max() < (1 << 20)
    s = dg.scan_input_i32(n)
    assert s.min() == 0 and s.max() == 15
    f = dg.scan_input_f32(n)
    assert f.dtype == np.float32 and f.min() >= 0 and f.max() < 1
    k = dg.sort_keys_u64_40bit(n)
    assert k.max() < (1 << 40) and k.max() > (1 << 39)
    c = dg.compaction_input(n)
    assert c.min() >= 0 and abs((c % 2 == 0).mean() - 0.5) < 0.02
    r = dg.run_keys(n)
    assert (np.diff(r) >= 0).all() and abs(n / (r[-1] + 1) - 4.0) < 0.2
    m = dg.merge_keys_u64(n, 4)
    assert (np.diff(m.astype(np.int64)) >= 0).all() and m.max() < (1 << 48)
