"""Parity of the CUDA sorts (radix and merge sort, through the C ABI) with the CPU oracle."""
import numpy as np
import pytest
import torch

from thrust_b200 import datagen as dg
from gpu_util import EDGE_SIZES, dev, host, rand_of

pytestmark = pytest.mark.gpu
KEY_TYPES = [np.int8, np.uint8, np.int16, np.uint16, np.int32, np.uint32, np.float32, np.int64, np.uint64, np.float64]
WIDE_KEY_TYPES = KEY_TYPES[4:]


@pytest.mark.parametrize("n", EDGE_SIZES)
def test_sort_by_key_u32_bit_exact_and_stable(tb, oracles, n):
    k = dg.sort_keys_u32(n)
    v = np.arange(n, dtype=np.uint32)             # value = original index: equality proves stability
    kd, vd = dev(k), dev(v)
    tb.sort_by_key(kd, vd)
    for o in oracles:
        ok, ov = o.sort_by_key(k, v)
        assert np.array_equal(host(kd), ok) and np.array_equal(host(vd), ov)


@pytest.mark.parametrize("n", [0, 1, 1000, 8193, 200003])
def test_sort_by_key_u64_40bit_skips_empty_digits(tb, port, n):
    k = dg.sort_keys_u64_40bit(n)
    v = np.arange(n, dtype=np.uint32)
    kd, vd = dev(k), dev(v)
    tb.sort_by_key(kd, vd)
    ok, ov = port.sort_by_key(k, v)
    assert np.array_equal(host(kd), ok) and np.array_equal(host(vd), ov)


def test_sort_all_key_types_orders_and_payloads(tb, port):
    n = 70001
    for dt in KEY_TYPES:
        k = rand_of(dt, n, 51)
        for desc in (False, True):
            kd = dev(k)
            tb.sort(kd, desc)
            ok, _ = port.sort_by_key(k, None, desc)
            assert np.array_equal(host(kd), ok), (dt, desc)
            for vt in (np.uint32, np.uint64):
                few = rand_of(dt, n, 52, small=True)   # many equal keys: stability visible
                v = np.arange(n, dtype=vt)
                kd, vd = dev(few), dev(v)
                tb.sort_by_key(kd, vd, desc)
                ok, ov = port.sort_by_key(few, v, desc)
                assert np.array_equal(host(kd), ok) and np.array_equal(host(vd), ov), (dt, vt, desc)


def test_sort_special_values(tb, port):
    k = np.array([3.5, -0.0, 0.0, -1e30, np.inf, -np.inf, 1e-40, -1e-40, 2.0, -2.0], np.float32)
    k = np.concatenate([k, rand_of(np.float32, 5000, 53)])
    v = np.arange(k.size, dtype=np.uint32)
    kd, vd = dev(k), dev(v)
    tb.sort_by_key(kd, vd)
    ok, ov = port.sort_by_key(k, v)                    # the radix code puts -0.0 before +0.0 on both sides
    assert np.array_equal(host(kd).view(np.uint32), ok.view(np.uint32)) and np.array_equal(host(vd), ov)
    same = np.full(20000, 42, np.int32)                # every digit degenerate: all passes skipped
    kd, vd = dev(same), dev(np.arange(20000, dtype=np.uint32))
    tb.sort_by_key(kd, vd)
    assert np.array_equal(host(vd), np.arange(20000, dtype=np.uint32))
    ext = np.array([np.iinfo(np.int64).min, -1, 0, 1, np.iinfo(np.int64).max] * 700, np.int64)
    kd = dev(ext)
    tb.sort(kd)
    assert np.array_equal(host(kd), np.sort(ext))


def test_sort_bit_range(tb, port):
    """testing/sort_by_key_variable_bits.cu: keys masked to few bits; and an explicit bit window."""
    n = 30011
    for bits in (1, 5, 8, 13, 24):
        k = (dg.sort_keys_u32(n) & np.uint32((1 << bits) - 1)).astype(np.uint32)
        v = np.arange(n, dtype=np.uint32)
        kd, vd = dev(k), dev(v)
        tb.sort_by_key(kd, vd)
        ok, ov = port.sort_by_key(k, v)
        assert np.array_equal(host(kd), ok) and np.array_equal(host(vd), ov), bits
    k = dg.sort_keys_u32(n)
    v = np.arange(n, dtype=np.uint32)
    kd, vd = dev(k), dev(v)
    tb.sort_by_key(kd, vd, begin_bit=8, end_bit=24)    # orders on bits 8..23 only, stably
    order = np.argsort((k >> 8) & 0xFFFF, kind="stable")
    assert np.array_equal(host(vd), v[order]) and np.array_equal(host(kd), k[order])


@pytest.mark.parametrize("n", [0, 1, 2, 33, 4095, 4096, 4097, 8193, 65536 + 17, (1 << 20) + 3])
def test_merge_sort_zip_by_first(tb, oracles, n):
    """stable_sort(zip(u32 key, float value), get<0>(a) < get<0>(b)) on the comparison-sort route."""
    k, v = dg.zip_sort_input(n)
    k = (k >> np.uint32(18)).astype(np.uint32)         # 14-bit keys: ties everywhere
    kd, vd = dev(k), dev(v)
    tb.stable_sort_zip_by_first(kd, vd, method="merge")
    kr, vr = dev(k), dev(v)
    tb.stable_sort_zip_by_first(kr, vr, method="radix")
    for o in oracles:
        ok, ov = o.stable_sort_zip_by_first(k, v.view(np.uint32))
        assert np.array_equal(host(kd), ok) and np.array_equal(host(vd).view(np.uint32), ov)
        assert np.array_equal(host(kr), ok) and np.array_equal(host(vr).view(np.uint32), ov)


def test_merge_sort_types(tb, port):
    n = 50021
    for dt in WIDE_KEY_TYPES:
        k = rand_of(dt, n, 55, small=True)
        v = np.arange(n, dtype=np.uint64)
        for desc in (False, True):
            kd, vd = dev(k), dev(v)
            tb.merge_sort_by_key(kd, vd, desc)
            ok, ov = port.sort_by_key(k, v, desc)
            assert np.array_equal(host(kd), ok) and np.array_equal(host(vd), ov), (dt, desc)
            kd = dev(k)
            tb.merge_sort_by_key(kd, None, desc)
            assert np.array_equal(host(kd), ok)


def test_golden_sorts(tb, golden):
    for n in (1, 777, 12345):
        v = np.arange(n, dtype=np.uint32)
        kd, vd = dev(golden[f"sort_keys_in_{n}"]), dev(v)
        tb.sort_by_key(kd, vd)
        assert np.array_equal(host(kd), golden[f"sort_keys_out_{n}"]) and np.array_equal(host(vd), golden[f"sort_vals_out_{n}"])
        kd, vd = dev(golden[f"sort64_keys_in_{n}"]), dev(v)
        tb.sort_by_key(kd, vd)
        assert np.array_equal(host(kd), golden[f"sort64_keys_out_{n}"]) and np.array_equal(host(vd), golden[f"sort64_vals_out_{n}"])
        kd, vd = dev(golden[f"zip_keys_in_{n}"]), dev(golden[f"zip_vals_in_{n}"])
        tb.stable_sort_zip_by_first(kd, vd)
        assert np.array_equal(host(kd), golden[f"zip_keys_out_{n}"])
        assert np.array_equal(host(vd).view(np.uint32), golden[f"zip_vals_out_{n}"])


def test_full_size_sort_properties(tb):
    """2^28 pairs: sorted, a permutation of the input (keys[i] == original[value[i]]), and stable
    (values increase inside every run of equal keys)."""
    n = 1 << 28
    k0 = dev(dg.sort_keys_u32(n))
    k = k0.clone()
    v = torch.arange(n, dtype=torch.int32, device="cuda").view(torch.uint32)
    tb.sort_by_key(k, v)
    ki, vi = k.view(torch.int32), v.view(torch.int32)
    flipped = ki ^ torch.tensor(-(1 << 31), dtype=torch.int32, device="cuda")      # unsigned order as signed
    assert bool((flipped[1:] >= flipped[:-1]).all())
    assert torch.equal(k0.view(torch.int32)[vi.long()], ki)
    ties = ki[1:] == ki[:-1]
    assert bool((vi[1:][ties] > vi[:-1][ties]).all())
    assert int(vi.long().sum()) == n * (n - 1) // 2


def _sorted_permutation_stable(k0, k, v, as_signed_flip):
    """k is sorted, k == k0[v] (v is the permutation applied) and v increases inside equal keys."""
    if as_signed_flip is not None:                     # unsigned keys compared as signed integers
        f = k ^ as_signed_flip
        assert bool((f[1:] >= f[:-1]).all())
    else:
        assert bool((k[1:] >= k[:-1]).all())
    assert torch.equal(k0[v.long()], k)
    ties = k[1:] == k[:-1]
    assert bool((v[1:][ties] > v[:-1][ties]).all())
    n = k.numel()
    assert int(v.long().sum()) == n * (n - 1) // 2


def test_full_size_sort_u64_40bit_properties(tb):
    """The second sort configuration at its size: 2^27 uint64 keys with 40 random bits (three digit
    places are skipped on the device) and uint32 values = original index."""
    n = 1 << 27
    k0 = dev(dg.sort_keys_u64_40bit(n)).view(torch.int64)     # < 2^40: signed and unsigned order agree
    k = k0.clone()
    v = torch.arange(n, dtype=torch.int32, device="cuda")
    tb.sort_by_key(k.view(torch.uint64), v.view(torch.uint32))
    _sorted_permutation_stable(k0, k, v, None)


def test_full_size_sort_u32_half_size_properties(tb):
    n = 1 << 27
    k0 = dev(dg.sort_keys_u32(n, seed=12)).view(torch.int32)
    k = k0.clone()
    v = torch.arange(n, dtype=torch.int32, device="cuda")
    tb.sort_by_key(k.view(torch.uint32), v.view(torch.uint32))
    _sorted_permutation_stable(k0, k, v, torch.tensor(-(1 << 31), dtype=torch.int32, device="cuda"))


def test_full_size_stable_sort_zip_both_routes(tb):
    """stable_sort of 2^26 zip(u32 key, float value) pairs by the key alone, on the comparison
    (merge sort) route and on the radix route: each result sorted, a permutation, stable; the float
    payload is the original index as a bit pattern, which must travel bit for bit."""
    n = 1 << 26
    k0 = dev(dg.zip_sort_input(n)[0] >> np.uint32(8)).view(torch.int32)      # 24-bit keys: plenty of ties
    idx = torch.arange(n, dtype=torch.int32, device="cuda")
    outs = []
    for method in ("merge", "radix"):
        k, v = k0.clone(), idx.clone()
        tb.stable_sort_zip_by_first(k.view(torch.uint32), v.view(torch.float32), method=method)
        _sorted_permutation_stable(k0, k, v, None)
        outs.append((k, v))
    assert torch.equal(outs[0][0], outs[1][0]) and torch.equal(outs[0][1], outs[1][1])


@pytest.mark.parametrize("n", [0, 1, 4097, 200003, (1 << 22) + 5])
def test_sort_by_key_host_buffers_match_the_oracle(tb, port, n):
    """The host-buffer call (keys and values in pinned host memory; values permuted by the sorted
    positions) gives exactly what the reference's stable sort_by_key gives, ties included."""
    for kdt, vdt, desc in ((np.uint32, np.uint32, False), (np.float32, np.int64, True), (np.int64, np.float32, False)):
        k = rand_of(kdt, n, 77, small=(kdt == np.int64))          # small: many equal keys, so stability shows
        v = rand_of(vdt, n, 78)
        hk, hv = torch.from_numpy(k.copy()).pin_memory(), torch.from_numpy(v.copy()).pin_memory()
        ok_, ov_ = torch.empty_like(hk).pin_memory(), torch.empty_like(hv).pin_memory()
        tb.sort_by_key_host(hk, hv, ok_, ov_, descending=desc)
        wk, wv = port.sort_by_key(k, v, descending=desc)
        assert np.array_equal(ok_.numpy().view(np.uint8), wk.view(np.uint8)) and np.array_equal(ov_.numpy().view(np.uint8), wv.view(np.uint8)), (kdt, n)
        assert np.array_equal(hk.numpy().view(np.uint8), k.view(np.uint8))             # inputs untouched when outputs are given
        tb.sort_by_key_host(hk, hv, descending=desc)                                   # in place
        assert np.array_equal(hk.numpy().view(np.uint8), wk.view(np.uint8)) and np.array_equal(hv.numpy().view(np.uint8), wv.view(np.uint8))
