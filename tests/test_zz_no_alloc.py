"""tb200_inclusive_scan_static: the scan for callers that cannot allocate device memory (a plug-in
without an allocator, a loop that must not hit cudaMalloc's synchronisation, a process whose data
already fills the device).  Its scratch is a fixed array inside the library, so this test checks,
through the C ABI, that it gives the CPU oracle's answer and the ordinary entry point's -- twice in
a row, because the second call finds the array as the first one left it -- that its status
read-out works, and that it refuses inputs whose descriptors would not fit.  This file sorts last so that every other test has already run
when it starts; it also passes on its own in a fresh process."""
import ctypes as C

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

EXCEEDS = 100001


def _scan_with_workspace(lib, torch, x, t, op, init):
    out = torch.empty_like(x)
    need = C.c_size_t(0)
    h = None if init is None else C.c_void_p(init.ctypes.data)
    assert lib.tb200_inclusive_scan(None, None, x.numel(), t, op, h, None, C.byref(need), None) == 0
    ws = torch.empty(need.value, dtype=torch.uint8, device="cuda")
    rc = lib.tb200_inclusive_scan(C.c_void_p(x.data_ptr()), C.c_void_p(out.data_ptr()), x.numel(), t, op, h,
                                  C.c_void_p(ws.data_ptr()), C.byref(need), None)
    assert rc == 0
    torch.cuda.synchronize()
    return out


def _scan_static(lib, torch, x, t, op, init):
    out = torch.empty_like(x)
    h = None if init is None else C.c_void_p(init.ctypes.data)
    rc = lib.tb200_inclusive_scan_static(C.c_void_p(x.data_ptr()), C.c_void_p(out.data_ptr()), x.numel(), t, op, h, None)
    assert rc == 0, rc
    torch.cuda.synchronize()
    return out


def _status(lib):
    st = C.c_uint(99)
    assert lib.tb200_inclusive_scan_static_status(None, C.byref(st)) == 0
    return st.value


def test_static_scratch_scan_matches_oracle_and_workspace_scan_twice(tb, port):
    import torch
    from thrust_b200 import datagen as dg
    lib = tb._lib.load()
    # first call: an input large enough for the windowed route leaves many descriptors behind in
    # the shared array
    big_h = dg.scan_input_i32((1 << 24) + 12345)
    big = torch.from_numpy(big_h).cuda()
    got = _scan_static(lib, torch, big, 4, 0, None)
    assert np.array_equal(got.cpu().numpy(), port.inclusive_scan(big_h))           # bit-exact against the oracle
    assert torch.equal(got, _scan_with_workspace(lib, torch, big, 4, 0, None))
    assert _status(lib) == 0
    # second call, straight after, on different data and a shorter length (single-pass kernel):
    # stale descriptors of the first call must not leak into it
    small_h = dg.scan_input_i32(300001, seed=8)
    small = torch.from_numpy(small_h).cuda()
    init = np.asarray(17, dtype=np.int32)
    got = _scan_static(lib, torch, small, 4, 0, init)
    assert np.array_equal(got.cpu().numpy(), port.inclusive_scan(small_h) + 17)
    assert torch.equal(got, _scan_with_workspace(lib, torch, small, 4, 0, init))
    assert _status(lib) == 0
    # and once more with another type and operator (fp32 max is exact, so bit-equality holds)
    f = torch.from_numpy(dg.scan_input_f32(777777)).cuda()
    assert torch.equal(_scan_static(lib, torch, f, 8, 2, None), _scan_with_workspace(lib, torch, f, 8, 2, None))
    # fp32 plus: same tolerance as the scan parity test (1e-5 relative of the fp64-accumulated yardstick)
    a = _scan_static(lib, torch, f, 8, 0, None).double().cpu().numpy()
    yard = port.scan_f32_via_f64(f.cpu().numpy()).astype(np.float64)
    assert float(np.max(np.abs(a - yard) / np.maximum(yard, 1.0))) < 1e-5
    # empty input is fine and touches nothing
    e = torch.empty(0, dtype=torch.int32, device="cuda")
    assert _scan_static(lib, torch, e, 4, 0, None).numel() == 0


def test_static_scratch_scan_rejects_oversized_input(tb):
    import torch
    lib = tb._lib.load()
    x = torch.zeros(16, dtype=torch.int64, device="cuda")
    p = C.c_void_p(x.data_ptr())
    lim4, lim8 = C.c_size_t(0), C.c_size_t(0)
    assert lib.tb200_inclusive_scan_static_limit(4, C.byref(lim4)) == 0 and lib.tb200_inclusive_scan_static_limit(6, C.byref(lim8)) == 0
    assert (1 << 28) <= lim4.value < (1 << 30) and (1 << 26) <= lim8.value < lim4.value     # the benchmark size fits
    assert lib.tb200_inclusive_scan_static(p, p, lim4.value + 1, 4, 0, None, None) == EXCEEDS   # one past the limit, 4-byte type
    assert lib.tb200_inclusive_scan_static(p, p, lim8.value + 1, 6, 0, None, None) == EXCEEDS   # 8-byte type hits it sooner
    assert lib.tb200_inclusive_scan_static(p, p, 1 << 30, 4, 0, None, None) == EXCEEDS
    assert lib.tb200_inclusive_scan_static(p, p, 16, 0, 0, None, None) == 801             # int8 is not a scan type
    torch.cuda.synchronize()
    assert int(x.sum()) == 0                                                               # refused calls did nothing
