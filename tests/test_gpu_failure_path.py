"""A bounded wait that runs out: the kernel returns, the status word says so, the host raises.

Every inter-CTA wait in the library gives up after a fixed number of polls, records status 1 in the
workspace header and carries on, so a broken launch can never hang the device.  This test makes one
run out without faulting or hanging anything: it loads the TEST build of the scan entry points
(thrust_b200.build.build_shortwait: 64 polls instead of 2^23) and switches on its hook that makes
the first tile of a single-pass scan withhold its descriptor.  Every index stays in bounds; the later
tiles' polls of tile 0 simply expire after a few microseconds.  Afterwards the same workspace serves
an ordinary call again."""
import ctypes as C
import os

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def test_lookback_timeout_is_reported_and_recoverable(tb, port, monkeypatch):
    import torch
    from thrust_b200 import _lib, api, build, datagen as dg
    if not os.path.isfile(build.SHORTWAIT_LIB):
        pytest.fail("%s is missing -- python -m thrust_b200.build makes it" % build.SHORTWAIT_LIB)
    short = _lib.load_partial(build.SHORTWAIT_LIB)
    short.tb200_test_hooks.argtypes = [C.c_uint]
    short.tb200_test_hooks.restype = C.c_int
    n = 5 * 8192 + 123                                   # six tiles of the single-pass kernel
    x_h = dg.scan_input_i32(n)
    x = torch.from_numpy(x_h).cuda()
    out = torch.empty_like(x)
    need = C.c_size_t(0)
    assert short.tb200_inclusive_scan(None, None, n, 4, 0, None, None, C.byref(need), None) == 0
    ws = torch.zeros(need.value, dtype=torch.uint8, device="cuda")
    p = lambda t: C.c_void_p(t.data_ptr())  # noqa: E731
    status = C.c_uint(7)

    # 1. the wait runs out: the call itself succeeds (it only enqueues), the kernel returns, status = 1
    assert short.tb200_test_hooks(1) == 0
    assert short.tb200_inclusive_scan(p(x), p(out), n, 4, 0, None, p(ws), C.byref(need), None) == 0
    assert short.tb200_workspace_status(p(ws), None, C.byref(status)) == 0
    assert status.value == 1
    torch.cuda.synchronize()                              # the context is alive and well

    # 2. the host side of the library turns that status into an exception
    monkeypatch.setattr(_lib, "_lib", short)
    with pytest.raises(api.Tb200Error):
        tb.inclusive_scan(x)

    # 3. hook off: the same workspace and the same (short-wait) kernels give the right answer again
    assert short.tb200_test_hooks(0) == 0
    got = tb.inclusive_scan(x)
    assert np.array_equal(got.cpu().numpy(), port.inclusive_scan(x_h))
    assert short.tb200_inclusive_scan(p(x), p(out), n, 4, 0, None, p(ws), C.byref(need), None) == 0
    assert short.tb200_workspace_status(p(ws), None, C.byref(status)) == 0 and status.value == 0
    assert np.array_equal(out.cpu().numpy(), port.inclusive_scan(x_h))
