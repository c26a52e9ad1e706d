"""Helpers for the GPU parity tests."""
import numpy as np
import torch

from thrust_b200 import datagen as dg

# sizes that cross every tile boundary used by the kernels (4096-, 3840-, 8192-item tiles, warp
# chunks of 512 items), plus empty and single-element inputs
EDGE_SIZES = [0, 1, 2, 31, 32, 33, 511, 513, 3839, 3841, 4095, 4096, 4097, 8191, 8193, 65536 + 17, (1 << 20) + 3]
WIDE = [np.int32, np.uint32, np.int64, np.uint64, np.float32, np.float64]
ALL = [np.int8, np.uint8, np.int16, np.uint16] + WIDE


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def host(t):
    return t.cpu().numpy()


def rand_of(dtype, n, seed, small=False):
    u = dg.rand64(seed, n)
    if small:
        u = u % np.uint64(7)
    dt = np.dtype(dtype)
    if dt.kind == "f":
        x = ((u >> np.uint64(40)).astype(np.float64) / 2.0 ** 23 - 1.0)
        x = (np.round(x * 8) / 8 if small else x).astype(dt)
        x[x == 0] = 0.0
        return x
    return u.astype(dt)


def misaligned(a, offset=1):
    """A device tensor whose data pointer is `offset` elements past a 16-byte boundary."""
    buf = torch.empty(a.size + 64, dtype=dev(a[:0]).dtype, device="cuda")
    view = buf[offset:offset + a.size]
    view.copy_(dev(a))
    return view
