"""The exchange step of the multi-GPU sort_by_key, run for G emulated ranks on ONE GPU: the three
kernels (digit histogram, plan, scatter) are plain independent launches that never wait on one
another, so the ranks' steps run one after the other with every receive buffer in local memory.
The concatenation of the locally sorted receive buffers must be, bit for bit, the oracle's stable
sort of the concatenated shards -- for rank counts a test box with fewer GPUs cannot otherwise reach."""
import ctypes as C

import numpy as np
import pytest
import torch

from thrust_b200 import api, datagen as dg
from thrust_b200.sharded import DeviceOps
from gpu_util import dev, host

pytestmark = pytest.mark.gpu


def _run(tb, shards_k, shards_v, descending=False):
    ops = DeviceOps()
    G = len(shards_k)
    kdt, vdt = shards_k[0].dtype, shards_v[0].dtype
    st = ops.exchange_state(shards_k[0].device, kdt, vdt)
    rows = []
    for r in range(G):
        rows.append(ops.exchange_hist(st, shards_k[r], descending, (1 << 32) | 7).clone())
    rows = torch.cat(rows)
    plans = []
    for r in range(G):
        plans.append(ops.exchange_plan(st, rows, G, r, kdt).clone())
    head = plans[0][:st["head_bytes"]].cpu().numpy()
    table = head[8:].view(np.uint64).reshape(3, -1)
    recv_total = table[1, :G].astype(np.int64)
    assert int(recv_total.sum()) == sum(k.numel() for k in shards_k)
    recv_k = [torch.empty(max(int(t), 1), dtype=kdt, device="cuda") for t in recv_total]
    recv_v = [torch.empty(max(int(t), 1), dtype=vdt, device="cuda") for t in recv_total]
    for r in range(G):
        if shards_k[r].numel():
            ops.exchange_scatter(shards_k[r], shards_v[r], plans[r], [t.data_ptr() for t in recv_k], [t.data_ptr() for t in recv_v], descending)
    torch.cuda.synchronize()
    out_k, out_v = [], []
    for d in range(G):
        k, v = recv_k[d][:int(recv_total[d])], recv_v[d][:int(recv_total[d])]
        tb.sort_by_key(k, v, descending)
        out_k.append(host(k)); out_v.append(host(v))
    return np.concatenate(out_k), np.concatenate(out_v), recv_total


@pytest.mark.parametrize("G", [2, 3, 8, 16])
def test_emulated_ranks_exchange_then_local_sort_equals_the_oracle(tb, port, G):
    per = 150001
    for kind in ("u32", "ties", "u64", "f32desc"):
        ks, vs = [], []
        for r in range(G):
            u = dg.rand64(900 + r, per if r != 1 else per // 3)          # one short shard
            if kind == "u32":
                k = (u >> np.uint64(32)).astype(np.uint32)
            elif kind == "ties":
                k = (u % np.uint64(1000)).astype(np.uint32) << np.uint32(18)
            elif kind == "u64":
                k = (u >> np.uint64(24)).astype(np.uint64)
            else:
                k = ((u >> np.uint64(40)).astype(np.float64) / 2.0 ** 23 - 1.0).astype(np.float32)
            ks.append(k)
            vs.append((np.arange(k.size, dtype=np.uint32) + np.uint32(r << 24)))
        desc = kind == "f32desc"
        gk, gv, totals = _run(tb, [dev(k) for k in ks], [dev(v) for v in vs], desc)
        wk, wv = port.sort_by_key(np.concatenate(ks), np.concatenate(vs), descending=desc)
        assert np.array_equal(gk.view(np.uint8), wk.view(np.uint8)) and np.array_equal(gv, wv), (G, kind)
        if kind == "u32":
            assert totals.max() <= 1.1 * totals.mean() + 4096, totals        # balanced to about one bin
