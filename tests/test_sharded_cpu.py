"""The multi-GPU orchestration (thrust_b200/sharded.py) run as two gloo ranks on CPU, with the
oracle standing in for the per-GPU kernels: checks the carry logic of the sharded scan, the
splitter / all-to-all / merge plumbing of the sharded sort (bit-exact and stable against a
single-process sort of the concatenation), and the sharded reduce."""
import os
import socket
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


class HostOps:
    """Same interface as sharded.DeviceOps, computed by the CPU oracle on CPU tensors."""

    def __init__(self):
        from oracle import oracle
        self.o = oracle.load_port()

    @staticmethod
    def _np(t):
        from thrust_b200 import api
        return t.numpy().view(api.NP_OF[t.dtype]) if t is not None else None

    def reduce(self, x, init, op):
        return self.o.reduce(self._np(x), init, op)

    def inclusive_scan(self, x, op, init):
        a = self._np(x)
        if init is None:
            return torch.from_numpy(self.o.inclusive_scan(a, op))
        ex = self.o.exclusive_scan(np.concatenate([a, a[:1]]), init, op)   # inclusive with carry = shifted exclusive
        return torch.from_numpy(ex[1:].copy()) if a.size else x.clone()

    def exclusive_scan(self, x, op, init):
        return torch.from_numpy(self.o.exclusive_scan(self._np(x), init, op))

    def sort_by_key(self, keys, vals, descending):
        k, v = self.o.sort_by_key(self._np(keys), self._np(vals), descending)
        self._np(keys)[:] = k
        if vals is not None:
            self._np(vals)[:] = v

    def merge_by_key(self, ka, kb, va, vb, descending):
        k, v = self.o.merge_by_key(self._np(ka), self._np(kb), self._np(va), self._np(vb), descending)
        return torch.from_numpy(k), None if v is None else torch.from_numpy(v)

    def lower_bound(self, sorted_keys, needles, descending):
        s, nd = self._np(sorted_keys), self._np(needles)
        if descending:
            return torch.from_numpy(np.array([int(np.sum(s > x)) for x in nd], dtype=np.int64))
        return torch.from_numpy(np.searchsorted(s, nd, side="left").astype(np.int64))


def _worker(rank, world, port, case, out_dir):
    sys.path.insert(0, ROOT)
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from thrust_b200 import datagen as dg, sharded
    ops = HostOps()
    try:
        n_total = 50000 + 13
        lo, hi = rank * n_total // world, (rank + 1) * n_total // world
        if case == "reduce":
            x = torch.from_numpy(dg.reduce_input(hi - lo, start=lo))
            got = sharded.sharded_reduce(x, np.int64(5), "plus", ops=ops)
            want = np.int64(5) + dg.reduce_input(n_total).sum(dtype=np.int64)
            assert got == want, (got, want)
            assert sharded.sharded_reduce(x, np.int64(0), "max", ops=ops) == dg.reduce_input(n_total).max()
            # unsigned accumulators with the top bit set, one empty shard: a signed all-reduce would get these wrong
            for dt, top in ((np.uint32, np.uint32(1 << 31)), (np.uint64, np.uint64(1 << 63))):
                full = (dg.rand64(9, n_total).astype(dt) | top).astype(dt)
                mine = full[lo:hi] if rank != world - 1 else full[:0]
                seen = full[:(world - 1) * n_total // world]
                assert sharded.sharded_reduce(torch.from_numpy(mine.copy()), np.asarray(np.iinfo(dt).max, dt)[()], "min", ops=ops) == seen.min()
                assert sharded.sharded_reduce(torch.from_numpy(mine.copy()), np.asarray(0, dt)[()], "max", ops=ops) == seen.max()
            f = np.full(4, -np.inf, np.float32)
            assert sharded.sharded_reduce(torch.from_numpy(f), np.float32(-np.inf), "max", ops=ops) == -np.inf
        elif case == "scan":
            full = dg.scan_input_i32(n_total)
            x = torch.from_numpy(full[lo:hi].copy())
            inc = sharded.sharded_scan(x, ops=ops).numpy()
            assert np.array_equal(inc, np.cumsum(full, dtype=np.int32)[lo:hi])
            exc = sharded.sharded_scan(x, exclusive=True, init=7, ops=ops).numpy()
            assert np.array_equal(exc, (np.cumsum(full, dtype=np.int32) - full + 7)[lo:hi])
            mx = sharded.sharded_scan(x, op="max", ops=ops).numpy()
            assert np.array_equal(mx, np.maximum.accumulate(full)[lo:hi])
        elif case in ("sort", "sort_desc_ties"):
            desc = case == "sort_desc_ties"
            keys_full = dg.sort_keys_u32(n_total)
            if desc:
                keys_full = (keys_full >> np.uint32(24)).astype(np.uint32)        # 8-bit keys: heavy ties across ranks
            vals_full = np.arange(n_total, dtype=np.uint32)
            k, v = sharded.sharded_sort_by_key(torch.from_numpy(keys_full[lo:hi].copy()), torch.from_numpy(vals_full[lo:hi].copy()),
                                               descending=desc, ops=ops, samples_per_rank=64)
            np.save(os.path.join(out_dir, f"k{rank}.npy"), ops._np(k))
            np.save(os.path.join(out_dir, f"v{rank}.npy"), ops._np(v))
            dist.barrier()
            if rank == 0:
                kk = np.concatenate([np.load(os.path.join(out_dir, f"k{r}.npy")) for r in range(world)])
                vv = np.concatenate([np.load(os.path.join(out_dir, f"v{r}.npy")) for r in range(world)])
                wk, wv = ops.o.sort_by_key(keys_full, vals_full, desc)
                assert np.array_equal(kk, wk) and np.array_equal(vv, wv)
    finally:
        dist.destroy_process_group()


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


@pytest.mark.parametrize("case", ["reduce", "scan", "sort", "sort_desc_ties"])
@pytest.mark.parametrize("world", [2, 3])
def test_sharded_orchestration_on_gloo(case, world, tmp_path):
    mp.spawn(_worker, args=(world, _free_port(), case, str(tmp_path)), nprocs=world, join=True)


def test_choose_splitters():
    from thrust_b200.sharded import choose_splitters
    s = choose_splitters(np.array([5, 1, 9, 3, 7, 2, 8, 4], np.uint32), 4)
    assert s.tolist() == [3, 5, 8]
    assert choose_splitters(np.array([1, 2, 3, 4], np.uint32), 2, descending=True).tolist() == [2]
    assert choose_splitters(np.empty(0, np.uint32), 4).size == 0
