"""Multi-GPU reduce, scan and sort_by_key (thrust_b200/sharded.py over NCCL) against the oracle run on
the concatenated input.  Needs at least two GPUs; skipped otherwise."""
import os
import socket
import sys

import numpy as np
import pytest

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _worker(rank, world, port, out_dir):
    sys.path.insert(0, ROOT)
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    import torch
    import torch.distributed as dist
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        from thrust_b200 import datagen as dg, sharded
        from oracle import oracle
        o = oracle.load_best()
        n_total = (1 << 22) + 4321
        lo, hi = rank * n_total // world, (rank + 1) * n_total // world
        dev = lambda a: torch.from_numpy(np.ascontiguousarray(a)).cuda()  # noqa: E731
        x = dg.reduce_input(n_total)
        assert sharded.sharded_reduce(dev(x[lo:hi]), np.int64(3)) == o.reduce(x, np.int64(3))
        s = dg.scan_input_i32(n_total)
        assert np.array_equal(sharded.sharded_scan(dev(s[lo:hi])).cpu().numpy(), o.inclusive_scan(s)[lo:hi])
        assert np.array_equal(sharded.sharded_scan(dev(s[lo:hi]), exclusive=True, init=9).cpu().numpy(), o.exclusive_scan(s, 9)[lo:hi])
        # unsigned min/max with the top bit set and an empty shard (the all-reduce of the collective library would compare them as signed)
        u = (dg.sort_keys_u32(n_total) | np.uint32(0x80000000)).astype(np.uint32)
        part = u[lo:hi] if rank != world - 1 else u[:0]
        ref_part = np.concatenate([u[r * n_total // world:(r + 1) * n_total // world] for r in range(world - 1)])
        assert sharded.sharded_reduce(dev(part), np.uint32(0xFFFFFFFF), "min") == ref_part.min()
        assert sharded.sharded_reduce(dev(part), np.uint32(0), "max") == ref_part.max()
        skew = dg.sort_keys_u32(n_total).copy()
        skew[: (7 * n_total) // 8] = 123456789           # 7/8 of the keys equal: one rank's receive buffer would overflow, sampled splitters take over
        for case, keys in (("uniform", dg.sort_keys_u32(n_total)), ("ties", (dg.sort_keys_u32(n_total) >> np.uint32(22)).astype(np.uint32)),
                           ("u64", dg.sort_keys_u64_40bit(n_total)), ("skew", skew),
                           ("f32", dg.sort_keys_u32(n_total).view(np.int32).astype(np.float32))):
            vals = np.arange(n_total, dtype=np.uint32)
            # "histogram": splitters from a digit histogram, one kernel per GPU stores every pair into its owner's receive buffer, local sort;
            # "scatter": the same with sampled splitters;
            # "peer": merges read the pieces straight out of the other GPUs' memory (CUDA IPC + NVLink);
            # "collective": NCCL all-to-all first.  All must give the single-GPU result.
            for mode in ("histogram", "scatter", "peer", "collective"):
                for repeat in range(3):                      # later calls alternate receive buffers and reuse cached IPC mappings
                    k, v = sharded.sharded_sort_by_key(dev(keys[lo:hi]), dev(vals[lo:hi]), exchange=mode)
                np.save(os.path.join(out_dir, f"{case}_k{rank}.npy"), k.cpu().numpy())
                np.save(os.path.join(out_dir, f"{case}_v{rank}.npy"), v.cpu().numpy())
                dist.barrier()
                if rank == 0:
                    kk = np.concatenate([np.load(os.path.join(out_dir, f"{case}_k{r}.npy")) for r in range(world)])
                    vv = np.concatenate([np.load(os.path.join(out_dir, f"{case}_v{r}.npy")) for r in range(world)])
                    wk, wv = o.sort_by_key(keys, vals)
                    assert np.array_equal(kk, wk) and np.array_equal(vv, wv), (case, mode)
                dist.barrier()
    finally:
        dist.destroy_process_group()


def test_sharded_algorithms_over_nccl(tb, tmp_path):
    import torch
    import torch.multiprocessing as mp
    world = min(torch.cuda.device_count(), 4)
    if world < 2:
        pytest.skip("needs at least two GPUs")
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    mp.spawn(_worker, args=(world, port, str(tmp_path)), nprocs=world, join=True)
