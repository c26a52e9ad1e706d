"""Runs one hot-path algorithm a few times on its synthetic benchmark input, for profilers.

    python -m thrust_b200.profile_case <algorithm> <log2 n> [repetitions]

algorithm: reduce | scan | sort | sort64 | copy_if | partition_copy | unique | reduce_by_key | merge |
merge_sort | scan_by_key | unique_by_key | minmax.  Intended for captures such as
    ncu --set full --clock-control none -k regex:<kernel> -s 1 -c 1 -o out python -m thrust_b200.profile_case scan 26
on a case small enough for the profiler (a few hundred MB) yet larger than the 126 MB L2.
"""
import sys

import numpy as np
import torch

import thrust_b200 as tb
from thrust_b200 import datagen as dg


def main():
    algo = sys.argv[1]
    n = 1 << int(sys.argv[2])
    reps = int(sys.argv[3]) if len(sys.argv) > 3 else 2
    dev = lambda a: torch.from_numpy(a).cuda()  # noqa: E731
    if algo == "reduce":
        x = dev(dg.reduce_input(n))
        run = lambda: tb.reduce(x, np.int64(0))  # noqa: E731
    elif algo == "scan":
        x = dev(dg.scan_input_i32(n))
        run = lambda: tb.inclusive_scan(x)  # noqa: E731
    elif algo in ("sort", "sort64"):
        k0 = dev(dg.sort_keys_u32(n) if algo == "sort" else dg.sort_keys_u64_40bit(n))
        v0 = torch.arange(n, dtype=torch.int32, device="cuda")
        run = lambda: tb.sort_by_key(k0.clone(), v0.clone())  # noqa: E731
    elif algo == "copy_if":
        x = dev(dg.compaction_input(n))
        run = lambda: tb.copy_if(x, "mod_eq", 2, 0)  # noqa: E731
    elif algo == "partition_copy":
        x = dev(dg.compaction_input(n))
        run = lambda: tb.partition_copy(x, "mod_eq", 2, 0)  # noqa: E731
    elif algo == "unique":
        x = dev(dg.run_keys(n))
        run = lambda: tb.unique_copy(x)  # noqa: E731
    elif algo == "reduce_by_key":
        k, v = dev(dg.run_keys(n)), dev(dg.run_values_f32(n))
        run = lambda: tb.reduce_by_key(k, v)  # noqa: E731
    elif algo == "scan_by_key":
        k, v = dev(dg.run_keys(n)), dev(dg.run_values_f32(n))
        run = lambda: tb.inclusive_scan_by_key(k, v)  # noqa: E731
    elif algo == "unique_by_key":
        k, v = dev(dg.run_keys(n)), dev(dg.run_values_f32(n))
        run = lambda: tb.unique_by_key_copy(k, v)  # noqa: E731
    elif algo == "minmax":
        x = dev(dg.reduce_input(n))
        run = lambda: tb.minmax_element(x)  # noqa: E731
    elif algo == "merge":
        a, b = dev(dg.merge_keys_u64(n, 4)), dev(dg.merge_keys_u64(n, 5))
        va = torch.arange(n, dtype=torch.int32, device="cuda")
        vb = va + n
        run = lambda: tb.merge_by_key(a, b, va, vb)  # noqa: E731
    elif algo == "merge_sort":
        zk, zv = dg.zip_sort_input(n)
        k0, v0 = dev(zk), dev(zv)
        run = lambda: tb.merge_sort_by_key(k0.clone(), v0.clone())  # noqa: E731
    else:
        raise SystemExit("unknown algorithm " + algo)
    for _ in range(reps):
        run()
    torch.cuda.synchronize()
    print("done", algo, n)


if __name__ == "__main__":
    main()
