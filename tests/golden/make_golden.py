"""Generates tests/golden/golden_v1.npz: inputs and the outputs of the REFERENCE Thrust (1.14.0,
OpenMP device system, via oracle/_ref/liboracle_ref.so) for every algorithm on the hot path.

    python tests/golden/make_golden.py        (needs the reference checkout to build oracle/_ref)

The file travels with the repository, so the parity tests can check the CUDA kernels and the C
restatement against reference outputs on machines where the reference itself is absent.  Inputs
come from thrust_b200.datagen with the seeds of the benchmark configurations, at sizes that cross
every tile boundary of the kernels but keep the file small.
"""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
from oracle import oracle  # noqa: E402
from thrust_b200 import datagen as dg  # noqa: E402

SIZES = (1, 777, 12345)


def main():
    ref = oracle.load_ref()
    if ref is None:
        raise SystemExit("the reference oracle could not be built")
    assert ref.kind == "reference"
    g = {}
    for n in SIZES:
        x = dg.reduce_input(n)
        g[f"reduce_in_{n}"] = x
        g[f"reduce_out_{n}"] = np.asarray(ref.reduce(x, np.int64(0)))
        s = dg.scan_input_i32(n)
        g[f"scan_in_{n}"] = s
        g[f"scan_incl_{n}"] = ref.inclusive_scan(s)
        g[f"scan_excl_{n}"] = ref.exclusive_scan(s, 0)
        k = dg.sort_keys_u32(n)
        v = np.arange(n, dtype=np.uint32)
        sk, sv = ref.sort_by_key(k, v)
        g[f"sort_keys_in_{n}"] = k
        g[f"sort_keys_out_{n}"] = sk
        g[f"sort_vals_out_{n}"] = sv
        k64 = dg.sort_keys_u64_40bit(n) & np.uint64(0xFFFF)   # few distinct keys: exercises stability
        sk, sv = ref.sort_by_key(k64, v)
        g[f"sort64_keys_in_{n}"] = k64
        g[f"sort64_keys_out_{n}"] = sk
        g[f"sort64_vals_out_{n}"] = sv
        c = dg.compaction_input(n)
        g[f"compact_in_{n}"] = c
        g[f"copy_if_out_{n}"] = ref.copy_if(c, "mod_eq", 2, 0)
        sp, cnt = ref.stable_partition(c, "mod_eq", 2, 0)
        g[f"stable_partition_out_{n}"] = sp
        g[f"partition_count_{n}"] = np.asarray(cnt)
        up, ucnt = ref.partition(c, "mod_eq", 2, 0)
        g[f"partition_out_{n}"] = up
        rk = dg.run_keys(n)
        rv = dg.scan_input_i32(n, 7)
        g[f"run_keys_{n}"] = rk
        g[f"run_vals_{n}"] = rv
        g[f"unique_out_{n}"] = ref.unique_copy(rk)
        ko, vo = ref.reduce_by_key(rk, rv)
        g[f"rbk_keys_out_{n}"] = ko
        g[f"rbk_vals_out_{n}"] = vo
        a = dg.merge_keys_u64(n, 4) >> np.uint64(36)         # 12-bit keys: many ties between A and B
        b = dg.merge_keys_u64(n // 2 + 1, 5) >> np.uint64(36)
        va = np.arange(a.size, dtype=np.uint32)
        vb = np.arange(b.size, dtype=np.uint32) + np.uint32(1 << 27)
        mk, mv = ref.merge_by_key(a, b, va, vb)
        g[f"merge_a_{n}"] = a
        g[f"merge_b_{n}"] = b
        g[f"merge_keys_out_{n}"] = mk
        g[f"merge_vals_out_{n}"] = mv
        zk, zv = dg.zip_sort_input(n)
        zk = zk >> np.uint32(22)                              # 10-bit keys: stability visible
        sk, sv = ref.stable_sort_zip_by_first(zk, zv.view(np.uint32))
        g[f"zip_keys_in_{n}"] = zk
        g[f"zip_vals_in_{n}"] = zv
        g[f"zip_keys_out_{n}"] = sk
        g[f"zip_vals_out_{n}"] = sv
    out = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden_v1.npz")
    np.savez_compressed(out, **g)
    print("wrote", out, os.path.getsize(out), "bytes")


if __name__ == "__main__":
    main()
