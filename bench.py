#!/usr/bin/env python
"""Benchmark of the hot path: thrust::sort_by_key of 2^28 (uint32 key, uint32 value) pairs.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--no-extras]
    python bench.py --case ALGO LOG2N [REPS]        (one algorithm, a few calls, for profilers)

A step is one stable sort_by_key of the whole workload (uniform random 32-bit keys from seed 2,
value = original index).  Rank 0 prints ONE JSON line:

  value        Gkeys/s with the inputs resident in HBM, CUDA-event time of the C-ABI call only
               (the pristine input is restored by a device copy between steps, outside the events;
               that 2 GiB copy also flushes L2);
  e2e          the same metric through the host API with HOST buffers (thrust_b200.sort_by_key_host):
               pinned host -> device copy of keys and values, sort, device -> pinned host copy of
               both, all inside the events; the call sorts (key, position) pairs while the values
               are still coming up and sends the sorted keys down meanwhile, so the two directions
               of the host link overlap (N > 1: every rank copies its shard up, the sharded sort,
               every rank copies its slice of the result down);
  roofline     the dominant kernel (one onesweep digit pass), timed live with CUDA events through
               the library's per-kernel timing switch: algorithmic bytes = 2 * (4 + 4) * n per pass;
  cpu_baseline the reference Thrust's OpenMP sort_by_key (oracle/_ref) on a bounded sample, N=1 only;
  others       the remaining hot-path algorithms at their benchmark sizes (N=1 only).

With N > 1 (torchrun, one rank per GPU) the same 2^28 pairs are split across the ranks and sorted
by thrust_b200.sharded.sharded_sort_by_key: splitters from an all-gathered digit histogram, one scatter
kernel per GPU that stores each pair into its owner's receive buffer over NVLink (CUDA IPC), then a
stable per-GPU radix sort ("scaling": "strong"); the sharded result is verified after the timed steps.  `--impl reference` times the
reference's own CPU implementation (OpenMP backend) on the host cores instead.
"""
import argparse
import ctypes as C
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

N_KEYS = 1 << 28
METRIC = "sort_by_key_gkeys_per_s"
UNIT = "Gkeys/s"
WORKLOAD = "thrust::sort_by_key, 2^28 uint32 keys (uniform random 32 bits, seed 2) + uint32 values (original index)"
CPU_SAMPLE = 1 << 26
FALLBACK_HBM_GBS = 6650.0
# DRAM bytes per onesweep launch per key, from the ncu capture summarised in
# profiles/onesweep_u32_u32_2p25.md (dram read + write of one pass at 2^25 pairs, divided by 2^25)
ONESWEEP_TRAFFIC_BYTES_PER_KEY = 14.47


def hbm_peak():
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except Exception:
        return FALLBACK_HBM_GBS, "fallback"


class ClockSampler:
    """Samples SM clock and throttle reasons of one GPU with nvidia-smi while a region runs."""
    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index = index
        self.proc = None
        self.lines = []

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.index), "--query-gpu=" + self.FIELDS,
                                          "--format=csv,noheader,nounits", "-lms", "100"], stdout=subprocess.PIPE, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        self.proc.wait()
        mhz, mx, reasons = [], None, set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for ln in self.lines:
            p = [x.strip() for x in ln.split(",")]
            if len(p) < 6:
                continue
            try:
                mhz.append(float(p[0]))
                mx = float(p[1])
            except ValueError:
                continue
            for nm, val in zip(names, p[2:6]):
                if val.lower().startswith("active"):
                    reasons.add(nm)
        return {"sm_mhz": float(np.median(mhz)) if mhz else None, "sm_max_mhz": mx, "reasons": sorted(reasons), "samples": len(mhz)}


def run_reference(args):
    """The reference arm: Thrust 1.14.0 OpenMP backend on the host cores (oracle/_ref), or the C
    restatement if that library was never built.  Each step sorts a bounded sample."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    from oracle import oracle
    from thrust_b200 import datagen as dg
    o = oracle.load_best()
    n = CPU_SAMPLE
    keys = dg.sort_keys_u32(n)
    vals = np.arange(n, dtype=np.uint32)
    for _ in range(min(args.warmup, 1)):
        o.sort_by_key(keys, vals)
    times = []
    for _ in range(args.steps):
        k, v = keys.copy(), vals.copy()
        t0 = time.perf_counter()
        o.lib.ora_sort_by_key(C.c_void_p(k.ctypes.data), C.c_void_p(v.ctypes.data), C.c_size_t(n), 5, 4, 0)
        times.append(time.perf_counter() - t0)
    ms = 1e3 * float(np.mean(times))
    value = n / ms / 1e6
    sample = "2^26 of the 2^28 pairs per step (same generator and seed)"
    print(json.dumps({
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
        "dtype": "u32", "data": "synthetic", "config": {"workload": WORKLOAD, "sample": sample},
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": o.threads, "kind": o.kind, "sample": sample},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }))


def _mark(torch):
    e = torch.cuda.Event(enable_timing=True)
    e.record()
    return e


def _events(torch):
    return torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)


def time_calls(torch, fn, reps, setup=None):
    """CUDA-event time (ms) of each of `reps` calls of fn on the current stream."""
    out = []
    for _ in range(reps):
        if setup:
            setup()
        e0, e1 = _events(torch)
        e0.record()
        fn()
        e1.record()
        e1.synchronize()
        out.append(e0.elapsed_time(e1))
    return out


def read_kernel_times(lib, kernel_id):
    cap = 256
    ids = (C.c_int * cap)()
    ms = (C.c_float * cap)()
    cnt = C.c_int(0)
    rc = lib.tb200_kernel_timing_read(cap, ids, ms, C.byref(cnt))
    assert rc == 0, rc
    return [ms[i] for i in range(cnt.value) if ids[i] == kernel_id]


def bench_others(torch, tb, lib, peak):
    """The other hot-path algorithms at their benchmark sizes; median of 10 C-ABI calls each.  Each
    line also carries the reference Thrust's OpenMP backend on the host cores (oracle/_ref), timed
    once after a warm-up on a bounded sample of the same workload."""
    from thrust_b200 import datagen as dg
    from oracle import oracle
    ora = oracle.load_best()
    cpu_n = 1 << 25

    def cpu_time(fn, units):
        fn()
        t0 = time.perf_counter()
        fn()
        dt = time.perf_counter() - t0
        return {"value": units / dt / 1e9, "cores": ora.threads, "kind": ora.kind, "sample_units": units, "seconds": dt}
    st = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    p = lambda t: None if t is None else C.c_void_p(t.data_ptr())  # noqa: E731
    dev = lambda a: torch.from_numpy(a).cuda()  # noqa: E731
    res = []

    def ws_for(fn, *a):
        need = C.c_size_t(0)
        assert getattr(lib, fn)(*a, None, C.byref(need), None) == 0
        return torch.empty(max(need.value, 256), dtype=torch.uint8, device="cuda"), need

    def record(name, n_units, bytes_per_unit, fn, setup=None, reps=10, unit="Gelem/s", cpu=None):
        for _ in range(3):
            if setup:
                setup()
            fn()
        ts = time_calls(torch, fn, reps, setup)
        ms = float(np.median(ts))
        gbs = n_units * bytes_per_unit / ms / 1e6
        res.append({"name": name, "value": n_units / ms / 1e6, "unit": unit, "ms": ms, "algorithmic_bytes_per_unit": bytes_per_unit,
                    "achieved_gbs": gbs, "frac_of_hbm_peak": gbs / peak, "cpu_reference": cpu})

    n = 1 << 28
    x = dev(dg.reduce_input(n))
    out8 = torch.empty(1, dtype=torch.int64, device="cuda")
    init = np.zeros((), np.int64)
    ws, need = ws_for("tb200_reduce", None, n, 4, 6, 0, None, None)
    hx = dg.reduce_input(cpu_n)
    record("reduce int32->int64 2^28", n, 4,
           lambda: lib.tb200_reduce(p(x), n, 4, 6, 0, C.c_void_p(init.ctypes.data), p(out8), p(ws), C.byref(need), st),
           cpu=cpu_time(lambda: ora.reduce(hx, np.int64(0)), cpu_n))
    del x
    s = dev(dg.scan_input_i32(n))
    o = torch.empty_like(s)
    ws, need = ws_for("tb200_inclusive_scan", None, None, n, 4, 0, None)
    hs = dg.scan_input_i32(cpu_n)
    hso = np.empty_like(hs)
    record("inclusive_scan int32 2^28", n, 8, lambda: lib.tb200_inclusive_scan(p(s), p(o), n, 4, 0, None, p(ws), C.byref(need), st),
           cpu=cpu_time(lambda: ora.inclusive_scan(hs, out=hso), cpu_n))
    zero = np.zeros((), np.int32)
    record("exclusive_scan int32 2^28", n, 8,
           lambda: lib.tb200_exclusive_scan(p(s), p(o), n, 4, 0, C.c_void_p(zero.ctypes.data), p(ws), C.byref(need), st))
    f = dev(dg.scan_input_f32(n))
    of = torch.empty_like(f)
    record("inclusive_scan fp32 2^28", n, 8, lambda: lib.tb200_inclusive_scan(p(f), p(of), n, 8, 0, None, p(ws), C.byref(need), st))
    del s, o, f, of
    c = dev(dg.compaction_input(n))
    o1, o2 = torch.empty_like(c), torch.empty_like(c)
    cnt = torch.zeros(1, dtype=torch.int64, device="cuda")
    ws, need = ws_for("tb200_partition", None, n, 4, 0, 2, 0, None)
    hc = dg.compaction_input(cpu_n)
    record("copy_if x%2==0 int32 2^28", n, 6, lambda: lib.tb200_copy_if(p(c), None, p(o1), n, 4, 0, 0, 2, 0, p(cnt), p(ws), C.byref(need), st),
           cpu=cpu_time(lambda: ora.copy_if(hc, "mod_eq", 2, 0), cpu_n))
    record("partition_copy x%2==0 int32 2^28", n, 8,
           lambda: lib.tb200_partition_copy(p(c), None, p(o1), p(o2), n, 4, 0, 0, 2, 0, p(cnt), p(ws), C.byref(need), st))
    record("partition (in place) x%2==0 int32 2^28", n, 8, lambda: lib.tb200_partition(p(o1), n, 4, 0, 2, 0, p(cnt), p(ws), C.byref(need), st),
           setup=lambda: o1.copy_(c), cpu=cpu_time(lambda: ora.stable_partition(hc, "mod_eq", 2, 0), cpu_n))
    del c
    keys = dev(dg.run_keys(n))
    hk = dg.run_keys(cpu_n)
    hv = dg.run_values_f32(cpu_n)
    record("unique_copy int32 runs(mean 4) 2^28", n, 5, lambda: lib.tb200_unique_copy(p(keys), p(o1), n, 4, p(cnt), p(ws), C.byref(need), st),
           cpu=cpu_time(lambda: ora.unique_copy(hk), cpu_n))
    vals = dev(dg.run_values_f32(n))
    vo = o2.view(torch.float32)
    ws2, need2 = ws_for("tb200_reduce_by_key", None, None, None, None, n, 4, 8, 0, None)
    record("reduce_by_key int32/fp32 runs(mean 4) 2^28", n, 10,
           lambda: lib.tb200_reduce_by_key(p(keys), p(vals), p(o1), p(vo), n, 4, 8, 0, p(cnt), p(ws2), C.byref(need2), st),
           cpu=cpu_time(lambda: ora.reduce_by_key(hk, hv), cpu_n))
    # the "next" components built so far: scan_by_key, unique_by_key, minmax_element
    ws3, need3 = ws_for("tb200_scan_by_key", None, None, None, n, 4, 8, 0, 0, None)
    record("inclusive_scan_by_key int32/fp32 runs(mean 4) 2^28", n, 12,
           lambda: lib.tb200_scan_by_key(p(keys), p(vals), p(vo), n, 4, 8, 0, 0, None, p(ws3), C.byref(need3), st),
           cpu=cpu_time(lambda: ora.scan_by_key(hk, hv), cpu_n))
    del ws3
    ko4 = torch.empty_like(keys)
    ws4, need4 = ws_for("tb200_unique_by_key_copy", None, None, None, None, n, 4, 4, None)
    record("unique_by_key_copy int32/4-byte runs(mean 4) 2^28", n, 10,
           lambda: lib.tb200_unique_by_key_copy(p(keys), p(vals), p(ko4), p(vo), n, 4, 4, p(cnt), p(ws4), C.byref(need4), st),
           cpu=cpu_time(lambda: ora.unique_by_key_copy(hk, hv), cpu_n))
    del ko4, ws4
    idx2 = torch.zeros(2, dtype=torch.int64, device="cuda")
    ws5, need5 = ws_for("tb200_minmax_element", None, n, 4, None)
    record("minmax_element int32 2^28", n, 4, lambda: lib.tb200_minmax_element(p(keys), n, 4, p(idx2), p(ws5), C.byref(need5), st),
           cpu=cpu_time(lambda: ora.minmax_element(hk), cpu_n))
    del keys, vals, o1, o2, vo, ws5
    na = 1 << 27
    hma, hmb = dg.merge_keys_u64(cpu_n // 2, 4), dg.merge_keys_u64(cpu_n // 2, 5)
    hmva = np.arange(cpu_n // 2, dtype=np.uint32)
    hmvb = hmva + np.uint32(cpu_n // 2)
    ka, kb = dev(dg.merge_keys_u64(na, 4)), dev(dg.merge_keys_u64(na, 5))
    va = torch.arange(na, dtype=torch.int32, device="cuda")
    vb = va + na
    ko = torch.empty(2 * na, dtype=torch.uint64, device="cuda")
    vo = torch.empty(2 * na, dtype=torch.int32, device="cuda")
    ws, need = ws_for("tb200_merge_by_key", None, None, na, None, None, na, None, None, 7, 4, 0)
    record("merge_by_key 2 x 2^27 (u64, u32)", 2 * na, 24,
           lambda: lib.tb200_merge_by_key(p(ka), p(va), na, p(kb), p(vb), na, p(ko), p(vo), 7, 4, 0, p(ws), C.byref(need), st),
           cpu=cpu_time(lambda: ora.merge_by_key(hma, hmb, hmva, hmvb), cpu_n))
    # the set operations on the same two sorted ranges (keys only): 8 B in and at most 8 B out per input item
    cnt = torch.zeros(1, dtype=torch.int64, device="cuda")
    ws, need = ws_for("tb200_set_operation", 0, None, na, None, na, None, None, None, None, 7, 0, 0, None)
    for code, nm in ((0, "set_union"), (1, "set_intersection")):
        record("%s 2 x 2^27 u64" % nm, 2 * na, 16 if code == 0 else 8,
               lambda c=code: lib.tb200_set_operation(c, p(ka), na, p(kb), na, None, None, p(ko), None, 7, 0, 0, p(cnt), p(ws), C.byref(need), st))
    del ka, kb, va, vb, ko, vo
    n64 = 1 << 27
    k0 = dev(dg.sort_keys_u64_40bit(n64))
    v0 = torch.arange(n64, dtype=torch.int32, device="cuda")
    k, v, kalt, valt = torch.empty_like(k0), torch.empty_like(v0), torch.empty_like(k0), torch.empty_like(v0)
    ws, need = ws_for("tb200_sort_by_key", None, None, None, None, n64, 7, 4, 0, 0, 64)

    def restore():
        k.copy_(k0)
        v.copy_(v0)
    record("sort_by_key 2^27 u64 (40 random bits) + u32", n64, 128,
           lambda: lib.tb200_sort_by_key(p(k), p(kalt), p(v), p(valt), n64, 7, 4, 0, 0, 64, p(ws), C.byref(need), st), setup=restore, reps=5,
           unit="Gkeys/s")
    del k0, v0, k, v, kalt, valt
    nz = 1 << 26
    zk, zv = dg.zip_sort_input(nz)
    k0, v0 = dev(zk), dev(zv)
    k, v, kalt, valt = torch.empty_like(k0), torch.empty_like(v0), torch.empty_like(k0), torch.empty_like(v0)

    def restore2():
        k.copy_(k0)
        v.copy_(v0)
    ws, need = ws_for("tb200_merge_sort_by_key", None, None, None, None, nz, 5, 4, 0)
    passes = 1 + int(np.ceil(np.log2(nz / 4096)))
    record("stable_sort zip(u32,f32) by key 2^26, merge-sort route", nz, 16 * passes,
           lambda: lib.tb200_merge_sort_by_key(p(k), p(kalt), p(v), p(valt), nz, 5, 4, 0, p(ws), C.byref(need), st), setup=restore2, reps=5,
           cpu=cpu_time(lambda: ora.stable_sort_zip_by_first(zk[:cpu_n], zv[:cpu_n].view(np.uint32)), cpu_n))
    ws, need = ws_for("tb200_sort_by_key", None, None, None, None, nz, 5, 4, 0, 0, 32)
    record("stable_sort zip(u32,f32) by key 2^26, radix route", nz, 68,
           lambda: lib.tb200_sort_by_key(p(k), p(kalt), p(v), p(valt), nz, 5, 4, 0, 0, 32, p(ws), C.byref(need), st), setup=restore2, reps=5)
    return res


def bench_sharded(torch, dist, sharded, dg, world, rank, peak, args):
    """The other two sharded paths at N > 1, on the same terms as the sort: the 2^28-element
    workloads of the reduce and scan configurations split across the ranks ("strong"), CUDA events
    around the public call, max over ranks, results checked against values computed on the host.
    reduce: per-GPU single-pass reduce, one all-gather of G accumulators, fold on the host (4 B/elem).
    scan: per-GPU reduce, all-gather of G totals on the stream, carry folded on the device and read
    by the scan kernels from device memory -- no host round trip; 12 B/elem by construction (the
    shard is read twice), reported against the 8 B/elem of the single-GPU algorithm."""
    n = 1 << 28
    lo, hi = rank * n // world, (rank + 1) * n // world
    res = []

    def timed(fn, reps=10):
        for _ in range(3):
            fn()
        dist.barrier()
        torch.cuda.synchronize()
        ts = time_calls(torch, fn, reps)
        t = torch.tensor([float(np.median(ts))], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    hx = dg.reduce_input(hi - lo, start=lo)
    x = torch.from_numpy(hx).cuda()
    part = torch.tensor([int(hx.sum(dtype=np.int64))], device="cuda")
    dist.all_reduce(part)
    got = sharded.sharded_reduce(x, np.int64(0))
    ok = int(got) == int(part.item())
    ms = timed(lambda: sharded.sharded_reduce(x, np.int64(0)))
    res.append({"name": "sharded reduce int32->int64 2^28", "ms": ms, "achieved_gbs": 4.0 * n / ms / 1e6, "frac_of_hbm_peak": 4.0 * n / ms / 1e6 / (peak * world),
                "algorithmic_bytes_per_unit": 4, "verified": bool(ok)})
    del x
    hs = dg.scan_input_i32(hi - lo, start=lo)
    s = torch.from_numpy(hs).cuda()
    sums = torch.zeros(world, dtype=torch.int64, device="cuda")
    sums[rank] = int(hs.sum(dtype=np.int64))
    dist.all_reduce(sums)
    before = int(sums[:rank].sum().item())
    out = sharded.sharded_scan(s)
    m32 = 1 << 32                                             # int32 sums wrap: compare modulo 2^32
    ok = int(out[0]) % m32 == (before + int(hs[0])) % m32 and torch.equal(out[1:] - out[:-1], s[1:]) and \
        int(out[-1]) % m32 == (before + int(hs.sum(dtype=np.int64))) % m32
    flag = torch.tensor([1 if ok else 0], device="cuda")
    dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    ms = timed(lambda: sharded.sharded_scan(s))
    res.append({"name": "sharded inclusive_scan int32 2^28", "ms": ms, "achieved_gbs": 8.0 * n / ms / 1e6, "frac_of_hbm_peak": 8.0 * n / ms / 1e6 / (peak * world),
                "algorithmic_bytes_per_unit": 8, "bytes_moved_per_unit": 12, "verified": bool(flag.item())})
    return res


def run_case(args):
    """`--case ALGO LOG2N [REPS]`: runs one hot-path algorithm a few times on its synthetic benchmark
    input and exits -- the command that the profiler captures under profiles/ wrap, on a case small
    enough for the profiler (a few hundred MB) yet larger than the 126 MB L2.
    ALGO: reduce | scan | sort | sort64 | copy_if | partition_copy | unique | reduce_by_key | merge |
    merge_sort | scan_by_key | unique_by_key | minmax."""
    import torch
    import thrust_b200 as tb
    from thrust_b200 import datagen as dg
    algo = args.case[0]
    n = 1 << int(args.case[1])
    reps = int(args.case[2]) if len(args.case) > 2 else 2
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
    elif algo in ("reduce_by_key", "scan_by_key", "unique_by_key"):
        k, v = dev(dg.run_keys(n)), dev(dg.run_values_f32(n))
        run = {"reduce_by_key": lambda: tb.reduce_by_key(k, v), "scan_by_key": lambda: tb.inclusive_scan_by_key(k, v),
               "unique_by_key": lambda: tb.unique_by_key_copy(k, v)}[algo]
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


def run_ours(args):
    import torch
    import torch.distributed as dist
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        if world == 1 and args.gpus > 1:
            raise SystemExit("launch with torch.distributed.run --nproc-per-node %d for --gpus %d" % (args.gpus, args.gpus))
    torch.cuda.set_device(local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    import thrust_b200 as tb
    from thrust_b200 import datagen as dg, sharded
    lib = tb._lib.load()
    peak, peak_kind = hbm_peak()

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # one process per GPU: keep each rank's pinned buffers and copies on its GPU's socket (N = 1 keeps
    # every host thread for the CPU baseline leg)
    numa_node = sharded.bind_to_gpu_numa_node(local_rank) if world > 1 else None
    lo, hi = rank * N_KEYS // world, (rank + 1) * N_KEYS // world
    n_local = hi - lo
    h_keys = torch.from_numpy(dg.sort_keys_u32(n_local, start=lo)).pin_memory()
    h_vals = torch.from_numpy(np.arange(lo, hi, dtype=np.uint32)).pin_memory()
    k0, v0 = h_keys.cuda(), h_vals.cuda()
    st = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    p = lambda t: C.c_void_p(t.data_ptr())  # noqa: E731
    launches_per_step = 0

    if world == 1:
        k, v = torch.empty_like(k0), torch.empty_like(v0)
        kalt, valt = torch.empty_like(k0), torch.empty_like(v0)
        need = C.c_size_t(0)
        assert lib.tb200_sort_by_key(None, None, None, None, n_local, 5, 4, 0, 0, 32, None, C.byref(need), None) == 0
        ws = torch.empty(need.value, dtype=torch.uint8, device="cuda")

        def restore():
            k.copy_(k0)
            v.copy_(v0)

        def step():
            rc = lib.tb200_sort_by_key(p(k), p(kalt), p(v), p(valt), n_local, 5, 4, 0, 0, 32, p(ws), C.byref(need), st)
            assert rc == 0, rc
        launches_per_step = 2 + 4 + 1     # histogram, bucket-base scan, four onesweep passes, copy-back check
    else:
        out = {}
        k, v = torch.empty_like(k0), torch.empty_like(v0)

        def restore():
            k.copy_(k0)
            v.copy_(v0)

        def step():
            # like thrust::sort_by_key, the sharded sort may consume its input
            out["k"], out["v"] = sharded.sharded_sort_by_key(k, v, consume_input=True)
        # per rank: digit histogram (1) + plan (1) + scatter (1) + local sort (histogram, bases, four passes, copy-back check: 7)
        launches_per_step = 1 + 1 + 1 + 7

    # the clock sampler runs from before the warm-up to after the timed steps, so that even a timed
    # region of a few tens of milliseconds is covered by samples taken under the same load
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
        time.sleep(0.3)
    for _ in range(max(args.warmup, 3)):
        restore()
        step()
    t_load = time.perf_counter()
    while time.perf_counter() - t_load < 1.0:      # keep the GPU under this load for a second of samples
        restore()
        step()
    barrier()
    t_wall = time.perf_counter()
    times = time_calls(torch, step, args.steps, restore)
    barrier()
    t_wall = time.perf_counter() - t_wall
    clocks = sampler.stop() if rank == 0 else None
    ms = float(np.mean(times))
    if world > 1:
        t = torch.tensor([ms], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    value = N_KEYS / ms / 1e6

    # correctness guard on the last step's output (cheap, outside every timed region)
    if world == 1:
        status = C.c_uint(9)
        assert lib.tb200_workspace_status(p(ws), st, C.byref(status)) == 0 and status.value == 0
        ki = k.view(torch.int32) ^ torch.tensor(-(1 << 31), dtype=torch.int32, device="cuda")
        assert bool((ki[1:] >= ki[:-1]).all()), "output is not sorted"
        del ki
    verified = None
    stages = None
    if world > 1:
        # the whole sharded result: genuine pairs, sorted and stable inside every shard, shards in
        # rank order, values a permutation of 0 .. n-1 (thrust_b200.sharded.check_sharded_sort)
        verified = sharded.check_sharded_sort(out["k"], out["v"], N_KEYS, dg.sort_keys_u32_at)
        # where a step's time goes: CUDA events at the stage boundaries of one more step
        marks = [("start", lambda: _mark(torch))]
        restore()
        marks.append(("begin", _mark(torch)))
        sharded.sharded_sort_by_key(k, v, consume_input=True, stage_marks=marks)
        torch.cuda.synchronize()
        evs = marks[1:]
        stages = {evs[i + 1][0] + "_ms": evs[i][1].elapsed_time(evs[i + 1][1]) for i in range(len(evs) - 1)}

    # ---- roofline of the dominant kernel: one onesweep digit pass, timed with the library's events
    lib.tb200_kernel_timing(1)
    pass_ms = []
    for _ in range(max(2, min(args.steps, 5))):
        restore()
        step()
        torch.cuda.synchronize()
        pass_ms += read_kernel_times(lib, 3)
    lib.tb200_kernel_timing(0)
    avg_pass = float(np.mean(pass_ms))
    algo_bytes = 16.0 * n_local
    achieved = algo_bytes / avg_pass / 1e6
    roofline = {"bound": "hbm", "kernel": "onesweep_kernel (one 8-bit digit pass over key/value pairs)", "achieved": achieved, "peak": peak,
                "unit": "GB/s", "frac": achieved / peak, "peak_kind": peak_kind, "algorithmic_bytes_per_launch": algo_bytes,
                "avg_launch_ms": avg_pass, "launches_timed": len(pass_ms), "traffic": ONESWEEP_TRAFFIC_BYTES_PER_KEY * n_local}

    # ---- end to end through the host API with host buffers
    h_out_k = torch.empty_like(h_keys).pin_memory()
    h_out_v = torch.empty_like(h_vals).pin_memory()
    if world == 1:
        def e2e_step():
            tb.sort_by_key_host(h_keys, h_vals, h_out_k, h_out_v)
        d2h = 8 * n_local
        e2e_api = ("thrust_b200.sort_by_key_host on pinned host tensors: keys up, (key, position) pairs sorted while the values follow on a second "
                   "stream, sorted keys down while the values arrive, values permuted by position and sent down")
        # the host-buffer call must give what the device call gave on the same data (k, v hold its result)
        e2e_step()
        if not (torch.equal(h_out_k.cuda(), k) and torch.equal(h_out_v.cuda(), v)):
            raise SystemExit("sort_by_key_host disagrees with sort_by_key")
    else:
        dk, dv = torch.empty_like(k0), torch.empty_like(v0)
        # this rank's slice of the result is about n_local long; leave room for splitter imbalance
        h_res_k = torch.empty(2 * n_local, dtype=h_keys.dtype).pin_memory()
        h_res_v = torch.empty(2 * n_local, dtype=h_vals.dtype).pin_memory()

        def e2e_step():
            dk.copy_(h_keys, non_blocking=True)
            dv.copy_(h_vals, non_blocking=True)
            rk, rv = sharded.sharded_sort_by_key(dk, dv, consume_input=True)
            h_res_k[:rk.numel()].copy_(rk, non_blocking=True)
            h_res_v[:rv.numel()].copy_(rv, non_blocking=True)
        d2h = 8 * n_local
        e2e_api = "thrust_b200.sharded.sharded_sort_by_key on shards filled from pinned host memory; every rank's slice of the result copied back to pinned host memory"
    e2e_step()
    barrier()
    e2e_times = time_calls(torch, e2e_step, max(1, min(args.steps, 3)))
    barrier()
    e2e_ms = float(np.mean(e2e_times))
    if world > 1:
        t = torch.tensor([e2e_ms], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e_ms = float(t.item())
    e2e = {"value": N_KEYS / e2e_ms / 1e6, "unit": UNIT, "ms_per_step": e2e_ms, "h2d_bytes_per_step": 8 * n_local, "d2h_bytes_per_step": d2h,
           "api": e2e_api}

    line = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "u32", "data": "synthetic",
        "config": {"workload": WORKLOAD, "n": N_KEYS, "per_gpu": n_local,
                   "l2": "2 GiB of input per step (> 126 MB L2); the pristine input is restored by a 2 GiB device copy between timed steps",
                   "host_numa_node_of_rank0": numa_node,
                   "parallelism": "1 GPU" if world == 1 else "%d GPUs: splitters from an all-gathered 12-bit digit histogram, one scatter kernel per GPU storing each pair into the owning GPU's receive buffer over NVLink (CUDA IPC), local radix sort of what arrived" % world},
        "roofline": roofline, "e2e": e2e, "gpu_launches": launches_per_step * args.steps, "clocks": clocks,
        "wall_s_timed_region": t_wall, "verified": verified, "stages_ms": stages,
        "sort_roofline": {"algorithmic_bytes_per_key": 68, "achieved_gbs": 68.0 * N_KEYS / ms / 1e6, "frac_of_hbm_peak": 68.0 * N_KEYS / ms / 1e6 / peak / world},
    }

    if world > 1:
        line["sharded_others"] = bench_sharded(torch, dist, sharded, dg, world, rank, peak, args)
    if world == 1:
        del k, v, kalt, valt, ws, k0, v0
        torch.cuda.empty_cache()
        # ---- CPU baseline on the host cores of this box: the reference Thrust (OpenMP) when built
        from oracle import oracle
        o = oracle.load_best()
        ck = dg.sort_keys_u32(CPU_SAMPLE)
        cv = np.arange(CPU_SAMPLE, dtype=np.uint32)
        cpu_t = []
        for _ in range(3):
            a, b = ck.copy(), cv.copy()
            t0 = time.perf_counter()
            o.lib.ora_sort_by_key(C.c_void_p(a.ctypes.data), C.c_void_p(b.ctypes.data), C.c_size_t(CPU_SAMPLE), 5, 4, 0)
            cpu_t.append(time.perf_counter() - t0)
        line["cpu_baseline"] = {"value": CPU_SAMPLE / (1e3 * float(np.median(cpu_t))) / 1e6, "unit": UNIT, "cores": o.threads,
                                "kind": o.kind, "sample": "2^26 of the 2^28 pairs, 3 repetitions, median"}
        if not args.no_extras:
            line["others"] = bench_others(torch, tb, lib, peak)
    if rank == 0:
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-extras", action="store_true")
    ap.add_argument("--case", nargs="+", metavar=("ALGO", "LOG2N"), help="run one algorithm a few times for a profiler and exit (see run_case)")
    args = ap.parse_args()
    if args.case:
        return run_case(args)
    if args.impl == "reference":
        # a launcher may have pinned OpenMP to one thread for its ranks; the reference arm runs on rank 0
        # alone and is meant to use every host core (read when the oracle library loads its OpenMP runtime)
        os.environ["OMP_NUM_THREADS"] = str(os.cpu_count() or 1)
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
