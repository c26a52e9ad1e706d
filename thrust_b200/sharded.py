"""Multi-GPU forms of the three paths that shard: reduce, scan and sort_by_key.

One process per GPU (torch.distributed, NCCL over NVLink); each rank owns a contiguous slice of
the global sequence, rank order being sequence order.  The reference has no multi-GPU path at all;
the semantics here are "the result the single-GPU algorithm would give on the concatenation":

  reduce       per-GPU single-pass reduce, then an all-reduce of one accumulator per GPU;
  scan         per-GPU reduce -> all-gather of the G totals -> each GPU folds the totals of the
               ranks before it into a carry -> per-GPU look-back scan seeded with that carry
               (12 bytes of HBM traffic per 4-byte element instead of 8);
  sort_by_key  per-GPU radix sort -> regular samples -> G-1 global splitters -> lower bounds cut
               each sorted shard into G pieces -> all-to-all of keys and values over NVLink ->
               each GPU merges the G sorted pieces it received, in source-rank order, with the
               stable merge-path merge.  Equal keys all land on one GPU and keep (rank, index)
               order, so the global result is the stable sort of the concatenation.

The collectives move only what has to move: 8 bytes per GPU for reduce, 8*G for scan, the keys and
values themselves for sort.  The compute steps go through an `ops` object: DeviceOps (the C-ABI
kernels, the default and the only one shipped) or, in the CPU tests of this orchestration, a
stand-in with the same methods.
"""
import numpy as np
import torch
import torch.distributed as dist

from . import api

_NP_IDENTITY = {
    "plus": lambda dt: np.zeros((), dt),
    "min": lambda dt: np.array(np.inf if np.issubdtype(dt, np.floating) else np.iinfo(dt).max, dt),
    "max": lambda dt: np.array(-np.inf if np.issubdtype(dt, np.floating) else np.iinfo(dt).min, dt),
}
_NP_OP = {"plus": np.add, "min": np.minimum, "max": np.maximum}
_REDUCE_OP = {"plus": dist.ReduceOp.SUM, "min": dist.ReduceOp.MIN, "max": dist.ReduceOp.MAX}

# integer views NCCL and torch indexing are happy with (uint32/uint64 tensors support few torch ops)
_SIGNED_VIEW = {torch.uint32: torch.int32, torch.uint64: torch.int64, torch.uint16: torch.int16}


def _plumbing_view(t):
    return t.view(_SIGNED_VIEW[t.dtype]) if t.dtype in _SIGNED_VIEW else t


def bind_to_gpu_numa_node(device_index):
    """Host-side placement for one-process-per-GPU jobs: restricts this process to the CPUs of the
    NUMA node that the GPU's PCIe link hangs off, so that the pinned buffers it allocates afterwards
    (first touch) and its copies stay on that socket instead of crossing the inter-socket link.
    Reads sysfs only; returns the node, or None when the topology is not visible, the node has no
    CPU this process may use, or there is a single node (nothing is changed then)."""
    import os
    try:
        props = torch.cuda.get_device_properties(device_index)
        dev = "%04x:%02x:%02x.0" % (props.pci_domain_id, props.pci_bus_id, props.pci_device_id)
        with open("/sys/bus/pci/devices/%s/numa_node" % dev) as f:
            node = int(f.read().strip())
        nodes = [d for d in os.listdir("/sys/devices/system/node") if d.startswith("node") and d[4:].isdigit()]
        if node < 0 or len(nodes) < 2:
            return None
        with open("/sys/devices/system/node/node%d/cpulist" % node) as f:
            cpus = set()
            for part in f.read().strip().split(","):
                lo, _, hi = part.partition("-")
                cpus.update(range(int(lo), int(hi or lo) + 1))
        usable = cpus & os.sched_getaffinity(0)
        if not usable:
            return None
        os.sched_setaffinity(0, usable)
        return node
    except (OSError, ValueError, AttributeError, RuntimeError, AssertionError):
        return None


class DeviceOps:
    """The product path: every compute step is a C-ABI call on CUDA tensors."""

    def reduce(self, x, init, op):
        return api.reduce(x, init, op)

    def inclusive_scan(self, x, op, init):
        return api.inclusive_scan(x, op=op, init=init)

    def exclusive_scan(self, x, op, init):
        return api.exclusive_scan(x, init=init, op=op)

    carries_on_device = True

    def reduce_to_device(self, x, identity, op, acc_dtype=None):
        return api.reduce_to_device(x, identity, op, acc_dtype=acc_dtype)

    def sort_by_key(self, keys, vals, descending):
        # enqueued only: the sharded algorithms wait for the GPU where they need a value on the host
        if vals is None:
            api.sort(keys, descending, sync=False)
        else:
            api.sort_by_key(keys, vals, descending, sync=False)

    def merge_by_key(self, ka, kb, va, vb, descending):
        return api.merge_by_key(ka, kb, va, vb, descending, sync=False)

    supports_peer_reads = True

    def export_buffer(self, t):
        """64-byte IPC handle (as 8 int64) + byte offset of tensor t inside its allocation."""
        import ctypes as C
        lib = api._lib.load()
        handle = np.zeros(8, dtype=np.int64)
        off = C.c_size_t(0)
        api._check(lib.tb200_ipc_export(api._ptr(t), C.c_void_p(handle.ctypes.data), C.byref(off)), "tb200_ipc_export")
        return handle, int(off.value)

    def open_buffer(self, handle, offset):
        """Device pointer (int) in this process of a peer's exported buffer."""
        import ctypes as C
        lib = api._lib.load()
        h = np.ascontiguousarray(handle, dtype=np.int64)
        out = C.c_void_p(0)
        api._check(lib.tb200_ipc_open(C.c_void_p(h.ctypes.data), int(offset), C.byref(out)), "tb200_ipc_open")
        return int(out.value)

    def close_buffer(self, handle):
        """Unmaps a peer's buffer (every pointer open_buffer returned for this handle dies)."""
        import ctypes as C
        h = np.ascontiguousarray(handle, dtype=np.int64)
        api._check(api._lib.load().tb200_ipc_close(C.c_void_p(h.ctypes.data)), "tb200_ipc_close")

    def merge_by_key_raw(self, ka, na, kb, nb, va, vb, key_dtype, val_dtype, descending, device):
        """merge_by_key on raw device pointers (which may point into a peer GPU's memory)."""
        import ctypes as C
        lib = api._lib.load()
        ko = torch.empty(na + nb, dtype=key_dtype, device=device)
        vo = None if val_dtype is None else torch.empty(na + nb, dtype=val_dtype, device=device)
        vbytes = 0 if vo is None else vo.element_size()
        args = (C.c_void_p(ka), None if va is None else C.c_void_p(va), na, C.c_void_p(kb), None if vb is None else C.c_void_p(vb), nb,
                api._ptr(ko), api._ptr(vo), api.DTYPE_CODE[key_dtype], vbytes, int(descending))
        api._call_with_ws("merge", "tb200_merge_by_key", *args)
        return ko, vo

    def bucket_count(self, keys, splitters, buckets, descending):
        import ctypes as C
        lib = api._lib.load()
        counts = torch.zeros(buckets, dtype=torch.int64, device=keys.device)
        api._check(lib.tb200_bucket_count(api._ptr(keys), keys.numel(), api.DTYPE_CODE[keys.dtype], int(descending), api._ptr(splitters), buckets,
                                          api._ptr(counts), api._stream()), "tb200_bucket_count")
        return counts

    def bucket_scatter(self, keys, vals, splitters, dst_keys, dst_vals, dst_offsets, descending):
        """Stable scatter of this rank's pairs into the receive buffers (device pointers, possibly on peers)."""
        import ctypes as C
        m = len(dst_keys)
        kp = (C.c_void_p * m)(*dst_keys)
        vp = None if vals is None else (C.c_void_p * m)(*dst_vals)
        off = (C.c_ulonglong * m)(*[int(o) for o in dst_offsets])
        api._call_with_ws("scatter", "tb200_bucket_scatter", api._ptr(keys), api._ptr(vals), keys.numel(), api.DTYPE_CODE[keys.dtype],
                          0 if vals is None else vals.element_size(), int(descending), api._ptr(splitters), m, kp, vp, off)

    supports_histogram_exchange = True
    _exchange_state = {}

    def exchange_state(self, device, key_dtype, val_dtype):
        """Per (device, types) state of the histogram exchange that outlives a call: two sets of receive
        buffers used alternately (a result stays valid until the call after next, and a sender never
        writes into a buffer its owner may still be sorting), their IPC handles, the peers' opened
        pointers, and the small device arrays of the plan."""
        key = (str(device), key_dtype, val_dtype)
        st = self._exchange_state.get(key)
        if st is None:
            import ctypes as C
            lib = api._lib.load()
            words, plan_bytes, head = C.c_size_t(0), C.c_size_t(0), C.c_size_t(0)
            api._check(lib.tb200_exchange_sizes(api.DTYPE_CODE[key_dtype], C.byref(words), C.byref(plan_bytes), C.byref(head)), "tb200_exchange_sizes")
            st = {"sets": [None, None], "generation": [0, 0], "turn": 0, "known_tags": [None, None], "peer_ptrs": [None, None],
                  "peer_handles": [set(), set()],
                  "row_words": int(words.value), "plan_bytes": int(plan_bytes.value), "head_bytes": int(head.value),
                  "row": torch.empty(int(words.value), dtype=torch.int32, device=device),
                  "plan": torch.empty(int(plan_bytes.value), dtype=torch.uint8, device=device)}
            self._exchange_state[key] = st
        return st

    def exchange_receive_set(self, st, device, key_dtype, val_dtype, capacity):
        """The receive buffers of this call (alternating sets), (re)allocated when too small."""
        i = st["turn"]
        st["turn"] ^= 1
        have = st["sets"][i]
        if have is None or have[0].numel() < capacity:
            k = torch.empty(capacity, dtype=key_dtype, device=device)
            v = None if val_dtype is None else torch.empty(capacity, dtype=val_dtype, device=device)
            st["sets"][i] = (k, v, self.export_buffer(k), None if v is None else self.export_buffer(v))
            st["generation"][i] += 1
        return i, st["sets"][i]

    def exchange_hist(self, st, keys, descending, tag):
        import ctypes as C
        lib = api._lib.load()
        api._check(lib.tb200_exchange_hist(api._ptr(keys), keys.numel(), api.DTYPE_CODE[keys.dtype], int(descending), C.c_ulonglong(tag),
                                           api._ptr(st["row"]), api._stream()), "tb200_exchange_hist")
        return st["row"]

    def exchange_plan(self, st, rows, world, rank, key_dtype):
        lib = api._lib.load()
        api._check(lib.tb200_exchange_plan(api._ptr(rows), world, rank, api.DTYPE_CODE[key_dtype], api._ptr(st["plan"]), api._stream()),
                   "tb200_exchange_plan")
        return st["plan"]

    def exchange_scatter(self, keys, vals, plan, dst_keys, dst_vals, descending):
        import ctypes as C
        m = len(dst_keys)
        kp = (C.c_void_p * m)(*dst_keys)
        vp = None if vals is None else (C.c_void_p * m)(*dst_vals)
        api._call_with_ws("scatter", "tb200_exchange_scatter", api._ptr(keys), api._ptr(vals), keys.numel(), api.DTYPE_CODE[keys.dtype],
                          0 if vals is None else vals.element_size(), int(descending), api._ptr(plan), m, kp, vp)

    _recv_cache = {}

    def receive_buffers(self, device, key_dtype, val_dtype, capacity):
        """Receive buffers of the scatter exchange, kept across calls so that their IPC handles stay valid."""
        key = (str(device), key_dtype, val_dtype)
        have = self._recv_cache.get(key)
        if have is None or have[0].numel() < capacity:
            k = torch.empty(capacity, dtype=key_dtype, device=device)
            v = None if val_dtype is None else torch.empty(capacity, dtype=val_dtype, device=device)
            have = (k, v, self.export_buffer(k), None if v is None else self.export_buffer(v))
            self._recv_cache[key] = have
        return have

    def merge_runs_raw(self, runs, key_dtype, val_dtype, descending, device):
        """Stable merge of many runs [(keys_ptr, vals_ptr or None, count)] with ONE library call."""
        import ctypes as C
        lib = api._lib.load()
        m = len(runs)
        total = sum(r[2] for r in runs)
        ko = torch.empty(total, dtype=key_dtype, device=device)
        kt = torch.empty(total, dtype=key_dtype, device=device)
        vo = None if val_dtype is None else torch.empty(total, dtype=val_dtype, device=device)
        vt = None if val_dtype is None else torch.empty(total, dtype=val_dtype, device=device)
        kp = (C.c_void_p * m)(*[r[0] for r in runs])
        vp = None if val_dtype is None else (C.c_void_p * m)(*[r[1] for r in runs])
        cn = (C.c_size_t * m)(*[r[2] for r in runs])
        vbytes = 0 if vo is None else vo.element_size()
        api._call_with_ws("merge", "tb200_merge_runs", kp, vp, cn, m, api._ptr(ko), api._ptr(vo), api._ptr(kt), api._ptr(vt),
                          api.DTYPE_CODE[key_dtype], vbytes, int(descending))
        return ko, vo

    def lower_bound(self, sorted_keys, needles, descending):
        import ctypes as C
        lib = api._lib.load()
        out = torch.empty(needles.numel(), dtype=torch.int64, device=sorted_keys.device)
        rc = lib.tb200_lower_bound(api._ptr(sorted_keys), sorted_keys.numel(), api._ptr(needles), needles.numel(),
                                   api._ptr(out), api.DTYPE_CODE[sorted_keys.dtype], int(descending), api._stream())
        api._check(rc, "tb200_lower_bound")
        return out


def _world(group):
    return dist.get_world_size(group), dist.get_rank(group)


def _np_dtype(t):
    return np.dtype(api.NP_OF[t.dtype])


def sharded_reduce(x_local, init, op="plus", group=None, ops=None):
    """thrust::reduce over the concatenation of every rank's x_local.  `init` is a numpy scalar
    whose dtype is the accumulator type.  Every rank returns the same numpy scalar."""
    ops = ops or DeviceOps()
    init = np.asarray(init)
    acc = init.dtype
    world, _ = _world(group)
    # The G partials are gathered bit for bit and folded on the host in the accumulator type: an
    # all-reduce would compare unsigned partials as signed integers (the collective library has no
    # unsigned min/max), and one word per rank costs the same either way.
    if getattr(ops, "carries_on_device", False) and x_local.is_cuda and dist.get_backend(group) == "nccl":
        # the partial never leaves the device before the gather: one host wait in all
        mine = ops.reduce_to_device(x_local, _NP_IDENTITY[op](acc)[()], op, acc_dtype=api.TORCH_OF[np.dtype(acc)])
        gathered = torch.empty(world, dtype=mine.dtype, device=x_local.device)
        dist.all_gather_into_tensor(_plumbing_view(gathered), _plumbing_view(mine), group=group)
        total = init
        with np.errstate(over="ignore"):
            for g in gathered.cpu().numpy().view(acc):
                total = _NP_OP[op](total, g).astype(acc)[()]
        return total
    partial = ops.reduce(x_local, _NP_IDENTITY[op](acc)[()], op)
    mine = torch.from_numpy(np.asarray(partial, dtype=acc).reshape(1).copy()).to(x_local.device)
    gathered = [torch.empty_like(mine) for _ in range(world)]
    dist.all_gather([_plumbing_view(g) for g in gathered], _plumbing_view(mine), group=group)
    total = init
    with np.errstate(over="ignore"):
        for g in gathered:
            total = _NP_OP[op](total, g.cpu().numpy().view(acc)[0]).astype(acc)[()]
    return total


def sharded_scan(x_local, op="plus", exclusive=False, init=None, group=None, ops=None):
    """Inclusive or exclusive scan of the concatenation; returns this rank's slice of the result.
    Accumulates in x_local's dtype, like the single-GPU scan."""
    ops = ops or DeviceOps()
    world, rank = _world(group)
    dt = _np_dtype(x_local)
    if getattr(ops, "carries_on_device", False) and x_local.is_cuda and dist.get_backend(group) == "nccl":
        # Nothing visits the host: the local total stays on the device, the all-gather runs on the
        # stream, the totals of the ranks before this one are folded by the library's own reduce
        # (seeded with init), and the scan reads its initial value from device memory.
        ident = _NP_IDENTITY[op](dt)[()]
        mine = ops.reduce_to_device(x_local, ident, op)
        totals = torch.empty(world, dtype=x_local.dtype, device=x_local.device)
        dist.all_gather_into_tensor(_plumbing_view(totals), _plumbing_view(mine), group=group)
        seed = ident if init is None else np.asarray(init, dtype=dt)[()]
        if rank == 0 and init is None:
            carry = None if not exclusive else torch.from_numpy(np.zeros(1, dt)).to(x_local.device)
        else:
            carry = ops.reduce_to_device(totals[:rank], seed, op)
        if exclusive:
            return api.exclusive_scan(x_local, init=carry, op=op)
        return api.inclusive_scan(x_local, op=op, init=carry)
    total = ops.reduce(x_local, _NP_IDENTITY[op](dt)[()], op)
    mine = torch.from_numpy(np.asarray(total, dtype=dt).reshape(1).copy()).to(x_local.device)
    gathered = [torch.empty_like(mine) for _ in range(world)]
    dist.all_gather([_plumbing_view(g) for g in gathered], _plumbing_view(mine), group=group)
    totals = [g.cpu().numpy().astype(dt)[0] for g in gathered]
    # carry = init (+) totals of the ranks before this one, folded left to right in the element type
    carry = None if init is None else np.asarray(init, dtype=dt)[()]
    with np.errstate(over="ignore"):
        for r in range(rank):
            carry = totals[r] if carry is None else _NP_OP[op](carry, totals[r]).astype(dt)[()]
    if exclusive:
        if carry is None:
            carry = np.zeros((), dt)[()]
        return ops.exclusive_scan(x_local, op, carry)
    return ops.inclusive_scan(x_local, op, carry)


def _exchange(pieces_send, send_counts, recv_counts, group):
    """All-to-all of variable-sized pieces of one tensor.  pieces_send is the local tensor laid out
    destination-major; returns the received tensor laid out source-major."""
    world, rank = _world(group)
    out = torch.empty(int(sum(recv_counts)), dtype=pieces_send.dtype, device=pieces_send.device)
    if dist.get_backend(group) == "nccl":
        dist.all_to_all_single(_plumbing_view(out), _plumbing_view(pieces_send), [int(c) for c in recv_counts],
                               [int(c) for c in send_counts], group=group)
        return out
    # gloo has no all-to-all: pairwise send/recv (CPU tests of the orchestration only)
    send_off = np.concatenate([[0], np.cumsum(send_counts)]).astype(np.int64)
    recv_off = np.concatenate([[0], np.cumsum(recv_counts)]).astype(np.int64)
    out[recv_off[rank]:recv_off[rank + 1]] = pieces_send[send_off[rank]:send_off[rank + 1]]
    reqs = []
    for peer in range(world):
        if peer == rank:
            continue
        if send_counts[peer]:
            reqs.append(dist.isend(_plumbing_view(pieces_send[send_off[peer]:send_off[peer + 1]]).contiguous(), peer, group=group))
        if recv_counts[peer]:
            reqs.append(dist.irecv(_plumbing_view(out[recv_off[peer]:recv_off[peer + 1]]), peer, group=group))
    for r in reqs:
        r.wait()
    return out


def choose_splitters(all_samples, world, descending=False):
    """G-1 splitters from the gathered regular samples (a numpy array, any order): the elements at
    every (len/G)-th position of the sorted sample."""
    s = np.sort(all_samples, kind="stable")
    if descending:
        s = s[::-1]
    if s.size == 0:
        return s[:0]
    pos = [(i * s.size) // world for i in range(1, world)]
    return np.ascontiguousarray(s[pos])


def _gather_rows(row, world, group):
    """all-gather of one int64 row per rank; returns the [world, width] table on the host (the host wait)."""
    width = row.numel()
    table = torch.empty(world * width, dtype=torch.int64, device=row.device)
    if dist.get_backend(group) == "nccl":
        dist.all_gather_into_tensor(table, row, group=group)
    else:
        dist.all_gather(list(table.view(world, width).unbind(0)), row, group=group)
    return table.cpu().numpy().reshape(world, width)


def _device_splitters(keys, n, world, descending, group, ops, samples_per_rank):
    """G-1 splitters on the device: regular samples of every shard, all-gathered, sorted with the
    library's own sort, every (len/G)-th element taken.  No host wait."""
    dev = keys.device
    s = samples_per_rank
    pick = torch.from_numpy(((np.arange(s, dtype=np.int64) * 2 + 1) * max(n, 1) // (2 * s))).to(dev)
    kview = _plumbing_view(keys)
    mine = kview[pick] if n else torch.zeros(s, dtype=kview.dtype, device=dev)
    gathered = torch.empty(world * s, dtype=kview.dtype, device=dev)
    if dist.get_backend(group) == "nccl":
        dist.all_gather_into_tensor(gathered, mine, group=group)
    else:
        dist.all_gather(list(gathered.view(world, s).unbind(0)), mine, group=group)
    sample_keys = gathered.view(keys.dtype)
    ops.sort_by_key(sample_keys, None, descending)
    pos = torch.tensor([i * s for i in range(1, world)], dtype=torch.int64, device=dev)
    return _plumbing_view(sample_keys)[pos].view(keys.dtype), gathered


def _sort_by_histogram_exchange(keys, vals, descending, group, ops, mark):
    """The default route of sharded_sort_by_key on GPUs: splitters from a 12-bit digit histogram.
    One read of the shard builds the histogram; ONE all-gather gives every rank all histograms, from
    which each derives the same plan (bin ranges per rank, its offsets into every receive buffer,
    every rank's receive total); the host waits once, for ~400 bytes of that plan; one kernel per
    GPU then stores every pair straight into its owner's receive buffer over NVLink; a collective
    fences the stores; a stable local radix sort of what arrived finishes.  Returns None when some
    receive buffer would overflow (heavily skewed keys): the caller then samples splitters instead.
    The result is a view of a receive buffer that the call after next reuses."""
    world, rank = _world(group)
    dev = keys.device
    n = keys.numel()
    if n >= (1 << 30) or keys.element_size() not in (4, 8):
        return None
    vdt = None if vals is None else vals.dtype
    st = ops.exchange_state(dev, keys.dtype, vdt)
    capacity = int(1.25 * n) + 65536
    which, (rk, rv, kexp, vexp) = ops.exchange_receive_set(st, dev, keys.dtype, vdt, capacity)
    tag = (st["generation"][which] << 32) | rk.numel()
    row = ops.exchange_hist(st, keys, descending, tag)
    rows = torch.empty(world * st["row_words"], dtype=torch.int32, device=dev)
    dist.all_gather_into_tensor(rows, row, group=group)
    plan = ops.exchange_plan(st, rows, world, rank, keys.dtype)
    mark("splitters")
    head = plan[:st["head_bytes"]].cpu().numpy()                               # the one host wait
    mark("host_wait")
    table = head[8:].view(np.uint64).reshape(3, -1)                            # send_offset, recv_total, tag; 16 entries each
    recv_total = table[1, :world].astype(np.int64)
    tags = table[2, :world].copy()
    caps = (tags & np.uint64(0xFFFFFFFF)).astype(np.int64)
    if (recv_total > caps).any():
        st["turn"] ^= 1                                                       # this set was not used
        return None
    if st["known_tags"][which] is None or not np.array_equal(st["known_tags"][which], tags):
        # some rank (re)allocated this receive set: exchange the IPC handles (every rank sees the same tags and takes this branch together)
        mine = np.concatenate([kexp[0], [kexp[1]], (vexp[0] if vexp else np.zeros(8, np.int64)), [vexp[1] if vexp else 0]]).astype(np.int64)
        handles = _gather_rows(torch.from_numpy(mine).to(dev), world, group)
        # the peers' previous buffers of this set are gone (or about to be): unmap the ones that are not
        # among the new handles or the other set's.  Nothing of this process is still writing into
        # them: the last scatter into this set was two calls ago and a fence followed it.
        fresh = set()
        for d in range(world):
            if d != rank:
                fresh.add(handles[d, 0:8].astype(np.int64).tobytes())
                if rv is not None:
                    fresh.add(handles[d, 9:17].astype(np.int64).tobytes())
        stale = st["peer_handles"][which] - fresh - st["peer_handles"][which ^ 1]
        if stale:
            torch.cuda.current_stream().synchronize()
            for hb in stale:
                ops.close_buffer(np.frombuffer(hb, dtype=np.int64))
        st["peer_handles"][which] = fresh
        ptrs_k, ptrs_v = [], []
        for d in range(world):
            if d == rank:
                ptrs_k.append(rk.data_ptr())
                ptrs_v.append(None if rv is None else rv.data_ptr())
            else:
                ptrs_k.append(ops.open_buffer(handles[d, 0:8], int(handles[d, 8])))
                ptrs_v.append(None if rv is None else ops.open_buffer(handles[d, 9:17], int(handles[d, 17])))
        st["peer_ptrs"][which] = (ptrs_k, ptrs_v)
        st["known_tags"][which] = tags
    dst_k, dst_v = st["peer_ptrs"][which]
    ops.exchange_scatter(keys, vals, plan, dst_k, dst_v, descending)
    # every sender's stores must have landed before a receiver sorts its buffer
    fence = torch.zeros(1, dtype=torch.int32, device=dev)
    dist.all_reduce(fence, group=group)
    mark("exchange")
    m = int(recv_total[rank])
    out_k = rk[:m]
    out_v = None if rv is None else rv[:m]
    ops.sort_by_key(out_k, out_v, descending)
    mark("local_sort")
    return out_k, out_v


def _sort_by_scatter(keys, vals, descending, group, ops, samples_per_rank, mark):
    """The scatter route of sharded_sort_by_key; returns None if some receive buffer is too small
    (every rank takes the same decision from the same table)."""
    world, rank = _world(group)
    dev = keys.device
    n = keys.numel()
    if n == 0 or n >= (1 << 30):
        flag = torch.tensor([1], dtype=torch.int64, device=dev)
    else:
        flag = torch.tensor([0], dtype=torch.int64, device=dev)
    splitters, _ = _device_splitters(keys, n, world, descending, group, ops, samples_per_rank)
    counts = ops.bucket_count(keys, splitters, world, descending)
    capacity = int(1.5 * n) + 65536
    rk, rv, kexp, vexp = ops.receive_buffers(dev, keys.dtype, None if vals is None else vals.dtype, capacity)
    extra = np.concatenate([[rk.numel()], kexp[0], [kexp[1]], (vexp[0] if vexp else np.zeros(8, np.int64)), [vexp[1] if vexp else 0]]).astype(np.int64)
    row = torch.cat([counts, flag, torch.from_numpy(extra).to(dev)])
    mark("splitters")
    meta = _gather_rows(row, world, group)                                     # the one host wait
    mark("host_wait")
    count_matrix = meta[:, :world]                                             # [src][dst]
    unusable = meta[:, world].any()
    caps = meta[:, world + 1]
    handles = meta[:, world + 2:]
    recv_total = count_matrix.sum(axis=0)
    if unusable or (recv_total > caps).any():
        return None
    offsets = np.cumsum(count_matrix, axis=0) - count_matrix                   # rows before mine, per destination
    dst_k, dst_v = [], []
    for d in range(world):
        if d == rank:
            dst_k.append(rk.data_ptr())
            dst_v.append(None if rv is None else rv.data_ptr())
        else:
            dst_k.append(ops.open_buffer(handles[d, 0:8], int(handles[d, 8])))
            dst_v.append(None if rv is None else ops.open_buffer(handles[d, 9:17], int(handles[d, 17])))
    ops.bucket_scatter(keys, vals, splitters, dst_k, dst_v, offsets[rank], descending)
    # every sender's stores must have landed before a receiver sorts its buffer
    fence = torch.zeros(1, dtype=torch.int32, device=dev)
    dist.all_reduce(fence, group=group)
    mark("exchange")
    m = int(recv_total[rank])
    out_k = rk[:m]
    out_v = None if rv is None else rv[:m]
    ops.sort_by_key(out_k, out_v, descending)
    res = (out_k.clone(), None if out_v is None else out_v.clone())          # the receive buffers are reused by the next call
    mark("local_sort")
    return res


def sharded_sort_by_key(keys_local, vals_local=None, descending=False, group=None, ops=None, samples_per_rank=1024, stage_marks=None,
                        consume_input=False, exchange="auto"):
    """Stable sort of the concatenation of every rank's (keys_local, vals_local).  Returns this
    rank's slice (keys, vals) of the sorted sequence; slices are contiguous in rank order, sized by
    the splitters (about 1/G of the data each for sampled splitters).

    Everything up to the exchange is enqueued without waiting for the GPU: local sort, sample
    gather, all-gather of the samples, sort of the gathered sample and splitter pick, lower bounds,
    all-gather of the cut positions.  The host blocks once, to read the G x (G-1) cut positions that
    size the all-to-all; the merges after the exchange are enqueued without waiting again.
    exchange: "histogram" (the default on GPUs, see _sort_by_histogram_exchange) takes splitters from
    a digit histogram of the unsorted shard: one collective, one short host wait, then the same
    scatter kernel; its result is a view of a receive buffer that the call after next reuses.
    "scatter" does not sort first either: it samples splitters from
    the unsorted shard, counts and exchanges bucket sizes, and then ONE kernel per GPU splits its
    pairs by key range and stores each pair straight into the owning GPU's receive buffer over
    NVLink (stable: source-rank-major, input order inside a source); a stable local radix sort of
    what was received finishes the job.  "collective" moves the pieces with an all-to-all (NCCL; pairwise send/recv on gloo) and
    merges local copies; "peer" skips that copy: every rank publishes its sorted shard through CUDA
    IPC and the first round of merges reads the pieces it needs directly out of the peers' memory
    over NVLink with ordinary loads -- the exchange is fused into the merge kernel; "auto" picks
    "peer" when the ops object supports it.
    consume_input=True sorts the local shard in place first (thrust::sort_by_key itself is an in-place
    algorithm) and so saves one copy of the shard; by default the inputs are left untouched.
    stage_marks, if a list, receives (label, callable) pairs where the callable records a marker on
    the current stream (the caller supplies what a marker is, e.g. a CUDA event)."""
    ops = ops or DeviceOps()
    mark = (lambda label: stage_marks.append((label, stage_marks[0][1]()))) if stage_marks else (lambda label: None)
    world, rank = _world(group)
    can_peer = getattr(ops, "supports_peer_reads", False) and keys_local.is_cuda
    if world > 1 and world <= 16 and keys_local.is_cuda and getattr(ops, "supports_histogram_exchange", False) and exchange in ("auto", "histogram"):
        done = _sort_by_histogram_exchange(keys_local, vals_local, descending, group, ops, mark)
        if done is not None:
            return done
        exchange = "scatter"                    # skewed keys: sampled splitters balance better
    if world > 1 and (exchange == "scatter" or (exchange == "auto" and can_peer and world <= 16)):
        done = _sort_by_scatter(keys_local, vals_local, descending, group, ops, samples_per_rank, mark)
        if done is not None:
            return done
        exchange = "peer"                       # a receive buffer would have overflowed: take the merge route
    dev = keys_local.device
    n = keys_local.numel()
    keys = keys_local if consume_input else keys_local.clone()
    vals = None if vals_local is None else (vals_local if consume_input else vals_local.clone())
    mark("copy")
    ops.sort_by_key(keys, vals, descending)
    mark("local_sort")
    if world == 1:
        return keys, vals

    # regular samples of the sorted shard; a rank without data contributes copies of nothing (flagged)
    s = samples_per_rank
    pick = torch.from_numpy(((np.arange(s, dtype=np.int64) * 2 + 1) * max(n, 1) // (2 * s))).to(dev)
    kview = _plumbing_view(keys)
    mine = kview[pick] if n else torch.zeros(s, dtype=kview.dtype, device=dev)
    gathered = torch.empty(world * s, dtype=kview.dtype, device=dev)
    dist.all_gather_into_tensor(gathered, mine, group=group) if dist.get_backend(group) == "nccl" else \
        dist.all_gather(list(gathered.view(world, s).unbind(0)), mine, group=group)
    sizes_t = torch.tensor([n], dtype=torch.int64, device=dev)

    # sort the gathered sample with the same kernels and take every (len/G)-th element as a splitter.
    # (ranks without data are rare; they are handled by the host path below)
    sample_keys = gathered.view(keys.dtype)
    ops.sort_by_key(sample_keys, None, descending)
    pos = torch.tensor([i * s for i in range(1, world)], dtype=torch.int64, device=dev)
    splitters = _plumbing_view(sample_keys)[pos].view(keys.dtype)

    peer = exchange == "peer" or (exchange == "auto" and can_peer)
    extra = np.zeros(0, np.int64)
    if peer:
        kh, koff = ops.export_buffer(keys)
        vh, voff = (np.zeros(8, np.int64), 0) if vals is None else ops.export_buffer(vals)
        extra = np.concatenate([kh, [koff], vh, [voff]]).astype(np.int64)
    cuts = ops.lower_bound(keys, splitters, descending)                       # [G-1] on the device
    row = torch.cat([cuts, sizes_t, torch.from_numpy(extra).to(dev)])
    width = row.numel()
    table = torch.empty(world * width, dtype=torch.int64, device=dev)
    dist.all_gather_into_tensor(table, row, group=group) if dist.get_backend(group) == "nccl" else \
        dist.all_gather(list(table.view(world, width).unbind(0)), row, group=group)
    mark("splitters")
    # the one host wait: cut positions, shard sizes and buffer handles of every rank
    meta = table.cpu().numpy().reshape(world, width)
    cut_matrix = meta[:, :world - 1]
    sizes_host = meta[:, world - 1]
    handles = meta[:, world:]
    if (sizes_host == 0).any():
        # a rank without data contributed placeholder samples: redo the splitters on the host from the real ones
        real = np.concatenate([gathered.view(world, s)[r].cpu().numpy().view(_np_dtype(keys)) for r in range(world) if sizes_host[r] > 0]) \
            if (sizes_host > 0).any() else np.empty(0, _np_dtype(keys))
        if real.size == 0:
            return keys, vals
        sp = choose_splitters(real, world, descending)
        cuts = ops.lower_bound(keys, torch.from_numpy(sp.copy()).to(dev), descending)
        all_cuts = torch.empty(world * (world - 1), dtype=torch.int64, device=dev)
        dist.all_gather_into_tensor(all_cuts, cuts, group=group) if dist.get_backend(group) == "nccl" else \
            dist.all_gather(list(all_cuts.view(world, world - 1).unbind(0)), cuts, group=group)
        cut_matrix = all_cuts.cpu().numpy().reshape(world, world - 1)
    bounds = np.concatenate([np.zeros((world, 1), np.int64), cut_matrix, sizes_host.reshape(world, 1)], axis=1)
    count_matrix = np.diff(bounds, axis=1)                                    # [src][dst]
    send_counts = count_matrix[rank]
    recv_counts = count_matrix[:, rank]

    mark("host_wait")
    if peer:
        # runs stay where they are: (pointer, length) pairs into the peers' published shards
        ksz = keys.element_size()
        vsz = 0 if vals is None else vals.element_size()
        runs = []
        opened = set()
        for src in range(world):
            start = int(bounds[src, rank])
            cnt = int(count_matrix[src, rank])
            if src == rank:
                kp = keys.data_ptr()
                vp = None if vals is None else vals.data_ptr()
            else:
                kp = ops.open_buffer(handles[src, 0:8], int(handles[src, 8]))
                vp = None if vals is None else ops.open_buffer(handles[src, 9:17], int(handles[src, 17]))
                opened.add(handles[src, 0:8].astype(np.int64).tobytes())
                if vals is not None:
                    opened.add(handles[src, 9:17].astype(np.int64).tobytes())
            runs.append((kp + start * ksz, None if vp is None else vp + start * vsz, cnt, None))
        mark("exchange")
        vdtype = None if vals is None else vals.dtype
        if hasattr(ops, "merge_runs_raw"):
            owner = ops.merge_runs_raw([(r[0], r[1], r[2]) for r in runs], keys.dtype, vdtype, descending, dev)
        else:
            while len(runs) > 1:
                nxt = []
                for i in range(0, len(runs) - 1, 2):
                    (ka, va, na, _), (kb, vb, nb, _) = runs[i], runs[i + 1]
                    ko, vo = ops.merge_by_key_raw(ka, na, kb, nb, va, vb, keys.dtype, vdtype, descending, dev)
                    nxt.append((ko.data_ptr(), None if vo is None else vo.data_ptr(), na + nb, (ko, vo)))   # keep the tensors alive
                if len(runs) % 2:
                    nxt.append(runs[-1])
                runs = nxt
            kp, vp, cnt, owner = runs[0]
            if owner is None:                                     # a lone run that was never merged is still a view of a shard: copy it
                owner = ops.merge_by_key_raw(kp, cnt, kp, 0, vp, vp, keys.dtype, vdtype, descending, dev)
        # nobody may reuse a shard while a peer still reads it: a collective on the stream orders
        # every rank's merges before whatever the callers enqueue next
        fence = torch.zeros(1, dtype=torch.int32, device=dev)
        dist.all_reduce(fence, group=group)
        mark("merge")
        # the shards were the callers' own tensors, which they may free or reuse at any time: unmap
        # them once this rank's merges have read them (a stale mapping must never be served again)
        if hasattr(ops, "close_buffer") and opened:
            torch.cuda.current_stream().synchronize()
            for hb in opened:
                ops.close_buffer(np.frombuffer(hb, dtype=np.int64))
        return owner

    rk = _exchange(keys, send_counts, recv_counts, group)
    rv = None if vals is None else _exchange(vals, send_counts, recv_counts, group)
    mark("exchange")

    # merge the G sorted runs received, pairwise in source-rank order (ties keep the lower rank first)
    off = np.concatenate([[0], np.cumsum(recv_counts)]).astype(np.int64)
    runs = [(rk[off[i]:off[i + 1]], None if rv is None else rv[off[i]:off[i + 1]]) for i in range(world)]
    while len(runs) > 1:
        nxt = []
        for i in range(0, len(runs) - 1, 2):
            (ka, va), (kb, vb) = runs[i], runs[i + 1]
            nxt.append(ops.merge_by_key(ka, kb, va, vb, descending))
        if len(runs) % 2:
            nxt.append(runs[-1])
        runs = nxt
    mark("merge")
    return runs[0]


def check_sharded_sort(keys_out, vals_out, n_total, key_of_index, group=None, descending=False):
    """Checks a sharded sort_by_key whose values were the original global indices 0 .. n_total-1 and
    whose keys can be recomputed from an index (key_of_index: numpy index array -> numpy key array):
    every output pair is an input pair; each shard is sorted, values increasing inside equal keys
    (stable); shards are in rank order; the shard sizes add up and the values are, by count, sum and
    sum of squares, the indices 0 .. n_total-1.  Together: the stable sort of the whole input.
    Collective (every rank calls it); returns True on every rank or raises."""
    world, rank = _world(group)
    k = keys_out.cpu().numpy()
    v = vals_out.cpu().numpy()
    assert np.array_equal(key_of_index(v), k), "an output pair is not an input pair"
    if k.size > 1:
        a, b = (k[1:], k[:-1]) if not descending else (k[:-1], k[1:])
        assert bool((a >= b).all()), "a shard is not sorted"
        ties = k[1:] == k[:-1]
        assert bool((v[1:][ties] > v[:-1][ties]).all()), "equal keys are not in input order"
    v64 = v.astype(np.uint64)
    with np.errstate(over="ignore"):
        mine = np.array([k.size, int(v64.sum(dtype=np.uint64) & np.uint64(0x7FFFFFFFFFFFFFFF)),
                         int((v64 * v64).sum(dtype=np.uint64) & np.uint64(0x7FFFFFFFFFFFFFFF)),
                         int(k[0]) if k.size else -1, int(k[-1]) if k.size else -1,
                         int(v[0]) if k.size else -1, int(v[-1]) if k.size else -1], dtype=np.int64)
    rows = _gather_rows(torch.from_numpy(mine).to(keys_out.device), world, group)
    assert int(rows[:, 0].sum()) == n_total, "shard sizes do not add up"
    want1 = (n_total * (n_total - 1) // 2) % (1 << 63)                        # closed forms, modulo 2^63 like the sums above
    want2 = ((n_total - 1) * n_total * (2 * n_total - 1) // 6) % (1 << 63)
    with np.errstate(over="ignore"):
        got1 = int(np.sum(rows[:, 1].astype(np.uint64), dtype=np.uint64) & np.uint64(0x7FFFFFFFFFFFFFFF))
        got2 = int(np.sum(rows[:, 2].astype(np.uint64), dtype=np.uint64) & np.uint64(0x7FFFFFFFFFFFFFFF))
    assert got1 == want1 and got2 == want2, "the values are not a permutation of the indices"
    full = [r for r in range(world) if rows[r, 0] > 0]
    for a, b in zip(full[:-1], full[1:]):
        last, first = rows[a, 4], rows[b, 3]
        assert (first >= last) if not descending else (first <= last), "shards are not in rank order"
        assert first != last or rows[b, 5] > rows[a, 6], "equal keys across a shard boundary are not in input order"
    return True
