"""Host-side mirror of the Thrust algorithms on the hot path, over the C ABI.

Function names, argument meaning and return conventions follow the reference's CUDA backend
(thrust/system/cuda/detail/{reduce,scan,sort,copy_if,partition,unique,reduce_by_key,merge}.h):
synchronous on return, results that are counts come back as Python ints, "end iterators" come
back as the output tensor sliced to its logical length.  Inputs are CUDA torch tensors; torch is
used only to own device memory and to name the stream.  Every call goes through
libthrust_b200.so; there is no fallback path.
"""
import ctypes as C

import numpy as np
import torch

from . import _lib

DTYPE_CODE = {
    torch.int8: 0, torch.uint8: 1, torch.int16: 2, torch.uint16: 3, torch.int32: 4,
    torch.uint32: 5, torch.int64: 6, torch.uint64: 7, torch.float32: 8, torch.float64: 9,
}
NP_OF = {
    torch.int8: np.int8, torch.uint8: np.uint8, torch.int16: np.int16, torch.uint16: np.uint16,
    torch.int32: np.int32, torch.uint32: np.uint32, torch.int64: np.int64, torch.uint64: np.uint64,
    torch.float32: np.float32, torch.float64: np.float64,
}
TORCH_OF = {np.dtype(v): k for k, v in NP_OF.items()}
OPS = {"plus": 0, "min": 1, "max": 2}
PREDS = {"mod_eq": 0, "lt": 1, "ge": 2, "ne": 3}


class Tb200Error(RuntimeError):
    """A C-ABI call returned a CUDA error, or a kernel reported a failed wait."""


def _check(rc, what):
    if rc != 0:
        raise Tb200Error("%s failed with cudaError %d" % (what, rc))


def _ptr(t):
    return None if t is None else C.c_void_p(t.data_ptr())


def _stream():
    return C.c_void_p(torch.cuda.current_stream().cuda_stream)


def _require_cuda(*tensors):
    for t in tensors:
        if t is not None and (not t.is_cuda or not t.is_contiguous()):
            raise ValueError("thrust_b200 operates on contiguous CUDA tensors")


class _Workspaces:
    """Scratch buffers cached per (device, stream, call site) and grown on demand, standing in for
    the reference's per-call temporary_array (thrust/system/cuda/detail/reduce.h:959)."""

    def __init__(self):
        self._bufs = {}

    def get(self, tag, nbytes):
        key = (torch.cuda.current_device(), torch.cuda.current_stream().cuda_stream, tag)
        buf = self._bufs.get(key)
        if buf is None or buf.numel() < nbytes:
            buf = torch.empty(max(int(nbytes), 256), dtype=torch.uint8, device="cuda")
            self._bufs[key] = buf
        return buf

    def clear(self):
        self._bufs.clear()


workspaces = _Workspaces()


def _call_with_ws(tag, fn, *args):
    """fn(*args, d_ws, &ws_bytes, stream): size query, then the real call.  Returns the workspace."""
    lib_fn = getattr(_lib.load(), fn)
    need = C.c_size_t(0)
    _check(lib_fn(*args, None, C.byref(need), _stream()), fn + " (size query)")
    ws = workspaces.get(tag, need.value)
    have = C.c_size_t(ws.numel())
    _check(lib_fn(*args, _ptr(ws), C.byref(have), _stream()), fn)
    return ws


def _sync_and_check(ws, what):
    status = C.c_uint(0)
    _check(_lib.load().tb200_workspace_status(_ptr(ws), _stream(), C.byref(status)), what + " (status)")
    if status.value != 0:
        raise Tb200Error("%s: device reported status %d (an inter-CTA wait ran out)" % (what, status.value))


# ------------------------------------------------------------------------------------- reduce
def reduce(x, init=None, op="plus", acc_dtype=None):
    """thrust::reduce(first, last, init, op): returns init (+) x[0] (+) ... as a numpy scalar of the
    accumulator type (the type of `init`; default: x's type and 0, as in reduce.h:1057-1067)."""
    _require_cuda(x)
    if acc_dtype is None:
        acc_dtype = x.dtype if init is None or not isinstance(init, np.generic) else TORCH_OF[np.dtype(init.dtype)]
    h_init = np.asarray(0 if init is None else init, dtype=NP_OF[acc_dtype])
    out = torch.empty(1, dtype=acc_dtype, device=x.device)
    ws = _call_with_ws("reduce", "tb200_reduce", _ptr(x), x.numel(), DTYPE_CODE[x.dtype], DTYPE_CODE[acc_dtype],
                       OPS[op], C.c_void_p(h_init.ctypes.data), _ptr(out))
    _sync_and_check(ws, "reduce")
    return out.cpu().numpy().view(NP_OF[acc_dtype])[0]


def reduce_to_device(x, init, op="plus", acc_dtype=None, out=None):
    """The same reduction with the result left in device memory (a 1-element tensor of the accumulator
    type) and nothing waited for: for callers that feed it to later work on the stream."""
    _require_cuda(x)
    acc_dtype = acc_dtype or x.dtype
    h_init = np.asarray(init, dtype=NP_OF[acc_dtype])
    out = torch.empty(1, dtype=acc_dtype, device=x.device) if out is None else out
    _call_with_ws("reduce", "tb200_reduce", _ptr(x), x.numel(), DTYPE_CODE[x.dtype], DTYPE_CODE[acc_dtype], OPS[op],
                  C.c_void_p(h_init.ctypes.data), _ptr(out))
    return out


# ------------------------------------------------------------------------------------- scan
def inclusive_scan(x, out=None, op="plus", init=None, sync=True):
    """thrust::inclusive_scan(first, last, result, op); out may be x (in place).  Returns out.
    `init`, if given, is combined in front of the first element (the carry of a sharded scan): a
    host scalar, or a 1-element CUDA tensor of x's type that earlier work on the stream fills in."""
    _require_cuda(x, out)
    out = torch.empty_like(x) if out is None else out
    if isinstance(init, torch.Tensor):
        ws = _call_with_ws("scan", "tb200_inclusive_scan_dinit", _ptr(x), _ptr(out), x.numel(), DTYPE_CODE[x.dtype], OPS[op], _ptr(init))
    else:
        h_init = None if init is None else np.asarray(init, dtype=NP_OF[x.dtype])
        ws = _call_with_ws("scan", "tb200_inclusive_scan", _ptr(x), _ptr(out), x.numel(), DTYPE_CODE[x.dtype], OPS[op],
                           None if h_init is None else C.c_void_p(h_init.ctypes.data))
    if sync:
        _sync_and_check(ws, "inclusive_scan")
    return out


def exclusive_scan(x, init=0, out=None, op="plus", sync=True):
    """thrust::exclusive_scan(first, last, result, init, op); init as for inclusive_scan."""
    _require_cuda(x, out)
    out = torch.empty_like(x) if out is None else out
    if isinstance(init, torch.Tensor):
        ws = _call_with_ws("scan", "tb200_exclusive_scan_dinit", _ptr(x), _ptr(out), x.numel(), DTYPE_CODE[x.dtype], OPS[op], _ptr(init))
    else:
        h_init = np.asarray(init, dtype=NP_OF[x.dtype])
        ws = _call_with_ws("scan", "tb200_exclusive_scan", _ptr(x), _ptr(out), x.numel(), DTYPE_CODE[x.dtype], OPS[op],
                           C.c_void_p(h_init.ctypes.data))
    if sync:
        _sync_and_check(ws, "exclusive_scan")
    return out


# ------------------------------------------------------------------------------------- sort
def _sort_impl(keys, vals, descending, begin_bit, end_bit, sync=True):
    _require_cuda(keys, vals)
    if vals is not None and vals.numel() != keys.numel():
        raise ValueError("keys and values differ in length")
    n = keys.numel()
    vb = 0 if vals is None else vals.element_size()
    kalt = workspaces.get("sort_keys_alt", n * keys.element_size())
    valt = None if vals is None else workspaces.get("sort_vals_alt", n * vb)
    end_bit = 8 * keys.element_size() if end_bit is None else end_bit
    ws = _call_with_ws("sort", "tb200_sort_by_key", _ptr(keys), _ptr(kalt), _ptr(vals), _ptr(valt), n,
                       DTYPE_CODE[keys.dtype], vb, int(descending), begin_bit, end_bit)
    if sync:
        _sync_and_check(ws, "sort")


def sort(keys, descending=False, sync=True):
    """thrust::sort / thrust::stable_sort(first, last[, greater]) in place.  sync=False only
    enqueues the work (for callers that chain several calls on one stream)."""
    _sort_impl(keys, None, descending, 0, None, sync)
    return keys


stable_sort = sort


def sort_by_key(keys, vals, descending=False, begin_bit=0, end_bit=None, sync=True):
    """thrust::sort_by_key / stable_sort_by_key(keys_first, keys_last, values_first[, greater]) in
    place; stable."""
    _sort_impl(keys, vals, descending, begin_bit, end_bit, sync)
    return keys, vals


stable_sort_by_key = sort_by_key

_side_streams = {}


def sort_by_key_host(h_keys, h_vals, h_keys_out=None, h_vals_out=None, descending=False):
    """thrust::sort_by_key for keys and values that start and end in (pinned) host memory: the call
    a host-side caller makes when the data does not live on the device.  The keys go up first and are
    sorted together with their positions while the values are still on their way up on a second
    stream; the sorted keys then travel back down while the values finish arriving (PCIe carries
    both directions at once), the values are permuted by the sorted positions (tb200_gather) and
    follow.  The result equals sort_by_key's on the same data (the sort is stable).  h_*_out default
    to the inputs (in place).  Returns (h_keys_out, h_vals_out) after synchronising."""
    if h_keys.is_cuda or h_vals.is_cuda:
        raise ValueError("sort_by_key_host takes host tensors; device tensors go to sort_by_key")
    n = h_keys.numel()
    if h_vals.numel() != n or h_vals.element_size() not in (4, 8) or n > 0xFFFFFFFF:
        raise ValueError("need one 4- or 8-byte value per key and at most 2^32 - 1 pairs")
    h_keys_out = h_keys if h_keys_out is None else h_keys_out
    h_vals_out = h_vals if h_vals_out is None else h_vals_out
    if n == 0:
        return h_keys_out, h_vals_out
    lib = _lib.load()
    dev = torch.cuda.current_device()
    main = torch.cuda.current_stream()
    side = _side_streams.get(dev)
    if side is None:
        side = _side_streams[dev] = torch.cuda.Stream()
    vb = h_vals.element_size()
    d_keys = workspaces.get("host_sort_keys", n * h_keys.element_size()).view(h_keys.dtype)[:n]
    d_pos = workspaces.get("host_sort_pos", n * 4).view(torch.int32)[:n]
    d_vals = workspaces.get("host_sort_vals", n * vb).view(h_vals.dtype)[:n]
    d_vals_out = workspaces.get("host_sort_vals_out", n * vb).view(h_vals.dtype)[:n]
    d_keys.copy_(h_keys.view(-1), non_blocking=True)
    keys_up = torch.cuda.Event()
    keys_up.record(main)
    side.wait_stream(main)                              # the value buffer may still be read by an earlier call's gather
    with torch.cuda.stream(side):
        side.wait_event(keys_up)                        # keys first: the sort can start while the values follow
        d_vals.copy_(h_vals.view(-1), non_blocking=True)
        vals_up = torch.cuda.Event()
        vals_up.record(side)
    _check(lib.tb200_sequence_u32(_ptr(d_pos), n, _stream()), "tb200_sequence_u32")
    sort_by_key(d_keys, d_pos, descending, sync=False)
    h_keys_out.view(-1).copy_(d_keys, non_blocking=True)
    main.wait_event(vals_up)
    _check(lib.tb200_gather(_ptr(d_vals), _ptr(d_pos), _ptr(d_vals_out), n, vb, _stream()), "tb200_gather")
    h_vals_out.view(-1).copy_(d_vals_out, non_blocking=True)
    _sync_and_check(workspaces.get("sort", 1), "sort_by_key_host")      # waits for the stream
    return h_keys_out, h_vals_out


# ------------------------------------------------------------------------------------- compaction
def _count_word():
    return torch.zeros(1, dtype=torch.int64, device="cuda")


def _read_count(cnt):
    return int(cnt.cpu().item())


def copy_if(x, pred, a=0, b=0, stencil=None, out=None):
    """thrust::copy_if(first, last, [stencil,] result, pred): returns out[:count] (stable)."""
    _require_cuda(x, stencil, out)
    out = torch.empty_like(x) if out is None else out
    cnt = _count_word()
    ws = _call_with_ws("select", "tb200_copy_if", _ptr(x), _ptr(stencil), _ptr(out), x.numel(), DTYPE_CODE[x.dtype],
                       0 if stencil is None else DTYPE_CODE[stencil.dtype], PREDS[pred], a, b, _ptr(cnt))
    _sync_and_check(ws, "copy_if")
    return out[:_read_count(cnt)]


def partition_copy(x, pred, a=0, b=0, stencil=None):
    """thrust::stable_partition_copy: returns (selected, rejected), both in input order."""
    _require_cuda(x, stencil)
    out_t, out_f = torch.empty_like(x), torch.empty_like(x)
    cnt = _count_word()
    ws = _call_with_ws("select", "tb200_partition_copy", _ptr(x), _ptr(stencil), _ptr(out_t), _ptr(out_f), x.numel(),
                       DTYPE_CODE[x.dtype], 0 if stencil is None else DTYPE_CODE[stencil.dtype], PREDS[pred], a, b, _ptr(cnt))
    _sync_and_check(ws, "partition_copy")
    k = _read_count(cnt)
    return out_t[:k], out_f[:x.numel() - k]


stable_partition_copy = partition_copy


def partition(x, pred, a=0, b=0):
    """thrust::partition / thrust::stable_partition in place; returns the split point."""
    _require_cuda(x)
    cnt = _count_word()
    ws = _call_with_ws("partition", "tb200_partition", _ptr(x), x.numel(), DTYPE_CODE[x.dtype], PREDS[pred], a, b, _ptr(cnt))
    _sync_and_check(ws, "partition")
    return _read_count(cnt)


stable_partition = partition


def unique_copy(x, out=None):
    """thrust::unique_copy(first, last, result): returns out[:count]."""
    _require_cuda(x, out)
    out = torch.empty_like(x) if out is None else out
    cnt = _count_word()
    ws = _call_with_ws("select", "tb200_unique_copy", _ptr(x), _ptr(out), x.numel(), DTYPE_CODE[x.dtype], _ptr(cnt))
    _sync_and_check(ws, "unique_copy")
    return out[:_read_count(cnt)]


def unique(x):
    """thrust::unique(first, last) in place: returns x[:count]."""
    return unique_copy(x, out=x)


def reduce_by_key(keys, vals, op="plus"):
    """thrust::reduce_by_key(keys_first, keys_last, values_first, keys_out, values_out, equal_to, op):
    returns (keys_out[:runs], values_out[:runs])."""
    _require_cuda(keys, vals)
    ko, vo = torch.empty_like(keys), torch.empty_like(vals)
    cnt = _count_word()
    ws = _call_with_ws("rbk", "tb200_reduce_by_key", _ptr(keys), _ptr(vals), _ptr(ko), _ptr(vo), keys.numel(),
                       DTYPE_CODE[keys.dtype], DTYPE_CODE[vals.dtype], OPS[op], _ptr(cnt))
    _sync_and_check(ws, "reduce_by_key")
    k = _read_count(cnt)
    return ko[:k], vo[:k]


def inclusive_scan_by_key(keys, vals, out=None, op="plus"):
    """thrust::inclusive_scan_by_key(keys_first, keys_last, values_first, result, equal_to, op)."""
    _require_cuda(keys, vals, out)
    out = torch.empty_like(vals) if out is None else out
    ws = _call_with_ws("rbk", "tb200_scan_by_key", _ptr(keys), _ptr(vals), _ptr(out), keys.numel(), DTYPE_CODE[keys.dtype],
                       DTYPE_CODE[vals.dtype], OPS[op], 0, None)
    _sync_and_check(ws, "inclusive_scan_by_key")
    return out


def exclusive_scan_by_key(keys, vals, init=0, out=None, op="plus"):
    """thrust::exclusive_scan_by_key(keys_first, keys_last, values_first, result, init, equal_to, op)."""
    _require_cuda(keys, vals, out)
    out = torch.empty_like(vals) if out is None else out
    h_init = np.asarray(init, dtype=NP_OF[vals.dtype])
    ws = _call_with_ws("rbk", "tb200_scan_by_key", _ptr(keys), _ptr(vals), _ptr(out), keys.numel(), DTYPE_CODE[keys.dtype],
                       DTYPE_CODE[vals.dtype], OPS[op], 1, C.c_void_p(h_init.ctypes.data))
    _sync_and_check(ws, "exclusive_scan_by_key")
    return out


def unique_by_key_copy(keys, vals, keys_out=None, vals_out=None):
    """thrust::unique_by_key_copy: returns (keys_out[:runs], vals_out[:runs])."""
    _require_cuda(keys, vals, keys_out, vals_out)
    ko = torch.empty_like(keys) if keys_out is None else keys_out
    vo = torch.empty_like(vals) if vals_out is None else vals_out
    cnt = _count_word()
    ws = _call_with_ws("rbk", "tb200_unique_by_key_copy", _ptr(keys), _ptr(vals), _ptr(ko), _ptr(vo), keys.numel(),
                       DTYPE_CODE[keys.dtype], vals.element_size(), _ptr(cnt))
    _sync_and_check(ws, "unique_by_key_copy")
    k = _read_count(cnt)
    return ko[:k], vo[:k]


def unique_by_key(keys, vals):
    """thrust::unique_by_key in place: returns (keys[:runs], vals[:runs])."""
    return unique_by_key_copy(keys, vals, keys, vals)


# ------------------------------------------------------------------------------------- extrema
def _extrema(fn, x, words):
    _require_cuda(x)
    idx = torch.zeros(words, dtype=torch.int64, device="cuda")
    ws = _call_with_ws("reduce", fn, _ptr(x), x.numel(), DTYPE_CODE[x.dtype], _ptr(idx))
    _sync_and_check(ws, fn)
    return [int(v) for v in idx.cpu().tolist()]


def min_element(x):
    """thrust::min_element(first, last): position of the first smallest element (0 when empty)."""
    return _extrema("tb200_min_element", x, 1)[0]


def max_element(x):
    """thrust::max_element(first, last): position of the first largest element (0 when empty)."""
    return _extrema("tb200_max_element", x, 1)[0]


def minmax_element(x):
    """thrust::minmax_element(first, last): (position of the first smallest, of the first largest)."""
    lo, hi = _extrema("tb200_minmax_element", x, 2)
    return lo, hi


# ------------------------------------------------------------------------------------- merge
def merge_by_key(keys_a, keys_b, vals_a=None, vals_b=None, descending=False, sync=True):
    """thrust::merge_by_key(A, B, payload A, payload B, keys_out, payload_out[, greater]); with no
    payloads it is thrust::merge.  Returns (keys_out, payload_out or None)."""
    _require_cuda(keys_a, keys_b, vals_a, vals_b)
    if keys_a.dtype != keys_b.dtype:
        raise ValueError("key types differ")
    na, nb = keys_a.numel(), keys_b.numel()
    ko = torch.empty(na + nb, dtype=keys_a.dtype, device=keys_a.device)
    vo = None if vals_a is None else torch.empty(na + nb, dtype=vals_a.dtype, device=keys_a.device)
    vb = 0 if vals_a is None else vals_a.element_size()
    ws = _call_with_ws("merge", "tb200_merge_by_key", _ptr(keys_a), _ptr(vals_a), na, _ptr(keys_b), _ptr(vals_b), nb, _ptr(ko),
                       _ptr(vo), DTYPE_CODE[keys_a.dtype], vb, int(descending))
    if sync:
        _sync_and_check(ws, "merge_by_key")
    return ko, vo


def merge(a, b, descending=False):
    """thrust::merge(A, B, out[, greater])."""
    return merge_by_key(a, b, None, None, descending)[0]


SET_OPS = {"union": 0, "intersection": 1, "difference": 2, "symmetric_difference": 3}


def set_operation(op, keys_a, keys_b, vals_a=None, vals_b=None, descending=False):
    """thrust::set_union / set_intersection / set_difference / set_symmetric_difference (op names
    as in SET_OPS) of two sorted ranges, and their _by_key forms when vals_a is given (vals_b for the
    union and the symmetric difference, whose results also take items from B).  Returns
    (keys_out, vals_out or None) cut to the result's length."""
    _require_cuda(keys_a, keys_b, vals_a, vals_b)
    if keys_a.dtype != keys_b.dtype:
        raise ValueError("key types differ")
    code = SET_OPS[op]
    na, nb = keys_a.numel(), keys_b.numel()
    cap = {0: na + nb, 1: min(na, nb), 2: na, 3: na + nb}[code]
    ko = torch.empty(cap, dtype=keys_a.dtype, device=keys_a.device)
    vo = None if vals_a is None else torch.empty(cap, dtype=vals_a.dtype, device=keys_a.device)
    vb = 0 if vals_a is None else vals_a.element_size()
    cnt = _count_word()
    ws = _call_with_ws("setop", "tb200_set_operation", code, _ptr(keys_a), na, _ptr(keys_b), nb, _ptr(vals_a), _ptr(vals_b), _ptr(ko), _ptr(vo),
                       DTYPE_CODE[keys_a.dtype], vb, int(descending), _ptr(cnt))
    _sync_and_check(ws, "set_" + op)
    m = _read_count(cnt)
    return ko[:m], (None if vo is None else vo[:m])


def merge_sort_by_key(keys, vals=None, descending=False):
    """The comparison-sort route of thrust::stable_sort(_by_key): stable merge sort in place."""
    _require_cuda(keys, vals)
    n = keys.numel()
    vb = 0 if vals is None else vals.element_size()
    kalt = workspaces.get("sort_keys_alt", n * keys.element_size())
    valt = None if vals is None else workspaces.get("sort_vals_alt", n * vb)
    ws = _call_with_ws("merge_sort", "tb200_merge_sort_by_key", _ptr(keys), _ptr(kalt), _ptr(vals), _ptr(valt), n,
                       DTYPE_CODE[keys.dtype], vb, int(descending))
    _sync_and_check(ws, "merge_sort_by_key")
    return keys, vals


def stable_sort_zip_by_first(keys, vals, method="merge"):
    """thrust::stable_sort(zip(keys, vals), comp) with comp ordering on get<0> alone, in place.
    method "merge" follows the reference's comparator route (merge sort); "radix" uses the fact
    that the comparator is a plain less on an arithmetic key and takes the radix path."""
    if method == "radix":
        return sort_by_key(keys, vals)
    return merge_sort_by_key(keys, vals)
