"""ctypes front end of the CPU oracle libraries -- TEST INFRASTRUCTURE, NOT PRODUCT CODE.

Loads oracle/_ref/liboracle_ref.so (the reference Thrust 1.14.0 compiled with its OpenMP device
system) and oracle/_build/liboracle_port.so (the plain-C restatement, oracle/port.c).  Both export
the interface of oracle/oracle_api.h; `Oracle` wraps it with numpy arrays in, numpy arrays out.
Only tests, the smoke check and the CPU-baseline legs of the benchmark may import this module.
"""
import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
REF_SO = os.path.join(_HERE, "_ref", "liboracle_ref.so")
PORT_SO = os.path.join(_HERE, "_build", "liboracle_port.so")

DTYPES = {
    np.dtype(np.int8): 0, np.dtype(np.uint8): 1, np.dtype(np.int16): 2, np.dtype(np.uint16): 3,
    np.dtype(np.int32): 4, np.dtype(np.uint32): 5, np.dtype(np.int64): 6, np.dtype(np.uint64): 7,
    np.dtype(np.float32): 8, np.dtype(np.float64): 9,
}
OPS = {"plus": 0, "min": 1, "max": 2}
PREDS = {"mod_eq": 0, "lt": 1, "ge": 2, "ne": 3}


def build(which=("port", "ref"), thrust_ref=None):
    """Compile the oracle libraries with oracle/Makefile.  `ref` needs a checkout of the reference
    (Thrust 1.14.0): the directory named by THRUST_REF, else baseline/_ref in this repository, else a
    directory `reference` beside the repository; it is skipped silently when none has the headers."""
    env = dict(os.environ)
    repo = os.path.dirname(_HERE)
    candidates = [thrust_ref, env.get("THRUST_REF"), os.path.join(repo, "baseline", "_ref"), os.path.join(os.path.dirname(repo), "reference")]
    ref_dir = next((c for c in candidates if c and os.path.isfile(os.path.join(c, "thrust", "version.h"))), "")
    if "port" in which:
        subprocess.check_call(["make", "-C", _HERE, "port"], env=env)
    if "ref" in which and os.path.isfile(os.path.join(ref_dir, "thrust", "version.h")):
        subprocess.check_call(["make", "-C", _HERE, "ref", "THRUST_REF=" + ref_dir], env=env)


def _ptr(a):
    return None if a is None else C.c_void_p(a.ctypes.data)


class Oracle:
    """One loaded oracle library."""

    def __init__(self, path):
        self.path = path
        lib = C.CDLL(path)
        self.lib = lib
        lib.ora_kind.restype = C.c_char_p
        lib.ora_threads.restype = C.c_int
        for name in ("ora_copy_if", "ora_partition", "ora_stable_partition", "ora_partition_copy",
                     "ora_unique_copy", "ora_reduce_by_key", "ora_reduce_by_key_f32_via_f64", "ora_unique_by_key_copy"):
            getattr(lib, name).restype = C.c_int64
        self.kind = lib.ora_kind().decode()
        self.threads = lib.ora_threads()

    # -- reduce / scan -------------------------------------------------------------------------
    def reduce(self, x, init, op="plus"):
        """init is a numpy scalar; its dtype is the accumulator / result type."""
        x = np.ascontiguousarray(x)
        init = np.asarray(init)
        out = np.zeros((), dtype=init.dtype)
        rc = self.lib.ora_reduce(_ptr(x), C.c_size_t(x.size), DTYPES[x.dtype], DTYPES[init.dtype],
                                 OPS[op], _ptr(init), _ptr(out))
        if rc != 0:
            raise ValueError("oracle: unsupported reduce types %s -> %s" % (x.dtype, init.dtype))
        return out[()]

    def inclusive_scan(self, x, op="plus", out=None):
        x = np.ascontiguousarray(x)
        out = np.empty_like(x) if out is None else out
        rc = self.lib.ora_inclusive_scan(_ptr(x), _ptr(out), C.c_size_t(x.size), DTYPES[x.dtype],
                                         OPS[op])
        assert rc == 0
        return out

    def exclusive_scan(self, x, init=0, op="plus", out=None):
        x = np.ascontiguousarray(x)
        out = np.empty_like(x) if out is None else out
        i0 = np.asarray(init, dtype=x.dtype)
        rc = self.lib.ora_exclusive_scan(_ptr(x), _ptr(out), C.c_size_t(x.size), DTYPES[x.dtype],
                                         OPS[op], _ptr(i0))
        assert rc == 0
        return out

    def scan_f32_via_f64(self, x, exclusive=False, init=0.0):
        x = np.ascontiguousarray(x, dtype=np.float32)
        out = np.empty_like(x)
        self.lib.ora_scan_f32_via_f64(_ptr(x), _ptr(out), C.c_size_t(x.size), int(exclusive),
                                      C.c_float(init))
        return out

    # -- sort ----------------------------------------------------------------------------------
    def sort_by_key(self, keys, vals=None, descending=False):
        """Stable sort; returns sorted copies (keys, vals)."""
        k = np.array(keys, copy=True)
        v = None if vals is None else np.array(vals, copy=True)
        rc = self.lib.ora_sort_by_key(_ptr(k), _ptr(v), C.c_size_t(k.size), DTYPES[k.dtype],
                                      0 if v is None else v.dtype.itemsize, int(descending))
        assert rc == 0
        return k, v

    def stable_sort_zip_by_first(self, keys, vals):
        k = np.array(keys, dtype=np.uint32, copy=True)
        v = np.array(vals, copy=True)
        assert v.dtype.itemsize == 4
        self.lib.ora_stable_sort_zip_u32_by_first(_ptr(k), _ptr(v), C.c_size_t(k.size))
        return k, v

    # -- compaction ----------------------------------------------------------------------------
    def copy_if(self, x, pred, a=0, b=0, stencil=None):
        x = np.ascontiguousarray(x)
        out = np.empty_like(x)
        st = None if stencil is None else np.ascontiguousarray(stencil)
        n = self.lib.ora_copy_if(_ptr(x), _ptr(st), _ptr(out), C.c_size_t(x.size), DTYPES[x.dtype],
                                 0 if st is None else DTYPES[st.dtype], PREDS[pred],
                                 C.c_int64(a), C.c_int64(b))
        assert n >= 0
        return out[:n].copy()

    def partition(self, x, pred, a=0, b=0):
        d = np.array(x, copy=True)
        n = self.lib.ora_partition(_ptr(d), C.c_size_t(d.size), DTYPES[d.dtype], PREDS[pred],
                                   C.c_int64(a), C.c_int64(b))
        return d, int(n)

    def stable_partition(self, x, pred, a=0, b=0):
        d = np.array(x, copy=True)
        n = self.lib.ora_stable_partition(_ptr(d), C.c_size_t(d.size), DTYPES[d.dtype],
                                          PREDS[pred], C.c_int64(a), C.c_int64(b))
        return d, int(n)

    def partition_copy(self, x, pred, a=0, b=0):
        x = np.ascontiguousarray(x)
        ot = np.empty_like(x)
        of = np.empty_like(x)
        n = self.lib.ora_partition_copy(_ptr(x), _ptr(ot), _ptr(of), C.c_size_t(x.size),
                                        DTYPES[x.dtype], PREDS[pred], C.c_int64(a), C.c_int64(b))
        return ot[:n].copy(), of[:x.size - n].copy()

    def unique_copy(self, x):
        x = np.ascontiguousarray(x)
        out = np.empty_like(x)
        n = self.lib.ora_unique_copy(_ptr(x), _ptr(out), C.c_size_t(x.size), DTYPES[x.dtype])
        return out[:n].copy()

    def reduce_by_key(self, keys, vals, op="plus"):
        k = np.ascontiguousarray(keys)
        v = np.ascontiguousarray(vals)
        ko = np.empty_like(k)
        vo = np.empty_like(v)
        n = self.lib.ora_reduce_by_key(_ptr(k), _ptr(v), _ptr(ko), _ptr(vo), C.c_size_t(k.size),
                                       DTYPES[k.dtype], DTYPES[v.dtype], OPS[op])
        assert n >= 0
        return ko[:n].copy(), vo[:n].copy()

    def reduce_by_key_f32_via_f64(self, keys, vals):
        k = np.ascontiguousarray(keys)
        v = np.ascontiguousarray(vals, dtype=np.float32)
        ko = np.empty_like(k)
        vo = np.empty_like(v)
        n = self.lib.ora_reduce_by_key_f32_via_f64(_ptr(k), _ptr(v), _ptr(ko), _ptr(vo),
                                                   C.c_size_t(k.size), DTYPES[k.dtype])
        return ko[:n].copy(), vo[:n].copy()

    def scan_by_key(self, keys, vals, op="plus", exclusive=False, init=0):
        k = np.ascontiguousarray(keys)
        v = np.ascontiguousarray(vals)
        out = np.empty_like(v)
        i0 = np.asarray(init, dtype=v.dtype)
        rc = self.lib.ora_scan_by_key(_ptr(k), _ptr(v), _ptr(out), C.c_size_t(k.size), DTYPES[k.dtype], DTYPES[v.dtype], OPS[op],
                                      int(exclusive), _ptr(i0))
        assert rc == 0
        return out

    def unique_by_key_copy(self, keys, vals):
        k = np.ascontiguousarray(keys)
        v = np.ascontiguousarray(vals)
        ko = np.empty_like(k)
        vo = np.empty_like(v)
        n = self.lib.ora_unique_by_key_copy(_ptr(k), _ptr(v), _ptr(ko), _ptr(vo), C.c_size_t(k.size), DTYPES[k.dtype], v.dtype.itemsize)
        assert n >= 0
        return ko[:n].copy(), vo[:n].copy()

    # -- extrema -------------------------------------------------------------------------------
    def minmax_element(self, x):
        """(position of the first smallest element, position of the first largest)."""
        x = np.ascontiguousarray(x)
        idx = np.zeros(2, dtype=np.uint64)
        rc = self.lib.ora_minmax_element(_ptr(x), C.c_size_t(x.size), DTYPES[x.dtype], _ptr(idx))
        assert rc == 0
        return int(idx[0]), int(idx[1])

    # -- merge ---------------------------------------------------------------------------------
    def merge_by_key(self, ka, kb, va=None, vb=None, descending=False):
        ka = np.ascontiguousarray(ka)
        kb = np.ascontiguousarray(kb)
        assert ka.dtype == kb.dtype
        ko = np.empty(ka.size + kb.size, dtype=ka.dtype)
        vo = None
        vbytes = 0
        if va is not None:
            va = np.ascontiguousarray(va)
            vb = np.ascontiguousarray(vb)
            vo = np.empty(ka.size + kb.size, dtype=va.dtype)
            vbytes = va.dtype.itemsize
        rc = self.lib.ora_merge_by_key(_ptr(ka), _ptr(va), C.c_size_t(ka.size), _ptr(kb), _ptr(vb),
                                       C.c_size_t(kb.size), _ptr(ko), _ptr(vo), DTYPES[ka.dtype],
                                       vbytes, int(descending))
        assert rc == 0
        return ko, vo


def load_port():
    if not os.path.isfile(PORT_SO):
        build(("port",))
    return Oracle(PORT_SO)


def load_ref():
    """The reference-built oracle, or None when it has not been built and cannot be."""
    if not os.path.isfile(REF_SO):
        try:
            build(("ref",))
        except Exception:
            return None
    return Oracle(REF_SO) if os.path.isfile(REF_SO) else None


def load_best():
    """The reference-built oracle when present, else the port."""
    return load_ref() or load_port()
