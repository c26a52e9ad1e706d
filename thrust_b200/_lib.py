"""Loads libthrust_b200.so and declares the C-ABI prototypes (include/thrust_b200.h).

There is no fallback: if the library is missing or a symbol is absent this raises, so that a
caller can never silently run anything but the sm_100a kernels.
"""
import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libthrust_b200.so")

_vp, _sz, _i, _ll = C.c_void_p, C.c_size_t, C.c_int, C.c_longlong
_szp = C.POINTER(C.c_size_t)

# name -> argtypes; every function returns int (cudaError_t)
PROTOTYPES = {
    "tb200_version": [],
    "tb200_sm_arch": [],
    "tb200_workspace_status": [_vp, _vp, C.POINTER(C.c_uint)],
    "tb200_reduce": [_vp, _sz, _i, _i, _i, _vp, _vp, _vp, _szp, _vp],
    "tb200_inclusive_scan": [_vp, _vp, _sz, _i, _i, _vp, _vp, _szp, _vp],
    "tb200_exclusive_scan": [_vp, _vp, _sz, _i, _i, _vp, _vp, _szp, _vp],
    "tb200_inclusive_scan_dinit": [_vp, _vp, _sz, _i, _i, _vp, _vp, _szp, _vp],
    "tb200_exclusive_scan_dinit": [_vp, _vp, _sz, _i, _i, _vp, _vp, _szp, _vp],
    "tb200_sort_by_key": [_vp, _vp, _vp, _vp, _sz, _i, _i, _i, _i, _i, _vp, _szp, _vp],
    "tb200_copy_if": [_vp, _vp, _vp, _sz, _i, _i, _i, _ll, _ll, _vp, _vp, _szp, _vp],
    "tb200_partition_copy": [_vp, _vp, _vp, _vp, _sz, _i, _i, _i, _ll, _ll, _vp, _vp, _szp, _vp],
    "tb200_partition": [_vp, _sz, _i, _i, _ll, _ll, _vp, _vp, _szp, _vp],
    "tb200_unique_copy": [_vp, _vp, _sz, _i, _vp, _vp, _szp, _vp],
    "tb200_reduce_by_key": [_vp, _vp, _vp, _vp, _sz, _i, _i, _i, _vp, _vp, _szp, _vp],
    "tb200_scan_by_key": [_vp, _vp, _vp, _sz, _i, _i, _i, _i, _vp, _vp, _szp, _vp],
    "tb200_unique_by_key_copy": [_vp, _vp, _vp, _vp, _sz, _i, _i, _vp, _vp, _szp, _vp],
    "tb200_min_element": [_vp, _sz, _i, _vp, _vp, _szp, _vp],
    "tb200_max_element": [_vp, _sz, _i, _vp, _vp, _szp, _vp],
    "tb200_minmax_element": [_vp, _sz, _i, _vp, _vp, _szp, _vp],
    "tb200_merge_by_key": [_vp, _vp, _sz, _vp, _vp, _sz, _vp, _vp, _i, _i, _i, _vp, _szp, _vp],
    "tb200_merge_sort_by_key": [_vp, _vp, _vp, _vp, _sz, _i, _i, _i, _vp, _szp, _vp],
    "tb200_merge_runs": [_vp, _vp, _vp, _i, _vp, _vp, _vp, _vp, _i, _i, _i, _vp, _szp, _vp],
    "tb200_bucket_count": [_vp, _sz, _i, _i, _vp, _i, _vp, _vp],
    "tb200_bucket_scatter": [_vp, _vp, _sz, _i, _i, _i, _vp, _i, _vp, _vp, _vp, _vp, _szp, _vp],
    "tb200_set_operation": [_i, _vp, _sz, _vp, _sz, _vp, _vp, _vp, _vp, _i, _i, _i, _vp, _vp, _szp, _vp],
    "tb200_exchange_sizes": [_i, _szp, _szp, _szp],
    "tb200_exchange_hist": [_vp, _sz, _i, _i, C.c_ulonglong, _vp, _vp],
    "tb200_exchange_plan": [_vp, _i, _i, _i, _vp, _vp],
    "tb200_exchange_scatter": [_vp, _vp, _sz, _i, _i, _i, _vp, _i, _vp, _vp, _vp, _szp, _vp],
    "tb200_lower_bound": [_vp, _sz, _vp, _sz, _vp, _i, _i, _vp],
    "tb200_inclusive_scan_static": [_vp, _vp, _sz, _i, _i, _vp, _vp],
    "tb200_inclusive_scan_static_limit": [_i, _szp],
    "tb200_inclusive_scan_static_status": [_vp, C.POINTER(C.c_uint)],
    "tb200_ipc_export": [_vp, _vp, _szp],
    "tb200_ipc_open": [_vp, _sz, C.POINTER(C.c_void_p)],
    "tb200_ipc_close": [_vp],
    "tb200_ipc_close_all": [],
    "tb200_sequence_u32": [_vp, _sz, _vp],
    "tb200_gather": [_vp, _vp, _vp, _sz, _i, _vp],
    "tb200_kernel_timing": [_i],
    "tb200_kernel_timing_read": [_i, C.POINTER(C.c_int), C.POINTER(C.c_float), C.POINTER(C.c_int)],
}

_lib = None


def load_partial(path):
    """A ctypes handle of another build of the library that exports only some of the entry points
    (the short-wait test build): prototypes are declared for the symbols it has."""
    lib = C.CDLL(path)
    for name, args in PROTOTYPES.items():
        fn = getattr(lib, name, None)
        if fn is not None:
            fn.argtypes = args
            fn.restype = C.c_int
    return lib


def load():
    """Returns the ctypes handle, loading the library on first use."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.isfile(LIB_PATH):
        raise RuntimeError(
            "thrust_b200: %s is missing -- build it with `python -m thrust_b200.build`; "
            "there is no CPU or library fallback" % LIB_PATH)
    lib = C.CDLL(LIB_PATH)
    for name, args in PROTOTYPES.items():
        fn = getattr(lib, name)  # AttributeError if the symbol is not exported
        fn.argtypes = args
        fn.restype = C.c_int
    _lib = lib
    return lib
