"""Builds libthrust_b200.so (the C-ABI library of sm_100a kernels) in-tree with nvcc.

    python -m thrust_b200.build [--force]

Every csrc/*.cu is compiled to an object for sm_100a (-gencode arch=compute_100a,code=sm_100a
-lineinfo) and linked into thrust_b200/libthrust_b200.so.  Objects are rebuilt only when the
source or a header is newer.  nvcc cross-compiles, so no GPU is needed to build.
"""
import concurrent.futures as cf
import glob
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
CSRC = os.path.join(HERE, "csrc")
INCLUDE = os.path.join(ROOT, "include")
OBJ_DIR = os.path.join(HERE, "build")
LIB = os.path.join(HERE, "libthrust_b200.so")

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-I" + INCLUDE, "-I" + CSRC, "-Xcompiler", "-fPIC,-fvisibility=hidden", "--expt-relaxed-constexpr",
]


def _nvcc():
    for cand in (os.environ.get("NVCC"), "/usr/local/cuda/bin/nvcc", "nvcc"):
        if cand and (os.path.sep not in cand or os.path.isfile(cand)):
            return cand
    return "nvcc"


def _newest_header():
    hdrs = glob.glob(os.path.join(INCLUDE, "**", "*.*h"), recursive=True) + glob.glob(os.path.join(CSRC, "*.cuh"))
    return max(os.path.getmtime(h) for h in hdrs)


def _compile(src, obj):
    cmd = [_nvcc()] + NVCC_FLAGS + ["-c", src, "-o", obj]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError("nvcc failed for %s:\n%s\n%s" % (src, r.stdout, r.stderr))
    return obj


def build(force=False, verbose=False):
    os.makedirs(OBJ_DIR, exist_ok=True)
    srcs = sorted(glob.glob(os.path.join(CSRC, "*.cu")))
    hdr_time = _newest_header()
    jobs, objs = [], []
    for s in srcs:
        o = os.path.join(OBJ_DIR, os.path.basename(s)[:-3] + ".o")
        objs.append(o)
        if force or not os.path.isfile(o) or os.path.getmtime(o) < max(os.path.getmtime(s), hdr_time):
            jobs.append((s, o))
    if jobs:
        if verbose:
            print("compiling", [os.path.basename(s) for s, _ in jobs], file=sys.stderr)
        with cf.ThreadPoolExecutor(max_workers=min(8, len(jobs))) as ex:
            list(ex.map(lambda so: _compile(*so), jobs))
    if jobs or not os.path.isfile(LIB):
        cmd = [_nvcc(), "-shared", "-o", LIB] + objs + ["-lcudart"]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError("link failed:\n%s\n%s" % (r.stdout, r.stderr))
    return LIB


SHORTWAIT_LIB = os.path.join(HERE, "libthrust_b200_shortwait.so")
SHORTWAIT_SOURCES = ["abi_scan.cu", "abi_reduce.cu", "abi_util.cu"]
SHORTWAIT_FLAGS = ["-DTB200_SPIN_LIMIT=64", "-DTB200_TEST_HOOKS"]


def build_shortwait(force=False):
    """A TEST build of the scan entry points: the bound on every inter-CTA wait is 64 polls instead
    of 2^23, and tb200_test_hooks(1) makes the first tile of a single-pass scan withhold its
    descriptor.  tests/test_gpu_failure_path.py uses it to show that a wait that runs out makes the
    kernel RETURN with the status word set, which the host turns into an exception.  Nothing else
    loads this library."""
    obj_dir = os.path.join(OBJ_DIR, "shortwait")
    os.makedirs(obj_dir, exist_ok=True)
    hdr_time = _newest_header()
    objs, stale = [], False
    for name in SHORTWAIT_SOURCES:
        src = os.path.join(CSRC, name)
        obj = os.path.join(obj_dir, name[:-3] + ".o")
        objs.append(obj)
        if force or not os.path.isfile(obj) or os.path.getmtime(obj) < max(os.path.getmtime(src), hdr_time):
            cmd = [_nvcc()] + NVCC_FLAGS + SHORTWAIT_FLAGS + ["-c", src, "-o", obj]
            r = subprocess.run(cmd, capture_output=True, text=True)
            if r.returncode != 0:
                raise RuntimeError("nvcc failed for %s:\n%s\n%s" % (src, r.stdout, r.stderr))
            stale = True
    if stale or not os.path.isfile(SHORTWAIT_LIB):
        r = subprocess.run([_nvcc(), "-shared", "-o", SHORTWAIT_LIB] + objs + ["-lcudart"], capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError("link failed:\n%s\n%s" % (r.stdout, r.stderr))
    return SHORTWAIT_LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose=True))
    print(build_shortwait(force="--force" in sys.argv))
