"""The reference's OWN unit tests on this library's kernels.

oracle/ref_tests/Makefile compiles testing/<name>.cu of the reference (Thrust 1.14.0) -- its
reduce, scan, sort, sort_by_key, stable_sort(_by_key), copy (copy_if), partition, unique,
reduce_by_key, merge, merge_by_key tests and those of their callers (count, inner_product,
transform_reduce, transform_scan, remove, extrema, scan_by_key, unique_by_key) and the set
operations -- against the CUDA
toolkit's Thrust with include/thrust_b200/thrust_overlay.cuh force-included, one executable each.
The executables are built where the reference checkout is available and shipped as files; this
test runs them and requires (1) exit code 0, i.e. every test case of the file passed, and (2) that
the overlay served calls, i.e. the cases ran on this library's kernels and not on the stock ones."""
import os
import re
import subprocess

import pytest

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
BIN = os.path.join(ROOT, "oracle", "_ref", "tests")
NAMES = ["reduce", "scan", "sort", "sort_by_key", "stable_sort", "stable_sort_by_key", "copy", "partition", "unique", "reduce_by_key",
         "merge", "merge_by_key", "count", "inner_product", "transform_reduce", "transform_scan", "remove", "min_element", "max_element",
         "minmax_element", "scan_by_key", "unique_by_key", "set_union", "set_union_by_key", "set_intersection", "set_intersection_by_key",
         "set_difference", "set_difference_by_key", "set_symmetric_difference", "set_symmetric_difference_by_key", "set_union_descending",
         "set_intersection_descending"]


@pytest.mark.parametrize("name", NAMES)
def test_reference_unit_tests_pass_on_the_overlay(tb, name):
    exe = os.path.join(BIN, name)
    if not os.path.isfile(exe):
        pytest.skip("oracle/_ref/tests/%s is not built (make -C oracle/ref_tests THRUST_REF=<reference checkout>)" % name)
    r = subprocess.run([exe, "--sizes=default"], capture_output=True, text=True, timeout=1500)
    tail = (r.stdout + r.stderr)[-3000:]
    assert r.returncode == 0, tail
    m = re.search(r"thrust_b200 overlay served (\d+) calls", r.stdout)
    assert m and int(m.group(1)) > 0, tail
