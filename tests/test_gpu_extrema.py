"""min_element / max_element / minmax_element against the oracle: positions are exact, ties go to the
first occurrence (thrust/system/cuda/detail/extrema.h:48-108)."""
import numpy as np
import pytest

from gpu_util import ALL, EDGE_SIZES, dev, misaligned
from thrust_b200 import datagen as dg

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("n", EDGE_SIZES)
def test_extrema_positions_exact(tb, oracles, n):
    x = dg.compaction_input(n)
    got = tb.minmax_element(dev(x))
    lo, hi = tb.min_element(dev(x)), tb.max_element(dev(x))
    for o in oracles:
        assert got == o.minmax_element(x)
        assert (lo, hi) == o.minmax_element(x)


def test_extrema_known_answers_types_and_ties(tb, port):
    assert tb.minmax_element(dev(np.array([3, 5, 1, 2, 5, 1], np.int32))) == (2, 1)   # testing/minmax_element.cu:8-20
    rng = np.random.default_rng(5)
    for dt in ALL:
        for n in (1, 7, 4099, 300001):
            x = rng.integers(0, 100, n).astype(dt)          # many ties: the first occurrence must win
            assert tb.minmax_element(dev(x)) == port.minmax_element(x), (dt, n)
            y = (rng.standard_normal(n) * 50).astype(dt)
            assert tb.minmax_element(dev(y)) == port.minmax_element(y), (dt, n)
    x = rng.integers(-5, 5, 100001).astype(np.int32)
    for off in (1, 3):
        assert tb.minmax_element(misaligned(x, off)) == port.minmax_element(x)
    const = np.full(1 << 20, 9, np.float32)
    assert tb.minmax_element(dev(const)) == (0, 0)
    const[123457] = -1.0
    const[(1 << 20) - 1] = 10.0
    assert tb.minmax_element(dev(const)) == (123457, (1 << 20) - 1)


def test_extrema_full_size(tb, oracles):
    """2^28 int32 (the reduce configuration's input): the positions match the reference's."""
    n = 1 << 28
    x = dg.reduce_input(n)
    got = tb.minmax_element(dev(x))
    assert got == oracles[-1].minmax_element(x)
