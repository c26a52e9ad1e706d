"""Seeded synthetic inputs for the benchmark configurations (numpy, counter based).

u(seed, i) = mix64(i + (seed + 1) * 0x9E3779B97F4A7C15), mix64 being the splitmix64 finaliser, so
element i of any stream can be produced anywhere (host, any GPU shard) without shipping data.
The workload shapes and value ranges are the ones the benchmark configurations name; no external
dataset is involved.
"""
import numpy as np

_GOLDEN = 0x9E3779B97F4A7C15
_M1 = np.uint64(0xBF58476D1CE4E5B9)
_M2 = np.uint64(0x94D049BB133111EB)


def rand64(seed, n, start=0):
    """n 64-bit values of stream `seed`, starting at counter `start`."""
    with np.errstate(over="ignore"):
        z = np.arange(start, start + n, dtype=np.uint64) + np.uint64(((seed + 1) * _GOLDEN) & 0xFFFFFFFFFFFFFFFF)
        z = (z ^ (z >> np.uint64(30))) * _M1
        z = (z ^ (z >> np.uint64(27))) * _M2
        return z ^ (z >> np.uint64(31))


def rand64_at(seed, idx):
    """The 64-bit values of stream `seed` at the counters in `idx` (any integer array)."""
    with np.errstate(over="ignore"):
        z = np.asarray(idx).astype(np.uint64) + np.uint64(((seed + 1) * _GOLDEN) & 0xFFFFFFFFFFFFFFFF)
        z = (z ^ (z >> np.uint64(30))) * _M1
        z = (z ^ (z >> np.uint64(27))) * _M2
        return z ^ (z >> np.uint64(31))


def reduce_input(n, seed=0, start=0):
    """config 1: int32 uniform in [-2^20, 2^20)."""
    return ((rand64(seed, n, start) >> np.uint64(43)).astype(np.int64) - (1 << 20)).astype(np.int32)


def scan_input_i32(n, seed=1, start=0):
    """config 2a: int32 uniform in [0, 16)."""
    return (rand64(seed, n, start) >> np.uint64(60)).astype(np.int32)


def scan_input_f32(n, seed=1, start=0):
    """config 2b: fp32 uniform in [0, 1) with 24 random mantissa bits."""
    return ((rand64(seed, n, start) >> np.uint64(40)).astype(np.float32) * np.float32(2.0 ** -24))


def sort_keys_u32(n, seed=2, start=0):
    """config 3a: uniform random 32-bit keys (values are the original index)."""
    return (rand64(seed, n, start) >> np.uint64(32)).astype(np.uint32)


def sort_keys_u32_at(idx, seed=2):
    """config 3a: the keys at the given original indices."""
    return (rand64_at(seed, idx) >> np.uint64(32)).astype(np.uint32)


def sort_keys_u64_40bit(n, seed=2, start=0):
    """config 3b: uint64 keys with only the low 40 bits random."""
    return rand64(seed, n, start) >> np.uint64(24)


def compaction_input(n, seed=3, start=0):
    """config 4a/4b: int32 uniform in [0, 2^31); the predicate is x % 2 == 0."""
    return (rand64(seed, n, start) >> np.uint64(33)).astype(np.int32)


def run_keys(n, seed=3):
    """config 4c/4d: sorted int32 keys whose run lengths are geometric with mean 4: a new run
    starts at each position with probability 1/4, the key is the run index."""
    heads = (rand64(seed + 100, n) >> np.uint64(62)) == 0
    if n:
        heads[0] = True
    return (np.cumsum(heads, dtype=np.int64) - 1).astype(np.int32)


def run_values_f32(n, seed=3):
    """config 4d: fp32 values uniform in [0, 1)."""
    return scan_input_f32(n, seed + 200)


def merge_keys_u64(n, seed):
    """config 5a: uint64 uniform in [0, 2^48), sorted ascending (seeds 4 and 5)."""
    k = rand64(seed, n) >> np.uint64(16)
    k.sort(kind="stable")
    return k


def zip_sort_input(n, seed=6):
    """config 5b: (uint32 random key, fp32 value in [0, 1)) pairs."""
    return sort_keys_u32(n, seed), scan_input_f32(n, seed + 300)
