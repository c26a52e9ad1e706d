"""thrust_b200: a B200-native (sm_100a) backend for Thrust's core parallel algorithms.

The product is the C-ABI library libthrust_b200.so (include/thrust_b200.h) and the Thrust header
overlay under include/thrust/; this package is the Python host layer over the C ABI that the
tests and the benchmark drive.
"""
from . import _lib  # noqa: F401
from .api import *  # noqa: F401,F403
from .api import Tb200Error, workspaces  # noqa: F401
