"""Names a jit-decorated function body may use (python/parpy/operators.py).
When such a function runs un-jitted in the interpreter they evaluate with
NumPy, which is how the reference's tests build expected values
(test/test_reduce.py:72-85); the native kernels never call them.
"""
from builtins import abs  # noqa: F401
import contextlib

import numpy as np
from numpy import cos, exp, inf, log, sin, sqrt, tanh  # noqa: F401
from numpy import arctan2 as atan2  # noqa: F401

gpu = contextlib.nullcontext()


def min(x, y=None, axis=None):
    if y is None:
        return np.min(x) if axis is None else np.min(x, axis=axis)
    assert axis is None
    return np.minimum(x, y)


def max(x, y=None, axis=None):
    if y is None:
        return np.max(x) if axis is None else np.max(x, axis=axis)
    assert axis is None
    return np.maximum(x, y)


def sum(x, axis=None):
    return np.sum(x) if axis is None else np.sum(x, axis=axis)


def prod(x, axis=None):
    return np.prod(x) if axis is None else np.prod(x, axis=axis)


def _as_float(x):
    return float(x)


def _as_int(x):
    return int(x)


float16 = float32 = float64 = _as_float
int8 = int16 = int32 = int64 = _as_int
uint8 = uint16 = uint32 = uint64 = _as_int


def label(x):
    assert x is not None, "parpy.label expects one argument"
