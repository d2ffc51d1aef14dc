"""Shared builders for parity cases: seeded inputs, shapeInfo layouts and comparison helpers."""
import numpy as np

from libnd4j_b200 import shape as S

DTYPES = {"f32": np.float32, "f64": np.float64, "f16": np.float16}
SUFFIX = {"f32": "Float", "f64": "Double", "f16": "Half"}


def ulp_distance(a, b):
    """Distance in units in the last place between two float32/float16/float64 arrays."""
    a = np.ascontiguousarray(a)
    b = np.ascontiguousarray(b)
    it = {2: np.int16, 4: np.int32, 8: np.int64}[a.dtype.itemsize]
    ai = a.view(it).astype(np.int64)
    bi = b.view(it).astype(np.int64)
    sign = np.int64(1) << (8 * a.dtype.itemsize - 1)
    ai = np.where(ai < 0, -(ai & (sign - 1)), ai)
    bi = np.where(bi < 0, -(bi & (sign - 1)), bi)
    d = np.abs(ai - bi)
    both_nan = np.isnan(a) & np.isnan(b)
    return np.where(both_nan, 0, d)


class Layout:
    """A logical array placed in a flat buffer: contiguous c/f order or a strided view of a
    larger parent. `buffer` is what goes to the device; `info` is the shapeInfo."""

    def __init__(self, logical, kind="c"):
        logical = np.asarray(logical)
        self.kind = kind
        self.shape = logical.shape
        dt = logical.dtype
        if kind == "c":
            self.buffer = np.ascontiguousarray(logical).ravel()
            self.info = S.shape_info(self.shape, "c")
        elif kind == "f":
            self.buffer = np.asfortranarray(logical).ravel(order="K").copy()
            self.info = S.shape_info(self.shape, "f")
        elif kind == "fview2":
            # every second index of the LAST axis of an f-order parent twice as wide
            pshape = list(self.shape)
            pshape[-1] *= 2
            parent = np.full(pshape, np.nan, dtype=dt, order="F")
            parent[..., ::2] = logical
            self.buffer = parent.ravel(order="K").copy()
            strides = S.default_strides(pshape, "f")
            strides[-1] *= 2
            self.info = S.shape_info(self.shape, "f", strides, ews=-1 if len(self.shape) > 1 else strides[-1])
        elif kind == "cview2":
            # every second index of the LAST axis of a c-order parent twice as wide
            pshape = list(self.shape)
            pshape[-1] *= 2
            parent = np.full(pshape, np.nan, dtype=dt, order="C")
            parent[..., ::2] = logical
            self.buffer = parent.ravel().copy()
            strides = S.default_strides(pshape, "c")
            strides[-1] *= 2
            self.info = S.shape_info(self.shape, "c", strides)
        elif kind == "rowview2":
            # every second index of the FIRST axis of a c-order parent twice as tall
            pshape = list(self.shape)
            pshape[0] *= 2
            parent = np.full(pshape, np.nan, dtype=dt, order="C")
            parent[::2] = logical
            self.buffer = parent.ravel().copy()
            strides = S.default_strides(pshape, "c")
            strides[0] *= 2
            self.info = S.shape_info(self.shape, "c", strides)
        else:
            raise ValueError(kind)

    def read(self, buffer=None):
        """Logical array gathered back out of a (possibly modified) flat buffer."""
        buf = self.buffer if buffer is None else buffer
        strides = S.strides_of(self.info)
        return np.lib.stride_tricks.as_strided(buf, self.shape, [s * buf.dtype.itemsize for s in strides]).copy()


def result_info(x_shape, dims):
    return S.reduced_shape_info(S.shape_info(x_shape), dims)


def rand_input(rng, shape, dtype, kind="normal"):
    if kind == "normal":
        a = rng.standard_normal(shape)
    elif kind == "uniform":
        a = rng.uniform(-1, 1, shape)
    elif kind == "positive":
        a = rng.uniform(0.1, 2.0, shape)
    elif kind == "levels":
        a = (rng.integers(0, 16, shape) / 8.0) - 1.0
    else:
        raise ValueError(kind)
    return a.astype(dtype)
