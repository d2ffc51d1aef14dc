"""Expected results of NativeOps::convertTypes restated in numpy (include/loops/type_conversions.h:592-610,
696-880 and the saturating integer wrappers of include/types/impl/). tests/test_oracle.py pins this
restatement against the reference compiled in place; the GPU tests compare the CUDA path with it."""
import numpy as np

CODES = {np.int8: 1, np.uint8: 2, np.float16: 3, np.int16: 4, np.uint16: 5, np.float32: 6, np.float64: 7}


def _x86_int(f):
    """(int) of a float as the reference's x86 build does it: truncation, INT_MIN outside int32 and for NaN."""
    f = f.astype(np.float32)
    bad = ~(f < np.float32(2147483648.0)) | (f < np.float32(-2147483648.0))
    with np.errstate(invalid="ignore"):
        t = np.where(bad, 0, np.trunc(np.where(bad, 0, f))).astype(np.int64)
    return np.where(bad, -2 ** 31, t)


def convert_truth(x, dst):
    """z = (D)(float) x with the reference's saturating integer wrappers (include/types/impl/*.cpp)."""
    with np.errstate(over="ignore"):
        f = x.astype(np.float32)
        if dst in (np.float16, np.float32, np.float64):
            return f.astype(dst)
    t = _x86_int(f)
    if dst == np.int8:
        return np.clip(t, -128, 127).astype(np.int8)
    if dst == np.uint8:
        return np.clip(t, 0, 255).astype(np.uint8)
    if dst == np.int16:
        return np.clip(t, -32768, 32767).astype(np.int16)
    # uint16: clamped to 65536, then returned through a uint8_t (uint16.cpp:13-19): the low byte survives
    return (np.clip(t, 0, 65536) & 0xff).astype(np.uint16)


SOURCES = [np.int8, np.uint8, np.float16, np.int16, np.float32, np.float64]
RESULTS = SOURCES + [np.uint16]


def convert_inputs(src):
    """Seeded inputs that cover every range edge of the result types, NaN and the infinities."""
    rng = np.random.default_rng(1)
    if np.issubdtype(src, np.integer):
        info = np.iinfo(src)
        return np.concatenate([rng.integers(info.min, info.max + 1, 10003), [info.min, info.max, 0, 1]]).astype(src)
    x = np.concatenate([rng.standard_normal(6001) * 100, rng.standard_normal(4000) * 40000,
                        [0.0, -0.0, 65504.0, 70000.0, 1e-7, 6e-8, 1e300, -1e300, 1 / 3, 127.9, -128.9, 255.5, 65535.5,
                         65536.0, 65537.0, 3e9, -3e9, np.nan, np.inf, -np.inf, 0.0]])
    with np.errstate(over="ignore"):
        return x.astype(src)
