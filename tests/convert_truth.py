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


# ---- float8 ("quarter": sign, 3 exponent bits, 4 mantissa bits; type code 0), carried in uint8 arrays ----------
FLOAT8 = 0


def float8_to_float(b):
    """include/types/impl/float8.cpp:8-35, vectorised."""
    b = np.asarray(b, np.uint8).astype(np.uint32)
    sign, e, m = (b >> 7) & 1, (b >> 4) & 7, (b & 0xF) << 19
    out = np.zeros(b.shape, np.uint32)
    special = e == 7
    nan = special & (m != 0)
    out[special] = ((sign << 31) | (0xFF << 23))[special]
    out[nan] = 0x7FFFFFFF
    normal = (e != 0) & ~special
    out[normal] = ((sign << 31) | ((e + 0x7C) << 23) | m)[normal]
    sub = (e == 0) & (m != 0)
    lead = np.zeros(b.shape, np.int64)
    mm = m.astype(np.int64)
    for p in range(19, 23):
        lead[(mm >> p) & 1 == 1] = p
    up = 23 - lead
    subv = (sign.astype(np.int64) << 31) | ((0x7D - up) << 23) | ((mm << up) & 0x7FFFFF)
    out[sub] = subv[sub].astype(np.uint32)
    zero = (e == 0) & (m == 0)
    out[zero] = (sign << 31)[zero]
    return out.view(np.float32)


def float_to_float8(f):
    """include/types/impl/float8.cpp:39-96, vectorised, with the x86 shifter's modulo-32 shift counts."""
    x = np.ascontiguousarray(f, np.float32).view(np.uint32).astype(np.int64)
    u = x & 0x7FFFFFFF
    sign = (x >> 24) & 0x80
    e = (u >> 23) & 0xFF
    m = u & 0x7FFFFF
    big = e > 0x7C
    shift = np.where(big, 19, (0x90 - e) & 31)
    e2 = np.where(big, e - 0x7C, 0)
    m2 = np.where(big, m, m | 0x800000)
    lsb = (np.int64(1) << shift) & 0xFFFFFFFF
    rest = m2 & ((lsb - 1) & 0xFFFFFFFF)
    half = lsb >> 1
    m3 = m2 >> shift
    up = (rest > half) | ((rest == half) & ((m3 & 1) == 1))
    m4 = np.where(up, m3 + 1, m3)
    carry = up & ((m4 & 0xF) == 0)
    e3 = np.where(carry, e2 + 1, e2)
    m5 = np.where(carry, 0, m4)
    out = (sign | (e3 << 4) | m5) & 0xFF
    out = np.where(u < 0x33000001, sign, out)
    out = np.where(u > 0x477FEFFF, sign | 0x70, out)
    out = np.where(u > 0x7F800000, 0x7F, out)
    return out.astype(np.uint8)


def float8_inputs():
    """Every float8 bit pattern, several times over so that vector and scalar code paths both see all of them."""
    return np.tile(np.arange(256, dtype=np.uint8), 5)[:1277]


def convert_truth_from_float8(x, dst):
    return convert_truth(float8_to_float(x), dst)


def convert_truth_to_float8(x):
    with np.errstate(over="ignore"):
        return float_to_float8(x.astype(np.float32))
