"""GPU parity of the elementwise families (transform, pairwise, scalar, broadcast,
scalar-along-dimension) against the reference's CPU loops, called through the C ABI.

Tolerances: +, -, *, / and comparisons must be bit-exact (the library is built without FMA
contraction); functions that go through libm (tanh, exp, pow, ...) must stay within 2 ulp in
float32, the bound stated for fp32 transforms. float16 results may differ by one half-ulp more
because the reference rounds to half after every operation while the GPU rounds once.
"""
import numpy as np
import pytest
import torch

from libnd4j_b200 import shape as S
from tests.cases import Layout, rand_input, ulp_distance

pytestmark = pytest.mark.gpu


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def host(t):
    return t.cpu().numpy()


# opNum -> (input kind, extra params) for every elementwise transform functor
TRANSFORMS = {
    0: ("normal", None), 1: ("normal", None), 2: ("normal", None), 3: ("normal", None), 4: ("normal", None),
    5: ("positive", None), 6: ("normal", None), 7: ("positive", [2.5]), 8: ("normal", None),
    9: ("normal", [0.0, 1.0]), 10: ("normal", None), 11: ("normal", None), 12: ("normal", None),
    13: ("normal", None), 14: ("positive", None), 15: ("normal", None), 16: ("uniform", None),
    17: ("uniform", None), 18: ("normal", None), 19: ("normal", None), 20: ("normal", None), 21: ("normal", None),
    22: ("normal", None), 23: ("normal", None), 24: ("normal", None), 25: ("normal", None), 26: ("normal", None),
    27: ("normal", None), 28: ("normal", [2.0]), 29: ("normal", None), 30: ("normal", None), 31: ("normal", [0.01]),
    32: ("normal", [0.01]), 33: ("normal", [0.0]), 34: ("normal", [0.1]), 35: ("normal", None), 42: ("normal", None),
    45: ("levels", [0.25, 7.0, 1e-5, 0.0]), 46: ("normal", [3.0]), 47: ("normal", None), 49: ("normal", None),
    50: ("normal", None), 51: ("normal", None), 52: ("normal", None), 53: ("normal", None), 54: ("normal", None),
    55: ("positive", [3.0]), 59: ("levels", [0.25]), 61: ("normal", None), 62: ("normal", None), 63: ("normal", None),
    64: ("normal", None), 65: ("uniform", None), 66: ("uniform", None), 67: ("normal", None), 68: ("normal", None),
    72: ("levels", [0.25, 1e-5, 2.0]), 73: ("normal", [-0.5, 0.5]), 74: ("normal", None), 75: ("normal", None),
    76: ("positive", None), 77: ("positive", None), 78: ("normal", None), 79: ("normal", None), 80: ("normal", None),
    81: ("normal", None), 82: ("positive+1", None), 83: ("positive+1", None), 84: ("normal", None),
    85: ("normal", None), 86: ("normal", None), 87: ("normal", None), 88: ("normal", None), 89: ("normal", None),
    90: ("normal", None), 91: ("normal", None), 92: ("positive", [2.5]), 93: ("uniform*0.9", None),
    94: ("positive", None), 95: ("normal", None), 96: ("normal", [0.0]),
}
# functions computed through libm on the host and the CUDA math library on the device
LIBM = {2, 3, 5, 7, 10, 12, 13, 15, 16, 17, 18, 21, 22, 23, 29, 53, 54, 55, 61, 62, 63, 64, 65, 66, 67, 68, 74, 75,
        77, 78, 82, 84, 85, 86, 88, 89, 90, 91, 92, 93, 9}
# Formulas that subtract nearly equal intermediates (exp(x) - 1 near 0, 1 - tanh^2, log(1 + e^x),
# 1 - 1/(1 + ...)) turn a last-ulp difference of exp/log/tanh between the two math libraries into
# many ulps of a tiny result. For those the distance is measured in ulps of max(|result|, floor),
# floor being the magnitude of the intermediate that is being cancelled: op -> (ulps, floor).
CANCELLING = {13: (4, 1.0), 21: (2, 1.0), 22: (2, 0.0), 23: (4, 1.0), 29: (4, 0.25), 53: (4, 1.7159), 54: (8, 1.0),
              61: (2, 0.0), 62: (4, 1.0), 67: (4, 1.7581), 68: (4, 0.0), 75: (8, 1.0), 88: (4, 1.0), 91: (2, 1.0),
              84: (4, 1.0), 85: (4, 0.0), 66: (8, 0.0), 77: (2, 1.0), 74: (4, 0.0), 89: (4, 0.0), 10: (2, 0.0),
              7: (4, 0.0), 92: (8, 0.0), 55: (4, 0.0), 63: (4, 0.0), 64: (4, 0.0), 65: (4, 0.0), 90: (8, 0.0),
              82: (4, 0.0), 93: (4, 0.0),
              # 3*x*x: the reference's associative-math build groups the product differently in its
              # single-thread and OpenMP code paths, so either grouping is two roundings away at most
              50: (2, 0.0)}


def ulps_at(got, want, floor):
    """|got - want| in units of the float32 spacing at max(|want|, floor)."""
    scale = np.maximum(np.abs(want.astype(np.float64)), floor).astype(np.float32)
    return np.abs(got.astype(np.float64) - want.astype(np.float64)) / np.spacing(scale).astype(np.float64)


def make_input(rng, kind, n, dtype):
    if kind == "positive+1":
        return (rand_input(rng, n, np.float64, "positive") + 1.0).astype(dtype)
    if kind == "uniform*0.9":
        return (rand_input(rng, n, np.float64, "uniform") * 0.9).astype(dtype)
    return rand_input(rng, n, dtype, kind)


@pytest.mark.parametrize("op", sorted(TRANSFORMS))
def test_transform_float_all_ops(ops, real_ref, op):
    kind, extra = TRANSFORMS[op]
    rng = np.random.default_rng(100 + op)
    n = 40003  # ragged: not a multiple of the 128-bit pack
    x = make_input(rng, kind, n, np.float32)
    if op in (79, 80, 81, 46):
        x[::7] = np.nan
        x[3::11] = np.inf
    info = S.shape_info([1, n])
    ex = None if extra is None else np.array(extra, dtype=np.float32)
    want = real_ref.transform(op, x, info, np.empty_like(x), info, ex)
    dz = torch.empty(n, device="cuda")
    ops.execTransformFloat(None, op, dev(x), info, dz, info, None if ex is None else dev(ex))
    got = host(dz)
    assert np.array_equal(np.isnan(got), np.isnan(want))
    assert np.array_equal(np.isinf(got), np.isinf(want))
    finite = np.isfinite(want)
    limit, floor = CANCELLING.get(op, (2 if op in LIBM else 0, 0.0))
    d = ulps_at(got[finite], want[finite], floor) if floor > 0 else ulp_distance(got[finite], want[finite])
    assert d.max(initial=0) <= limit, "op %d: max ulp %g (limit %d at floor %g)" % (op, d.max(), limit, floor)


@pytest.mark.parametrize("dt,name", [(np.float64, "Double"), (np.float16, "Half")])
@pytest.mark.parametrize("op", [0, 3, 10, 15, 19, 33, 51, 73, 94, 95])
def test_transform_other_types(ops, real_ref, dt, name, op):
    kind, extra = TRANSFORMS[op]
    rng = np.random.default_rng(7 + op)
    n = 8191
    x = make_input(rng, kind, n, dt)
    info = S.shape_info([n])
    ex = None if extra is None else np.array(extra, dtype=dt)
    want = real_ref.transform(op, x, info, np.empty_like(x), info, ex)
    dz = dev(np.zeros(n, dt))
    getattr(ops, "execTransform" + name)(None, op, dev(x), info, dz, info, None if ex is None else dev(ex))
    if dt == np.float16 and op == 51:
        # HardSigmoid: the reference rounds the constant 0.2 and every intermediate to half, the
        # GPU rounds once at the end; near the zero crossing that is many ulps of a tiny result
        # but at most two half-ulps of the intermediates (magnitude 0.5)
        assert np.abs(host(dz).astype(np.float64) - want.astype(np.float64)).max() <= 2 * 2.0 ** -11
        return
    d = ulp_distance(host(dz), want)
    # the reference rounds to half after every operation of a composite functor, the GPU once
    assert d.max() <= (3 if dt == np.float16 else 2), d.max()


def test_transform_tanh_dense_sweep(ops, real_ref):
    """Tanh over 4M inputs spread across the whole active range: <= 2 ulp from the host libm."""
    rng = np.random.default_rng(5)
    x = np.concatenate([rng.standard_normal(1 << 21) * 1.5, rng.uniform(-12, 12, 1 << 20),
                        rng.uniform(-0.6, 0.6, 1 << 20)]).astype(np.float32)
    info = S.shape_info([1, x.size])
    want = real_ref.transform(15, x, info, np.empty_like(x), info)
    dz = torch.empty(x.size, device="cuda")
    ops.execTransformFloat(None, 15, dev(x), info, dz, info, None)
    d = ulp_distance(host(dz), want)
    assert d.max() <= 2, np.bincount(d)[:6]


@pytest.mark.parametrize("xk,zk", [("c", "c"), ("f", "f"), ("c", "f"), ("cview2", "c"), ("fview2", "fview2"),
                                    ("rowview2", "cview2")])
@pytest.mark.parametrize("shape", [(37, 53), (5, 7, 11), (3, 4, 5, 6)])
def test_transform_layouts(ops, real_ref, xk, zk, shape):
    rng = np.random.default_rng(3)
    lx = Layout(rand_input(rng, shape, np.float32), xk)
    lz = Layout(np.zeros(shape, np.float32), zk)
    zb = lz.buffer.copy()
    real_ref.transform(6, lx.buffer, lx.info, zb, lz.info)  # Neg
    dz = dev(lz.buffer)
    ops.execTransformFloat(None, 6, dev(lx.buffer), lx.info, dz, lz.info, None)
    np.testing.assert_array_equal(lz.read(host(dz)), -lx.read())
    np.testing.assert_array_equal(lz.read(host(dz)), lz.read(zb))


def test_transform_in_place_and_strided_overload(ops):
    x = np.arange(1, 1025, dtype=np.float32)
    d = dev(x)
    info = S.shape_info([1, 1024])
    ops.execTransformFloat(None, 95, d, info, d, info, None)  # Sqr in place
    np.testing.assert_array_equal(host(d), x * x)
    src = dev(np.arange(64, dtype=np.float32))
    dst = torch.zeros(32, device="cuda")
    ops.execTransformFloat(None, 6, src, 2, dst, 1, None, 32)  # (x, xStride, z, zStride, extra, n)
    np.testing.assert_array_equal(host(dst), -np.arange(0, 64, 2, dtype=np.float32))


PAIRWISE = {0: None, 1: None, 2: None, 3: None, 4: None, 5: None, 6: None, 7: None, 8: None, 9: None, 10: None,
            11: None, 12: None, 13: None, 14: None, 15: None, 16: None, 17: [0.75], 18: None,
            45: [0.25, 0.0, 1e-5, 0.0], 46: [0.25, 0.0, 1e-5, 3.0], 56: [0.0], 57: [0.0], 58: [0.0], 59: None,
            60: None, 69: None, 19: None, 20: None, 21: None, 22: None, 23: None, 24: None, 25: None, 26: None,
            27: [0.1], 28: [0.1, 0.05], 92: None, 93: None, 94: None}
PAIRWISE_LIBM = {7: 4, 69: 2, 92: 8, 22: 0, 59: 0, 60: 0, 21: 0}
# exp(y) - x*y cancels: measured in ulps of the larger intermediate
PAIRWISE_FLOOR = {93, 94}


@pytest.mark.parametrize("op", sorted(PAIRWISE))
def test_pairwise_float_all_ops(ops, real_ref, op):
    rng = np.random.default_rng(200 + op)
    n = 30011
    positive = op in (7, 92, 94)
    x = rand_input(rng, n, np.float32, "positive" if positive else "levels" if op in (3, 15, 45, 46, 56, 57, 58) else "normal")
    y = rand_input(rng, n, np.float32, "positive" if positive else "levels" if op in (3, 15, 45, 46, 56, 57, 58) else "normal")
    if op in (19, 23, 25):
        x = np.round(x * 10).astype(np.float32)
        y = (np.round(np.abs(y) * 5) + 1).astype(np.float32)
        if op == 23:
            x, y = y, x
    info = S.shape_info([n, 1])
    ex = None if PAIRWISE[op] is None else np.array(PAIRWISE[op], dtype=np.float32)
    want = real_ref.pairwise(op, x, info, y, info, np.empty_like(x), info, ex)
    dz = torch.empty(n, device="cuda")
    ops.execPairwiseTransformFloat(None, op, dev(x), info, dev(y), info, dz, info, None if ex is None else dev(ex))
    ok = np.isfinite(want)
    if op in PAIRWISE_FLOOR:
        floor = np.maximum(np.exp(y.astype(np.float64)), np.abs(x.astype(np.float64) * y))[ok]
        d = ulps_at(host(dz)[ok], want[ok], floor)
        assert d.max(initial=0) <= 8, "op %d max ulp %g" % (op, d.max())
    else:
        d = ulp_distance(host(dz), want)
        assert d[ok].max(initial=0) <= PAIRWISE_LIBM.get(op, 0), "op %d max ulp %d" % (op, d[ok].max())


@pytest.mark.parametrize("kinds", [("c", "c", "c"), ("f", "f", "f"), ("c", "f", "c"), ("cview2", "c", "fview2"),
                                    ("rowview2", "rowview2", "c")])
def test_pairwise_layouts(ops, real_ref, kinds):
    rng = np.random.default_rng(11)
    shape = (29, 31)
    lx = Layout(rand_input(rng, shape, np.float32), kinds[0])
    ly = Layout(rand_input(rng, shape, np.float32), kinds[1])
    lz = Layout(np.zeros(shape, np.float32), kinds[2])
    dz = dev(lz.buffer)
    ops.execPairwiseTransformFloat(None, 9, dev(lx.buffer), lx.info, dev(ly.buffer), ly.info, dz, lz.info, None)
    np.testing.assert_array_equal(lz.read(host(dz)), lx.read() - ly.read())
    zb = lz.buffer.copy()
    real_ref.pairwise(9, lx.buffer, lx.info, ly.buffer, ly.info, zb, lz.info)
    np.testing.assert_array_equal(lz.read(host(dz)), lz.read(zb))


def test_pairwise_scalar_y_and_half(ops, real_ref):
    rng = np.random.default_rng(12)
    x = rand_input(rng, (64, 33), np.float16)
    y = np.array([1.5], dtype=np.float16)
    xi, yi = S.shape_info(x.shape), S.shape_info([1, 1])
    want = real_ref.pairwise(6, x.ravel(), xi, y, yi, np.empty(x.size, np.float16), xi)
    dz = dev(np.zeros(x.size, np.float16))
    ops.execPairwiseTransformHalf(None, 6, dev(x), xi, dev(y), yi, dz, xi, None)
    np.testing.assert_array_equal(host(dz), want)


@pytest.mark.parametrize("op", range(24))
def test_scalar_float_all_ops(ops, real_ref, op):
    rng = np.random.default_rng(300 + op)
    n = 20001
    x = rand_input(rng, n, np.float32, "normal")
    scalar = 1.75
    if op in (14, 15, 19):
        x = (np.round(x * 10) + (0.0 if op != 15 else 0.0)).astype(np.float32)
        x[x == 0] = 3.0
        scalar = 3.0
    info = S.shape_info([1, n])
    want = real_ref.scalar(op, x, info, np.empty_like(x), info, scalar)
    dz = torch.empty(n, device="cuda")
    ops.execScalarFloat(None, op, dev(x), info, dz, info, scalar, None)
    d = ulp_distance(host(dz), want)
    # x / scalar: the reference is compiled with reciprocal-math, so its loop multiplies by a
    # hoisted 1/scalar and can be one ulp away from the IEEE quotient computed here
    limit = 2 if op in (17, 18, 21, 22) else (1 if op in (3, 23) else 0)
    assert d[np.isfinite(want)].max(initial=0) <= limit, "op %d" % op
    if op == 3:
        np.testing.assert_array_equal(host(dz), x / np.float32(scalar))


@pytest.mark.parametrize("op", range(24))
def test_broadcast_float_all_ops(ops, real_ref, op):
    rng = np.random.default_rng(400 + op)
    shape = (45, 68)
    x = rand_input(rng, shape, np.float32, "normal")
    y = rand_input(rng, shape[1], np.float32, "normal")
    if op in (20, 22, 23):
        x = (np.round(x * 10)).astype(np.float32)
        y = (np.round(np.abs(y) * 5) + 1).astype(np.float32)
        x[x == 0] = 2.0
    xi, yi = S.shape_info(shape), S.shape_info([1, shape[1]])
    want = real_ref.broadcast(op, x.ravel(), xi, y, yi, np.empty(x.size, np.float32), xi, [1])
    dz = torch.empty(x.size, device="cuda")
    ops.execBroadcastFloat(None, op, dev(x), xi, dev(y), yi, dz, xi, [1], 1)
    d = ulp_distance(host(dz), want)
    assert d[np.isfinite(want)].max(initial=0) <= (2 if op in (17, 18) else 0), "op %d" % op


@pytest.mark.parametrize("shape,dims,kind", [
    ((16, 4096), [1], "c"), ((16, 4096), [0], "c"), ((33, 65), [1], "f"), ((33, 65), [0], "f"),
    ((6, 7, 8), [1], "c"), ((6, 7, 8), [0, 2], "c"), ((6, 7, 8), [1, 2], "f"), ((4, 5, 6, 7), [1, 3], "c"),
    ((24, 40), [1], "cview2"), ((24, 40), [1], "fview2"), ((24, 40), [0], "rowview2")])
def test_broadcast_layouts(ops, real_ref, shape, dims, kind):
    rng = np.random.default_rng(13)
    x = rand_input(rng, shape, np.float32)
    yshape = [shape[d] for d in dims]
    y = rand_input(rng, yshape, np.float32)
    lx = Layout(x, kind)
    lz = Layout(np.zeros(shape, np.float32), kind)
    yi = S.shape_info(yshape if len(yshape) > 1 else [1, yshape[0]])
    dz = dev(lz.buffer)
    ops.execBroadcastFloat(None, 0, dev(lx.buffer), lx.info, dev(y), yi, dz, lz.info, dims, len(dims))
    expand = [shape[i] if i in dims else 1 for i in range(len(shape))]
    np.testing.assert_array_equal(lz.read(host(dz)), x + y.reshape(expand))
    zb = lz.buffer.copy()
    real_ref.broadcast(0, lx.buffer, lx.info, y.ravel(), yi, zb, lz.info, dims)
    np.testing.assert_array_equal(lz.read(host(dz)), lz.read(zb))


@pytest.mark.parametrize("shape,dims", [((31, 64), [1]), ((31, 64), [0]), ((5, 6, 8), [2]), ((5, 6, 8), [0, 1])])
def test_scalar_along_dimension(ops, real_ref, shape, dims):
    rng = np.random.default_rng(14)
    x = rand_input(rng, shape, np.float32)
    ntads = x.size // int(np.prod([shape[d] for d in dims]))
    scalars = rand_input(rng, ntads, np.float32)
    xi = S.shape_info(shape)
    dz = torch.empty(x.size, device="cuda")
    ops.execScalarAlongDimensionFloat(None, 2, dev(x), xi, dz, xi, dev(scalars), None, dims, len(dims))
    keep = [i for i in range(len(shape)) if i not in dims]
    expand = [shape[i] if i in keep else 1 for i in range(len(shape))]
    np.testing.assert_array_equal(host(dz).reshape(shape), x * scalars.reshape(expand))
    if len(dims) == 1:
        # the reference's CPU loop only handles TADs with a linear stride (loops/cpu/scalar.cpp:38-60)
        want = real_ref.scalar_along_dimension(2, x.ravel(), xi, np.empty(x.size, np.float32), xi, scalars, dims)
        np.testing.assert_array_equal(host(dz), want)


def test_elementwise_chain_config_exact_and_two_ulp(ops, real_ref):
    """The benchmark's chain (broadcast Add -> Tanh -> pairwise Multiply) on a slab of the
    configured width: the two arithmetic steps are bit-exact, Tanh stays within 2 ulp."""
    rng1, rng2, rng3 = (np.random.default_rng(s) for s in (1, 2, 3))
    rows, cols = 1024, 4096
    x = rng1.standard_normal((rows, cols)).astype(np.float32)
    b = rng2.standard_normal(cols).astype(np.float32)
    y = rng3.uniform(0, 1, (rows, cols)).astype(np.float32)
    xi, bi = S.shape_info(x.shape), S.shape_info([1, cols])
    r1 = real_ref.broadcast(0, x.ravel(), xi, b, bi, np.empty(x.size, np.float32), xi, [1])
    r2 = real_ref.transform(15, r1, xi, np.empty_like(r1), xi)
    d1, d2, d3 = (torch.empty(x.size, device="cuda") for _ in range(3))
    ops.execBroadcastFloat(None, 0, dev(x), xi, dev(b), bi, d1, xi, [1], 1)
    ops.execTransformFloat(None, 15, d1, xi, d2, xi, None)
    ops.execPairwiseTransformFloat(None, 6, d2, xi, dev(y), xi, d3, xi, None)
    np.testing.assert_array_equal(host(d1), r1)
    assert ulp_distance(host(d2), r2).max() <= 2
    np.testing.assert_array_equal(host(d3), host(d2) * y.ravel())


def test_errors_are_reported_not_fatal(ops):
    from libnd4j_b200.native_ops import Nd4jError
    x = torch.zeros(16, device="cuda")
    info = S.shape_info([4, 4])
    with pytest.raises(Nd4jError) as e:
        ops.execTransformFloat(None, 57, x, info, x, info, None)   # hole in the transform table
    assert e.value.code == 2
    with pytest.raises(Nd4jError) as e:
        ops.execTransformFloat(None, 43, x, info, x, info, None)   # DropOut by rand(): recognised, not served
    assert e.value.code == 3
    with pytest.raises(Nd4jError) as e:
        ops.execTransformFloat(None, 36, x, info, x, info, None)   # Col2Im wants a six-axis x
    assert e.value.code == 1
    with pytest.raises(Nd4jError) as e:
        ops.execPairwiseTransformFloat(None, 0, x, info, x, S.shape_info([3, 3]), x, info, None)
    assert e.value.code == 1
    # the context is still usable
    ops.execTransformFloat(None, 26, x, info, x, info, None)
    assert host(x).sum() == 16


# ---- indexed overloads ----------------------------------------------------------------------------
@pytest.mark.parametrize("op", [0, 1, 6, 13])
def test_pairwise_indexed_gather_scatter(ops, op):
    """z[zIdx[i]] = op(x[xIdx[i]], y[yIdx[i]]) (include/loops/pairwise_transform.h:136-152): checked against the
    reference's shaped call on the gathered operands, since the indexed loop applies the same functor."""
    rng = np.random.default_rng(op)
    n, span = 5000, 12000
    x, y = rng.standard_normal(span).astype(np.float32), rng.standard_normal(span).astype(np.float32) + 3
    xi_, yi_ = rng.integers(0, span, n), rng.integers(0, span, n)
    zi_ = rng.permutation(span)[:n]
    z = np.full(span, -7, np.float32)
    dz = dev(z)
    info = S.shape_info([1, n])
    ops.execPairwiseTransformFloat(None, op, dev(x), info, dev(y), info, dz, info, None,
                                   dev(xi_.astype(np.int64)), dev(yi_.astype(np.int64)), dev(zi_.astype(np.int64)))
    dense = torch.zeros(n, device="cuda")
    ops.execPairwiseTransformFloat(None, op, dev(x[xi_]), info, dev(y[yi_]), info, dense, info, None)
    want = z.copy()
    want[zi_] = host(dense)
    np.testing.assert_array_equal(host(dz), want)


def test_scalar_indexed(ops):
    rng = np.random.default_rng(3)
    n, span = 3000, 9000
    x = rng.standard_normal(span).astype(np.float32)
    xi_ = rng.integers(0, span, n)
    zi_ = rng.permutation(span)[:n]
    z = np.zeros(span, np.float32)
    dz = dev(z)
    info = S.shape_info([1, n])
    ops.execScalarFloat(None, 2, dev(x), info, dz, info, 1.5, None, dev(xi_.astype(np.int64)), dev(zi_.astype(np.int64)))
    want = z.copy()
    want[zi_] = x[xi_] * np.float32(1.5)
    np.testing.assert_array_equal(host(dz), want)


# ---- row softmax family (special transforms 38, 39, 40) -------------------------------------------
def _softmax_truth(op, x):
    x = x.astype(np.float64)
    e = np.exp(x - x.max(axis=1, keepdims=True))
    y = e / e.sum(axis=1, keepdims=True)
    with np.errstate(divide="ignore"):
        return y if op == 38 else (y * (1 - y) if op == 39 else np.log(y))


@pytest.mark.parametrize("op", [38, 39, 40])
@pytest.mark.parametrize("shape", [(64, 10), (300, 1000), (160, 4096), (150, 2052), (7, 3000), (1, 777), (513, 1)])
@pytest.mark.parametrize("dt,name,tol", [(np.float32, "Float", 1e-5), (np.float64, "Double", 1e-12), (np.float16, "Half", 1e-2)])
def test_softmax_family_rows(ops, real_ref, op, shape, dt, name, tol):
    """Fused row softmax against the reference's composite (include/ops/special_ops.h:1484-1940). The
    derivative is called in place: out of place the reference subtracts the row maximum from the
    result buffer's previous content instead of x (special_ops.h:1826)."""
    rng = np.random.default_rng(op + shape[1])
    x = (rng.standard_normal(shape) * 3).astype(dt)
    info = S.shape_info(shape)
    want = x.copy().ravel()
    real_ref.transform(op, want, info, want, info)
    if op == 39:
        dz = dev(x)
        getattr(ops, "execTransform" + name)(None, op, dz, info, dz, info, None)
    else:
        dz = dev(np.zeros(x.size, dt))
        getattr(ops, "execTransform" + name)(None, op, dev(x), info, dz, info, None)
    # a column vector is one "row" of its whole length, like a row vector
    truth = _softmax_truth(op, x.reshape(1, -1) if 1 in shape else x).reshape(shape)
    got = host(dz).astype(np.float64).reshape(shape)
    ref = want.astype(np.float64).reshape(shape)
    finite = np.isfinite(truth) & np.isfinite(ref)
    scale = np.maximum(np.abs(truth), 1e-30 if op != 40 else 1.0)
    bound = np.maximum(tol * scale, np.abs(ref - truth) * 1.0000001)
    if dt == np.float16:
        # x - max is stored as a half before Exp reads it (spacing 2^-6 at magnitude 16..32), which alone
        # moves a probability by up to 0.8 %; the stored probability adds half an ulp (or the 6e-8 quantum)
        bound = np.maximum(bound, 3e-2 * scale + (1.2e-7 if op != 40 else 0.0))
        # probabilities near half's subnormal quantum (6e-8) round to different neighbours, or to
        # zero, depending on the last bits of the row sum: those elements only have to be tiny
        y = _softmax_truth(38, x.reshape(1, -1) if 1 in shape else x).reshape(shape)
        tiny = y < 2e-6
        finite &= ~tiny
        small = host(dz).astype(np.float64).reshape(shape)[tiny]
        if op != 40:
            assert (np.abs(small) <= 4e-6).all()
        else:
            assert (small <= np.log(4e-6)).all()
    else:
        assert (np.isneginf(got) == np.isneginf(ref))[~finite].all()
    assert (np.abs(got - truth)[finite] <= bound[finite]).all()


def test_softmax_f_order_rows(ops, real_ref):
    rng = np.random.default_rng(9)
    x = rng.standard_normal((40, 33)).astype(np.float32)
    lay = Layout(x, "f")
    want = lay.buffer.copy()
    real_ref.transform(38, want, lay.info, want, lay.info)
    dz = dev(np.zeros_like(lay.buffer))
    ops.execTransformFloat(None, 38, dev(lay.buffer), lay.info, dz, lay.info, None)
    np.testing.assert_allclose(host(dz), want, rtol=1e-5, atol=1e-9)
    np.testing.assert_allclose(host(dz).reshape(33, 40).T.sum(axis=1), 1.0, rtol=1e-5)


# ---- IsMax (special transform 41) -----------------------------------------------------------------
@pytest.mark.parametrize("shape,extra", [((1, 777), None), ((40, 33), None), ((40, 33), [1, 1]), ((40, 33), [1, 0]),
                                         ((6, 7, 8), [1, 2]), ((6, 7, 8), [2, 0, 2]), ((6, 7, 8), [2, 1, 2]),
                                         ((9, 11), [2, 0, 1])])
def test_ismax_first_maximum_wins(ops, real_ref, shape, extra):
    """One-hot of the maximum over the whole array or along dimensions, ties resolved to the first position,
    against the reference (include/ops/special_ops.h:2001-2400)."""
    rng = np.random.default_rng(len(shape) + (0 if extra is None else sum(extra)))
    x = rng.integers(0, 6, shape).astype(np.float32)          # few levels: many ties
    info = S.shape_info(list(shape))
    ex = None if extra is None else np.array(extra, np.float32)
    want = real_ref.transform(41, x.ravel().copy(), info, np.full(x.size, 7, np.float32), info, ex)
    dz = dev(np.full(x.size, 7, np.float32))
    ops.execTransformFloat(None, 41, dev(x), info, dz, info, None if ex is None else dev(ex))
    np.testing.assert_array_equal(host(dz), want)
    if extra is None:
        assert host(dz).sum() == 1 and host(dz)[int(x.argmax())] == 1


def test_ismax_positions_beyond_what_the_element_type_can_hold(ops, real_ref):
    """The winning position is carried as a 64-bit integer: half cannot represent positions above 2048 and
    float none above 2^24 exactly, and the reference scans with an integer index (special_ops.h:2199-2260)."""
    # half rows of 5001 elements with the maximum at odd positions far beyond 2048
    rows, cols = 6, 5001
    x = np.zeros((rows, cols), np.float16)
    where = [2049, 3001, 4097, 4999, 5000, 2051]
    for r, j in enumerate(where):
        x[r, j] = 3.0
        x[r, (j + 7) % cols if (j + 7) % cols > j else j] = 3.0          # a later duplicate where it fits
    info = S.shape_info([rows, cols])
    ex = np.array([1, 1], np.float16)
    dz = dev(np.full(x.size, 7, np.float16))
    ops.execTransformHalf(None, 41, dev(x), info, dz, info, dev(ex))
    got = host(dz).reshape(rows, cols)
    assert (got.sum(1) == 1).all()
    assert [int(g.argmax()) for g in got] == where
    # float, whole array of 2^24 + 1025 elements with the maximum at an odd position above 2^24
    n = (1 << 24) + 1025
    xf = np.zeros(n, np.float32)
    xf[(1 << 24) + 1001] = 2.0
    xf[(1 << 24) + 1003] = 2.0
    finfo = S.shape_info([1, n])
    dz = torch.full((n,), 7.0, device="cuda")
    ops.execTransformFloat(None, 41, dev(xf), finfo, dz, finfo, None)
    assert int(dz.sum().item()) == 1 and int(dz.argmax().item()) == (1 << 24) + 1001
    want = real_ref.transform(41, xf.copy(), finfo, np.full(n, 7, np.float32), finfo, None)
    np.testing.assert_array_equal(host(dz), want)
