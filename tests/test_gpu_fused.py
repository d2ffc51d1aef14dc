"""Fused elementwise chains on the GPU. nd4jb200_exec_chain must give, bit for bit, what the three launches it
replaces give (execBroadcast -> execTransform -> execPairwiseTransform), and the meta-predicate entry points
what execPairwiseTransform -> execScalar give; the separate launches are themselves held against the reference
in tests/test_gpu_elementwise.py and tests/test_gpu_full_configs.py. The benchmark's chain is also compared with
the reference's CPU loops directly."""
import numpy as np
import pytest
import torch

from libnd4j_b200 import shape as S
from tests.cases import Layout, ulp_distance

pytestmark = pytest.mark.gpu

NAMES = {np.float32: ("Float", 0), np.float64: ("Double", 1), np.float16: ("Half", 2)}


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def host(t):
    return t.cpu().numpy()


def same_bits(a, b):
    a, b = np.ascontiguousarray(a), np.ascontiguousarray(b)
    it = {2: np.uint16, 4: np.uint32, 8: np.uint64}[a.dtype.itemsize]
    nan = np.isnan(a) & np.isnan(b)
    return np.array_equal(np.where(nan, 0, a.view(it)), np.where(nan, 0, b.view(it)))


def three_calls(ops, name, bc, tr, pw, lx, lb, ly, lz, dims, tr_extra=None):
    """The chain as separate launches, through a scratch copy laid out like z."""
    fb, ft, fp = (getattr(ops, f + name) for f in ("execBroadcast", "execTransform", "execPairwiseTransform"))
    t = dev(lz.buffer)
    fb(None, bc, dev(lx.buffer), lx.info, dev(lb.buffer), lb.info, t, lz.info, dims, len(dims))
    ft(None, tr, t, lz.info, t, lz.info, None if tr_extra is None else dev(tr_extra))
    fp(None, pw, t, lz.info, dev(ly.buffer), ly.info, t, lz.info, None)
    return host(t)


# (broadcast op, transform op, pairwise op): arithmetic, comparison and min / max steps around transforms with and
# without transcendental arithmetic; the last two fall back to separate launches (FloorMod / PowB are not light ops)
TRIPLES = [(0, 15, 6), (2, 10, 0), (1, 2, 2), (14, 0, 14), (3, 18, 9), (5, 19, 8), (13, 4, 13), (6, 23, 18), (8, 6, 3),
           (17, 42, 22), (18, 0, 6), (0, 15, 7)]


@pytest.mark.parametrize("dt", [np.float32, np.float64, np.float16])
@pytest.mark.parametrize("triple", TRIPLES)
@pytest.mark.parametrize("kind,shape,dims", [("c", (37, 64), [1]), ("c", (37, 61), [1]), ("c", (64, 24), [0]),
                                             ("f", (24, 40), [1]), ("cview2", (16, 48), [1]), ("c", (5, 6, 8), [2]),
                                             ("c", (5, 6, 8), [0, 2]), ("rowview2", (20, 32), [1])])
def test_chain_equals_three_launches(ops, dt, triple, kind, shape, dims):
    bc, tr, pw = triple
    name, code = NAMES[dt]
    rng = np.random.default_rng(sum(shape) + bc + tr + pw)
    x = rng.standard_normal(shape).astype(dt)
    y = rng.uniform(0.25, 2.0, shape).astype(dt)
    bshape = [shape[d] for d in dims]
    b = rng.uniform(0.5, 1.5, bshape).astype(dt)
    lx, ly, lz = Layout(x, kind), Layout(y, kind), Layout(np.zeros(shape, dt), kind)
    lb = Layout(b.reshape(1, -1) if len(dims) == 1 else b, "c")
    want = three_calls(ops, name, bc, tr, pw, lx, lb, ly, lz, dims)
    dz = dev(lz.buffer)
    ops.execChain(code, None, bc, dev(lx.buffer), lx.info, dev(lb.buffer), lb.info, dims, len(dims), tr, None, pw,
                  dev(ly.buffer), ly.info, None, dz, lz.info)
    assert same_bits(lz.read(host(dz)), lz.read(want)), (triple, kind, shape, dims)


@pytest.mark.parametrize("alias", ["x", "y"])
def test_chain_in_place(ops, alias):
    rng = np.random.default_rng(9)
    shape = (33, 128)
    x, y = rng.standard_normal(shape).astype(np.float32), rng.uniform(0, 1, shape).astype(np.float32)
    b = rng.standard_normal((1, 128)).astype(np.float32)
    info, bi = S.shape_info(shape), S.shape_info([1, 128])
    lx, ly, lb, lz = Layout(x, "c"), Layout(y, "c"), Layout(b, "c"), Layout(np.zeros(shape, np.float32), "c")
    want = three_calls(ops, "Float", 0, 15, 6, lx, lb, ly, lz, [1])
    dx, dy = dev(x), dev(y)
    dz = dx if alias == "x" else dy
    ops.execChain(0, None, 0, dx, info, dev(b), bi, [1], 1, 15, None, 6, dy, info, None, dz, info)
    assert same_bits(host(dz).ravel(), want)


def test_chain_with_transform_parameters_and_errors(ops):
    rng = np.random.default_rng(10)
    shape = (16, 256)
    x, y = rng.standard_normal(shape).astype(np.float32), rng.uniform(0, 1, shape).astype(np.float32)
    b = rng.standard_normal((1, 256)).astype(np.float32)
    info, bi = S.shape_info(shape), S.shape_info([1, 256])
    lx, ly, lb, lz = Layout(x, "c"), Layout(y, "c"), Layout(b, "c"), Layout(np.zeros(shape, np.float32), "c")
    alpha = np.array([0.3], np.float32)                       # LeakyRELU (opNum 31) takes its slope from extraParams
    want = three_calls(ops, "Float", 0, 31, 6, lx, lb, ly, lz, [1], tr_extra=alpha)
    dz = torch.zeros(x.size, device="cuda")
    ops.execChain(0, None, 0, dev(x), info, dev(b), bi, [1], 1, 31, dev(alpha), 6, dev(y), info, None, dz, info)
    assert same_bits(host(dz), want)
    with pytest.raises(RuntimeError):                          # b does not match the TAD length
        ops.execChain(0, None, 0, dev(x), info, dev(b[:, :100]), S.shape_info([1, 100]), [1], 1, 15, None, 6, dev(y), info,
                      None, dz, info)
    with pytest.raises(RuntimeError):                          # y has another shape
        ops.execChain(0, None, 0, dev(x), info, dev(b), bi, [1], 1, 15, None, 6, dev(y), S.shape_info([256, 16]), None, dz, info)
    with pytest.raises(RuntimeError):                          # hole in the transform table
        ops.execChain(0, None, 0, dev(x), info, dev(b), bi, [1], 1, 57, None, 6, dev(y), info, None, dz, info)


def test_chain_full_config_against_the_reference(ops, real_ref):
    """f32 [16384,4096], seeds 1/2/3: the fused pass equals the three launches exactly and stays within Tanh's
    2 ulp (carried through the product) of the reference's CPU loops."""
    rows, cols = 16384, 4096
    x = np.random.default_rng(1).standard_normal((rows, cols), dtype=np.float32)
    b = np.random.default_rng(2).standard_normal(cols, dtype=np.float32)
    y = np.random.default_rng(3).random((rows, cols), dtype=np.float32)
    xi, bi = S.shape_info([rows, cols]), S.shape_info([1, cols])
    dx, db, dy = dev(x), dev(b), dev(y)
    t = torch.empty(x.size, device="cuda")
    ops.execBroadcastFloat(None, 0, dx, xi, db, bi, t, xi, [1], 1)
    ops.execTransformFloat(None, 15, t, xi, t, xi, None)
    ops.execPairwiseTransformFloat(None, 6, t, xi, dy, xi, t, xi, None)
    dz = torch.empty(x.size, device="cuda")
    before = ops.launchCount()
    ops.execChain(0, None, 0, dx, xi, db, bi, [1], 1, 15, None, 6, dy, xi, None, dz, xi)
    assert ops.launchCount() - before == 1
    assert torch.equal(dz, t)
    r1 = real_ref.broadcast(0, x.ravel(), xi, b, bi, np.empty(x.size, np.float32), xi, [1])
    r2 = real_ref.transform(15, r1, xi, np.empty_like(r1), xi)
    r3 = real_ref.pairwise(6, r2, xi, y.ravel(), xi, np.empty_like(r1), xi)
    g3 = host(dz)
    bound = 2 * np.spacing(np.abs(r2)).astype(np.float64) * y.ravel() + np.spacing(np.abs(r3)).astype(np.float64)
    assert (np.abs(g3.astype(np.float64) - r3) <= bound).all()


# (pairwise opNumA, scalar opNumB): the last two use a scalar op outside the light set (two launches)
META = [(0, 2), (6, 0), (9, 6), (2, 12), (13, 3), (17, 1), (7, 5), (0, 14), (6, 21)]


@pytest.mark.parametrize("dt", [np.float32, np.float64, np.float16])
@pytest.mark.parametrize("pair", META)
@pytest.mark.parametrize("kind", ["c", "f", "cview2"])
def test_meta_predicate_shape_equals_pairwise_then_scalar(ops, dt, pair, kind):
    pw, sc = pair
    name, _ = NAMES[dt]
    rng = np.random.default_rng(pw * 31 + sc)
    shape = (23, 40)
    x = rng.uniform(0.5, 3.0, shape).astype(dt)
    y = rng.uniform(0.5, 2.0, shape).astype(dt)
    lx, ly, lz = Layout(x, kind), Layout(y, kind), Layout(np.zeros(shape, dt), kind)
    extra_a = np.array([1.5], dt) if pw == 17 else None       # Axpy: alpha
    scalar = 1.75
    t = dev(lz.buffer)
    getattr(ops, "execPairwiseTransform" + name)(None, pw, dev(lx.buffer), lx.info, dev(ly.buffer), ly.info, t, lz.info,
                                                 None if extra_a is None else dev(extra_a))
    getattr(ops, "execScalar" + name)(None, sc, t, lz.info, t, lz.info, scalar, None)
    dz = dev(lz.buffer)
    getattr(ops, "execMetaPredicateShape" + name)(None, 2, pw, 0, sc, x.size, dev(lx.buffer), lx.info, dev(ly.buffer), ly.info,
                                                  dz, lz.info, None if extra_a is None else dev(extra_a), None, 0.0, scalar)
    assert same_bits(lz.read(host(dz)), lz.read(host(t))), (pair, kind)


@pytest.mark.parametrize("strides", [(1, 1, 1), (2, 1, 3)])
def test_meta_predicate_strided_and_type_errors(ops, strides):
    rng = np.random.default_rng(5)
    n = 10007
    sx, sy, sz = strides
    x, y = rng.standard_normal(n * sx).astype(np.float32), rng.standard_normal(n * sy).astype(np.float32)
    z = np.zeros(n * sz, np.float32)
    dz = dev(z)
    ops.execMetaPredicateStridedFloat(None, 2, 6, 0, 0, n, dev(x), sx, dev(y), sy, dz, sz, None, None, 0.0, 0.5)
    want = z.copy()
    want[::sz] = (x[::sx] * y[::sy]).astype(np.float32) + np.float32(0.5)
    assert same_bits(host(dz), want)
    with pytest.raises(RuntimeError, match="pairwise"):        # the reference defines no other type pair
        ops.execMetaPredicateStridedFloat(None, 0, 6, 2, 0, n, dev(x), sx, dev(y), sy, dz, sz, None, None, 0.0, 0.5)
