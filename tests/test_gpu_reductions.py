"""GPU parity of the reduction families (reduce, indexreduce, summarystats, reduce3) against the
reference's CPU loops, called through the C ABI.

Floating-point reductions are compared the way the tolerance has to be read for sums: the
reference folds sequentially in T, so both sides are held against an fp64 ground truth and the
GPU must satisfy |gpu - truth| <= max(tol * sum|terms|, |ref - truth|) with tol = 1e-5 (float32),
1e-2 (float16), 1e-12 (float64). Index reductions must be bit-exact, including ties.
"""
import numpy as np
import pytest
import torch

from libnd4j_b200 import shape as S
from tests.cases import Layout, rand_input, result_info

pytestmark = pytest.mark.gpu

TOL = {np.float32: 1e-5, np.float16: 1e-2, np.float64: 1e-12}
NAME = {np.float32: "Float", np.float16: "Double", np.float64: "Double"}
NAME[np.float16] = "Half"


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def host(t):
    return t.cpu().numpy()


def moved(x, dims):
    """[numTads, tadLen] float64 matrix of the TADs along `dims` in reference order."""
    keep = [i for i in range(x.ndim) if i not in dims]
    t = np.transpose(x, keep + list(dims)).astype(np.float64)
    return t.reshape(int(np.prod([x.shape[i] for i in keep], dtype=np.int64)), -1)


# opNum -> (truth(tads, extra), magnitude(tads, extra), input kind, extra)
def _var(t, e):
    n = t.shape[1]
    return (((t - e[0]) ** 2).sum(1) - e[1] ** 2 / n) / (n - 1)


REDUCE = {
    0: (lambda t, e: t.mean(1), lambda t, e: np.abs(t).mean(1), "normal", None),
    1: (lambda t, e: t.sum(1), lambda t, e: np.abs(t).sum(1), "normal", None),
    3: (lambda t, e: t.max(1), None, "normal", None),
    4: (lambda t, e: t.min(1), None, "normal", None),
    5: (lambda t, e: np.abs(t).sum(1), None, "normal", None),
    6: (lambda t, e: np.sqrt((t * t).sum(1)), None, "normal", None),
    7: (lambda t, e: np.abs(t).max(1), None, "normal", None),
    8: (lambda t, e: t.prod(1), None, "near1", None),
    9: (lambda t, e: np.sqrt(_var(t, e)), None, "normal", [0.1, 0.0]),
    10: (_var, None, "normal", [0.1, 0.0]),
    11: (lambda t, e: np.abs(t).sum(1), None, "normal", None),
    12: (lambda t, e: (np.abs(t - e[0]) <= e[1]).sum(1).astype(np.float64), None, "levels", [0.25, 1e-5, 0.0]),
    13: (lambda t, e: np.abs(t).max(1), None, "normal", None),
    14: (lambda t, e: np.abs(t).min(1), None, "normal", None),
    15: (lambda t, e: np.abs(t).mean(1), None, "normal", None),
    16: (lambda t, e: (t * np.log(t)).sum(1), lambda t, e: np.abs(t * np.log(t)).sum(1), "positive", None),
    17: (lambda t, e: np.log(t * t).sum(1), lambda t, e: np.abs(np.log(t * t)).sum(1), "positive", None),
    18: (lambda t, e: -(t * t * np.log(t * t)).sum(1), lambda t, e: np.abs(t * t * np.log(t * t)).sum(1), "positive", None),
    19: (lambda t, e: np.log(np.exp(t - t.max(1, keepdims=True)).sum(1)) + t.max(1), None, "normal", None),
    20: (lambda t, e: (t.sum(1) > 0).astype(np.float64), None, "bits", None),
    21: (lambda t, e: (t.prod(1) > 0).astype(np.float64), None, "bits", None),
    22: (lambda t, e: (t != 0).sum(1).astype(np.float64), None, "levels", None),
    23: (lambda t, e: np.sqrt((t * t).sum(1)), None, "normal", None),
    24: (lambda t, e: (np.abs(t) ** e[0]).sum(1) ** (1.0 / e[0]), None, "normal", [3.0]),
    25: (lambda t, e: (t * t).sum(1), None, "normal", None),
    26: (lambda t, e: (t == 0).sum(1).astype(np.float64), None, "levels", None),
}


def reduce_input(rng, shape, dt, kind):
    if kind == "near1":
        return (1.0 + rng.uniform(-0.01, 0.01, shape)).astype(dt)
    if kind == "bits":
        return (rng.uniform(0, 1, shape) > 0.7).astype(dt)
    return rand_input(rng, shape, dt, kind)


def check_against_truth(got, want, truth, mag, tol):
    got, want = got.astype(np.float64), want.astype(np.float64)
    bound = np.maximum(tol * np.maximum(mag, 1e-30), np.abs(want - truth) * 1.0000001)
    bad = np.abs(got - truth) > bound
    assert not bad.any(), "worst: got %r ref %r truth %r" % (got[bad][:3], want[bad][:3], truth[bad][:3])


@pytest.mark.parametrize("op", sorted(REDUCE))
@pytest.mark.parametrize("shape,dims", [((64, 1000), [1]), ((300, 96), [0]), ((12, 20, 30), [0, 2])])
def test_reduce_float_all_ops(ops, real_ref, op, shape, dims):
    truth_fn, mag_fn, kind, extra = REDUCE[op]
    rng = np.random.default_rng(op * 13 + len(shape))
    x = reduce_input(rng, shape, np.float32, kind)
    xi, zi = S.shape_info(shape), result_info(shape, dims)
    n = S.length(zi)
    ex = None if extra is None else np.array(extra, dtype=np.float32)
    want = real_ref.reduce(op, x.ravel(), xi, np.zeros(n, np.float32), zi, dims, ex)
    dz = torch.zeros(n, device="cuda")
    ops.execReduceFloat(None, op, dev(x), xi, None if ex is None else dev(ex), dz, zi, dims, len(dims))
    t = moved(x, dims)
    truth = truth_fn(t, extra)
    mag = mag_fn(t, extra) if mag_fn else np.abs(truth)
    check_against_truth(host(dz), want, truth, mag, 1e-5)


@pytest.mark.parametrize("dt", [np.float64, np.float16])
@pytest.mark.parametrize("op", [0, 1, 3, 4, 6, 13, 25])
def test_reduce_other_types(ops, real_ref, dt, op):
    truth_fn, mag_fn, kind, extra = REDUCE[op]
    rng = np.random.default_rng(op)
    shape, dims = (48, 200), [1]
    x = reduce_input(rng, shape, dt, kind)
    xi, zi = S.shape_info(shape), result_info(shape, dims)
    want = real_ref.reduce(op, x.ravel(), xi, np.zeros(48, dt), zi, dims)
    dz = dev(np.zeros(48, dt))
    getattr(ops, "execReduce" + NAME[dt])(None, op, dev(x), xi, None, dz, zi, dims, 1)
    t = moved(x, dims)
    truth = truth_fn(t, extra)
    mag = mag_fn(t, extra) if mag_fn else np.abs(truth)
    check_against_truth(host(dz), want, truth, mag, TOL[dt])


@pytest.mark.parametrize("kind", ["c", "f", "cview2", "fview2", "rowview2"])
@pytest.mark.parametrize("shape,dims", [((40, 72), [1]), ((40, 72), [0]), ((6, 10, 14), [1]), ((6, 10, 14), [0, 1]),
                                        ((6, 10, 14), [2]), ((3, 4, 5, 6), [1, 2]), ((3, 4, 5, 6), [0, 3])])
def test_reduce_layouts_sum_and_tad_order(ops, real_ref, kind, shape, dims):
    rng = np.random.default_rng(21)
    x = np.round(rng.standard_normal(shape) * 8).astype(np.float32)  # small integers: sums are exact
    lx = Layout(x, kind)
    zi = result_info(shape, dims)
    n = S.length(zi)
    dz = torch.zeros(n, device="cuda")
    ops.execReduceFloat(None, 1, dev(lx.buffer), lx.info, None, dz, zi, dims, len(dims))
    np.testing.assert_array_equal(host(dz), moved(x, dims).sum(1).astype(np.float32))
    want = real_ref.reduce(1, lx.buffer, lx.info, np.zeros(n, np.float32), zi, dims)
    np.testing.assert_array_equal(host(dz), want)


@pytest.mark.parametrize("n", [1, 5, 1023, 1 << 20, (1 << 22) + 3])
def test_reduce_scalar_sum_and_max(ops, real_ref, n):
    rng = np.random.default_rng(n)
    x = rng.uniform(-1, 1, n).astype(np.float32)
    xi = S.shape_info([1, n])
    got = ops.execReduceScalarFloat(None, 1, dev(x), xi, None)
    want = real_ref.reduce_scalar(1, x, xi)
    truth = x.astype(np.float64).sum()
    assert abs(got - truth) <= max(1e-5 * np.abs(x).astype(np.float64).sum(), abs(float(want) - truth))
    assert ops.execReduceScalarFloat(None, 3, dev(x), xi, None) == x.max()
    zi = S.shape_info([1, 1])
    dz = torch.zeros(1, device="cuda")
    ops.execReduceFloat(None, 4, dev(x), xi, None, dz, zi, [S.MAX_DIMENSION], 1)
    assert host(dz)[0] == x.min()


def test_reduce_scalar_is_reproducible(ops):
    x = np.random.default_rng(0).uniform(-1, 1, 1 << 23).astype(np.float32)
    d = dev(x)
    xi = S.shape_info([1, x.size])
    a = ops.execReduceScalarFloat(None, 1, d, xi, None)
    assert all(ops.execReduceScalarFloat(None, 1, d, xi, None) == a for _ in range(5))


# ---- index reduce -----------------------------------------------------------------------------
@pytest.mark.parametrize("op", [0, 1, 2, 3])
@pytest.mark.parametrize("shape,dims,kind", [((128, 1024), [1], "c"), ((257, 33), [0], "c"), ((64, 96), [1], "f"),
                                             ((9, 10, 11), [0, 2], "c"), ((9, 10, 11), [1, 2], "f"),
                                             ((50, 70), [1], "cview2"), ((50, 70), [1], "fview2")])
def test_index_reduce_ties_first_index_wins(ops, real_ref, op, shape, dims, kind):
    rng = np.random.default_rng(op + len(shape))
    x = rand_input(rng, shape, np.float32, "levels")  # 16 levels: every TAD has ties
    lx = Layout(x, kind)
    zi = result_info(shape, dims)
    n = S.length(zi)
    want = real_ref.index_reduce(op, lx.buffer, lx.info, np.zeros(n, np.float32), zi, dims)
    dz = torch.zeros(n, device="cuda")
    ops.execIndexReduceFloat(None, op, dev(lx.buffer), lx.info, None, dz, zi, dims, len(dims))
    np.testing.assert_array_equal(host(dz), want)
    t = moved(x, dims)
    key = {0: t, 1: -t, 2: np.abs(t), 3: -np.abs(t)}[op]
    np.testing.assert_array_equal(host(dz), key.argmax(1).astype(np.float32))


@pytest.mark.parametrize("op", [4, 5])
def test_first_last_index(ops, real_ref, op):
    rng = np.random.default_rng(op)
    x = rand_input(rng, (77, 130), np.float32, "levels")
    x[5] = 3.0   # no match in this row -> -1
    xi, zi = S.shape_info(x.shape), result_info(x.shape, [1])
    ex = np.array([0.25, 1e-5, 0.0], dtype=np.float32)   # equals 0.25 within eps
    want = real_ref.index_reduce(op, x.ravel(), xi, np.zeros(77, np.float32), zi, [1], ex)
    dz = torch.zeros(77, device="cuda")
    ops.execIndexReduceFloat(None, op, dev(x), xi, dev(ex), dz, zi, [1], 1)
    np.testing.assert_array_equal(host(dz), want)
    assert host(dz)[5] == -1


@pytest.mark.parametrize("n", [1, 1000, 1 << 20, (1 << 21) + 7])
def test_index_reduce_scalar(ops, n):
    """Whole-array argmax. The reference merges per-thread partials in arrival order here
    (include/loops/cpu/indexreduce.cpp:79-110), so ties are nondeterministic on its side; the
    first maximal index, which its sequential path produces, is the contract."""
    rng = np.random.default_rng(n)
    x = rand_input(rng, n, np.float32, "levels")
    xi = S.shape_info([1, n])
    assert ops.execIndexReduceScalarFloat(None, 0, dev(x), xi, None) == int(x.argmax())
    assert ops.execIndexReduceScalarFloat(None, 1, dev(x), xi, None) == int(x.argmin())


def test_index_reduce_full_config_rows(ops, real_ref):
    rng = np.random.default_rng(4)
    levels = (np.arange(16) / 8.0 - 1.0).astype(np.float32)
    x = levels[rng.integers(0, 16, (65536, 1024))]
    xi, zi = S.shape_info(x.shape), result_info(x.shape, [1])
    dz = torch.zeros(65536, device="cuda")
    ops.execIndexReduceFloat(None, 0, dev(x), xi, None, dz, zi, [1], 1)
    np.testing.assert_array_equal(host(dz), x.argmax(1).astype(np.float32))
    sample = slice(0, 4096)
    xs = np.ascontiguousarray(x[sample])
    want = real_ref.index_reduce(0, xs.ravel(), S.shape_info(xs.shape), np.zeros(4096, np.float32),
                                 result_info(xs.shape, [1]), [1])
    np.testing.assert_array_equal(host(dz)[sample], want)


# ---- summary stats ------------------------------------------------------------------------------
@pytest.mark.parametrize("op", [0, 1])
@pytest.mark.parametrize("bias", [True, False])
@pytest.mark.parametrize("shape,dims,kind", [((4096, 64), [0], "c"), ((64, 4096), [1], "c"), ((50, 60), [0], "f"),
                                             ((7, 8, 9), [0, 2], "c"), ((200, 48), [0], "cview2")])
def test_summary_stats(ops, real_ref, op, bias, shape, dims, kind):
    rng = np.random.default_rng(op + shape[0])
    x = (rand_input(rng, shape, np.float64) * 3 + 100).astype(np.float32)   # mean >> spread
    lx = Layout(x, kind)
    zi = result_info(shape, dims)
    n = S.length(zi)
    want = real_ref.summary_stats(op, lx.buffer, lx.info, np.zeros(n, np.float32), zi, dims, bias)
    dz = torch.zeros(n, device="cuda")
    ops.execSummaryStatsFloat(None, op, dev(lx.buffer), lx.info, None, dz, zi, dims, len(dims), bias)
    t = moved(x, dims)
    truth = t.var(1, ddof=1 if bias else 0)
    if op == 1:
        truth = np.sqrt(truth)
    np.testing.assert_allclose(host(dz), truth, rtol=1e-5)
    np.testing.assert_allclose(host(dz), want, rtol=1e-5)


def test_summary_stats_scalar_and_degenerate(ops, real_ref):
    x = np.random.default_rng(2).standard_normal(100001).astype(np.float32)
    xi = S.shape_info([1, x.size])
    got = ops.execSummaryStatsScalarFloat(None, 0, dev(x), xi, None, True)
    assert abs(got - x.astype(np.float64).var(ddof=1)) <= 1e-5 * got
    assert abs(got - float(real_ref.summary_stats_scalar(0, x, xi, True))) <= 1e-5 * got
    one = np.array([3.0], dtype=np.float32)
    assert ops.execSummaryStatsScalarFloat(None, 0, dev(one), S.shape_info([1, 1]), None, True) == 0.0


def test_summary_stats_full_config_columns(ops):
    rng = np.random.default_rng(4)
    levels = (np.arange(16) / 8.0 - 1.0).astype(np.float32)
    x = levels[rng.integers(0, 16, (65536, 1024))]
    xi, zi = S.shape_info(x.shape), result_info(x.shape, [0])
    dz = torch.zeros(1024, device="cuda")
    ops.execSummaryStatsFloat(None, 0, dev(x), xi, None, dz, zi, [0], 1, True)
    np.testing.assert_allclose(host(dz), x.astype(np.float64).var(0, ddof=1), rtol=1e-5)


# ---- reduce3 --------------------------------------------------------------------------------------
def reduce3_truth(op, a, b, eps=0.0):
    d = a - b
    if op == 0: return np.abs(d).sum(1)
    if op == 1: return np.sqrt((d * d).sum(1))
    if op == 2: return (a * b).sum(1) / (np.sqrt((a * a).sum(1)) * np.sqrt((b * b).sum(1)))
    if op == 3: return (a * b).sum(1)
    if op == 4:
        diff = np.abs(d)
        same = (diff <= eps) | (diff <= np.maximum(np.abs(a), np.abs(b)) * eps)
        return (~same).sum(1).astype(np.float64)
    if op == 5: return 1 - (a * b).sum(1) / (np.sqrt((a * a).sum(1)) * np.sqrt((b * b).sum(1)))
    if op == 6: return 1 - np.minimum(a, b).sum(1) / np.maximum(a, b).sum(1)
    if op == 7: return (a != b).sum(1) / a.shape[1]
    raise ValueError(op)


@pytest.mark.parametrize("op", range(8))
@pytest.mark.parametrize("dt", [np.float32, np.float64, np.float16])
def test_reduce3_rows_all_ops(ops, real_ref, op, dt):
    rng = np.random.default_rng(op)
    shape = (96, 512)
    kind = "positive" if op == 6 else ("levels" if op in (4, 7) else "normal")
    x, y = rand_input(rng, shape, dt, kind), rand_input(rng, shape, dt, kind)
    xi, zi = S.shape_info(shape), result_info(shape, [1])
    if op == 4:
        # along a dimension the reference hands EqualsWithEps a null parameter block and reads
        # index 2 of it (include/loops/reduce3.h:1238-1250, ops.h:2846): it cannot be run here.
        want = reduce3_truth(op, x.astype(np.float64), y.astype(np.float64)).astype(dt)
    else:
        want = real_ref.reduce3(op, x.ravel(), xi, y.ravel(), xi, np.zeros(96, dt), zi, [1])
    dz = dev(np.zeros(96, dt))
    getattr(ops, "execReduce3" + NAME[dt])(None, op, dev(x), xi, None, dev(y), xi, dz, zi, [1], 1)
    truth = reduce3_truth(op, x.astype(np.float64), y.astype(np.float64))
    tol = TOL[dt]
    got = host(dz).astype(np.float64)
    scale = np.maximum(np.abs(truth), 1.0 if op in (2, 5) else 1e-30)
    bound = np.maximum(tol * scale, np.abs(want.astype(np.float64) - truth) * 1.0000001)
    if op in (0, 3):
        bound = np.maximum(bound, tol * np.abs(x.astype(np.float64) * (1 if op == 0 else y)).sum(1))
    assert (np.abs(got - truth) <= bound).all()


@pytest.mark.parametrize("op", [1, 2])
@pytest.mark.parametrize("kind", ["f", "fview2", "cview2", "rowview2"])
def test_reduce3_views(ops, real_ref, op, kind):
    """Strided operands. Euclidean distance is compared with the reference on the view itself;
    cosine similarity is compared with the reference run on a contiguous copy, because the
    reference's non-contiguous path shares one pair of norm accumulators across all rows
    (include/loops/reduce3.h:1112, 1320-1338) and is wrong from row 1 on."""
    rng = np.random.default_rng(31)
    shape = (128, 96)
    x, y = rand_input(rng, shape, np.float32), rand_input(rng, shape, np.float32)
    lx, ly = Layout(x, kind), Layout(y, kind)
    zi = result_info(shape, [1])
    dz = torch.zeros(128, device="cuda")
    ops.execReduce3Float(None, op, dev(lx.buffer), lx.info, None, dev(ly.buffer), ly.info, dz, zi, [1], 1)
    ci = S.shape_info(shape)
    want = real_ref.reduce3(op, x.ravel(), ci, y.ravel(), ci, np.zeros(128, np.float32), zi, [1])
    np.testing.assert_allclose(host(dz), want, rtol=1e-5, atol=1e-6)
    if op == 1 and kind != "f":
        direct = real_ref.reduce3(op, lx.buffer, lx.info, ly.buffer, ly.info, np.zeros(128, np.float32), zi, [1])
        np.testing.assert_allclose(host(dz), direct, rtol=1e-5)


def test_reduce3_reference_fixture_euclidean(ops):
    """tests_cpu/layers_tests/Reduce3Tests.cpp:10-45 of the reference: EuclideanDistance (op 1)
    of x[1,4] = {1,2,3,4} against every row of y[4,4] = 1..16 along dimension 1 gives
    {0, 8, 16, 24} exactly."""
    x = np.array([1, 2, 3, 4], dtype=np.float32)
    y = np.arange(1, 17, dtype=np.float32).reshape(4, 4)
    xi, yi, zi = S.shape_info([1, 4]), S.shape_info([4, 4]), S.shape_info([4, 1])
    dz = torch.zeros(4, device="cuda")
    ops.execReduce3Float(None, 1, dev(x), xi, None, dev(y), yi, dz, zi, [1], 1)
    np.testing.assert_array_equal(host(dz), np.array([0, 8, 16, 24], dtype=np.float32))


def test_reduce3_scalar_and_equals_with_eps(ops, real_ref):
    rng = np.random.default_rng(33)
    x = rand_input(rng, 50001, np.float32)
    y = x.copy()
    y[::1000] += 0.5
    xi = S.shape_info([1, x.size])
    eps = np.array([1e-3], dtype=np.float32)
    got = ops.execReduce3ScalarFloat(None, 4, dev(x), xi, dev(eps), dev(y), xi)
    assert got == float(real_ref.reduce3_scalar(4, x, xi, y, xi, eps)) == 51.0
    got = ops.execReduce3ScalarFloat(None, 3, dev(x), xi, None, dev(y), xi)
    truth = (x.astype(np.float64) * y).sum()
    assert abs(got - truth) <= 1e-5 * np.abs(x.astype(np.float64) * y).sum()


def test_reduce3_full_config(ops, real_ref):
    rng5, rng6 = np.random.default_rng(5), np.random.default_rng(6)
    shape = (32768, 512)
    x, y = rng5.standard_normal(shape).astype(np.float32), rng6.standard_normal(shape).astype(np.float32)
    zi = result_info(shape, [1])
    for dt in (np.float32, np.float16):
        xd, yd = x.astype(dt), y.astype(dt)
        x64, y64 = xd.astype(np.float64), yd.astype(np.float64)
        for kind in ("c", "fview2"):
            lx, ly = Layout(xd, kind), Layout(yd, kind)
            for op in (2, 1):
                dz = dev(np.zeros(shape[0], dt))
                getattr(ops, "execReduce3" + NAME[dt])(None, op, dev(lx.buffer), lx.info, None, dev(ly.buffer),
                                                        ly.info, dz, zi, [1], 1)
                truth = reduce3_truth(op, x64, y64)
                tol = TOL[dt]
                scale = np.maximum(np.abs(truth), 1.0 if op == 2 else 0.0)
                assert (np.abs(host(dz).astype(np.float64) - truth) <= tol * scale).all(), (dt, kind, op)


# ---- reduce3 over all TAD pairs -------------------------------------------------------------------
def reduce3_all_truth(op, a, b):
    """a [xTads, len], b [yTads, len] -> [xTads, yTads] in float64."""
    return np.stack([reduce3_truth(op, np.broadcast_to(a[r], b.shape), b) for r in range(a.shape[0])])


@pytest.mark.parametrize("op", range(8))
@pytest.mark.parametrize("dt", [np.float32, np.float64, np.float16])
def test_reduce3_all_pairs(ops, real_ref, op, dt):
    """execReduce3All: ragged tile edges (70 x 45 TADs, 129 elements) against the reference's own
    loop (include/loops/reduce3.h:919-990)."""
    rng = np.random.default_rng(100 + op)
    xs, ys = (70, 129), (45, 129)
    kind = "positive" if op == 6 else ("levels" if op in (4, 7) else "normal")
    x, y = rand_input(rng, xs, dt, kind), rand_input(rng, ys, dt, kind)
    xi, yi, zi = S.shape_info(xs), S.shape_info(ys), S.shape_info([70, 45])
    truth = reduce3_all_truth(op, x.astype(np.float64), y.astype(np.float64))
    if op == 4:
        # EqualsWithEps reads index 2 of a parameter block the reference never allocates here
        # (extraParamsLen is 0, include/ops/ops.h:2839-2859): the truth stands in for it, eps = 0
        want = truth.astype(dt)
    else:
        want = real_ref.reduce3_all(op, x.ravel(), xi, y.ravel(), yi, np.zeros(70 * 45, dt), zi, [1]).reshape(70, 45)
    dz = dev(np.full(70 * 45, 7, dt))
    getattr(ops, "execReduce3All" + NAME[dt])(None, op, dev(x), xi, None, dev(y), yi, dz, zi, [1], 1, None, None, None, None)
    got = host(dz).astype(np.float64).reshape(70, 45)
    tol = TOL[dt]
    scale = np.maximum(np.abs(truth), 1.0 if op in (2, 5) else 1e-30)
    bound = np.maximum(tol * scale, np.abs(want.astype(np.float64) - truth) * 1.0000001)
    if op in (0, 3):
        ax, ay = np.abs(x.astype(np.float64)), np.abs(y.astype(np.float64))
        mag = ax.sum(1)[:, None] + ay.sum(1)[None, :] if op == 0 else ax @ ay.T
        bound = np.maximum(bound, tol * mag)
    assert (np.abs(got - truth) <= bound).all()


@pytest.mark.parametrize("kind", ["f", "fview2", "cview2"])
def test_reduce3_all_pairs_views_and_columns(ops, real_ref, kind):
    """TADs along dimension 0 of strided operands: every column of x against every column of y."""
    rng = np.random.default_rng(77)
    x, y = rand_input(rng, (200, 33), np.float32), rand_input(rng, (200, 70), np.float32)
    lx, ly = Layout(x, kind), Layout(y, kind)
    zi = S.shape_info([33, 70])
    dz = torch.zeros(33 * 70, device="cuda")
    ops.execReduce3AllFloat(None, 1, dev(lx.buffer), lx.info, None, dev(ly.buffer), ly.info, dz, zi, [0], 1,
                            None, None, None, None)
    want = real_ref.reduce3_all(1, lx.buffer, lx.info, ly.buffer, ly.info, np.zeros(33 * 70, np.float32), zi, [0])
    truth = reduce3_all_truth(1, x.T.astype(np.float64), y.T.astype(np.float64)).ravel()
    np.testing.assert_allclose(host(dz), truth, rtol=1e-5)
    np.testing.assert_allclose(host(dz), want, rtol=1e-5)


def test_reduce3_all_pairs_rejects_mismatched_tads(ops):
    xi, yi, zi = S.shape_info([4, 8]), S.shape_info([4, 9]), S.shape_info([4, 4])
    z = torch.zeros(16, device="cuda")
    with pytest.raises(RuntimeError):
        ops.execReduce3AllFloat(None, 1, torch.zeros(32, device="cuda"), xi, None, torch.zeros(36, device="cuda"), yi,
                                z, zi, [1], 1, None, None, None, None)


# ---- along-TAD reductions over thousands of back-to-back TADs ---------------------------------------
@pytest.mark.parametrize("dt", [np.float32, np.float64, np.float16])
@pytest.mark.parametrize("rows,cols", [(8191, 1000), (4099, 4096), (40000, 64), (70001, 24)])
def test_dimension_reductions_on_many_back_to_back_tads(ops, real_ref, dt, rows, cols):
    """Shapes with thousands of contiguous TADs (ragged row counts, lengths that leave partial trips): Sum, Max,
    IMax with ties, Variance and Euclidean distance against the reference."""
    if dt != np.float32 and rows > 10000:
        pytest.skip("the float run covers the long shapes")
    rng = np.random.default_rng(rows + cols)
    x = rng.integers(-8, 9, (rows, cols)).astype(dt)          # small integers: ties for IMax, exact sums
    y = rng.integers(-8, 9, (rows, cols)).astype(dt)
    xi, zi = S.shape_info([rows, cols]), S.shape_info([rows, 1])
    name = NAME[dt]
    dx, dy = dev(x), dev(y)
    out = dev(np.zeros(rows, dt))
    getattr(ops, "execReduce" + name)(None, 1, dx, xi, None, out, zi, [1], 1)
    np.testing.assert_array_equal(host(out).astype(np.float64), x.astype(np.float64).sum(1))
    getattr(ops, "execReduce" + name)(None, 3, dx, xi, None, out, zi, [1], 1)
    np.testing.assert_array_equal(host(out), x.max(1))
    getattr(ops, "execIndexReduce" + name)(None, 0, dx, xi, None, out, zi, [1], 1)
    np.testing.assert_array_equal(host(out).astype(np.int64), x.argmax(1))
    getattr(ops, "execSummaryStats" + name)(None, 0, dx, xi, None, out, zi, [1], 1, True)
    np.testing.assert_allclose(host(out).astype(np.float64), x.astype(np.float64).var(1, ddof=1), rtol=TOL[dt] * 10)
    getattr(ops, "execReduce3" + name)(None, 1, dx, xi, None, dy, xi, out, zi, [1], 1)
    want = np.sqrt(((x.astype(np.float64) - y.astype(np.float64)) ** 2).sum(1))
    np.testing.assert_allclose(host(out).astype(np.float64), want, rtol=TOL[dt])
    if dt == np.float32 and rows < 10000:
        ref = real_ref.reduce3(1, x.ravel(), xi, y.ravel(), xi, np.zeros(rows, dt), zi, [1])
        np.testing.assert_allclose(host(out), ref, rtol=1e-5)
