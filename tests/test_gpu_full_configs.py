"""Every benchmark configuration at its full size, with the expected values taken from the reference's own
CPU loops (oracle/_ref) on the same seeded inputs:

  C1  execReduceFloat Sum along dimension 1, f32 [8192,4096], U(-1,1) seed 0
  C2  execBroadcast Add -> execTransform Tanh -> execPairwiseTransform Multiply, f32 [16384,4096], seeds 1/2/3
  C3  execIndexReduce IMax dim 1 (bit-exact) and execSummaryStats Variance dim 0, f32 [65536,1024], 16 levels
  C4  execReduce3 Cosine / Euclidean dim 1, [32768,512] f32 and f16, c-order and f-order stride-2 column views
  C5a execRandom Uniform / Gaussian / Bernoulli / inverted DropOut, seed 119 (2^27 outputs here: the CPU needs
      about 10 ns per draw; the 2^30 call differs only in length, and tests/test_gpu_random.py checks probe
      windows of it)
  C5b execReduceScalar Sum over U(-1,1): 2^28 floats against the reference, 2^31 against an fp64 truth

Tolerances are the stated ones: bit-exact indices and random bits, <= 2 ulp for Tanh, relative 1e-5 (f32) /
1e-2 (f16) for reductions, read as |gpu - truth| <= max(tol * sum|terms|, |ref - truth|) for sums."""
import numpy as np
import pytest
import torch

from libnd4j_b200 import shape as S
from tests.cases import Layout, result_info, ulp_distance

pytestmark = pytest.mark.gpu


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def host(t):
    return t.cpu().numpy()


def test_c1_reduce_sum_rows(ops, real_ref):
    x = np.random.default_rng(0).uniform(-1, 1, (8192, 4096)).astype(np.float32)
    xi, zi = S.shape_info(x.shape), result_info(x.shape, [1])
    want = real_ref.reduce(1, x.ravel(), xi, np.zeros(8192, np.float32), zi, [1])
    dz = torch.zeros(8192, device="cuda")
    ops.execReduceFloat(None, 1, dev(x), xi, None, dz, zi, [1], 1)
    x64 = x.astype(np.float64)
    truth, mag = x64.sum(1), np.abs(x64).sum(1)
    got = host(dz).astype(np.float64)
    bound = np.maximum(1e-5 * mag, np.abs(want - truth) * 1.0000001)
    assert (np.abs(got - truth) <= bound).all()
    assert (np.abs(got - want) <= 2e-5 * mag).all()


def test_c2_elementwise_chain(ops, real_ref):
    rows, cols = 16384, 4096
    x = np.random.default_rng(1).standard_normal((rows, cols), dtype=np.float32)
    b = np.random.default_rng(2).standard_normal(cols, dtype=np.float32)
    y = np.random.default_rng(3).random((rows, cols), dtype=np.float32)
    xi, bi = S.shape_info([rows, cols]), S.shape_info([1, cols])
    r1 = real_ref.broadcast(0, x.ravel(), xi, b, bi, np.empty(x.size, np.float32), xi, [1])
    r2 = real_ref.transform(15, r1, xi, np.empty_like(r1), xi)
    r3 = real_ref.pairwise(6, r2, xi, y.ravel(), xi, np.empty_like(r1), xi)
    d1, d2, d3 = (torch.empty(x.size, device="cuda") for _ in range(3))
    dy = dev(y)
    ops.execBroadcastFloat(None, 0, dev(x), xi, dev(b), bi, d1, xi, [1], 1)
    ops.execTransformFloat(None, 15, d1, xi, d2, xi, None)
    ops.execPairwiseTransformFloat(None, 6, d2, xi, dy, xi, d3, xi, None)
    g1, g2, g3 = host(d1), host(d2), host(d3)
    np.testing.assert_array_equal(g1, r1)                       # Add: exact
    ulps = ulp_distance(g2, r2)
    assert ulps.max() <= 2, "Tanh: %d ulp" % ulps.max()          # Tanh: <= 2 ulp from the host libm
    np.testing.assert_array_equal(g3, g2 * y.ravel())            # Multiply: exact on the GPU's own Tanh output
    # against the reference's chain: Tanh's 2 ulp carried through the product, plus the product's own rounding
    bound = 2 * np.spacing(np.abs(r2)).astype(np.float64) * y.ravel() + np.spacing(np.abs(r3)).astype(np.float64)
    assert (np.abs(g3.astype(np.float64) - r3) <= bound).all()


def test_c3_imax_rows_and_variance_columns(ops, real_ref):
    levels = (np.arange(16) / 8.0 - 1.0).astype(np.float32)
    x = levels[np.random.default_rng(4).integers(0, 16, (65536, 1024))]
    xi = S.shape_info(x.shape)
    dx = dev(x)
    zi = result_info(x.shape, [1])
    want = real_ref.index_reduce(0, x.ravel(), xi, np.zeros(65536, np.float32), zi, [1])
    dz = torch.zeros(65536, device="cuda")
    ops.execIndexReduceFloat(None, 0, dx, xi, None, dz, zi, [1], 1)
    np.testing.assert_array_equal(host(dz), want)                # every row, ties included
    zi0 = result_info(x.shape, [0])
    want = real_ref.summary_stats(0, x.ravel(), xi, np.zeros(1024, np.float32), zi0, [0], True)
    dz = torch.zeros(1024, device="cuda")
    ops.execSummaryStatsFloat(None, 0, dx, xi, None, dz, zi0, [0], 1, True)
    truth = x.astype(np.float64).var(0, ddof=1)
    np.testing.assert_allclose(host(dz), want, rtol=1e-5)
    np.testing.assert_allclose(host(dz), truth, rtol=1e-5)


def _reduce3_truth(op, a, b):
    if op == 1:
        d = a - b
        return np.sqrt((d * d).sum(1))
    return (a * b).sum(1) / (np.sqrt((a * a).sum(1)) * np.sqrt((b * b).sum(1)))


@pytest.mark.parametrize("dt,name,tol", [(np.float32, "Float", 1e-5), (np.float16, "Half", 1e-2)])
def test_c4_reduce3_rows_and_views(ops, real_ref, dt, name, tol):
    shape = (32768, 512)
    x = np.random.default_rng(5).standard_normal(shape).astype(np.float32).astype(dt)
    y = np.random.default_rng(6).standard_normal(shape).astype(np.float32).astype(dt)
    zi = result_info(shape, [1])
    x64, y64 = x.astype(np.float64), y.astype(np.float64)
    cx, cy = Layout(x, "c"), Layout(y, "c")
    for kind in ("c", "fview2"):
        lx, ly = Layout(x, kind), Layout(y, kind)
        dx, dy = dev(lx.buffer), dev(ly.buffer)
        for op in (2, 1):
            # the reference's cosine on non-contiguous operands carries its accumulators from row to row
            # (include/loops/reduce3.h:1112, 1320-1338): there it runs on a contiguous copy of the same arrays
            rx, ry = (cx, cy) if (op == 2 and kind != "c") else (lx, ly)
            want = real_ref.reduce3(op, rx.buffer, rx.info, ry.buffer, ry.info, np.zeros(shape[0], dt), zi, [1])
            dz = dev(np.zeros(shape[0], dt))
            getattr(ops, "execReduce3" + name)(None, op, dx, lx.info, None, dy, ly.info, dz, zi, [1], 1)
            got = host(dz).astype(np.float64)
            truth = _reduce3_truth(op, x64, y64)
            scale = np.maximum(np.abs(truth), 1.0 if op == 2 else 0.0)
            bound = np.maximum(tol * scale, np.abs(want.astype(np.float64) - truth) * 1.0000001)
            assert (np.abs(got - truth) <= bound).all(), (kind, op)
            # and directly against the reference, whose half arithmetic rounds after every step
            assert (np.abs(got - want.astype(np.float64)) <= 2 * tol * np.maximum(scale, np.abs(want.astype(np.float64)))).all(), (kind, op)


def test_c5a_random_ops_seed_119(ops, real_ref):
    n = 1 << 27
    zi = S.shape_info([1, n])
    st = ops.initRandom(None, 119, 100000, None)
    rs, _ = real_ref.init_random(119, 100000)
    try:
        ones = np.ones(n, np.float32)
        dones = dev(ones)
        for op, extra, arity in ((0, [0, 1], 0), (6, [0, 1], 2), (7, [0.3], 0), (2, [0.5], 1)):
            ex = np.array(extra, np.float32)
            want = np.zeros(n, np.float32)
            dz = torch.zeros(n, device="cuda")
            if arity == 0:
                real_ref.random(op, rs, want, zi, ex)
                ops.execRandomFloat(None, op, st, dz, zi, dev(ex))
            elif arity == 1:
                real_ref.random_x(op, rs, ones, zi, want, zi, ex)
                ops.execRandomFloat(None, op, st, dones, zi, dz, zi, dev(ex))
            else:
                real_ref.random_xy(op, rs, want, zi, want, zi, want, zi, ex)
                ops.execRandomFloat(None, op, st, dz, zi, dz, zi, dz, zi, dev(ex))
            got = host(dz)
            if op == 6:
                # uniforms are bit-exact; logf / cosf / sinf come from the device library instead of glibc
                assert np.abs(got - want).max() <= 1e-5
            else:
                np.testing.assert_array_equal(got, want)
            assert ops.rngState(st)[1:3] == (real_ref.rng_position(rs), real_ref.rng_generation(rs))
    finally:
        ops.destroyRandom(st)
        real_ref.destroy_random(rs)


def test_c5b_whole_array_sum(ops, real_ref):
    n = 1 << 31
    st = ops.initRandom(None, 8, 100000, None)
    big = torch.empty(n, device="cuda")
    chunk = 1 << 26
    ci = S.shape_info([1, chunk])
    em1 = torch.tensor([-1.0, 1.0], device="cuda")
    for off in range(0, n, chunk):
        ops.execRandomFloat(None, 0, st, big[off:off + chunk], ci, em1)
    ops.destroyRandom(st)
    # the full 2^31 against an fp64 truth accumulated on the device
    truth = sum(float(big[o:o + chunk].double().sum()) for o in range(0, n, chunk))
    mag = sum(float(big[o:o + chunk].double().abs().sum()) for o in range(0, n, chunk))
    got = ops.execReduceScalarFloat(None, 1, big, S.shape_info([1, n]), None)
    assert abs(got - truth) <= 1e-5 * mag
    # a 2^28 shard (what one of eight GPUs holds) against the reference's own whole-array loop
    m = 1 << 28
    shard = host(big[:m])
    mi = S.shape_info([1, m])
    want = float(real_ref.reduce_scalar(1, shard, mi))
    t = float(shard.astype(np.float64).sum())
    smag = float(np.abs(shard).astype(np.float64).sum())
    got = ops.execReduceScalarFloat(None, 1, big[:m], mi, None)
    assert abs(got - t) <= max(1e-5 * smag, abs(want - t) * 1.0000001)
