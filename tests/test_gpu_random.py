"""GPU parity of the random family against the reference's RandomBuffer / execRandom: uniform
bits, Bernoulli and dropout masks bit-exact (including the wrap-around hash path, generations
above 1 and re-seeded states); Gaussian / LogNormal within 1e-5 absolute because log/cos/sin
come from different math libraries."""
import numpy as np
import pytest
import torch

from libnd4j_b200 import shape as S
from libnd4j_b200.native_ops import FLOAT

pytestmark = pytest.mark.gpu

SEED, TABLE = 119, 100000   # fixture of the reference's RNGTests.cpp:22-34


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def host(t):
    return t.cpu().numpy()


@pytest.fixture()
def pair(ops, real_ref):
    st = ops.initRandom(None, SEED, TABLE, None)
    rs, table = real_ref.init_random(SEED, TABLE)
    yield st, rs, table
    ops.destroyRandom(st)
    real_ref.destroy_random(rs)


def test_table_matches_reference(ops, real_ref, pair):
    st, rs, table = pair
    got = torch.zeros(TABLE, dtype=torch.int64, device="cuda")
    ops.memcpy(got, ops.lib.nd4jb200_rng_device_table(st), TABLE * 8, 3)
    np.testing.assert_array_equal(host(got).view(np.uint64), table)
    # values printed by the reference for this fixture
    assert table[0] == 7465776281147007380 and table[99999] == 2165072995135488967


def run_both(ops, ref, st, rs, op, n, extra, x=None, y=None, dt=np.float32, name="Float", gaussian=False):
    zi = S.shape_info([1, n])
    z = np.zeros(n, dt)
    dz = dev(z)
    ex = np.array(extra, dtype=dt)
    dex = dev(ex)
    fn = getattr(ops, "execRandom" + name)
    if gaussian:
        fn(None, op, st, dz, zi, dz, zi, dz, zi, dex)
        ref.random_xy(op, rs, z, zi, z, zi, z, zi, ex)
    elif x is None:
        fn(None, op, st, dz, zi, dex)
        ref.random(op, rs, z, zi, ex)
    elif y is None:
        fn(None, op, st, dev(x), zi, dz, zi, dex)
        ref.random_x(op, rs, x, zi, z, zi, ex)
    else:
        fn(None, op, st, dev(x), zi, dev(y), zi, dz, zi, dex)
        ref.random_xy(op, rs, x, zi, y, zi, z, zi, ex)
    return host(dz), z


def test_sequence_of_calls_bit_exact(ops, real_ref, pair):
    """Uniform -> Gaussian -> Bernoulli -> DropOutInverted -> DropOut -> AlphaDropOut ->
    ProbablisticMerge -> Linspace -> Exponential on one evolving state; the call lengths make the
    position wrap the 100000-entry table several times (generation > 1)."""
    st, rs, _ = pair
    rng = np.random.default_rng(7)
    n = 70001
    x = rng.standard_normal(n).astype(np.float32)
    y = rng.standard_normal(n).astype(np.float32)
    g, r = run_both(ops, real_ref, st, rs, 0, n, [0, 1])
    np.testing.assert_array_equal(g, r)
    g, r = run_both(ops, real_ref, st, rs, 0, n, [-3, 5])
    np.testing.assert_array_equal(g, r)
    g, r = run_both(ops, real_ref, st, rs, 6, n, [0, 1], gaussian=True)
    np.testing.assert_allclose(g, r, atol=1e-5, rtol=0)
    g, r = run_both(ops, real_ref, st, rs, 7, n, [0.3])
    np.testing.assert_array_equal(g, r)
    g, r = run_both(ops, real_ref, st, rs, 2, n, [0.5], x=x)
    np.testing.assert_array_equal(g, r)
    g, r = run_both(ops, real_ref, st, rs, 1, n, [0.8], x=x)
    np.testing.assert_array_equal(g, r)
    g, r = run_both(ops, real_ref, st, rs, 12, n, [0.6, 1.1, -0.2, 1.7], x=x)
    np.testing.assert_array_equal(g, r)
    g, r = run_both(ops, real_ref, st, rs, 3, n, [0.4], x=x, y=y)
    np.testing.assert_array_equal(g, r)
    g, r = run_both(ops, real_ref, st, rs, 4, n, [2, 9])
    # Linspace divides by a loop-invariant (length - 1); the reference's reciprocal-math build
    # multiplies by a hoisted reciprocal instead, so the last bit can differ
    np.testing.assert_allclose(g, r, rtol=3e-7, atol=0)
    g, r = run_both(ops, real_ref, st, rs, 13, n, [1.5])
    np.testing.assert_allclose(g, r, rtol=1e-5, atol=1e-6)   # pow() of two math libraries
    g, r = run_both(ops, real_ref, st, rs, 10, n, [0, 0.5], gaussian=True)
    np.testing.assert_allclose(g, r, rtol=1e-5, atol=1e-6)
    seed, pos, gen, amp, size = ops.rngState(st)
    assert (pos, gen) == (real_ref.rng_position(rs), real_ref.rng_generation(rs))
    assert gen > 1


def test_reseed_and_refresh(ops, real_ref, pair):
    st, rs, _ = pair
    ops.reSeedBuffer(None, 4242, st)
    real_ref.reseed(rs, 4242)
    g, r = run_both(ops, real_ref, st, rs, 0, 5000, [0, 1])
    np.testing.assert_array_equal(g, r)
    ops.refreshBuffer(None, 77, st)
    real_ref.refresh(rs, 77)
    g, r = run_both(ops, real_ref, st, rs, 0, 250007, [0, 1])
    np.testing.assert_array_equal(g, r)
    ops.reSeedBuffer(None, -5, st)   # a negative amplifier becomes a huge unsigned multiplier
    real_ref.reseed(rs, -5)
    g, r = run_both(ops, real_ref, st, rs, 7, 1000, [0.5])
    np.testing.assert_array_equal(g, r)


@pytest.mark.parametrize("dt,name", [(np.float64, "Double"), (np.float16, "Half")])
def test_other_types(ops, real_ref, pair, dt, name):
    st, rs, _ = pair
    g, r = run_both(ops, real_ref, st, rs, 0, 150001, [0, 1], dt=dt, name=name)
    np.testing.assert_array_equal(g, r)
    g, r = run_both(ops, real_ref, st, rs, 7, 1001, [0.25], dt=dt, name=name)
    np.testing.assert_array_equal(g, r)


def test_uniform_closed_interval_and_known_values(ops, pair):
    st, _, _ = pair
    dz = torch.zeros(8, device="cuda")
    ops.execRandomFloat(None, 0, st, dz, S.shape_info([1, 8]), dev(np.array([0, 1], np.float32)))
    # first uniforms of the reference for seed 119 / table 100000
    np.testing.assert_array_equal(host(dz)[:4], np.array([0.404720545, 0.550942004, 0.127938554, 0.622450352], np.float32))
    assert ops.rngState(st)[1] == 8


def test_strided_output_uses_f_order_coordinates(ops, real_ref, pair):
    """A non-linear output view is filled through f-order coordinates, which fixes which element
    receives which draw (include/loops/cpu/random.cpp:175)."""
    st, rs, _ = pair
    shape = (6, 10)
    parent = np.zeros((6, 20), np.float32)
    info = S.shape_info(shape, "c", [20, 2], ews=-1)
    want = parent.ravel().copy()
    real_ref.random(0, rs, want, info, np.array([0, 1], np.float32))
    dz = dev(parent.ravel())
    ops.execRandomFloat(None, 0, st, dz, info, dev(np.array([0, 1], np.float32)))
    np.testing.assert_array_equal(host(dz), want)


def test_sharded_ranges_reassemble_the_full_call(ops, real_ref, pair):
    """Offset-sharding: G independent range calls with global indices reproduce one full call
    bit for bit (Gaussian within tolerance), and a single rewind matches the reference state."""
    st, rs, _ = pair
    n, G = 1 << 20, 8
    zi = S.shape_info([1, n])
    for op, extra, arity in ((0, [0, 1], 0), (7, [0.3], 0), (2, [0.5], 1), (6, [0, 1], 2)):
        ex = np.array(extra, np.float32)
        x = np.random.default_rng(op).standard_normal(n).astype(np.float32)
        want = np.zeros(n, np.float32)
        if arity == 0:
            real_ref.random(op, rs, want, zi, ex)
        elif arity == 1:
            real_ref.random_x(op, rs, x, zi, want, zi, ex)
        else:
            real_ref.random_xy(op, rs, want, zi, want, zi, want, zi, ex)
        dz = torch.zeros(n, device="cuda")
        dx = dev(x)
        per = n // G
        for g in range(G):
            zs = dz[g * per:(g + 1) * per]
            xs = dx[g * per:(g + 1) * per] if arity == 1 else (zs if arity == 2 else None)
            ys = zs if arity == 2 else None
            ops.execRandomRange(FLOAT, None, op, arity, st, xs, ys, zs, dev(ex), g * per, per, n)
        ops.rngRewind(st, n)
        if op == 6:
            np.testing.assert_allclose(host(dz), want, atol=1e-5, rtol=0)
        else:
            np.testing.assert_array_equal(host(dz), want)
        assert ops.rngState(st)[1:3] == (real_ref.rng_position(rs), real_ref.rng_generation(rs))


def test_large_uniform_properties(ops, pair):
    """2^26 draws: mean/variance of U(0,1), every value inside the closed interval, and a
    re-run from the same state reproduces the same bits."""
    st, _, _ = pair
    n = 1 << 26
    zi = S.shape_info([1, n])
    ex = dev(np.array([0, 1], np.float32))
    state = ops.rngState(st)
    a = torch.zeros(n, device="cuda")
    ops.execRandomFloat(None, 0, st, a, zi, ex)
    assert 0.0 <= float(a.min()) and float(a.max()) <= 1.0
    assert abs(float(a.double().mean()) - 0.5) < 2e-4
    assert abs(float(a.double().var()) - 1 / 12) < 2e-4
    ops.rngSetState(st, *state[:4])
    b = torch.zeros(n, device="cuda")
    ops.execRandomFloat(None, 0, st, b, zi, ex)
    assert torch.equal(a, b)




@pytest.mark.parametrize("dt,name", [(np.float32, "Float"), (np.float64, "Double"), (np.float16, "Half")])
def test_binomial_and_binomial_ex_bit_exact(ops, real_ref, pair, dt, name):
    """BinomialDistribution with one probability (y aliases z) and with per-trial probabilities,
    BinomialDistributionEx with per-element probabilities; then a Uniform call, which only matches
    if the state advanced by zLength * trials as in the reference (special_random_ops.h:474-650)."""
    st, rs, _ = pair
    n, trials = 5000, 7
    zi = S.shape_info([1, n])
    fn = getattr(ops, "execRandom" + name)
    rng = np.random.default_rng(5)
    # 8, scalar probability: x, y and z are the same buffer
    ex = np.array([trials, 0.35], dtype=dt)
    z = np.zeros(n, dt); dz = dev(z)
    fn(None, 8, st, dz, zi, dz, zi, dz, zi, dev(ex))
    real_ref.random_xy(8, rs, z, zi, z, zi, z, zi, ex)
    np.testing.assert_array_equal(host(dz), z)
    assert 0 < z.mean() < trials
    # 8, one probability per trial
    probs = rng.uniform(0.1, 0.9, trials).astype(dt)
    pi = S.shape_info([1, trials])
    z = np.zeros(n, dt); dz = dev(z)
    fn(None, 8, st, dz, zi, dev(probs), pi, dz, zi, dev(ex))
    real_ref.random_xy(8, rs, z, zi, probs, pi, z, zi, ex)
    np.testing.assert_array_equal(host(dz), z)
    # 9, one probability per element
    probs = rng.uniform(0.0, 1.0, n).astype(dt)
    z = np.zeros(n, dt); dz = dev(z)
    fn(None, 9, st, dz, zi, dev(probs), zi, dz, zi, dev(ex))
    real_ref.random_xy(9, rs, z, zi, probs, zi, z, zi, ex)
    np.testing.assert_array_equal(host(dz), z)
    # the states moved in step
    got, want = run_both(ops, real_ref, st, rs, 0, 1000, [0.0, 1.0], dt=dt, name=name)
    np.testing.assert_array_equal(got, want)


@pytest.mark.parametrize("dt,name", [(np.float32, "Float"), (np.float64, "Double"), (np.float16, "Half")])
def test_choice_bit_exact(ops, real_ref, pair, dt, name):
    """Choice: z[e] = x[f] for the first f whose running probability sum reaches the draw; the sums are
    accumulated in the element type (special_random_ops.h:176-190)."""
    st, rs, _ = pair
    n, k = 20000, 37
    rng = np.random.default_rng(6)
    values = rng.standard_normal(k).astype(dt)
    probs = rng.uniform(0.0, 1.0, k)
    probs = (probs / probs.sum()).astype(dt)
    zi, ki = S.shape_info([1, n]), S.shape_info([1, k])
    ex = np.array([1.0], dtype=dt)
    z = np.zeros(n, dt); dz = dev(z)
    getattr(ops, "execRandom" + name)(None, 5, st, dev(values), ki, dev(probs), ki, dz, zi, dev(ex))
    real_ref.random_xy(5, rs, values, ki, probs, ki, z, zi, ex)
    np.testing.assert_array_equal(host(dz), z)
    assert len(np.unique(z)) > k // 2
    got, want = run_both(ops, real_ref, st, rs, 0, 1000, [0.0, 1.0], dt=dt, name=name)
    np.testing.assert_array_equal(got, want)


@pytest.mark.parametrize("dt,name,n", [(np.float32, "Float", 200001), (np.float64, "Double", 100000), (np.float32, "Float", 2)])
def test_truncated_normal_matches_up_to_boundary_flips(ops, real_ref, pair, dt, name, n):
    """TruncatedNormalDistribution (special_random_ops.h:654-806): pairs (e, e + middle) are redrawn until both
    samples lie within two standard deviations. The uniforms are bit-exact, so the GPU takes the same draws as
    the reference except where a sample is within rounding of the boundary (device log / cos / sin against
    glibc's): those elements are counted, everything else agrees to 1e-5 like the Gaussian op."""
    st, rs, _ = pair
    zi = S.shape_info([1, n])
    ex = np.array([0.25, 1.5], dtype=dt)
    z = np.zeros(n, dt)
    dz = dev(z)
    getattr(ops, "execRandom" + name)(None, 11, st, dz, zi, dz, zi, dz, zi, dev(ex))
    real_ref.random_xy(11, rs, z, zi, z, zi, z, zi, ex)
    got = host(dz)
    assert (np.abs(got) + 0.25 <= 3.0 + 1e-5).all()                       # |mean| + |result| <= 2 stddev
    flipped = int((np.abs(got - z) > 1e-5).sum())
    assert flipped <= max(2, n // 20000), "%d of %d elements took another draw than the reference" % (flipped, n)
    assert n < 100 or 0.5 < float(got.std()) < 1.5
    # the state moved by n on both sides
    a, b = run_both(ops, real_ref, st, rs, 0, 1000, [0.0, 1.0], dt=dt, name=name)
    np.testing.assert_array_equal(a, b)


def test_truncated_normal_per_element_means_and_refusals(ops, real_ref, pair):
    st, rs, _ = pair
    n = 50001                                                             # odd: the last pair has one member
    zi = S.shape_info([1, n])
    ex = np.array([0.0, 2.0], np.float32)
    means = np.random.default_rng(3).uniform(-1, 1, n).astype(np.float32)
    z = np.zeros(n, np.float32)
    dz = dev(z)
    ops.execRandomFloat(None, 11, st, dz, zi, dev(means), zi, dz, zi, dev(ex))
    real_ref.random_xy(11, rs, z, zi, np.concatenate([means, means[-1:]]), zi, z, zi, ex)
    got = host(dz)
    assert int((np.abs(got - z) > 1e-5).sum()) <= 3
    with pytest.raises(RuntimeError, match="ever accepted"):              # the reference would loop forever
        ops.execRandomFloat(None, 11, st, dz, zi, dz, zi, dz, zi, dev(np.array([5.0, 1.0], np.float32)))
