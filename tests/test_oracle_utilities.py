"""Pins the numpy restatements of the memory-movement utilities (tests/utility_truth.py) against the
reference's own CPU `NativeOps` members (blas/cpu/NativeOps.cpp, compiled in place into oracle/_ref behind
oracle/ref_nativeops.cpp). The GPU tests use the same restatements and, where oracle/_ref is present, the
reference itself as expected values; this file is what makes the restatements trustworthy. CPU only."""
import numpy as np
import pytest

from libnd4j_b200 import shape as S
from tests.cases import Layout
from tests import utility_truth as U

DTS = [np.float32, np.float64]


@pytest.mark.parametrize("dt", DTS)
@pytest.mark.parametrize("order", ["c", "f"])
@pytest.mark.parametrize("kind", ["c", "f", "cview2"])
def test_flatten_restatement(real_ref, dt, order, kind):
    rng = np.random.default_rng(3)
    x = rng.standard_normal((6, 5, 4)).astype(dt)
    lay = Layout(x, kind)
    total = x.size + 17
    z = np.full(total, -1, dt)
    got = real_ref.flatten(9, order, z.copy(), S.shape_info([1, total]), lay.buffer.copy(), lay.info)
    np.testing.assert_array_equal(got, U.flatten_truth(z, 9, order, x))


@pytest.mark.parametrize("dt", DTS + [np.float16])
@pytest.mark.parametrize("dim", [0, 1, 2])
def test_concat_restatement(real_ref, dt, dim):
    rng = np.random.default_rng(dim)
    parts = []
    for extent in (2, 1, 4):
        shp = [3, 4, 5]
        shp[dim] = extent
        parts.append(rng.standard_normal(shp).astype(dt))
    want = np.concatenate(parts, axis=dim)
    lays = [Layout(parts[0], "c"), Layout(parts[1], "f"), Layout(parts[2], "cview2")]
    z = np.zeros(want.size, dt)
    real_ref.concat(dim, [l.buffer for l in lays], [l.info for l in lays], z, S.shape_info(list(want.shape)))
    np.testing.assert_array_equal(z.reshape(want.shape), want)


@pytest.mark.parametrize("dt", DTS)
@pytest.mark.parametrize("kind,dim", [("c", 1), ("f", 1), ("c", 0)])
def test_pull_rows_restatement(real_ref, dt, kind, dim):
    rng = np.random.default_rng(5)
    x = rng.standard_normal((50, 24)).astype(dt)
    lay = Layout(x, kind)
    tad_info, tad_offsets = real_ref.tad(lay.info, [dim])
    picks = rng.integers(0, len(tad_offsets), 13)
    rows = x[picks] if dim == 1 else x[:, picks].T
    zinfo = S.shape_info(list(rows.shape))
    ztad_info, ztad_offsets = real_ref.tad(zinfo, [1])
    z = np.zeros(rows.size, dt)
    real_ref.pull_rows(lay.buffer.copy(), lay.info, z, zinfo, picks, tad_info, tad_offsets, ztad_info, ztad_offsets)
    np.testing.assert_array_equal(z.reshape(rows.shape), rows)


@pytest.mark.parametrize("dt", DTS + [np.float16])
@pytest.mark.parametrize("kind,dim,zorder", [("c", 1, "c"), ("f", 1, "c"), ("c", 0, "c"), ("cview2", 1, "c"), ("c", 1, "f")])
def test_tear_restatement(real_ref, dt, kind, dim, zorder):
    rng = np.random.default_rng(21)
    x = rng.standard_normal((12, 40)).astype(dt)
    lay = Layout(x, kind)
    tad_info, tad_offsets = real_ref.tad(lay.info, [dim])
    pieces = [x[k] if dim == 1 else x[:, k] for k in range(len(tad_offsets))]
    targets = [np.zeros(p.size, dt) for p in pieces]
    real_ref.tear(lay.buffer.copy(), lay.info, targets, S.shape_info([1, pieces[0].size], zorder), tad_info, tad_offsets)
    for t, p in zip(targets, pieces):
        np.testing.assert_array_equal(t, p)


def test_tear_matrices_restatement(real_ref):
    rng = np.random.default_rng(22)
    x = rng.standard_normal((5, 6, 7)).astype(np.float32)
    lay = Layout(x, "cview2")
    tad_info, tad_offsets = real_ref.tad(lay.info, [1, 2])
    zlay = Layout(np.zeros((6, 7), np.float32), "fview2")
    targets = [zlay.buffer.copy() for _ in range(5)]
    real_ref.tear(lay.buffer.copy(), lay.info, targets, zlay.info, tad_info, tad_offsets)
    for k, t in enumerate(targets):
        np.testing.assert_array_equal(zlay.read(t), x[k])


@pytest.mark.parametrize("dt", DTS)
@pytest.mark.parametrize("which", sorted(U.MAPS))
@pytest.mark.parametrize("kind,dim", [("c", 1), ("f", 1), ("c", 0)])
def test_shuffle_restatement(real_ref, dt, which, kind, dim):
    rng = np.random.default_rng(31)
    n = 21
    feats = rng.standard_normal((n, 36) if dim == 1 else (36, n)).astype(dt)
    labels = rng.standard_normal((n, 5) if dim == 1 else (5, n)).astype(dt)
    shuffle_map = U.MAPS[which](n, rng)
    lays = [Layout(feats, kind), Layout(labels, kind)]
    bufs = [l.buffer.copy() for l in lays]
    tads = [real_ref.tad(l.info, [dim]) for l in lays]
    real_ref.shuffle(bufs, [l.info for l in lays], shuffle_map, [t[0] for t in tads], [t[1] for t in tads])
    axis = 0 if dim == 1 else 1
    for lay, buf, a in zip(lays, bufs, (feats, labels)):
        np.testing.assert_array_equal(lay.read(buf), U.shuffled(a, axis, shuffle_map))


@pytest.mark.parametrize("dt", DTS)
def test_average_and_accumulate_restatement(real_ref, dt):
    rng = np.random.default_rng(11)
    n, length = 5, 10007
    xs = [rng.standard_normal(length).astype(dt) for _ in range(n)]
    z = np.full(length, 3, dt)
    real_ref.average([x.copy() for x in xs], z, False)
    want = U.average_truth(xs, dt)
    # the reference's build may replace x / n by x * (1 / n): one ulp per term at most
    assert np.abs(z.astype(np.float64) - want.astype(np.float64)).max() <= n * np.spacing(np.abs(want).max())
    srcs = [x.copy() for x in xs]
    real_ref.average(srcs, z, True)
    for s in srcs:
        np.testing.assert_array_equal(s, z)
    start = rng.standard_normal(length).astype(dt)
    z = start.copy()
    real_ref.accumulate([x.copy() for x in xs], z)
    np.testing.assert_array_equal(z, U.accumulate_truth(xs, start, dt))


def test_accumulate_half_restatement(real_ref):
    rng = np.random.default_rng(12)
    xs = [rng.standard_normal(4099).astype(np.float16) for _ in range(4)]
    start = rng.standard_normal(4099).astype(np.float16)
    z = start.copy()
    real_ref.accumulate([x.copy() for x in xs], z)
    np.testing.assert_array_equal(z, U.accumulate_truth(xs, start, np.float16))


@pytest.mark.parametrize("dt", DTS)
@pytest.mark.parametrize("n", [1, 2, 3, 31, 257, 2049, 20000, 100003])
@pytest.mark.parametrize("descending", [False, True])
def test_sort_is_numpy_sort(real_ref, dt, n, descending):
    """The reference's quicksort (include/ops/impl/specials.cpp:457-549) yields the sorted sequence of the
    same values, which is what numpy's sort gives: this holds the GPU tests' expectation against it."""
    x = U.sort_values(np.random.default_rng(n), n, dt)
    got = real_ref.sort(x.copy(), S.shape_info([1, n]), descending)
    want = np.sort(x)[::-1] if descending else np.sort(x)
    np.testing.assert_array_equal(got, want)


@pytest.mark.parametrize("kind", ["c", "f", "cview2"])
def test_sort_positions_restatement(real_ref, kind):
    rng = np.random.default_rng(4)
    x = rng.standard_normal((37, 53)).astype(np.float32)
    lay = Layout(x, kind)
    buf = real_ref.sort(lay.buffer.copy(), lay.info, False)
    flat = lay.read(buf).ravel(order="F" if kind == "f" else "C")
    np.testing.assert_array_equal(flat, np.sort(x.ravel()))


@pytest.mark.parametrize("dt", DTS)
@pytest.mark.parametrize("shape,dim", [((64, 10), 1), ((64, 10), 0), ((33, 300), 1), ((3, 9000), 1), ((5, 6, 7), 2), ((5, 6, 7), 0)])
@pytest.mark.parametrize("kind", ["c", "f"])
@pytest.mark.parametrize("descending", [False, True])
def test_sort_tad_is_numpy_sort_along_axis(real_ref, dt, shape, dim, kind, descending):
    rng = np.random.default_rng(sum(shape) + dim)
    x = (rng.standard_normal(shape) * 50).astype(dt)
    lay = Layout(x, kind)
    buf = real_ref.sort_tad(lay.buffer.copy(), lay.info, [dim], descending)
    want = np.sort(x, axis=dim)
    if descending:
        want = np.flip(want, axis=dim)
    np.testing.assert_array_equal(lay.read(buf), want)


@pytest.mark.parametrize("dt", DTS)
@pytest.mark.parametrize("rank,length", [(1, 30), (2, 1000), (3, 4097)])
def test_sort_coo_indices_keeps_pairs_but_is_not_a_full_sort(real_ref, dt, rank, length):
    """The reference's COO quicksort (include/ops/impl/specials_sparse.cpp:82-113) compares against the
    element at the pivot POSITION, which the partition loop itself swaps away, so its output is a permutation
    that keeps every (coordinates, value) pair together but is in general not in lexicographic order. The GPU
    entry point sorts fully (U.coo_sorted); what is common to both, and checked here, is the pairing."""
    rng = np.random.default_rng(rank * 1000 + length)
    flat = rng.choice(40 ** rank, length, replace=False)       # distinct coordinate tuples, as a COO array has them
    idx = np.stack(np.unravel_index(flat, [40] * rank), axis=1).astype(np.int64)
    vals = rng.standard_normal(length).astype(dt)
    gi, gv = real_ref.sort_coo_indices(idx.copy(), vals.copy(), rank)
    lin = np.ravel_multi_index(gi.T, [40] * rank)
    assert dict(zip(lin.tolist(), gv.tolist())) == dict(zip(flat.tolist(), vals.tolist()))
    wi, wv = U.coo_sorted(idx, vals)
    assert np.array_equal(np.ravel_multi_index(wi.T, [40] * rank), np.sort(flat))
