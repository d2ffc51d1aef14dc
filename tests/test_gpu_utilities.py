"""flatten / concat / pullRows / tear / shuffle / average / accumulate / convertTypes on the GPU. They move or
add elements without any transcendental arithmetic, so every result must be bit-exact. Expected values come
from the reference's own CPU NativeOps members (oracle/_ref, when it was built) and from numpy restatements of
the same loops (tests/utility_truth.py), which tests/test_oracle_utilities.py holds against the reference."""
import numpy as np
import pytest
import torch

from libnd4j_b200 import shape as S
from tests.cases import Layout
from tests import utility_truth as U

pytestmark = pytest.mark.gpu

NAMES = [(np.float32, "Float"), (np.float64, "Double"), (np.float16, "Half")]


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def host(t):
    return t.cpu().numpy()


@pytest.mark.parametrize("dt,name", NAMES)
@pytest.mark.parametrize("order", ["c", "f"])
@pytest.mark.parametrize("kind", ["c", "f", "cview2"])
def test_flatten_orders_and_offset(ops, maybe_ref, dt, name, order, kind):
    rng = np.random.default_rng(3)
    x = rng.standard_normal((6, 5, 4)).astype(dt)
    lay = Layout(x, kind)
    total = x.size + 17
    z = np.full(total, -1, dt)
    dz = dev(z)
    getattr(ops, "flatten" + name)(None, 9, order, dz, S.shape_info([1, total]), dev(lay.buffer), lay.info)
    np.testing.assert_array_equal(host(dz), U.flatten_truth(z, 9, order, x))
    if maybe_ref is not None and dt != np.float16:          # flattenHalf is empty in the reference's CPU build
        want = maybe_ref.flatten(9, order, z.copy(), S.shape_info([1, total]), lay.buffer.copy(), lay.info)
        np.testing.assert_array_equal(host(dz), want)


@pytest.mark.parametrize("dt,name", NAMES)
@pytest.mark.parametrize("dim", [0, 1, 2])
def test_concat_along_each_axis(ops, maybe_ref, dt, name, dim):
    rng = np.random.default_rng(dim)
    base = [3, 4, 5]
    parts = []
    for extent in (2, 1, 4):
        shp = list(base)
        shp[dim] = extent
        parts.append(rng.standard_normal(shp).astype(dt))
    want = np.concatenate(parts, axis=dim)
    # inputs in mixed layouts: c-order, f-order, strided view
    lays = [Layout(parts[0], "c"), Layout(parts[1], "f"), Layout(parts[2], "cview2")]
    dz = dev(np.zeros(want.size, dt))
    getattr(ops, "concat" + name)(None, dim, 3, [dev(l.buffer) for l in lays], [l.info for l in lays], dz,
                                  S.shape_info(list(want.shape)))
    np.testing.assert_array_equal(host(dz).reshape(want.shape), want)
    if maybe_ref is not None:
        zr = maybe_ref.concat(dim, [l.buffer for l in lays], [l.info for l in lays], np.zeros(want.size, dt),
                              S.shape_info(list(want.shape)))
        np.testing.assert_array_equal(host(dz), zr)


def test_concat_large_rows_takes_the_dense_path(ops):
    a = np.arange(4096 * 256, dtype=np.float32).reshape(4096, 256)
    b = -a[:1024]
    dz = torch.zeros(5120 * 256, device="cuda")
    ops.concatFloat(None, 0, 2, [dev(a), dev(b)], [S.shape_info([4096, 256]), S.shape_info([1024, 256])], dz,
                    S.shape_info([5120, 256]))
    np.testing.assert_array_equal(host(dz).reshape(5120, 256), np.concatenate([a, b]))
    with pytest.raises(RuntimeError):      # the inputs do not fill the result
        ops.concatFloat(None, 0, 1, [dev(a)], [S.shape_info([4096, 256])], dz, S.shape_info([5120, 256]))


@pytest.mark.parametrize("dt,name", NAMES)
@pytest.mark.parametrize("kind,dim", [("c", 1), ("f", 1), ("c", 0)])
def test_pull_rows(ops, maybe_ref, dt, name, kind, dim):
    rng = np.random.default_rng(5)
    x = rng.standard_normal((50, 24)).astype(dt)
    lay = Layout(x, kind)
    tad_info, tad_offsets = ops.tadOnlyShapeInfo(lay.info, [dim], 1)
    picks = rng.integers(0, len(tad_offsets), 13)
    rows = x[picks] if dim == 1 else x[:, picks].T
    zshape = list(rows.shape)
    zinfo = S.shape_info(zshape)
    ztad_info, ztad_offsets = ops.tadOnlyShapeInfo(zinfo, [1], 1)
    dz = dev(np.zeros(rows.size, dt))
    getattr(ops, "pullRows" + name)(None, dev(lay.buffer), lay.info, dz, zinfo, len(picks), dev(picks.astype(np.int64)),
                                    tad_info, dev(tad_offsets.astype(np.int64)), ztad_info,
                                    dev(ztad_offsets.astype(np.int64)))
    np.testing.assert_array_equal(host(dz).reshape(zshape), rows)
    if maybe_ref is not None and dt != np.float16:          # pullRowsHalf is empty in the reference's CPU build
        zr = maybe_ref.pull_rows(lay.buffer.copy(), lay.info, np.zeros(rows.size, dt), zinfo, picks, tad_info,
                                 tad_offsets, ztad_info, ztad_offsets)
        np.testing.assert_array_equal(host(dz), zr)


def test_pull_rows_pairs_by_coordinates_unless_both_sides_have_a_stride(ops, maybe_ref):
    """Source TADs with an elementWiseStride (matrices of an f-order array, walked first axis fastest) against
    target TADs without one (rows padded by one element): the reference then pairs the i-th c-order coordinate
    of both (blas/cpu/NativeOps.cpp:2072-2101), so z[k, p, q] = x[p, q, pick[k]]."""
    rng = np.random.default_rng(6)
    a, b, n, k = 5, 7, 9, 4
    x = rng.standard_normal((a, b, n)).astype(np.float32)
    lay = Layout(x, "f")
    _, tad_offsets = ops.tadOnlyShapeInfo(lay.info, [0, 1], 2)
    tad_info = S.shape_info([a, b], "f", [1, a], ews=1)               # the source TAD has a stride
    picks = rng.integers(0, n, k)
    zinfo = S.shape_info([k, a, b], "c", [a * (b + 1), b + 1, 1])     # parent [k, a, b + 1]
    ztad_info, ztad_offsets = ops.tadOnlyShapeInfo(zinfo, [1, 2], 2)
    assert ztad_info[2 * 2 + 2] < 1                                   # the target TAD has none
    zbuf = np.zeros(k * a * (b + 1), np.float32)
    dz = dev(zbuf)
    ops.pullRowsFloat(None, dev(lay.buffer), lay.info, dz, zinfo, k, dev(picks.astype(np.int64)), tad_info,
                      dev(np.asarray(tad_offsets, dtype=np.int64)), ztad_info, dev(np.asarray(ztad_offsets, dtype=np.int64)))
    got = host(dz).reshape(k, a, b + 1)[:, :, :b]
    np.testing.assert_array_equal(got, np.moveaxis(x[:, :, picks], 2, 0))
    if maybe_ref is not None:
        zr = maybe_ref.pull_rows(lay.buffer.copy(), lay.info, zbuf.copy(), zinfo, picks, tad_info, tad_offsets, ztad_info,
                                 ztad_offsets)
        np.testing.assert_array_equal(host(dz), zr)


@pytest.mark.parametrize("dt,name", NAMES)
def test_average_and_accumulate(ops, maybe_ref, dt, name):
    rng = np.random.default_rng(11)
    n, length = 5, 10007
    xs = [rng.standard_normal(length).astype(dt) for _ in range(n)]
    want_avg = U.average_truth(xs, dt)
    dxs = [dev(x) for x in xs]
    dz = dev(np.full(length, 3, dt))
    getattr(ops, "average" + name)(None, dxs, dz, n, length, False)
    got = host(dz)
    # the reference's build may replace x / n by x * (1 / n): one ulp per term at most
    assert np.abs(got.astype(np.float64) - want_avg.astype(np.float64)).max() <= n * np.spacing(np.abs(want_avg).max())
    if maybe_ref is not None and dt != np.float16:          # averageHalf is empty in the reference's CPU build
        zr = maybe_ref.average([x.copy() for x in xs], np.zeros(length, dt), False)
        assert np.abs(got.astype(np.float64) - zr.astype(np.float64)).max() <= n * np.spacing(np.abs(zr).max())
    for x, d in zip(xs, dxs):
        np.testing.assert_array_equal(host(d), x)             # sources untouched without propagate
    getattr(ops, "average" + name)(None, dxs, dz, n, length, True)
    for d in dxs:
        np.testing.assert_array_equal(host(d), host(dz))       # propagated
    # accumulate adds onto what z holds
    dxs = [dev(x) for x in xs]
    start = rng.standard_normal(length).astype(dt)
    dz = dev(start)
    getattr(ops, "accumulate" + name)(None, dxs, dz, n, length)
    np.testing.assert_array_equal(host(dz), U.accumulate_truth(xs, start, dt))
    if maybe_ref is not None:
        np.testing.assert_array_equal(host(dz), maybe_ref.accumulate([x.copy() for x in xs], start.copy()))


def test_average_into_first_source_and_limits(ops):
    xs = [np.full(1000, v, np.float32) for v in (1.0, 2.0, 6.0)]
    dxs = [dev(x) for x in xs]
    ops.averageFloat(None, dxs, None, 3, 1000, True)
    for d in dxs:
        np.testing.assert_array_equal(host(d), np.full(1000, 3.0, np.float32))
    with pytest.raises(RuntimeError):
        ops.averageFloat(None, [dxs[0]] * 129, None, 129, 1000, False)


from tests.convert_truth import CODES, SOURCES, RESULTS, convert_truth, convert_inputs


@pytest.mark.parametrize("src", SOURCES)
@pytest.mark.parametrize("dst", RESULTS)
@pytest.mark.parametrize("misalign", [0, 1])
def test_convert_types_goes_through_float(ops, src, dst, misalign):
    """z = (D)(float) x (include/loops/type_conversions.h:592-610, 696-880): bit-exact against numpy's IEEE
    conversions (overflow to infinity, subnormal halves) and the saturating integer wrappers. The pairs the
    reference's dispatch leaves out (int8 -> int8, float32 -> float32, double -> double) leave z untouched."""
    x = convert_inputs(src)
    untouched = src == dst and src in (np.int8, np.float32, np.float64)
    # `misalign` shifts both buffers by one element so that the four-element vector path cannot be taken
    dx = dev(np.concatenate([x[:1], x]))[misalign:]
    dz = dev(np.full(x.size + 1, 7, dst))[misalign:]
    n = x.size + 1 - misalign
    xs = host(dx)
    ops.convertTypes(None, CODES[src], dx, n, CODES[dst], dz)
    got = host(dz)
    if untouched:
        assert (got == 7).all()
    else:
        want = convert_truth(xs, dst)
        if np.issubdtype(dst, np.floating):
            # a NaN stays a NaN; its payload bits are not compared (the reference's float16 class and IEEE
            # hardware conversions pick different ones)
            nan = np.isnan(want)
            assert np.array_equal(np.isnan(got), nan)
            got, want = np.where(nan, 0, got).astype(dst), np.where(nan, 0, want).astype(dst)
        assert np.array_equal(got.view(np.uint8), want.view(np.uint8))


@pytest.mark.parametrize("misalign", [0, 1])
def test_convert_types_float8(ops, maybe_ref, misalign):
    """The 8-bit float of include/types/float8.h (type code 0) as source and as result, bit for bit, including
    the reference's half-precision thresholds and x86 shift counts in its float -> float8 routine."""
    from tests import convert_truth as C
    q = C.float8_inputs()
    for dst in RESULTS:
        dx = dev(np.concatenate([q[:1], q]))[misalign:]
        dz = dev(np.full(q.size + 1, 7, dst))[misalign:]
        n = q.size + 1 - misalign
        src_host = host(dx)
        ops.convertTypes(None, C.FLOAT8, dx, n, CODES[dst], dz)
        got, want = host(dz), C.convert_truth_from_float8(src_host, dst)
        if np.issubdtype(dst, np.floating):
            nan = np.isnan(want)
            assert np.array_equal(np.isnan(got), nan)
            got, want = np.where(nan, 0, got).astype(dst), np.where(nan, 0, want).astype(dst)
        assert np.array_equal(got.view(np.uint8), want.view(np.uint8)), dst
    rng = np.random.default_rng(0)
    f = rng.integers(0, 2 ** 32, 100001, dtype=np.uint64).astype(np.uint32).view(np.float32)
    for src in SOURCES:
        x = f if src == np.float32 else convert_inputs(src)
        dx = dev(np.concatenate([x[:1], x]))[misalign:]
        dz = dev(np.full(x.size + 1, 9, np.uint8))[misalign:]
        ops.convertTypes(None, CODES[src], dx, x.size + 1 - misalign, C.FLOAT8, dz)
        xs = host(dx)
        np.testing.assert_array_equal(host(dz), C.convert_truth_to_float8(xs), err_msg=str(src))
        if maybe_ref is not None:
            np.testing.assert_array_equal(host(dz), maybe_ref.convert_types(CODES[src], xs.copy(), C.FLOAT8, np.full(xs.size, 9, np.uint8)))
    z = dev(np.full(16, 7, np.uint8))
    ops.convertTypes(None, 0, dev(q[:16]), 16, 0, z)          # float8 -> float8 is left out by the reference's dispatch
    assert (host(z) == 7).all()


def test_convert_types_unserved_encodings(ops):
    x = dev(np.zeros(16, np.float32))
    z = dev(np.zeros(16, np.float32))
    for src, dst in ((8, 6), (6, 8), (5, 6), (9, 6)):      # threshold encodings; no conversion from uint16
        with pytest.raises(RuntimeError):
            ops.convertTypes(None, src, x, 16, dst, z)


def _tad_view(x, lay, ops, dims):
    """TAD descriptors of a laid-out array, plus a function giving TAD k of the logical array."""
    tad_info, tad_offsets = ops.tadOnlyShapeInfo(lay.info, dims, len(dims))
    return tad_info, np.asarray(tad_offsets, dtype=np.int64)


@pytest.mark.parametrize("dt,name", NAMES)
@pytest.mark.parametrize("kind,dim,zorder", [("c", 1, "c"), ("f", 1, "c"), ("c", 0, "c"), ("cview2", 1, "c"), ("c", 1, "f")])
def test_tear_rows_and_columns(ops, maybe_ref, dt, name, kind, dim, zorder):
    # TAD k of x lands in its own array (blas/cpu/NativeOps.cpp:2119-2162)
    rng = np.random.default_rng(21)
    x = rng.standard_normal((12, 40)).astype(dt)
    lay = Layout(x, kind)
    tad_info, tad_offsets = _tad_view(x, lay, ops, [dim])
    pieces = [x[k] if dim == 1 else x[:, k] for k in range(len(tad_offsets))]
    zshape = [1, pieces[0].size]
    zinfo = S.shape_info(zshape, zorder)
    targets = [dev(np.zeros(p.size, dt)) for p in pieces]
    getattr(ops, "tear" + name)(None, dev(lay.buffer), lay.info, targets, zinfo, tad_info, dev(tad_offsets))
    for t, p in zip(targets, pieces):
        np.testing.assert_array_equal(host(t), p)
    if maybe_ref is not None:
        rt = maybe_ref.tear(lay.buffer.copy(), lay.info, [np.zeros(p.size, dt) for p in pieces], zinfo, tad_info, tad_offsets)
        for t, r in zip(targets, rt):
            np.testing.assert_array_equal(host(t), r)


def test_tear_matrices_in_f_order_enumeration(ops, maybe_ref):
    # neither side addressable by one stride: element j of a TAD in f-order goes to element j of the target in f-order
    rng = np.random.default_rng(22)
    x = rng.standard_normal((5, 6, 7)).astype(np.float32)
    lay = Layout(x, "cview2")
    tad_info, tad_offsets = _tad_view(x, lay, ops, [1, 2])
    zlay = Layout(np.zeros((6, 7), np.float32), "fview2")
    targets = [dev(zlay.buffer) for _ in range(5)]
    ops.tearFloat(None, dev(lay.buffer), lay.info, targets, zlay.info, tad_info, dev(tad_offsets))
    for k, t in enumerate(targets):
        np.testing.assert_array_equal(zlay.read(host(t)), x[k])
    if maybe_ref is not None:
        rt = maybe_ref.tear(lay.buffer.copy(), lay.info, [zlay.buffer.copy() for _ in range(5)], zlay.info, tad_info, tad_offsets)
        for t, r in zip(targets, rt):
            np.testing.assert_array_equal(zlay.read(host(t)), zlay.read(r))


def test_tear_few_long_tads_are_cut_into_chunks(ops):
    x = np.arange(3 * 100003, dtype=np.float32).reshape(3, 100003)      # odd length: no 16-byte rows
    y = np.arange(4 * 65536, dtype=np.float64).reshape(4, 65536)
    for a, name in ((x, "Float"), (y, "Double")):
        info = S.shape_info(list(a.shape))
        tad_info, tad_offsets = ops.tadOnlyShapeInfo(info, [1], 1)
        targets = [dev(np.zeros(a.shape[1], a.dtype)) for _ in range(a.shape[0])]
        getattr(ops, "tear" + name)(None, dev(a), info, targets, S.shape_info([1, a.shape[1]]), tad_info,
                                    dev(np.asarray(tad_offsets, dtype=np.int64)))
        for k, t in enumerate(targets):
            np.testing.assert_array_equal(host(t), a[k])


_shuffled, _half_map, MAPS = U.shuffled, U.half_map, U.MAPS


@pytest.mark.parametrize("dt,name", NAMES)
@pytest.mark.parametrize("which", sorted(MAPS))
@pytest.mark.parametrize("kind,dim", [("c", 1), ("f", 1), ("c", 0)])
def test_shuffle_features_and_labels_together(ops, maybe_ref, dt, name, which, kind, dim):
    rng = np.random.default_rng(31)
    n = 21
    feats = rng.standard_normal((n, 36) if dim == 1 else (36, n)).astype(dt)
    labels = rng.standard_normal((n, 5) if dim == 1 else (5, n)).astype(dt)
    shuffle_map = MAPS[which](n, rng)
    lays = [Layout(feats, kind), Layout(labels, kind)]
    bufs = [dev(l.buffer) for l in lays]
    tads = [ops.tadOnlyShapeInfo(l.info, [dim], 1) for l in lays]
    getattr(ops, "shuffle" + name)(None, bufs, [l.info for l in lays], None, None, 2, shuffle_map,
                                   [t[0] for t in tads], [dev(np.asarray(t[1], dtype=np.int64)) for t in tads])
    axis = 0 if dim == 1 else 1
    for lay, buf, a in zip(lays, bufs, (feats, labels)):
        np.testing.assert_array_equal(lay.read(host(buf)), _shuffled(a, axis, shuffle_map))
    if maybe_ref is not None and dt != np.float16:          # shuffleHalf is empty in the reference's CPU build
        rb = maybe_ref.shuffle([l.buffer.copy() for l in lays], [l.info for l in lays], shuffle_map, [t[0] for t in tads],
                               [t[1] for t in tads])
        for lay, buf, r in zip(lays, bufs, rb):
            np.testing.assert_array_equal(lay.read(host(buf)), lay.read(r))


def test_shuffle_long_rows_and_bad_map(ops):
    rng = np.random.default_rng(32)
    x = rng.standard_normal((64, 8192)).astype(np.float32)        # 32 KB rows: two chunks each, dense packs
    info = S.shape_info([64, 8192])
    tad_info, tad_offsets = ops.tadOnlyShapeInfo(info, [1], 1)
    offs = dev(np.asarray(tad_offsets, dtype=np.int64))
    shuffle_map = _half_map(64, rng)
    dx = dev(x)
    ops.shuffleFloat(None, [dx], [info], None, None, 1, shuffle_map, [tad_info], [offs])
    np.testing.assert_array_equal(host(dx), _shuffled(x, 0, shuffle_map))
    bad = shuffle_map.copy()
    bad[3] = 64
    with pytest.raises(RuntimeError):
        ops.shuffleFloat(None, [dx], [info], None, None, 1, bad, [tad_info], [offs])
