"""Host-side shapeInfo / TAD decoding (the C ABI's nd4jb200_tad_only_shape_info) against the
reference's shape::TAD: known answers from the reference's tests, the committed golden
descriptors, and, where oracle/_ref is present, a randomized sweep against the live reference."""
import os

import numpy as np
import pytest

from libnd4j_b200 import native_ops, shape as S
from tests import golden_cases as G

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "legacy_ops_golden.npz")


class HostOps(native_ops.NativeOps):
    """NativeOps without touching CUDA: only the host helpers are used here."""


@pytest.fixture(scope="module")
def host_ops():
    if not os.path.exists(native_ops.LIB_PATH):
        import __graft_entry__
        __graft_entry__.build()
    return HostOps()


def test_golden_tad_descriptors(host_ops):
    gold = np.load(GOLDEN)
    for i, (shape, order, dims) in enumerate(G.TAD_CASES):
        info, offs = host_ops.tadOnlyShapeInfo(S.shape_info(shape, order), dims, len(dims))
        np.testing.assert_array_equal(info, gold["tad/%d/info" % i], err_msg=str((shape, order, dims)))
        np.testing.assert_array_equal(offs, gold["tad/%d/offsets" % i], err_msg=str((shape, order, dims)))


def test_reference_test_vectors(host_ops):
    # TadTests.cpp:22-48 of the reference: a [2,1,4,4] view with strides {80,16,4,1}, dimension 1
    bad = np.array([4, 2, 1, 4, 4, 80, 16, 4, 1, 0, -1, 99], dtype=np.int64)
    _, offs = host_ops.tadOnlyShapeInfo(bad, [1], 1)
    np.testing.assert_array_equal(offs, list(range(16)) + list(range(80, 96)))
    # descriptors printed by the reference for the benchmark's reduce input
    info, offs = host_ops.tadOnlyShapeInfo(S.shape_info([8192, 4096]), [1], 1)
    np.testing.assert_array_equal(info, [2, 1, 4096, 1, 1, 0, 1, 102])
    np.testing.assert_array_equal(offs[:4], [0, 4096, 8192, 12288])
    info, offs = host_ops.tadOnlyShapeInfo(S.shape_info([8192, 4096]), [0], 1)
    np.testing.assert_array_equal(info, [2, 1, 8192, 1, 4096, 0, 4096, 99])
    np.testing.assert_array_equal(offs[:4], [0, 1, 2, 3])
    view = S.shape_info([8, 6], "f", [1, 16], ews=-1)
    info, offs = host_ops.tadOnlyShapeInfo(view, [1], 1)
    np.testing.assert_array_equal(info, [2, 1, 6, 1, 16, 0, 16, 99])
    np.testing.assert_array_equal(offs, np.arange(8))


def test_random_sweep_against_live_reference(host_ops, real_ref):
    rng = np.random.default_rng(0)
    for _ in range(300):
        rank = int(rng.integers(2, 6))
        shape = [int(v) for v in rng.integers(2, 6, rank)]
        order = "c" if rng.random() < 0.5 else "f"
        nd = int(rng.integers(1, rank))
        dims = sorted(int(d) for d in rng.choice(rank, nd, replace=False))
        info = S.shape_info(shape, order)
        want_info, want_off = real_ref.tad(info, dims)
        got_info, got_off = host_ops.tadOnlyShapeInfo(info, dims, len(dims))
        np.testing.assert_array_equal(got_off, want_off, err_msg=str((shape, order, dims)))
        np.testing.assert_array_equal(got_info, want_info, err_msg=str((shape, order, dims)))


def test_dimension_list_recovered_from_the_tad_descriptor(host_ops, real_ref):
    """nd4jb200_dims_from_tad: given the array's shapeInfo and the REFERENCE's TAD shapeInfo for some dimension
    list (what a caller of the CUDA build keeps on the host), the recovered list must produce the same TADs:
    same count, same length, same base offsets and the same element offsets inside a TAD."""
    rng = np.random.default_rng(1)
    for trial in range(400):
        rank = int(rng.integers(1, 6))
        shape = [int(v) for v in rng.integers(1, 5, rank)]
        if trial % 3 == 0:
            shape = [int(v) for v in rng.integers(2, 5, rank)]     # no unit axes
        order = "c" if rng.random() < 0.5 else "f"
        nd = int(rng.integers(1, rank + 1))
        dims = sorted(int(d) for d in rng.choice(rank, nd, replace=False))
        info = S.shape_info(shape, order)
        ref_tad, ref_off = real_ref.tad(info, dims)
        got = host_ops.dimsFromTad(info, ref_tad)
        assert got is not None, (shape, order, dims, ref_tad)
        what = str((shape, order, dims, got))
        if not got:                                                 # whole array
            assert int(np.prod(shape)) == int(np.prod(S.shape_of(ref_tad))), what
            continue
        _, off = host_ops.tadOnlyShapeInfo(info, got, len(got))
        np.testing.assert_array_equal(off, ref_off, err_msg=what)
        strides = S.strides_of(info)
        inner = lambda dd: sorted(int(np.dot(c, [strides[d] for d in dd]))
                                  for c in np.ndindex(*[shape[d] for d in dd]))
        assert inner(got) == inner(dims), what


def test_dimension_list_recovery_on_views_and_failures(host_ops):
    # f-order parent [32768, 1024], every second column: the benchmark's reduce3 view, TAD along dimension 1
    view = S.shape_info([32768, 512], "f", [1, 65536], ews=-1)
    tad, _ = host_ops.tadOnlyShapeInfo(view, [1], 1)
    assert host_ops.dimsFromTad(view, tad) == [1]
    tad, _ = host_ops.tadOnlyShapeInfo(view, [0], 1)
    assert host_ops.dimsFromTad(view, tad) == [0]
    # a descriptor that belongs to another array is refused instead of guessed
    other, _ = host_ops.tadOnlyShapeInfo(S.shape_info([7, 9]), [1], 1)
    assert host_ops.dimsFromTad(view, other) is None


def test_offsets_with_unit_axes_match_reference(host_ops, real_ref):
    for shape, dims in (((3, 1, 4), [2]), ((3, 1, 4), [0, 1]), ((1, 5), [0]), ((5, 1), [1]), ((2, 1, 1, 3), [3])):
        info = S.shape_info(shape)
        _, want_off = real_ref.tad(info, dims)
        _, got_off = host_ops.tadOnlyShapeInfo(info, dims, len(dims))
        np.testing.assert_array_equal(got_off, want_off, err_msg=str((shape, dims)))


def test_shape_helpers():
    np.testing.assert_array_equal(S.shape_info([4, 3]), [2, 4, 3, 3, 1, 0, 1, 99])   # shape::shapeBuffer(2,{4,3})
    np.testing.assert_array_equal(S.shape_info([4, 3], "f"), [2, 4, 3, 1, 4, 0, 1, 102])
    assert S.element_wise_stride([8, 6], [1, 16], "f") == -1
    assert S.element_wise_stride([8, 6], [12, 2], "c") == 2
    assert S.element_wise_stride([1, 6], [6, 1], "c") == 1
    np.testing.assert_array_equal(S.reduced_shape_info(S.shape_info([8, 6]), [1]), S.shape_info([8, 1]))
    np.testing.assert_array_equal(S.reduced_shape_info(S.shape_info([8, 6]), [0]), S.shape_info([1, 6]))
