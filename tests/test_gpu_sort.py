"""sort / sortTad on the GPU (NativeOps.h:2940-2952; include/ops/impl/specials.cpp:457-564). A sorted
sequence does not depend on the sorting algorithm, so the expectation is numpy's sort of the same values laid
out over the same positions (tests/test_oracle_utilities.py holds that expectation against the reference's own
quicksort), and where oracle/_ref is present the reference's CPU sort is run on the same buffer as well;
inputs have no NaN, and equal values are interchangeable."""
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


_values = U.sort_values


@pytest.mark.parametrize("dt,name", NAMES)
@pytest.mark.parametrize("n", [1, 2, 3, 31, 256, 257, 2048, 2049, 8192, 8193, 20000, 65536, 100003])
@pytest.mark.parametrize("descending", [False, True])
def test_sort_whole_array(ops, maybe_ref, dt, name, n, descending):
    rng = np.random.default_rng(n)
    x = _values(rng, n, dt)
    dx = dev(x)
    getattr(ops, "sort" + name)(None, dx, S.shape_info([1, n]), descending)
    want = np.sort(x)[::-1] if descending else np.sort(x)
    np.testing.assert_array_equal(host(dx), want)
    if maybe_ref is not None and dt != np.float16:          # sortHalf is empty in the reference's CPU build
        np.testing.assert_array_equal(host(dx), maybe_ref.sort(x.copy(), S.shape_info([1, n]), descending))


def test_sort_small_known_answer(ops):
    x = np.array([5, 2, 4, 7, 1, 3, 6, 9, 8, 0], np.float32)
    dx = dev(x)
    ops.sortFloat(None, dx, S.shape_info([1, 10]), False)
    np.testing.assert_array_equal(host(dx), np.arange(10, dtype=np.float32))
    ops.sortFloat(None, dx, S.shape_info([1, 10]), True)
    np.testing.assert_array_equal(host(dx), np.arange(10, dtype=np.float32)[::-1])


@pytest.mark.parametrize("kind", ["c", "f", "cview2"])
def test_sort_walks_linear_positions(ops, maybe_ref, kind):
    # positions are i * ews, or c-order coordinates where there is no element-wise stride
    rng = np.random.default_rng(4)
    x = rng.standard_normal((37, 53)).astype(np.float32)
    lay = Layout(x, kind)
    dx = dev(lay.buffer)
    ops.sortFloat(None, dx, lay.info, False)
    got = lay.read(host(dx))
    flat = got.ravel(order="F" if kind == "f" else "C")
    np.testing.assert_array_equal(flat, np.sort(x.ravel()))
    if maybe_ref is not None:
        np.testing.assert_array_equal(got, lay.read(maybe_ref.sort(lay.buffer.copy(), lay.info, False)))


@pytest.mark.parametrize("dt,name", NAMES)
@pytest.mark.parametrize("shape,dim", [((64, 10), 1), ((64, 10), 0), ((33, 300), 1), ((7, 3000), 1), ((3, 9000), 1),
                                       ((2, 20001), 1), ((3, 20000), 1), ((5, 6, 7), 2), ((5, 6, 7), 0)])
@pytest.mark.parametrize("kind", ["c", "f"])
@pytest.mark.parametrize("descending", [False, True])
def test_sort_tad(ops, maybe_ref, dt, name, shape, dim, kind, descending):
    rng = np.random.default_rng(sum(shape) + dim)
    x = (rng.standard_normal(shape) * 50).astype(dt)
    lay = Layout(x, kind)
    dx = dev(lay.buffer)
    getattr(ops, "sortTad" + name)(None, dx, lay.info, [dim], 1, None, None, descending)
    want = np.sort(x, axis=dim)
    if descending:
        want = np.flip(want, axis=dim)
    np.testing.assert_array_equal(lay.read(host(dx)), want)
    if maybe_ref is not None and dt != np.float16:          # sortTadHalf is empty in the reference's CPU build
        np.testing.assert_array_equal(lay.read(host(dx)), lay.read(maybe_ref.sort_tad(lay.buffer.copy(), lay.info, [dim], descending)))


@pytest.mark.parametrize("dt,name", NAMES)
@pytest.mark.parametrize("descending", [False, True])
def test_sort_long_arrays_take_the_radix_path(ops, dt, name, descending):
    """From 65536 elements on a dense array is radix-sorted (8-bit digits over an order-preserving integer key):
    ragged last tile, many duplicates (every half value occurs dozens of times) and both directions."""
    n = (1 << 21) + 4097 + 13
    rng = np.random.default_rng(21)
    x = (rng.standard_normal(n) * 300).astype(dt)
    x[:6] = [np.inf, -np.inf, 0.0, -0.0, x[10], x[10]]
    dx = dev(x)
    getattr(ops, "sort" + name)(None, dx, S.shape_info([1, n]), descending)
    want = np.sort(x)[::-1] if descending else np.sort(x)
    got = host(dx)
    np.testing.assert_array_equal(got, want)
    zeros = np.flatnonzero(got == 0)
    if len(zeros) >= 2:
        assert np.signbit(got[zeros[0]]) != descending               # -0 sorts before +0


def test_sort_large_is_sorted_and_a_permutation(ops):
    # 2^24 + 5 floats: 12 stages beyond the shared-memory chunks; sortedness plus an order-independent checksum
    n = (1 << 24) + 5
    g = torch.Generator(device="cuda")
    g.manual_seed(5)
    x = torch.randn(n, device="cuda", generator=g)
    before = (x.double().sum().item(), x.double().abs().sum().item(), x.max().item(), x.min().item())
    ops.sortFloat(None, x, S.shape_info([1, n]), False)
    assert bool((x[1:] >= x[:-1]).all())
    after = (x.double().sum().item(), x.double().abs().sum().item(), x.max().item(), x.min().item())
    assert before[2:] == after[2:]
    assert abs(before[0] - after[0]) <= 1e-6 * before[1] and abs(before[1] - after[1]) <= 1e-9 * before[1]
    want = torch.sort(torch.randn(n, device="cuda", generator=g.manual_seed(5)))[0]
    assert torch.equal(x, want)


@pytest.mark.parametrize("n", [40, 5000, 30000, 70001, (1 << 20) + 9])
def test_sort_total_order_of_zeros_and_nans(ops, n):
    # on-chip keys are totally ordered: -0 before +0, NaNs (sign bit clear) after +inf; nothing is lost
    rng = np.random.default_rng(n)
    x = rng.standard_normal(n).astype(np.float32)
    x[rng.choice(n, 12, replace=False)] = [0.0, -0.0, 0.0, -0.0, np.nan, np.nan, np.inf, -np.inf, 0.0, -0.0, np.nan, 1.0]
    for descending in (False, True):
        dx = dev(x)
        ops.sortFloat(None, dx, S.shape_info([1, n]), descending)
        got = host(dx)
        if descending:
            got = got[::-1]
        want = np.sort(x)                          # numpy: NaNs last
        assert np.array_equal(np.isnan(got), np.isnan(want))
        ok = ~np.isnan(want)
        np.testing.assert_array_equal(got[ok], want[ok])
        zeros = got[got == 0]
        assert len(zeros) == 6 and np.signbit(zeros[:3]).all() and not np.signbit(zeros[3:]).any()
