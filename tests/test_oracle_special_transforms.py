"""The numpy restatements of the whole-array transforms (tests/special_truth.py) against the reference's own CPU
code (include/ops/special_ops.h through execTransform of oracle/_ref). CPU only."""
import numpy as np
import pytest

from libnd4j_b200 import shape as S
from tests import special_truth as T
from tests.cases import Layout

GEOMETRIES = [
    # b, c, h, w, kH, kW, sH, sW, pH, pW, dH, dW
    (2, 3, 8, 9, 3, 3, 1, 1, 0, 0, 1, 1),
    (1, 2, 7, 7, 3, 2, 2, 1, 1, 1, 1, 1),
    (2, 1, 10, 12, 2, 3, 2, 3, 1, 2, 2, 1),
    (1, 4, 5, 6, 5, 5, 1, 1, 2, 2, 1, 1),
    (3, 2, 9, 9, 3, 3, 2, 2, 0, 1, 2, 2),
    (1, 1, 4, 4, 1, 1, 1, 1, 0, 0, 1, 1),
]


def offsets(layout):
    """Buffer offsets of the layout's linear positions in its own order."""
    info = [int(v) for v in layout.info]
    return T.own_order_offsets(layout.shape, S.strides_of(layout.info), chr(info[-1]), info[-2])


def geometry(g):
    b, c, h, w, kH, kW, sH, sW, pH, pW, dH, dW = g
    return T.out_size(h, kH, sH, pH, dH), T.out_size(w, kW, sW, pW, dW)


@pytest.mark.parametrize("dt", [np.float32, np.float64])
@pytest.mark.parametrize("g", GEOMETRIES)
@pytest.mark.parametrize("kinds", [("c", "c"), ("f", "c"), ("c", "f"), ("cview2", "c"), ("f", "cview2"), ("fview2", "fview2")])
def test_im2col(real_ref, dt, g, kinds):
    b, c, h, w, kH, kW, sH, sW, pH, pW, dH, dW = g
    oH, oW = geometry(g)
    x = np.random.default_rng(sum(g)).standard_normal((b, c, h, w)).astype(dt)
    lx, lz = Layout(x, kinds[0]), Layout(np.full((b, c, kH, kW, oH, oW), 7, dt), kinds[1])
    extra = np.array([kH, kW, sH, sW, pH, pW, dH, dW, 0, 0], dt)
    got = real_ref.transform(37, lx.buffer.copy(), lx.info, lz.buffer.copy(), lz.info, extra)
    want = T.im2col(x, kH, kW, sH, sW, pH, pW, dH, dW, oH, oW)
    assert np.array_equal(lz.read(got).reshape(want.shape), want)


@pytest.mark.parametrize("dt", [np.float32, np.float64])
@pytest.mark.parametrize("g", GEOMETRIES)
@pytest.mark.parametrize("kinds", [("c", "c"), ("f", "c"), ("c", "f"), ("fview2", "f")])
def test_col2im(real_ref, dt, g, kinds):
    """Dense results only: the reference zeroes the first `length` elements of the result buffer, whatever its
    strides, before it adds."""
    b, c, h, w, kH, kW, sH, sW, pH, pW, dH, dW = g
    oH, oW = geometry(g)
    cols = np.random.default_rng(sum(g) + 1).standard_normal((b, c, kH, kW, oH, oW)).astype(dt)
    lx, lz = Layout(cols, kinds[0]), Layout(np.full((b, c, h, w), 7, dt), kinds[1])
    extra = np.array([sH, sW, pH, pW, h, w, dH, dW, 0], dt)
    got = real_ref.transform(36, lx.buffer.copy(), lx.info, lz.buffer.copy(), lz.info, extra)
    want = T.col2im(cols, sH, sW, pH, pW, h, w, dH, dW)
    assert np.array_equal(lz.read(got).reshape(want.shape), want)


@pytest.mark.parametrize("dt", [np.float32, np.float64])
@pytest.mark.parametrize("g", GEOMETRIES)
@pytest.mark.parametrize("mode,extra0", [(0, 0.0), (1, 0.0), (1, 1.0), (2, 2.0), (2, 3.0)])
@pytest.mark.parametrize("kinds", [("c", "c"), ("f", "f")])
def test_pooling2d(real_ref, dt, g, mode, extra0, kinds):
    b, c, h, w, kH, kW, sH, sW, pH, pW, dH, dW = g
    if pH >= kH + (kH - 1) * (dH - 1) or pW >= kW + (kW - 1) * (dW - 1):
        pytest.skip("window entirely inside the padding")
    oH, oW = geometry(g)
    x = np.random.default_rng(sum(g) + 2).standard_normal((b, c, h, w)).astype(dt)
    lx, lz = Layout(x, kinds[0]), Layout(np.zeros((b, c, oH, oW), dt), kinds[1])
    extra = np.array([kH, kW, sH, sW, pH, pW, dH, dW, 0, mode, extra0], dt)
    got = real_ref.transform(71, lx.buffer.copy(), lx.info, lz.buffer.copy(), lz.info, extra)
    want = T.pooling2d(x, kH, kW, sH, sW, pH, pW, dH, dW, oH, oW, mode, extra0)
    got = lz.read(got).reshape(want.shape).astype(np.float64)
    if mode == 0:
        assert np.array_equal(got, want)
    else:
        assert np.allclose(got, want, rtol=1e-5 if dt == np.float32 else 1e-12, atol=1e-6 if dt == np.float32 else 1e-13)


@pytest.mark.parametrize("dt", [np.float32, np.float64])
@pytest.mark.parametrize("n,bins", [(1000, 10), (4099, 64), (65536, 256), (17, 3)])
def test_histogram(real_ref, dt, n, bins):
    x = np.random.default_rng(n).uniform(-2, 3, n).astype(dt)
    z0 = np.arange(bins).astype(dt)                            # the reference adds to what the result holds
    extra = np.array([bins, -1.5, 2.5], dt)
    got = real_ref.transform(48, x.copy(), S.shape_info([1, n]), z0.copy(), S.shape_info([1, bins]), extra)
    assert np.array_equal(got, T.histogram(x, z0, bins, -1.5, 2.5))


@pytest.mark.parametrize("dt", [np.float32, np.float64])
@pytest.mark.parametrize("shape", [(1, 17), (6, 7), (3, 4, 5)])
@pytest.mark.parametrize("kinds", [("c", "c"), ("f", "f"), ("c", "f"), ("cview2", "c"), ("f", "cview2"), ("fview2", "fview2")])
def test_reverse(real_ref, dt, shape, kinds):
    x = np.random.default_rng(len(shape)).standard_normal(shape).astype(dt)
    lx, lz = Layout(x, kinds[0]), Layout(np.zeros(shape, dt), kinds[1])
    got = real_ref.transform(70, lx.buffer.copy(), lx.info, lz.buffer.copy(), lz.info, None)
    xo, zo = offsets(lx), offsets(lz)
    want = lz.buffer.copy()
    want[zo[::-1]] = lx.buffer[xo]
    assert np.array_equal(got, want, equal_nan=True)


@pytest.mark.parametrize("kind", ["c", "f", "cview2", "fview2"])
@pytest.mark.parametrize("shape", [(1, 16), (1, 17), (5, 6)])
def test_reverse_in_place(real_ref, kind, shape):
    x = np.random.default_rng(3).standard_normal(shape).astype(np.float32)
    lx = Layout(x, kind)
    buf = lx.buffer.copy()
    got = real_ref.transform(70, buf, lx.info, buf, lx.info, None)
    o = offsets(lx)
    n = x.size
    want = lx.buffer.copy()
    if int(lx.info[-2]) >= 1:
        want[o] = lx.buffer[o[::-1]]
    else:                                                      # the first half is copied over the second, not swapped
        half = n // 2
        want[o[::-1][:half]] = lx.buffer[o[:half]]
    assert np.array_equal(got, want, equal_nan=True)
