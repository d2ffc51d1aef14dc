"""The whole-array ("special") transforms on the GPU, through execTransform*: Col2Im 36, Im2col 37, Histogram 48,
Reverse 70, Pooling2D 71, against the numpy restatements of tests/special_truth.py (which
tests/test_oracle_special_transforms.py pins to the reference's CPU code) and, where oracle/_ref is present,
against that code directly. Data movement, integer counts and sums whose order the reference fixes are compared
bit for bit; the average and p-norm pooling, whose summation order the reference leaves to the compiler, within
1e-5 (float) / 1e-12 (double) / 2e-3 (half) relative."""
import numpy as np
import pytest
import torch

from libnd4j_b200 import shape as S
from tests import special_truth as T
from tests.cases import Layout
from tests.test_oracle_special_transforms import GEOMETRIES, geometry, offsets

pytestmark = pytest.mark.gpu

NAMES = {np.float32: "Float", np.float64: "Double", np.float16: "Half"}
BIG = [(4, 16, 28, 28, 3, 3, 1, 1, 1, 1, 1, 1), (2, 8, 57, 43, 5, 3, 2, 2, 2, 1, 1, 2), (3, 5, 64, 64, 2, 2, 2, 2, 0, 0, 1, 1),
       (1, 3, 224, 224, 7, 7, 2, 2, 3, 3, 1, 1),
       # rows whose length is a multiple of the 16-byte run of every element type, so that whole warps take the span
       # forms: seven taps per kernel row, a single tap, dilated kernel rows, four-tap pooling windows, mixed strides
       (2, 4, 32, 40, 7, 7, 1, 1, 3, 3, 1, 1), (2, 4, 32, 32, 1, 1, 1, 1, 0, 0, 1, 1), (1, 4, 40, 48, 5, 5, 1, 1, 2, 2, 2, 1),
       (2, 4, 32, 32, 4, 4, 2, 2, 1, 1, 1, 1), (2, 3, 33, 64, 3, 3, 2, 1, 1, 1, 1, 1), (2, 2, 16, 128, 2, 2, 1, 2, 0, 0, 1, 1)]


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def host(t):
    return t.cpu().numpy()


def run(ops, dt, op, lx, lz, extra, in_place=False):
    dx = dev(lx.buffer)
    dz = dx if in_place else dev(lz.buffer)
    getattr(ops, "execTransform" + NAMES[dt])(None, op, dx, lx.info, dz, lz.info, None if extra is None else dev(extra))
    return host(dz)


@pytest.mark.parametrize("dt", [np.float32, np.float64, np.float16])
@pytest.mark.parametrize("g", GEOMETRIES + BIG)
@pytest.mark.parametrize("kinds", [("c", "c"), ("f", "c"), ("c", "f"), ("cview2", "c"), ("f", "cview2"), ("fview2", "fview2")])
def test_im2col(ops, maybe_ref, dt, g, kinds):
    b, c, h, w, kH, kW, sH, sW, pH, pW, dH, dW = g
    oH, oW = geometry(g)
    x = np.random.default_rng(sum(g)).standard_normal((b, c, h, w)).astype(dt)
    lx, lz = Layout(x, kinds[0]), Layout(np.full((b, c, kH, kW, oH, oW), 7, dt), kinds[1])
    extra = np.array([kH, kW, sH, sW, pH, pW, dH, dW, 0, 0], dt)
    got = run(ops, dt, 37, lx, lz, extra)
    want = T.im2col(x, kH, kW, sH, sW, pH, pW, dH, dW, oH, oW)
    assert np.array_equal(lz.read(got).reshape(want.shape), want)
    if maybe_ref is not None and dt != np.float16 and g in GEOMETRIES:
        assert np.array_equal(got, maybe_ref.transform(37, lx.buffer.copy(), lx.info, lz.buffer.copy(), lz.info, extra), equal_nan=True)


def test_im2col_dense_walk_of_a_strided_result_and_padding_value(ops, real_ref):
    """Both arrays c-order with descending strides: the reference writes the result as one dense run per batch entry
    even when its strides say otherwise; and the CUDA build's padding value (extraParams[9])."""
    g = GEOMETRIES[1]
    b, c, h, w, kH, kW, sH, sW, pH, pW, dH, dW = g
    oH, oW = geometry(g)
    x = np.random.default_rng(1).standard_normal((b, c, h, w)).astype(np.float32)
    lx, lz = Layout(x, "cview2"), Layout(np.full((b, c, kH, kW, oH, oW), 7, np.float32), "cview2")
    extra = np.array([kH, kW, sH, sW, pH, pW, dH, dW, 0, 0], np.float32)
    got = run(ops, np.float32, 37, lx, lz, extra)
    assert np.array_equal(got, real_ref.transform(37, lx.buffer.copy(), lx.info, lz.buffer.copy(), lz.info, extra), equal_nan=True)
    extra[9] = -3.5
    lz = Layout(np.zeros((b, c, kH, kW, oH, oW), np.float32), "c")
    got = run(ops, np.float32, 37, Layout(x, "c"), lz, extra)
    assert np.array_equal(got.reshape(b, c, kH, kW, oH, oW), T.im2col(x, kH, kW, sH, sW, pH, pW, dH, dW, oH, oW, pad=-3.5))


@pytest.mark.parametrize("dt", [np.float32, np.float64, np.float16])
@pytest.mark.parametrize("g", GEOMETRIES + BIG)
@pytest.mark.parametrize("kinds", [("c", "c"), ("f", "c"), ("c", "f"), ("fview2", "f"), ("c", "cview2")])
def test_col2im(ops, maybe_ref, dt, g, kinds):
    b, c, h, w, kH, kW, sH, sW, pH, pW, dH, dW = g
    oH, oW = geometry(g)
    cols = np.random.default_rng(sum(g) + 1).standard_normal((b, c, kH, kW, oH, oW)).astype(dt)
    lx, lz = Layout(cols, kinds[0]), Layout(np.full((b, c, h, w), 7, dt), kinds[1])
    extra = np.array([sH, sW, pH, pW, h, w, dH, dW, 0], dt)
    got = lz.read(run(ops, dt, 36, lx, lz, extra)).reshape(b, c, h, w)
    if dt == np.float16:        # the sum is kept in float and rounded once; the reference rounds every addition
        want = T.col2im(cols.astype(np.float32), sH, sW, pH, pW, h, w, dH, dW)
        assert np.allclose(got.astype(np.float32), want, rtol=2e-3, atol=2e-3)
        return
    assert np.array_equal(got, T.col2im(cols, sH, sW, pH, pW, h, w, dH, dW))
    if maybe_ref is not None and g in GEOMETRIES and kinds[1] != "cview2":
        ref = maybe_ref.transform(36, lx.buffer.copy(), lx.info, lz.buffer.copy(), lz.info, extra)
        assert np.array_equal(lz.read(ref).reshape(b, c, h, w), got)


@pytest.mark.parametrize("dt", [np.float32, np.float64, np.float16])
@pytest.mark.parametrize("g", GEOMETRIES + BIG[:3] + BIG[4:])
@pytest.mark.parametrize("mode,extra0", [(0, 0.0), (1, 0.0), (1, 1.0), (2, 2.0), (2, 3.0)])
@pytest.mark.parametrize("kinds", [("c", "c"), ("f", "f"), ("cview2", "c")])
def test_pooling2d(ops, maybe_ref, dt, g, mode, extra0, kinds):
    b, c, h, w, kH, kW, sH, sW, pH, pW, dH, dW = g
    if pH >= kH + (kH - 1) * (dH - 1) or pW >= kW + (kW - 1) * (dW - 1):
        pytest.skip("window entirely inside the padding")
    oH, oW = geometry(g)
    x = np.random.default_rng(sum(g) + 2).standard_normal((b, c, h, w)).astype(dt)
    lx, lz = Layout(x, kinds[0]), Layout(np.zeros((b, c, oH, oW), dt), kinds[1])
    extra = np.array([kH, kW, sH, sW, pH, pW, dH, dW, 0, mode, extra0], dt)
    raw = run(ops, dt, 71, lx, lz, extra)
    got = lz.read(raw).reshape(b, c, oH, oW).astype(np.float64)
    want = T.pooling2d(x, kH, kW, sH, sW, pH, pW, dH, dW, oH, oW, mode, extra0)
    if mode == 0:
        assert np.array_equal(got, want)
    else:
        tol = {np.float32: 1e-5, np.float64: 1e-12, np.float16: 2e-3}[dt]
        assert np.allclose(got, want, rtol=tol, atol=tol)
    if maybe_ref is not None and dt != np.float16 and g in GEOMETRIES:
        ref = maybe_ref.transform(71, lx.buffer.copy(), lx.info, lz.buffer.copy(), lz.info, extra)
        if mode == 0:
            assert np.array_equal(raw, ref)
        else:
            assert np.allclose(raw, ref, rtol=1e-5 if dt == np.float32 else 1e-12, atol=1e-6)


@pytest.mark.parametrize("dt", [np.float32, np.float64, np.float16])
@pytest.mark.parametrize("n,bins", [(1000, 10), (4099, 64), (65536, 256), (17, 3), (1 << 22, 1000), (1 << 20, 20000)])
def test_histogram(ops, maybe_ref, dt, n, bins):
    if dt == np.float16 and (bins > 2048 or n > 65536):
        pytest.skip("half cannot hold the bin number or the counts")
    x = np.random.default_rng(n).uniform(-2, 3, n).astype(dt)
    z0 = (np.arange(bins) % 5).astype(dt)                      # the reference adds to what the result holds
    extra = np.array([bins, -1.5, 2.5], dt)
    dz = dev(z0)
    getattr(ops, "execTransform" + NAMES[dt])(None, 48, dev(x), S.shape_info([1, n]), dz, S.shape_info([1, bins]), dev(extra))
    got = host(dz)
    if dt == np.float16:
        # every operation of the reference rounds to half: restated with numpy's half arithmetic
        lo, hi = np.float16(-1.5), np.float16(2.5)
        size = np.float16(np.float16(hi - lo) / np.float16(bins))
        idx = np.clip(((x - lo).astype(np.float16) / size).astype(np.float16).astype(np.int64), 0, bins - 1)
        counts = np.bincount(idx, minlength=bins)
        assert np.array_equal(got.astype(np.float32), (z0.astype(np.float32) + counts).astype(np.float16).astype(np.float32))
        return
    assert np.array_equal(got, T.histogram(x, z0, bins, -1.5, 2.5))
    if maybe_ref is not None and n <= 65536:
        assert np.array_equal(got, maybe_ref.transform(48, x.copy(), S.shape_info([1, n]), z0.copy(), S.shape_info([1, bins]), extra))


@pytest.mark.parametrize("dt", [np.float32, np.float64, np.float16])
@pytest.mark.parametrize("shape", [(1, 17), (6, 7), (3, 4, 5), (1, 1 << 20), (300, 1001)])
@pytest.mark.parametrize("kinds", [("c", "c"), ("f", "f"), ("c", "f"), ("cview2", "c"), ("f", "cview2"), ("fview2", "fview2")])
def test_reverse(ops, maybe_ref, dt, shape, kinds):
    x = np.random.default_rng(len(shape)).standard_normal(shape).astype(dt)
    lx, lz = Layout(x, kinds[0]), Layout(np.zeros(shape, dt), kinds[1])
    got = run(ops, dt, 70, lx, lz, None)
    xo, zo = offsets(lx), offsets(lz)
    want = lz.buffer.copy()
    want[zo[::-1]] = lx.buffer[xo]
    assert np.array_equal(got, want, equal_nan=True)
    if maybe_ref is not None and dt != np.float16 and x.size < 1000:
        assert np.array_equal(got, maybe_ref.transform(70, lx.buffer.copy(), lx.info, lz.buffer.copy(), lz.info, None), equal_nan=True)


@pytest.mark.parametrize("kind", ["c", "f", "cview2", "fview2"])
@pytest.mark.parametrize("shape", [(1, 16), (1, 17), (5, 6), (1, 12), (1, 20), (1, 1 << 20), (1, (1 << 20) + 4), (1, (1 << 20) + 1),
                                   (257, 513), (256, 516)])
def test_reverse_in_place(ops, maybe_ref, kind, shape):
    x = np.random.default_rng(3).standard_normal(shape).astype(np.float32)
    lx = Layout(x, kind)
    got = run(ops, np.float32, 70, lx, lx, None, in_place=True)
    o = offsets(lx)
    want = lx.buffer.copy()
    if int(lx.info[-2]) >= 1:
        want[o] = lx.buffer[o[::-1]]
    else:                                                      # the first half is copied over the second, not swapped
        half = x.size // 2
        want[o[::-1][:half]] = lx.buffer[o[:half]]
    assert np.array_equal(got, want, equal_nan=True)
    if maybe_ref is not None and x.size < 1000:
        buf = lx.buffer.copy()
        assert np.array_equal(got, maybe_ref.transform(70, buf, lx.info, buf, lx.info, None), equal_nan=True)


def test_errors(ops):
    x = torch.zeros(2 * 3 * 4 * 4, device="cuda")
    z = torch.zeros(2 * 3 * 2 * 2 * 3 * 3, device="cuda")
    extra = torch.tensor([2, 2, 1, 1, 0, 0, 1, 1, 0, 0], dtype=torch.float32, device="cuda")
    with pytest.raises(RuntimeError, match="rank"):
        ops.execTransformFloat(None, 37, x, S.shape_info([2, 3, 16]), z, S.shape_info([2, 3, 2, 2, 3, 3]), extra)
    with pytest.raises(RuntimeError, match="batch"):
        ops.execTransformFloat(None, 37, x, S.shape_info([2, 3, 4, 4]), z, S.shape_info([3, 2, 2, 2, 3, 3]), extra)
    with pytest.raises(RuntimeError, match="extraParams"):
        ops.execTransformFloat(None, 71, x, S.shape_info([2, 3, 4, 4]), x, S.shape_info([2, 3, 4, 4]), None)
