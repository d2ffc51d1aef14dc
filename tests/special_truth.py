"""numpy restatements of the reference's whole-array ("special") transforms, include/ops/special_ops.h: Col2Im
(opNum 36, :891-1120), Im2col (37, :414-640), Histogram (48, :713-880), Reverse (70, :1178-1415) and Pooling2D
(71, :31-330). Test infrastructure: tests/test_oracle_special_transforms.py holds every function here against the
reference's own CPU code (oracle/_ref), and the GPU tests compare with both."""
import numpy as np


def out_size(size, k, s, p, d):
    return (size + 2 * p - (k + (k - 1) * (d - 1))) // s + 1


def _taps(k_index, dilation, pad, stride, out, size):
    """Image coordinates read by kernel tap k_index for every output coordinate, and which of them lie inside."""
    at = -pad + k_index * dilation + stride * np.arange(out)
    inside = np.nonzero((at >= 0) & (at < size))[0]
    return at[inside], inside


def im2col(x, kH, kW, sH, sW, pH, pW, dH, dW, oH, oW, pad=0.0):
    """x [b, c, h, w] -> [b, c, kH, kW, oH, oW]; positions outside the image hold `pad`."""
    b, c, iH, iW = x.shape
    z = np.full((b, c, kH, kW, oH, oW), pad, dtype=x.dtype)
    for kr in range(kH):
        rows, oh = _taps(kr, dH, pH, sH, oH, iH)
        for kc in range(kW):
            cols, ow = _taps(kc, dW, pW, sW, oW, iW)
            if len(oh) and len(ow):
                z[:, :, kr, kc, oh[:, None], ow[None, :]] = x[:, :, rows[:, None], cols[None, :]]
    return z


def col2im(cols, sH, sW, pH, pW, iH, iW, dH, dW):
    """cols [b, c, kH, kW, oH, oW] -> [b, c, iH, iW]; additions in the reference's order (kernel row, then kernel
    column), each in the element type."""
    b, c, kH, kW, oH, oW = cols.shape
    z = np.zeros((b, c, iH, iW), dtype=cols.dtype)
    for kr in range(kH):
        rows, oh = _taps(kr, dH, pH, sH, oH, iH)
        for kc in range(kW):
            cs, ow = _taps(kc, dW, pW, sW, oW, iW)
            if len(oh) and len(ow):
                z[:, :, rows[:, None], cs[None, :]] += cols[:, :, kr, kc, oh[:, None], ow[None, :]]
    return z


def pooling2d(x, kH, kW, sH, sW, pH, pW, dH, dW, oH, oW, mode, extra0):
    """mode 0 max, 1 average (extra0 0: divide by the positions inside the image, 1: by kH * kW), 2 p-norm with
    p = extra0. Sums in double, so compare the average and the p-norm with a tolerance."""
    b, c, iH, iW = x.shape
    z = np.zeros((b, c, oH, oW), dtype=np.float64)
    kHe, kWe = kH + (kH - 1) * (dH - 1), kW + (kW - 1) * (dW - 1)
    xd = x.astype(np.float64)
    for yy in range(oH):
        for xx in range(oW):
            hs, ws = yy * sH - pH, xx * sW - pW
            he, we = hs + kHe, ws + kWe
            if hs < 0:
                hs += -(hs // dH) * dH
            if ws < 0:
                ws += -(ws // dW) * dW
            if he > iH:
                he -= -((iH - he) // dH) * dH
            if we > iW:
                we -= -((iW - we) // dW) * dW
            win = xd[:, :, hs:he:dH, ws:we:dW]
            n = win.shape[2] * win.shape[3]
            if mode == 0:
                z[:, :, yy, xx] = np.maximum(win.reshape(b, c, -1).max(axis=2), -1e37) if n else -1e37
            elif mode == 1:
                div = n if int(extra0) == 0 else kH * kW
                z[:, :, yy, xx] = win.reshape(b, c, -1).sum(axis=2) / div
            else:
                z[:, :, yy, xx] = (np.abs(win.reshape(b, c, -1)) ** extra0).sum(axis=2) ** (1.0 / extra0)
    return z


def histogram(x, z, num_bins, lo, hi):
    """Adds the counts to z (the reference's CPU code accumulates into the result). Arithmetic in x's type."""
    t = x.dtype.type
    bin_size = t(t(hi) - t(lo)) / t(num_bins)
    idx = ((x.ravel() - t(lo)) / t(bin_size)).astype(np.int64)
    idx = np.clip(idx, 0, num_bins - 1)
    return (z + np.bincount(idx, minlength=num_bins).astype(z.dtype)).astype(z.dtype)


def own_order_offsets(shape, strides, order, ews):
    """Buffer offset of linear position e, for every e, in the array's own order."""
    n = int(np.prod(shape))
    if ews >= 1:
        return np.arange(n, dtype=np.int64) * ews
    coords = np.unravel_index(np.arange(n), shape, order="C" if order == "c" else "F")
    return sum(c.astype(np.int64) * s for c, s in zip(coords, strides))
