"""The cases behind tests/golden/special_transforms_golden.npz (the reference's outputs for the whole-array
transforms): each case names the op, the geometry and the layouts; build() turns it into the buffers of the
execTransform call. Used by the generator, by the CPU test of the numpy restatements and by the GPU test."""
import numpy as np

from libnd4j_b200 import shape as S
from tests import special_truth as T
from tests.cases import Layout

GEOMETRIES = [
    # b, c, h, w, kH, kW, sH, sW, pH, pW, dH, dW
    (2, 3, 8, 12, 3, 3, 1, 1, 1, 1, 1, 1),
    (1, 2, 9, 9, 3, 2, 2, 1, 1, 0, 1, 1),
    (2, 2, 12, 16, 2, 2, 2, 2, 0, 0, 1, 1),
    (1, 3, 10, 11, 3, 3, 2, 2, 1, 1, 2, 2),
]


def cases():
    for gi, g in enumerate(GEOMETRIES):
        for kinds in (("c", "c"), ("f", "c"), ("c", "f")):
            yield "im2col/%d/%s%s" % (gi, *kinds), ("im2col", g, kinds)
            yield "col2im/%d/%s%s" % (gi, *kinds), ("col2im", g, kinds)
        for mode, extra0 in ((0, 0.0), (1, 0.0), (1, 1.0), (2, 2.0)):
            for kinds in (("c", "c"), ("f", "f")):
                yield "pooling/%d/%d_%d/%s%s" % (gi, mode, int(extra0), *kinds), ("pooling", g, kinds, mode, extra0)
    for n, bins in ((1000, 10), (4099, 64)):
        yield "histogram/%d_%d" % (n, bins), ("histogram", n, bins)
    for shape in ((1, 17), (6, 7), (3, 4, 5)):
        for kinds in (("c", "c"), ("f", "f"), ("c", "f"), ("cview2", "c"), ("fview2", "fview2")):
            yield "reverse/%s/%s_%s" % ("x".join(map(str, shape)), *kinds), ("reverse", shape, kinds)


def build(case):
    """-> (opNum, x buffer, x shapeInfo, z buffer, z shapeInfo, extraParams), all float32."""
    kind = case[0]
    dt = np.float32
    if kind in ("im2col", "col2im", "pooling"):
        g, kinds = case[1], case[2]
        b, c, h, w, kH, kW, sH, sW, pH, pW, dH, dW = g
        oH, oW = T.out_size(h, kH, sH, pH, dH), T.out_size(w, kW, sW, pW, dW)
        rng = np.random.default_rng(sum(g) + len(kind))
        if kind == "im2col":
            x = rng.standard_normal((b, c, h, w)).astype(dt)
            lx, lz = Layout(x, kinds[0]), Layout(np.full((b, c, kH, kW, oH, oW), 7, dt), kinds[1])
            return 37, lx.buffer, lx.info, lz.buffer, lz.info, np.array([kH, kW, sH, sW, pH, pW, dH, dW, 0, 0], dt)
        if kind == "col2im":
            x = rng.standard_normal((b, c, kH, kW, oH, oW)).astype(dt)
            lx, lz = Layout(x, kinds[0]), Layout(np.full((b, c, h, w), 7, dt), kinds[1])
            return 36, lx.buffer, lx.info, lz.buffer, lz.info, np.array([sH, sW, pH, pW, h, w, dH, dW, 0], dt)
        mode, extra0 = case[3], case[4]
        x = rng.standard_normal((b, c, h, w)).astype(dt)
        lx, lz = Layout(x, kinds[0]), Layout(np.zeros((b, c, oH, oW), dt), kinds[1])
        return 71, lx.buffer, lx.info, lz.buffer, lz.info, np.array([kH, kW, sH, sW, pH, pW, dH, dW, 0, mode, extra0], dt)
    if kind == "histogram":
        n, bins = case[1], case[2]
        x = np.random.default_rng(n).uniform(-2, 3, n).astype(dt)
        z = (np.arange(bins) % 5).astype(dt)
        return 48, x, S.shape_info([1, n]), z, S.shape_info([1, bins]), np.array([bins, -1.5, 2.5], dt)
    shape, kinds = case[1], case[2]
    x = np.random.default_rng(len(shape)).standard_normal(shape).astype(dt)
    lx, lz = Layout(x, kinds[0]), Layout(np.zeros(shape, dt), kinds[1])
    return 70, lx.buffer, lx.info, lz.buffer, lz.info, None
