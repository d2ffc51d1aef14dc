"""Host-side helpers for the reference's shapeInfo descriptors.

A shapeInfo is an int64 vector ``[rank, shape..., stride..., offset, elementWiseStride, order]``
of length ``2*rank + 4`` (include/helpers/shape.h:2558-2617 of the reference). Strides count
elements, not bytes. ``order`` is ``ord('c')`` = 99 or ``ord('f')`` = 102.
"""
import numpy as np

MAX_DIMENSION = 0x7FFFFFFF


def default_strides(shape, order="c"):
    shape = list(shape)
    strides = [0] * len(shape)
    acc = 1
    rng = range(len(shape) - 1, -1, -1) if order == "c" else range(len(shape))
    for i in rng:
        strides[i] = acc
        acc *= shape[i]
    return strides


def element_wise_stride(shape, strides, order="c"):
    """Stride that walks every element linearly in `order`, or -1 when the view has none.

    Unit axes are ignored; the remaining axes must chain (c: stride[k] == shape[k+1]*stride[k+1],
    f: stride[k+1] == shape[k]*stride[k]). This is what nd4j's Java side stores in the ews slot.
    """
    dims = [(s, t) for s, t in zip(shape, strides) if s != 1]
    if not dims:
        return 1
    if order == "f":
        dims = dims[::-1]
    for (s0, t0), (s1, t1) in zip(dims[:-1], dims[1:]):
        if t0 != s1 * t1:
            return -1
    return dims[-1][1]


def shape_info(shape, order="c", strides=None, ews=None, offset=0):
    shape = [int(s) for s in shape]
    if strides is None:
        strides = default_strides(shape, order)
        if ews is None:
            ews = 1
    else:
        strides = [int(s) for s in strides]
        if ews is None:
            ews = element_wise_stride(shape, strides, order)
    return np.array([len(shape)] + shape + strides + [offset, ews, ord(order)], dtype=np.int64)


def shape_info_of(array, order=None):
    """shapeInfo describing a numpy array (or view) in element strides."""
    item = array.dtype.itemsize
    strides = [s // item for s in array.strides]
    if order is None:
        order = "f" if (array.flags["F_CONTIGUOUS"] and not array.flags["C_CONTIGUOUS"]) else "c"
    return shape_info(array.shape, order, strides)


def rank(info):
    return int(info[0])


def shape_of(info):
    r = int(info[0])
    return [int(v) for v in info[1:1 + r]]


def strides_of(info):
    r = int(info[0])
    return [int(v) for v in info[1 + r:1 + 2 * r]]


def length(info):
    n = 1
    for s in shape_of(info):
        n *= s
    return n


def reduced_shape_info(x_info, dimension, old_shapes=True):
    """shapeInfo of a reduction result: rank-2 "old shapes" ([1,n] when axis 0 is reduced,
    [n,1] otherwise) as the legacy callers pass them, or the keep-remaining-axes shape."""
    shp = shape_of(x_info)
    dims = sorted(set(d % len(shp) for d in dimension)) if dimension else list(range(len(shp)))
    keep = [s for i, s in enumerate(shp) if i not in dims]
    n = 1
    for s in keep:
        n *= s
    if not keep:
        return shape_info([1, 1])
    if old_shapes and len(keep) == 1:
        return shape_info([1, n]) if 0 in dims else shape_info([n, 1])
    return shape_info(keep)
