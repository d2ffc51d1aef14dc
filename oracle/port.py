"""TEST INFRASTRUCTURE ONLY. Restatement ("port") of the reference's CPU algorithms for the legacy
op families: shapeInfo / TAD decoding in Python (below) and the arithmetic in plain C
(oracle/port.c, compiled on first use with gcc into oracle/_port.so).

Parity status: pinned. tests/test_oracle.py checks this port against the reference's own CPU
build (oracle/_ref) wherever that library is present, and against the golden vectors under
tests/golden/ (generated from that build by tests/golden/make_golden.py) everywhere else.

`Port` offers the same methods as oracle.reference.Reference for float32 arrays, so the tests and
the smoke check can use either. Only tests/, the smoke check and the benchmark's CPU arm may
import this module.

What is restated, with the reference lines each part follows:
  * shapeInfo layout, c-order coordinates and offsets: include/helpers/shape.h:1860-1892 (ind2subC),
    3271-3294 (getOffset), 2558-2617 (layout);
  * TAD shape and base offsets: include/helpers/TAD.h:325-372 (init), 577-720 (tadOffset,
    tad2Sub via ind2subC, createOffsets), 723-896 (shape of the TAD);
  * which elements a loop visits for an operand: ews >= 1 walks the buffer linearly, otherwise
    c-order coordinates (include/loops/cpu/transform.cpp:30-91, pairwise_transform.h:155-367,
    reduce.cpp:14-60); random ops use f-order coordinates (loops/cpu/random.cpp:175).
"""
import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_SO = os.path.join(_HERE, "_port.so")
_SRC = os.path.join(_HERE, "port.c")


def build():
    if not os.path.exists(_SO) or os.path.getmtime(_SO) < os.path.getmtime(_SRC):
        subprocess.run(["gcc", "-O2", "-fPIC", "-shared", "-ffp-contract=off", "-o", _SO, _SRC, "-lm"], check=True)
    return _SO


# ---- shapeInfo / TAD decoding -------------------------------------------------------------------
def _parts(info):
    info = [int(v) for v in info]
    r = info[0]
    return r, info[1:1 + r], info[1 + r:1 + 2 * r], info[2 * r + 2], chr(info[2 * r + 3])


def linear_offsets(info, f_order_coords=False):
    """Offsets of the elements in the order a whole-array loop visits them."""
    r, shape, stride, ews, order = _parts(info)
    n = int(np.prod(shape, dtype=np.int64)) if r else 1
    if ews >= 1:
        return np.arange(n, dtype=np.int64) * ews
    return coord_offsets(shape, stride, f_order_coords)


def coord_offsets(shape, stride, f_order=False):
    """Offsets in c-order (last axis fastest) or f-order (first axis fastest) coordinate order;
    axes of extent 1 contribute nothing, as in getOffset."""
    if not shape:
        return np.zeros(1, dtype=np.int64)
    grids = np.indices(shape, dtype=np.int64)
    off = np.zeros(shape, dtype=np.int64)
    for d, st in enumerate(stride):
        if shape[d] != 1:
            off += grids[d] * st
    return off.ravel(order="F" if f_order else "C")


def normalise_dims(rank, dims):
    if dims is None or len(dims) == 0 or (len(dims) == 1 and dims[0] == 0x7FFFFFFF):
        return list(range(rank))
    return sorted(set(int(d) % rank for d in dims))


def tad_offsets(info, dims):
    """(base offsets [numTads], element offsets inside a TAD [tadLen]) for the given axes."""
    r, shape, stride, ews, order = _parts(info)
    dims = normalise_dims(r, dims)
    if len(dims) == r:
        return np.zeros(1, dtype=np.int64), linear_offsets(info)
    keep = [i for i in range(r) if i not in dims]
    base = coord_offsets([shape[i] for i in keep], [stride[i] for i in keep])
    inner = coord_offsets([shape[i] for i in dims], [stride[i] for i in dims])
    return base, inner


def tad_shape_info(info, dims):
    """The TAD's own shapeInfo as the reference reports it for arrays without unit axes."""
    r, shape, stride, ews, order = _parts(info)
    dims = normalise_dims(r, dims)
    if len(dims) == r:
        return np.array(info, dtype=np.int64)

    def order_of(shp, st):
        c = f = True
        sd = 1
        for i in range(len(shp) - 1, -1, -1):
            if st[i] != sd:
                c = False
                break
            sd *= shp[i]
        sd = 1
        for i in range(len(shp)):
            if st[i] != sd:
                f = False
            sd *= shp[i]
        return "a" if (f and c) else ("f" if f else "c")

    if len(dims) == 1:
        d = dims[0]
        if shape[d] == 1:
            return np.array([1, 1, 1, 0, 1, 99], dtype=np.int64)
        shp, st = [1, shape[d]], [1, stride[d]]
        return np.array([2] + shp + st + [0, stride[d], ord(order_of(shp, st))], dtype=np.int64)
    shp, st = [shape[i] for i in dims], [stride[i] for i in dims]
    return np.array([len(dims)] + shp + st + [0, -1, ord(order_of(shp, st))], dtype=np.int64)


def _c(a):
    return a.ctypes.data_as(ctypes.c_void_p)


class PortRng(ctypes.Structure):
    _fields_ = [("size", ctypes.c_longlong), ("position", ctypes.c_longlong), ("generation", ctypes.c_longlong),
                ("seed", ctypes.c_longlong), ("amplifier", ctypes.c_longlong), ("table", ctypes.c_void_p)]


class Port:
    """float32 restatement with the calling conventions of oracle.reference.Reference."""

    def __init__(self):
        self.lib = ctypes.CDLL(build())
        self.lib.port_rng_element.restype = ctypes.c_ulonglong
        self._rng = {}

    def threads(self):
        return 1

    def set_threads(self, n):
        pass

    # ---- shape ---------------------------------------------------------------------------------
    def tad(self, x_info, dims):
        base, _ = tad_offsets(x_info, dims)
        return tad_shape_info(x_info, dims), base

    @staticmethod
    def _need_f32(*arrays):
        for a in arrays:
            if a is not None and a.dtype != np.float32:
                raise NotImplementedError("the port restates the float32 flavour")

    def _gather(self, x, info, dims):
        base, inner = tad_offsets(info, dims)
        return np.ascontiguousarray(x[base[:, None] + inner[None, :]]), base, inner

    @staticmethod
    def _params(extra, n=4):
        p = np.zeros(n, dtype=np.float32)
        if extra is not None:
            p[:min(n, len(extra))] = np.asarray(extra, dtype=np.float32)[:n]
        return p

    # ---- reductions ----------------------------------------------------------------------------
    def _dims_for(self, x_info, z_info, dims):
        n = int(np.prod(_parts(z_info)[1], dtype=np.int64)) if z_info is not None else 0
        return None if n == 1 else dims

    def reduce(self, op, x, x_info, z, z_info, dims, extra=None):
        self._need_f32(x)
        m, _, _ = self._gather(x, x_info, self._dims_for(x_info, z_info, dims))
        out = np.zeros(m.shape[0], dtype=np.float32)
        rc = self.lib.port_reduce_f32(op, _c(m), ctypes.c_longlong(m.shape[0]), ctypes.c_longlong(m.shape[1]), _c(out),
                                      _c(self._params(extra)))
        assert rc == 0, "unknown reduce op %d" % op
        z[:out.size] = out
        return z

    def reduce_scalar(self, op, x, x_info, extra=None):
        out = np.zeros(1, dtype=np.float32)
        return self.reduce(op, x, x_info, out, np.array([2, 1, 1, 1, 1, 0, 1, 99]), None, extra)[0]

    def index_reduce(self, op, x, x_info, z, z_info, dims, extra=None):
        self._need_f32(x)
        m, _, _ = self._gather(x, x_info, self._dims_for(x_info, z_info, dims))
        out = np.zeros(m.shape[0], dtype=np.float32)
        rc = self.lib.port_index_reduce_f32(op, _c(m), ctypes.c_longlong(m.shape[0]), ctypes.c_longlong(m.shape[1]),
                                            _c(out), _c(self._params(extra)))
        assert rc == 0
        z[:out.size] = out
        return z

    def index_reduce_scalar(self, op, x, x_info, extra=None):
        out = np.zeros(1, dtype=np.float32)
        return self.index_reduce(op, x, x_info, out, np.array([2, 1, 1, 1, 1, 0, 1, 99]), None, extra)[0]

    def summary_stats(self, op, x, x_info, z, z_info, dims, bias_corrected, extra=None):
        self._need_f32(x)
        m, _, _ = self._gather(x, x_info, self._dims_for(x_info, z_info, dims))
        out = np.zeros(m.shape[0], dtype=np.float32)
        rc = self.lib.port_summary_stats_f32(op, _c(m), ctypes.c_longlong(m.shape[0]), ctypes.c_longlong(m.shape[1]),
                                             _c(out), 1 if bias_corrected else 0)
        assert rc == 0
        z[:out.size] = out
        return z

    def summary_stats_scalar(self, op, x, x_info, bias_corrected, extra=None):
        out = np.zeros(1, dtype=np.float32)
        return self.summary_stats(op, x, x_info, out, np.array([2, 1, 1, 1, 1, 0, 1, 99]), None, bias_corrected)[0]

    def reduce3(self, op, x, x_info, y, y_info, z, z_info, dims, extra=None):
        """Row-against-row semantics (the reference's contiguous path, reduce3.h:1236-1262)."""
        self._need_f32(x, y)
        d = self._dims_for(x_info, z_info, dims)
        mx, _, _ = self._gather(x, x_info, d)
        my, _, _ = self._gather(y, y_info, d)
        if mx.shape[0] == 1 and my.shape[0] > 1:
            mx = np.ascontiguousarray(np.broadcast_to(mx, my.shape))
        ystep = my.shape[1] if my.shape[0] == mx.shape[0] else 0
        out = np.zeros(mx.shape[0], dtype=np.float32)
        eps = float(extra[0]) if (extra is not None and d is None) else 0.0
        rc = self.lib.port_reduce3_f32(op, _c(mx), _c(np.ascontiguousarray(my)), ctypes.c_longlong(ystep),
                                       ctypes.c_longlong(mx.shape[0]), ctypes.c_longlong(mx.shape[1]), _c(out),
                                       ctypes.c_float(eps))
        assert rc == 0
        z[:out.size] = out
        return z

    def reduce3_all(self, op, x, x_info, y, y_info, z, z_info, dims, extra=None):
        """Every TAD of x against every TAD of y, z[r * yTads + g] (reduce3.h:919-990); the functors see a
        zeroed parameter block, as in the reference."""
        self._need_f32(x, y)
        mx, _, _ = self._gather(x, x_info, list(dims))
        my, _, _ = self._gather(y, y_info, list(dims))
        my = np.ascontiguousarray(my)
        out = np.zeros(my.shape[0], dtype=np.float32)
        for r in range(mx.shape[0]):
            row = np.ascontiguousarray(np.broadcast_to(mx[r], my.shape))
            rc = self.lib.port_reduce3_f32(op, _c(row), _c(my), ctypes.c_longlong(my.shape[1]),
                                           ctypes.c_longlong(my.shape[0]), ctypes.c_longlong(my.shape[1]), _c(out),
                                           ctypes.c_float(0.0))
            assert rc == 0
            z[r * my.shape[0]:(r + 1) * my.shape[0]] = out
        return z

    def reduce3_scalar(self, op, x, x_info, y, y_info, extra=None):
        out = np.zeros(1, dtype=np.float32)
        return self.reduce3(op, x, x_info, y, y_info, out, np.array([2, 1, 1, 1, 1, 0, 1, 99]), None, extra)[0]

    # ---- elementwise ---------------------------------------------------------------------------
    def _softmax(self, op, x, x_info, z, z_info):
        """SoftMax (38), SoftMaxDerivative (39), LogSoftMax (40) on matrices (row-wise) and vectors
        (include/ops/special_ops.h:1484-1940): max, subtract, exp, sequential float row sum, divide, then
        y (1 - y) or log."""
        shp = _parts(x_info)[1]
        rows, cols = (1, int(np.prod(shp))) if 1 in shp else (int(shp[0]), int(shp[1]))
        offs = coord_offsets(*_parts(x_info)[1:3])
        m = np.ascontiguousarray(x[offs]).reshape(rows, cols).astype(np.float32)
        e = np.exp((m - m.max(axis=1, keepdims=True)).astype(np.float32)).astype(np.float32)
        sums = np.cumsum(e, axis=1, dtype=np.float32)[:, -1:]
        yv = (e / sums).astype(np.float32)
        with np.errstate(divide="ignore"):
            out = yv if op == 38 else ((yv * (np.float32(1) - yv)).astype(np.float32) if op == 39 else np.log(yv).astype(np.float32))
        z[coord_offsets(*_parts(z_info)[1:3])] = out.ravel()
        return z

    def transform(self, op, x, x_info, z, z_info, extra=None):
        self._need_f32(x)
        if op in (38, 39, 40):
            return self._softmax(op, x, x_info, z, z_info)
        xo, zo = linear_offsets(x_info), linear_offsets(z_info)
        if _parts(x_info)[4] != _parts(z_info)[4] and _parts(x_info)[0] > 1:
            xo, zo = coord_offsets(*_parts(x_info)[1:3]), coord_offsets(*_parts(z_info)[1:3])
        src = np.ascontiguousarray(x[xo])
        out = np.empty_like(src)
        self.lib.port_transform_f32(op, _c(src), _c(out), ctypes.c_longlong(src.size), _c(self._params(extra)))
        z[zo] = out
        return z

    def _binary(self, table, op, xs, ys, ystep, extra):
        out = np.empty_like(xs)
        rc = self.lib.port_binary_f32(table, op, _c(xs), _c(ys), ctypes.c_longlong(ystep), _c(out),
                                      ctypes.c_longlong(xs.size), _c(self._params(extra)))
        assert rc == 0, "unknown binary op %d in table %d" % (op, table)
        return out

    def pairwise(self, op, x, x_info, y, y_info, z, z_info, extra=None):
        self._need_f32(x, y)
        infos = (x_info, y_info, z_info)
        linear = all(_parts(i)[3] >= 1 for i in infos) and len({_parts(i)[4] for i in infos if _parts(i)[0] > 1}) <= 1
        if linear:
            xo, yo, zo = (linear_offsets(i) for i in infos)
        else:
            xo, yo, zo = (coord_offsets(*_parts(i)[1:3]) for i in infos)
        if yo.size == 1 and xo.size > 1:
            out = self._binary(0, op, np.ascontiguousarray(x[xo]), np.ascontiguousarray(y[yo]), 0, extra)
        else:
            out = self._binary(0, op, np.ascontiguousarray(x[xo]), np.ascontiguousarray(y[yo]), 1, extra)
        z[zo] = out
        return z

    def scalar(self, op, x, x_info, z, z_info, scalar, extra=None):
        self._need_f32(x)
        xo, zo = linear_offsets(x_info), linear_offsets(z_info)
        out = self._binary(1, op, np.ascontiguousarray(x[xo]), np.array([scalar], dtype=np.float32), 0, extra)
        z[zo] = out
        return z

    def broadcast(self, op, x, x_info, y, y_info, z, z_info, dims):
        self._need_f32(x, y)
        mx, _, _ = self._gather(x, x_info, dims)
        zb, zi = tad_offsets(z_info, dims)
        yo = coord_offsets(*_parts(y_info)[1:3])
        yrow = np.ascontiguousarray(y[yo])
        tiled = np.ascontiguousarray(np.broadcast_to(yrow, mx.shape)).ravel()
        out = self._binary(2, op, mx.ravel(), tiled, 1, None)
        z[(zb[:, None] + zi[None, :]).ravel()] = out
        return z

    def scalar_along_dimension(self, op, x, x_info, z, z_info, scalars, dims, extra=None):
        self._need_f32(x)
        mx, _, _ = self._gather(x, x_info, dims)
        zb, zi = tad_offsets(z_info, dims)
        per = np.ascontiguousarray(np.repeat(np.asarray(scalars, dtype=np.float32), mx.shape[1]))
        out = self._binary(1, op, mx.ravel(), per, 1, extra)
        z[(zb[:, None] + zi[None, :]).ravel()] = out
        return z

    # ---- random --------------------------------------------------------------------------------
    def init_random(self, seed, size):
        table = np.zeros(size, dtype=np.uint64)
        g = PortRng(size, 0, 1, seed, seed, table.ctypes.data)
        self.lib.port_rng_fill(ctypes.byref(g))
        handle = len(self._rng) + 1
        self._rng[handle] = (g, table)
        return handle, table

    def refresh(self, state, seed):
        g, _ = self._rng[state]
        g.seed, g.amplifier, g.generation, g.position = seed, seed, 1, 0
        self.lib.port_rng_fill(ctypes.byref(g))

    def reseed(self, state, seed):
        self._rng[state][0].amplifier = seed

    def destroy_random(self, state):
        self._rng.pop(state, None)

    def rng_position(self, state):
        return self._rng[state][0].position

    def rng_generation(self, state):
        return self._rng[state][0].generation

    def rng_set_position(self, state, pos):
        self._rng[state][0].position = pos

    def rng_element(self, state, pos):
        return self.lib.port_rng_element(ctypes.byref(self._rng[state][0]), ctypes.c_longlong(pos))

    def _random(self, op, arity, state, x, y, y_is_z, z, z_info, extra, x_info=None, y_info=None):
        self._need_f32(z)
        g, _ = self._rng[state]
        special = op in (6, 10)

        def offs(info):
            if _parts(info)[3] >= 1 or special:
                return np.arange(int(np.prod(_parts(z_info)[1], dtype=np.int64)), dtype=np.int64) * max(_parts(info)[3], 1)
            return coord_offsets(*_parts(info)[1:3], f_order=True)

        zo = offs(z_info)
        n = zo.size
        xs = np.ascontiguousarray(x[offs(x_info)[:n]]) if x is not None and arity >= 1 and x_info is not None else None
        ys = np.ascontiguousarray(y[offs(y_info)[:n]]) if y is not None and arity == 2 and y_info is not None else None
        out = np.zeros(n, dtype=np.float32)
        rc = self.lib.port_random_f32(op, arity, ctypes.byref(g), _c(xs) if xs is not None else None,
                                      _c(ys) if ys is not None else None, 1 if y_is_z else 0, _c(out),
                                      ctypes.c_longlong(n), _c(self._params(extra)))
        assert rc == 0, "random op %d is not restated" % op
        z[zo] = out
        self.lib.port_rng_rewind(ctypes.byref(g), ctypes.c_longlong(n))
        return z

    def random(self, op, state, z, z_info, extra):
        return self._random(op, 0, state, None, None, False, z, z_info, extra)

    def random_x(self, op, state, x, x_info, z, z_info, extra):
        return self._random(op, 1, state, x, None, False, z, z_info, extra, x_info)

    def _unit(self, state, indices):
        """relativeT<float>: (float) element / (float) MAX, with the float of 2^64 - 1 being 2^64 (helper_generator.h:481-486)."""
        raw = np.array([self.rng_element(state, int(i)) & 0xFFFFFFFFFFFFFFFF for i in indices], dtype=np.uint64)
        return raw.astype(np.float32) * np.float32(2.0 ** -64)

    def _special_random(self, op, state, x, x_info, y, y_info, z, z_info, extra):
        """Choice (5), BinomialDistribution (8), BinomialDistributionEx (9): special_random_ops.h:153-245, 474-650,
        operands addressed by their elementWiseStride."""
        self._need_f32(z)
        g, _ = self._rng[state]
        n = int(np.prod(_parts(z_info)[1], dtype=np.int64))
        zews = max(_parts(z_info)[3], 1)
        if op == 5:
            k = int(np.prod(_parts(y_info)[1], dtype=np.int64))
            xs = x[::max(_parts(x_info)[3], 1)][:k]
            sums = np.zeros(k, np.float32)
            acc = np.float32(0)
            for f in range(k):                       # running sums in float, in order
                acc = np.float32(acc + y[f * max(_parts(y_info)[3], 1)])
                sums[f] = acc
            u = self._unit(state, range(n))
            hit = np.array([int(np.argmax(u[e] <= sums)) if (u[e] <= sums).any() else k - 1 for e in range(n)])
            z[:n * zews:zews] = xs[hit]
            self.lib.port_rng_rewind(ctypes.byref(g), ctypes.c_longlong(n))
            return z
        trials = int(extra[0])
        out = np.zeros(n, np.float32)
        e1 = np.arange(1, n + 1, dtype=np.int64)
        for t in range(1, trials + 1):
            u = self._unit(state, e1 * t)
            if y is z:
                prob = np.float32(extra[1])
            elif op == 8:
                prob = y[(t - 1) * max(_parts(y_info)[3], 1)]
            else:
                prob = y[:n * max(_parts(y_info)[3], 1):max(_parts(y_info)[3], 1)]
            out += (u < prob).astype(np.float32)
        z[:n * zews:zews] = out
        if trials > 0:
            self.lib.port_rng_rewind(ctypes.byref(g), ctypes.c_longlong(n * trials))
        return z

    def random_xy(self, op, state, x, x_info, y, y_info, z, z_info, extra):
        if op in (5, 8, 9):
            return self._special_random(op, state, x, x_info, y, y_info, z, z_info, extra)
        y_is_z = y is z
        xs = None if x is z else x
        return self._random(op, 2, state, x if xs is not None else np.array(z), None if y_is_z else y, y_is_z, z, z_info,
                            extra, x_info, None if y_is_z else y_info)
