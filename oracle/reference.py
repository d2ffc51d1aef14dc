"""TEST INFRASTRUCTURE ONLY. ctypes front-end to oracle/_ref/libnd4jref.so, the reference's own
CPU implementation of the legacy-op path compiled in place by oracle/Makefile (see ref_shim.cpp).

Only tests/, the smoke check and the benchmark's CPU arm may import this module; the product
package (libnd4j_b200) never does. All arrays are host numpy buffers; ``info`` arguments are
shapeInfo vectors (libnd4j_b200.shape.shape_info).
"""
import ctypes
import os

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "_ref", "libnd4jref.so")

_SFX = {np.dtype(np.float32): "f32", np.dtype(np.float64): "f64", np.dtype(np.float16): "f16"}


def available():
    return os.path.exists(LIB_PATH)


def _p(a):
    if a is None:
        return None
    return ctypes.c_void_p(a.ctypes.data)


def _li(a):
    return None if a is None else np.ascontiguousarray(a, dtype=np.int64)


def _ii(a):
    return None if a is None else np.ascontiguousarray(a, dtype=np.int32)


class Reference:
    def __init__(self, path=None):
        self.lib = ctypes.CDLL(path or LIB_PATH)
        L = self.lib
        L.ref_omp_max_threads.restype = ctypes.c_int
        L.ref_tad_num.restype = ctypes.c_longlong
        L.ref_initRandom.restype = ctypes.c_void_p
        L.ref_initRandom.argtypes = [ctypes.c_longlong, ctypes.c_longlong, ctypes.c_void_p]
        for name in ("ref_refreshBuffer", "ref_reSeedBuffer"):
            getattr(L, name).argtypes = [ctypes.c_longlong, ctypes.c_void_p]
        L.ref_destroyRandom.argtypes = [ctypes.c_void_p]
        L.ref_rng_offset.restype = ctypes.c_longlong
        L.ref_rng_offset.argtypes = [ctypes.c_void_p]
        L.ref_rng_generation.restype = ctypes.c_longlong
        L.ref_rng_generation.argtypes = [ctypes.c_void_p]
        L.ref_rng_set_offset.argtypes = [ctypes.c_void_p, ctypes.c_longlong]
        L.ref_rng_rewind.argtypes = [ctypes.c_void_p, ctypes.c_longlong]
        L.ref_rng_element.restype = ctypes.c_ulonglong
        L.ref_rng_element.argtypes = [ctypes.c_void_p, ctypes.c_longlong]
        L.ref_rng_relative_f32.restype = ctypes.c_float
        L.ref_rng_relative_f32.argtypes = [ctypes.c_void_p, ctypes.c_longlong]
        L.ref_rng_relative_f64.restype = ctypes.c_double
        L.ref_rng_relative_f64.argtypes = [ctypes.c_void_p, ctypes.c_longlong]

    def convert_types(self, src_type, x, dst_type, z):
        """NativeOps::convertTypes (include/loops/type_conversions.h:696-880); z is written in place."""
        self.lib.ref_convertTypes(int(src_type), _p(x), ctypes.c_longlong(x.size), int(dst_type), _p(z))
        return z

    # ---- memory-movement utilities: the CPU NativeOps members themselves (oracle/ref_nativeops.cpp) ----
    @staticmethod
    def _ptrs(arrays):
        return (ctypes.c_void_p * len(arrays))(*[a.ctypes.data for a in arrays])

    def flatten(self, offset, order, z, z_info, x, x_info):
        """NativeOps::flatten* (blas/cpu/NativeOps.cpp:1530-1660, 1797-1860); float and double."""
        zi, xi = _li(z_info), _li(x_info)
        self._f("ref_flatten", x)(int(offset), ctypes.c_char(order.encode()), _p(z), _p(zi), _p(x), _p(xi))
        return z

    def concat(self, dimension, arrays, infos, z, z_info):
        """NativeOps::concat* -> SpecialMethods<T>::concatCpuGeneric (include/ops/impl/specials.cpp:17-120)."""
        keep = [_li(i) for i in infos]
        zi = _li(z_info)
        self._f("ref_concat", z)(int(dimension), len(arrays), self._ptrs(arrays), self._ptrs(keep), _p(z), _p(zi))
        return z

    def pull_rows(self, x, x_info, z, z_info, indexes, tad_info, tad_offsets, ztad_info, ztad_offsets):
        """NativeOps::pullRows* (blas/cpu/NativeOps.cpp:2045-2116); float and double."""
        a = [_li(v) for v in (x_info, z_info, indexes, tad_info, tad_offsets, ztad_info, ztad_offsets)]
        self._f("ref_pullRows", x)(_p(x), _p(a[0]), _p(z), _p(a[1]), ctypes.c_longlong(len(a[2])), _p(a[2]), _p(a[3]),
                                   _p(a[4]), _p(a[5]), _p(a[6]))
        return z

    def tear(self, x, x_info, targets, z_info, tad_info, tad_offsets):
        """NativeOps::tear* (blas/cpu/NativeOps.cpp:2119-2174)."""
        xi, zi, ti, to = _li(x_info), _li(z_info), _li(tad_info), _li(tad_offsets)
        self._f("ref_tear", x)(_p(x), _p(xi), self._ptrs(targets), _p(zi), _p(ti), _p(to))
        return targets

    def shuffle(self, arrays, infos, shuffle_map, tad_infos, tad_offsets):
        """NativeOps::shuffle* in place (blas/cpu/NativeOps.cpp:2266-2380); float and double."""
        ki, kt, ko = [_li(i) for i in infos], [_li(i) for i in tad_infos], [_li(i) for i in tad_offsets]
        m = _ii(shuffle_map)
        self._f("ref_shuffle", arrays[0])(self._ptrs(arrays), self._ptrs(ki), self._ptrs(arrays), self._ptrs(ki),
                                          len(arrays), _p(m), self._ptrs(kt), self._ptrs(ko))
        return arrays

    def average(self, arrays, z, propagate):
        """NativeOps::average* -> SpecialMethods<T>::averageGeneric (specials.cpp:374-433); float and double."""
        self._f("ref_average", arrays[0])(self._ptrs(arrays), _p(z), len(arrays), ctypes.c_longlong(arrays[0].size),
                                          1 if propagate else 0)
        return z

    def accumulate(self, arrays, z):
        """NativeOps::accumulate* -> SpecialMethods<T>::accumulateGeneric (specials.cpp:344-371)."""
        self._f("ref_accumulate", z)(self._ptrs(arrays), _p(z), len(arrays), ctypes.c_longlong(z.size))
        return z

    def sort(self, x, x_info, descending):
        """NativeOps::sort* -> SpecialMethods<T>::sortGeneric (specials.cpp:547-549), in place; float and double."""
        xi = _li(x_info)
        self._f("ref_sort", x)(_p(x), _p(xi), 1 if descending else 0)
        return x

    def sort_tad(self, x, x_info, dims, descending):
        """NativeOps::sortTad* -> SpecialMethods<T>::sortTadGeneric (specials.cpp:552-564), in place."""
        xi, d = _li(x_info), _ii(dims)
        tad_info, tad_off = self.tad(x_info, dims)
        self._f("ref_sortTad", x)(_p(x), _p(xi), _p(d), len(d), _p(tad_info), _p(tad_off), 1 if descending else 0)
        return x

    def sort_coo_indices(self, indices, values, rank):
        """NativeOps::sortCooIndices* (include/ops/impl/specials_sparse.cpp), in place: `indices` holds
        length x rank coordinates, `values` the matching values."""
        self._f("ref_sortCooIndices", values)(_p(indices), _p(values), ctypes.c_longlong(values.size), int(rank))
        return indices, values

    def threads(self):
        return self.lib.ref_omp_max_threads()

    def set_threads(self, n):
        self.lib.ref_omp_set_threads(int(n))

    def _f(self, name, arr):
        return getattr(self.lib, "%s_%s" % (name, _SFX[arr.dtype]))

    # ---- shape / TAD ------------------------------------------------------------------------
    def tad(self, x_info, dims):
        xi, d = _li(x_info), _ii(dims)
        n = self.lib.ref_tad_num(_p(xi), _p(d), len(d))
        target = np.zeros(80, dtype=np.int64)
        offsets = np.zeros(max(int(n), 1), dtype=np.int64)
        self.lib.ref_tadOnlyShapeInfo(_p(xi), _p(d), len(d), _p(target), _p(offsets))
        r = int(target[0])
        return target[:2 * r + 4].copy(), offsets[:int(n)].copy()

    # ---- reductions ---------------------------------------------------------------------------
    def reduce(self, op, x, x_info, z, z_info, dims, extra=None):
        xi, zi, d = _li(x_info), _li(z_info), _ii(dims)
        self._f("ref_execReduce", x)(op, _p(x), _p(xi), _p(extra), _p(z), _p(zi), _p(d), len(d), None, None)
        return z

    def reduce_scalar(self, op, x, x_info, extra=None):
        xi = _li(x_info)
        out = np.zeros(1, dtype=x.dtype)
        self._f("ref_execReduceScalarOut", x)(op, _p(x), _p(xi), _p(extra), _p(out))
        return out[0]

    def index_reduce(self, op, x, x_info, z, z_info, dims, extra=None):
        xi, zi, d = _li(x_info), _li(z_info), _ii(dims)
        self._f("ref_execIndexReduce", x)(op, _p(x), _p(xi), _p(extra), _p(z), _p(zi), _p(d), len(d), None, None)
        return z

    def index_reduce_scalar(self, op, x, x_info, extra=None):
        xi = _li(x_info)
        out = np.zeros(1, dtype=x.dtype)
        self._f("ref_execIndexReduceScalarOut", x)(op, _p(x), _p(xi), _p(extra), _p(out))
        return out[0]

    def summary_stats(self, op, x, x_info, z, z_info, dims, bias_corrected, extra=None):
        xi, zi, d = _li(x_info), _li(z_info), _ii(dims)
        self._f("ref_execSummaryStats", x)(op, _p(x), _p(xi), _p(extra), _p(z), _p(zi), _p(d), len(d),
                                           1 if bias_corrected else 0)
        return z

    def summary_stats_scalar(self, op, x, x_info, bias_corrected, extra=None):
        xi = _li(x_info)
        out = np.zeros(1, dtype=x.dtype)
        self._f("ref_execSummaryStatsScalarOut", x)(op, _p(x), _p(xi), _p(extra), 1 if bias_corrected else 0, _p(out))
        return out[0]

    def reduce3(self, op, x, x_info, y, y_info, z, z_info, dims, extra=None):
        xi, yi, zi, d = _li(x_info), _li(y_info), _li(z_info), _ii(dims)
        self._f("ref_execReduce3", x)(op, _p(x), _p(xi), _p(extra), _p(y), _p(yi), _p(z), _p(zi), _p(d), len(d))
        return z

    def reduce3_all(self, op, x, x_info, y, y_info, z, z_info, dims, extra=None):
        """execReduce3All (include/loops/reduce3.h:919-990): z[r * yTads + g]; z is zeroed first because
        the reference accumulates onto whatever the result buffer holds."""
        xi, yi, zi, d = _li(x_info), _li(y_info), _li(z_info), _ii(dims)
        xt, xo = self.tad(x_info, dims)
        yt, yo = self.tad(y_info, dims)
        z[...] = 0
        self._f("ref_execReduce3All", x)(op, _p(x), _p(xi), _p(extra), _p(y), _p(yi), _p(z), _p(zi), _p(d), len(d),
                                         _p(xt), _p(xo), _p(yt), _p(yo))
        return z

    def reduce3_scalar(self, op, x, x_info, y, y_info, extra=None):
        xi, yi = _li(x_info), _li(y_info)
        out = np.zeros(1, dtype=x.dtype)
        self._f("ref_execReduce3ScalarOut", x)(op, _p(x), _p(xi), _p(extra), _p(y), _p(yi), _p(out))
        return out[0]

    # ---- elementwise --------------------------------------------------------------------------
    def transform(self, op, x, x_info, z, z_info, extra=None):
        xi, zi = _li(x_info), _li(z_info)
        self._f("ref_execTransform", x)(op, _p(x), _p(xi), _p(z), _p(zi), _p(extra))
        return z

    def pairwise(self, op, x, x_info, y, y_info, z, z_info, extra=None):
        xi, yi, zi = _li(x_info), _li(y_info), _li(z_info)
        self._f("ref_execPairwise", x)(op, _p(x), _p(xi), _p(y), _p(yi), _p(z), _p(zi), _p(extra))
        return z

    def broadcast(self, op, x, x_info, y, y_info, z, z_info, dims):
        xi, yi, zi, d = _li(x_info), _li(y_info), _li(z_info), _ii(dims)
        self._f("ref_execBroadcast", x)(op, _p(x), _p(xi), _p(y), _p(yi), _p(z), _p(zi), _p(d), len(d), None, None,
                                        None, None)
        return z

    def scalar(self, op, x, x_info, z, z_info, scalar, extra=None):
        xi, zi = _li(x_info), _li(z_info)
        s = np.array([scalar], dtype=x.dtype)
        self._f("ref_execScalar", x)(op, _p(x), _p(xi), _p(z), _p(zi), _p(s), _p(extra))
        return z

    def scalar_along_dimension(self, op, x, x_info, z, z_info, scalars, dims, extra=None):
        xi, zi, d = _li(x_info), _li(z_info), _ii(dims)
        tad_info, tad_off = self.tad(x_info, dims)
        ztad_info, ztad_off = self.tad(z_info, dims)
        self._f("ref_execScalarAlongDim", x)(op, _p(x), _p(xi), _p(extra), _p(z), _p(zi), _p(scalars), _p(d), len(d),
                                             _p(tad_info), _p(tad_off), _p(ztad_info), _p(ztad_off))
        return z

    # ---- random ---------------------------------------------------------------------------------
    def init_random(self, seed, size):
        table = np.zeros(size, dtype=np.uint64)
        state = self.lib.ref_initRandom(seed, size, _p(table))
        return state, table

    def refresh(self, state, seed):
        self.lib.ref_refreshBuffer(seed, state)

    def reseed(self, state, seed):
        self.lib.ref_reSeedBuffer(seed, state)

    def destroy_random(self, state):
        self.lib.ref_destroyRandom(state)

    def rng_position(self, state):
        return self.lib.ref_rng_offset(state)

    def rng_generation(self, state):
        return self.lib.ref_rng_generation(state)

    def rng_set_position(self, state, pos):
        self.lib.ref_rng_set_offset(state, pos)

    def rng_element(self, state, pos):
        return self.lib.ref_rng_element(state, pos)

    def random(self, op, state, z, z_info, extra):
        zi = _li(z_info)
        self._f("ref_execRandom", z)(op, ctypes.c_void_p(state), _p(z), _p(zi), _p(extra))
        return z

    def random_x(self, op, state, x, x_info, z, z_info, extra):
        xi, zi = _li(x_info), _li(z_info)
        self._f("ref_execRandomX", z)(op, ctypes.c_void_p(state), _p(x), _p(xi), _p(z), _p(zi), _p(extra))
        return z

    def random_xy(self, op, state, x, x_info, y, y_info, z, z_info, extra):
        xi, yi, zi = _li(x_info), _li(y_info), _li(z_info)
        # pass z itself where the caller aliases it, so that the "y == z" test of the Gaussian family holds
        xp = _p(z) if x is z else _p(x)
        yp = _p(z) if y is z else _p(y)
        self._f("ref_execRandomXY", z)(op, ctypes.c_void_p(state), xp, _p(xi), yp, _p(yi), _p(z), _p(zi), _p(extra))
        return z
