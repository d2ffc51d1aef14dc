"""Host-side mirror of the reference's ``NativeOps`` interface for the legacy op families.

The class below keeps the reference's member names, argument order and op numbers
(blas/NativeOps.h: ``execReduceFloat``, ``execBroadcastFloat``, ``execTransformFloat`` ...), so a
test written against the reference reads the same here. Every call goes through the C ABI of
``libnd4jb200.so`` (include/nd4j_b200.h); there is no CPU path. If the library cannot be loaded
the import of this module still succeeds (so tooling can inspect it) but constructing
``NativeOps`` raises.

Pointer arguments accept a torch CUDA tensor, an object with ``data_ptr()``, or a raw integer
device address. shapeInfo and dimension arguments are host arrays (numpy int64 / int32 or
sequences); in the reference's CUDA build the same host copies travel in ``extraPointers``.
``extraPointers`` is accepted for signature compatibility: slot 1, when present and non-zero,
is used as the CUDA stream, exactly as the reference does (blas/cuda/NativeOps.cu:2107).
"""
import ctypes
import os

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libnd4jb200.so")

FLOAT, DOUBLE, HALF = 0, 1, 2
_SUFFIX = {"Float": FLOAT, "Double": DOUBLE, "Half": HALF}

# copy directions of NativeOps::memcpy* (blas/cuda/NativeOps.cu:4038-4075)
HOST_TO_HOST, HOST_TO_DEVICE, DEVICE_TO_HOST, DEVICE_TO_DEVICE = 0, 1, 2, 3


class Nd4jError(RuntimeError):
    """A call into the backend failed; ``code`` is the ND4JB200_E* status."""

    def __init__(self, code, message):
        super().__init__("nd4jb200 status %d: %s" % (code, message))
        self.code = code


def _ptr(obj):
    if obj is None:
        return None
    if isinstance(obj, int):
        return ctypes.c_void_p(obj)
    if hasattr(obj, "data_ptr"):
        return ctypes.c_void_p(obj.data_ptr())
    if isinstance(obj, ctypes.c_void_p):
        return obj
    raise TypeError("expected a device pointer (int, torch tensor or c_void_p), got %r" % type(obj))


def _longs(a):
    if a is None:
        return None, None
    arr = np.ascontiguousarray(a, dtype=np.int64)
    return arr, arr.ctypes.data_as(ctypes.POINTER(ctypes.c_longlong))


def _ints(a):
    if a is None:
        return None, None
    arr = np.ascontiguousarray(a, dtype=np.int32)
    return arr, arr.ctypes.data_as(ctypes.POINTER(ctypes.c_int))


def load_library(path=None):
    """Loads libnd4jb200.so and declares the argument types of every entry point."""
    path = path or LIB_PATH
    if not os.path.exists(path):
        raise Nd4jError(-1, "%s is missing: build it with `python -m libnd4j_b200.build`" % path)
    lib = ctypes.CDLL(path)
    vp, ll, i, d = ctypes.c_void_p, ctypes.c_longlong, ctypes.c_int, ctypes.c_double
    llp, ip, dp = ctypes.POINTER(ll), ctypes.POINTER(i), ctypes.POINTER(d)
    sig = {
        "nd4jb200_last_error": (ctypes.c_char_p, []),
        "nd4jb200_launch_count": (ctypes.c_ulonglong, []),
        "nd4jb200_convert_types": (i, [vp, i, vp, ll, i, vp]),
        "nd4jb200_flatten": (i, [vp, i, ll, ctypes.c_char, vp, llp, vp, llp]),
        "nd4jb200_concat": (i, [vp, i, i, i, vp, vp, vp, llp]),
        "nd4jb200_pull_rows": (i, [vp, i, vp, vp, ll, vp, llp, vp, llp, vp]),
        "nd4jb200_tear": (i, [vp, i, vp, llp, vp, llp, llp, vp]),
        "nd4jb200_shuffle": (i, [vp, i, i, vp, vp, ip, vp, vp]),
        "nd4jb200_sort": (i, [vp, i, vp, llp, i]),
        "nd4jb200_sort_tad": (i, [vp, i, vp, llp, ip, i, i]),
        "nd4jb200_average": (i, [vp, i, vp, vp, i, ll, i]),
        "nd4jb200_accumulate": (i, [vp, i, vp, vp, i, ll]),
        "nd4jb200_set_tuning": (ctypes.c_int, [ctypes.c_int, ctypes.c_longlong]),
        "nd4jb200_exec_reduce": (i, [vp, i, i, vp, llp, vp, vp, llp, ip, i]),
        "nd4jb200_exec_reduce_scalar": (i, [vp, i, i, vp, llp, vp, dp]),
        "nd4jb200_exec_index_reduce": (i, [vp, i, i, vp, llp, vp, vp, llp, ip, i]),
        "nd4jb200_exec_index_reduce_scalar": (i, [vp, i, i, vp, llp, vp, dp]),
        "nd4jb200_exec_summary_stats": (i, [vp, i, i, vp, llp, vp, vp, llp, ip, i, i]),
        "nd4jb200_exec_summary_stats_scalar": (i, [vp, i, i, vp, llp, vp, i, dp]),
        "nd4jb200_exec_reduce3": (i, [vp, i, i, vp, llp, vp, vp, llp, vp, llp, ip, i]),
        "nd4jb200_exec_reduce3_all": (i, [vp, i, i, vp, llp, vp, vp, llp, vp, llp, ip, i]),
        "nd4jb200_exec_reduce3_scalar": (i, [vp, i, i, vp, llp, vp, vp, llp, dp]),
        "nd4jb200_exec_transform": (i, [vp, i, i, vp, llp, vp, llp, vp]),
        "nd4jb200_exec_transform_strided": (i, [vp, i, i, vp, ll, vp, ll, vp, ll]),
        "nd4jb200_exec_pairwise": (i, [vp, i, i, vp, llp, vp, llp, vp, llp, vp]),
        "nd4jb200_exec_pairwise_strided": (i, [vp, i, i, vp, ll, vp, ll, vp, ll, vp, ll]),
        "nd4jb200_exec_pairwise_indexed": (i, [vp, i, i, vp, llp, vp, vp, vp, vp, vp, vp]),
        "nd4jb200_exec_scalar_indexed": (i, [vp, i, i, vp, llp, vp, d, vp, vp, vp]),
        "nd4jb200_exec_chain": (i, [vp, i, i, vp, llp, vp, llp, ip, i, i, vp, i, vp, llp, vp, vp, llp]),
        "nd4jb200_exec_meta_predicate_shape": (i, [vp, i, i, i, i, i, vp, llp, vp, llp, vp, llp, vp, vp, d, d]),
        "nd4jb200_exec_meta_predicate_strided": (i, [vp, i, i, i, i, i, ll, vp, ll, vp, ll, vp, ll, vp, vp, d, d]),
        "nd4jb200_comm_unique_id": (i, [vp]),
        "nd4jb200_comm_init": (i, [vp, i, i]),
        "nd4jb200_comm_destroy": (i, []),
        "nd4jb200_comm_rank": (i, []),
        "nd4jb200_comm_world": (i, []),
        "nd4jb200_exec_reduce_scalar_sharded": (i, [vp, i, i, vp, ll, vp, i, ll, vp, dp]),
        "nd4jb200_accumulate_across": (i, [vp, i, vp, vp, ll]),
        "nd4jb200_average_across": (i, [vp, i, vp, vp, ll, i]),
        "nd4jb200_exec_broadcast": (i, [vp, i, i, vp, llp, vp, llp, vp, llp, ip, i]),
        "nd4jb200_exec_scalar": (i, [vp, i, i, vp, llp, vp, llp, d, vp]),
        "nd4jb200_exec_scalar_strided": (i, [vp, i, i, vp, ll, vp, ll, d, vp, ll]),
        "nd4jb200_exec_scalar_along_dimension": (i, [vp, i, i, vp, llp, vp, vp, llp, vp, ip, i]),
        "nd4jb200_init_random": (vp, [vp, ll, ll, vp, vp]),
        "nd4jb200_refresh_buffer": (i, [vp, ll, vp]),
        "nd4jb200_reseed_buffer": (i, [ll, vp]),
        "nd4jb200_destroy_random": (i, [vp]),
        "nd4jb200_exec_random": (i, [vp, i, i, vp, vp, llp, vp]),
        "nd4jb200_exec_random_x": (i, [vp, i, i, vp, vp, llp, vp, llp, vp]),
        "nd4jb200_exec_random_xy": (i, [vp, i, i, vp, vp, llp, vp, llp, vp, llp, vp]),
        "nd4jb200_exec_random_range": (i, [vp, i, i, i, vp, vp, vp, vp, vp, ll, ll, ll]),
        "nd4jb200_rng_rewind": (i, [vp, ll]),
        "nd4jb200_rng_get_state": (i, [vp, llp]),
        "nd4jb200_rng_set_state": (i, [vp, llp]),
        "nd4jb200_rng_device_table": (vp, [vp]),
        "nd4jb200_tad_only_shape_info": (i, [llp, ip, i, llp, llp]),
        "nd4jb200_tad_count": (ll, [llp, ip, i]),
        "nd4jb200_dims_from_tad": (i, [llp, llp, ip]),
        "nd4jb200_metadata_reads": (ctypes.c_ulonglong, []),
        "nd4jb200_check_p2p": (i, []),
        "nd4jb200_is_p2p_available": (i, []),
        "nd4jb200_enable_p2p": (i, [i]),
        "nd4jb200_memcpy_constant_async": (i, [ll, vp, ll, i, vp]),
        "nd4jb200_get_constant_space": (vp, []),
        "nd4jb200_get_available_devices": (i, []),
        "nd4jb200_set_device": (i, [i]),
        "nd4jb200_get_device": (i, []),
        "nd4jb200_malloc_device": (vp, [ll]),
        "nd4jb200_free_device": (i, [vp]),
        "nd4jb200_malloc_host": (vp, [ll]),
        "nd4jb200_free_host": (i, [vp]),
        "nd4jb200_create_stream": (vp, []),
        "nd4jb200_destroy_stream": (i, [vp]),
        "nd4jb200_stream_synchronize": (i, [vp]),
        "nd4jb200_create_event": (vp, []),
        "nd4jb200_register_event": (i, [vp, vp]),
        "nd4jb200_event_synchronize": (i, [vp]),
        "nd4jb200_destroy_event": (i, [vp]),
        "nd4jb200_event_elapsed_ms": (i, [vp, vp, ctypes.POINTER(ctypes.c_float)]),
        "nd4jb200_memcpy_async": (i, [vp, vp, ll, i, vp]),
        "nd4jb200_memcpy": (i, [vp, vp, ll, i]),
        "nd4jb200_memset_async": (i, [vp, i, ll, vp]),
        "nd4jb200_device_free_memory": (ll, [i]),
        "nd4jb200_device_total_memory": (ll, [i]),
        "nd4jb200_device_major": (i, [i]),
        "nd4jb200_device_minor": (i, [i]),
        "nd4jb200_device_name": (ctypes.c_char_p, [i]),
    }
    for name, (res, args) in sig.items():
        fn = getattr(lib, name)
        fn.restype = res
        fn.argtypes = args
    return lib


#: every extern "C" symbol include/nd4j_b200.h declares (checked by the CPU test suite)
EXPORTED_SYMBOLS = None


class NativeOps:
    """Mirror of the reference's NativeOps for the legacy families (see module docstring)."""

    def __init__(self, lib_path=None):
        self.lib = load_library(lib_path)
        self.stream = None  # default stream unless extraPointers[1] overrides it per call

    # ---- plumbing ---------------------------------------------------------------------------
    def _check(self, code):
        if code != 0:
            raise Nd4jError(code, self.lib.nd4jb200_last_error().decode())

    def _stream(self, extraPointers):
        if extraPointers is not None and len(extraPointers) > 1 and extraPointers[1]:
            return _ptr(extraPointers[1])
        return _ptr(self.stream)

    def lastError(self):
        return self.lib.nd4jb200_last_error().decode()

    def launchCount(self):
        return int(self.lib.nd4jb200_launch_count())

    # ---- families (dtype-generic bodies; the Float/Double/Half members are generated below) ---
    def _execReduce(self, dt, extraPointers, opNum, x, xShapeInfo, extraParams, result, resultShapeInfo,
                    dimension=None, dimensionLength=0):
        xs, xsp = _longs(xShapeInfo)
        zs, zsp = _longs(resultShapeInfo)
        dm, dmp = _ints(dimension)
        self._check(self.lib.nd4jb200_exec_reduce(self._stream(extraPointers), dt, opNum, _ptr(x), xsp,
                                                  _ptr(extraParams), _ptr(result), zsp, dmp, dimensionLength))

    def _execReduceScalar(self, dt, extraPointers, opNum, x, xShapeInfo, extraParams):
        xs, xsp = _longs(xShapeInfo)
        out = ctypes.c_double()
        self._check(self.lib.nd4jb200_exec_reduce_scalar(self._stream(extraPointers), dt, opNum, _ptr(x), xsp,
                                                         _ptr(extraParams), ctypes.byref(out)))
        return out.value

    def _execIndexReduce(self, dt, extraPointers, opNum, x, xShapeInfo, extraParams, result, resultShapeInfo,
                         dimension=None, dimensionLength=0):
        xs, xsp = _longs(xShapeInfo)
        zs, zsp = _longs(resultShapeInfo)
        dm, dmp = _ints(dimension)
        self._check(self.lib.nd4jb200_exec_index_reduce(self._stream(extraPointers), dt, opNum, _ptr(x), xsp,
                                                        _ptr(extraParams), _ptr(result), zsp, dmp, dimensionLength))

    def _execIndexReduceScalar(self, dt, extraPointers, opNum, x, xShapeInfo, extraParams):
        xs, xsp = _longs(xShapeInfo)
        out = ctypes.c_double()
        self._check(self.lib.nd4jb200_exec_index_reduce_scalar(self._stream(extraPointers), dt, opNum, _ptr(x), xsp,
                                                               _ptr(extraParams), ctypes.byref(out)))
        return out.value

    def _execSummaryStats(self, dt, extraPointers, opNum, x, xShapeInfo, extraParams, result, resultShapeInfo,
                          dimension=None, dimensionLength=0, biasCorrected=True):
        # the reference also has an overload without dimension; there biasCorrected comes 8th
        if isinstance(dimension, bool):
            dimension, biasCorrected = None, dimension
        xs, xsp = _longs(xShapeInfo)
        zs, zsp = _longs(resultShapeInfo)
        dm, dmp = _ints(dimension)
        self._check(self.lib.nd4jb200_exec_summary_stats(self._stream(extraPointers), dt, opNum, _ptr(x), xsp,
                                                         _ptr(extraParams), _ptr(result), zsp, dmp, dimensionLength,
                                                         1 if biasCorrected else 0))

    def _execSummaryStatsScalar(self, dt, extraPointers, opNum, x, xShapeInfo, extraParams, biasCorrected):
        xs, xsp = _longs(xShapeInfo)
        out = ctypes.c_double()
        self._check(self.lib.nd4jb200_exec_summary_stats_scalar(self._stream(extraPointers), dt, opNum, _ptr(x), xsp,
                                                                _ptr(extraParams), 1 if biasCorrected else 0,
                                                                ctypes.byref(out)))
        return out.value

    def _execReduce3(self, dt, extraPointers, opNum, x, xShapeInfo, extraParamsVals, y, yShapeInfo, result,
                     resultShapeInfo, dimension=None, dimensionLength=0):
        xs, xsp = _longs(xShapeInfo)
        ys, ysp = _longs(yShapeInfo)
        zs, zsp = _longs(resultShapeInfo)
        dm, dmp = _ints(dimension)
        self._check(self.lib.nd4jb200_exec_reduce3(self._stream(extraPointers), dt, opNum, _ptr(x), xsp,
                                                   _ptr(extraParamsVals), _ptr(y), ysp, _ptr(result), zsp, dmp,
                                                   dimensionLength))

    def _execReduce3All(self, dt, extraPointers, opNum, x, xInfo, extraParamsVals, y, yInfo, result,
                        resultShapeInfoBuffer, dimension, dimensionLength, xTadShapeInfo=None, xOffsets=None,
                        yTadShapeInfo=None, yOffsets=None):
        """Every TAD of x against every TAD of y; the TAD descriptors of the reference's signature are
        accepted and ignored (the geometry is derived from the shapeInfos and the dimension list)."""
        xs, xsp = _longs(xInfo)
        ys, ysp = _longs(yInfo)
        zs, zsp = _longs(resultShapeInfoBuffer)
        dm, dmp = _ints(dimension)
        self._check(self.lib.nd4jb200_exec_reduce3_all(self._stream(extraPointers), dt, opNum, _ptr(x), xsp,
                                                       _ptr(extraParamsVals), _ptr(y), ysp, _ptr(result), zsp, dmp,
                                                       dimensionLength))

    def _execReduce3Scalar(self, dt, extraPointers, opNum, x, xShapeInfo, extraParamsVals, y, yShapeInfo):
        xs, xsp = _longs(xShapeInfo)
        ys, ysp = _longs(yShapeInfo)
        out = ctypes.c_double()
        self._check(self.lib.nd4jb200_exec_reduce3_scalar(self._stream(extraPointers), dt, opNum, _ptr(x), xsp,
                                                          _ptr(extraParamsVals), _ptr(y), ysp, ctypes.byref(out)))
        return out.value

    def _execTransform(self, dt, extraPointers, opNum, dx, xShapeInfo, result, resultShapeInfo, extraParams, n=None):
        st = self._stream(extraPointers)
        if n is not None:  # strided overload: (dx, xStride, result, resultStride, extraParams, n)
            self._check(self.lib.nd4jb200_exec_transform_strided(st, dt, opNum, _ptr(dx), int(xShapeInfo), _ptr(result),
                                                                 int(resultShapeInfo), _ptr(extraParams), int(n)))
            return
        xs, xsp = _longs(xShapeInfo)
        zs, zsp = _longs(resultShapeInfo)
        self._check(self.lib.nd4jb200_exec_transform(st, dt, opNum, _ptr(dx), xsp, _ptr(result), zsp, _ptr(extraParams)))

    def _execPairwiseTransform(self, dt, extraPointers, opNum, dx, xShapeInfo, y, yShapeInfo, result, resultShapeInfo,
                               extraParams, n=None, yIndexes=None, resultIndexes=None):
        """Three overloads, as in the reference: shaped (nine arguments), strided (`n` = element count, the
        three shapeInfo slots carry strides) and indexed (`n`, `yIndexes`, `resultIndexes` carry the device
        index arrays xIndexes, yIndexes, resultIndexes)."""
        st = self._stream(extraPointers)
        if yIndexes is not None:  # indexed overload
            xs, xsp = _longs(xShapeInfo)
            self._check(self.lib.nd4jb200_exec_pairwise_indexed(st, dt, opNum, _ptr(dx), xsp, _ptr(y), _ptr(result),
                                                                _ptr(extraParams), _ptr(n), _ptr(yIndexes),
                                                                _ptr(resultIndexes)))
            return
        if n is not None:  # strided overload
            self._check(self.lib.nd4jb200_exec_pairwise_strided(st, dt, opNum, _ptr(dx), int(xShapeInfo), _ptr(y),
                                                                int(yShapeInfo), _ptr(result), int(resultShapeInfo),
                                                                _ptr(extraParams), int(n)))
            return
        xs, xsp = _longs(xShapeInfo)
        ys, ysp = _longs(yShapeInfo)
        zs, zsp = _longs(resultShapeInfo)
        self._check(self.lib.nd4jb200_exec_pairwise(st, dt, opNum, _ptr(dx), xsp, _ptr(y), ysp, _ptr(result), zsp,
                                                    _ptr(extraParams)))

    def _execBroadcast(self, dt, extraPointers, opNum, x, xShapeInfo, y, yShapeInfo, result, resultShapeInfo,
                       dimension, dimensionLength):
        xs, xsp = _longs(xShapeInfo)
        ys, ysp = _longs(yShapeInfo)
        zs, zsp = _longs(resultShapeInfo)
        dm, dmp = _ints(dimension)
        self._check(self.lib.nd4jb200_exec_broadcast(self._stream(extraPointers), dt, opNum, _ptr(x), xsp, _ptr(y), ysp,
                                                     _ptr(result), zsp, dmp, dimensionLength))

    # ---- several GPUs (nd4jb200_comm_*) ---------------------------------------------------------
    def commUniqueId(self):
        buf = ctypes.create_string_buffer(128)
        self._check(self.lib.nd4jb200_comm_unique_id(buf))
        return buf.raw

    def commInit(self, unique_id, rank, world):
        self._check(self.lib.nd4jb200_comm_init(unique_id, rank, world))

    def commDestroy(self):
        self._check(self.lib.nd4jb200_comm_destroy())

    def execReduceScalarSharded(self, dt, extraPointers, opNum, x, localLength, extraParams, shardsPerRank, totalLength,
                                z=None, fetch=True):
        """Whole-array reduce over world * shardsPerRank shards (nd4jb200_exec_reduce_scalar_sharded); returns the
        value when `fetch`, else None (asynchronous, value in z)."""
        out = ctypes.c_double()
        self._check(self.lib.nd4jb200_exec_reduce_scalar_sharded(self._stream(extraPointers), dt, opNum, _ptr(x), localLength,
                                                                 _ptr(extraParams), shardsPerRank, totalLength, _ptr(z),
                                                                 ctypes.byref(out) if fetch else None))
        return out.value if fetch else None

    def accumulateAcross(self, dt, extraPointers, x, z, length):
        self._check(self.lib.nd4jb200_accumulate_across(self._stream(extraPointers), dt, _ptr(x), _ptr(z), length))

    def averageAcross(self, dt, extraPointers, x, z, length, propagate):
        self._check(self.lib.nd4jb200_average_across(self._stream(extraPointers), dt, _ptr(x), _ptr(z), length, 1 if propagate else 0))

    def execChain(self, dt, extraPointers, broadcastOp, x, xShapeInfo, b, bShapeInfo, dimension, dimensionLength,
                  transformOp, transformExtra, pairwiseOp, y, yShapeInfo, pairwiseExtra, z, zShapeInfo):
        """z = pairwise(transform(broadcast(x, b)), y) in one pass (nd4jb200_exec_chain): what execBroadcast ->
        execTransform -> execPairwiseTransform would compute, bit for bit."""
        xs, xsp = _longs(xShapeInfo)
        bs, bsp = _longs(bShapeInfo)
        ys, ysp = _longs(yShapeInfo)
        zs, zsp = _longs(zShapeInfo)
        dm, dmp = _ints(dimension)
        self._check(self.lib.nd4jb200_exec_chain(self._stream(extraPointers), dt, broadcastOp, _ptr(x), xsp, _ptr(b), bsp,
                                                 dmp, dimensionLength, transformOp, _ptr(transformExtra), pairwiseOp,
                                                 _ptr(y), ysp, _ptr(pairwiseExtra), _ptr(z), zsp))

    def _execMetaPredicateShape(self, dt, extras, opTypeA, opNumA, opTypeB, opNumB, N, dx, xShapeInfo, dy, yShapeInfo,
                                dz, zShapeInfo, extraA, extraB, scalarA, scalarB):
        xs, xsp = _longs(xShapeInfo)
        ys, ysp = _longs(yShapeInfo)
        zs, zsp = _longs(zShapeInfo)
        self._check(self.lib.nd4jb200_exec_meta_predicate_shape(self._stream(extras), dt, opTypeA, opNumA, opTypeB, opNumB,
                                                                _ptr(dx), xsp, _ptr(dy), ysp, _ptr(dz), zsp, _ptr(extraA),
                                                                _ptr(extraB), float(scalarA), float(scalarB)))

    def _execMetaPredicateStrided(self, dt, extras, opTypeA, opNumA, opTypeB, opNumB, N, dx, xStride, dy, yStride, dz,
                                  zStride, extraA, extraB, scalarA, scalarB):
        self._check(self.lib.nd4jb200_exec_meta_predicate_strided(self._stream(extras), dt, opTypeA, opNumA, opTypeB,
                                                                  opNumB, N, _ptr(dx), xStride, _ptr(dy), yStride, _ptr(dz),
                                                                  zStride, _ptr(extraA), _ptr(extraB), float(scalarA),
                                                                  float(scalarB)))

    def _execScalar(self, dt, extraPointers, opNum, x, xShapeInfo, result, resultShapeInfo, scalar, extraParams,
                    n=None, resultIndexes=None):
        """Shaped, strided (`n` = element count) and indexed (`n`, `resultIndexes` carry the device index
        arrays xIndexes, resultIndexes) overloads."""
        st = self._stream(extraPointers)
        if resultIndexes is not None:  # indexed overload
            xs, xsp = _longs(xShapeInfo)
            self._check(self.lib.nd4jb200_exec_scalar_indexed(st, dt, opNum, _ptr(x), xsp, _ptr(result), float(scalar),
                                                              _ptr(extraParams), _ptr(n), _ptr(resultIndexes)))
            return
        if n is not None:  # strided overload
            self._check(self.lib.nd4jb200_exec_scalar_strided(st, dt, opNum, _ptr(x), int(xShapeInfo), _ptr(result),
                                                              int(resultShapeInfo), float(scalar), _ptr(extraParams),
                                                              int(n)))
            return
        xs, xsp = _longs(xShapeInfo)
        zs, zsp = _longs(resultShapeInfo)
        self._check(self.lib.nd4jb200_exec_scalar(st, dt, opNum, _ptr(x), xsp, _ptr(result), zsp, float(scalar),
                                                  _ptr(extraParams)))

    def _execScalarAlongDimension(self, dt, extraPointers, opNum, x, xShapeInfo, z, zShapeInfo, scalars, extraParams,
                                  dimension, dimensionLength):
        xs, xsp = _longs(xShapeInfo)
        zs, zsp = _longs(zShapeInfo)
        dm, dmp = _ints(dimension)
        self._check(self.lib.nd4jb200_exec_scalar_along_dimension(self._stream(extraPointers), dt, opNum, _ptr(x), xsp,
                                                                  _ptr(extraParams), _ptr(z), zsp, _ptr(scalars), dmp,
                                                                  dimensionLength))

    def _execRandom(self, dt, extraPointers, opNum, state, *args):
        """execRandom{T}(extra, op, state, z, zShape, extraArgs)
        | (extra, op, state, x, xShape, z, zShape, extraArgs)
        | (extra, op, state, x, xShape, y, yShape, z, zShape, extraArgs)"""
        st = self._stream(extraPointers)
        if len(args) == 3:
            z, zShape, extra = args
            zs, zsp = _longs(zShape)
            self._check(self.lib.nd4jb200_exec_random(st, dt, opNum, _ptr(state), _ptr(z), zsp, _ptr(extra)))
        elif len(args) == 5:
            x, xShape, z, zShape, extra = args
            xs, xsp = _longs(xShape)
            zs, zsp = _longs(zShape)
            self._check(self.lib.nd4jb200_exec_random_x(st, dt, opNum, _ptr(state), _ptr(x), xsp, _ptr(z), zsp,
                                                        _ptr(extra)))
        elif len(args) == 7:
            x, xShape, y, yShape, z, zShape, extra = args
            xs, xsp = _longs(xShape)
            ys, ysp = _longs(yShape)
            zs, zsp = _longs(zShape)
            self._check(self.lib.nd4jb200_exec_random_xy(st, dt, opNum, _ptr(state), _ptr(x), xsp, _ptr(y), ysp,
                                                         _ptr(z), zsp, _ptr(extra)))
        else:
            raise TypeError("execRandom takes 3, 5 or 7 arguments after the state")

    def execRandomRange(self, dt, extraPointers, opNum, arity, state, x, y, z, extraArguments, first, count, length):
        """Offset-sharded generation (no counterpart in the reference): elements
        [first, first+count) of a logical call of `length` elements; the state is not advanced."""
        self._check(self.lib.nd4jb200_exec_random_range(self._stream(extraPointers), dt, opNum, arity, _ptr(state),
                                                        _ptr(x), _ptr(y), _ptr(z), _ptr(extraArguments), first, count,
                                                        length))

    # ---- RNG state (blas/NativeOps.h:2510-2539) ------------------------------------------------
    def initRandom(self, extraPointers, seed, bufferSize, ptrToBuffer=None):
        host = extraPointers[0] if extraPointers is not None and len(extraPointers) > 0 else None
        state = self.lib.nd4jb200_init_random(self._stream(extraPointers), seed, bufferSize, _ptr(host),
                                              _ptr(ptrToBuffer))
        if not state:
            raise Nd4jError(-1, self.lastError())
        return state

    def refreshBuffer(self, extraPointers, seed, ptrRandom):
        self._check(self.lib.nd4jb200_refresh_buffer(self._stream(extraPointers), seed, _ptr(ptrRandom)))

    def reSeedBuffer(self, extraPointers, seed, ptrRandom):
        self._check(self.lib.nd4jb200_reseed_buffer(seed, _ptr(ptrRandom)))

    def destroyRandom(self, ptrRandom):
        self._check(self.lib.nd4jb200_destroy_random(_ptr(ptrRandom)))

    def rngRewind(self, ptrRandom, count):
        self._check(self.lib.nd4jb200_rng_rewind(_ptr(ptrRandom), count))

    def rngState(self, ptrRandom):
        """(seed, currentPosition, generation, amplifier, size)"""
        words = (ctypes.c_longlong * 5)()
        self._check(self.lib.nd4jb200_rng_get_state(_ptr(ptrRandom), words))
        return tuple(int(w) for w in words)

    def rngSetState(self, ptrRandom, seed, position, generation, amplifier):
        words = (ctypes.c_longlong * 4)(seed, position, generation, amplifier)
        self._check(self.lib.nd4jb200_rng_set_state(_ptr(ptrRandom), words))

    # ---- shape helpers ---------------------------------------------------------------------
    def tadOnlyShapeInfo(self, xShapeInfo, dimension, dimensionLength, target=None, offsets=None):
        """Returns (tadShapeInfo, tadOffsets) as numpy arrays (NativeOps.h:1880)."""
        xs, xsp = _longs(xShapeInfo)
        dm, dmp = _ints(dimension)
        n = self.lib.nd4jb200_tad_count(xsp, dmp, dimensionLength)
        if n < 0:
            raise Nd4jError(1, self.lastError())
        tgt = np.zeros(2 * 32 + 4, dtype=np.int64)
        off = np.zeros(max(int(n), 1), dtype=np.int64)
        self._check(self.lib.nd4jb200_tad_only_shape_info(
            xsp, dmp, dimensionLength, tgt.ctypes.data_as(ctypes.POINTER(ctypes.c_longlong)),
            off.ctypes.data_as(ctypes.POINTER(ctypes.c_longlong))))
        r = int(tgt[0])
        return tgt[:2 * r + 4].copy(), off[:int(n)].copy()

    def dimsFromTad(self, xShapeInfo, tadShapeInfo):
        """The dimension list that yields the given TADs of x, recovered from the two host descriptors, or None
        when they do not determine it (nd4jb200_dims_from_tad). An empty list means the whole array."""
        xs, xsp = _longs(xShapeInfo)
        ts, tsp = _longs(tadShapeInfo)
        out = np.zeros(32, dtype=np.int32)
        n = self.lib.nd4jb200_dims_from_tad(xsp, tsp, out.ctypes.data_as(ctypes.POINTER(ctypes.c_int)))
        return None if n < 0 else [int(v) for v in out[:n]]

    # ---- device / memory / stream utilities (blas/NativeOps.h:1607-1870) ---------------------
    def getAvailableDevices(self):
        return self.lib.nd4jb200_get_available_devices()

    def setDevice(self, device):
        self._check(self.lib.nd4jb200_set_device(int(device)))

    def getDevice(self):
        return self.lib.nd4jb200_get_device()

    def mallocDevice(self, memorySize, ptrToDeviceId=None, flags=0):
        p = self.lib.nd4jb200_malloc_device(memorySize)
        if not p:
            raise Nd4jError(4, self.lastError())
        return p

    def freeDevice(self, pointer, ptrToDeviceId=None):
        self._check(self.lib.nd4jb200_free_device(_ptr(pointer)))

    def mallocHost(self, memorySize, flags=0):
        p = self.lib.nd4jb200_malloc_host(memorySize)
        if not p:
            raise Nd4jError(4, self.lastError())
        return p

    def freeHost(self, pointer):
        self._check(self.lib.nd4jb200_free_host(_ptr(pointer)))

    def createStream(self):
        s = self.lib.nd4jb200_create_stream()
        if not s:
            raise Nd4jError(4, self.lastError())
        return s

    def destroyStream(self, stream):
        self._check(self.lib.nd4jb200_destroy_stream(_ptr(stream)))

    def streamSynchronize(self, stream):
        self._check(self.lib.nd4jb200_stream_synchronize(_ptr(stream)))

    def createEvent(self):
        e = self.lib.nd4jb200_create_event()
        if not e:
            raise Nd4jError(4, self.lastError())
        return e

    def registerEvent(self, event, stream):
        self._check(self.lib.nd4jb200_register_event(_ptr(event), _ptr(stream)))

    def eventSynchronize(self, event):
        self._check(self.lib.nd4jb200_event_synchronize(_ptr(event)))

    def destroyEvent(self, event):
        self._check(self.lib.nd4jb200_destroy_event(_ptr(event)))

    def eventElapsedMs(self, start, stop):
        ms = ctypes.c_float()
        self._check(self.lib.nd4jb200_event_elapsed_ms(_ptr(start), _ptr(stop), ctypes.byref(ms)))
        return ms.value

    # ---- memory-movement utilities (generic bodies; Float / Double / Half names are bound below) ----
    def _flatten(self, dt, extraPointers, offset, order, result, resultShapeInfo, input, inputShapeInfo):
        zs, zsp = _longs(resultShapeInfo)
        xs, xsp = _longs(inputShapeInfo)
        o = order.encode() if isinstance(order, str) else order
        self._check(self.lib.nd4jb200_flatten(self._stream(extraPointers), dt, offset, o, _ptr(result), zsp, _ptr(input), xsp))

    def _concat(self, dt, extraPointers, dimension, numArrays, data, inputShapeInfo, result, resultShapeInfo,
                tadPointers=None, offsetPointers=None):
        """`data`: sequence of device arrays; `inputShapeInfo`: sequence of shapeInfo arrays."""
        ptrs = (ctypes.c_void_p * numArrays)(*[_ptr(d).value for d in data])
        keep = [_longs(s) for s in inputShapeInfo]
        infos = (ctypes.c_void_p * numArrays)(*[ctypes.cast(k[1], ctypes.c_void_p).value for k in keep])
        zs, zsp = _longs(resultShapeInfo)
        self._check(self.lib.nd4jb200_concat(self._stream(extraPointers), dt, dimension, numArrays, ptrs, infos,
                                             _ptr(result), zsp))

    def _pullRows(self, dt, extraPointers, x, xShapeInfo, z, zShapeInfo, n, indexes, tadShapeInfo, tadOffsets,
                  zTadShapeInfo, zTadOffsets):
        ts, tsp = _longs(tadShapeInfo)
        zts, ztsp = _longs(zTadShapeInfo)
        self._check(self.lib.nd4jb200_pull_rows(self._stream(extraPointers), dt, _ptr(x), _ptr(z), n, _ptr(indexes), tsp,
                                                _ptr(tadOffsets), ztsp, _ptr(zTadOffsets)))

    def _tear(self, dt, extraPointers, x, xShapeInfo, targets, zShapeInfo, tadShapeInfo, tadOffsets):
        """`targets`: sequence of device arrays, one per TAD of x; `tadOffsets`: device array."""
        xs, xsp = _longs(xShapeInfo)
        zs, zsp = _longs(zShapeInfo)
        ts, tsp = _longs(tadShapeInfo)
        ptrs = (ctypes.c_void_p * len(targets))(*[_ptr(t).value for t in targets])
        self._check(self.lib.nd4jb200_tear(self._stream(extraPointers), dt, _ptr(x), xsp, ptrs, zsp, tsp, _ptr(tadOffsets)))

    def _shuffle(self, dt, extras, dx, xShapeInfo, dz, zShapeInfo, N, shuffleMap, tadShapeInfo, tadOffsets):
        """`dx`, `xShapeInfo`, `tadShapeInfo`, `tadOffsets`: sequences of N entries; `shuffleMap`: host ints.
        The arrays are shuffled in place; `dz` / `zShapeInfo` are unused, as in the reference."""
        ptrs = (ctypes.c_void_p * N)(*[_ptr(d).value for d in dx])
        keepX = [_longs(s) for s in xShapeInfo]
        keepT = [_longs(s) for s in tadShapeInfo]
        infos = (ctypes.c_void_p * N)(*[ctypes.cast(k[1], ctypes.c_void_p).value for k in keepX])
        tads = (ctypes.c_void_p * N)(*[ctypes.cast(k[1], ctypes.c_void_p).value for k in keepT])
        offs = (ctypes.c_void_p * N)(*[_ptr(o).value for o in tadOffsets])
        m, mp = _ints(shuffleMap)
        self._check(self.lib.nd4jb200_shuffle(self._stream(extras), dt, N, ptrs, infos, mp, tads, offs))

    def _sort(self, dt, extraPointers, x, xShapeInfo, descending):
        xs, xsp = _longs(xShapeInfo)
        self._check(self.lib.nd4jb200_sort(self._stream(extraPointers), dt, _ptr(x), xsp, 1 if descending else 0))

    def _sortTad(self, dt, extraPointers, x, xShapeInfo, dimension, dimensionLength, tadShapeInfo=None, tadOffsets=None,
                 descending=False):
        xs, xsp = _longs(xShapeInfo)
        d, dp = _ints(dimension)
        self._check(self.lib.nd4jb200_sort_tad(self._stream(extraPointers), dt, _ptr(x), xsp, dp, dimensionLength,
                                               1 if descending else 0))

    def _average(self, dt, extras, dx, dz, n, length, propagate):
        ptrs = (ctypes.c_void_p * n)(*[_ptr(d).value for d in dx])
        self._check(self.lib.nd4jb200_average(self._stream(extras), dt, ptrs, _ptr(dz), n, length, 1 if propagate else 0))

    def _accumulate(self, dt, extras, dx, dz, n, length):
        ptrs = (ctypes.c_void_p * n)(*[_ptr(d).value for d in dx])
        self._check(self.lib.nd4jb200_accumulate(self._stream(extras), dt, ptrs, _ptr(dz), n, length))

    def convertTypes(self, extras, srcType, x, N, dstType, z):
        """ND4J_INT8 = 1, UINT8 = 2, FLOAT16 = 3, INT16 = 4, UINT16 = 5 (result only), FLOAT32 = 6, DOUBLE = 7
        (NativeOps.h:2144; include/loops/type_conversions.h:11-19)."""
        self._check(self.lib.nd4jb200_convert_types(self._stream(extras), srcType, _ptr(x), N, dstType, _ptr(z)))

    def memcpyAsync(self, dst, src, size, flags, reserved=None):
        self._check(self.lib.nd4jb200_memcpy_async(_ptr(dst), _ptr(src), size, flags, _ptr(reserved)))

    def memcpy(self, dst, src, size, flags, reserved=None):
        self._check(self.lib.nd4jb200_memcpy(_ptr(dst), _ptr(src), size, flags))

    def memsetAsync(self, dst, value, size, flags=0, reserved=None):
        self._check(self.lib.nd4jb200_memset_async(_ptr(dst), value, size, _ptr(reserved)))

    def memcpyConstantAsync(self, dst, src, size, flags, reserved=None):
        self._check(self.lib.nd4jb200_memcpy_constant_async(int(dst), _ptr(src), int(size), int(flags), _ptr(reserved)))
        return 1

    def getConstantSpace(self):
        p = self.lib.nd4jb200_get_constant_space()
        if not p:
            raise Nd4jError(4, self.lastError())
        return p

    def enableP2P(self, enable):
        self._check(self.lib.nd4jb200_enable_p2p(1 if enable else 0))

    def checkP2P(self):
        self._check(self.lib.nd4jb200_check_p2p())

    def isP2PAvailable(self):
        return bool(self.lib.nd4jb200_is_p2p_available())

    def getDeviceFreeMemory(self, device=0):
        return self.lib.nd4jb200_device_free_memory(int(device))

    def getDeviceTotalMemory(self, device=0):
        return self.lib.nd4jb200_device_total_memory(int(device))

    def getDeviceMajor(self, device=0):
        return self.lib.nd4jb200_device_major(int(device))

    def getDeviceMinor(self, device=0):
        return self.lib.nd4jb200_device_minor(int(device))

    def getDeviceName(self, device=0):
        return self.lib.nd4jb200_device_name(int(device)).decode()


def _bind(generic, dt):
    def method(self, *args, **kwargs):
        return getattr(self, generic)(dt, *args, **kwargs)
    return method


for _fam in ("execReduce", "execReduceScalar", "execIndexReduce", "execIndexReduceScalar", "execSummaryStats",
             "execSummaryStatsScalar", "execReduce3", "execReduce3All", "execReduce3Scalar", "execTransform", "execPairwiseTransform",
             "execBroadcast", "execScalar", "execScalarAlongDimension", "execRandom", "flatten", "concat", "pullRows",
             "tear", "shuffle", "sort", "sortTad", "average", "accumulate", "execMetaPredicateShape",
             "execMetaPredicateStrided"):
    for _sfx, _dt in _SUFFIX.items():
        _m = _bind("_" + _fam, _dt)
        _m.__name__ = _fam + _sfx
        _m.__doc__ = "NativeOps::%s%s of the reference (blas/NativeOps.h); see the generic body _%s." % (_fam, _sfx, _fam)
        setattr(NativeOps, _fam + _sfx, _m)
