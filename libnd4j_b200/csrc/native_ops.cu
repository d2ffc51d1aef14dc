// The reference-facing C++ surface: NativeOps members with the reference's signatures
// (include/NativeOps.h), each a thin forwarder to the C ABI. The only logic here is recovering
// HOST copies of the shapeInfo / dimension arguments, which the reference's CUDA build receives
// as device pointers plus host copies in extraPointers.
#include "../../include/NativeOps.h"
#include <cuda_runtime.h>
#include <map>
#include <mutex>
#include <stdexcept>
#include <string>
#include <vector>

#include <atomic>

namespace {

// Blocking device-to-host reads of call metadata (shapeInfo, dimension lists) made because a caller left the
// host copies out of extraPointers; read through nd4jb200_metadata_reads().
std::atomic<unsigned long long> g_metadataReads{0};

[[noreturn]] void fail(const char *where) {
    throw std::runtime_error(std::string(where) + ": " + nd4jb200_last_error());
}
inline void check(int status, const char *where) { if (status != 0) fail(where); }

inline void *stream_of(Nd4jPointer *extra) { return extra ? extra[1] : nullptr; }

bool is_device_pointer(const void *p) {
    // descriptors staged in the constant space (memcpyConstantAsync) are device memory whatever the driver
    // reports for addresses of __constant__ symbols
    thread_local const char *constBase[16] = {nullptr};
    int device = 0;
    if (cudaGetDevice(&device) == cudaSuccess && device >= 0 && device < 16) {
        if (!constBase[device]) constBase[device] = static_cast<const char *>(nd4jb200_get_constant_space());
        const char *c = static_cast<const char *>(p);
        if (constBase[device] && c >= constBase[device] && c < constBase[device] + 49152) return true;
    }
    cudaPointerAttributes attr;
    if (cudaPointerGetAttributes(&attr, p) != cudaSuccess) { cudaGetLastError(); return false; }
    return attr.type == cudaMemoryTypeDevice;
}

// Host view of a shapeInfo: the copy in extraPointers[slot] when the caller provided one, otherwise the
// argument itself if it is host memory, otherwise a fresh download. Downloads are not cached by address: a
// caller may free a descriptor and get the same address back for a different shape. The returned pointer
// stays valid until the calling thread has asked for kKeep further descriptors (one call needs at most 4).
constexpr int kKeep = 16;
const Nd4jLong *host_info(Nd4jPointer *extra, int slot, const Nd4jLong *arg) {
    if (extra && slot >= 0 && extra[slot]) return static_cast<const Nd4jLong *>(extra[slot]);
    if (arg == nullptr) return nullptr;
    if (!is_device_pointer(arg)) return arg;
    thread_local std::vector<Nd4jLong> ring[kKeep];
    thread_local int next = 0;
    std::vector<Nd4jLong> &v = ring[next];
    next = (next + 1) % kKeep;
    g_metadataReads.fetch_add(1, std::memory_order_relaxed);
    Nd4jLong rank = 0;
    if (cudaMemcpy(&rank, arg, sizeof(Nd4jLong), cudaMemcpyDeviceToHost) != cudaSuccess || rank < 0 || rank > 32)
        throw std::runtime_error("could not read shapeInfo from the device");
    v.resize(2 * rank + 4);
    if (cudaMemcpy(v.data(), arg, sizeof(Nd4jLong) * v.size(), cudaMemcpyDeviceToHost) != cudaSuccess)
        throw std::runtime_error("could not read shapeInfo from the device");
    return v.data();
}

// The dimension list lives on the device in the reference's CUDA build, while TAD geometry is decoded on the
// host here. Callers of that build keep host copies of x's shapeInfo and of its TAD shapeInfo in
// extraPointers[0] and [9] (blas/cuda/NativeOps.cu:2107-2118); the list is recovered from those two without
// touching the device. Only when a slot is missing, or the descriptors do not determine the list, is the
// device array read back (a blocking copy; dimension buffers are routinely reused with other contents, so the
// download is never cached).
struct HostDims {
    const int *p;
    int n;
};
HostDims host_dims(Nd4jPointer *extra, const int *dimension, int n) {
    if (dimension == nullptr || n <= 0) return HostDims{nullptr, 0};
    thread_local int recovered[32];
    if (extra && extra[0] && extra[9]) {
        const Nd4jLong *xInfo = static_cast<const Nd4jLong *>(extra[0]);
        const int got = nd4jb200_dims_from_tad(xInfo, static_cast<const Nd4jLong *>(extra[9]), recovered);
        if (got > 0) return HostDims{recovered, got};
        if (got == 0) {                       // the TAD is the whole array: every axis is listed
            const int rank = (int) xInfo[0];
            for (int i = 0; i < rank; i++) recovered[i] = i;
            return HostDims{recovered, rank};
        }
    }
    if (!is_device_pointer(dimension)) return HostDims{dimension, n};
    g_metadataReads.fetch_add(1, std::memory_order_relaxed);
    thread_local std::vector<int> v;
    v.resize(n);
    if (cudaMemcpy(v.data(), dimension, sizeof(int) * n, cudaMemcpyDeviceToHost) != cudaSuccess)
        throw std::runtime_error("could not read the dimension array from the device");
    return HostDims{v.data(), n};
}

// A host copy the caller owns: calls that take many descriptors (concat, shuffle) would outrun the ring.
std::vector<Nd4jLong> owned_info(const void *arg) {
    const Nd4jLong *h = host_info(nullptr, -1, static_cast<const Nd4jLong *>(arg));
    if (!h) return std::vector<Nd4jLong>();
    const Nd4jLong rank = h[0] < 0 || h[0] > 32 ? 0 : h[0];
    return std::vector<Nd4jLong>(h, h + 2 * rank + 4);
}

template <class T> struct TypeCode;
template <> struct TypeCode<float> { static constexpr int v = ND4JB200_FLOAT; };
template <> struct TypeCode<double> { static constexpr int v = ND4JB200_DOUBLE; };
template <> struct TypeCode<float16> { static constexpr int v = ND4JB200_HALF; };

}  // namespace

extern "C" __attribute__((visibility("default"))) unsigned long long nd4jb200_metadata_reads(void) {
    return g_metadataReads.load(std::memory_order_relaxed);
}

#define X_INFO host_info(extraPointers, 0, xShapeInfo)
#define Y_INFO host_info(extraPointers, 7, yShapeInfo)
#define Z_INFO(arg) host_info(extraPointers, 8, arg)
#define STREAM stream_of(extraPointers)
#define DIMS host_dims(extraPointers, dimension, dimensionLength)

#define ND4JB200_DEFINE_FAMILIES(T, S, R)                                                                              \
    R NativeOps::execIndexReduceScalar##S(Nd4jPointer *extraPointers, int opNum, T *x, Nd4jLong *xShapeInfo,          \
                                          T *extraParams) {                                                           \
        double out = 0;                                                                                                \
        check(nd4jb200_exec_index_reduce_scalar(STREAM, TypeCode<T>::v, opNum, x, X_INFO, extraParams, &out),         \
              "execIndexReduceScalar" #S);                                                                             \
        return (R) out;                                                                                                \
    }                                                                                                                  \
    void NativeOps::execIndexReduce##S(Nd4jPointer *extraPointers, int opNum, T *x, Nd4jLong *xShapeInfo,             \
                                       T *extraParams, T *result, Nd4jLong *resultShapeInfoBuffer, int *dimension,    \
                                       int dimensionLength) {                                                         \
        const HostDims dims = DIMS;                                                                                    \
        check(nd4jb200_exec_index_reduce(STREAM, TypeCode<T>::v, opNum, x, X_INFO, extraParams, result,               \
                                         Z_INFO(resultShapeInfoBuffer), dims.p,        \
                                         dims.n), "execIndexReduce" #S);                                      \
    }                                                                                                                  \
    void NativeOps::execBroadcast##S(Nd4jPointer *extraPointers, int opNum, T *x, Nd4jLong *xShapeInfo, T *y,         \
                                     Nd4jLong *yShapeInfo, T *result, Nd4jLong *resultShapeInfo, int *dimension,      \
                                     int dimensionLength) {                                                           \
        const HostDims dims = DIMS;                                                                                    \
        check(nd4jb200_exec_broadcast(STREAM, TypeCode<T>::v, opNum, x, X_INFO, y, Y_INFO, result,                    \
                                      Z_INFO(resultShapeInfo), dims.p,                 \
                                      dims.n), "execBroadcast" #S);                                           \
    }                                                                                                                  \
    void NativeOps::execPairwiseTransform##S(Nd4jPointer *extraPointers, int opNum, T *dx, Nd4jLong xStride, T *y,    \
                                             Nd4jLong yStride, T *result, Nd4jLong resultStride, T *extraParams,      \
                                             Nd4jLong n) {                                                            \
        check(nd4jb200_exec_pairwise_strided(STREAM, TypeCode<T>::v, opNum, dx, xStride, y, yStride, result,          \
                                             resultStride, extraParams, n), "execPairwiseTransform" #S);               \
    }                                                                                                                  \
    void NativeOps::execPairwiseTransform##S(Nd4jPointer *extraPointers, int opNum, T *dx, Nd4jLong *xShapeInfo,      \
                                             T *y, Nd4jLong *yShapeInfo, T *result, Nd4jLong *resultShapeInfo,        \
                                             T *extraParams) {                                                        \
        check(nd4jb200_exec_pairwise(STREAM, TypeCode<T>::v, opNum, dx, X_INFO, y, Y_INFO, result,                    \
                                     Z_INFO(resultShapeInfo), extraParams), "execPairwiseTransform" #S);               \
    }                                                                                                                  \
    void NativeOps::execPairwiseTransform##S(Nd4jPointer *extraPointers, int opNum, T *dx, Nd4jLong *xShapeInfo,      \
                                             T *y, Nd4jLong *, T *result, Nd4jLong *, T *extraParams,                 \
                                             Nd4jLong *xIndexes, Nd4jLong *yIndexes, Nd4jLong *resultIndexes) {       \
        check(nd4jb200_exec_pairwise_indexed(STREAM, TypeCode<T>::v, opNum, dx, X_INFO, y, result, extraParams,       \
                                             xIndexes, yIndexes, resultIndexes), "execPairwiseTransform" #S);          \
    }                                                                                                                  \
    void NativeOps::execReduce##S(Nd4jPointer *extraPointers, int opNum, T *x, Nd4jLong *xShapeInfo, T *extraParams,  \
                                  T *result, Nd4jLong *resultShapeInfo) {                                             \
        check(nd4jb200_exec_reduce(STREAM, TypeCode<T>::v, opNum, x, X_INFO, extraParams, result,                     \
                                   Z_INFO(resultShapeInfo), nullptr, 0), "execReduce" #S);                             \
    }                                                                                                                  \
    void NativeOps::execReduce##S(Nd4jPointer *extraPointers, int opNum, T *x, Nd4jLong *xShapeInfo, T *extraParams,  \
                                  T *result, Nd4jLong *resultShapeInfo, int *dimension, int dimensionLength) {        \
        const HostDims dims = DIMS;                                                                                    \
        check(nd4jb200_exec_reduce(STREAM, TypeCode<T>::v, opNum, x, X_INFO, extraParams, result,                     \
                                   Z_INFO(resultShapeInfo), dims.p, dims.n),  \
              "execReduce" #S);                                                                                        \
    }                                                                                                                  \
    R NativeOps::execReduceScalar##S(Nd4jPointer *extraPointers, int opNum, T *x, Nd4jLong *xShapeInfo,               \
                                     T *extraParams) {                                                                \
        double out = 0;                                                                                                \
        check(nd4jb200_exec_reduce_scalar(STREAM, TypeCode<T>::v, opNum, x, X_INFO, extraParams, &out),               \
              "execReduceScalar" #S);                                                                                  \
        return (R) out;                                                                                                \
    }                                                                                                                  \
    void NativeOps::execReduce3##S(Nd4jPointer *extraPointers, int opNum, T *x, Nd4jLong *xShapeInfo,                 \
                                   T *extraParamsVals, T *y, Nd4jLong *yShapeInfo, T *result,                         \
                                   Nd4jLong *resultShapeInfo) {                                                       \
        check(nd4jb200_exec_reduce3(STREAM, TypeCode<T>::v, opNum, x, X_INFO, extraParamsVals, y, Y_INFO, result,     \
                                    Z_INFO(resultShapeInfo), nullptr, 0), "execReduce3" #S);                           \
    }                                                                                                                  \
    R NativeOps::execReduce3Scalar##S(Nd4jPointer *extraPointers, int opNum, T *x, Nd4jLong *xShapeInfo,              \
                                      T *extraParamsVals, T *y, Nd4jLong *yShapeInfo) {                               \
        double out = 0;                                                                                                \
        check(nd4jb200_exec_reduce3_scalar(STREAM, TypeCode<T>::v, opNum, x, X_INFO, extraParamsVals, y, Y_INFO,      \
                                           &out), "execReduce3Scalar" #S);                                             \
        return (R) out;                                                                                                \
    }                                                                                                                  \
    void NativeOps::execReduce3##S(Nd4jPointer *extraPointers, int opNum, T *x, Nd4jLong *xShapeInfo,                 \
                                   T *extraParamsVals, T *y, Nd4jLong *yShapeInfo, T *result,                         \
                                   Nd4jLong *resultShapeInfoBuffer, int *dimension, int dimensionLength) {            \
        const HostDims dims = DIMS;                                                                                    \
        check(nd4jb200_exec_reduce3(STREAM, TypeCode<T>::v, opNum, x, X_INFO, extraParamsVals, y, Y_INFO, result,     \
                                    Z_INFO(resultShapeInfoBuffer), dims.p,             \
                                    dims.n), "execReduce3" #S);                                               \
    }                                                                                                                  \
    void NativeOps::execReduce3All##S(Nd4jPointer *extraPointers, int opNum, T *x, Nd4jLong *xShapeInfo,              \
                                      T *extraParamsVals, T *y, Nd4jLong *yShapeInfo, T *result,                      \
                                      Nd4jLong *resultShapeInfoBuffer, int *dimension, int dimensionLength,           \
                                      Nd4jLong *, Nd4jLong *, Nd4jLong *, Nd4jLong *) {                               \
        const HostDims dims = DIMS;                                                                                    \
        check(nd4jb200_exec_reduce3_all(STREAM, TypeCode<T>::v, opNum, x, X_INFO, extraParamsVals, y, Y_INFO,         \
                                        result, Z_INFO(resultShapeInfoBuffer), dims.p, \
                                        dims.n), "execReduce3All" #S);                                        \
    }                                                                                                                  \
    void NativeOps::flatten##S(Nd4jPointer *extraPointers, int offset, char order, T *result,                         \
                               Nd4jLong *resultShapeInfo, T *input, Nd4jLong *inputShapeInfo) {                       \
        check(nd4jb200_flatten(STREAM, TypeCode<T>::v, offset, order, result, host_info(nullptr, -1, resultShapeInfo),\
                               input, host_info(nullptr, -1, inputShapeInfo)), "flatten" #S);                          \
    }                                                                                                                  \
    void NativeOps::concat##S(Nd4jPointer *extraPointers, int dimension, int numArrays, Nd4jPointer *data,            \
                              Nd4jPointer *inputShapeInfo, T *result, Nd4jLong *resultShapeInfo, Nd4jPointer *,       \
                              Nd4jPointer *) {                                                                        \
        std::vector<std::vector<Nd4jLong> > keep(numArrays > 0 ? numArrays : 0);                                      \
        std::vector<const Nd4jLong *> infos(keep.size());                                                              \
        for (size_t k = 0; k < keep.size(); k++) {                                                                     \
            keep[k] = owned_info(inputShapeInfo[k]);                                                                   \
            infos[k] = keep[k].empty() ? nullptr : keep[k].data();                                                     \
        }                                                                                                              \
        check(nd4jb200_concat(STREAM, TypeCode<T>::v, dimension, numArrays, data, infos.data(), result,               \
                              host_info(nullptr, -1, resultShapeInfo)), "concat" #S);                                  \
    }                                                                                                                  \
    void NativeOps::pullRows##S(Nd4jPointer *extraPointers, T *x, Nd4jLong *, T *z, Nd4jLong *, Nd4jLong n,           \
                                Nd4jLong *indexes, Nd4jLong *tadShapeInfo, Nd4jLong *tadOffsets,                      \
                                Nd4jLong *zTadShapeInfo, Nd4jLong *zTadOffsets) {                                     \
        check(nd4jb200_pull_rows(STREAM, TypeCode<T>::v, x, z, n, indexes, host_info(nullptr, -1, tadShapeInfo),      \
                                 tadOffsets, host_info(nullptr, -1, zTadShapeInfo), zTadOffsets), "pullRows" #S);      \
    }                                                                                                                  \
    void NativeOps::tear##S(Nd4jPointer *extraPointers, T *x, Nd4jLong *xShapeInfo, Nd4jPointer *targets,             \
                            Nd4jLong *zShapeInfo, Nd4jLong *tadShapeInfo, Nd4jLong *tadOffsets) {                     \
        const Nd4jLong *xi = host_info(nullptr, -1, xShapeInfo);                                                      \
        const Nd4jLong *zi = host_info(nullptr, -1, zShapeInfo);                                                      \
        check(nd4jb200_tear(STREAM, TypeCode<T>::v, x, xi, targets, zi, host_info(nullptr, -1, tadShapeInfo),         \
                            tadOffsets), "tear" #S);                                                                   \
    }                                                                                                                  \
    void NativeOps::shuffle##S(Nd4jPointer *extras, Nd4jPointer *dx, Nd4jPointer *xShapeInfo, Nd4jPointer *,          \
                               Nd4jPointer *, int N, int *shuffleMap, Nd4jPointer *tadShapeInfo,                      \
                               Nd4jPointer *tadOffsets) {                                                             \
        std::vector<std::vector<Nd4jLong> > keepX(N > 0 ? N : 0), keepT(keepX.size());                                \
        std::vector<const Nd4jLong *> infos(keepX.size()), tads(keepX.size()), offs(keepX.size());                     \
        for (size_t k = 0; k < keepX.size(); k++) {                                                                    \
            keepX[k] = owned_info(xShapeInfo[k]);                                                                      \
            keepT[k] = owned_info(tadShapeInfo[k]);                                                                    \
            infos[k] = keepX[k].empty() ? nullptr : keepX[k].data();                                                   \
            tads[k] = keepT[k].empty() ? nullptr : keepT[k].data();                                                    \
            offs[k] = static_cast<const Nd4jLong *>(tadOffsets[k]);                                                    \
        }                                                                                                              \
        check(nd4jb200_shuffle(stream_of(extras), TypeCode<T>::v, N, dx, infos.data(), shuffleMap, tads.data(),       \
                               offs.data()), "shuffle" #S);                                                            \
    }                                                                                                                  \
    void NativeOps::sort##S(Nd4jPointer *extraPointers, T *x, Nd4jLong *xShapeInfo, bool descending) {                \
        check(nd4jb200_sort(STREAM, TypeCode<T>::v, x, X_INFO, descending ? 1 : 0), "sort" #S);                       \
    }                                                                                                                  \
    void NativeOps::sortTad##S(Nd4jPointer *extraPointers, T *x, Nd4jLong *xShapeInfo, int *dimension,                \
                               int dimensionLength, Nd4jLong *, Nd4jLong *, bool descending) {                        \
        const HostDims dims = DIMS;                                                                                    \
        check(nd4jb200_sort_tad(STREAM, TypeCode<T>::v, x, X_INFO, dims.p,             \
                                dims.n, descending ? 1 : 0), "sortTad" #S);                                   \
    }                                                                                                                  \
    void NativeOps::average##S(Nd4jPointer *extras, Nd4jPointer *dx, T *dz, int n, Nd4jLong length,                   \
                               bool propagate) {                                                                      \
        check(nd4jb200_average(stream_of(extras), TypeCode<T>::v, dx, dz, n, length, propagate ? 1 : 0),              \
              "average" #S);                                                                                           \
    }                                                                                                                  \
    void NativeOps::accumulate##S(Nd4jPointer *extras, Nd4jPointer *dx, T *dz, int n, Nd4jLong length) {              \
        check(nd4jb200_accumulate(stream_of(extras), TypeCode<T>::v, dx, dz, n, length), "accumulate" #S);             \
    }                                                                                                                  \
    void NativeOps::execScalar##S(Nd4jPointer *extraPointers, int opNum, T *x, Nd4jLong *xShapeInfo, T *z,            \
                                  Nd4jLong *zShapeInfo, T *scalars, T *extraParams, int *dimension,                   \
                                  int dimensionLength) {                                                              \
        const HostDims dims = DIMS;                                                                                    \
        check(nd4jb200_exec_scalar_along_dimension(STREAM, TypeCode<T>::v, opNum, x, X_INFO, extraParams, z,          \
                                                   Z_INFO(zShapeInfo), scalars,                                       \
                                                   dims.p, dims.n),           \
              "execScalar" #S);                                                                                        \
    }                                                                                                                  \
    R NativeOps::execSummaryStatsScalar##S(Nd4jPointer *extraPointers, int opNum, T *x, Nd4jLong *xShapeInfo,         \
                                           T *extraParams, bool biasCorrected) {                                      \
        double out = 0;                                                                                                \
        check(nd4jb200_exec_summary_stats_scalar(STREAM, TypeCode<T>::v, opNum, x, X_INFO, extraParams,               \
                                                 biasCorrected ? 1 : 0, &out), "execSummaryStatsScalar" #S);           \
        return (R) out;                                                                                                \
    }                                                                                                                  \
    void NativeOps::execSummaryStats##S(Nd4jPointer *extraPointers, int opNum, T *x, Nd4jLong *xShapeInfo,            \
                                        T *extraParams, T *result, Nd4jLong *resultShapeInfo, bool biasCorrected) {   \
        check(nd4jb200_exec_summary_stats(STREAM, TypeCode<T>::v, opNum, x, X_INFO, extraParams, result,              \
                                          Z_INFO(resultShapeInfo), nullptr, 0, biasCorrected ? 1 : 0),                \
              "execSummaryStats" #S);                                                                                  \
    }                                                                                                                  \
    void NativeOps::execSummaryStats##S(Nd4jPointer *extraPointers, int opNum, T *x, Nd4jLong *xShapeInfo,            \
                                        T *extraParams, T *result, Nd4jLong *resultShapeInfoBuffer, int *dimension,   \
                                        int dimensionLength, bool biasCorrected) {                                    \
        const HostDims dims = DIMS;                                                                                    \
        check(nd4jb200_exec_summary_stats(STREAM, TypeCode<T>::v, opNum, x, X_INFO, extraParams, result,              \
                                          Z_INFO(resultShapeInfoBuffer), dims.p,       \
                                          dims.n, biasCorrected ? 1 : 0), "execSummaryStats" #S);             \
    }                                                                                                                  \
    void NativeOps::execTransform##S(Nd4jPointer *extraPointers, int opNum, T *dx, Nd4jLong xStride, T *result,       \
                                     Nd4jLong resultStride, T *extraParams, Nd4jLong n) {                             \
        check(nd4jb200_exec_transform_strided(STREAM, TypeCode<T>::v, opNum, dx, xStride, result, resultStride,       \
                                              extraParams, n), "execTransform" #S);                                    \
    }                                                                                                                  \
    void NativeOps::execTransform##S(Nd4jPointer *extraPointers, int opNum, T *dx, Nd4jLong *xShapeInfo, T *result,   \
                                     Nd4jLong *resultShapeInfo, T *extraParams) {                                     \
        check(nd4jb200_exec_transform(STREAM, TypeCode<T>::v, opNum, dx, X_INFO, result, Z_INFO(resultShapeInfo),     \
                                      extraParams), "execTransform" #S);                                               \
    }                                                                                                                  \
    void NativeOps::execRandom##S(Nd4jPointer *extraPointers, int opNum, Nd4jPointer state, T *z,                     \
                                  Nd4jLong *zShapeBuffer, T *extraArguments) {                                        \
        check(nd4jb200_exec_random(STREAM, TypeCode<T>::v, opNum, state, z, host_info(extraPointers, 0, zShapeBuffer),\
                                   extraArguments), "execRandom" #S);                                                  \
    }                                                                                                                  \
    void NativeOps::execRandom##S(Nd4jPointer *extraPointers, int opNum, Nd4jPointer state, T *x,                     \
                                  Nd4jLong *xShapeBuffer, T *y, Nd4jLong *yShapeBuffer, T *z,                         \
                                  Nd4jLong *zShapeBuffer, T *extraArguments) {                                        \
        check(nd4jb200_exec_random_xy(STREAM, TypeCode<T>::v, opNum, state, x, host_info(nullptr, -1, xShapeBuffer),  \
                                      y, host_info(nullptr, -1, yShapeBuffer), z,                                     \
                                      host_info(nullptr, -1, zShapeBuffer), extraArguments), "execRandom" #S);         \
    }                                                                                                                  \
    void NativeOps::execRandom##S(Nd4jPointer *extraPointers, int opNum, Nd4jPointer state, T *x,                     \
                                  Nd4jLong *xShapeBuffer, T *z, Nd4jLong *zShapeBuffer, T *extraArguments) {          \
        check(nd4jb200_exec_random_x(STREAM, TypeCode<T>::v, opNum, state, x, host_info(nullptr, -1, xShapeBuffer),   \
                                     z, host_info(nullptr, -1, zShapeBuffer), extraArguments), "execRandom" #S);       \
    }

ND4JB200_DEFINE_FAMILIES(double, Double, double)
ND4JB200_DEFINE_FAMILIES(float, Float, float)
ND4JB200_DEFINE_FAMILIES(float16, Half, float)

#define ND4JB200_DEFINE_SCALAR(T, S, ST)                                                                               \
    void NativeOps::execScalar##S(Nd4jPointer *extraPointers, int opNum, T *x, Nd4jLong xStride, T *result,           \
                                  Nd4jLong resultStride, ST scalar, T *extraParams, Nd4jLong n) {                     \
        check(nd4jb200_exec_scalar_strided(STREAM, TypeCode<T>::v, opNum, x, xStride, result, resultStride,           \
                                           (double) scalar, extraParams, n), "execScalar" #S);                         \
    }                                                                                                                  \
    void NativeOps::execScalar##S(Nd4jPointer *extraPointers, int opNum, T *x, Nd4jLong *xShapeInfo, T *result,       \
                                  Nd4jLong *resultShapeInfo, ST scalar, T *extraParams) {                             \
        check(nd4jb200_exec_scalar(STREAM, TypeCode<T>::v, opNum, x, X_INFO, result, Z_INFO(resultShapeInfo),         \
                                   (double) scalar, extraParams), "execScalar" #S);                                    \
    }
ND4JB200_DEFINE_SCALAR(double, Double, double)
ND4JB200_DEFINE_SCALAR(float, Float, float)
ND4JB200_DEFINE_SCALAR(float16, Half, float)

void NativeOps::execScalarFloat(Nd4jPointer *extraPointers, int opNum, float *x, Nd4jLong *xShapeInfo, float *result,
                                Nd4jLong *, float scalar, float *extraParams, Nd4jLong *xIndexes, Nd4jLong *resultIndexes) {
    check(nd4jb200_exec_scalar_indexed(STREAM, ND4JB200_FLOAT, opNum, x, X_INFO, result, (double) scalar, extraParams,
                                       xIndexes, resultIndexes), "execScalarFloat");
}
void NativeOps::execScalarDouble(Nd4jPointer *extraPointers, int opNum, double *x, Nd4jLong *xShapeInfo, double *result,
                                 Nd4jLong *, double scalar, double *extraParams, Nd4jLong, Nd4jLong *xIndexes,
                                 Nd4jLong *resultIndexes) {
    // the element count is that of xShapeInfo, as for the Float member
    check(nd4jb200_exec_scalar_indexed(STREAM, ND4JB200_DOUBLE, opNum, x, X_INFO, result, scalar, extraParams, xIndexes,
                                       resultIndexes), "execScalarDouble");
}
void NativeOps::execTransformDouble(Nd4jPointer *, int, double *, Nd4jLong *, double *, Nd4jLong *, double *, Nd4jLong *,
                                    Nd4jLong *) {}
void NativeOps::execTransformFloat(Nd4jPointer *, int, float *, Nd4jLong *, float *, Nd4jLong *, float *, Nd4jLong *,
                                   Nd4jLong *) {}
void NativeOps::execTransformHalf(Nd4jPointer *, int, float16 *, Nd4jLong *, float16 *, Nd4jLong *, float16 *, Nd4jLong *,
                                  Nd4jLong *) {}

#define ND4JB200_DEFINE_META(T, S, ST)                                                                                 \
    void NativeOps::execMetaPredicateStrided##S(Nd4jPointer *extraPointers, const int opTypeA, const int opNumA,      \
                                                const int opTypeB, const int opNumB, Nd4jLong N, T *dx,               \
                                                Nd4jLong xStride, T *dy, Nd4jLong yStride, T *dz, Nd4jLong zStride,   \
                                                T *extraA, T *extraB, ST scalarA, ST scalarB) {                       \
        check(nd4jb200_exec_meta_predicate_strided(STREAM, TypeCode<T>::v, opTypeA, opNumA, opTypeB, opNumB, N, dx,   \
                                                   xStride, dy, yStride, dz, zStride, extraA, extraB,                 \
                                                   (double) scalarA, (double) scalarB), "execMetaPredicateStrided" #S); \
    }                                                                                                                  \
    void NativeOps::execMetaPredicateShape##S(Nd4jPointer *extraPointers, const int opTypeA, const int opNumA,        \
                                              const int opTypeB, const int opNumB, Nd4jLong, T *dx,                   \
                                              Nd4jLong *xShapeInfo, T *dy, Nd4jLong *yShapeInfo, T *dz,               \
                                              Nd4jLong *zShapeInfo, T *extraA, T *extraB, ST scalarA, ST scalarB) {   \
        check(nd4jb200_exec_meta_predicate_shape(STREAM, TypeCode<T>::v, opTypeA, opNumA, opTypeB, opNumB, dx,        \
                                                 X_INFO, dy, Y_INFO, dz, Z_INFO(zShapeInfo), extraA, extraB,          \
                                                 (double) scalarA, (double) scalarB), "execMetaPredicateShape" #S);    \
    }
ND4JB200_DEFINE_META(float, Float, float)
ND4JB200_DEFINE_META(double, Double, double)
ND4JB200_DEFINE_META(float16, Half, float)
void NativeOps::execMetaPredicateReduceFloat(Nd4jPointer *, const int, const int, const int, const int, float *, Nd4jLong *,
                                             float *, Nd4jLong *, float *, Nd4jLong *, int *, int, Nd4jLong *, Nd4jLong *,
                                             float *, float *, float, float, bool) {}

void NativeOps::sortCooIndicesFloat(Nd4jPointer *, Nd4jLong *, float *, Nd4jLong, int) { throw std::runtime_error("Not implemented yet"); }
void NativeOps::sortCooIndicesDouble(Nd4jPointer *, Nd4jLong *, double *, Nd4jLong, int) { throw std::runtime_error("Not implemented yet"); }
void NativeOps::sortCooIndicesHalf(Nd4jPointer *, Nd4jLong *, float16 *, Nd4jLong, int) { throw std::runtime_error("Not implemented yet"); }

void NativeOps::convertTypes(Nd4jPointer *extras, int srcType, Nd4jPointer x, Nd4jLong N, int dstType, Nd4jPointer z) {
    check(nd4jb200_convert_types(stream_of(extras), srcType, x, N, dstType, z), "convertTypes");
}

Nd4jPointer NativeOps::initRandom(Nd4jPointer *extraPointers, long seed, long bufferSize, Nd4jPointer ptrToBuffer) {
    Nd4jPointer state = nd4jb200_init_random(stream_of(extraPointers), seed, bufferSize,
                                             extraPointers ? extraPointers[0] : nullptr, ptrToBuffer);
    if (!state) fail("initRandom");
    return state;
}
void NativeOps::refreshBuffer(Nd4jPointer *extraPointers, long seed, Nd4jPointer ptrRandom) {
    check(nd4jb200_refresh_buffer(stream_of(extraPointers), seed, ptrRandom), "refreshBuffer");
}
void NativeOps::reSeedBuffer(Nd4jPointer *extraPointers, long seed, Nd4jPointer ptrRandom) {
    check(nd4jb200_reseed_buffer(seed, ptrRandom), "reSeedBuffer");
}
void NativeOps::destroyRandom(Nd4jPointer ptrRandom) { nd4jb200_destroy_random(ptrRandom); }

void NativeOps::tadOnlyShapeInfo(Nd4jLong *xShapeInfo, int *dimension, int dimensionLength, Nd4jLong *targetBuffer,
                                 Nd4jLong *offsetsBuffer) {
    check(nd4jb200_tad_only_shape_info(xShapeInfo, dimension, dimensionLength, targetBuffer, offsetsBuffer),
          "tadOnlyShapeInfo");
}

static int device_of(Nd4jPointer p) { return (int) (Nd4jLong) p; }

void NativeOps::initializeDevicesAndFunctions() {}
Nd4jPointer NativeOps::mallocHost(Nd4jLong memorySize, int) { return nd4jb200_malloc_host(memorySize); }
Nd4jPointer NativeOps::mallocDevice(Nd4jLong memorySize, Nd4jPointer, int) { return nd4jb200_malloc_device(memorySize); }
int NativeOps::freeHost(Nd4jPointer pointer) { return nd4jb200_free_host(pointer) == 0 ? 1 : 0; }
int NativeOps::freeDevice(Nd4jPointer pointer, Nd4jPointer) { return nd4jb200_free_device(pointer) == 0 ? 1 : 0; }
Nd4jPointer NativeOps::createContext() { return nullptr; }
Nd4jPointer NativeOps::createStream() {
    Nd4jPointer s = nd4jb200_create_stream();
    if (!s) fail("createStream");
    return s;
}
Nd4jPointer NativeOps::createEvent() {
    Nd4jPointer e = nd4jb200_create_event();
    if (!e) fail("createEvent");
    return e;
}
int NativeOps::registerEvent(Nd4jPointer event, Nd4jPointer stream) { check(nd4jb200_register_event(event, stream), "registerEvent"); return 1; }
int NativeOps::destroyEvent(Nd4jPointer event) { check(nd4jb200_destroy_event(event), "destroyEvent"); return 1; }
int NativeOps::setDevice(Nd4jPointer ptrToDeviceId) { check(nd4jb200_set_device(device_of(ptrToDeviceId)), "setDevice"); return 1; }
int NativeOps::getDevice() { return nd4jb200_get_device(); }
int NativeOps::streamSynchronize(Nd4jPointer stream) { check(nd4jb200_stream_synchronize(stream), "streamSynchronize"); return 1; }
int NativeOps::eventSynchronize(Nd4jPointer event) { check(nd4jb200_event_synchronize(event), "eventSynchronize"); return 1; }
Nd4jLong NativeOps::getDeviceFreeMemory(Nd4jPointer p) { return nd4jb200_device_free_memory(device_of(p)); }
Nd4jLong NativeOps::getDeviceTotalMemory(Nd4jPointer p) { return nd4jb200_device_total_memory(device_of(p)); }
int NativeOps::getDeviceMajor(Nd4jPointer p) { return nd4jb200_device_major(device_of(p)); }
int NativeOps::getDeviceMinor(Nd4jPointer p) { return nd4jb200_device_minor(device_of(p)); }
const char *NativeOps::getDeviceName(Nd4jPointer p) { return nd4jb200_device_name(device_of(p)); }
int NativeOps::memcpy(Nd4jPointer dst, Nd4jPointer src, Nd4jLong size, int flags, Nd4jPointer) {
    check(nd4jb200_memcpy(dst, src, size, flags), "memcpy"); return 1;
}
int NativeOps::memcpyAsync(Nd4jPointer dst, Nd4jPointer src, Nd4jLong size, int flags, Nd4jPointer reserved) {
    check(nd4jb200_memcpy_async(dst, src, size, flags, reserved), "memcpyAsync"); return 1;
}
int NativeOps::memset(Nd4jPointer dst, int value, Nd4jLong size, int, Nd4jPointer) {
    check(nd4jb200_memset_async(dst, value, size, nullptr), "memset");
    check(nd4jb200_stream_synchronize(nullptr), "memset");
    return 1;
}
int NativeOps::memsetAsync(Nd4jPointer dst, int value, Nd4jLong size, int, Nd4jPointer reserved) {
    check(nd4jb200_memset_async(dst, value, size, reserved), "memsetAsync"); return 1;
}
int NativeOps::memcpyConstantAsync(Nd4jLong dst, Nd4jPointer src, Nd4jLong size, int flags, Nd4jPointer reserved) {
    check(nd4jb200_memcpy_constant_async(dst, src, size, flags, reserved), "memcpyConstantAsync"); return 1;
}
Nd4jPointer NativeOps::getConstantSpace() {
    Nd4jPointer p = nd4jb200_get_constant_space();
    if (!p) fail("getConstantSpace");
    return p;
}
void NativeOps::enableP2P(bool enable) { check(nd4jb200_enable_p2p(enable ? 1 : 0), "enableP2P"); }
void NativeOps::checkP2P() { check(nd4jb200_check_p2p(), "checkP2P"); }
bool NativeOps::isP2PAvailable() { return nd4jb200_is_p2p_available() != 0; }
int NativeOps::getAvailableDevices() { return nd4jb200_get_available_devices(); }
// The reference's tuning knobs for its own launch heuristics and OpenMP loops have no effect on
// these kernels; they are accepted so that callers need no change.
void NativeOps::enableDebugMode(bool) {}
void NativeOps::enableVerboseMode(bool) {}
void NativeOps::setGridLimit(int) {}
void NativeOps::setElementThreshold(int) {}
void NativeOps::setTADThreshold(int) {}
void NativeOps::setOmpNumThreads(int) {}
void NativeOps::setOmpMinThreads(int) {}
