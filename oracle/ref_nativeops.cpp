// TEST INFRASTRUCTURE ONLY -- never linked into or called from the product library.
//
// extern "C" shim over the reference's own CPU `NativeOps` class (blas/cpu/NativeOps.cpp, compiled in
// place by oracle/Makefile with -DLIBND4J_ALL_OPS so that no custom op registers itself at load time).
// It gives the parity tests the reference's results for the memory-movement utilities whose bodies are
// templates private to that translation unit (flattenGeneric :1530, pullRowsGeneric :2045, tearGeneric
// :2119, shuffleGeneric :2266) and for the ones it forwards to nd4j::SpecialMethods<T>
// (include/ops/impl/specials.cpp: concat :17, accumulate :344, average :374, sort :547, sortTad :552)
// and to sparse::SparseUtils<T>::sortCooIndicesGeneric (include/ops/impl/specials_sparse.cpp).
//
// The graph / custom-op members of that translation unit reference symbols of the graph runtime and
// of the declarable ops, which are not built here. The Makefile points every such symbol at
// ref_unreachable() below; none of them is on a path these wrappers call.
#include <cstdio>
#include <cstdlib>
#include <NativeOps.h>

extern "C" {

void ref_unreachable() {
    std::fprintf(stderr, "oracle: a graph / custom-op symbol that is not built into libnd4jref.so was called\n");
    std::abort();
}

void ref_convertTypes(int srcType, void *x, long long n, int dstType, void *z) {
    NativeOps ops;
    ops.convertTypes(nullptr, srcType, x, n, dstType, z);
}

#define DEFINE_UTILITIES(T, S, N)                                                                                \
    void ref_flatten_##S(int offset, char order, T *z, long long *zInfo, T *x, long long *xInfo) {               \
        NativeOps ops;                                                                                            \
        ops.flatten##N(nullptr, offset, order, z, zInfo, x, xInfo);                                               \
    }                                                                                                             \
    void ref_concat_##S(int dimension, int numArrays, void **data, void **infos, T *z, long long *zInfo) {       \
        NativeOps ops;                                                                                            \
        ops.concat##N(nullptr, dimension, numArrays, data, infos, z, zInfo, nullptr, nullptr);                    \
    }                                                                                                             \
    void ref_pullRows_##S(T *x, long long *xInfo, T *z, long long *zInfo, long long n, long long *indexes,       \
                          long long *tadInfo, long long *tadOffsets, long long *zTadInfo,                        \
                          long long *zTadOffsets) {                                                               \
        NativeOps ops;                                                                                            \
        ops.pullRows##N(nullptr, x, xInfo, z, zInfo, n, indexes, tadInfo, tadOffsets, zTadInfo, zTadOffsets);     \
    }                                                                                                             \
    void ref_tear_##S(T *x, long long *xInfo, void **targets, long long *zInfo, long long *tadInfo,              \
                      long long *tadOffsets) {                                                                    \
        NativeOps ops;                                                                                            \
        ops.tear##N(nullptr, x, xInfo, targets, zInfo, tadInfo, tadOffsets);                                      \
    }                                                                                                             \
    void ref_shuffle_##S(void **x, void **xInfos, void **z, void **zInfos, int n, int *shuffleMap,               \
                         void **tadInfos, void **tadOffsets) {                                                    \
        NativeOps ops;                                                                                            \
        ops.shuffle##N(nullptr, x, xInfos, z, zInfos, n, shuffleMap, tadInfos, tadOffsets);                       \
    }                                                                                                             \
    void ref_average_##S(void **x, T *z, int n, long long length, int propagate) {                               \
        NativeOps ops;                                                                                            \
        ops.average##N(nullptr, x, z, n, length, propagate != 0);                                                 \
    }                                                                                                             \
    void ref_accumulate_##S(void **x, T *z, int n, long long length) {                                           \
        NativeOps ops;                                                                                            \
        ops.accumulate##N(nullptr, x, z, n, length);                                                              \
    }                                                                                                             \
    void ref_sort_##S(T *x, long long *xInfo, int descending) {                                                  \
        NativeOps ops;                                                                                            \
        ops.sort##N(nullptr, x, xInfo, descending != 0);                                                          \
    }                                                                                                             \
    void ref_sortTad_##S(T *x, long long *xInfo, int *dimension, int dimensionLength, long long *tadInfo,        \
                         long long *tadOffsets, int descending) {                                                 \
        NativeOps ops;                                                                                            \
        ops.sortTad##N(nullptr, x, xInfo, dimension, dimensionLength, tadInfo, tadOffsets, descending != 0);      \
    }                                                                                                             \
    void ref_sortCooIndices_##S(long long *indices, T *values, long long length, int rank) {                     \
        NativeOps ops;                                                                                            \
        ops.sortCooIndices##N(nullptr, indices, values, length, rank);                                            \
    }

DEFINE_UTILITIES(float, f32, Float)
DEFINE_UTILITIES(double, f64, Double)
// The Half members of the CPU build are empty for flatten, pullRows, average, shuffle, sort and sortTad
// (blas/cpu/NativeOps.cpp:1815, 2106, 2176, 2381, 3009, 3021); the ones with a body:
void ref_concat_f16(int dimension, int numArrays, void **data, void **infos, float16 *z, long long *zInfo) {
    NativeOps ops;
    ops.concatHalf(nullptr, dimension, numArrays, data, infos, z, zInfo, nullptr, nullptr);
}
void ref_tear_f16(float16 *x, long long *xInfo, void **targets, long long *zInfo, long long *tadInfo,
                  long long *tadOffsets) {
    NativeOps ops;
    ops.tearHalf(nullptr, x, xInfo, targets, zInfo, tadInfo, tadOffsets);
}
void ref_accumulate_f16(void **x, float16 *z, int n, long long length) {
    NativeOps ops;
    ops.accumulateHalf(nullptr, x, z, n, length);
}

}  // extern "C"
