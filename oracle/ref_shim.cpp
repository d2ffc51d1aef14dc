// TEST INFRASTRUCTURE ONLY -- never linked into or called from the product library.
//
// extern "C" shim over the reference's own CPU implementation (NativeOpExcutioner<T>,
// shape::TAD, nd4j::random::RandomBuffer / Xoroshiro128). It is compiled together with the
// reference's translation units, taken from the reference checkout where they lie, by
// oracle/Makefile into oracle/_ref/libnd4jref.so. The parity tests call these entry points
// through ctypes to obtain the reference's results for the same inputs, and the benchmark's
// CPU arm times them.
//
// Each wrapper forwards to the function that blas/cpu/NativeOps.cpp forwards to (the
// NativeOps::*Half CPU members are empty, blas/cpu/NativeOps.cpp:319-329, so the float16
// entry points here go straight to NativeOpExcutioner<float16>).
#include <cstring>
#include <omp.h>
#include <NativeOpExcutioner.h>
#include <helpers/TAD.h>
#include <helpers/shape.h>
#include <helpers/helper_generator.h>
#include <Environment.h>

#define EACH_TYPE(M) M(float, f32) M(double, f64) M(float16, f16)

extern "C" {

int ref_omp_max_threads() { return omp_get_max_threads(); }
void ref_omp_set_threads(int n) { omp_set_num_threads(n); }

// ---- shape / TAD (blas/cpu/NativeOps.cpp:2022-2032) -------------------------------------
long long ref_tad_num(long long *xShapeInfo, int *dimension, int dimensionLength) {
    shape::TAD tad;
    tad.init(xShapeInfo, dimension, dimensionLength);
    tad.createTadOnlyShapeInfo();
    return tad.numTads;
}
void ref_tadOnlyShapeInfo(long long *xShapeInfo, int *dimension, int dimensionLength,
                          long long *target, long long *offsets) {
    shape::TAD tad;
    tad.init(xShapeInfo, dimension, dimensionLength);
    tad.createTadOnlyShapeInfo();
    tad.createOffsets();
    std::memcpy(target, tad.tadOnlyShapeInfo, shape::shapeInfoByteLength(tad.tadOnlyShapeInfo));
    std::memcpy(offsets, tad.tadOffsets, tad.numTads * sizeof(Nd4jLong));
}
void ref_shapeBuffer(int rank, long long *shape, char order, long long *out) {
    Nd4jLong *b = order == 'f' ? shape::shapeBufferFortran(rank, shape) : shape::shapeBuffer(rank, shape);
    std::memcpy(out, b, shape::shapeInfoByteLength(rank));
    delete[] b;
}
int ref_computeElementWiseStride(int rank, long long *shape, long long *stride, int isFOrder) {
    return shape::computeElementWiseStride(rank, shape, stride, isFOrder);
}
long long ref_getOffset(long long *shapeInfo, long long *coords) {
    return shape::getOffset(0, shape::shapeOf(shapeInfo), shape::stride(shapeInfo), coords, shape::rank(shapeInfo));
}
void ref_ind2subC(long long *shapeInfo, long long index, long long *out) {
    shape::ind2subC(shape::rank(shapeInfo), shape::shapeOf(shapeInfo), index, out);
}
void ref_ind2sub(long long *shapeInfo, long long index, long long *out) {
    shape::ind2sub(shape::rank(shapeInfo), shape::shapeOf(shapeInfo), index, out);
}

// ---- RNG state (blas/cpu/NativeOps.cpp:2877-2906) ---------------------------------------
void *ref_initRandom(long long seed, long long bufferSize, void *ptrToBuffer) {
    auto buffer = new nd4j::random::RandomBuffer(seed, bufferSize, reinterpret_cast<uint64_t *>(ptrToBuffer));
    nd4j::random::Xoroshiro128 generator(buffer);
    generator.refreshBuffer();
    return buffer;
}
void ref_refreshBuffer(long long seed, void *ptrRandom) {
    auto buffer = reinterpret_cast<nd4j::random::RandomBuffer *>(ptrRandom);
    buffer->setSeed(seed);
    buffer->setOffset(0);
    nd4j::random::Xoroshiro128 generator(buffer);
    generator.refreshBuffer();
}
void ref_reSeedBuffer(long long seed, void *ptrRandom) {
    reinterpret_cast<nd4j::random::RandomBuffer *>(ptrRandom)->reSeed(seed);
}
void ref_destroyRandom(void *ptrRandom) {
    delete reinterpret_cast<nd4j::random::RandomBuffer *>(ptrRandom);
}
long long ref_rng_offset(void *p) { return reinterpret_cast<nd4j::random::RandomBuffer *>(p)->getOffset(); }
void ref_rng_set_offset(void *p, long long o) { reinterpret_cast<nd4j::random::RandomBuffer *>(p)->setOffset(o); }
void ref_rng_rewind(void *p, long long n) { reinterpret_cast<nd4j::random::RandomBuffer *>(p)->rewindH(n); }
unsigned long long ref_rng_element(void *p, long long pos) {
    return reinterpret_cast<nd4j::random::RandomBuffer *>(p)->getElement(pos);
}
float ref_rng_relative_f32(void *p, long long pos) {
    return reinterpret_cast<nd4j::random::RandomBuffer *>(p)->relativeT<float>(pos);
}
double ref_rng_relative_f64(void *p, long long pos) {
    return reinterpret_cast<nd4j::random::RandomBuffer *>(p)->relativeT<double>(pos);
}
// The generation counter is private; recover it the way a caller can: it is the 8th 8-byte
// field of the CPU-build object (devHolder,size,buffer,devBuffer,offset,seed,position,generation).
long long ref_rng_generation(void *p) { return reinterpret_cast<long long *>(p)[7]; }

// ---- the exec* families, one set per element type ----------------------------------------
#define DEFINE_FAMILIES(T, S)                                                                                   \
    void ref_execReduce_##S(int op, T *x, long long *xs, T *extra, T *z, long long *zs, int *dim, int dimLen,   \
                            long long *tadShape, long long *tadOffsets) {                                       \
        NativeOpExcutioner<T>::execReduce(op, x, xs, extra, z, zs, dim, dimLen, tadShape, tadOffsets);         \
    }                                                                                                           \
    double ref_execReduceScalar_##S(int op, T *x, long long *xs, T *extra) {                                    \
        return (double) (float) NativeOpExcutioner<T>::execReduceScalar(op, x, xs, extra);                      \
    }                                                                                                           \
    void ref_execReduceScalarOut_##S(int op, T *x, long long *xs, T *extra, T *out) {                           \
        *out = NativeOpExcutioner<T>::execReduceScalar(op, x, xs, extra);                                       \
    }                                                                                                           \
    void ref_execIndexReduce_##S(int op, T *x, long long *xs, T *extra, T *z, long long *zs, int *dim,          \
                                 int dimLen, long long *tadShape, long long *tadOffsets) {                      \
        NativeOpExcutioner<T>::execIndexReduce(op, x, xs, extra, z, zs, dim, dimLen, tadShape, tadOffsets);    \
    }                                                                                                           \
    void ref_execIndexReduceScalarOut_##S(int op, T *x, long long *xs, T *extra, T *out) {                      \
        *out = NativeOpExcutioner<T>::execIndexReduceScalar(op, x, xs, extra);                                  \
    }                                                                                                           \
    void ref_execSummaryStats_##S(int op, T *x, long long *xs, T *extra, T *z, long long *zs, int *dim,         \
                                  int dimLen, int biasCorrected) {                                              \
        NativeOpExcutioner<T>::execSummaryStats(op, x, xs, extra, z, zs, dim, dimLen, biasCorrected != 0);     \
    }                                                                                                           \
    void ref_execSummaryStatsScalarOut_##S(int op, T *x, long long *xs, T *extra, int biasCorrected, T *out) {  \
        *out = NativeOpExcutioner<T>::execSummaryStatsScalar(op, x, xs, extra, biasCorrected != 0);             \
    }                                                                                                           \
    void ref_execReduce3_##S(int op, T *x, long long *xs, T *extra, T *y, long long *ys, T *z, long long *zs,   \
                             int *dim, int dimLen) {                                                            \
        NativeOpExcutioner<T>::execReduce3(op, x, xs, extra, y, ys, z, zs, dim, dimLen);                        \
    }                                                                                                           \
    void ref_execReduce3TAD_##S(int op, T *x, long long *xs, T *extra, T *y, long long *ys, T *z,               \
                                long long *zs, int *dim, int dimLen, long long *tadShape,                       \
                                long long *tadOffsets) {                                                        \
        NativeOpExcutioner<T>::execReduce3TAD(op, x, xs, extra, y, ys, z, zs, dim, dimLen, tadShape,            \
                                              tadOffsets);                                                      \
    }                                                                                                           \
    void ref_execReduce3ScalarOut_##S(int op, T *x, long long *xs, T *extra, T *y, long long *ys, T *out) {     \
        *out = NativeOpExcutioner<T>::execReduce3Scalar(op, x, xs, extra, y, ys);                               \
    }                                                                                                           \
    void ref_execReduce3All_##S(int op, T *x, long long *xs, T *extra, T *y, long long *ys, T *z,               \
                                long long *zs, int *dim, int dimLen, long long *xTadShape, long long *xOffsets, \
                                long long *yTadShape, long long *yOffsets) {                                    \
        NativeOpExcutioner<T>::execReduce3All(op, x, xs, extra, y, ys, z, zs, dim, dimLen, xTadShape, xOffsets, \
                                              yTadShape, yOffsets);                                             \
    }                                                                                                           \
    void ref_execTransform_##S(int op, T *x, long long *xs, T *z, long long *zs, T *extra) {                    \
        NativeOpExcutioner<T>::execTransform(op, x, xs, z, zs, extra, nullptr, nullptr);                        \
    }                                                                                                           \
    void ref_execTransformStrided_##S(int op, T *x, long long xStride, T *z, long long zStride, T *extra,       \
                                      long long n) {                                                            \
        NativeOpExcutioner<T>::execTransform(op, x, xStride, z, zStride, extra, n);                             \
    }                                                                                                           \
    void ref_execPairwise_##S(int op, T *x, long long *xs, T *y, long long *ys, T *z, long long *zs,            \
                              T *extra) {                                                                       \
        NativeOpExcutioner<T>::execPairwiseTransform(op, x, xs, y, ys, z, zs, extra);                           \
    }                                                                                                           \
    void ref_execPairwiseStrided_##S(int op, T *x, long long xStride, T *y, long long yStride, T *z,            \
                                     long long zStride, T *extra, long long n) {                                \
        NativeOpExcutioner<T>::execPairwiseTransform(op, x, xStride, y, yStride, z, zStride, extra, n);         \
    }                                                                                                           \
    void ref_execBroadcast_##S(int op, T *x, long long *xs, T *y, long long *ys, T *z, long long *zs, int *dim, \
                               int dimLen, long long *tadShape, long long *tadOffsets, long long *tadShapeZ,    \
                               long long *tadOffsetsZ) {                                                        \
        NativeOpExcutioner<T>::execBroadcast(op, x, xs, y, ys, z, zs, dim, dimLen, tadShape, tadOffsets,        \
                                             tadShapeZ, tadOffsetsZ);                                           \
    }                                                                                                           \
    void ref_execScalar_##S(int op, T *x, long long *xs, T *z, long long *zs, T *scalar, T *extra) {            \
        NativeOpExcutioner<T>::execScalar(op, x, xs, z, zs, *scalar, extra);                                    \
    }                                                                                                           \
    void ref_execScalarStrided_##S(int op, T *x, long long xStride, T *z, long long zStride, T *scalar,         \
                                   T *extra, long long n) {                                                     \
        NativeOpExcutioner<T>::execScalar(op, x, xStride, z, zStride, *scalar, extra, n);                       \
    }                                                                                                           \
    void ref_execScalarAlongDim_##S(int op, T *x, long long *xs, T *extra, T *z, long long *zs, T *scalars,     \
                                    int *dim, int dimLen, long long *tadShape, long long *tadOffsets,           \
                                    long long *tadShapeZ, long long *tadOffsetsZ) {                             \
        NativeOpExcutioner<T>::execScalar(op, x, xs, extra, z, zs, scalars, dim, dimLen, tadShape, tadOffsets,  \
                                          tadShapeZ, tadOffsetsZ);                                              \
    }                                                                                                           \
    void ref_execRandom_##S(int op, void *state, T *z, long long *zs, T *extra) {                               \
        NativeOpExcutioner<T>::execRandom(op, state, z, zs, extra);                                             \
    }                                                                                                           \
    void ref_execRandomX_##S(int op, void *state, T *x, long long *xs, T *z, long long *zs, T *extra) {         \
        NativeOpExcutioner<T>::execRandom(op, state, x, xs, z, zs, extra);                                      \
    }                                                                                                           \
    void ref_execRandomXY_##S(int op, void *state, T *x, long long *xs, T *y, long long *ys, T *z,              \
                              long long *zs, T *extra) {                                                        \
        NativeOpExcutioner<T>::execRandom(op, state, x, xs, y, ys, z, zs, extra);                               \
    }

EACH_TYPE(DEFINE_FAMILIES)

}  // extern "C"
