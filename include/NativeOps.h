/*
 * The subset of the reference's NativeOps class (blas/NativeOps.h:56) served by this backend,
 * declared with identical member names and parameter types so that the shared library exports
 * the same Itanium-mangled symbols JavaCPP binds in libnd4jcuda (for example
 * _ZN9NativeOps15execReduceFloatEPPviPfPxS2_S2_S3_Pii). Members of the reference class that are
 * not listed here (custom ops, graph execution, aggregates, the threshold / bitmap / float8 codecs, numpy and
 * memory-mapping helpers, specialConcat) are outside this backend.
 *
 * Semantics follow the reference's CUDA build (blas/cuda/NativeOps.cu):
 *   - x / y / z / extraParams / scalars / dimension / *ShapeInfo arguments are DEVICE pointers;
 *   - extraPointers[0], [7], [8] carry HOST copies of the x, y and z shapeInfo, [9] the HOST copy of x's TAD
 *     shapeInfo and [1] the cudaStream_t (stored in the slot itself). With those slots filled no call reads
 *     metadata from the device: the dimension list is recovered from [0] and [9]. When a slot is absent the
 *     descriptor (or the dimension array) is read back with a blocking copy on every call and never cached,
 *     because descriptor and dimension buffers get reused with other contents;
 *   - calls are asynchronous on that stream; the *Scalar* members synchronise it and return the
 *     value; failures throw std::runtime_error carrying nd4jb200_last_error().
 * Each member forwards to the C entry point of include/nd4j_b200.h named in its comment.
 */
#ifndef ND4J_B200_NATIVEOPS_H
#define ND4J_B200_NATIVEOPS_H

#include "nd4j_b200.h"

/* 16-bit IEEE half, layout-compatible with the reference's float16 (include/types/float16.h:201). */
struct float16 {
    unsigned short bits;
};

#define ND4JB200_EXPORT __attribute__((visibility("default")))

#define ND4JB200_DECLARE_FAMILIES(T, S, R)                                                                          \
    /* nd4jb200_exec_index_reduce_scalar / nd4jb200_exec_index_reduce (NativeOps.h:544-602) */                      \
    R execIndexReduceScalar##S(Nd4jPointer *extraPointers, int opNum, T *x, Nd4jLong *xShapeInfo, T *extraParams);  \
    void execIndexReduce##S(Nd4jPointer *extraPointers, int opNum, T *x, Nd4jLong *xShapeInfo, T *extraParams,      \
                            T *result, Nd4jLong *resultShapeInfoBuffer, int *dimension, int dimensionLength);       \
    /* nd4jb200_exec_broadcast (NativeOps.h:615-649) */                                                             \
    void execBroadcast##S(Nd4jPointer *extraPointers, int opNum, T *x, Nd4jLong *xShapeInfo, T *y,                  \
                          Nd4jLong *yShapeInfo, T *result, Nd4jLong *resultShapeInfo, int *dimension,               \
                          int dimensionLength);                                                                     \
    /* nd4jb200_exec_pairwise_strided / nd4jb200_exec_pairwise (NativeOps.h:665-798) */                             \
    void execPairwiseTransform##S(Nd4jPointer *extraPointers, int opNum, T *dx, Nd4jLong xStride, T *y,             \
                                  Nd4jLong yStride, T *result, Nd4jLong resultStride, T *extraParams, Nd4jLong n);  \
    void execPairwiseTransform##S(Nd4jPointer *extraPointers, int opNum, T *dx, Nd4jLong *xShapeInfo, T *y,         \
                                  Nd4jLong *yShapeInfo, T *result, Nd4jLong *resultShapeInfo, T *extraParams);      \
    /* nd4jb200_exec_pairwise_indexed (NativeOps.h:167-178, 715-754): index arrays live on the device */          \
    void execPairwiseTransform##S(Nd4jPointer *extraPointers, int opNum, T *dx, Nd4jLong *xShapeInfo, T *y,         \
                                  Nd4jLong *yShapeInfo, T *result, Nd4jLong *resultShapeInfo, T *extraParams,       \
                                  Nd4jLong *xIndexes, Nd4jLong *yIndexes, Nd4jLong *resultIndexes);                 \
    /* nd4jb200_exec_reduce / nd4jb200_exec_reduce_scalar (NativeOps.h:809-906) */                                  \
    void execReduce##S(Nd4jPointer *extraPointers, int opNum, T *x, Nd4jLong *xShapeInfo, T *extraParams,           \
                       T *result, Nd4jLong *resultShapeInfo);                                                       \
    void execReduce##S(Nd4jPointer *extraPointers, int opNum, T *x, Nd4jLong *xShapeInfo, T *extraParams,           \
                       T *result, Nd4jLong *resultShapeInfo, int *dimension, int dimensionLength);                  \
    R execReduceScalar##S(Nd4jPointer *extraPointers, int opNum, T *x, Nd4jLong *xShapeInfo, T *extraParams);       \
    /* nd4jb200_exec_reduce3 / nd4jb200_exec_reduce3_scalar (NativeOps.h:918-1034) */                               \
    void execReduce3##S(Nd4jPointer *extraPointers, int opNum, T *x, Nd4jLong *xShapeInfo, T *extraParamsVals,      \
                        T *y, Nd4jLong *yShapeInfo, T *result, Nd4jLong *resultShapeInfo);                          \
    R execReduce3Scalar##S(Nd4jPointer *extraPointers, int opNum, T *x, Nd4jLong *xShapeInfo, T *extraParamsVals,   \
                           T *y, Nd4jLong *yShapeInfo);                                                             \
    void execReduce3##S(Nd4jPointer *extraPointers, int opNum, T *x, Nd4jLong *xShapeInfo, T *extraParamsVals,      \
                        T *y, Nd4jLong *yShapeInfo, T *result, Nd4jLong *resultShapeInfoBuffer, int *dimension,     \
                        int dimensionLength);                                                                       \
    /* nd4jb200_exec_reduce3_all (NativeOps.h:314-360); the TAD descriptors are not needed */                       \
    void execReduce3All##S(Nd4jPointer *extraPointers, int opNum, T *x, Nd4jLong *xInfo, T *extraParamsVals,        \
                           T *y, Nd4jLong *yInfo, T *result, Nd4jLong *resultShapeInfoBuffer, int *dimension,       \
                           int dimensionLength, Nd4jLong *xTadShapeInfo, Nd4jLong *xOffsets,                        \
                           Nd4jLong *yTadShapeInfo, Nd4jLong *yOffsets);                                            \
    /* nd4jb200_flatten / _concat / _pull_rows / _average / _accumulate (NativeOps.h:1457-1601, 1904-2037) */      \
    void flatten##S(Nd4jPointer *extraPointers, int offset, char order, T *result, Nd4jLong *resultShapeInfo,       \
                    T *input, Nd4jLong *inputShapeInfo);                                                            \
    void concat##S(Nd4jPointer *extraPointers, int dimension, int numArrays, Nd4jPointer *data,                     \
                   Nd4jPointer *inputShapeInfo, T *result, Nd4jLong *resultShapeInfo, Nd4jPointer *tadPointers,     \
                   Nd4jPointer *offsetPointers);                                                                    \
    void pullRows##S(Nd4jPointer *extraPointers, T *x, Nd4jLong *xShapeInfo, T *z, Nd4jLong *zShapeInfo,            \
                     Nd4jLong n, Nd4jLong *indexes, Nd4jLong *tadShapeInfo, Nd4jLong *tadOffsets,                   \
                     Nd4jLong *zTadShapeInfo, Nd4jLong *zTadOffsets);                                               \
    /* nd4jb200_tear / nd4jb200_shuffle (NativeOps.h:2076-2129, 2876-2899); pointer arrays are host arrays */       \
    void tear##S(Nd4jPointer *extraPointers, T *x, Nd4jLong *xShapeInfo, Nd4jPointer *targets,                      \
                 Nd4jLong *zShapeInfo, Nd4jLong *tadShapeInfo, Nd4jLong *tadOffsets);                               \
    void shuffle##S(Nd4jPointer *extras, Nd4jPointer *dx, Nd4jPointer *xShapeInfo, Nd4jPointer *dz,                 \
                    Nd4jPointer *zShapeInfo, int N, int *shuffleMap, Nd4jPointer *tadShapeInfo,                     \
                    Nd4jPointer *tadOffsets);                                                                       \
    /* nd4jb200_sort / nd4jb200_sort_tad (NativeOps.h:2940-2952) */                                                 \
    void sort##S(Nd4jPointer *extraPointers, T *x, Nd4jLong *xShapeInfo, bool descending);                          \
    void sortTad##S(Nd4jPointer *extraPointers, T *x, Nd4jLong *xShapeInfo, int *dimension, int dimensionLength,    \
                    Nd4jLong *tadShapeInfo, Nd4jLong *tadOffsets, bool descending);                                 \
    void average##S(Nd4jPointer *extras, Nd4jPointer *dx, T *dz, int n, Nd4jLong length, bool propagate);           \
    void accumulate##S(Nd4jPointer *extras, Nd4jPointer *dx, T *dz, int n, Nd4jLong length);                        \
    /* nd4jb200_exec_scalar_along_dimension (NativeOps.h:1160-1214) */                                              \
    void execScalar##S(Nd4jPointer *extraPointers, int opNum, T *x, Nd4jLong *xShapeInfo, T *z,                     \
                       Nd4jLong *zShapeInfo, T *scalars, T *extraParams, int *dimension, int dimensionLength);      \
    /* nd4jb200_exec_summary_stats_scalar / nd4jb200_exec_summary_stats (NativeOps.h:1223-1325) */                  \
    R execSummaryStatsScalar##S(Nd4jPointer *extraPointers, int opNum, T *x, Nd4jLong *xShapeInfo, T *extraParams,  \
                                bool biasCorrected);                                                                \
    void execSummaryStats##S(Nd4jPointer *extraPointers, int opNum, T *x, Nd4jLong *xShapeInfo, T *extraParams,     \
                             T *result, Nd4jLong *resultShapeInfo, bool biasCorrected);                             \
    void execSummaryStats##S(Nd4jPointer *extraPointers, int opNum, T *x, Nd4jLong *xShapeInfo, T *extraParams,     \
                             T *result, Nd4jLong *resultShapeInfoBuffer, int *dimension, int dimensionLength,       \
                             bool biasCorrected);                                                                   \
    /* nd4jb200_exec_transform_strided / nd4jb200_exec_transform (NativeOps.h:1337-1443) */                         \
    void execTransform##S(Nd4jPointer *extraPointers, int opNum, T *dx, Nd4jLong xStride, T *result,                \
                          Nd4jLong resultStride, T *extraParams, Nd4jLong n);                                       \
    void execTransform##S(Nd4jPointer *extraPointers, int opNum, T *dx, Nd4jLong *xShapeInfo, T *result,            \
                          Nd4jLong *resultShapeInfo, T *extraParams);                                               \
    /* nd4jb200_exec_random / _x / _xy (NativeOps.h:2327-2505) */                                                   \
    void execRandom##S(Nd4jPointer *extraPointers, int opNum, Nd4jPointer state, T *z, Nd4jLong *zShapeBuffer,      \
                       T *extraArguments);                                                                          \
    void execRandom##S(Nd4jPointer *extraPointers, int opNum, Nd4jPointer state, T *x, Nd4jLong *xShapeBuffer,      \
                       T *y, Nd4jLong *yShapeBuffer, T *z, Nd4jLong *zShapeBuffer, T *extraArguments);              \
    void execRandom##S(Nd4jPointer *extraPointers, int opNum, Nd4jPointer state, T *x, Nd4jLong *xShapeBuffer,      \
                       T *z, Nd4jLong *zShapeBuffer, T *extraArguments);

class ND4JB200_EXPORT NativeOps {
public:
    ND4JB200_DECLARE_FAMILIES(double, Double, double)
    ND4JB200_DECLARE_FAMILIES(float, Float, float)
    ND4JB200_DECLARE_FAMILIES(float16, Half, float)

    /* nd4jb200_exec_scalar_strided / nd4jb200_exec_scalar (NativeOps.h:1046-1150): the scalar
     * travels by value, as double / float / float respectively */
    void execScalarDouble(Nd4jPointer *extraPointers, int opNum, double *x, Nd4jLong xStride, double *result,
                          Nd4jLong resultStride, double scalar, double *extraParams, Nd4jLong n);
    void execScalarDouble(Nd4jPointer *extraPointers, int opNum, double *x, Nd4jLong *xShapeInfo, double *result,
                          Nd4jLong *resultShapeInfo, double scalar, double *extraParams);
    void execScalarFloat(Nd4jPointer *extraPointers, int opNum, float *x, Nd4jLong xStride, float *result,
                         Nd4jLong resultStride, float scalar, float *extraParams, Nd4jLong n);
    void execScalarFloat(Nd4jPointer *extraPointers, int opNum, float *x, Nd4jLong *xShapeInfo, float *result,
                         Nd4jLong *resultShapeInfo, float scalar, float *extraParams);
    void execScalarHalf(Nd4jPointer *extraPointers, int opNum, float16 *x, Nd4jLong xStride, float16 *result,
                        Nd4jLong resultStride, float scalar, float16 *extraParams, Nd4jLong n);
    void execScalarHalf(Nd4jPointer *extraPointers, int opNum, float16 *x, Nd4jLong *xShapeInfo, float16 *result,
                        Nd4jLong *resultShapeInfo, float scalar, float16 *extraParams);
    /* nd4jb200_exec_scalar_indexed (NativeOps.h:420-430, 1132-1141): the Double member carries an element count,
     * the Float member does not, and the reference declares none for Half */
    void execScalarDouble(Nd4jPointer *extraPointers, int opNum, double *x, Nd4jLong *xShapeInfo, double *result,
                          Nd4jLong *resultShapeInfo, double scalar, double *extraParams, Nd4jLong n,
                          Nd4jLong *xIndexes, Nd4jLong *resultIndexes);
    void execScalarFloat(Nd4jPointer *extraPointers, int opNum, float *x, Nd4jLong *xShapeInfo, float *result,
                         Nd4jLong *resultShapeInfo, float scalar, float *extraParams, Nd4jLong *xIndexes,
                         Nd4jLong *resultIndexes);
    /* the indexed transform members (NativeOps.h:327-360, 1400-1443) do nothing in the reference, in its CUDA build
     * (blas/cuda/NativeOps.cu:3598-3624) as in its CPU build (the call is commented out,
     * blas/cpu/NativeOpExcutioner.cpp:345-346); they are exported with the same empty behaviour */
    void execTransformDouble(Nd4jPointer *extraPointers, int opNum, double *dx, Nd4jLong *xShapeInfo, double *result,
                             Nd4jLong *resultShapeInfo, double *extraParams, Nd4jLong *xIndexes,
                             Nd4jLong *resultIndexes);
    void execTransformFloat(Nd4jPointer *extraPointers, int opNum, float *dx, Nd4jLong *xShapeInfo, float *result,
                            Nd4jLong *resultShapeInfo, float *extraParams, Nd4jLong *xIndexes,
                            Nd4jLong *resultIndexes);
    void execTransformHalf(Nd4jPointer *extraPointers, int opNum, float16 *dx, Nd4jLong *xShapeInfo, float16 *result,
                           Nd4jLong *resultShapeInfo, float16 *extraParams, Nd4jLong *xIndexes,
                           Nd4jLong *resultIndexes);

    /* nd4jb200_exec_meta_predicate_strided / _shape (NativeOps.h:2564-2759): pairwise opNumA (opTypeA 2) followed by
     * scalar opNumB (opTypeB 0) in one launch; shapeInfo arguments are device pointers with host copies in
     * extraPointers[0], [7], [8] like everywhere else */
#define ND4JB200_DECLARE_META(T, S, ST)                                                                             \
    void execMetaPredicateStrided##S(Nd4jPointer *extras, const int opTypeA, const int opNumA, const int opTypeB,    \
                                     const int opNumB, Nd4jLong N, T *dx, Nd4jLong xStride, T *dy, Nd4jLong yStride, \
                                     T *dz, Nd4jLong zStride, T *extraA, T *extraB, ST scalarA, ST scalarB);         \
    void execMetaPredicateShape##S(Nd4jPointer *extras, const int opTypeA, const int opNumA, const int opTypeB,      \
                                   const int opNumB, Nd4jLong N, T *dx, Nd4jLong *xShapeInfo, T *dy,                 \
                                   Nd4jLong *yShapeInfo, T *dz, Nd4jLong *zShapeInfo, T *extraA, T *extraB,          \
                                   ST scalarA, ST scalarB);
    ND4JB200_DECLARE_META(float, Float, float)
    ND4JB200_DECLARE_META(double, Double, double)
    ND4JB200_DECLARE_META(float16, Half, float)
    /* does nothing in the reference either (blas/cuda/NativeOps.cu:5065-5078, blas/cpu/NativeOps.cpp:2393-2417) */
    void execMetaPredicateReduceFloat(Nd4jPointer *extras, const int opTypeA, const int opNumA, const int opTypeB,
                                      const int opNumB, float *dx, Nd4jLong *xShapeInfo, float *dy, Nd4jLong *yShapeInfo,
                                      float *dz, Nd4jLong *zShapeInfo, int *dimension, int dimensionLength,
                                      Nd4jLong *tadShapeInfo, Nd4jLong *tadOffsets, float *extraA, float *extraB,
                                      float scalarA, float scalarB, bool scalarReturned);

    /* The reference's CUDA build throws "Not implemented yet" from these three (blas/cuda/NativeOps.cu:6072-6082) and
     * its CPU build does not leave the coordinates sorted (include/ops/impl/specials_sparse.cpp:82-113 compares
     * against a pivot position that its own partition loop moves); they are exported with the CUDA build's behaviour. */
    void sortCooIndicesFloat(Nd4jPointer *extraPointers, Nd4jLong *indices, float *values, Nd4jLong length, int rank);
    void sortCooIndicesDouble(Nd4jPointer *extraPointers, Nd4jLong *indices, double *values, Nd4jLong length, int rank);
    void sortCooIndicesHalf(Nd4jPointer *extraPointers, Nd4jLong *indices, float16 *values, Nd4jLong length, int rank);

    /* nd4jb200_init_random and friends (NativeOps.h:2510-2539). extraPointers[0] = host table,
     * [1] = stream, ptrToBuffer = device table (blas/cuda/NativeOps.cu:5384-5391). */
    Nd4jPointer initRandom(Nd4jPointer *extraPointers, long seed, long bufferSize, Nd4jPointer ptrToBuffer);
    void refreshBuffer(Nd4jPointer *extraPointers, long seed, Nd4jPointer ptrRandom);
    void reSeedBuffer(Nd4jPointer *extraPointers, long seed, Nd4jPointer ptrRandom);
    void destroyRandom(Nd4jPointer ptrRandom);

    /* nd4jb200_tad_only_shape_info (NativeOps.h:1880): host pointers in, host buffers out */
    void tadOnlyShapeInfo(Nd4jLong *xShapeInfo, int *dimension, int dimensionLength, Nd4jLong *targetBuffer,
                          Nd4jLong *offsetsBuffer);

    /* device / memory / stream utilities (NativeOps.h:1607-1870) over the nd4jb200_* helpers.
     * ptrToDeviceId is the device ordinal stored in the pointer (blas/cuda/NativeOps.cu:106-108);
     * `reserved` of memcpyAsync / memsetAsync is the stream (blas/cuda/NativeOps.cu:4263-4264). */
    void initializeDevicesAndFunctions();
    Nd4jPointer mallocHost(Nd4jLong memorySize, int flags);
    Nd4jPointer mallocDevice(Nd4jLong memorySize, Nd4jPointer ptrToDeviceId, int flags);
    int freeHost(Nd4jPointer pointer);
    int freeDevice(Nd4jPointer pointer, Nd4jPointer ptrToDeviceId);
    Nd4jPointer createContext();
    Nd4jPointer createStream();
    Nd4jPointer createEvent();
    int registerEvent(Nd4jPointer event, Nd4jPointer stream);
    int destroyEvent(Nd4jPointer event);
    int setDevice(Nd4jPointer ptrToDeviceId);
    int getDevice();
    int streamSynchronize(Nd4jPointer stream);
    int eventSynchronize(Nd4jPointer event);
    Nd4jLong getDeviceFreeMemory(Nd4jPointer ptrToDeviceId);
    Nd4jLong getDeviceTotalMemory(Nd4jPointer ptrToDeviceId);
    int getDeviceMajor(Nd4jPointer ptrToDeviceId);
    int getDeviceMinor(Nd4jPointer ptrToDeviceId);
    const char *getDeviceName(Nd4jPointer ptrToDeviceId);
    int memcpy(Nd4jPointer dst, Nd4jPointer src, Nd4jLong size, int flags, Nd4jPointer reserved);
    int memcpyAsync(Nd4jPointer dst, Nd4jPointer src, Nd4jLong size, int flags, Nd4jPointer reserved);
    int memset(Nd4jPointer dst, int value, Nd4jLong size, int flags, Nd4jPointer reserved);
    int memsetAsync(Nd4jPointer dst, int value, Nd4jLong size, int flags, Nd4jPointer reserved);
    /* nd4jb200_convert_types (NativeOps.h:2144) */
    void convertTypes(Nd4jPointer *extras, int srcType, Nd4jPointer x, Nd4jLong N, int dstType, Nd4jPointer z);
    /* nd4jb200_memcpy_constant_async / nd4jb200_get_constant_space (NativeOps.h:1836-1846) */
    int memcpyConstantAsync(Nd4jLong dst, Nd4jPointer src, Nd4jLong size, int flags, Nd4jPointer reserved);
    Nd4jPointer getConstantSpace();
    /* nd4jb200_enable_p2p / nd4jb200_check_p2p / nd4jb200_is_p2p_available (NativeOps.h:2047-2058) */
    void enableP2P(bool enable);
    void checkP2P();
    bool isP2PAvailable();
    int getAvailableDevices();
    void enableDebugMode(bool reallyEnable);
    void enableVerboseMode(bool reallyEnable);
    void setGridLimit(int gridSize);
    void setElementThreshold(int num);
    void setTADThreshold(int num);
    void setOmpNumThreads(int threads);
    void setOmpMinThreads(int threads);
};

#endif /* ND4J_B200_NATIVEOPS_H */
