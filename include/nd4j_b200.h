/*
 * C ABI of the sm_100a backend for libnd4j's legacy op families.
 *
 * Each entry point replaces one family of member functions of the reference's NativeOps class
 * (blas/NativeOps.h; CUDA implementation blas/cuda/NativeOps.cu). The Float / Double / Half
 * flavours of the reference collapse into one function with a `dtype` argument
 * (ND4JB200_FLOAT / _DOUBLE / _HALF); op numbers are the reference's (include/loops/legacy_ops.h).
 *
 * Conventions, identical for every call:
 *   - x, y, z, scalars, extraParams / extraArguments are DEVICE pointers owned by the caller
 *     (as in the reference's CUDA build). extraParams may be NULL when the op reads none.
 *   - every *ShapeInfo and `dimension` argument is a HOST pointer. The reference's CUDA build
 *     receives the same host copies through extraPointers[0], [7], [8], [9]
 *     (blas/cuda/NativeOps.cu:2107-2118); here they are explicit arguments.
 *   - `stream` is a cudaStream_t (NULL = default stream). Calls are asynchronous on it, except
 *     the *_scalar calls, which synchronise the stream and return the value through `result`,
 *     as the reference's scalar calls do (blas/cuda/NativeOps.cu:2209-2232).
 *   - the return value is 0 on success, otherwise one of the ND4JB200_E* codes;
 *     nd4jb200_last_error() then describes the failure (thread-local string).
 *   - nothing here falls back to the CPU: without a usable GPU every compute call fails with
 *     ND4JB200_ECUDA.
 */
#ifndef ND4J_B200_H
#define ND4J_B200_H

#ifdef __cplusplus
extern "C" {
#endif

typedef long long Nd4jLong;   /* include/pointercast.h:10-12 */
typedef void *Nd4jPointer;

enum { ND4JB200_FLOAT = 0, ND4JB200_DOUBLE = 1, ND4JB200_HALF = 2 };
enum {
    ND4JB200_OK = 0, ND4JB200_EARG = 1, ND4JB200_EOP = 2, ND4JB200_EUNSUPPORTED = 3,
    ND4JB200_ECUDA = 4, ND4JB200_ETOOLARGE = 5
};

const char *nd4jb200_last_error(void);
/* kernels launched by this library since it was loaded */
unsigned long long nd4jb200_launch_count(void);
/* Launch heuristics (no counterpart in the reference). key 0: CTAs per SM the across-TAD reduction
 * kernel aims for when it cuts TADs into segments (default 3); key 1: resident threads per SM the
 * along-TAD reduction kernel aims for (default 1024); key 2: most segments per TAD that are still
 * merged inside the reduction launch instead of by a separate pass (default 32); key 3: 1 (default)
 * launches kernels with programmatic stream serialisation so that a kernel's launch overlaps the
 * tail of the previous kernel on the stream, 0 launches them plainly; key 4: largest thread-block cluster
 * (1, 2, 4 or 8, default 4) the across-TAD reduction uses to merge segments in distributed shared memory.
 * key 5: CTAs per SM the along-TAD reduction launches at most (default 16; 8 for half precision).
 * Results do not
 * depend on these values beyond the summation order of floating-point reductions. */
int nd4jb200_set_tuning(int key, long long value);

/* ---- reduce: NativeOps::execReduce{Float,Double,Half} along dimension
 *      (blas/NativeOps.h:845-876; blas/cuda/NativeOps.cu:2098-2185) ------------------------- */
int nd4jb200_exec_reduce(void *stream, int dtype, int opNum, const void *x, const Nd4jLong *xShapeInfo,
                         const void *extraParams, void *z, const Nd4jLong *zShapeInfo,
                         const int *dimension, int dimensionLength);
/* NativeOps::execReduceScalar* (blas/NativeOps.h:886-906; blas/cuda/NativeOps.cu:2195-2233) */
int nd4jb200_exec_reduce_scalar(void *stream, int dtype, int opNum, const void *x,
                                const Nd4jLong *xShapeInfo, const void *extraParams, double *result);

/* Whole-array reduction that allocates nothing. It has no counterpart in the reference: the
 * reference's CUDA build takes its reduction scratch from the caller (extraPointers[4]), this
 * library normally allocates its own. Callers that cannot allocate on the device - code running
 * inside a pool that owns all device memory, loops that must not trigger a device-wide
 * synchronisation, processes without allocation rights - use this form instead: partial states
 * live in a fixed 64 KiB device array inside the library and the result is written to `z`, a
 * DEVICE location for one element of the call's type (asynchronous on `stream`).
 * Arrays longer than 2^27 elements are refused with ND4JB200_ETOOLARGE. Calls on one device
 * share the array, so calls that overlap on the GPU must be ordered by the caller. The first
 * call on each device looks up the array's address and should precede any stream capture. */
int nd4jb200_exec_reduce_scalar_noalloc(void *stream, int dtype, int opNum, const void *x,
                                        const Nd4jLong *xShapeInfo, const void *extraParams, void *z);

/* ---- indexreduce: NativeOps::execIndexReduce* (blas/NativeOps.h:576-602;
 *      blas/cuda/NativeOps.cu:1699-1781). Indices are written in the element type, as in the
 *      reference (include/loops/cpu/indexreduce.cpp:206,223). ---------------------------------- */
int nd4jb200_exec_index_reduce(void *stream, int dtype, int opNum, const void *x, const Nd4jLong *xShapeInfo,
                               const void *extraParams, void *z, const Nd4jLong *zShapeInfo,
                               const int *dimension, int dimensionLength);
/* NativeOps::execIndexReduceScalar* (blas/NativeOps.h:544-563) */
int nd4jb200_exec_index_reduce_scalar(void *stream, int dtype, int opNum, const void *x,
                                      const Nd4jLong *xShapeInfo, const void *extraParams, double *result);

/* ---- summarystats: NativeOps::execSummaryStats* (blas/NativeOps.h:1291-1325;
 *      blas/cuda/NativeOps.cu:2957-3020) and execSummaryStatsScalar* (:1223-1242) ---------- */
int nd4jb200_exec_summary_stats(void *stream, int dtype, int opNum, const void *x, const Nd4jLong *xShapeInfo,
                                const void *extraParams, void *z, const Nd4jLong *zShapeInfo,
                                const int *dimension, int dimensionLength, int biasCorrected);
int nd4jb200_exec_summary_stats_scalar(void *stream, int dtype, int opNum, const void *x,
                                       const Nd4jLong *xShapeInfo, const void *extraParams,
                                       int biasCorrected, double *result);

/* ---- reduce3: NativeOps::execReduce3* along dimension (blas/NativeOps.h:998-1034;
 *      blas/cuda/NativeOps.cu:2502-2629) and execReduce3Scalar* (blas/NativeOps.h:962-986).
 *      When one operand holds exactly one TAD it is paired with every TAD of the other. ---- */
int nd4jb200_exec_reduce3(void *stream, int dtype, int opNum, const void *x, const Nd4jLong *xShapeInfo,
                          const void *extraParams, const void *y, const Nd4jLong *yShapeInfo,
                          void *z, const Nd4jLong *zShapeInfo, const int *dimension, int dimensionLength);
/* every TAD of x against every TAD of y: z[r * yTads + g]; NativeOps::execReduce3All{Float,Double,Half}
 * (blas/NativeOps.h:314-360; include/loops/reduce3.h:919-990). z must be dense. */
int nd4jb200_exec_reduce3_all(void *stream, int dtype, int opNum, const void *x, const Nd4jLong *xShapeInfo,
                              const void *extraParams, const void *y, const Nd4jLong *yShapeInfo, void *z,
                              const Nd4jLong *zShapeInfo, const int *dimension, int dimensionLength);
int nd4jb200_exec_reduce3_scalar(void *stream, int dtype, int opNum, const void *x, const Nd4jLong *xShapeInfo,
                                 const void *extraParams, const void *y, const Nd4jLong *yShapeInfo,
                                 double *result);

/* ---- transform: NativeOps::execTransform* shaped and strided (blas/NativeOps.h:1337-1443;
 *      blas/cuda/NativeOps.cu:3033-3343) --------------------------------------------------------
 * The shaped call also serves the whole-array ("special") transforms of include/ops/special_ops.h, where x and z
 * may differ in shape: SoftMax 38, SoftMaxDerivative 39, LogSoftMax 40, IsMax 41 and
 *   Col2Im 36    x [b, c, kH, kW, oH, oW] -> z [b, c, h, w]; extraParams {sH, sW, pH, pW, h, w, dH, dW}
 *   Im2col 37    x [b, c, h, w] -> z [b, c, kH, kW, oH, oW]; extraParams {kH, kW, sH, sW, pH, pW, dH, dW, -, padValue}
 *   Histogram 48 x dense -> z [numBins] (added to); extraParams {numBins, min, max}
 *   Reverse 70   z at linear position n - 1 - e = x at linear position e; no extraParams
 *   Pooling2D 71 x [b, c, h, w] -> z [b, c, oH, oW]; extraParams {kH, kW, sH, sW, pH, pW, dH, dW, -, mode, extra0},
 *                mode 0 max, 1 average (extra0 0: divide by the taps inside the image, 1: by kH * kW), 2 p-norm (p = extra0)
 * extraParams is a device pointer to values of the element type, as in the reference. */
int nd4jb200_exec_transform(void *stream, int dtype, int opNum, const void *x, const Nd4jLong *xShapeInfo,
                            void *z, const Nd4jLong *zShapeInfo, const void *extraParams);
int nd4jb200_exec_transform_strided(void *stream, int dtype, int opNum, const void *x, Nd4jLong xStride,
                                    void *z, Nd4jLong zStride, const void *extraParams, Nd4jLong n);

/* ---- pairwise transform: NativeOps::execPairwiseTransform* (blas/NativeOps.h:665-798;
 *      blas/cuda/NativeOps.cu:1883-2005) -------------------------------------------------------- */
int nd4jb200_exec_pairwise(void *stream, int dtype, int opNum, const void *x, const Nd4jLong *xShapeInfo,
                           const void *y, const Nd4jLong *yShapeInfo, void *z, const Nd4jLong *zShapeInfo,
                           const void *extraParams);
/* indexed overloads: z[zIndexes[i]] = op(x[xIndexes[i]], y[yIndexes[i]]) for i < length(x); the index arrays
 * are DEVICE arrays of element offsets (NativeOps::execPairwiseTransform* with xIndexes/yIndexes/resultIndexes,
 * blas/NativeOps.h:167-178, 715-754; include/loops/pairwise_transform.h:136-152) */
int nd4jb200_exec_pairwise_indexed(void *stream, int dtype, int opNum, const void *x, const Nd4jLong *xShapeInfo,
                                   const void *y, void *z, const void *extraParams, const Nd4jLong *xIndexes,
                                   const Nd4jLong *yIndexes, const Nd4jLong *zIndexes);
int nd4jb200_exec_pairwise_strided(void *stream, int dtype, int opNum, const void *x, Nd4jLong xStride,
                                   const void *y, Nd4jLong yStride, void *z, Nd4jLong zStride,
                                   const void *extraParams, Nd4jLong n);

/* ---- broadcast: NativeOps::execBroadcast* (blas/NativeOps.h:615-649;
 *      blas/cuda/NativeOps.cu:1795-1867) -------------------------------------------------------- */
int nd4jb200_exec_broadcast(void *stream, int dtype, int opNum, const void *x, const Nd4jLong *xShapeInfo,
                            const void *y, const Nd4jLong *yShapeInfo, void *z, const Nd4jLong *zShapeInfo,
                            const int *dimension, int dimensionLength);

/* ---- scalar: NativeOps::execScalar* shaped / strided / along dimension
 *      (blas/NativeOps.h:1046-1214; blas/cuda/NativeOps.cu:2642-2816, 5135-5190) ------------ */
int nd4jb200_exec_scalar(void *stream, int dtype, int opNum, const void *x, const Nd4jLong *xShapeInfo,
                         void *z, const Nd4jLong *zShapeInfo, double scalar, const void *extraParams);
/* z[zIndexes[i]] = op(x[xIndexes[i]], scalar) (NativeOps::execScalar* with xIndexes/resultIndexes,
 * blas/NativeOps.h:1132-1141; include/loops/cpu/scalar.cpp:118-131) */
int nd4jb200_exec_scalar_indexed(void *stream, int dtype, int opNum, const void *x, const Nd4jLong *xShapeInfo, void *z,
                                 double scalar, const void *extraParams, const Nd4jLong *xIndexes,
                                 const Nd4jLong *zIndexes);
int nd4jb200_exec_scalar_strided(void *stream, int dtype, int opNum, const void *x, Nd4jLong xStride,
                                 void *z, Nd4jLong zStride, double scalar, const void *extraParams, Nd4jLong n);
int nd4jb200_exec_scalar_along_dimension(void *stream, int dtype, int opNum, const void *x,
                                         const Nd4jLong *xShapeInfo, const void *extraParams, void *z,
                                         const Nd4jLong *zShapeInfo, const void *scalars,
                                         const int *dimension, int dimensionLength);

/* ---- random: NativeOps::initRandom / refreshBuffer / reSeedBuffer / destroyRandom
 *      (blas/NativeOps.h:2510-2539; blas/cuda/NativeOps.cu:5384-5447) and execRandom* in its
 *      three arities (blas/NativeOps.h:2327-2505; blas/cuda/NativeOps.cu:5312-5382).
 *      hostTable / deviceTable may be NULL, in which case the library allocates them. The state
 *      handle is a host object; execRandom advances it by length(z) like RandomBuffer::rewindH
 *      (include/helpers/helper_generator.h:322-334). ------------------------------------------- */
Nd4jPointer nd4jb200_init_random(void *stream, Nd4jLong seed, Nd4jLong bufferSize, void *hostTable,
                                 void *deviceTable);
int nd4jb200_refresh_buffer(void *stream, Nd4jLong seed, Nd4jPointer state);
int nd4jb200_reseed_buffer(Nd4jLong seed, Nd4jPointer state);
int nd4jb200_destroy_random(Nd4jPointer state);
int nd4jb200_exec_random(void *stream, int dtype, int opNum, Nd4jPointer state, void *z,
                         const Nd4jLong *zShapeInfo, const void *extraArguments);
int nd4jb200_exec_random_x(void *stream, int dtype, int opNum, Nd4jPointer state, const void *x,
                           const Nd4jLong *xShapeInfo, void *z, const Nd4jLong *zShapeInfo,
                           const void *extraArguments);
int nd4jb200_exec_random_xy(void *stream, int dtype, int opNum, Nd4jPointer state, const void *x,
                            const Nd4jLong *xShapeInfo, const void *y, const Nd4jLong *yShapeInfo,
                            void *z, const Nd4jLong *zShapeInfo, const void *extraArguments);
/* Offset-sharded generation: produces elements [first, first+count) of a logical call of
 * `length` elements into dense buffers that hold only that range (x, y, z point at the range's
 * first element). The state is NOT advanced; the owner of the logical call advances it once
 * with nd4jb200_rng_rewind(state, length). `first` must be even for the Gaussian family.
 * arity: 0 = z only, 1 = x, 2 = x and y (pass y == z to take the mean from extraArguments[0]). */
int nd4jb200_exec_random_range(void *stream, int dtype, int opNum, int arity, Nd4jPointer state,
                               const void *x, const void *y, void *z, const void *extraArguments,
                               Nd4jLong first, Nd4jLong count, Nd4jLong length);
int nd4jb200_rng_rewind(Nd4jPointer state, Nd4jLong count);
/* words: seed, currentPosition, generation, amplifier, size (RandomBuffer fields,
 * include/helpers/helper_generator.h:64-74) */
int nd4jb200_rng_get_state(Nd4jPointer state, Nd4jLong words[5]);
int nd4jb200_rng_set_state(Nd4jPointer state, const Nd4jLong words[4]);
void *nd4jb200_rng_device_table(Nd4jPointer state);

/* ---- shape helpers: NativeOps::tadOnlyShapeInfo (blas/NativeOps.h:1880;
 *      blas/cuda/NativeOps.cu:4781-4791). target needs 2*rank+4 longs, offsets numTads. ------- */
int nd4jb200_tad_only_shape_info(const Nd4jLong *xShapeInfo, const int *dimension, int dimensionLength,
                                 Nd4jLong *target, Nd4jLong *offsets);
Nd4jLong nd4jb200_tad_count(const Nd4jLong *xShapeInfo, const int *dimension, int dimensionLength);
/* The dimension list that yields the given TADs of x, recovered on the host from the two descriptors (both host
 * pointers): the reference's CUDA callers keep a host copy of the TAD shapeInfo in extraPointers[9]
 * (blas/cuda/NativeOps.cu:2111) while `dimension` itself lives on the device. Returns the number of axes written
 * to `dimension` (room for 32), 0 when the TAD is the whole array, -1 when the descriptors do not determine it. */
/* Diagnostics: how many blocking device-to-host reads of shapeInfo / dimension arrays the NativeOps members
 * (include/NativeOps.h) have made since load because a call came without the host copies the reference's CUDA
 * callers provide in extraPointers[0], [7], [8] and [9]. A caller that fills those slots keeps this at zero. */
unsigned long long nd4jb200_metadata_reads(void);
int nd4jb200_dims_from_tad(const Nd4jLong *xShapeInfo, const Nd4jLong *tadShapeInfo, int *dimension);

/* ---- memory-movement utilities on the same boundary (blas/NativeOps.h:1457-1601, 1904-2037). Pointer
 *      arrays (`sources`, `data`, `inputShapeInfo`) are HOST arrays; what they point to follows the usual
 *      rule (data on the device, shapeInfo on the host). `indexes` and the TAD offset arrays of pullRows are
 *      DEVICE arrays, as in the reference's CUDA build; the TAD shapeInfos are host arrays. ------------------ */
/* NativeOps::flatten{Float,Double,Half}: z[offset + i * zEws] = element i of x walked in `order` ('c' / 'f')
 * (blas/NativeOps.h:1457-1500; blas/cpu/NativeOps.cpp:1530-1700) */
int nd4jb200_flatten(void *stream, int dtype, Nd4jLong offset, char order, void *z, const Nd4jLong *zShapeInfo,
                     const void *x, const Nd4jLong *xShapeInfo);
/* NativeOps::concat{Float,Double,Half}: inputs side by side along `dimension` of z
 * (blas/NativeOps.h:1510-1555; include/ops/impl/specials.cpp concatCpuGeneric) */
int nd4jb200_concat(void *stream, int dtype, int dimension, int numArrays, const void *const *data,
                    const Nd4jLong *const *inputShapeInfo, void *z, const Nd4jLong *zShapeInfo);
/* NativeOps::pullRows{Float,Double,Half}: TAD indexes[k] of x onto TAD k of z
 * (blas/NativeOps.h:1930-1980; blas/cpu/NativeOps.cpp:2045-2104) */
int nd4jb200_pull_rows(void *stream, int dtype, const void *x, void *z, Nd4jLong n, const Nd4jLong *indexes,
                       const Nd4jLong *tadShapeInfo, const Nd4jLong *tadOffsets, const Nd4jLong *zTadShapeInfo,
                       const Nd4jLong *zTadOffsets);
/* NativeOps::tear{Float,Double,Half}: TAD k of x is copied into the array targets[k], all of shape zShapeInfo
 * (blas/NativeOps.h:2876-2899; blas/cpu/NativeOps.cpp:2119-2162). `targets` is a host array of device
 * pointers, `tadOffsets` a device array. */
int nd4jb200_tear(void *stream, int dtype, const void *x, const Nd4jLong *xShapeInfo, void *const *targets,
                  const Nd4jLong *zShapeInfo, const Nd4jLong *tadShapeInfo, const Nd4jLong *tadOffsets);
/* NativeOps::shuffle{Float,Double}: in every array x[f], for r = 0, 1, ... in this order, TAD r changes places
 * with TAD shuffleMap[r] unless shuffleMap[r] < 0 (blas/NativeOps.h:2076-2129; blas/cpu/NativeOps.cpp:2266-2326;
 * the reference's result arrays are not used by it and are not part of this call). `x`, `xShapeInfo`,
 * `tadShapeInfo`, `tadOffsets` and `shuffleMap` are host arrays; tadOffsets[f] is a device array. */
int nd4jb200_shuffle(void *stream, int dtype, int numArrays, void *const *x, const Nd4jLong *const *xShapeInfo,
                     const int *shuffleMap, const Nd4jLong *const *tadShapeInfo, const Nd4jLong *const *tadOffsets);
/* NativeOps::convertTypes among ND4J_INT8 (1), UINT8 (2), FLOAT16 (3), INT16 (4), FLOAT32 (6), DOUBLE (7) and, as a
 * result only, UINT16 (5): z[i] = (D)(float) x[i] with the reference's saturating integer wrappers
 * (blas/NativeOps.h:2144; include/loops/type_conversions.h:592-610, 696-880; include/types/impl/). The pairs its
 * dispatch leaves out (1->1, 6->6, 7->7) leave z untouched. FLOAT8 (0) and THRESHOLD (8): ND4JB200_EUNSUPPORTED. */
int nd4jb200_convert_types(void *stream, int srcType, const void *x, Nd4jLong n, int dstType, void *z);
/* NativeOps::sort{Float,Double,Half}: the whole array sorted in place over its linear positions (i * ews, or c-order
 * coordinates), ascending or descending (blas/NativeOps.h:2940-2944; include/ops/impl/specials.cpp:457-549) */
int nd4jb200_sort(void *stream, int dtype, void *x, const Nd4jLong *xShapeInfo, int descending);
/* NativeOps::sortTad{Float,Double,Half}: every TAD along `dimension` sorted in place
 * (blas/NativeOps.h:2948-2952; include/ops/impl/specials.cpp:551-564). The TAD descriptors are derived from
 * xShapeInfo and the dimension list on the host. */
int nd4jb200_sort_tad(void *stream, int dtype, void *x, const Nd4jLong *xShapeInfo, const int *dimension,
                      int dimensionLength, int descending);
/* NativeOps::average{Float,Double,Half}: z[i] = sum_k sources[k][i] / n (z == NULL: into sources[0]); with
 * `propagate` the result is also written over every source (blas/NativeOps.h:1996-2025;
 * include/ops/impl/specials.cpp:374-433). At most 128 sources, all on this device or peer-mapped. */
int nd4jb200_average(void *stream, int dtype, const void *const *sources, void *z, int n, Nd4jLong length, int propagate);
/* NativeOps::accumulate{Float,Double,Half}: z[i] += sum_k sources[k][i] (blas/NativeOps.h:2027-2037;
 * include/ops/impl/specials.cpp:343-359) */
int nd4jb200_accumulate(void *stream, int dtype, const void *const *sources, void *z, int n, Nd4jLong length);

/* ---- device / memory / stream utilities the same object offers
 *      (blas/NativeOps.h:1607-1870; blas/cuda/NativeOps.cu:3854-4260) ------------------------- */
int nd4jb200_get_available_devices(void);
int nd4jb200_set_device(int device);
int nd4jb200_get_device(void);
Nd4jPointer nd4jb200_malloc_device(Nd4jLong bytes);
int nd4jb200_free_device(Nd4jPointer p);
Nd4jPointer nd4jb200_malloc_host(Nd4jLong bytes);   /* pinned */
int nd4jb200_free_host(Nd4jPointer p);
Nd4jPointer nd4jb200_create_stream(void);
int nd4jb200_destroy_stream(Nd4jPointer stream);
int nd4jb200_stream_synchronize(Nd4jPointer stream);
Nd4jPointer nd4jb200_create_event(void);
int nd4jb200_register_event(Nd4jPointer event, Nd4jPointer stream);
int nd4jb200_event_synchronize(Nd4jPointer event);
int nd4jb200_destroy_event(Nd4jPointer event);
/* milliseconds between two recorded events (cudaEventElapsedTime) */
int nd4jb200_event_elapsed_ms(Nd4jPointer start, Nd4jPointer stop, float *ms);
/* flags: 0 host->host, 1 host->device, 2 device->host, 3 device->device (NativeOps.cu:4038-4075) */
int nd4jb200_memcpy_async(Nd4jPointer dst, Nd4jPointer src, Nd4jLong bytes, int flags, Nd4jPointer stream);
int nd4jb200_memcpy(Nd4jPointer dst, Nd4jPointer src, Nd4jLong bytes, int flags);
int nd4jb200_memset_async(Nd4jPointer dst, int value, Nd4jLong bytes, Nd4jPointer stream);
Nd4jLong nd4jb200_device_free_memory(int device);
Nd4jLong nd4jb200_device_total_memory(int device);
int nd4jb200_device_major(int device);
int nd4jb200_device_minor(int device);
const char *nd4jb200_device_name(int device);

/* ---- fused elementwise chains --------------------------------------------------------------------------------
 * exec_chain has no counterpart among the reference's members: it runs what a caller would otherwise issue as
 *   execBroadcast(broadcastOp, x, b, dimension) -> execTransform(transformOp) -> execPairwiseTransform(pairwiseOp, ., y)
 * (blas/NativeOps.h:615-649, 1337-1443, 665-798) as ONE pass that reads x and y once and writes z once, with results
 * bit-identical to the three calls. x, y and z must have one shape; z may alias x or y. Fused for the arithmetic /
 * comparison / min / max broadcast and pairwise ops and every elementwise transform; any other op combination is
 * executed as the three separate launches (through z, which must then not alias y).
 * exec_meta_predicate_* serve the reference's own fusion hook, NativeOps::execMetaPredicateShape* / Strided*
 * (blas/NativeOps.h:2564-2785): opTypeA 2 (pairwise opNumA on x, y with extraA) followed by opTypeB 0 (scalar
 * opNumB with scalarB), the only pair the reference implements (include/loops/cuda/grid_shaped.cu:159-211).
 * Unlike the reference's kernel, out-of-place calls write every element of z (grid_shaped.cu:283 writes
 * result[0] only). */
int nd4jb200_exec_chain(void *stream, int dtype, int broadcastOp, const void *x, const Nd4jLong *xShapeInfo,
                        const void *b, const Nd4jLong *bShapeInfo, const int *dimension, int dimensionLength,
                        int transformOp, const void *transformExtra, int pairwiseOp, const void *y,
                        const Nd4jLong *yShapeInfo, const void *pairwiseExtra, void *z, const Nd4jLong *zShapeInfo);
int nd4jb200_exec_meta_predicate_shape(void *stream, int dtype, int opTypeA, int opNumA, int opTypeB, int opNumB,
                                       const void *x, const Nd4jLong *xShapeInfo, const void *y,
                                       const Nd4jLong *yShapeInfo, void *z, const Nd4jLong *zShapeInfo,
                                       const void *extraA, const void *extraB, double scalarA, double scalarB);
int nd4jb200_exec_meta_predicate_strided(void *stream, int dtype, int opTypeA, int opNumA, int opTypeB, int opNumB,
                                         Nd4jLong n, const void *x, Nd4jLong xStride, const void *y, Nd4jLong yStride,
                                         void *z, Nd4jLong zStride, const void *extraA, const void *extraB,
                                         double scalarA, double scalarB);

/* ---- several GPUs: one process per GPU, one communicator per process -------------------------------------------
 * The exec* families shard without any exchange (TADs, elements and random indices are independent; see
 * nd4jb200_exec_random_range). The one exchange step of this path is the combine of per-GPU partials of a
 * whole-array reduction, and the across-GPU forms of average / accumulate; the reference does these by letting a
 * kernel read its peers' memory (blas/cuda/NativeOps.cu:4884-4968, include/loops/special_kernels.h:711-821;
 * peer access control blas/NativeOps.h:2047-2058). Here partial states travel through NCCL on the caller's stream
 * and no kernel reads another GPU's memory.
 *   comm_unique_id: rank 0 obtains 128 bytes and hands them to the other ranks by any means (it is ncclGetUniqueId);
 *   comm_init:      every rank, with its device current; collective. world == 1 needs neither an id nor NCCL;
 *   exec_reduce_scalar_sharded: the whole-array reduce (opNum of execReduceScalar*, blas/NativeOps.h:886-906) of
 *       an array cut into world * shardsPerRank equal contiguous shards, of which this rank holds shardsPerRank
 *       consecutive ones at x (localLength elements, dense). Every shard is reduced to an accumulator state, the
 *       states are all-gathered and every rank folds them in global shard order, so the value depends on the
 *       shard grid only: 8 shards give the same bits on 1, 2, 4 or 8 GPUs. totalLength is the n of Mean-like ops.
 *       The value goes to z (device, one element; may be null) and, if `result` is not null, to the host after a
 *       stream synchronisation; with result == null the call is asynchronous.
 *   accumulate_across: z = sum over ranks of x (ncclAllReduce; NativeOps::accumulate* across devices).
 *   average_across: z (or x when z is null) = sum over ranks of x / world, each term divided first as the
 *       reference's loop does (include/ops/impl/specials.cpp:392-400); propagate != 0 also writes it back to x.
 *       The order of the additions is NCCL's: results agree with the sequential loop to rounding, not bit for bit. */
int nd4jb200_comm_unique_id(void *id128);
int nd4jb200_comm_init(const void *id128, int rank, int world);
int nd4jb200_comm_destroy(void);
int nd4jb200_comm_rank(void);
int nd4jb200_comm_world(void);
int nd4jb200_exec_reduce_scalar_sharded(void *stream, int dtype, int opNum, const void *x, Nd4jLong localLength,
                                        const void *extraParams, int shardsPerRank, Nd4jLong totalLength, void *z,
                                        double *result);
int nd4jb200_accumulate_across(void *stream, int dtype, const void *x, void *z, Nd4jLong length);
int nd4jb200_average_across(void *stream, int dtype, void *x, void *z, Nd4jLong length, int propagate);

/* ---- peer access and the constant-memory staging area (blas/NativeOps.h:1836-1846, 2047-2058;
 *      blas/cuda/NativeOps.cu:87, 3854-3938, 4793-4834) -------------------------------------------------------
 * check_p2p probes every ordered device pair and records whether all of them can reach each other (one device
 * counts as supported); enable_p2p turns peer access on or off for every pair that supports it. The exec*
 * kernels never read another GPU's memory; these exist for callers that copy between devices themselves.
 * The constant space is a 49152-byte __constant__ array, as in the reference: memcpy_constant_async copies
 * `bytes` to byte offset `offset` of it (flags 1 host->device, 3 device->device) and get_constant_space returns
 * its device address, so that descriptors staged there can be passed as device pointers. */
int nd4jb200_check_p2p(void);
int nd4jb200_is_p2p_available(void);
int nd4jb200_enable_p2p(int enable);
int nd4jb200_memcpy_constant_async(Nd4jLong offset, const void *src, Nd4jLong bytes, int flags, void *stream);
void *nd4jb200_get_constant_space(void);

#ifdef __cplusplus
}
#endif
#endif /* ND4J_B200_H */
