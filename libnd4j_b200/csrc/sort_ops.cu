// In-place sorting of a whole array or of every TAD of an array (NativeOps::sort{Float,Double,Half},
// sortTad{Float,Double,Half}; blas/NativeOps.h:2940-2952). The reference's CPU build runs a quicksort over
// getPosition(shapeInfo, i) (include/ops/impl/specials.cpp:457-564); a sorted sequence does not depend on the
// algorithm, so the result is the reference's bit for bit wherever the values are distinct (equal values,
// such as -0 and +0, may come out in either order, as with any unstable sort; NaNs have no defined place in
// either implementation).
//
// Here: a bitonic network in its "mirror" form -- stage k first compares element i of every block of k
// with its mirror image k-1-i, then runs half-cleaners with strides k/4 ... 1 -- in which every comparator
// puts the earlier value at the lower position. Positions past the end behave like values that sort last
// and are never moved by such a comparator, so any length works without padding in memory.
//   * chunks of CN elements (8192 four-byte or 4096 eight-byte keys, 32 KB) are sorted entirely in shared
//     memory: one read and one write of the data for the first log2(CN) stages;
//   * every later stage k runs its strides >= CN as passes over global memory (coalesced: neighbouring
//     threads own neighbouring comparators) and its strides < CN again in shared memory, one pass.
// TADs of up to CN elements take a single launch with one CTA per TAD.
#include "../../include/nd4j_b200.h"
#include "device_utils.cuh"
#include "runtime.h"
#include <math_constants.h>
#include <vector>

namespace nd4jb200 {
namespace {

struct SortArgs {
    void *x;
    LL numTads, n;        // n: elements per TAD
    View outer, inner;    // TAD r -> base offset; position i of a TAD -> offset from the base
    int descending;
    LL k;                 // stage of the global / merge passes
    LL j;                 // stride of a global half-cleaner pass (0: the mirror step of stage k)
};

template <class C> ND_D bool sorts_before(C a, C b, int descending) { return descending ? a > b : a < b; }

template <class C> ND_D void order_pair(C &lo, C &hi, int descending) {
    if (sorts_before(hi, lo, descending)) { const C t = lo; lo = hi; hi = t; }
}

// The comparators of one step over a chunk held in shared memory. q numbers the CN/2 comparators.
template <class C, int CN, int THREADS> ND_D void mirror_step(C *s, int k, int descending) {
    const int half = k >> 1;
    for (int q = threadIdx.x; q < CN / 2; q += THREADS) {
        const int block = q / half, r = q - block * half;
        const int lo = block * k + r, hi = block * k + (k - 1 - r);
        order_pair(s[lo], s[hi], descending);
    }
    __syncthreads();
}
template <class C, int CN, int THREADS> ND_D void stride_steps(C *s, int jFirst, int descending) {
    for (int j = jFirst; j > 0; j >>= 1) {
        for (int q = threadIdx.x; q < CN / 2; q += THREADS) {
            const int lo = ((q & ~(j - 1)) << 1) | (q & (j - 1));
            order_pair(s[lo], s[lo + j], descending);
        }
        __syncthreads();
    }
}

// fullSort: sorts every chunk (stages 2 ... CN). Otherwise: the strides CN/2 ... 1 of a later stage.
template <class T, int CN, int THREADS>
__global__ void __launch_bounds__(THREADS) k_sort_chunks(const SortArgs a, int fullSort) {
    grid_dependency_sync();
    typedef typename Elem<T>::C C;
    __shared__ C s[CN];
    T *ax = static_cast<T *>(a.x);
    const C inf = sizeof(C) == 8 ? C(CUDART_INF) : C(CUDART_INF_F);
    const C last = a.descending ? -inf : inf;
    const LL chunks = (a.n + CN - 1) / CN, units = a.numTads * chunks;
    for (LL u = blockIdx.x; u < units; u += gridDim.x) {
        const LL tad = u / chunks, first = (u - tad * chunks) * CN;
        T *base = ax + view_offset(a.outer, tad);
        for (int t = threadIdx.x; t < CN; t += THREADS) {
            const LL i = first + t;
            s[t] = i < a.n ? Elem<T>::load(base + view_offset(a.inner, i)) : last;
        }
        __syncthreads();
        if (fullSort) {
            for (int k = 2; k <= CN; k <<= 1) {
                mirror_step<C, CN, THREADS>(s, k, a.descending);
                stride_steps<C, CN, THREADS>(s, k >> 2, a.descending);
            }
        } else {
            stride_steps<C, CN, THREADS>(s, CN / 2, a.descending);
        }
        for (int t = threadIdx.x; t < CN; t += THREADS) {
            const LL i = first + t;
            if (i < a.n) Elem<T>::store(base + view_offset(a.inner, i), s[t]);
        }
        __syncthreads();
    }
}

// One step of stage a.k over global memory: the mirror step (a.j == 0) or the half-cleaner of stride a.j.
// `half` = comparators per TAD (half of the length rounded up to a power of two), a power of two.
template <class T>
__global__ void __launch_bounds__(256) k_sort_global_step(const SortArgs a, LL half) {
    grid_dependency_sync();
    typedef typename Elem<T>::C C;
    T *ax = static_cast<T *>(a.x);
    const LL total = a.numTads * half, nthreads = (LL) gridDim.x * 256;
    for (LL u = (LL) blockIdx.x * 256 + threadIdx.x; u < total; u += nthreads) {
        const LL tad = u / half, q = u - tad * half;
        LL lo, hi;
        if (a.j == 0) {
            const LL hk = a.k >> 1, block = q / hk, r = q - block * hk;
            lo = block * a.k + r; hi = block * a.k + (a.k - 1 - r);
        } else {
            lo = ((q & ~(a.j - 1)) << 1) | (q & (a.j - 1)); hi = lo + a.j;
        }
        if (hi >= a.n) continue;      // the partner lies past the end: it sorts last and stays
        T *base = ax + view_offset(a.outer, tad);
        T *pl = base + view_offset(a.inner, lo), *ph = base + view_offset(a.inner, hi);
        const C vl = Elem<T>::load(pl), vh = Elem<T>::load(ph);
        if (sorts_before(vh, vl, a.descending)) { Elem<T>::store(pl, vh); Elem<T>::store(ph, vl); }
    }
}

template <class T, int CN, int THREADS>
void launch_chunks(const SortArgs &a, int fullSort, cudaStream_t st) {
    LL blocks = a.numTads * ceil_div(a.n, CN);
    const LL cap = (LL) kNumSMs * 32;
    if (blocks > cap) blocks = cap;
    launch_kernel(k_sort_chunks<T, CN, THREADS>, dim3((unsigned) blocks), dim3(THREADS), st, a, fullSort);
}

template <class T>
Status run_sort(SortArgs a, cudaStream_t st) {
    if (a.numTads <= 0 || a.n <= 1) return kOk;
    constexpr int kChunk = sizeof(typename Elem<T>::C) == 8 ? 4096 : 8192;
    // short TADs: the smallest chunk that holds one
    if (a.n <= 256) { launch_chunks<T, 256, 128>(a, 1, st); ND_CUDA(cudaGetLastError()); return kOk; }
    if (a.n <= 2048) { launch_chunks<T, 2048, 512>(a, 1, st); ND_CUDA(cudaGetLastError()); return kOk; }
    launch_chunks<T, kChunk, 512>(a, 1, st);
    ND_CUDA(cudaGetLastError());
    LL padded = kChunk;
    while (padded < a.n) padded <<= 1;
    const LL half = padded >> 1, total = a.numTads * half;
    LL blocks = ceil_div(total, 256);
    const LL cap = (LL) kNumSMs * 32;
    if (blocks > cap) blocks = cap;
    for (LL k = 2 * (LL) kChunk; k <= padded; k <<= 1) {
        a.k = k; a.j = 0;
        launch_kernel(k_sort_global_step<T>, dim3((unsigned) blocks), dim3(256), st, a, half);
        for (LL j = k >> 2; j >= kChunk; j >>= 1) {
            a.j = j;
            launch_kernel(k_sort_global_step<T>, dim3((unsigned) blocks), dim3(256), st, a, half);
        }
        launch_chunks<T, kChunk, 512>(a, 0, st);
        ND_CUDA(cudaGetLastError());
    }
    return kOk;
}

Status dispatch_sort(int dtype, const SortArgs &a, cudaStream_t st) {
    if (dtype == ND4JB200_FLOAT) return run_sort<float>(a, st);
    if (dtype == ND4JB200_DOUBLE) return run_sort<double>(a, st);
    if (dtype == ND4JB200_HALF) return run_sort<__half>(a, st);
    return bad_arg("dtype must be 0 (float), 1 (double) or 2 (half)");
}

}  // namespace
}  // namespace nd4jb200

using namespace nd4jb200;

#pragma GCC visibility push(default)
extern "C" {

int nd4jb200_sort(void *stream, int dtype, void *x, const Nd4jLong *xShapeInfo, int descending) {
    if (!x) return bad_arg("sort: null array");
    ShapeDesc xd;
    ND_TRY(parse_shape(xShapeInfo, "xShapeInfo", &xd));
    SortArgs a;
    a.x = x; a.numTads = 1; a.n = xd.length; a.descending = descending != 0; a.k = 0; a.j = 0;
    a.outer.rank = 0;
    ND_TRY(linear_view(xd, &a.inner));       // getPosition(): i * ews, or c-order coordinates (specials.cpp:461)
    return dispatch_sort(dtype, a, static_cast<cudaStream_t>(stream));
}

int nd4jb200_sort_tad(void *stream, int dtype, void *x, const Nd4jLong *xShapeInfo, const int *dimension,
                      int dimensionLength, int descending) {
    if (!x) return bad_arg("sortTad: null array");
    if (!dimension || dimensionLength < 1) return bad_arg("sortTad: no dimension");
    ShapeDesc xd, td;
    ND_TRY(parse_shape(xShapeInfo, "xShapeInfo", &xd));
    TadPlan plan;
    ND_TRY(make_tad_plan(xd, dimension, dimensionLength, &plan));
    // positions inside a TAD follow the TAD's own shapeInfo, as quickSort_parallel(dx, tadShapeInfo, ...) does
    std::vector<LL> tadInfo(2 * kMaxRank + 4);
    LL numTads = 0;
    ND_TRY(tad_only_shape_info(xShapeInfo, dimension, dimensionLength, tadInfo.data(), nullptr, &numTads));
    ND_TRY(parse_shape(tadInfo.data(), "tadShapeInfo", &td));
    SortArgs a;
    a.x = x; a.numTads = plan.numTads; a.n = plan.tadLen; a.descending = descending != 0; a.k = 0; a.j = 0;
    a.outer = plan.outer;
    ND_TRY(linear_view(td, &a.inner));
    return dispatch_sort(dtype, a, static_cast<cudaStream_t>(stream));
}

}  // extern "C"
#pragma GCC visibility pop
