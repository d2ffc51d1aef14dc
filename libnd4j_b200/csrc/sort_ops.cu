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
//   * chunks of CN elements (8192 four-byte or 4096 eight-byte keys) are sorted on chip, eight keys per
//     thread in registers, exchanged by warp shuffles and, beyond a warp, through shared memory: one read
//     and one write of the data for the first log2(CN) stages;
//   * every later stage k runs its strides >= CN as passes over global memory (coalesced: neighbouring
//     threads own neighbouring comparators) and its strides < CN again on chip, one pass.
// TADs of up to CN elements take a single launch (a warp per TAD up to 256 keys, a CTA per TAD above).
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

// ---- chunks in registers ------------------------------------------------------------------------------
// A chunk of CN = 8 G keys is held by G threads, thread t owning positions 8 t ... 8 t + 7. The partner of
// position i is i ^ m in every step (m = k - 1 for the mirror step of stage k, m = j for a half-cleaner), so
// a step is one of three kinds: m < 8 stays inside a thread's registers; a partner thread t ^ (m >> 3) in
// the same warp is reached with shuffles; anything further goes through shared memory. The member of a
// pair at the lower position keeps the value that sorts earlier; with equal (or unordered) values both
// keep their own, so the keys stay a permutation of the input whatever they are.
constexpr int kKeys = 8;

template <class C> ND_D void order_regs(C &lo, C &hi, int descending) {
    if (sorts_before(hi, lo, descending)) { const C t = lo; lo = hi; hi = t; }
}
// stages 2, 4 and 8 of a thread's own eight keys
template <class C> ND_D void head_stages(C (&v)[kKeys], int d) {
#pragma unroll
    for (int k = 2; k <= kKeys; k <<= 1) {
#pragma unroll
        for (int e = 0; e < kKeys; e++) {
            const int partner = e ^ (k - 1);
            if (e < partner) order_regs(v[e], v[partner], d);
        }
#pragma unroll
        for (int j = k >> 2; j > 0; j >>= 1)
#pragma unroll
            for (int e = 0; e < kKeys; e++)
                if ((e & j) == 0) order_regs(v[e], v[e + j], d);
    }
}
// half-cleaners of stride 4, 2, 1
template <class C> ND_D void tail_steps(C (&v)[kKeys], int d) {
#pragma unroll
    for (int j = kKeys >> 1; j > 0; j >>= 1)
#pragma unroll
        for (int e = 0; e < kKeys; e++)
            if ((e & j) == 0) order_regs(v[e], v[e + j], d);
}

template <int G> ND_D void group_sync() {
    if (G == 32) __syncwarp(); else __syncthreads();
}
// shared-memory slot of key e of thread t: rows of G + 4 so that both the per-thread and the linear access
// patterns are free of bank conflicts
template <int G> ND_D int slot(int e, int t) { return e * (G + 4) + t; }

// partner thread t ^ mt; MIRROR: the partner's keys are taken in reverse order (m = k - 1 flips the low bits)
template <class C, int G, bool MIRROR>
ND_D void cross_step(C (&v)[kKeys], C *s, int t, int mt, int highT, int d) {
    C p[kKeys];
    if (mt < 32) {
#pragma unroll
        for (int e = 0; e < kKeys; e++) p[e] = __shfl_xor_sync(0xffffffffu, v[MIRROR ? kKeys - 1 - e : e], mt);
    } else {
#pragma unroll
        for (int e = 0; e < kKeys; e++) s[slot<G>(e, t)] = v[e];
        group_sync<G>();
        const int pt = t ^ mt;
#pragma unroll
        for (int e = 0; e < kKeys; e++) p[e] = s[slot<G>(MIRROR ? kKeys - 1 - e : e, pt)];
        group_sync<G>();
    }
    const bool lower = (t & highT) == 0;
#pragma unroll
    for (int e = 0; e < kKeys; e++) {
        const bool take = lower ? sorts_before(p[e], v[e], d) : sorts_before(v[e], p[e], d);
        v[e] = take ? p[e] : v[e];
    }
}

// fullSort: sorts every chunk (stages 2 ... CN). Otherwise: the strides CN/2 ... 1 of a later stage.
// THREADS / G chunks are worked on by one CTA at a time (G = 32: a warp per chunk, no CTA barriers).
template <class T, int G, int THREADS>
__global__ void __launch_bounds__(THREADS) k_sort_chunks(const SortArgs a, int fullSort) {
    grid_dependency_sync();
    typedef typename Elem<T>::C C;
    constexpr int CN = G * kKeys, kGroups = THREADS / G;
    __shared__ C shared[kGroups * kKeys * (G + 4)];
    const int t = threadIdx.x % G, group = threadIdx.x / G;
    C *s = shared + group * kKeys * (G + 4);
    T *ax = static_cast<T *>(a.x);
    const C inf = sizeof(C) == 8 ? C(CUDART_INF) : C(CUDART_INF_F);
    const C last = a.descending ? -inf : inf;
    const int d = a.descending;
    const LL chunks = (a.n + CN - 1) / CN, units = a.numTads * chunks;
    for (LL u = (LL) blockIdx.x * kGroups + group; u < units; u += (LL) gridDim.x * kGroups) {
        const LL tad = u / chunks, first = (u - tad * chunks) * CN;
        T *base = ax + view_offset(a.outer, tad);
        // coalesced over linear positions, then every thread picks up its eight keys
        for (int idx = t; idx < CN; idx += G) {
            const LL i = first + idx;
            s[slot<G>(idx & (kKeys - 1), idx / kKeys)] = i < a.n ? Elem<T>::load(base + view_offset(a.inner, i)) : last;
        }
        group_sync<G>();
        C v[kKeys];
#pragma unroll
        for (int e = 0; e < kKeys; e++) v[e] = s[slot<G>(e, t)];
        group_sync<G>();
        if (fullSort) {
            head_stages(v, d);
            for (int k = 2 * kKeys; k <= CN; k <<= 1) {
                cross_step<C, G, true>(v, s, t, k / kKeys - 1, k / (2 * kKeys), d);
                for (int j = k >> 2; j >= kKeys; j >>= 1) cross_step<C, G, false>(v, s, t, j / kKeys, j / kKeys, d);
                tail_steps(v, d);
            }
        } else {
            for (int j = CN >> 1; j >= kKeys; j >>= 1) cross_step<C, G, false>(v, s, t, j / kKeys, j / kKeys, d);
            tail_steps(v, d);
        }
#pragma unroll
        for (int e = 0; e < kKeys; e++) s[slot<G>(e, t)] = v[e];
        group_sync<G>();
        for (int idx = t; idx < CN; idx += G) {
            const LL i = first + idx;
            if (i < a.n) Elem<T>::store(base + view_offset(a.inner, i), s[slot<G>(idx & (kKeys - 1), idx / kKeys)]);
        }
        group_sync<G>();
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

template <class T, int G, int THREADS>
void launch_chunks(const SortArgs &a, int fullSort, cudaStream_t st) {
    LL blocks = ceil_div(a.numTads * ceil_div(a.n, G * kKeys), THREADS / G);
    const LL cap = (LL) kNumSMs * 32;
    if (blocks > cap) blocks = cap;
    launch_kernel(k_sort_chunks<T, G, THREADS>, dim3((unsigned) blocks), dim3(THREADS), st, a, fullSort);
}

template <class T>
Status run_sort(SortArgs a, cudaStream_t st) {
    if (a.numTads <= 0 || a.n <= 1) return kOk;
    // threads per full-size chunk: 8192 four-byte or 4096 eight-byte keys
    constexpr int kBig = sizeof(typename Elem<T>::C) == 8 ? 512 : 1024;
    constexpr int kChunk = kBig * kKeys;
    // short TADs: the smallest chunk that holds one
    if (a.n <= 256) { launch_chunks<T, 32, 256>(a, 1, st); ND_CUDA(cudaGetLastError()); return kOk; }
    if (a.n <= 1024) { launch_chunks<T, 128, 128>(a, 1, st); ND_CUDA(cudaGetLastError()); return kOk; }
    if (a.n <= 2048) { launch_chunks<T, 256, 256>(a, 1, st); ND_CUDA(cudaGetLastError()); return kOk; }
    launch_chunks<T, kBig, kBig>(a, 1, st);
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
        launch_chunks<T, kBig, kBig>(a, 0, st);
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
