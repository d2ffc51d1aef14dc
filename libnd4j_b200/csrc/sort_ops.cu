// In-place sorting of a whole array or of every TAD of an array (NativeOps::sort{Float,Double,Half},
// sortTad{Float,Double,Half}; blas/NativeOps.h:2940-2952). The reference's CPU build runs a quicksort over
// getPosition(shapeInfo, i) (include/ops/impl/specials.cpp:457-564); a sorted sequence does not depend on the
// algorithm, so the result is the reference's bit for bit wherever the values are distinct (equal values,
// such as -0 and +0, may come out in either order there, as with any unstable sort, and NaNs have no defined
// place in it; here the order is total: -0 before +0, NaNs at the two ends by their sign).
//
// Here: a bitonic network in its "mirror" form -- stage k first compares element i of every block of k
// with its mirror image k-1-i, then runs half-cleaners with strides k/4 ... 1 -- in which every comparator
// puts the earlier value at the lower position. Positions past the end behave like values that sort last
// and are never moved by such a comparator, so any length works without padding in memory.
//   * chunks of CN elements (8192 four-byte or 4096 eight-byte keys) are sorted on chip, eight keys per
//     thread in registers, exchanged by warp shuffles and, beyond a warp, through shared memory: one read
//     and one write of the data for the first log2(CN) stages;
//   * every later stage k runs its strides >= 2048 as passes over global memory, three steps per pass (a
//     thread orders the eight positions those steps connect), and its strides < 2048 again on chip, one pass.
// TADs of up to CN elements take a single launch (a warp per TAD up to 256 keys, a CTA per TAD above).
#include "../../include/nd4j_b200.h"
#include "device_utils.cuh"
#include "runtime.h"
#include "radix_sort.cuh"
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


// ---- chunks in registers ------------------------------------------------------------------------------
// A chunk of CN = 8 G keys is held by G threads, thread t owning positions 8 t ... 8 t + 7. The partner of
// position i is i ^ m in every step (m = k - 1 for the mirror step of stage k, m = j for a half-cleaner), so
// a step is one of three kinds: m < 8 stays inside a thread's registers; a partner thread t ^ (m >> 3) in
// the same warp is reached with shuffles; anything further goes through shared memory. The member of a
// pair at the lower position keeps the smaller key.
constexpr int kKeys = 8;

// On chip the keys are integers whose signed order is the order wanted: the IEEE bit pattern with the
// magnitude bits of negative values flipped (so -0 sorts before +0 and NaNs sort to the ends by sign), and
// all bits inverted for a descending sort. Comparators are then an integer min and max, and no key can be
// lost or duplicated whatever its value. The transform is its own inverse.
template <class C> struct SortKey;
template <> struct SortKey<float> {
    typedef int K;
    static constexpr K kLast = 0x7fffffff;
    static ND_D K flip(K b, int descending) { b ^= (b >> 31) & 0x7fffffff; return descending ? ~b : b; }
    static ND_D K to_key(float v, int descending) { return flip(__float_as_int(v), descending); }
    static ND_D float from_key(K k, int descending) { if (descending) k = ~k; return __int_as_float(k ^ ((k >> 31) & 0x7fffffff)); }
};
template <> struct SortKey<double> {
    typedef long long K;
    static constexpr K kLast = 0x7fffffffffffffffll;
    static ND_D K to_key(double v, int descending) {
        K b = __double_as_longlong(v);
        b ^= (b >> 63) & 0x7fffffffffffffffll;
        return descending ? ~b : b;
    }
    static ND_D double from_key(K k, int descending) {
        if (descending) k = ~k;
        return __longlong_as_double(k ^ ((k >> 63) & 0x7fffffffffffffffll));
    }
};

template <class K> ND_D void order_regs(K &lo, K &hi) {
    const K a = min(lo, hi), b = max(lo, hi);
    lo = a; hi = b;
}
// stages 2, 4 and 8 of a thread's own eight keys
template <class K> ND_D void head_stages(K (&v)[kKeys]) {
#pragma unroll
    for (int k = 2; k <= kKeys; k <<= 1) {
#pragma unroll
        for (int e = 0; e < kKeys; e++) {
            const int partner = e ^ (k - 1);
            if (e < partner) order_regs(v[e], v[partner]);
        }
#pragma unroll
        for (int j = k >> 2; j > 0; j >>= 1)
#pragma unroll
            for (int e = 0; e < kKeys; e++)
                if ((e & j) == 0) order_regs(v[e], v[e + j]);
    }
}
// half-cleaners of stride 4, 2, 1
template <class K> ND_D void tail_steps(K (&v)[kKeys]) {
#pragma unroll
    for (int j = kKeys >> 1; j > 0; j >>= 1)
#pragma unroll
        for (int e = 0; e < kKeys; e++)
            if ((e & j) == 0) order_regs(v[e], v[e + j]);
}

template <int G> ND_D void group_sync() {
    if (G == 32) __syncwarp(); else __syncthreads();
}
// shared-memory slot of key e of thread t: rows of G + 4 so that both the per-thread and the linear access
// patterns are free of bank conflicts
template <int G> ND_D int slot(int e, int t) { return e * (G + 4) + t; }

// partner thread t ^ mt; MIRROR: the partner's keys are taken in reverse order (m = k - 1 flips the low bits)
template <class K, int G, bool MIRROR>
ND_D void cross_step(K (&v)[kKeys], K *s, int t, int mt, int highT) {
    K p[kKeys];
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
        const K a = min(v[e], p[e]), b = max(v[e], p[e]);
        v[e] = lower ? a : b;
    }
}

// fullSort: sorts every chunk (stages 2 ... CN). Otherwise: the strides CN/2 ... 1 of a later stage.
// THREADS / G chunks are worked on by one CTA at a time (G = 32: a warp per chunk, no CTA barriers).
template <class T, int G, int THREADS>
__global__ void __launch_bounds__(THREADS) k_sort_chunks(const SortArgs a, int fullSort, int dense) {
    grid_dependency_sync();
    typedef typename Elem<T>::C C;
    typedef SortKey<C> Key;
    typedef typename Key::K K;
    constexpr int CN = G * kKeys, kGroups = THREADS / G;
    __shared__ K shared[kGroups * kKeys * (G + 4)];
    const int t = threadIdx.x % G, group = threadIdx.x / G;
    K *s = shared + group * kKeys * (G + 4);
    T *ax = static_cast<T *>(a.x);
    const int d = a.descending;
    const LL chunks = (a.n + CN - 1) / CN, units = a.numTads * chunks;
    for (LL u = (LL) blockIdx.x * kGroups + group; u < units; u += (LL) gridDim.x * kGroups) {
        const LL tad = u / chunks, first = (u - tad * chunks) * CN;
        T *base = ax + view_offset(a.outer, tad);
        // dense chunks that lie wholly inside the TAD: a thread's eight keys are 16-byte packs of its own
        const bool direct = dense && first + CN <= a.n;
        K v[kKeys];
        if (direct) {
            constexpr int PER = 16 / sizeof(T), PACKS = kKeys / PER;
            struct alignas(16) Pack16 { T v[PER]; };
            const Pack16 *src = reinterpret_cast<const Pack16 *>(base + first + (LL) t * kKeys);
#pragma unroll
            for (int p = 0; p < PACKS; p++) {
                const Pack16 pk = src[p];
#pragma unroll
                for (int e = 0; e < PER; e++) v[p * PER + e] = Key::to_key(Elem<T>::to_c(pk.v[e]), d);
            }
        } else {
            // coalesced over linear positions through shared memory, then every thread picks up its eight keys
            for (int idx = t; idx < CN; idx += G) {
                const LL i = first + idx;
                s[slot<G>(idx & (kKeys - 1), idx / kKeys)] =
                    i < a.n ? Key::to_key(Elem<T>::load(base + view_offset(a.inner, i)), d) : Key::kLast;
            }
            group_sync<G>();
#pragma unroll
            for (int e = 0; e < kKeys; e++) v[e] = s[slot<G>(e, t)];
            group_sync<G>();
        }
        if (fullSort) {
            head_stages(v);
            for (int k = 2 * kKeys; k <= CN; k <<= 1) {
                cross_step<K, G, true>(v, s, t, k / kKeys - 1, k / (2 * kKeys));
                for (int j = k >> 2; j >= kKeys; j >>= 1) cross_step<K, G, false>(v, s, t, j / kKeys, j / kKeys);
                tail_steps(v);
            }
        } else {
            for (int j = CN >> 1; j >= kKeys; j >>= 1) cross_step<K, G, false>(v, s, t, j / kKeys, j / kKeys);
            tail_steps(v);
        }
        if (direct) {
            constexpr int PER = 16 / sizeof(T), PACKS = kKeys / PER;
            struct alignas(16) Pack16 { T v[PER]; };
            Pack16 *dst = reinterpret_cast<Pack16 *>(base + first + (LL) t * kKeys);
#pragma unroll
            for (int p = 0; p < PACKS; p++) {
                Pack16 pk;
#pragma unroll
                for (int e = 0; e < PER; e++) pk.v[e] = Elem<T>::from_c(Key::from_key(v[p * PER + e], d));
                dst[p] = pk;
            }
            // the exchanges of the next chunk reuse the shared-memory slots this one may still be reading
            group_sync<G>();
            continue;
        }
#pragma unroll
        for (int e = 0; e < kKeys; e++) s[slot<G>(e, t)] = v[e];
        group_sync<G>();
        for (int idx = t; idx < CN; idx += G) {
            const LL i = first + idx;
            if (i < a.n)
                Elem<T>::store(base + view_offset(a.inner, i), Key::from_key(s[slot<G>(idx & (kKeys - 1), idx / kKeys)], d));
        }
        group_sync<G>();
    }
}

// L consecutive steps of stage a.k in one pass over global memory: the mirror step (MIRROR) or the
// half-cleaner of stride a.j, followed by the next L - 1 half-cleaners. The 2^L positions that those steps
// connect (a position and its images under every combination of the steps' masks) are loaded by one thread,
// ordered in registers and written back, so a stage with s strides beyond the chunk size costs ceil(s / 3)
// passes instead of s. Neighbouring threads own neighbouring positions in each of the 2^L loads.
template <class T, int L, bool MIRROR>
__global__ void __launch_bounds__(256) k_sort_global_pass(const SortArgs a, LL padded) {
    grid_dependency_sync();
    typedef typename Elem<T>::C C;
    typedef SortKey<C> Key;
    typedef typename Key::K K;
    constexpr int N = 1 << L;
    T *ax = static_cast<T *>(a.x);
    const LL high = MIRROR ? a.k >> 1 : a.j;          // the highest position bit these steps act on
    LL mask[L];
    mask[0] = MIRROR ? a.k - 1 : a.j;
#pragma unroll
    for (int l = 1; l < L; l++) mask[l] = high >> l;
    const LL low = (high >> (L - 1)) - 1;             // position bits below the L bits a thread spans
    const LL per = padded >> L, total = a.numTads * per, nthreads = (LL) gridDim.x * 256;
    const int d = a.descending;
    for (LL u = (LL) blockIdx.x * 256 + threadIdx.x; u < total; u += nthreads) {
        const LL tad = u / per, q = u - tad * per;
        const LL first = ((q & ~low) << L) | (q & low);
        T *base = ax + view_offset(a.outer, tad);
        LL idx[N];
        K key[N];
#pragma unroll
        for (int c = 0; c < N; c++) {
            LL i = first;
#pragma unroll
            for (int l = 0; l < L; l++)
                if ((c >> l) & 1) i ^= mask[l];
            idx[c] = i;
            key[c] = i < a.n ? Key::to_key(Elem<T>::load(base + view_offset(a.inner, i)), d) : Key::kLast;
        }
#pragma unroll
        for (int l = 0; l < L; l++) {
#pragma unroll
            for (int c = 0; c < N; c++) {
                if ((c >> l) & 1) continue;
                // the mirror image has the lower position bits flipped, which turns the later pairs around
                if (MIRROR && l > 0 && (c & 1)) order_regs(key[c | (1 << l)], key[c]);
                else order_regs(key[c], key[c | (1 << l)]);
            }
        }
#pragma unroll
        for (int c = 0; c < N; c++)
            if (idx[c] < a.n) Elem<T>::store(base + view_offset(a.inner, idx[c]), Key::from_key(key[c], d));
    }
}

// The same pass for dense data, VK neighbouring positions per access: the steps treat neighbouring positions
// alike (all strides are far larger than VK), so lane e of every access is an independent instance of the
// scalar pass at position first + e. The mirror image of VK neighbouring positions is again VK neighbouring
// positions, in reverse order: those vectors are reversed after loading and before storing.
template <class T> struct SortVec {
    static constexpr int VK = sizeof(T) == 8 ? 2 : 4;
    struct alignas(sizeof(T) * VK) V { T v[VK]; };
};

template <class T, int L, bool MIRROR>
__global__ void __launch_bounds__(256) k_sort_global_pass_vec(const SortArgs a, LL padded) {
    grid_dependency_sync();
    typedef typename Elem<T>::C C;
    typedef SortKey<C> Key;
    typedef typename Key::K K;
    typedef typename SortVec<T>::V V;
    constexpr int N = 1 << L, VK = SortVec<T>::VK;
    T *ax = static_cast<T *>(a.x);
    const LL high = MIRROR ? a.k >> 1 : a.j;
    LL mask[L];
    mask[0] = MIRROR ? a.k - 1 : a.j;
#pragma unroll
    for (int l = 1; l < L; l++) mask[l] = high >> l;
    const LL low = (high >> (L - 1)) - 1;
    const LL per = (padded >> L) / VK, total = a.numTads * per, nthreads = (LL) gridDim.x * 256;
    const int d = a.descending;
    for (LL u = (LL) blockIdx.x * 256 + threadIdx.x; u < total; u += nthreads) {
        const LL tad = u / per, q = (u - tad * per) * VK;
        const LL first = ((q & ~low) << L) | (q & low);
        T *base = ax + view_offset(a.outer, tad);
        LL start[N];
        K key[N][VK];
#pragma unroll
        for (int c = 0; c < N; c++) {
            LL i = first;
#pragma unroll
            for (int l = 0; l < L; l++)
                if ((c >> l) & 1) i ^= mask[l];
            const bool reversed = MIRROR && (c & 1);
            start[c] = reversed ? i - (VK - 1) : i;         // the lowest of the VK positions
            if (start[c] + VK <= a.n) {
                const V pack = *reinterpret_cast<const V *>(base + start[c]);
#pragma unroll
                for (int e = 0; e < VK; e++) key[c][reversed ? VK - 1 - e : e] = Key::to_key(Elem<T>::to_c(pack.v[e]), d);
            } else {
#pragma unroll
                for (int e = 0; e < VK; e++) {
                    const LL pos = start[c] + e;
                    key[c][reversed ? VK - 1 - e : e] = pos < a.n ? Key::to_key(Elem<T>::load(base + pos), d) : Key::kLast;
                }
            }
        }
#pragma unroll
        for (int l = 0; l < L; l++) {
#pragma unroll
            for (int c = 0; c < N; c++) {
                if ((c >> l) & 1) continue;
                const bool turned = MIRROR && l > 0 && (c & 1);
#pragma unroll
                for (int e = 0; e < VK; e++) {
                    if (turned) order_regs(key[c | (1 << l)][e], key[c][e]);
                    else order_regs(key[c][e], key[c | (1 << l)][e]);
                }
            }
        }
#pragma unroll
        for (int c = 0; c < N; c++) {
            const bool reversed = MIRROR && (c & 1);
            if (start[c] + VK <= a.n) {
                V pack;
#pragma unroll
                for (int e = 0; e < VK; e++) pack.v[e] = Elem<T>::from_c(Key::from_key(key[c][reversed ? VK - 1 - e : e], d));
                *reinterpret_cast<V *>(base + start[c]) = pack;
            } else {
#pragma unroll
                for (int e = 0; e < VK; e++) {
                    const LL pos = start[c] + e;
                    if (pos < a.n) Elem<T>::store(base + pos, Key::from_key(key[c][reversed ? VK - 1 - e : e], d));
                }
            }
        }
    }
}

template <class T, bool MIRROR>
void launch_global(const SortArgs &a, int levels, LL padded, cudaStream_t st) {
    constexpr int VK = SortVec<T>::VK;
    const bool dense = (a.inner.rank == 0 || (a.inner.rank == 1 && a.inner.stride[0] == 1)) &&
                       reinterpret_cast<uintptr_t>(a.x) % (sizeof(T) * VK) == 0 && view_strides_multiple_of(a.outer, VK);
    LL blocks = ceil_div(a.numTads * (padded >> levels) / (dense ? VK : 1), 256);
    const LL cap = (LL) kNumSMs * 32;
    if (blocks > cap) blocks = cap;
    if (blocks < 1) blocks = 1;
    const dim3 grid((unsigned) blocks), block(256);
    if (dense) {
        if (levels == 1) launch_kernel(k_sort_global_pass_vec<T, 1, MIRROR>, grid, block, st, a, padded);
        else if (levels == 2) launch_kernel(k_sort_global_pass_vec<T, 2, MIRROR>, grid, block, st, a, padded);
        else launch_kernel(k_sort_global_pass_vec<T, 3, MIRROR>, grid, block, st, a, padded);
        return;
    }
    if (levels == 1) launch_kernel(k_sort_global_pass<T, 1, MIRROR>, grid, block, st, a, padded);
    else if (levels == 2) launch_kernel(k_sort_global_pass<T, 2, MIRROR>, grid, block, st, a, padded);
    else launch_kernel(k_sort_global_pass<T, 3, MIRROR>, grid, block, st, a, padded);
}

template <class T, int G, int THREADS>
void launch_chunks(const SortArgs &a, int fullSort, cudaStream_t st) {
    LL blocks = ceil_div(a.numTads * ceil_div(a.n, G * kKeys), THREADS / G);
    const LL cap = (LL) kNumSMs * 32;
    if (blocks > cap) blocks = cap;
    // unit-stride TADs whose starts keep 16-byte alignment
    constexpr int PER = 16 / sizeof(T);
    const int dense = (a.inner.rank == 0 || (a.inner.rank == 1 && a.inner.stride[0] == 1)) && aligned16(a.x) &&
                      view_strides_multiple_of(a.outer, PER);
    launch_kernel(k_sort_chunks<T, G, THREADS>, dim3((unsigned) blocks), dim3(THREADS), st, a, fullSort, dense);
}

// From this length on a single dense array goes to the radix sort: below it the network's few stages beyond a
// chunk cost less than the radix sort's fixed dozen launches.
constexpr LL kRadixMin = 1 << 16;

template <class T>
Status run_sort(SortArgs a, cudaStream_t st) {
    if (a.numTads <= 0 || a.n <= 1) return kOk;
    // one long dense array: radix sort (3 sweeps per 8-bit digit instead of a sweep per network step)
    static_assert(kRadixThreads == kRadixBins, "one thread per digit in the scans");
    if (a.numTads == 1 && a.n >= kRadixMin && a.inner.rank == 1 && a.inner.stride[0] == 1)
        return run_radix_sort<T>(static_cast<T *>(a.x), a.n, a.descending, st);
    // threads per full-size chunk: 8192 four-byte or 4096 eight-byte keys
    constexpr int kBig = sizeof(typename Elem<T>::C) == 8 ? 512 : 1024;
    constexpr int kChunk = kBig * kKeys;
    // short TADs: the smallest chunk that holds one
    if (a.n <= 256) { launch_chunks<T, 32, 256>(a, 1, st); ND_CUDA(cudaGetLastError()); return kOk; }
    if (a.n <= 1024) { launch_chunks<T, 128, 128>(a, 1, st); ND_CUDA(cudaGetLastError()); return kOk; }
    if (a.n <= 2048) { launch_chunks<T, 256, 256>(a, 1, st); ND_CUDA(cudaGetLastError()); return kOk; }
    launch_chunks<T, kBig, kBig>(a, 1, st);
    ND_CUDA(cudaGetLastError());
    // The later stages finish on chip in chunks of 2048 keys: CTAs of 256 threads, several of which fit an SM
    // and overlap their loads with each other's exchanges (one CTA of 1024 threads per SM cannot).
    constexpr int kMergeThreads = 256, kMerge = kMergeThreads * kKeys;
    LL padded = kChunk;
    while (padded < a.n) padded <<= 1;
    for (LL k = 2 * (LL) kChunk; k <= padded; k <<= 1) {
        a.k = k;
        // steps of this stage beyond a merge chunk: the mirror step, then strides k/4 ... kMerge; three per pass
        int steps = 1;
        for (LL j = k >> 2; j >= kMerge; j >>= 1) steps++;
        int levels = steps < 3 ? steps : 3;
        a.j = 0;
        launch_global<T, true>(a, levels, padded, st);
        LL j = k >> (1 + levels);          // the next stride after `levels` steps (k/2 is the mirror's high bit)
        for (int left = steps - levels; left > 0; left -= levels) {
            levels = left < 3 ? left : 3;
            a.j = j;
            launch_global<T, false>(a, levels, padded, st);
            j >>= levels;
        }
        launch_chunks<T, kMergeThreads, kMergeThreads>(a, 0, st);
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
