// Least-significant-digit radix sort for one long dense array: 8-bit digits, so 4 passes for float, 8 for double
// and 2 for half keys, each pass three launches (tile histograms, per-digit scan over the tiles, stable scatter).
// The bitonic network of sort_ops.cu needs log2(n)^2 / 2 compare steps per key, 45 sweeps of the array for 2^24
// keys; this needs 3 sweeps per pass whatever n is. The reference sorts with a quicksort on the host
// (include/ops/impl/specials.cpp:457-564); the sorted sequence is the same.
//
// Keys: the IEEE bit pattern made order-preserving as an unsigned integer (negative values inverted, the sign
// bit of the others set; all bits inverted again for a descending sort). That is the total order the network
// uses too: -0 before +0, NaNs at the two ends by their sign. The first pass reads the array's own values and
// the last pass writes them back, so that the data moves 2 x passes times, never more.
//
// A tile of kRadixThreads * KPT consecutive keys is owned by one CTA, warp w holding a contiguous run and
// lane l of round r the key at run offset r * 32 + l, so "earlier key" means "lower (warp, round, lane)".
// Ranks among equal digits come from __match_any_sync plus a per-warp counter table in shared memory; keys are
// first placed at their tile-local sorted position in shared memory and then written out in that order, which
// turns the scatter into runs of (on average) tile / 256 consecutive keys per digit.
#pragma once
#include "device_utils.cuh"
#include "runtime.h"

namespace nd4jb200 {

constexpr int kRadixThreads = 256;
constexpr int kRadixWarps = kRadixThreads / 32;
constexpr int kRadixBins = 256;

template <class T> struct RadixKey;
template <> struct RadixKey<float> {
    typedef unsigned K;
    static constexpr int kKpt = 16, kPasses = 4;
    static ND_D K load(const float *p, int descending) {
        const K b = __float_as_uint(*p);
        const K k = b ^ ((b >> 31) ? 0xffffffffu : 0x80000000u);
        return descending ? ~k : k;
    }
    static ND_D void store(float *p, K k, int descending) {
        if (descending) k = ~k;
        *p = __uint_as_float(k ^ ((k >> 31) ? 0x80000000u : 0xffffffffu));
    }
};
template <> struct RadixKey<double> {
    typedef unsigned long long K;
    static constexpr int kKpt = 8, kPasses = 8;
    static ND_D K load(const double *p, int descending) {
        const K b = (K) __double_as_longlong(*p);
        const K k = b ^ ((b >> 63) ? 0xffffffffffffffffull : 0x8000000000000000ull);
        return descending ? ~k : k;
    }
    static ND_D void store(double *p, K k, int descending) {
        if (descending) k = ~k;
        *p = __longlong_as_double((long long) (k ^ ((k >> 63) ? 0x8000000000000000ull : 0xffffffffffffffffull)));
    }
};
template <> struct RadixKey<__half> {
    typedef unsigned short K;
    static constexpr int kKpt = 16, kPasses = 2;
    static ND_D K load(const __half *p, int descending) {
        const K b = __half_as_ushort(*p);
        const K k = (K) (b ^ ((b >> 15) ? 0xffffu : 0x8000u));
        return descending ? (K) ~k : k;
    }
    static ND_D void store(__half *p, K k, int descending) {
        if (descending) k = (K) ~k;
        *p = __ushort_as_half((K) (k ^ ((k >> 15) ? 0x8000u : 0xffffu)));
    }
};

struct RadixArgs {
    const void *in;      // pass 0: the array's own values; later passes: keys
    void *out;           // last pass: values; earlier passes: keys
    unsigned *hist;      // [kRadixBins][tiles]: keys of tile t with digit d; after the scan, their exclusive prefix over t
    unsigned *totals;    // [kRadixBins]: keys with digit d in the whole array
    LL n;
    LL tiles;
    int shift;           // bit position of this pass's digit
    int descending;
};

template <class T, bool RAW> ND_D typename RadixKey<T>::K radix_read(const void *base, LL i, int descending) {
    typedef typename RadixKey<T>::K K;
    if (RAW) return RadixKey<T>::load(static_cast<const T *>(base) + i, descending);
    return static_cast<const K *>(base)[i];
}

// Step 1: hist[d][tile] = number of keys of the tile whose digit is d.
template <class T, bool IN_RAW>
__global__ void __launch_bounds__(kRadixThreads) k_radix_histogram(const RadixArgs a) {
    grid_dependency_sync();
    constexpr int KPT = RadixKey<T>::kKpt;
    __shared__ unsigned bins[kRadixWarps][kRadixBins];
    for (LL tile = blockIdx.x; tile < a.tiles; tile += gridDim.x) {
        for (int i = threadIdx.x; i < kRadixWarps * kRadixBins; i += kRadixThreads) (&bins[0][0])[i] = 0;
        __syncthreads();
        const int warp = threadIdx.x >> 5;
        const LL base = tile * (LL) (kRadixThreads * KPT);
#pragma unroll
        for (int r = 0; r < KPT; r++) {
            const LL i = base + (LL) r * kRadixThreads + threadIdx.x;     // any order serves a histogram
            if (i < a.n) atomicAdd(&bins[warp][(unsigned) (radix_read<T, IN_RAW>(a.in, i, a.descending) >> a.shift) & 0xffu], 1u);
        }
        __syncthreads();
        for (int d = threadIdx.x; d < kRadixBins; d += kRadixThreads) {
            unsigned s = 0;
#pragma unroll
            for (int w = 0; w < kRadixWarps; w++) s += bins[w][d];
            a.hist[(LL) d * a.tiles + tile] = s;
        }
        __syncthreads();
    }
}

// Step 2: one CTA per digit turns hist[d][*] into its exclusive prefix over the tiles and records the total.
__global__ void __launch_bounds__(kRadixThreads) k_radix_scan(const RadixArgs a) {
    grid_dependency_sync();
    __shared__ unsigned partial[kRadixThreads];
    const int d = blockIdx.x;
    unsigned *row = a.hist + (LL) d * a.tiles;
    const LL per = (a.tiles + kRadixThreads - 1) / kRadixThreads;
    const LL lo = (LL) threadIdx.x * per;
    LL hi = lo + per;
    if (hi > a.tiles) hi = a.tiles;
    unsigned s = 0;
    for (LL t = lo; t < hi; t++) s += row[t];
    partial[threadIdx.x] = s;
    __syncthreads();
    // exclusive scan of the per-thread sums (Hillis-Steele over 256 entries)
    unsigned mine = s;
    for (int off = 1; off < kRadixThreads; off <<= 1) {
        const unsigned add = threadIdx.x >= off ? partial[threadIdx.x - off] : 0u;
        __syncthreads();
        partial[threadIdx.x] += add;
        __syncthreads();
    }
    unsigned run = partial[threadIdx.x] - mine;
    if (threadIdx.x == kRadixThreads - 1) a.totals[d] = partial[threadIdx.x];
    for (LL t = lo; t < hi; t++) { const unsigned c = row[t]; row[t] = run; run += c; }
}

// Step 3: stable scatter of every tile.
template <class T, bool IN_RAW, bool OUT_RAW>
__global__ void __launch_bounds__(kRadixThreads) k_radix_scatter(const RadixArgs a) {
    grid_dependency_sync();
    typedef typename RadixKey<T>::K K;
    constexpr int KPT = RadixKey<T>::kKpt;
    constexpr int TILE = kRadixThreads * KPT;
    __shared__ K keys[TILE];
    __shared__ unsigned cnt[kRadixWarps][kRadixBins];
    __shared__ unsigned tileBase[kRadixBins];      // first tile-local position of digit d
    __shared__ unsigned digitBase[kRadixBins];     // first position of digit d in the whole array
    __shared__ unsigned scan[kRadixThreads];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const unsigned below = (1u << lane) - 1u;

    // first position of every digit in the whole array: exclusive scan of the totals (256 entries, one per thread)
    {
        const unsigned t = a.totals[threadIdx.x];
        scan[threadIdx.x] = t;
        __syncthreads();
        for (int off = 1; off < kRadixThreads; off <<= 1) {
            const unsigned add = threadIdx.x >= off ? scan[threadIdx.x - off] : 0u;
            __syncthreads();
            scan[threadIdx.x] += add;
            __syncthreads();
        }
        digitBase[threadIdx.x] = scan[threadIdx.x] - t;
        __syncthreads();
    }

    for (LL tile = blockIdx.x; tile < a.tiles; tile += gridDim.x) {
        for (int i = threadIdx.x; i < kRadixWarps * kRadixBins; i += kRadixThreads) (&cnt[0][0])[i] = 0;
        __syncthreads();
        const LL base = tile * (LL) TILE + (LL) warp * (32 * KPT);
        K key[KPT];
        unsigned short rank[KPT];
        // ranks among the warp's keys of equal digit, earlier rounds first, lower lanes first
#pragma unroll
        for (int r = 0; r < KPT; r++) {
            const LL i = base + r * 32 + lane;
            const bool valid = i < a.n;
            key[r] = valid ? radix_read<T, IN_RAW>(a.in, i, a.descending) : K(0);
            const unsigned d = valid ? ((unsigned) (key[r] >> a.shift) & 0xffu) : 256u;
            const unsigned peers = __match_any_sync(0xffffffffu, d);
            unsigned before = 0;
            if (valid) before = cnt[warp][d];
            __syncwarp();
            if (valid && (peers & below) == 0) cnt[warp][d] = before + __popc(peers);   // lowest lane of the group
            __syncwarp();
            rank[r] = (unsigned short) (before + __popc(peers & below));
        }
        __syncthreads();
        // per digit: exclusive prefix over the warps, and the tile's histogram
        {
            const int d = threadIdx.x;
            unsigned run = 0;
#pragma unroll
            for (int w = 0; w < kRadixWarps; w++) { const unsigned c = cnt[w][d]; cnt[w][d] = run; run += c; }
            scan[d] = run;
            __syncthreads();
            for (int off = 1; off < kRadixThreads; off <<= 1) {
                const unsigned add = d >= off ? scan[d - off] : 0u;
                __syncthreads();
                scan[d] += add;
                __syncthreads();
            }
            tileBase[d] = scan[d] - run;
            __syncthreads();
        }
        LL left = a.n - tile * (LL) TILE;
        const int count = left < TILE ? (int) left : TILE;
#pragma unroll
        for (int r = 0; r < KPT; r++) {
            const LL i = base + r * 32 + lane;
            if (i < a.n) {
                const unsigned d = (unsigned) (key[r] >> a.shift) & 0xffu;
                keys[tileBase[d] + cnt[warp][d] + rank[r]] = key[r];
            }
        }
        __syncthreads();
        for (int i = threadIdx.x; i < count; i += kRadixThreads) {
            const K k = keys[i];
            const unsigned d = (unsigned) (k >> a.shift) & 0xffu;
            const LL pos = (LL) digitBase[d] + a.hist[(LL) d * a.tiles + tile] + ((unsigned) i - tileBase[d]);
            if (OUT_RAW) RadixKey<T>::store(static_cast<T *>(a.out) + pos, k, a.descending);
            else static_cast<K *>(a.out)[pos] = k;
        }
        __syncthreads();
    }
}

// Sorts the dense array x[0 .. n) in place. `scratch` holds n keys plus the histogram table.
template <class T>
Status run_radix_sort(T *x, LL n, int descending, cudaStream_t st) {
    typedef typename RadixKey<T>::K K;
    constexpr int KPT = RadixKey<T>::kKpt, PASSES = RadixKey<T>::kPasses;
    constexpr LL TILE = (LL) kRadixThreads * KPT;
    if (n >= (1LL << 32)) { set_error("sort: arrays of 2^32 or more elements are not served"); return kTooLarge; }
    RadixArgs a;
    a.n = n; a.tiles = ceil_div(n, TILE); a.descending = descending;
    const size_t keyBytes = ((size_t) n * sizeof(K) + 255) / 256 * 256;
    const size_t histBytes = (size_t) kRadixBins * a.tiles * sizeof(unsigned);
    void *ws = nullptr;
    ND_TRY(workspace(st, kWorkspaceScratch + keyBytes + histBytes + kRadixBins * sizeof(unsigned), &ws, nullptr));
    char *scratch = static_cast<char *>(ws) + kWorkspaceScratch;
    K *tmp = reinterpret_cast<K *>(scratch);
    a.hist = reinterpret_cast<unsigned *>(scratch + keyBytes);
    a.totals = a.hist + (size_t) kRadixBins * a.tiles;
    LL blocks = a.tiles;
    const LL cap = (LL) kNumSMs * 32;
    if (blocks > cap) blocks = cap;
    // ping-pong x -> tmp -> x ...; the number of passes is even, so the last one lands in x
    for (int p = 0; p < PASSES; p++) {
        a.shift = 8 * p;
        a.in = (p & 1) ? static_cast<const void *>(tmp) : static_cast<const void *>(x);
        a.out = (p & 1) ? static_cast<void *>(x) : static_cast<void *>(tmp);
        const bool first = p == 0, last = p == PASSES - 1;
        if (first) launch_kernel(k_radix_histogram<T, true>, dim3((unsigned) blocks), dim3(kRadixThreads), st, a);
        else launch_kernel(k_radix_histogram<T, false>, dim3((unsigned) blocks), dim3(kRadixThreads), st, a);
        launch_kernel(k_radix_scan, dim3(kRadixBins), dim3(kRadixThreads), st, a);
        if (first) launch_kernel(k_radix_scatter<T, true, false>, dim3((unsigned) blocks), dim3(kRadixThreads), st, a);
        else if (last) launch_kernel(k_radix_scatter<T, false, true>, dim3((unsigned) blocks), dim3(kRadixThreads), st, a);
        else launch_kernel(k_radix_scatter<T, false, false>, dim3((unsigned) blocks), dim3(kRadixThreads), st, a);
    }
    ND_CUDA(cudaGetLastError());
    return kOk;
}

}  // namespace nd4jb200
