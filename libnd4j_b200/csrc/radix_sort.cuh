// Least-significant-digit radix sort for one long dense array: 8-bit digits, so 4 passes for float, 8 for double
// and 2 for half keys, each pass four launches (tile histograms, two-level scan of them over the tiles, stable scatter).
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
// Ranks among equal digits come from warp ballots plus a per-warp counter table in shared memory; keys are
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
    unsigned *hist;      // [tiles][kRadixBins]: keys of tile t with digit d; after the chunk scan, their exclusive
                         // prefix over the tiles of the same chunk
    unsigned *chunks;    // [numChunks][kRadixBins]: keys with digit d in chunk c; after the top scan, their exclusive
                         // prefix over the chunks
    unsigned *digitBase; // [kRadixBins]: first output position of digit d (written by the top scan)
    LL n;
    LL tiles;
    LL chunkTiles;       // tiles per chunk
    LL numChunks;
    int shift;           // bit position of this pass's digit
    int descending;
};

template <class T, bool RAW> ND_D typename RadixKey<T>::K radix_read(const void *base, LL i, int descending) {
    typedef typename RadixKey<T>::K K;
    if (RAW) return RadixKey<T>::load(static_cast<const T *>(base) + i, descending);
    return static_cast<const K *>(base)[i];
}

// Exclusive prefix sum over the CTA's 256 threads (one value each): shuffles inside a warp, one shared-memory round
// across the 8 warps. `warpSums` is 8 words of shared memory that no other code uses around the call.
ND_D unsigned radix_block_scan(unsigned v, unsigned *warpSums) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    unsigned inc = v;
#pragma unroll
    for (int off = 1; off < 32; off <<= 1) {
        const unsigned t = __shfl_up_sync(0xffffffffu, inc, off);
        if (lane >= off) inc += t;
    }
    if (lane == 31) warpSums[warp] = inc;
    __syncthreads();
    unsigned before = 0;
#pragma unroll
    for (int w = 0; w < kRadixWarps; w++) before += w < warp ? warpSums[w] : 0u;
    __syncthreads();
    return before + inc - v;
}

// Step 1: hist[tile][d] = number of keys of the tile whose digit is d.
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
        typename RadixKey<T>::K key[KPT];
#pragma unroll
        for (int r = 0; r < KPT; r++) {
            const LL i = base + (LL) r * kRadixThreads + threadIdx.x;     // any order serves a histogram
            key[r] = i < a.n ? radix_read<T, IN_RAW>(a.in, i, a.descending) : typename RadixKey<T>::K(0);
        }
#pragma unroll
        for (int r = 0; r < KPT; r++) {
            const LL i = base + (LL) r * kRadixThreads + threadIdx.x;
            if (i < a.n) atomicAdd(&bins[warp][(unsigned) (key[r] >> a.shift) & 0xffu], 1u);
        }
        __syncthreads();
        unsigned s = 0;
#pragma unroll
        for (int w = 0; w < kRadixWarps; w++) s += bins[w][threadIdx.x];
        a.hist[tile * kRadixBins + threadIdx.x] = s;
        __syncthreads();
    }
}

// Step 2a: one CTA per chunk of tiles, thread d: exclusive prefix of hist[*][d] over the chunk's tiles (in place)
// and the chunk's total.
__global__ void __launch_bounds__(kRadixThreads) k_radix_scan_chunks(const RadixArgs a) {
    grid_dependency_sync();
    const LL chunk = blockIdx.x;
    const LL t0 = chunk * a.chunkTiles;
    LL t1 = t0 + a.chunkTiles;
    if (t1 > a.tiles) t1 = a.tiles;
    unsigned *col = a.hist + threadIdx.x;
    unsigned run = 0;
    LL t = t0;
    for (; t + 8 <= t1; t += 8) {
        unsigned c[8];
#pragma unroll
        for (int u = 0; u < 8; u++) c[u] = col[(t + u) * kRadixBins];
#pragma unroll
        for (int u = 0; u < 8; u++) { col[(t + u) * kRadixBins] = run; run += c[u]; }
    }
    for (; t < t1; t++) { const unsigned c = col[t * kRadixBins]; col[t * kRadixBins] = run; run += c; }
    a.chunks[chunk * kRadixBins + threadIdx.x] = run;
}

// Step 2b: one CTA, thread d: exclusive prefix of chunks[*][d] over the chunks (in place), then the first output
// position of every digit.
__global__ void __launch_bounds__(kRadixThreads) k_radix_scan_top(const RadixArgs a) {
    grid_dependency_sync();
    __shared__ unsigned warpSums[kRadixWarps];
    unsigned *col = a.chunks + threadIdx.x;
    unsigned run = 0;
    for (LL c = 0; c < a.numChunks; c++) { const unsigned v = col[c * kRadixBins]; col[c * kRadixBins] = run; run += v; }
    a.digitBase[threadIdx.x] = radix_block_scan(run, warpSums);
}

// Step 3: stable scatter of every tile. The kernel is bound by instruction issue (about a hundred instructions per
// key, half of them the ballots), so the common case, a full tile, is compiled without any bounds checks and all
// tile-local arithmetic is 32-bit.
template <class T, bool IN_RAW, bool FULL, class K, int KPT>
ND_D void radix_rank_tile(const RadixArgs &a, const void *in, LL base, int live, K (&key)[KPT], unsigned (&rank)[KPT],
                          unsigned (*cnt)[kRadixBins], int warp, int lane) {
    const unsigned below = (1u << lane) - 1u;
#pragma unroll
    for (int r = 0; r < KPT; r++) {                       // all loads in flight before any ranking
        const int o = r * 32 + lane;
        key[r] = (FULL || o < live) ? radix_read<T, IN_RAW>(in, base + o, a.descending) : K(0);
    }
    // Rank among the warp's keys of equal digit, earlier rounds first, lower lanes first. The lanes that share a
    // digit are found with one ballot per digit bit (a match.any instruction serialises over the distinct values
    // of a warp, about thirty here); the lowest of them bumps the warp's counter for the digit and hands the old
    // value to the others.
#pragma unroll
    for (int r = 0; r < KPT; r++) {
        const bool valid = FULL || r * 32 + lane < live;
        const unsigned d = (unsigned) (key[r] >> a.shift) & 0xffu;
        unsigned peers = FULL ? 0xffffffffu : __ballot_sync(0xffffffffu, valid);
#pragma unroll
        for (int b = 0; b < 8; b++) {
            const bool bit = (d >> b) & 1u;
            const unsigned has = __ballot_sync(0xffffffffu, bit);
            peers &= bit ? has : ~has;
        }
        const int leader = FULL ? __ffs(peers) - 1 : max(__ffs(peers) - 1, 0);
        unsigned before = 0;
        if (valid && lane == leader) before = atomicAdd(&cnt[warp][d], (unsigned) __popc(peers));
        before = __shfl_sync(0xffffffffu, before, leader);
        rank[r] = before + __popc(peers & below);
    }
}

template <class T, bool IN_RAW, bool OUT_RAW>
__global__ void __launch_bounds__(kRadixThreads, 3) k_radix_scatter(const RadixArgs a) {
    grid_dependency_sync();
    typedef typename RadixKey<T>::K K;
    constexpr int KPT = RadixKey<T>::kKpt;
    constexpr int TILE = kRadixThreads * KPT;
    __shared__ K keys[TILE];
    __shared__ unsigned cnt[kRadixWarps][kRadixBins];   // per warp and digit: keys counted so far, then (after the scan)
                                                        // the tile-local position of the warp's first key of the digit
    __shared__ unsigned tileBase[kRadixBins];           // first tile-local position of digit d
    __shared__ LL outBase[kRadixBins];                  // output position of tile-local position 0 of digit d's run
    __shared__ unsigned warpSums[kRadixWarps];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    for (LL tile = blockIdx.x; tile < a.tiles; tile += gridDim.x) {
        for (int i = threadIdx.x; i < kRadixWarps * kRadixBins; i += kRadixThreads) (&cnt[0][0])[i] = 0;
        __syncthreads();
        const LL tileStart = tile * (LL) TILE;
        const LL left = a.n - tileStart;
        const int count = left < TILE ? (int) left : TILE;
        const LL base = tileStart + warp * (32 * KPT);
        const int live = count - warp * (32 * KPT);       // keys of this warp's run that exist
        K key[KPT];
        unsigned rank[KPT];
        if (count == TILE) radix_rank_tile<T, IN_RAW, true>(a, a.in, base, live, key, rank, cnt, warp, lane);
        else radix_rank_tile<T, IN_RAW, false>(a, a.in, base, live, key, rank, cnt, warp, lane);
        __syncthreads();
        // per digit: exclusive prefix over the warps, the tile's histogram, and where the digit's run goes
        {
            const int d = threadIdx.x;
            unsigned c[kRadixWarps], run = 0;
#pragma unroll
            for (int w = 0; w < kRadixWarps; w++) { c[w] = run; run += cnt[w][d]; }
            const unsigned first = radix_block_scan(run, warpSums);
#pragma unroll
            for (int w = 0; w < kRadixWarps; w++) cnt[w][d] = first + c[w];
            tileBase[d] = first;
            outBase[d] = (LL) a.digitBase[d] + a.chunks[(tile / a.chunkTiles) * kRadixBins + d] + a.hist[tile * kRadixBins + d] - first;
            __syncthreads();
        }
#pragma unroll
        for (int r = 0; r < KPT; r++) {
            if (count == TILE || r * 32 + lane < live) {
                const unsigned d = (unsigned) (key[r] >> a.shift) & 0xffu;
                keys[cnt[warp][d] + rank[r]] = key[r];
            }
        }
        __syncthreads();
        for (int i = threadIdx.x; i < count; i += kRadixThreads) {
            const K k = keys[i];
            const unsigned d = (unsigned) (k >> a.shift) & 0xffu;
            const LL pos = outBase[d] + i;
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
    // chunks of at least 64 tiles, and at most 1024 chunks for the single CTA of the top scan
    a.chunkTiles = 64;
    if (ceil_div(a.tiles, a.chunkTiles) > 1024) a.chunkTiles = ceil_div(a.tiles, 1024);
    a.numChunks = ceil_div(a.tiles, a.chunkTiles);
    const size_t histBytes = (size_t) kRadixBins * a.tiles * sizeof(unsigned);
    const size_t chunkBytes = (size_t) kRadixBins * a.numChunks * sizeof(unsigned);
    void *ws = nullptr;
    ND_TRY(workspace(st, kWorkspaceScratch + keyBytes + histBytes + chunkBytes + kRadixBins * sizeof(unsigned), &ws, nullptr));
    char *scratch = static_cast<char *>(ws) + kWorkspaceScratch;
    K *tmp = reinterpret_cast<K *>(scratch);
    a.hist = reinterpret_cast<unsigned *>(scratch + keyBytes);
    a.chunks = a.hist + (size_t) kRadixBins * a.tiles;
    a.digitBase = a.chunks + (size_t) kRadixBins * a.numChunks;
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
        launch_kernel(k_radix_scan_chunks, dim3((unsigned) a.numChunks), dim3(kRadixThreads), st, a);
        launch_kernel(k_radix_scan_top, dim3(1), dim3(kRadixThreads), st, a);
        if (first) launch_kernel(k_radix_scatter<T, true, false>, dim3((unsigned) blocks), dim3(kRadixThreads), st, a);
        else if (last) launch_kernel(k_radix_scatter<T, false, true>, dim3((unsigned) blocks), dim3(kRadixThreads), st, a);
        else launch_kernel(k_radix_scatter<T, false, false>, dim3((unsigned) blocks), dim3(kRadixThreads), st, a);
    }
    ND_CUDA(cudaGetLastError());
    return kOk;
}

}  // namespace nd4jb200
