// Least-significant-digit radix sort for one long dense array: 8-bit digits, so 4 passes for float, 8 for double
// and 2 for half keys, each pass four launches (tile histograms, two-level scan of them over the tiles, stable
// scatter). The bitonic network of sort_ops.cu needs log2(n)^2 / 2 compare steps per
// key, 45 sweeps of the array for 2^24 keys; this needs 3 sweeps per pass whatever n is. The reference sorts with
// a quicksort on the host (include/ops/impl/specials.cpp:457-564); the sorted sequence is the same.
//
// Keys: the IEEE bit pattern made order-preserving as an unsigned integer (negative values inverted, the sign
// bit of the others set; all bits inverted again for a descending sort). That is the total order the network
// uses too: -0 before +0, NaNs at the two ends by their sign. The first pass reads the array's own values and
// the last pass writes them back, so that the data moves 2 x passes times, never more.
//
// A tile of kRadixThreads * KPT consecutive keys is owned by one CTA, warp w holding a contiguous run and
// lane l of round r the key at run offset r * 32 + l, so "earlier key" means "lower (warp, round, lane)".
// Ranks among equal digits come from the set of lanes that hold the digit (found by warp ballots in one half of
// the rounds and through a word of shared memory in the other half) plus a per-warp counter table in shared
// memory; keys are first placed at their tile-local sorted position in shared memory and then written out in that
// order, which turns the scatter into runs of (on average) tile / 256 consecutive keys per digit.
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
    int descending;
};

template <class T, bool RAW> ND_D typename RadixKey<T>::K radix_read(const void *base, LL i, int descending) {
    typedef typename RadixKey<T>::K K;
    if (RAW) return RadixKey<T>::load(static_cast<const T *>(base) + i, descending);
    return static_cast<const K *>(base)[i];
}

template <int PASS, class K> ND_D unsigned radix_digit(K key) { return (unsigned) (key >> (8 * PASS)) & 0xffu; }

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
template <class T, int PASS>
__global__ void __launch_bounds__(kRadixThreads) k_radix_histogram(const RadixArgs a) {
    grid_dependency_sync();
    constexpr int KPT = RadixKey<T>::kKpt;
    typedef typename RadixKey<T>::K K;
    __shared__ unsigned bins[kRadixWarps][kRadixBins];
    for (LL tile = blockIdx.x; tile < a.tiles; tile += gridDim.x) {
        for (int i = threadIdx.x; i < kRadixWarps * kRadixBins; i += kRadixThreads) (&bins[0][0])[i] = 0;
        __syncthreads();
        const int warp = threadIdx.x >> 5;
        const LL base = tile * (LL) (kRadixThreads * KPT);
        K key[KPT];
#pragma unroll
        for (int r = 0; r < KPT; r++) {
            const LL i = base + (LL) r * kRadixThreads + threadIdx.x;     // any order serves a histogram
            key[r] = i < a.n ? radix_read<T, PASS == 0>(a.in, i, a.descending) : K(0);
        }
#pragma unroll
        for (int r = 0; r < KPT; r++) {
            const LL i = base + (LL) r * kRadixThreads + threadIdx.x;
            if (i < a.n) atomicAdd(&bins[warp][radix_digit<PASS>(key[r])], 1u);
        }
        __syncthreads();
        unsigned s = 0;
#pragma unroll
        for (int w = 0; w < kRadixWarps; w++) s += bins[w][threadIdx.x];
        a.hist[tile * kRadixBins + threadIdx.x] = s;
        __syncthreads();
    }
}

// Thread d: exclusive prefix of col[0], col[stride], ... (count entries, in place); returns their sum.
ND_D unsigned radix_scan_column(unsigned *col, LL count, LL stride) {
    unsigned run = 0;
    LL t = 0;
    for (; t + 16 <= count; t += 16) {                       // 16 independent loads per round trip to L2
        unsigned c[16];
#pragma unroll
        for (int u = 0; u < 16; u++) c[u] = col[(t + u) * stride];
#pragma unroll
        for (int u = 0; u < 16; u++) { col[(t + u) * stride] = run; run += c[u]; }
    }
    for (; t < count; t++) { const unsigned c = col[t * stride]; col[t * stride] = run; run += c; }
    return run;
}

// Step 2a: one CTA per chunk of tiles, thread d: exclusive prefix of hist[*][d] over the chunk's tiles (in place)
// and the chunk's total.
__global__ void __launch_bounds__(kRadixThreads) k_radix_scan_chunks(const RadixArgs a) {
    grid_dependency_sync();
    const LL first = blockIdx.x * a.chunkTiles;
    const LL inChunk = a.tiles - first < a.chunkTiles ? a.tiles - first : a.chunkTiles;
    a.chunks[blockIdx.x * kRadixBins + threadIdx.x] = radix_scan_column(a.hist + first * kRadixBins + threadIdx.x, inChunk, kRadixBins);
}

// Step 2b: one CTA, thread d: exclusive prefix of chunks[*][d] over the chunks (in place), then the first output
// position of every digit.
__global__ void __launch_bounds__(kRadixThreads) k_radix_scan_top(const RadixArgs a) {
    grid_dependency_sync();
    __shared__ unsigned warpSums[kRadixWarps];
    const unsigned total = radix_scan_column(a.chunks + threadIdx.x, a.numChunks, kRadixBins);
    a.digitBase[threadIdx.x] = radix_block_scan(total, warpSums);
}

// Rank of each of the warp's keys among the warp's keys of equal digit, earlier rounds first, lower lanes first.
// A round needs, for every lane, the set of lanes that hold the same digit. Even rounds find it with one ballot
// per digit bit (a match.any instruction serialises over the distinct values of a warp, about thirty here), which
// costs instruction issue (some forty instructions per key); odd rounds let the lanes set their bit in a word of
// shared memory per digit, which costs the shared-memory pipe instead (five accesses at random digits, each about
// three bank-conflict wavefronts). All ballots: 99 instructions per key and 78 us per pass for 2^24 keys; all
// shared words: 55 instructions but 29 wavefronts per warp and round, also 78 us; alternating: 70 us. The lowest
// lane of a set adds the set's size to the warp's running count of the digit. The common case, a full tile, is
// compiled without bounds checks and all tile-local arithmetic is 32-bit.
template <class T, int PASS, bool FULL, class K, int KPT>
ND_D void radix_rank_tile(const RadixArgs &a, LL base, int live, K (&key)[KPT], unsigned (&rank)[KPT], unsigned *cnt,
                          unsigned *match, int lane) {
    const unsigned below = (1u << lane) - 1u;
#pragma unroll
    for (int r = 0; r < KPT; r++) {                       // all loads in flight before any ranking
        const int o = r * 32 + lane;
        key[r] = (FULL || o < live) ? radix_read<T, PASS == 0>(a.in, base + o, a.descending) : K(0);
    }
#pragma unroll
    for (int r = 0; r < KPT; r++) {
        const bool valid = FULL || r * 32 + lane < live;
        const unsigned d = radix_digit<PASS>(key[r]);
        if (r & 1) {
            if (valid) atomicOr(&match[d], 1u << lane);
            __syncwarp();
            const unsigned peers = match[d], before = cnt[d];
            __syncwarp();
            const unsigned earlier = __popc(peers & below);
            if (valid && earlier == 0) { cnt[d] = before + __popc(peers); match[d] = 0; }
            rank[r] = before + earlier;
        } else {
            __syncwarp();                                 // the counter writes of the round before, ahead of the atomic
            unsigned peers = FULL ? 0xffffffffu : __ballot_sync(0xffffffffu, valid);
#pragma unroll
            for (int b = 0; b < 8; b++) {
                const bool bit = (d >> b) & 1u;
                const unsigned has = __ballot_sync(0xffffffffu, bit);
                peers &= bit ? has : ~has;
            }
            const int leader = FULL ? __ffs(peers) - 1 : max(__ffs(peers) - 1, 0);
            unsigned before = 0;
            if (valid && lane == leader) before = atomicAdd(&cnt[d], (unsigned) __popc(peers));
            before = __shfl_sync(0xffffffffu, before, leader);
            rank[r] = before + __popc(peers & below);
        }
    }
}

// Step 3: the stable scatter.
template <class T, int PASS>
__global__ void __launch_bounds__(kRadixThreads, 3) k_radix_scatter(const RadixArgs a) {
    grid_dependency_sync();
    typedef typename RadixKey<T>::K K;
    constexpr int KPT = RadixKey<T>::kKpt;
    constexpr int TILE = kRadixThreads * KPT;
    constexpr bool LAST = PASS == RadixKey<T>::kPasses - 1;
    __shared__ K keys[TILE];
    __shared__ unsigned cnt[kRadixWarps][kRadixBins];   // per warp and digit: keys counted so far, then (after the scan)
                                                        // the tile-local position of the warp's first key of the digit
    __shared__ unsigned match[kRadixWarps][kRadixBins]; // per warp and digit: the lanes of the round that hold it; zero
                                                        // between rounds
    __shared__ unsigned outBase[kRadixBins];            // output position of tile-local position 0, per digit (mod 2^32)
    __shared__ unsigned warpSums[kRadixWarps];
    for (int i = threadIdx.x; i < kRadixWarps * kRadixBins; i += kRadixThreads) (&match[0][0])[i] = 0;
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
        if (count == TILE) radix_rank_tile<T, PASS, true>(a, base, live, key, rank, cnt[warp], match[warp], lane);
        else radix_rank_tile<T, PASS, false>(a, base, live, key, rank, cnt[warp], match[warp], lane);
        __syncthreads();
        // per digit: exclusive prefix over the warps, the tile's count, and where the digit's run goes
        {
            const int d = threadIdx.x;
            unsigned c[kRadixWarps], run = 0;
#pragma unroll
            for (int w = 0; w < kRadixWarps; w++) { c[w] = run; run += cnt[w][d]; }
            const unsigned first = radix_block_scan(run, warpSums);
#pragma unroll
            for (int w = 0; w < kRadixWarps; w++) cnt[w][d] = first + c[w];
            outBase[d] = a.digitBase[d] + a.chunks[(tile / a.chunkTiles) * kRadixBins + d] + a.hist[tile * kRadixBins + d] - first;
            __syncthreads();
        }
#pragma unroll
        for (int r = 0; r < KPT; r++) {
            if (count == TILE || r * 32 + lane < live) keys[cnt[warp][radix_digit<PASS>(key[r])] + rank[r]] = key[r];
        }
        __syncthreads();
        if (count == TILE) {
#pragma unroll
            for (int r = 0; r < KPT; r++) {
                const unsigned i = r * kRadixThreads + threadIdx.x;
                const K k = keys[i];
                const unsigned pos = outBase[radix_digit<PASS>(k)] + i;
                if (LAST) RadixKey<T>::store(static_cast<T *>(a.out) + pos, k, a.descending);
                else static_cast<K *>(a.out)[pos] = k;
            }
        } else {
            for (unsigned i = threadIdx.x; i < (unsigned) count; i += kRadixThreads) {
                const K k = keys[i];
                const unsigned pos = outBase[radix_digit<PASS>(k)] + i;
                if (LAST) RadixKey<T>::store(static_cast<T *>(a.out) + pos, k, a.descending);
                else static_cast<K *>(a.out)[pos] = k;
            }
        }
        __syncthreads();
    }
}

template <class T, int PASS>
inline void launch_radix_passes(RadixArgs a, T *x, void *tmp, unsigned blocks, cudaStream_t st) {
    if constexpr (PASS < RadixKey<T>::kPasses) {
        // ping-pong x -> tmp -> x ...; the number of passes is even, so the last one lands in x
        a.in = (PASS & 1) ? static_cast<const void *>(tmp) : static_cast<const void *>(x);
        a.out = (PASS & 1) ? static_cast<void *>(x) : tmp;
        launch_kernel(k_radix_histogram<T, PASS>, dim3(blocks), dim3(kRadixThreads), st, a);
        launch_kernel(k_radix_scan_chunks, dim3((unsigned) a.numChunks), dim3(kRadixThreads), st, a);
        launch_kernel(k_radix_scan_top, dim3(1), dim3(kRadixThreads), st, a);
        launch_kernel(k_radix_scatter<T, PASS>, dim3(blocks), dim3(kRadixThreads), st, a);
        launch_radix_passes<T, PASS + 1>(a, x, tmp, blocks, st);
    }
}

// Sorts the dense array x[0 .. n) in place. The workspace holds n keys plus the histogram tables.
template <class T>
Status run_radix_sort(T *x, LL n, int descending, cudaStream_t st) {
    typedef typename RadixKey<T>::K K;
    constexpr int KPT = RadixKey<T>::kKpt, PASSES = RadixKey<T>::kPasses;
    constexpr LL TILE = (LL) kRadixThreads * KPT;
    static_assert(PASSES % 2 == 0, "the last pass must land in the array itself");
    if (n >= (1LL << 32)) { set_error("sort: arrays of 2^32 or more elements are not served"); return kTooLarge; }
    RadixArgs a;
    a.n = n; a.tiles = ceil_div(n, TILE); a.descending = descending;
    const size_t keyBytes = ((size_t) n * sizeof(K) + 255) / 256 * 256;
    // chunks of at least 64 tiles, and at most 1024 chunks for the single CTA of the top scan
    a.chunkTiles = 64;
    if (ceil_div(a.tiles, a.chunkTiles) > 1024) a.chunkTiles = ceil_div(a.tiles, 1024);
    a.numChunks = ceil_div(a.tiles, a.chunkTiles);
    const size_t histWords = (size_t) kRadixBins * a.tiles, chunkWords = (size_t) kRadixBins * a.numChunks;
    void *ws = nullptr;
    ND_TRY(workspace(st, kWorkspaceScratch + keyBytes + (histWords + chunkWords + kRadixBins) * sizeof(unsigned),
                     &ws, nullptr));
    char *scratch = static_cast<char *>(ws) + kWorkspaceScratch;
    void *tmp = scratch;
    a.hist = reinterpret_cast<unsigned *>(scratch + keyBytes);
    a.chunks = a.hist + histWords;
    a.digitBase = a.chunks + chunkWords;
    LL blocks = a.tiles;
    const LL cap = (LL) kNumSMs * 32;
    if (blocks > cap) blocks = cap;
    launch_radix_passes<T, 0>(a, x, tmp, (unsigned) blocks, st);
    ND_CUDA(cudaGetLastError());
    return kOk;
}

}  // namespace nd4jb200
