// Memory-movement utilities that sit on the same boundary as the legacy op families and share their
// shapeInfo / TAD decoding: flatten, concat, pullRows, and the parameter-averaging pair average /
// accumulate (NativeOps.h:1457-1601, 1904-2037). All of them are pure streams through HBM: each
// element is read once and written once, nothing is re-laid-out on the way.
//
//   flatten    z[offset + i * zEws] = element i of x walked in the requested order
//              (blas/cpu/NativeOps.cpp:1530-1700)
//   concat     the inputs are laid side by side along one axis of z (include/ops/impl/specials.cpp,
//              concatCpuGeneric): one strided block copy per input
//   pullRows   TAD number indexes[k] of x is copied onto TAD k of z (blas/cpu/NativeOps.cpp:2045-2104)
//   average    z[i] = sum_k x_k[i] / n, then (optionally) every x_k = z  (specials.cpp:374-433)
//   accumulate z[i] += sum_k x_k[i]  (onto what z already holds)          (specials.cpp:343-359)
//   convertTypes  z[i] = (D)(float) x[i] among float8 / int8 / uint8 / int16 / uint16 / float16 / float32 / double
//              (type_conversions.h:592-610, 696-880)
//   tear       TAD k of x is copied into the array targets[k]               (blas/cpu/NativeOps.cpp:2119-2162)
//   shuffle    TAD r and TAD map[r] of every array change places, r = 0, 1, ... (blas/cpu/NativeOps.cpp:2266-2326)
//
// Copies move raw 2-, 4- or 8-byte elements; only average / accumulate look at the values.
#include "../../include/nd4j_b200.h"
#include "device_utils.cuh"
#include "runtime.h"
#include <sstream>
#include <cstring>
#include <vector>

namespace nd4jb200 {
namespace {

template <int BYTES> struct Raw;
template <> struct Raw<2> { typedef unsigned short T; };
template <> struct Raw<4> { typedef unsigned int T; };
template <> struct Raw<8> { typedef unsigned long long T; };

struct CopyArgs {
    const void *x;
    void *z;
    LL n;
    int dense;        // both sides one unit-stride run, 16-byte aligned, n * size a multiple of 16
    View vx, vz;      // otherwise: linear index -> offset on either side
};

constexpr int kCopyBlock = 256;

template <int BYTES>
__global__ void __launch_bounds__(kCopyBlock) k_copy_views(const CopyArgs a) {
    grid_dependency_sync();
    typedef typename Raw<BYTES>::T E;
    const LL tid = (LL) blockIdx.x * kCopyBlock + threadIdx.x, nthreads = (LL) gridDim.x * kCopyBlock;
    if (a.dense) {
        const uint4 *src = static_cast<const uint4 *>(a.x);
        uint4 *dst = static_cast<uint4 *>(a.z);
        const LL packs = a.n * BYTES / 16;
        LL i = tid;
        for (; i + 3 * nthreads < packs; i += 4 * nthreads) {
            const uint4 p0 = src[i], p1 = src[i + nthreads], p2 = src[i + 2 * nthreads], p3 = src[i + 3 * nthreads];
            dst[i] = p0; dst[i + nthreads] = p1; dst[i + 2 * nthreads] = p2; dst[i + 3 * nthreads] = p3;
        }
        for (; i < packs; i += nthreads) dst[i] = src[i];
        return;
    }
    const E *src = static_cast<const E *>(a.x);
    E *dst = static_cast<E *>(a.z);
    for (LL i = tid; i < a.n; i += nthreads) dst[view_offset(a.vz, i)] = src[view_offset(a.vx, i)];
}

Status launch_copy(int bytes, CopyArgs a, cudaStream_t stream) {
    if (a.n <= 0) return kOk;
    LL work = a.dense ? ceil_div(a.n * bytes / 16, 4) : a.n;
    LL blocks = ceil_div(work, kCopyBlock);
    const LL cap = (LL) kNumSMs * 16;
    if (blocks > cap) blocks = cap;
    if (blocks < 1) blocks = 1;
    if (bytes == 2) launch_kernel(k_copy_views<2>, dim3((unsigned) blocks), dim3(kCopyBlock), stream, a);
    else if (bytes == 4) launch_kernel(k_copy_views<4>, dim3((unsigned) blocks), dim3(kCopyBlock), stream, a);
    else launch_kernel(k_copy_views<8>, dim3((unsigned) blocks), dim3(kCopyBlock), stream, a);
    ND_CUDA(cudaGetLastError());
    return kOk;
}

bool unit_run(const View &v) { return v.rank == 0 || (v.rank == 1 && v.stride[0] == 1); }

Status copy_between(int bytes, const void *x, const View &vx, void *z, const View &vz, LL n, cudaStream_t stream) {
    CopyArgs a;
    a.x = x; a.z = z; a.n = n; a.vx = vx; a.vz = vz;
    a.dense = unit_run(vx) && unit_run(vz) && aligned16(x) && aligned16(z) && (n * bytes) % 16 == 0;
    return launch_copy(bytes, a, stream);
}

// f-order traversal of an array: the same view with the axes reversed
Status forder_traversal(const ShapeDesc &d, View *out) {
    LL shp[kMaxRank], str[kMaxRank];
    for (int i = 0; i < d.rank; i++) { shp[i] = d.shape[d.rank - 1 - i]; str[i] = d.stride[d.rank - 1 - i]; }
    return collapse_view(d.rank, shp, str, out);
}

inline int dtype_bytes(int dtype) { return dtype == ND4JB200_DOUBLE ? 8 : (dtype == ND4JB200_FLOAT ? 4 : 2); }
inline Status check_dtype(int dtype) {
    if (dtype < 0 || dtype > 2) return bad_arg("dtype must be 0 (float), 1 (double) or 2 (half)");
    return kOk;
}
inline cudaStream_t as_stream(void *s) { return static_cast<cudaStream_t>(s); }

// ---- pullRows / tear ----------------------------------------------------------------------------
// A unit of work is one chunk of one TAD; a warp takes units grid-stride. TADs of up to kPullChunk
// bytes are one unit (a warp per TAD); longer ones are cut so that a few long TADs still fill the device.
constexpr LL kPullChunk = 16384;
struct PullArgs {
    const void *x;
    void *z;
    void *const *targets;                      // tear: TAD k goes to the array targets[k] (device array of pointers)
    LL n, tadLen, chunkLen, chunks;            // chunks per TAD, chunkLen elements each (a multiple of 16 bytes)
    const LL *indexes, *xOffsets, *zOffsets;   // device arrays; indexes == nullptr: TAD k itself
    View xInner, zInner;
    int dense;        // unit-stride TADs whose length keeps 16-byte alignment (bases are checked per TAD)
};

template <int BYTES>
__global__ void __launch_bounds__(kCopyBlock) k_pull_rows(const PullArgs a) {
    grid_dependency_sync();
    typedef typename Raw<BYTES>::T E;
    const int lane = threadIdx.x & 31;
    const LL warps = (LL) gridDim.x * (kCopyBlock / 32), units = a.n * a.chunks;
    for (LL u = (LL) blockIdx.x * (kCopyBlock / 32) + (threadIdx.x >> 5); u < units; u += warps) {
        const LL k = u / a.chunks, first = (u - k * a.chunks) * a.chunkLen;
        const LL len = min(a.chunkLen, a.tadLen - first);
        const E *src = static_cast<const E *>(a.x) + __ldg(a.xOffsets + (a.indexes ? __ldg(a.indexes + k) : k));
        E *dst = a.targets ? static_cast<E *>(a.targets[k]) : static_cast<E *>(a.z) + __ldg(a.zOffsets + k);
        const bool vec = a.dense && (reinterpret_cast<uintptr_t>(src) & 15) == 0 && (reinterpret_cast<uintptr_t>(dst) & 15) == 0;
        if (vec) {
            // four 16-byte packs in flight per lane
            const uint4 *s4 = reinterpret_cast<const uint4 *>(src + first);
            uint4 *d4 = reinterpret_cast<uint4 *>(dst + first);
            const LL packs = len * BYTES / 16;
            LL i = lane;
            for (; i + 96 < packs; i += 128) {
                const uint4 p0 = __ldg(s4 + i), p1 = __ldg(s4 + i + 32), p2 = __ldg(s4 + i + 64), p3 = __ldg(s4 + i + 96);
                d4[i] = p0; d4[i + 32] = p1; d4[i + 64] = p2; d4[i + 96] = p3;
            }
            for (; i < packs; i += 32) d4[i] = __ldg(s4 + i);
        } else {
            for (LL i = first + lane; i < first + len; i += 32)
                dst[view_offset(a.zInner, i)] = src[view_offset(a.xInner, i)];
        }
    }
}

Status launch_pull(int bytes, PullArgs a, cudaStream_t st) {
    const LL perChunk = kPullChunk / bytes;
    a.chunkLen = a.tadLen < perChunk ? a.tadLen : perChunk;
    a.chunks = ceil_div(a.tadLen, a.chunkLen);
    LL blocks = ceil_div(a.n * a.chunks, kCopyBlock / 32);
    const LL cap = (LL) kNumSMs * 16;
    if (blocks > cap) blocks = cap;
    if (bytes == 2) launch_kernel(k_pull_rows<2>, dim3((unsigned) blocks), dim3(kCopyBlock), st, a);
    else if (bytes == 4) launch_kernel(k_pull_rows<4>, dim3((unsigned) blocks), dim3(kCopyBlock), st, a);
    else launch_kernel(k_pull_rows<8>, dim3((unsigned) blocks), dim3(kCopyBlock), st, a);
    ND_CUDA(cudaGetLastError());
    return kOk;
}

// ---- shuffle -------------------------------------------------------------------------------------
// TAD pairs[p].x and TAD pairs[p].y of one array change places; the pairs of one launch are disjoint.
struct SwapArgs {
    void *x;
    const LL *offsets;        // device array of TAD offsets
    const int2 *pairs;        // device array
    LL n, tadLen, chunkLen, chunks;
    View inner;
    int dense;
};

template <int BYTES>
__global__ void __launch_bounds__(kCopyBlock) k_swap_tads(const SwapArgs a) {
    grid_dependency_sync();
    typedef typename Raw<BYTES>::T E;
    const int lane = threadIdx.x & 31;
    const LL warps = (LL) gridDim.x * (kCopyBlock / 32), units = a.n * a.chunks;
    for (LL u = (LL) blockIdx.x * (kCopyBlock / 32) + (threadIdx.x >> 5); u < units; u += warps) {
        const LL k = u / a.chunks, first = (u - k * a.chunks) * a.chunkLen;
        const LL len = min(a.chunkLen, a.tadLen - first);
        const int2 pr = a.pairs[k];
        E *p = static_cast<E *>(a.x) + __ldg(a.offsets + pr.x);
        E *q = static_cast<E *>(a.x) + __ldg(a.offsets + pr.y);
        const bool vec = a.dense && (reinterpret_cast<uintptr_t>(p) & 15) == 0 && (reinterpret_cast<uintptr_t>(q) & 15) == 0;
        if (vec) {
            uint4 *p4 = reinterpret_cast<uint4 *>(p + first), *q4 = reinterpret_cast<uint4 *>(q + first);
            const LL packs = len * BYTES / 16;
            LL i = lane;
            for (; i + 32 < packs; i += 64) {
                const uint4 a0 = p4[i], a1 = p4[i + 32], b0 = q4[i], b1 = q4[i + 32];
                p4[i] = b0; p4[i + 32] = b1; q4[i] = a0; q4[i + 32] = a1;
            }
            for (; i < packs; i += 32) { const uint4 a0 = p4[i], b0 = q4[i]; p4[i] = b0; q4[i] = a0; }
        } else {
            for (LL i = first + lane; i < first + len; i += 32) {
                const LL o = view_offset(a.inner, i);
                const E t = p[o]; p[o] = q[o]; q[o] = t;
            }
        }
    }
}

// The reference applies the swaps one after another (r = 0, 1, ...; blas/cpu/NativeOps.cpp:2289-2324), so a
// map whose swaps share TADs depends on that order. The swaps are sorted into rounds: a swap goes one round
// after the latest earlier swap that touches either of its TADs. The swaps of a round are disjoint and run
// as one launch; the usual map (disjoint pairs) is a single round.
// `flat` receives the swaps grouped by round (in map order inside a round), `counts` the swaps per round.
Status shuffle_rounds(const int *map, LL numTads, std::vector<int2> *flat, std::vector<size_t> *counts) {
    std::vector<int> last((size_t) numTads, 0), roundOf;
    std::vector<int2> swaps;
    swaps.reserve((size_t) numTads);
    roundOf.reserve((size_t) numTads);
    int rounds = 0;
    for (LL r = 0; r < numTads; r++) {
        const int m = map[r];
        if (m < 0 || m == r) continue;
        if (m >= numTads) return bad_arg("shuffle: the map names a TAD past the last one");
        const int round = (last[r] > last[m] ? last[r] : last[m]) + 1;
        last[r] = last[m] = round;
        if (round > rounds) rounds = round;
        swaps.push_back(make_int2((int) r, m));
        roundOf.push_back(round);
    }
    counts->assign((size_t) rounds, 0);
    if (rounds <= 1) {          // the usual map: disjoint pairs, one launch
        if (rounds == 1) (*counts)[0] = swaps.size();
        flat->swap(swaps);
        return kOk;
    }
    for (size_t i = 0; i < swaps.size(); i++) (*counts)[roundOf[i] - 1]++;
    std::vector<size_t> at((size_t) rounds, 0);
    for (int k = 1; k < rounds; k++) at[k] = at[k - 1] + (*counts)[k - 1];
    flat->resize(swaps.size());
    for (size_t i = 0; i < swaps.size(); i++) (*flat)[at[roundOf[i] - 1]++] = swaps[i];
    return kOk;
}

// ---- average / accumulate -----------------------------------------------------------------------
constexpr int kMaxSources = 128;
struct SumArgs {
    const void *src[kMaxSources];
    void *z;
    int n;
    LL length;
    int average;      // divide every term by n (the reference divides before adding)
    int propagate;    // write the result back over every source
};

// Terms are added in source order and every intermediate is rounded to the element type, as the
// reference's loop over T does; x / n is taken as x * (1 / n), which is what the reference's
// reciprocal-math build makes of it.
template <class T> ND_D typename Elem<T>::C sum_term(const SumArgs &a, typename Elem<T>::C acc, typename Elem<T>::C v,
                                                      typename Elem<T>::C inv) {
    if (a.average) v = Elem<T>::to_c(Elem<T>::from_c(v * inv));
    return Elem<T>::to_c(Elem<T>::from_c(acc + v));
}

template <class T, bool VEC>
__global__ void __launch_bounds__(kCopyBlock) k_sum_sources(const SumArgs a) {
    grid_dependency_sync();
    typedef typename Elem<T>::C C;
    constexpr int V = Elem<T>::kVec;
    T *az = static_cast<T *>(a.z);
    const C inv = C(1) / C(a.n);
    const LL tid = (LL) blockIdx.x * kCopyBlock + threadIdx.x, nthreads = (LL) gridDim.x * kCopyBlock;
    if (VEC) {
        // 16-byte packs; the loads of all sources for a pack are independent of each other
        const LL packs = a.length / V;
        for (LL i = tid; i < packs; i += nthreads) {
            C acc[V];
            if (a.average) {
#pragma unroll
                for (int j = 0; j < V; j++) acc[j] = C(0);
            } else {
                const Pack<T> pz = load_pack_rw(az + i * V);     // accumulate adds onto what z holds
#pragma unroll
                for (int j = 0; j < V; j++) acc[j] = Elem<T>::to_c(pz.v[j]);
            }
#pragma unroll 4
            for (int k = 0; k < a.n; k++) {
                const Pack<T> p = load_pack_rw(static_cast<const T *>(a.src[k]) + i * V);
#pragma unroll
                for (int j = 0; j < V; j++) acc[j] = sum_term<T>(a, acc[j], Elem<T>::to_c(p.v[j]), inv);
            }
            Pack<T> o;
#pragma unroll
            for (int j = 0; j < V; j++) o.v[j] = Elem<T>::from_c(acc[j]);
            store_pack(az + i * V, o);
            if (a.propagate)
                for (int k = 0; k < a.n; k++) store_pack(static_cast<T *>(const_cast<void *>(a.src[k])) + i * V, o);
        }
        return;
    }
    for (LL i = tid; i < a.length; i += nthreads) {
        C acc = a.average ? C(0) : Elem<T>::to_c(az[i]);
        for (int k = 0; k < a.n; k++) acc = sum_term<T>(a, acc, Elem<T>::to_c(static_cast<const T *>(a.src[k])[i]), inv);
        az[i] = Elem<T>::from_c(acc);
        if (a.propagate)
            for (int k = 0; k < a.n; k++) static_cast<T *>(const_cast<void *>(a.src[k]))[i] = Elem<T>::from_c(acc);
    }
}

Status sum_sources(void *stream, int dtype, const void *const *sources, void *z, int n, LL length, bool average, bool propagate) {
    ND_TRY(check_dtype(dtype));
    if (!sources) return bad_arg("null source pointer array");
    if (n < 1 || n > kMaxSources) {
        set_error("average / accumulate take between 1 and 128 source arrays");
        return kTooLarge;
    }
    if (length < 0) return bad_arg("negative length");
    SumArgs a;
    for (int k = 0; k < n; k++) {
        if (!sources[k]) return bad_arg("null source array");
        a.src[k] = sources[k];
    }
    // without a result array the first source receives it (specials.cpp:376-378)
    a.z = z ? z : const_cast<void *>(sources[0]);
    a.n = n; a.length = length; a.average = average; a.propagate = propagate;
    if (length == 0) return kOk;
    const int vlen = dtype == ND4JB200_DOUBLE ? 2 : (dtype == ND4JB200_FLOAT ? 4 : 8);
    bool vec = length % vlen == 0 && aligned16(a.z);
    for (int k = 0; k < n; k++) vec = vec && aligned16(a.src[k]);
    LL blocks = ceil_div(vec ? length / vlen : length, kCopyBlock);
    const LL cap = (LL) kNumSMs * 16;
    if (blocks > cap) blocks = cap;
    const cudaStream_t st = as_stream(stream);
    const dim3 grid((unsigned) blocks), block(kCopyBlock);
    if (dtype == ND4JB200_FLOAT) {
        if (vec) launch_kernel(k_sum_sources<float, true>, grid, block, st, a);
        else launch_kernel(k_sum_sources<float, false>, grid, block, st, a);
    } else if (dtype == ND4JB200_DOUBLE) {
        if (vec) launch_kernel(k_sum_sources<double, true>, grid, block, st, a);
        else launch_kernel(k_sum_sources<double, false>, grid, block, st, a);
    } else {
        if (vec) launch_kernel(k_sum_sources<__half, true>, grid, block, st, a);
        else launch_kernel(k_sum_sources<__half, false>, grid, block, st, a);
    }
    ND_CUDA(cudaGetLastError());
    return kOk;
}

// ---- convertTypes ------------------------------------------------------------------------------------
// z[i] = (D) ((float) x[i]): every conversion goes through float, as the reference's convertGeneric does
// (include/loops/type_conversions.h:592-610). The 8- and 16-bit integer types are the reference's saturating
// wrappers (include/types/impl/{int8,uint8,int16,uint16}.cpp): float -> int truncates like the x86 conversion
// the reference is compiled to (anything outside int32, and NaN, gives INT_MIN) and is then clamped to the
// type's range. Its uint16 wrapper clamps to 65536 and returns the value through a uint8_t, so only the low
// byte survives; that is reproduced, not repaired.
template <int CODE> struct ConvType;
template <> struct ConvType<0> { typedef unsigned char T; };     // float8 ("quarter"): sign, 3 exponent bits, 4 mantissa bits
template <> struct ConvType<1> { typedef signed char T; };
template <> struct ConvType<2> { typedef unsigned char T; };
template <> struct ConvType<3> { typedef __half T; };
template <> struct ConvType<4> { typedef short T; };
template <> struct ConvType<5> { typedef unsigned short T; };
template <> struct ConvType<6> { typedef float T; };
template <> struct ConvType<7> { typedef double T; };

ND_D int x86_float_to_int(float v) {
    return (v >= 2147483648.0f || v < -2147483648.0f || v != v) ? (int) 0x80000000 : __float2int_rz(v);
}
ND_D int clamp_int(int t, int lo, int hi) { return t > hi ? hi : (t < lo ? lo : t); }

// float8 <-> float exactly as the reference's software routines do it (include/types/impl/float8.cpp:8-96),
// quirks included: the overflow and underflow thresholds are those of half precision (values between 15.5 and
// 65520 keep exponent bits that spill into the sign, values below 2^-14 are shifted by 0x90 - exponent, which the
// x86 shifter the reference runs on takes modulo 32). Conversions are pinned bit for bit against the reference
// on every float8 value and on a dense sweep of floats.
ND_D float float8_to_float(unsigned char b) {
    unsigned sign = (b >> 7) & 1u, exponent = (b >> 4) & 7u, mantissa = (unsigned) (b & 0xfu) << 19;
    if (exponent == 7u) {                         // infinity, or NaN (which loses its sign)
        if (mantissa) { sign = 0u; mantissa = 0x7fffffu; }
        exponent = 0xffu;
    } else if (exponent == 0u) {
        if (mantissa) {                           // subnormal: normalise
            const int up = __clz(mantissa) - 8;   // shifts until bit 23 is set
            mantissa = (mantissa << up) & 0x7fffffu;
            exponent = 0x7du - (unsigned) up;
        }
    } else {
        exponent += 0x7cu;
    }
    return __uint_as_float((sign << 31) | (exponent << 23) | mantissa);
}
ND_D unsigned char float_to_float8(float f) {
    const unsigned x = __float_as_uint(f), u = x & 0x7fffffffu;
    if (u > 0x7f800000u) return 0x7fu;                                   // NaN
    const unsigned sign = (x >> 24) & 0x80u;
    if (u > 0x477fefffu) return (unsigned char) (sign | 0x70u);           // infinity
    if (u < 0x33000001u) return (unsigned char) sign;                     // zero
    unsigned exponent = (u >> 23) & 0xffu, mantissa = u & 0x7fffffu, shift;
    if (exponent > 0x7cu) { shift = 19u; exponent -= 0x7cu; }
    else { shift = (0x90u - exponent) & 31u; exponent = 0u; mantissa |= 0x800000u; }
    const unsigned lsb = 1u << shift, half = lsb >> 1, rest = mantissa & (lsb - 1u);
    mantissa >>= shift;
    if (rest > half || (rest == half && (mantissa & 1u))) {               // round to nearest even
        ++mantissa;
        if (!(mantissa & 0xfu)) { ++exponent; mantissa = 0u; }
    }
    return (unsigned char) (sign | (exponent << 4) | mantissa);
}

template <int CODE> ND_D float as_float(typename ConvType<CODE>::T v) { return (float) (int) v; }   // the integer types
template <> ND_D float as_float<0>(unsigned char v) { return float8_to_float(v); }
template <> ND_D float as_float<3>(__half v) { return __half2float(v); }
template <> ND_D float as_float<6>(float v) { return v; }
template <> ND_D float as_float<7>(double v) { return (float) v; }

template <int CODE> ND_D typename ConvType<CODE>::T from_float(float v);
template <> ND_D unsigned char from_float<0>(float v) { return float_to_float8(v); }
template <> ND_D signed char from_float<1>(float v) { return (signed char) clamp_int(x86_float_to_int(v), -128, 127); }
template <> ND_D unsigned char from_float<2>(float v) { return (unsigned char) clamp_int(x86_float_to_int(v), 0, 255); }
template <> ND_D __half from_float<3>(float v) { return __float2half_rn(v); }
template <> ND_D short from_float<4>(float v) { return (short) clamp_int(x86_float_to_int(v), -32768, 32767); }
template <> ND_D unsigned short from_float<5>(float v) {
    return (unsigned short) (unsigned char) (unsigned short) clamp_int(x86_float_to_int(v), 0, 65536);
}
template <> ND_D float from_float<6>(float v) { return v; }
template <> ND_D double from_float<7>(float v) { return (double) v; }

// four consecutive elements per thread as one (or two) vector accesses
template <class E> struct alignas(sizeof(E) * 4 > 16 ? 16 : sizeof(E) * 4) Quad { E v[4]; };

template <int SC, int DC>
__global__ void __launch_bounds__(kCopyBlock) k_convert(const void *x, void *z, LL n, int quads) {
    grid_dependency_sync();
    typedef typename ConvType<SC>::T S;
    typedef typename ConvType<DC>::T D;
    const LL tid = (LL) blockIdx.x * kCopyBlock + threadIdx.x, nthreads = (LL) gridDim.x * kCopyBlock;
    const S *sx = static_cast<const S *>(x);
    D *dz = static_cast<D *>(z);
    LL done = 0;
    if (quads) {
        const Quad<S> *qx = static_cast<const Quad<S> *>(x);
        Quad<D> *qz = static_cast<Quad<D> *>(z);
        const LL nq = n / 4;
        LL i = tid;
        for (; i + nthreads < nq; i += 2 * nthreads) {
            const Quad<S> a = qx[i], b = qx[i + nthreads];
            Quad<D> oa, ob;
#pragma unroll
            for (int k = 0; k < 4; k++) { oa.v[k] = from_float<DC>(as_float<SC>(a.v[k])); ob.v[k] = from_float<DC>(as_float<SC>(b.v[k])); }
            qz[i] = oa; qz[i + nthreads] = ob;
        }
        for (; i < nq; i += nthreads) {
            const Quad<S> a = qx[i];
            Quad<D> oa;
#pragma unroll
            for (int k = 0; k < 4; k++) oa.v[k] = from_float<DC>(as_float<SC>(a.v[k]));
            qz[i] = oa;
        }
        done = nq * 4;
    }
    for (LL i = done + tid; i < n; i += nthreads) dz[i] = from_float<DC>(as_float<SC>(sx[i]));
}

template <int SC, int DC>
Status launch_convert(const void *x, void *z, LL n, cudaStream_t stream) {
    typedef typename ConvType<SC>::T S;
    typedef typename ConvType<DC>::T D;
    const bool quads = reinterpret_cast<uintptr_t>(x) % alignof(Quad<S>) == 0 && reinterpret_cast<uintptr_t>(z) % alignof(Quad<D>) == 0;
    LL blocks = ceil_div(ceil_div(n, quads ? 8 : 1), kCopyBlock);
    const LL cap = (LL) kNumSMs * 16;
    if (blocks > cap) blocks = cap;
    if (blocks < 1) blocks = 1;
    launch_kernel(k_convert<SC, DC>, dim3((unsigned) blocks), dim3(kCopyBlock), stream, x, z, n, quads ? 1 : 0);
    ND_CUDA(cudaGetLastError());
    return kOk;
}

template <int SC>
Status convert_from(int dstType, const void *x, void *z, LL n, cudaStream_t stream) {
    switch (dstType) {
        case 0: return launch_convert<SC, 0>(x, z, n, stream);
        case 1: return launch_convert<SC, 1>(x, z, n, stream);
        case 2: return launch_convert<SC, 2>(x, z, n, stream);
        case 3: return launch_convert<SC, 3>(x, z, n, stream);
        case 4: return launch_convert<SC, 4>(x, z, n, stream);
        case 5: return launch_convert<SC, 5>(x, z, n, stream);
        case 6: return launch_convert<SC, 6>(x, z, n, stream);
        default: return launch_convert<SC, 7>(x, z, n, stream);
    }
}

}  // namespace
}  // namespace nd4jb200

using namespace nd4jb200;

#pragma GCC visibility push(default)
extern "C" {

int nd4jb200_flatten(void *stream, int dtype, Nd4jLong offset, char order, void *z, const Nd4jLong *zShapeInfo,
                     const void *x, const Nd4jLong *xShapeInfo) {
    ND_TRY(check_dtype(dtype));
    if (!x || !z) return bad_arg("flatten: null operand");
    if (order != 'c' && order != 'f') return bad_arg("flatten: order must be 'c' or 'f'");
    ShapeDesc xd, zd;
    ND_TRY(parse_shape(xShapeInfo, "xShapeInfo", &xd));
    ND_TRY(parse_shape(zShapeInfo, "zShapeInfo", &zd));
    if (offset < 0 || offset + xd.length > zd.length) return bad_arg("flatten: the input does not fit behind `offset` in the result");
    if (zd.ews < 1) return unsupported("flatten: the result must be addressable by elementWiseStride");
    View vx, vz;
    if (order == 'c') ND_TRY(coord_view(xd, &vx)); else ND_TRY(forder_traversal(xd, &vx));
    LL shp[1] = {xd.length}, str[1] = {zd.ews};
    ND_TRY(collapse_view(1, shp, str, &vz));
    const int bytes = dtype_bytes(dtype);
    return copy_between(bytes, x, vx, static_cast<char *>(z) + offset * zd.ews * bytes, vz, xd.length, as_stream(stream));
}

int nd4jb200_concat(void *stream, int dtype, int dimension, int numArrays, const void *const *data,
                    const Nd4jLong *const *inputShapeInfo, void *z, const Nd4jLong *zShapeInfo) {
    ND_TRY(check_dtype(dtype));
    if (!data || !inputShapeInfo || !z) return bad_arg("concat: null argument");
    if (numArrays < 1) return bad_arg("concat: no inputs");
    ShapeDesc zd;
    ND_TRY(parse_shape(zShapeInfo, "zShapeInfo", &zd));
    if (dimension < 0) dimension += zd.rank;
    if (dimension < 0 || dimension >= zd.rank) return bad_arg("concat: dimension out of range");
    const int bytes = dtype_bytes(dtype);
    LL at = 0;
    for (int k = 0; k < numArrays; k++) {
        ShapeDesc xd;
        ND_TRY(parse_shape(inputShapeInfo[k], "inputShapeInfo", &xd));
        if (!data[k]) return bad_arg("concat: null input array");
        if (xd.rank != zd.rank) return bad_arg("concat: inputs and result differ in rank");
        for (int d = 0; d < zd.rank; d++)
            if (d != dimension && xd.shape[d] != zd.shape[d]) return bad_arg("concat: an input does not match the result off the concatenation axis");
        if (at + xd.shape[dimension] > zd.shape[dimension]) return bad_arg("concat: the inputs overflow the result along the axis");
        // the block of z this input lands in: the input's shape with z's strides
        View vx, vz;
        ND_TRY(coord_view(xd, &vx));
        ND_TRY(collapse_view(zd.rank, xd.shape, zd.stride, &vz));
        ND_TRY(copy_between(bytes, data[k], vx, static_cast<char *>(z) + at * zd.stride[dimension] * bytes, vz, xd.length,
                            as_stream(stream)));
        at += xd.shape[dimension];
    }
    if (at != zd.shape[dimension]) return bad_arg("concat: the inputs do not fill the result along the axis");
    return kOk;
}

int nd4jb200_pull_rows(void *stream, int dtype, const void *x, void *z, Nd4jLong n, const Nd4jLong *indexes,
                       const Nd4jLong *tadShapeInfo, const Nd4jLong *tadOffsets, const Nd4jLong *zTadShapeInfo,
                       const Nd4jLong *zTadOffsets) {
    ND_TRY(check_dtype(dtype));
    if (!x || !z || !indexes || !tadOffsets || !zTadOffsets) return bad_arg("pullRows: null argument");
    if (n < 0) return bad_arg("pullRows: negative row count");
    ShapeDesc xt, zt;
    ND_TRY(parse_shape(tadShapeInfo, "tadShapeInfo", &xt));
    ND_TRY(parse_shape(zTadShapeInfo, "zTadShapeInfo", &zt));
    if (xt.length != zt.length) return bad_arg("pullRows: source and target TADs differ in length");
    if (n == 0 || xt.length == 0) return kOk;
    PullArgs a;
    a.x = x; a.z = z; a.targets = nullptr; a.n = n; a.tadLen = xt.length;
    a.indexes = indexes; a.xOffsets = tadOffsets; a.zOffsets = zTadOffsets;
    // both sides walk by elementWiseStride only when both have one; otherwise element i is the i-th c-order
    // coordinate of each TAD's own shape (blas/cpu/NativeOps.cpp:2072-2101)
    if (xt.ews >= 1 && zt.ews >= 1) {
        ND_TRY(linear_view(xt, &a.xInner));
        ND_TRY(linear_view(zt, &a.zInner));
    } else {
        ND_TRY(coord_view(xt, &a.xInner));
        ND_TRY(coord_view(zt, &a.zInner));
    }
    const int bytes = dtype_bytes(dtype);
    a.dense = unit_run(a.xInner) && unit_run(a.zInner) && (xt.length * bytes) % 16 == 0;
    return launch_pull(bytes, a, as_stream(stream));
}

int nd4jb200_tear(void *stream, int dtype, const void *x, const Nd4jLong *xShapeInfo, void *const *targets,
                  const Nd4jLong *zShapeInfo, const Nd4jLong *tadShapeInfo, const Nd4jLong *tadOffsets) {
    ND_TRY(check_dtype(dtype));
    if (!x || !targets || !tadOffsets) return bad_arg("tear: null argument");
    ShapeDesc xd, zd, xt;
    ND_TRY(parse_shape(xShapeInfo, "xShapeInfo", &xd));
    ND_TRY(parse_shape(zShapeInfo, "zShapeInfo", &zd));
    ND_TRY(parse_shape(tadShapeInfo, "tadShapeInfo", &xt));
    if (xt.length != zd.length) return bad_arg("tear: the targets and the TADs differ in length");
    if (xt.length == 0 || xd.length == 0) return kOk;
    PullArgs a;
    a.x = x; a.z = nullptr; a.n = xd.length / xt.length; a.tadLen = xt.length;
    // `targets` is a host array like the other pointer arrays of this boundary: the kernel reads a copy
    const cudaStream_t st = as_stream(stream);
    void *ws = nullptr;
    ND_TRY(workspace(st, kWorkspaceScratch + sizeof(void *) * (size_t) a.n, &ws, nullptr));
    void **devTargets = reinterpret_cast<void **>(static_cast<char *>(ws) + kWorkspaceScratch);
    for (LL k = 0; k < a.n; k++)
        if (!targets[k]) return bad_arg("tear: null target array");
    ND_TRY(staged_upload(st, devTargets, targets, sizeof(void *) * (size_t) a.n));
    a.targets = devTargets;
    a.indexes = nullptr; a.xOffsets = tadOffsets; a.zOffsets = nullptr;
    if (zd.ews > 0 && xt.ews > 0) {
        LL len[1] = {xt.length}, sx[1] = {xt.ews}, sz[1] = {zd.ews};
        ND_TRY(collapse_view(1, len, sx, &a.xInner));
        ND_TRY(collapse_view(1, len, sz, &a.zInner));
    } else {
        // element j of a TAD in f-order goes to element j of its target in f-order (blas/cpu/NativeOps.cpp:2147-2158)
        ND_TRY(forder_traversal(xt, &a.xInner));
        ND_TRY(forder_traversal(zd, &a.zInner));
    }
    const int bytes = dtype_bytes(dtype);
    a.dense = unit_run(a.xInner) && unit_run(a.zInner) && (xt.length * bytes) % 16 == 0;
    return launch_pull(bytes, a, st);
}

int nd4jb200_shuffle(void *stream, int dtype, int numArrays, void *const *x, const Nd4jLong *const *xShapeInfo,
                     const int *shuffleMap, const Nd4jLong *const *tadShapeInfo, const Nd4jLong *const *tadOffsets) {
    ND_TRY(check_dtype(dtype));
    if (!x || !xShapeInfo || !shuffleMap || !tadShapeInfo || !tadOffsets) return bad_arg("shuffle: null argument");
    if (numArrays < 0) return bad_arg("shuffle: negative array count");
    const int bytes = dtype_bytes(dtype);
    const cudaStream_t st = as_stream(stream);
    size_t used = 0;          // bytes of pair lists already placed in the workspace by this call
    for (int f = 0; f < numArrays; f++) {
        if (!x[f] || !tadOffsets[f]) return bad_arg("shuffle: null array or TAD offsets");
        ShapeDesc xd, xt;
        ND_TRY(parse_shape(xShapeInfo[f], "xShapeInfo", &xd));
        ND_TRY(parse_shape(tadShapeInfo[f], "tadShapeInfo", &xt));
        if (xt.length == 0) continue;
        const LL numTads = xd.length / xt.length;
        if (numTads > 0x7fffffffLL) return bad_arg("shuffle: more TADs than an int map can name");
        std::vector<int2> flat;
        std::vector<size_t> rounds;         // swaps per round
        // The usual map pairs every TAD with at most one other: one round, and the pair list is written straight
        // into a pinned staging buffer while a byte per TAD watches for a TAD that turns up twice. Any other map
        // takes the general ordering into rounds below.
        void *pinned = nullptr;
        int slot = 0;
        ND_TRY(staging_begin(st, (size_t) numTads * sizeof(int2), &pinned, &slot));
        int2 *pairs = static_cast<int2 *>(pinned);
        size_t total = 0;
        bool simple = true;
        {
            thread_local std::vector<unsigned char> tlSeen;
            std::vector<unsigned char> &seen = tlSeen;
            seen.assign((size_t) numTads, 0);
            for (LL r = 0; r < numTads; r++) {
                const int m = shuffleMap[r];
                if (m < 0 || m == r) continue;
                if (m >= numTads) return bad_arg("shuffle: the map names a TAD past the last one");
                if (seen[r] | seen[m]) { simple = false; break; }
                seen[r] = seen[m] = 1;
                pairs[total++] = make_int2((int) r, m);
            }
        }
        if (simple) {
            rounds.assign(total ? 1 : 0, total);
        } else {
            ND_TRY(shuffle_rounds(shuffleMap, numTads, &flat, &rounds));
            total = flat.size();
            if (total) memcpy(pairs, flat.data(), total * sizeof(int2));
        }
        if (total == 0) { ND_TRY(staging_commit(st, slot, nullptr, 0)); continue; }
        // every array's lists get their own part of the workspace: an earlier array's launches may still read theirs
        void *ws = nullptr;
        ND_TRY(workspace(st, kWorkspaceScratch + used + total * sizeof(int2), &ws, nullptr));
        int2 *dev = reinterpret_cast<int2 *>(static_cast<char *>(ws) + kWorkspaceScratch + used);
        ND_TRY(staging_commit(st, slot, dev, total * sizeof(int2)));
        used += total * sizeof(int2);
        SwapArgs a;
        a.x = x[f]; a.offsets = tadOffsets[f]; a.tadLen = xt.length;
        ND_TRY(linear_view(xt, &a.inner));
        a.dense = unit_run(a.inner) && (xt.length * bytes) % 16 == 0;
        const LL perChunk = kPullChunk / bytes;
        a.chunkLen = a.tadLen < perChunk ? a.tadLen : perChunk;
        a.chunks = ceil_div(a.tadLen, a.chunkLen);
        size_t at = 0;
        for (size_t r = 0; r < rounds.size(); r++) {
            a.pairs = dev + at; a.n = (LL) rounds[r];
            at += rounds[r];
            LL blocks = ceil_div(a.n * a.chunks, kCopyBlock / 32);
            const LL cap = (LL) kNumSMs * 16;
            if (blocks > cap) blocks = cap;
            if (bytes == 2) launch_kernel(k_swap_tads<2>, dim3((unsigned) blocks), dim3(kCopyBlock), st, a);
            else if (bytes == 4) launch_kernel(k_swap_tads<4>, dim3((unsigned) blocks), dim3(kCopyBlock), st, a);
            else launch_kernel(k_swap_tads<8>, dim3((unsigned) blocks), dim3(kCopyBlock), st, a);
            ND_CUDA(cudaGetLastError());
        }
    }
    return kOk;
}

int nd4jb200_convert_types(void *stream, int srcType, const void *x, Nd4jLong n, int dstType, void *z) {
    if (!x || !z) return bad_arg("convertTypes: null operand");
    if (n < 0) return bad_arg("convertTypes: negative length");
    // ND4J_FLOAT8 0, INT8 1, UINT8 2, FLOAT16 3, INT16 4, UINT16 5, FLOAT32 6, DOUBLE 7 (type_conversions.h:11-19)
    const bool srcServed = srcType == 0 || srcType == 1 || srcType == 2 || srcType == 3 || srcType == 4 || srcType == 6 || srcType == 7;
    if (!srcServed || dstType < 0 || dstType > 7)
        return unsupported("convertTypes serves float8 (0), int8 (1), uint8 (2), float16 (3), int16 (4), float32 (6) and double "
                           "(7) sources and the same plus uint16 (5) as results; the threshold encodings are not built, and "
                           "the reference has no conversion from uint16");
    // pairs the reference's dispatch leaves out: the result is not touched (type_conversions.h:701-702, 725-727,
    // 853-854; there is no float32 -> float32 branch at all)
    if (srcType == dstType && (srcType == 0 || srcType == 1 || srcType == 6 || srcType == 7)) return kOk;
    if (n == 0) return kOk;
    const cudaStream_t st = as_stream(stream);
    switch (srcType) {
        case 0: return convert_from<0>(dstType, x, z, n, st);
        case 1: return convert_from<1>(dstType, x, z, n, st);
        case 2: return convert_from<2>(dstType, x, z, n, st);
        case 3: return convert_from<3>(dstType, x, z, n, st);
        case 4: return convert_from<4>(dstType, x, z, n, st);
        case 6: return convert_from<6>(dstType, x, z, n, st);
        default: return convert_from<7>(dstType, x, z, n, st);
    }
}

int nd4jb200_average(void *stream, int dtype, const void *const *sources, void *z, int n, Nd4jLong length, int propagate) {
    return sum_sources(stream, dtype, sources, z, n, length, true, propagate != 0);
}

int nd4jb200_accumulate(void *stream, int dtype, const void *const *sources, void *z, int n, Nd4jLong length) {
    if (!z) return bad_arg("accumulate: null result array");
    return sum_sources(stream, dtype, sources, z, n, length, false, false);
}

}  // extern "C"
#pragma GCC visibility pop
