// Random family: a counter-style generator that reproduces the reference's RandomBuffer
// (include/helpers/helper_generator.h) bit for bit. Element e of a call depends only on the
// table, the state words and e, so any index range can be produced independently (which is what
// makes offset-sharding across GPUs possible).
//
//   position p = currentPosition + e;  wraps = p / size;  slot = p % size;  r = table[slot]
//   if wraps != 0:            r = shift(r, generation + wraps)
//   if generation > 1:        r = shift(r, generation)
//   if amplifier != seed:     r = shift(r, amplifier)
//   if any of the above:      r = mix(finalise(r))
//   shift(x, y)  = (y != 0 && x > MAX/y) ? x / y + 11 : x * y + 11       (helper_generator.h:238-242)
//   finalise     = splitmix64 finaliser                                   (helper_generator.h:244-250)
//   mix(s)       = one xoroshiro step on (s, s % (2^31-1) + 11), returning r0 + r1 (:222-232)
//   uniform      = rn_float(r) / 2^64  (the float of 2^64-1 is 2^64)      (:481-486)
//
// The arithmetic is 64-bit integer work (one division per draw once the table has wrapped), so
// this family is bound by the integer pipe, not by HBM. Two things keep the instruction count
// down on the dense path: every CTA walks a contiguous chunk of indices with a cursor
// (slot, wraps) that is advanced by additions, so the p / size and p % size divisions happen once
// per thread; and x / y is done by multiplying with floor(MAX / y), which only changes when the
// cursor wraps, followed by at most two corrections.
// Float arithmetic uses explicit round-to-nearest intrinsics so that nothing is contracted into
// an FMA: the reference's CPU build targets the x86-64 baseline, which has none.
#pragma once
#include "device_utils.cuh"
#include "runtime.h"

namespace nd4jb200 {

typedef unsigned long long U64;

struct RngParams {
    const U64 *table;
    LL size;
    LL position;    // currentPosition at the start of the call
    LL generation;
    LL seed;
    LL amplifier;
    U64 thrGeneration;   // MAX / generation (0 when generation == 0), filled by the host
    U64 thrAmplifier;    // MAX / amplifier  (0 when amplifier == 0)
};

constexpr U64 kMax64 = 0xffffffffffffffffull;

ND_D U64 rng_shift(U64 x, U64 y) {
    if (y != 0ull && x > kMax64 / y) return x / y + 11ull;
    return x * y + 11ull;
}
// Same value as rng_shift with thr = MAX / y precomputed: floor(x * thr / 2^64) is at most two
// below floor(x / y) for y >= 2, so two conditional corrections make it exact.
ND_D U64 rng_shift_pre(U64 x, U64 y, U64 thr) {
    if (y != 0ull && x > thr) {
        U64 q = __umul64hi(x, thr);
        if (y < (1ull << 30)) {
            // the remainder x - q*y is below 3y < 2^32, so its low 32 bits are all of it
            const unsigned y32 = (unsigned) y;
            unsigned rem = (unsigned) x - (unsigned) q * y32;
            unsigned up = 0;
            if (rem >= y32) { up = 1; rem -= y32; }
            if (rem >= y32) up++;
            return q + (U64) (up + 11u);
        }
        U64 rem = x - q * y;
        if (rem >= y) { q++; rem -= y; }
        if (rem >= y) q++;
        return q + 11ull;
    }
    return x * y + 11ull;
}
ND_D U64 rng_finalise(U64 x) {
    U64 z = x + 0x9E3779B97F4A7C15ull;
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    return z ^ (z >> 31);
}
ND_D U64 rotl64(U64 x, int k) { return (x << k) | (x >> (64 - k)); }
// s mod (2^31 - 1) by folding 31-bit digits (2^31 = 1 mod m)
ND_D U64 mod_mersenne31(U64 s) {
    // three 31-bit digits in 32-bit arithmetic: lo 31 bits, the next 31, the top 2
    const unsigned m = 2147483647u;
    const unsigned lo = (unsigned) s, hi = (unsigned) (s >> 32);
    const unsigned d0 = lo & m;
    const unsigned d1 = __funnelshift_r(lo, hi, 31) & m;        // bits 31..61
    const unsigned d2 = hi >> 30;                               // bits 62..63
    unsigned t = d0 + d1;                                       // <= 2^32 - 2
    t = (t & m) + (t >> 31) + d2;                               // <= m + 4
    return (U64) (t >= m ? t - m : t);
}
ND_D U64 rng_mix(U64 s0) {
    U64 s1 = mod_mersenne31(s0) + 11ull;
    s1 ^= s0;
    U64 r0 = rotl64(s0, 55) ^ s1 ^ (s1 << 14);
    U64 r1 = rotl64(s1, 36);
    return r0 + r1;
}

// Draw for an arbitrary index (general path).
ND_D U64 rng_element(const RngParams &g, LL e) {
    LL p = g.position + e;
    LL gen = g.generation;
    if (p >= g.size) { gen += p / g.size; p = p % g.size; }
    U64 r = g.table[p];
    const bool wrapped = gen != g.generation;
    if (wrapped) r = rng_shift(r, (U64) gen);
    if (g.generation > 1) r = rng_shift_pre(r, (U64) g.generation, g.thrGeneration);
    if (g.amplifier != g.seed) r = rng_shift_pre(r, (U64) g.amplifier, g.thrAmplifier);
    if (wrapped || g.generation > 1 || g.amplifier != g.seed) r = rng_mix(rng_finalise(r));
    return r;
}

// Cursor over consecutive indices (dense path).
struct RngCursor {
    LL slot;
    LL gen;
    U64 thr;
    ND_D void seek(const RngParams &g, LL e) {
        LL p = g.position + e;
        gen = g.generation;
        slot = p;
        if (p >= g.size) { LL q = p / g.size; gen += q; slot = p - q * g.size; }
        thr = gen != 0 ? kMax64 / (U64) gen : 0ull;
    }
    ND_D void advance(const RngParams &g, LL k) {
        slot += k;
        if (slot >= g.size) {
            LL q = slot / g.size;
            slot -= q * g.size;
            gen += q;
            thr = gen != 0 ? kMax64 / (U64) gen : 0ull;
        }
    }
    ND_D U64 draw(const RngParams &g) const {
        U64 r = g.table[slot];
        const bool wrapped = gen != g.generation;
        if (wrapped) r = rng_shift_pre(r, (U64) gen, thr);
        if (g.generation > 1) r = rng_shift_pre(r, (U64) g.generation, g.thrGeneration);
        if (g.amplifier != g.seed) r = rng_shift_pre(r, (U64) g.amplifier, g.thrAmplifier);
        if (wrapped || g.generation > 1 || g.amplifier != g.seed) r = rng_mix(rng_finalise(r));
        return r;
    }
};

template <class C> ND_D C rng_unit(U64 r);
template <> ND_D float rng_unit<float>(U64 r) { return __fmul_rn(__ull2float_rn(r), 5.421010862427522e-20f); }
template <> ND_D double rng_unit<double>(U64 r) { return __dmul_rn(__ull2double_rn(r), 5.421010862427522e-20); }

ND_D float rn_mul(float a, float b) { return __fmul_rn(a, b); }
ND_D double rn_mul(double a, double b) { return __dmul_rn(a, b); }
ND_D float rn_add(float a, float b) { return __fadd_rn(a, b); }
ND_D double rn_add(double a, double b) { return __dadd_rn(a, b); }
ND_D float rn_div(float a, float b) { return __fdiv_rn(a, b); }
ND_D double rn_div(double a, double b) { return __ddiv_rn(a, b); }

// Uniform draw in the element type's own precision: half draws are the float draw rounded to
// half (helper_generator.h:482-484).
template <class T> ND_D typename Elem<T>::C rng_uniform(U64 raw) {
    typedef typename Elem<T>::C C;
    C u = rng_unit<C>(raw);
    if (sizeof(T) == 2) u = Elem<T>::to_c(Elem<T>::from_c(u));
    return u;
}
template <class T> ND_D typename Elem<T>::C rng_uniform(U64 raw, typename Elem<T>::C from, typename Elem<T>::C to) {
    return rn_add(from, rn_mul(rng_uniform<T>(raw), rn_add(to, -from)));
}

struct RngArgs {
    RngParams g;
    const void *x;
    const void *y;
    void *z;
    const void *extra;
    LL first;      // global index of the first element this launch produces
    LL count;      // how many elements this launch produces
    LL length;     // length of the whole logical call (what the functors see as `length`)
    int mode;      // 0 unit-stride operands, 1 strided (ews), 2 views (f-order coordinates)
    LL sx, sy, sz;
    View vx, vy, vz;
    int yIsZ;      // Gaussian family: y aliases z, so the mean comes from extra[0]
    LL chunk;      // dense path: elements per CTA (a multiple of 256 * pack width)
    const void *aux;   // Choice: running sums of the probabilities (element type), auxLen of them
    LL auxLen;
};

// Does (op, arity) consume the uniform draw of its element?
template <int OP, int ARITY> struct RngNeedsDraw {
    static constexpr bool v = (OP == 0 && ARITY == 0) || (OP == 1 && ARITY == 1) || (OP == 2 && ARITY == 1) ||
                              (OP == 3 && ARITY == 2) || (OP == 7 && ARITY <= 1) || (OP == 12 && ARITY == 1) ||
                              (OP == 13 && ARITY == 0);
};

// opNum numbering: RANDOM_OPS (legacy_ops.h:225-239). arity 0: z only, 1: x, 2: x and y.
template <class T, int OP, int ARITY>
ND_D typename Elem<T>::C rng_value(LL length, const typename Elem<T>::C *p, LL e, U64 raw,
                                   typename Elem<T>::C xv, typename Elem<T>::C yv) {
    typedef typename Elem<T>::C C;
    if (OP == 100) {        // an op that has no body for this arity: the reference's defaults
        return ARITY == 0 ? C(-1) : (ARITY == 1 ? C(-2) : C(-3));
    } else if (OP == 0) {   // UniformDistribution (random_ops.h:59-72)
        if (ARITY == 0) return rng_uniform<T>(raw, p[0], p[1]);
        return ARITY == 1 ? C(-2) : C(-3);
    } else if (OP == 1) {   // DropOut (:122-137)
        if (ARITY == 1) return rng_uniform<T>(raw) >= p[0] ? C(0) : xv;
        return ARITY == 0 ? C(-1) : C(-3);
    } else if (OP == 2) {   // DropOutInverted (:161-176)
        if (ARITY == 1) return rng_uniform<T>(raw) >= p[0] ? C(0) : rn_div(xv, p[0]);
        return ARITY == 0 ? C(-1) : C(-3);
    } else if (OP == 3) {   // ProbablisticMerge (:36-53)
        if (ARITY == 2) return rng_uniform<T>(raw) <= p[0] ? yv : xv;
        return ARITY == 0 ? C(-1) : C(-2);
    } else if (OP == 4) {   // Linspace (:179-196)
        if (ARITY == 0) {
            C step = rn_div(C(e), rn_add(C(length), C(-1)));
            return rn_add(rn_mul(p[0], rn_add(C(1), -step)), rn_mul(step, p[1]));
        }
        return ARITY == 1 ? C(-2) : C(-3);
    } else if (OP == 7) {   // BernoulliDistribution (:77-91)
        if (ARITY == 0) return p[0] >= rng_uniform<T>(raw) ? C(1) : C(0);
        if (ARITY == 1) return xv >= rng_uniform<T>(raw) ? C(1) : C(0);
        return C(-3);
    } else if (OP == 12) {  // AlphaDropOut (:140-158): p = {prob, a, b, alphaPrime}
        if (ARITY == 1)
            return rng_uniform<T>(raw) >= p[0] ? rn_add(rn_mul(p[1], p[3]), p[2]) : rn_add(rn_mul(p[1], xv), p[2]);
        return ARITY == 0 ? C(-1) : C(-3);
    } else {                // 13 ExponentialDistribution (:96-117)
        if (ARITY == 0) {
            const C tiny = sizeof(T) == 8 ? C(2.2250738585072014e-308) : (sizeof(T) == 4 ? C(1.175494e-38f) : C(6.1035e-05f));
            C u = rng_uniform<T>(raw, tiny, C(1));
            return rn_add(C(1), -pow(C(2.7182818284590452354), -rn_mul(p[0], u)));
        }
        if (ARITY == 1) return xv <= C(0) ? C(0) : rn_add(C(1), -pow(C(2.7182818284590452354), -rn_mul(p[0], xv)));
        return C(-3);
    }
}

template <int OP> struct RngOpParams { static constexpr int n = (OP == 0 || OP == 4) ? 2 : (OP == 12 ? 4 : 1); };

constexpr int kRngBlock = 256;

template <class T, int OP, int ARITY>
__global__ void __launch_bounds__(kRngBlock) k_random(const RngArgs a) {
    grid_dependency_sync();
    typedef typename Elem<T>::C C;
    constexpr int V = Elem<T>::kVec;
    constexpr bool kDraw = RngNeedsDraw<OP, ARITY>::v;
    const T *ax = static_cast<const T *>(a.x);
    const T *ay = static_cast<const T *>(a.y);
    T *az = static_cast<T *>(a.z);
    C p[4] = {C(0), C(0), C(0), C(0)};
    load_params<T, RngOpParams<OP>::n>(static_cast<const T *>(a.extra), p);
    if (a.mode == 0) {
        // CTA b owns indices [b * chunk, (b + 1) * chunk); a thread walks them in packs of V,
        // 256 * V apart, with a cursor that never divides inside the loop
        const LL begin = (LL) blockIdx.x * a.chunk;
        LL end = begin + a.chunk;
        if (end > a.count) end = a.count;
        const LL full = end - (end - begin) % V;         // last index covered by whole packs
        RngCursor cur;
        LL i = begin + (LL) threadIdx.x * V;
        if (kDraw && i < end) cur.seek(a.g, a.first + i);
        for (; i < full; i += (LL) kRngBlock * V) {
            Pack<T> xv, yv, o;
            if (ARITY >= 1) xv = load_pack_rw(ax + i);
            if (ARITY == 2) yv = load_pack_rw(ay + i);
#pragma unroll
            for (int k = 0; k < V; k++) {
                U64 raw = 0;
                if (kDraw) { raw = cur.draw(a.g); cur.advance(a.g, 1); }
                C xc = ARITY >= 1 ? Elem<T>::to_c(xv.v[k]) : C(0);
                C yc = ARITY == 2 ? Elem<T>::to_c(yv.v[k]) : C(0);
                o.v[k] = Elem<T>::from_c(rng_value<T, OP, ARITY>(a.length, p, a.first + i + k, raw, xc, yc));
            }
            store_pack(az + i, o);
            if (kDraw) cur.advance(a.g, (LL) kRngBlock * V - V);
        }
        // ragged tail of the last CTA (fewer than V elements)
        const LL t = full + threadIdx.x;
        if (t < end) {
            U64 raw = kDraw ? rng_element(a.g, a.first + t) : 0;
            C xc = ARITY >= 1 ? Elem<T>::load(ax + t) : C(0);
            C yc = ARITY == 2 ? Elem<T>::load(ay + t) : C(0);
            Elem<T>::store(az + t, rng_value<T, OP, ARITY>(a.length, p, a.first + t, raw, xc, yc));
        }
    } else {
        const LL nthreads = (LL) gridDim.x * kRngBlock;
        for (LL i = (LL) blockIdx.x * kRngBlock + threadIdx.x; i < a.count; i += nthreads) {
            const LL e = a.first + i;
            LL ox = 0, oy = 0, oz;
            if (a.mode == 1) { oz = i * a.sz; if (ARITY >= 1) ox = i * a.sx; if (ARITY == 2) oy = i * a.sy; }
            else {
                oz = view_offset(a.vz, i);
                if (ARITY >= 1) ox = view_offset(a.vx, i);
                if (ARITY == 2) oy = view_offset(a.vy, i);
            }
            U64 raw = kDraw ? rng_element(a.g, e) : 0;
            C xc = ARITY >= 1 ? Elem<T>::load(ax + ox) : C(0);
            C yc = ARITY == 2 ? Elem<T>::load(ay + oy) : C(0);
            Elem<T>::store(az + oz, rng_value<T, OP, ARITY>(a.length, p, e, raw, xc, yc));
        }
    }
}

// GaussianDistribution (6) and LogNormalDistribution (10): Box-Muller on the pair of uniforms
// at global indices (2k, 2k+1), each mapped to [1e-5, 1] first; element 2k gets the cosine
// branch and 2k+1 the sine branch (special_random_ops.h:333-396). z = n * stddev + mean, where
// the mean is extra[0] when y aliases z and y[e] otherwise; LogNormal exponentiates the result.
// CTA b owns the pairs of indices [b * chunk, (b + 1) * chunk) (chunk is even).
template <class T, bool LOGNORMAL>
__global__ void __launch_bounds__(kRngBlock) k_random_gaussian(const RngArgs a) {
    grid_dependency_sync();
    typedef typename Elem<T>::C C;
    const T *ay = static_cast<const T *>(a.y);
    T *az = static_cast<T *>(a.z);
    C p[2];
    load_params<T, 2>(static_cast<const T *>(a.extra), p);
    const C mean = p[0], stddev = p[1];
    const C twoPi = C(2.0 * 3.14159265358979323846);
    const C eps = C(1e-5f);
    const LL begin = (LL) blockIdx.x * a.chunk;
    LL end = begin + a.chunk;
    if (end > a.count) end = a.count;
    RngCursor cur;
    LL li = begin + 2 * (LL) threadIdx.x;     // a.first is even (checked by the host), so li + first is too
    if (li < end) cur.seek(a.g, a.first + li);
    for (; li < end; li += 2 * (LL) kRngBlock) {
        const U64 raw0 = cur.draw(a.g);
        cur.advance(a.g, 1);
        const U64 raw1 = cur.draw(a.g);
        cur.advance(a.g, 2 * (LL) kRngBlock - 1);
        const C u0 = rng_uniform<T>(raw0, eps, C(1));
        const C u1 = rng_uniform<T>(raw1, eps, C(1));
        const C radius = sqrt(rn_mul(C(-2), log(u0)));
        const C angle = rn_mul(twoPi, u1);
        const C n0 = rn_mul(radius, cos(angle));
        const C n1 = rn_mul(radius, sin(angle));
#pragma unroll
        for (int h = 0; h < 2; h++) {
            const LL l = li + h;
            if (l >= a.count) break;
            LL oz, oy;
            if (a.mode == 0) { oz = l; oy = l; }
            else { oz = l * a.sz; oy = l * a.sy; }
            const C m = a.yIsZ ? mean : Elem<T>::load(ay + oy);
            C v = rn_add(rn_mul(h == 0 ? n0 : n1, stddev), m);
            if (LOGNORMAL) v = exp(v);
            Elem<T>::store(az + oz, v);
        }
    }
}

// TruncatedNormalDistribution (11): element e < middle = ceil(n / 2) and element e + middle share Box-Muller pairs
// drawn at global indices (e + t * n, e + middle + t * n) for t = 0, 1, ... until both results satisfy
// |mean| + |result| <= 2 |stddev| (special_random_ops.h:779-798). The uniforms are bit-exact; the normals go
// through the device log / cos / sin, so a pair within rounding of the acceptance boundary can be accepted one
// try earlier or later than on the host (counted in the tests: a few per million). The reference's loop has no
// exit when |mean| >= 2 |stddev|; here it ends after kTruncatedMaxTries tries and keeps the last pair.
constexpr int kTruncatedMaxTries = 4096;
template <class T>
__global__ void __launch_bounds__(kRngBlock) k_random_truncated_normal(const RngArgs a) {
    grid_dependency_sync();
    typedef typename Elem<T>::C C;
    const T *ay = static_cast<const T *>(a.y);
    T *az = static_cast<T *>(a.z);
    C p[2];
    load_params<T, 2>(static_cast<const T *>(a.extra), p);
    const C mean = p[0], stddev = p[1];
    const C twoPi = C(2.0 * 3.14159265358979323846);
    const C eps = C(1e-6f);
    const C ds = rn_mul(stddev < C(0) ? -stddev : stddev, C(2));
    const LL n = a.length;
    const LL middle = n - n / 2;
    const LL nthreads = (LL) gridDim.x * kRngBlock;
    for (LL e = (LL) blockIdx.x * kRngBlock + threadIdx.x; e < middle; e += nthreads) {
        const bool second = e + middle < n;
        const C m0 = a.yIsZ ? mean : Elem<T>::load(ay + e * a.sy);
        // the reference reads y[(e + middle) * yEWS] even for the unpaired last element of an odd length; the
        // value only enters the acceptance test there, and the mean stands in for it
        const C m1 = (a.yIsZ || !second) ? (a.yIsZ ? mean : m0) : Elem<T>::load(ay + (e + middle) * a.sy);
        const C am0 = m0 < C(0) ? -m0 : m0, am1 = m1 < C(0) ? -m1 : m1;
        C r0 = C(0), r1 = C(0);
        LL generation = 0;
        for (int t = 0; t < kTruncatedMaxTries; t++) {
            const C u0 = rng_uniform<T>(rng_element(a.g, e + generation), eps, C(1));
            const C u1 = rng_uniform<T>(rng_element(a.g, e + middle + generation), eps, C(1));
            const C radius = sqrt(rn_mul(C(-2), log(u0)));
            const C angle = rn_mul(twoPi, u1);
            r0 = rn_add(rn_mul(rn_mul(radius, cos(angle)), stddev), m0);
            r1 = rn_add(rn_mul(rn_mul(radius, sin(angle)), stddev), m1);
            generation += n;
            const C a0 = r0 < C(0) ? -r0 : r0, a1 = r1 < C(0) ? -r1 : r1;
            if (!(rn_add(am0, a0) > ds || rn_add(am1, a1) > ds)) break;
        }
        Elem<T>::store(az + e * a.sz, r0);
        if (second) Elem<T>::store(az + (e + middle) * a.sz, r1);
    }
}

// BinomialDistribution (8) and BinomialDistributionEx (9): z[e] = number of t in 1..trials whose
// uniform draw at global index (e + 1) * t is below the success probability. extra = {trials,
// probability}; when y does not alias z the probability is y[t - 1] (8: one per trial) or y[e]
// (9: one per element) instead (special_random_ops.h:474-520, 598-650). Operands are addressed by
// their elementWiseStride, as in the reference.
template <class T, bool PER_ELEMENT>
__global__ void __launch_bounds__(kRngBlock) k_random_binomial(const RngArgs a) {
    grid_dependency_sync();
    typedef typename Elem<T>::C C;
    const T *ay = static_cast<const T *>(a.y);
    T *az = static_cast<T *>(a.z);
    C p[2];
    load_params<T, 2>(static_cast<const T *>(a.extra), p);
    const int trials = (int) p[0];
    const LL nthreads = (LL) gridDim.x * kRngBlock;
    for (LL i = (LL) blockIdx.x * kRngBlock + threadIdx.x; i < a.count; i += nthreads) {
        const LL e = a.first + i;
        C prob = p[1];
        if (!a.yIsZ && PER_ELEMENT) prob = Elem<T>::load(ay + e * a.sy);
        int success = 0;
        for (int t = 1; t <= trials; t++) {
            const C u = rng_uniform<T>(rng_element(a.g, (e + 1) * t));
            if (!a.yIsZ && !PER_ELEMENT) prob = Elem<T>::load(ay + (LL) (t - 1) * a.sy);
            success += u < prob ? 1 : 0;
        }
        Elem<T>::store(az + e * a.sz, C(success));
    }
}

// Choice (5): z[e] = x[f] for the first f whose running probability sum reaches the uniform draw
// of element e, the last f if none does (special_random_ops.h:176-190). The running sums are
// accumulated once, in the reference's order and in the element type's own arithmetic (a half
// sum is rounded to half after every addition), by k_choice_sums; every element then scans them.
template <class T>
__global__ void k_choice_sums(const T *y, LL sy, LL n, T *sums) {
    grid_dependency_sync();
    typedef typename Elem<T>::C C;
    if (blockIdx.x != 0 || threadIdx.x != 0) return;
    C c = C(0);
    for (LL f = 0; f < n; f++) {
        c = Elem<T>::to_c(Elem<T>::from_c(c + Elem<T>::load(y + f * sy)));
        Elem<T>::store(sums + f, c);
    }
}

template <class T>
__global__ void __launch_bounds__(kRngBlock) k_random_choice(const RngArgs a) {
    grid_dependency_sync();
    typedef typename Elem<T>::C C;
    const T *ax = static_cast<const T *>(a.x);
    const T *sums = static_cast<const T *>(a.aux);
    T *az = static_cast<T *>(a.z);
    const LL nthreads = (LL) gridDim.x * kRngBlock;
    for (LL i = (LL) blockIdx.x * kRngBlock + threadIdx.x; i < a.count; i += nthreads) {
        const LL e = a.first + i;
        const C u = rng_uniform<T>(rng_element(a.g, e));
        LL f = 0;
        while (f < a.auxLen - 1 && !(u <= Elem<T>::load(sums + f))) f++;
        az[e * a.sz] = ax[f * a.sx];
    }
}

}  // namespace nd4jb200
