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
// Float arithmetic below uses explicit round-to-nearest intrinsics so that nothing is contracted
// into an FMA: the reference's CPU build targets the x86-64 baseline, which has none.
#pragma once
#include "device_utils.cuh"
#include "runtime.h"

namespace nd4jb200 {

struct RngParams {
    const unsigned long long *table;
    LL size;
    LL position;    // currentPosition at the start of the call
    LL generation;
    LL seed;
    LL amplifier;
};

ND_D unsigned long long rng_shift(unsigned long long x, unsigned long long y) {
    if (y != 0ull && x > 0xffffffffffffffffull / y) return x / y + 11ull;
    return x * y + 11ull;
}
ND_D unsigned long long rng_finalise(unsigned long long x) {
    unsigned long long z = x + 0x9E3779B97F4A7C15ull;
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    return z ^ (z >> 31);
}
ND_D unsigned long long rotl64(unsigned long long x, int k) { return (x << k) | (x >> (64 - k)); }
ND_D unsigned long long rng_mix(unsigned long long s0) {
    unsigned long long s1 = s0 % 2147483647ull + 11ull;
    s1 ^= s0;
    unsigned long long r0 = rotl64(s0, 55) ^ s1 ^ (s1 << 14);
    unsigned long long r1 = rotl64(s1, 36);
    return r0 + r1;
}

ND_D unsigned long long rng_element(const RngParams &g, LL e) {
    LL p = g.position + e;
    LL gen = g.generation;
    if (p >= g.size) { gen += p / g.size; p = p % g.size; }
    unsigned long long r = g.table[p];
    const bool wrapped = gen != g.generation;
    if (wrapped) r = rng_shift(r, (unsigned long long) gen);
    if (g.generation > 1) r = rng_shift(r, (unsigned long long) g.generation);
    if (g.amplifier != g.seed) r = rng_shift(r, (unsigned long long) g.amplifier);
    if (wrapped || g.generation > 1 || g.amplifier != g.seed) r = rng_mix(rng_finalise(r));
    return r;
}

template <class C> ND_D C rng_unit(unsigned long long r);
template <> ND_D float rng_unit<float>(unsigned long long r) { return __fmul_rn(__ull2float_rn(r), 5.421010862427522e-20f); }
template <> ND_D double rng_unit<double>(unsigned long long r) { return __dmul_rn(__ull2double_rn(r), 5.421010862427522e-20); }

ND_D float rn_mul(float a, float b) { return __fmul_rn(a, b); }
ND_D double rn_mul(double a, double b) { return __dmul_rn(a, b); }
ND_D float rn_add(float a, float b) { return __fadd_rn(a, b); }
ND_D double rn_add(double a, double b) { return __dadd_rn(a, b); }
ND_D float rn_div(float a, float b) { return __fdiv_rn(a, b); }
ND_D double rn_div(double a, double b) { return __ddiv_rn(a, b); }

// Uniform draw of element e in the element type's own precision: half draws are the float draw
// rounded to half (helper_generator.h:482-484).
template <class T> ND_D typename Elem<T>::C rng_uniform(const RngParams &g, LL e) {
    typedef typename Elem<T>::C C;
    C u = rng_unit<C>(rng_element(g, e));
    if (sizeof(T) == 2) u = Elem<T>::to_c(Elem<T>::from_c(u));
    return u;
}
template <class T> ND_D typename Elem<T>::C rng_uniform(const RngParams &g, LL e, typename Elem<T>::C from, typename Elem<T>::C to) {
    return rn_add(from, rn_mul(rng_uniform<T>(g, e), rn_add(to, -from)));
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
};

// opNum numbering: RANDOM_OPS (legacy_ops.h:225-239). arity 0: z only, 1: x, 2: x and y.
template <class T, int OP, int ARITY>
ND_D typename Elem<T>::C rng_value(const RngArgs &a, const typename Elem<T>::C *p, LL e,
                                   typename Elem<T>::C xv, typename Elem<T>::C yv) {
    typedef typename Elem<T>::C C;
    const RngParams &g = a.g;
    if (OP == 100) {        // an op that has no body for this arity: the reference's defaults
        return ARITY == 0 ? C(-1) : (ARITY == 1 ? C(-2) : C(-3));
    } else if (OP == 0) {   // UniformDistribution (random_ops.h:59-72)
        if (ARITY == 0) return rng_uniform<T>(g, e, p[0], p[1]);
        return ARITY == 1 ? C(-2) : C(-3);
    } else if (OP == 1) {   // DropOut (:122-137)
        if (ARITY == 1) return rng_uniform<T>(g, e) >= p[0] ? C(0) : xv;
        return ARITY == 0 ? C(-1) : C(-3);
    } else if (OP == 2) {   // DropOutInverted (:161-176)
        if (ARITY == 1) return rng_uniform<T>(g, e) >= p[0] ? C(0) : rn_div(xv, p[0]);
        return ARITY == 0 ? C(-1) : C(-3);
    } else if (OP == 3) {   // ProbablisticMerge (:36-53)
        if (ARITY == 2) return rng_uniform<T>(g, e) <= p[0] ? yv : xv;
        return ARITY == 0 ? C(-1) : C(-2);
    } else if (OP == 4) {   // Linspace (:179-196)
        if (ARITY == 0) {
            C step = rn_div(C(e), rn_add(C(a.length), C(-1)));
            return rn_add(rn_mul(p[0], rn_add(C(1), -step)), rn_mul(step, p[1]));
        }
        return ARITY == 1 ? C(-2) : C(-3);
    } else if (OP == 7) {   // BernoulliDistribution (:77-91)
        if (ARITY == 0) return p[0] >= rng_uniform<T>(g, e) ? C(1) : C(0);
        if (ARITY == 1) return xv >= rng_uniform<T>(g, e) ? C(1) : C(0);
        return C(-3);
    } else if (OP == 12) {  // AlphaDropOut (:140-158): p = {prob, a, b, alphaPrime}
        if (ARITY == 1)
            return rng_uniform<T>(g, e) >= p[0] ? rn_add(rn_mul(p[1], p[3]), p[2]) : rn_add(rn_mul(p[1], xv), p[2]);
        return ARITY == 0 ? C(-1) : C(-3);
    } else {                // 13 ExponentialDistribution (:96-117)
        if (ARITY == 0) {
            const C tiny = sizeof(T) == 8 ? C(2.2250738585072014e-308) : (sizeof(T) == 4 ? C(1.175494351e-38f) : C(6.103515625e-05f));
            C u = rng_uniform<T>(g, e, tiny, C(1));
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
    typedef typename Elem<T>::C C;
    constexpr int V = Elem<T>::kVec;
    const T *ax = static_cast<const T *>(a.x);
    const T *ay = static_cast<const T *>(a.y);
    T *az = static_cast<T *>(a.z);
    C p[4] = {C(0), C(0), C(0), C(0)};
    load_params<T, RngOpParams<OP>::n>(static_cast<const T *>(a.extra), p);
    const LL tid = (LL) blockIdx.x * kRngBlock + threadIdx.x;
    const LL nthreads = (LL) gridDim.x * kRngBlock;
    if (a.mode == 0) {
        const LL npacks = a.count / V;
        for (LL i = tid; i < npacks; i += nthreads) {
            Pack<T> xv, yv, o;
            if (ARITY >= 1) xv = load_pack_rw(ax + i * V);
            if (ARITY == 2) yv = load_pack_rw(ay + i * V);
#pragma unroll
            for (int k = 0; k < V; k++) {
                C xc = ARITY >= 1 ? Elem<T>::to_c(xv.v[k]) : C(0);
                C yc = ARITY == 2 ? Elem<T>::to_c(yv.v[k]) : C(0);
                o.v[k] = Elem<T>::from_c(rng_value<T, OP, ARITY>(a, p, a.first + i * V + k, xc, yc));
            }
            store_pack(az + i * V, o);
        }
        const LL i = npacks * V + tid;
        if (i < a.count) {
            C xc = ARITY >= 1 ? Elem<T>::load(ax + i) : C(0);
            C yc = ARITY == 2 ? Elem<T>::load(ay + i) : C(0);
            Elem<T>::store(az + i, rng_value<T, OP, ARITY>(a, p, a.first + i, xc, yc));
        }
    } else {
        for (LL i = tid; i < a.count; i += nthreads) {
            const LL e = a.first + i;
            LL ox = 0, oy = 0, oz;
            if (a.mode == 1) { oz = i * a.sz; if (ARITY >= 1) ox = i * a.sx; if (ARITY == 2) oy = i * a.sy; }
            else {
                oz = view_offset(a.vz, i);
                if (ARITY >= 1) ox = view_offset(a.vx, i);
                if (ARITY == 2) oy = view_offset(a.vy, i);
            }
            C xc = ARITY >= 1 ? Elem<T>::load(ax + ox) : C(0);
            C yc = ARITY == 2 ? Elem<T>::load(ay + oy) : C(0);
            Elem<T>::store(az + oz, rng_value<T, OP, ARITY>(a, p, e, xc, yc));
        }
    }
}

// GaussianDistribution (6) and LogNormalDistribution (10): Box-Muller on the pair of uniforms
// at global indices (2k, 2k+1), each mapped to [1e-5, 1] first; element 2k gets the cosine
// branch and 2k+1 the sine branch (special_random_ops.h:333-396). z = n * stddev + mean, where
// the mean is extra[0] when y aliases z and y[e] otherwise; LogNormal exponentiates the result.
template <class T, bool LOGNORMAL>
__global__ void __launch_bounds__(kRngBlock) k_random_gaussian(const RngArgs a) {
    typedef typename Elem<T>::C C;
    const T *ay = static_cast<const T *>(a.y);
    T *az = static_cast<T *>(a.z);
    C p[2];
    load_params<T, 2>(static_cast<const T *>(a.extra), p);
    const C mean = p[0], stddev = p[1];
    const C twoPi = C(2.0 * 3.14159265358979323846);
    const C eps = C(1e-5f);
    // a.first is even (checked by the host); thread i produces the pair (first + 2i, first + 2i + 1)
    const LL npairs = (a.count + 1) / 2;
    const LL nthreads = (LL) gridDim.x * kRngBlock;
    for (LL i = (LL) blockIdx.x * kRngBlock + threadIdx.x; i < npairs; i += nthreads) {
        const LL e0 = a.first + 2 * i;
        const C u0 = rng_uniform<T>(a.g, e0, eps, C(1));
        const C u1 = rng_uniform<T>(a.g, e0 + 1, eps, C(1));
        const C radius = sqrt(rn_mul(C(-2), log(u0)));
        const C angle = rn_mul(twoPi, u1);
        const C n0 = rn_mul(radius, cos(angle));
        const C n1 = rn_mul(radius, sin(angle));
#pragma unroll
        for (int h = 0; h < 2; h++) {
            const LL li = 2 * i + h;
            if (li >= a.count) break;
            LL oz, oy;
            if (a.mode == 0) { oz = li; oy = li; }
            else if (a.mode == 1) { oz = li * a.sz; oy = li * a.sy; }
            else { oz = view_offset(a.vz, li); oy = view_offset(a.vy, li); }
            const C m = a.yIsZ ? mean : Elem<T>::load(ay + oy);
            C v = rn_add(rn_mul(h == 0 ? n0 : n1, stddev), m);
            if (LOGNORMAL) v = exp(v);
            Elem<T>::store(az + oz, v);
        }
    }
}

}  // namespace nd4jb200
