// Accumulator policies plugged into the reduction engine (reduce_engine.cuh), one per family.
#pragma once
#include "functors.cuh"
#include "device_utils.cuh"

namespace nd4jb200 {
namespace pol {

using namespace fn;

// ---- reduce: wraps an identity/map/combine/post functor (functors.cuh) ----------------------
template <class Op, class C> struct Reduce {
    struct State { C v; };
    static constexpr int kInputs = 1;
    static constexpr int kColBytes = 8;    // bytes one lane loads per row in the across-TAD kernel
    static constexpr int kParams = Op::kParams;
    ND_D static void init(State &s) { s.v = Op::template identity<C>(); }
    ND_D static void accum(State &s, C x, C, LL, const C *p) { s.v = Op::template combine<C>(s.v, Op::template map<C>(x, p)); }
    template <int N> ND_D static void accum_many(State &s, const C (&x)[N], const C (&y)[N], LL j0, LL jstep, const C *p) {
#pragma unroll
        for (int i = 0; i < N; i++) accum(s, x[i], y[i], j0 + i * jstep, p);
    }
    ND_D static void merge(State &s, const State &o) { s.v = Op::template combine<C>(s.v, o.v); }
    ND_D static C finish(const State &s, LL n, const C *p) { return Op::template post<C>(s.v, n, p); }
};

// LogSumExp (reduce opNum 19). The reference runs a Max pass and then sums exp(x - max)
// (blas/cpu/NativeOpExcutioner.cpp:122-147, include/ops/special_accumulation_ops.h); here the
// running maximum and the rescaled sum travel together so the data is read once.
template <class C> struct LogSumExp {
    struct State { C m; C s; };
    static constexpr int kInputs = 1;
    static constexpr int kColBytes = 8;    // bytes one lane loads per row in the across-TAD kernel
    static constexpr int kParams = 0;
    ND_D static void init(State &s) { s.m = -ND_INF(C); s.s = C(0); }
    ND_D static void accum(State &s, C x, C, LL, const C *) {
        if (x > s.m) { s.s = s.s * exp(s.m - x) + C(1); s.m = x; }
        else if (x == s.m) s.s += C(1);      // also covers +-inf without producing inf-inf
        else s.s += exp(x - s.m);
    }
    template <int N> ND_D static void accum_many(State &s, const C (&x)[N], const C (&y)[N], LL j0, LL jstep, const C *p) {
#pragma unroll
        for (int i = 0; i < N; i++) accum(s, x[i], y[i], j0 + i * jstep, p);
    }
    ND_D static void merge(State &s, const State &o) {
        if (o.s == C(0)) return;
        if (s.s == C(0)) { s = o; return; }
        if (o.m > s.m) { s.s = s.s * exp(s.m - o.m) + o.s; s.m = o.m; }
        else if (o.m == s.m) s.s += o.s;
        else s.s += o.s * exp(o.m - s.m);
    }
    ND_D static C finish(const State &s, LL, const C *) { return s.m + log(s.s); }
};

// ---- reduce3: pairwise distances / similarities (REDUCE3_OPS; formulas ops.h:2567-2990) -----
// kind: 0 Manhattan, 1 Euclidean, 2 CosineSimilarity, 3 Dot, 4 EqualsWithEps, 5 CosineDistance,
//       6 JaccardDistance, 7 SimpleHammingDistance
template <int kind, class C> struct Reduce3 {
    struct State { C acc; C e0; C e1; };
    static constexpr int kInputs = 2;
    static constexpr int kColBytes = 8;    // bytes one lane loads per row in the across-TAD kernel
    static constexpr int kParams = kind == 4 ? 1 : 0;   // EqualsWithEps: p[0] = eps
    // the cosine kinds convert and multiply 16 half values per pack pair: 80 registers instead of 64
    static constexpr int kHalfRowCtas = (kind == 2 || kind == 5 || kind == 6) ? 3 : 4;
    ND_D static void init(State &s) { s.acc = C(0); s.e0 = C(0); s.e1 = C(0); }
    ND_D static void accum(State &s, C x, C y, LL, const C *p) {
        if (kind == 0) s.acc += absv(x - y);
        else if (kind == 1) { C d = x - y; s.acc = fmav(d, d, s.acc); }
        else if (kind == 2 || kind == 5) { s.acc = fmav(x, y, s.acc); s.e0 = fmav(x, x, s.e0); s.e1 = fmav(y, y, s.e1); }
        else if (kind == 3) s.acc = fmav(x, y, s.acc);
        else if (kind == 4) {
            C eps = p[0];
            C diff = absv(x - y);
            bool same = diff <= eps || diff <= maxv(absv(x), absv(y)) * eps;
            s.acc += same ? C(0) : C(1);
        } else if (kind == 6) { s.e0 += minv(x, y); s.e1 += maxv(x, y); }
        else s.acc += (x == y) ? C(0) : C(1);
    }
    template <int N> ND_D static void accum_many(State &s, const C (&x)[N], const C (&y)[N], LL j0, LL jstep, const C *p) {
#pragma unroll
        for (int i = 0; i < N; i++) accum(s, x[i], y[i], j0 + i * jstep, p);
    }
    ND_D static void merge(State &s, const State &o) { s.acc += o.acc; s.e0 += o.e0; s.e1 += o.e1; }
    ND_D static C finish(const State &s, LL n, const C *) {
        if (kind == 1) return sqrt(s.acc);
        if (kind == 2) return s.acc / (sqrt(s.e0) * sqrt(s.e1));
        if (kind == 5) return C(1) - s.acc / (sqrt(s.e0) * sqrt(s.e1));
        if (kind == 6) return C(1) - s.e0 / s.e1;
        if (kind == 7) return s.acc / C(n);
        return s.acc;
    }
};

// ---- indexreduce (INDEX_REDUCE_OPS; ops.h:2992-3470) ----------------------------------------
// kind: 0 IndexMax, 1 IndexMin, 2 IndexAbsoluteMax, 3 IndexAbsoluteMin. The winner is the
// extreme value with the LOWEST index among equals, which is what the reference's sequential
// strict-comparison scan produces (loops/cpu/indexreduce.cpp:208-224) and makes the result
// independent of how elements are spread over threads. Start values follow the reference:
// -1e37 / 1e37 for max / min, 1e-37 for absolute max (ops.h:3075, 3290, 3345, 3410).
template <int kind, class C> struct IndexExtreme {
    struct State { C v; int pad; LL i; };
    static constexpr bool kIndexResult = true;
    static constexpr int kInputs = 1;
    static constexpr int kColBytes = 8;    // bytes one lane loads per row in the across-TAD kernel
    static constexpr int kParams = 0;
    ND_D static void init(State &s) {
        s.v = kind == 0 ? C(-ND_MAX_FLOAT) : (kind == 2 ? C(ND_MIN_FLOAT) : C(ND_MAX_FLOAT));
        s.i = 0; s.pad = 0;
    }
    ND_D static bool better(C a, LL ia, C b, LL ib) {   // is (a, ia) preferred over (b, ib)?
        if (kind == 0 || kind == 2) return a > b || (a == b && ia < ib);
        return a < b || (a == b && ia < ib);
    }
    ND_D static void take(State &s, C v, LL j) {     // selects, not branches: lanes rarely agree
        const bool b = better(v, j, s.v, s.i);
        s.v = b ? v : s.v;
        s.i = b ? j : s.i;
    }
    ND_D static void accum(State &s, C x, C, LL j, const C *) { take(s, (kind >= 2) ? absv(x) : x, j); }
    // a run of ascending indices needs no tie-break: the first strictly better element wins, and
    // only the winner of the run is compared (with the index tie-break) against the state
    template <int N> ND_D static void accum_many(State &s, const C (&x)[N], const C (&y)[N], LL j0, LL jstep, const C *p) {
        C best = (kind >= 2) ? absv(x[0]) : x[0];
        int at = 0;
#pragma unroll
        for (int i = 1; i < N; i++) {
            C v = (kind >= 2) ? absv(x[i]) : x[i];
            bool b = (kind == 0 || kind == 2) ? v > best : v < best;
            best = b ? v : best;
            at = b ? i : at;
        }
        take(s, best, j0 + at * jstep);
    }
    // U packs of V consecutive elements, pack u starting at index j0 + u * ustep (ascending):
    // one index computation and one tie-break for the whole tile
    static constexpr bool kTile = true;
    template <int U, int V> ND_D static void accum_tile(State &s, const C (&x)[U * V], LL j0, int ustep, const C *) {
        C best = (kind >= 2) ? absv(x[0]) : x[0];
        int at = 0;
#pragma unroll
        for (int i = 1; i < U * V; i++) {
            C v = (kind >= 2) ? absv(x[i]) : x[i];
            bool b = (kind == 0 || kind == 2) ? v > best : v < best;
            best = b ? v : best;
            at = b ? i : at;
        }
        take(s, best, j0 + ((at / V) * ustep + (at % V)));
    }
    ND_D static void merge(State &s, const State &o) { take(s, o.v, o.i); }
    ND_D static C finish(const State &s, LL, const C *) { return C(s.i); }
};

// kind: 4 FirstIndex, 5 LastIndex of an element satisfying the MatchCondition predicate with
// extraParams {compare, eps, mode}; -1 when none does (ops.h:3079-3200).
template <int kind, class C> struct IndexMatch {
    struct State { LL i; };
    static constexpr bool kIndexResult = true;
    static constexpr int kInputs = 1;
    static constexpr int kColBytes = 8;    // bytes one lane loads per row in the across-TAD kernel
    static constexpr int kParams = 3;
    ND_D static void init(State &s) { s.i = -1; }
    ND_D static void take(State &s, LL j) {
        if (s.i < 0) s.i = j;
        else if (kind == 4) s.i = j < s.i ? j : s.i;
        else s.i = j > s.i ? j : s.i;
    }
    ND_D static void accum(State &s, C x, C, LL j, const C *p) {
        int c = condition(x, p[0], p[1], (int) p[2]);
        bool hit = c < 0 ? (x != C(0)) : (c != 0);
        if (hit) take(s, j);
    }
    template <int N> ND_D static void accum_many(State &s, const C (&x)[N], const C (&y)[N], LL j0, LL jstep, const C *p) {
#pragma unroll
        for (int i = 0; i < N; i++) accum(s, x[i], y[i], j0 + i * jstep, p);
    }
    ND_D static void merge(State &s, const State &o) { if (o.i >= 0) take(s, o.i); }
    ND_D static C finish(const State &s, LL, const C *) { return C(s.i); }
};

// ---- summarystats (SUMMARY_STATS_OPS; loops/summarystatsreduce.h:51-257, ops.h:3471-3518) ---
// The reference carries (n, mean, M2) in double and merges with Chan's formula per element.
// Here each thread keeps double sums of (x - k) and (x - k)^2 around a pivot k taken from its
// own data (3 flops per element), and partial states are re-centred when merged; the moments
// come out of the same fp64 arithmetic class as the reference's.
// kind: 0 variance, 1 standard deviation.
template <int kind, class C> struct Stats {
    struct State { double n, s1, s2, k; };
    static constexpr int kInputs = 1;
    static constexpr int kColBytes = 8;    // bytes one lane loads per row in the across-TAD kernel
    static constexpr int kParams = 0;
    ND_D static void init(State &s) { s.n = 0; s.s1 = 0; s.s2 = 0; s.k = 0; }
    ND_D static void accum(State &s, C x, C, LL, const C *) {
        double v = (double) x;
        if (s.n == 0) s.k = v;
        double d = v - s.k;
        s.n += 1.0; s.s1 += d; s.s2 += d * d;
    }
    // N elements at once: their offsets from the pivot are summed in the element's own compute
    // type first (N is at most 16, so this adds a few units in the last place of a short sum) and
    // only the two short sums enter the double accumulators
    template <int N> ND_D static void accum_many(State &s, const C (&x)[N], const C (&y)[N], LL j0, LL jstep, const C *p) {
        if (s.n == 0) s.k = (double) x[0];
        const C k = (C) s.k;
        C a = C(0), b = C(0);
#pragma unroll
        for (int i = 0; i < N; i++) { C d = x[i] - k; a += d; b = fmav(d, d, b); }
        s.n += (double) N; s.s1 += (double) a; s.s2 += (double) b;
    }
    ND_D static void merge(State &s, const State &o) {
        if (o.n == 0) return;
        if (s.n == 0) { s = o; return; }
        double d = o.k - s.k;                 // re-centre o's sums on s's pivot
        s.s1 += o.s1 + o.n * d;
        s.s2 += o.s2 + 2.0 * d * o.s1 + o.n * d * d;
        s.n += o.n;
    }
    // n carries the biasCorrected flag in bit 62 (the TAD length never reaches it)
    ND_D static C finish(const State &s, LL nflag, const C *) {
        bool bias = (nflag >> 62) & 1;
        double var = 0.0;
        if (s.n > 1.0) {
            double m2 = s.s2 - s.s1 * s.s1 / s.n;
            var = m2 / s.n;
            if (bias) { double vb = m2 / (s.n - 1.0); if (!(vb < 0.0)) var = vb; }
        }
        return C(kind == 1 ? sqrt(var) : var);
    }
};

}  // namespace pol
}  // namespace nd4jb200
