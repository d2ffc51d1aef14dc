// Device functors for the legacy op families. Each functor states what one opNum of the
// reference computes (formulas: include/ops/ops.h of the reference; numbering:
// include/loops/legacy_ops.h). They are written against a compute type C (float for the
// Float and Half entry points, double for Double); loads widen to C, stores round back once.
//
// Extra parameters arrive as a small register array `p` preloaded by the kernel
// (kParams entries, converted to C); functors never dereference global memory themselves.
#pragma once
#include <cuda_runtime.h>
#include <math_constants.h>
#include "common.h"

namespace nd4jb200 {
namespace fn {

// ---- constants of the reference (include/ops/ops.h:11-18, 41-42) ---------------------------
#define ND_MIN_EPS 1e-12
#define ND_MAX_FLOAT 1e37
#define ND_MIN_FLOAT 1e-37
#define ND_MIN_CUTOFF (-3.79297773665f)
#define ND_SELU_ALPHA 1.6732632423543772848170429916717
#define ND_SELU_LAMBDA 1.0507009873554804934193349852946
#define ND_E 2.7182818284590452354

template <class C> ND_D C absv(C x) { return x < C(0) ? -x : x; }
template <> ND_D float absv<float>(float x) { return fabsf(x); }
// a * b + c in one rounding; for accumulators whose tolerance is relative, not for elementwise results
ND_D float fmav(float a, float b, float c) { return __fmaf_rn(a, b, c); }
ND_D double fmav(double a, double b, double c) { return __fma_rn(a, b, c); }
template <class C> ND_D C maxv(C a, C b) { return a > b ? a : b; }   // nd4j_max: "a > b ? a : b"
template <class C> ND_D C minv(C a, C b) { return a < b ? a : b; }   // nd4j_min: "a < b ? a : b"
template <class C> ND_D C sgn(C x) { return x < C(0) ? C(-1) : (x > C(0) ? C(1) : C(0)); }
template <class C> ND_D bool isnanv(C x) { return x != x; }
template <class C> ND_D bool isinfv(C x) { return isinf(x); }
template <class C> ND_D C rel_err(C a, C b) {
    if (a == C(0) && b == C(0)) return C(0);
    return absv(a - b) / (absv(a) + absv(b));
}

// tanh for float with error well below one ulp, so that results stay within 2 ulp of the host
// libm the reference calls (templatemath.h:847). |x| < 11/32: odd polynomial. Otherwise
// |x| = k/16 + d with |d| <= 1/32, and
//     tanh(k/16 + d) = T + (1 - T^2) tanh(d) / (1 + T tanh(d)),   T = tanh(k/16),
// where T comes from a 141-entry table (k = 6..146) as an unevaluated float pair and the second term is
// at most 0.03 against T >= 0.36, so its rounding errors are a small fraction of an ulp of the result
// (0.78 ulp worst case over every float below 0.75 in an emulation that also perturbs the reciprocal by
// one ulp either way). Both chains are straight-line code (most warps hold arguments of both kinds).
static __device__ const float4 kTanhTable[141] = {
#include "tanh_table.inc"
};
ND_D float rcp_fast(float x) {
    float r;
    asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(x));
    return r;
}
// kShared: T (hi, lo) comes from the CTA's shared-memory copy of the table (tanh_table_to_shared must have
// run) and 1 - T^2 is recomputed (one FMA; its cancellation error near T = 1 scales a term below 1e-6).
// The global table is read through L1 as a 16-byte gather that costs up to one wavefront per distinct row
// and made the L1 data pipe, not the arithmetic, the limit of the Tanh transform (84 % busy in ncu).
ND_D float2 *tanh_shared_table() {
    __shared__ float2 table[144];
    return table;
}
ND_D void tanh_table_to_shared() {
    float2 *t = tanh_shared_table();
    const int tid = threadIdx.x + threadIdx.y * blockDim.x, n = blockDim.x * blockDim.y;
    for (int i = tid; i < 141; i += n) { const float4 e = kTanhTable[i]; t[i] = make_float2(e.x, e.y); }
    __syncthreads();
}
template <bool kShared> ND_D float tanh_core(float x) {
    const float ax = fabsf(x);
    // |x| < 11/32: odd polynomial x + x^3 P(x^2), P fitted to (tanh x - x) / x^3 (error 8e-10 relative)
    const float z = ax * ax;
    float ps = 0.01974657f;
    ps = fmaf(ps, z, -0.05379952f);
    ps = fmaf(ps, z, 0.13332911f);
    ps = fmaf(ps, z, -0.33333334f);
    const float ts = fmaf(ax * z, ps, ax);
    // otherwise k = round(16 |x|) in 6..146; adding 1.5 * 2^23 leaves k in the low mantissa bits. Arguments
    // above 9.125 are clamped: tanh is 1 to float precision from 9.011 on, and the table's last entries
    // round to exactly 1, so no separate saturation test is needed (infinity included).
    const float magic = 12582912.0f;
    const float ac = fminf(fmaxf(ax, 0.34375f), 9.125f);
    const float kb = fmaf(ac, 16.0f, magic);
    const float kf = kb - magic;
    const int k = (__float_as_int(kb) & 0xff) - 6;
    float th, tl, c;
    if (kShared) {
        const float2 e = tanh_shared_table()[k];
        th = e.x; tl = e.y; c = fmaf(-th, th, 1.0f);
    } else {
        const float4 e = __ldg(&kTanhTable[k]);                               // {T hi, T lo, 1 - T^2, 0}
        th = e.x; tl = e.y; c = e.z;
    }
    const float d = fmaf(-kf, 0.0625f, ac);                                  // exact, |d| <= 1/32
    const float d2 = d * d;
    const float td = fmaf(d * d2, fmaf(0.13333333f, d2, -0.33333334f), d);   // tanh(d)
    const float corr = (c * td) * rcp_fast(fmaf(th, td, 1.0f));
    const float tb = th + (tl + corr);
    const float t = copysignf(ax < 0.34375f ? ts : tb, x);
    return x != x ? x : t;
}
ND_D float tanh_accurate(float x) { return tanh_core<false>(x); }
// exp for float with error close to half an ulp (the host libm's expf is nearly correctly
// rounded, the CUDA library's is within 2 ulp): same range reduction and (hi, lo) bookkeeping as
// tanh_accurate, with the scaling by 2^n split in two so that subnormal results round once more.
ND_D float exp_accurate(float x) {
    if (!(x < 88.72284f)) return x == x ? CUDART_INF_F : x;
    if (x < -103.972f) return 0.0f;
    const float n = rintf(x * 1.4426950408889634f);
    const float rh = fmaf(-n, 0.693145751953125f, x);
    const float rl = -n * 1.42860682030941723212e-6f;
    const float r = rh + rl;
    const float rerr = (rh - r) + rl;
    float q = 0.0001989928507603579f;
    q = fmaf(q, r, 0.0013933650354159414f);
    q = fmaf(q, r, 0.008333298469720569f);
    q = fmaf(q, r, 0.04166646491457965f);
    q = fmaf(q, r, 0.16666666719031667f);
    q = fmaf(q, r, 0.5000000013468379f);
    const float p = (r * r) * q;
    const float sh = r + p;
    float sl = p - (sh - r);
    sl += fmaf(rerr, r, rerr);
    const float t = 1.0f + sh;
    const float e = (1.0f - t) + sh;
    float res = t + (e + sl);
    const int ni = (int) n, a = ni / 2, b = ni - a;
    res *= __int_as_float((a + 127) << 23);
    res *= __int_as_float((b + 127) << 23);
    return res;
}
template <class C> ND_D C expv(C x) { return exp(x); }
template <> ND_D float expv<float>(float x) { return exp_accurate(x); }

template <class C> ND_D C tanhv(C x) { return tanh(x); }
template <> ND_D float tanhv<float>(float x) { return tanh_accurate(x); }
template <class C> ND_D C sigmoid(C x) { return C(1) / (C(1) + expv(-x)); }

// The 14 comparison modes shared by MatchCondition, CompareAndSet, CompareAndReplace and the
// First/LastIndex reductions (ops.h:1534-1602). Returns <0 for an unknown mode.
template <class C> ND_D int condition(C v, C compare, C eps, int mode) {
    switch (mode) {
        case 0: return absv(v - compare) <= eps;
        case 1: return absv(v - compare) > eps;
        case 2: return v < compare;
        case 3: return v > compare;
        case 4: return v <= compare;
        case 5: return v >= compare;
        case 6: return absv(v) < compare;
        case 7: return absv(v) > compare;
        case 8: return isinfv(v);
        case 9: return isnanv(v);
        case 10: return v == compare;
        case 11: return v != compare;
        case 12: return absv(v) >= compare;
        case 13: return absv(v) <= compare;
        default: return -1;
    }
}

// =============================================================================================
// Unary transforms: z = f(x, p)           (TRANSFORM_OPS, legacy_ops.h:49-141)
// =============================================================================================
#define ND_UNARY(Name, NP, ...)                                              \
    struct Name {                                                            \
        static constexpr int kParams = NP;                                   \
        template <class C> ND_D static C f(C x, const C *p) { __VA_ARGS__ }  \
    };

ND_UNARY(Abs, 0, return absv(x);)
ND_UNARY(Ceiling, 0, return ceil(x);)
ND_UNARY(Cosine, 0, return cos(x);)
ND_UNARY(Exp, 0, return expv(x);)
ND_UNARY(Floor, 0, return floor(x);)
ND_UNARY(Log, 0, return log(x);)
ND_UNARY(Neg, 0, return -x;)
ND_UNARY(PowT, 1, return pow(x, p[0]);)
ND_UNARY(Round, 0, return round(x);)
ND_UNARY(SetRange, 2,
         C lo = p[0], hi = p[1];
         if (x >= lo && x <= hi) return x;
         if (lo == C(0) && hi == C(1)) { C v = C(1) / (C(1) + expv(-x)); return floor(v * (hi - lo)) + lo; }
         return floor(x * (hi - lo)) + lo;)
ND_UNARY(Sigmoid, 0, return sigmoid(x);)
ND_UNARY(Sign, 0, return C((x > C(0)) - (x < C(0)));)
ND_UNARY(Sin, 0, return sin(x);)
ND_UNARY(SoftPlus, 0, return log(C(1) + expv(x));)
ND_UNARY(Sqrt, 0, return sqrt(x);)
// Tanh keeps its table in shared memory: kernels that apply it call prepare() once per CTA (all threads).
struct Tanh {
    static constexpr int kParams = 0;
    static constexpr bool kPrepare = true;
    ND_D static void prepare() { tanh_table_to_shared(); }
    template <class C> ND_D static C f(C x, const C *) { return tanh(x); }
};
template <> ND_D float Tanh::f<float>(float x, const float *) { return tanh_core<true>(x); }
ND_UNARY(ACos, 0, return acos(x);)
ND_UNARY(ASin, 0, return asin(x);)
ND_UNARY(ATan, 0, return atan(x);)
ND_UNARY(HardTanh, 0, return x < C(-1) ? C(-1) : (x > C(1) ? C(1) : x);)
ND_UNARY(SoftSign, 0, return x / (C(1) + absv(x));)
ND_UNARY(ELU, 0, return x >= C(0) ? x : expv(x) - C(1);)
ND_UNARY(ELUDerivative, 0, return x >= C(0) ? C(1) : expv(x);)
ND_UNARY(TanhDerivative, 0, C t = tanhv(x); return C(1) - t * t;)
ND_UNARY(TimesOneMinus, 0, return x * (C(1) - x);)
ND_UNARY(HardTanhDerivative, 0, return (x >= C(-1) && x <= C(1)) ? C(1) : C(0);)
ND_UNARY(Ones, 0, return C(1);)
ND_UNARY(Identity, 0, return x;)
ND_UNARY(Stabilize, 1,
         C k = p[0];
         if (x * k > C(-ND_MIN_CUTOFF)) return C(-ND_MIN_CUTOFF) / k;
         if (x * k < C(ND_MIN_CUTOFF)) return C(ND_MIN_CUTOFF) / k;
         return x;)
ND_UNARY(SigmoidDerivative, 0, C s = sigmoid(x); return s * (C(1) - s);)
ND_UNARY(SoftSignDerivative, 0, C y = C(1) + absv(x); return C(1) / (y * y);)
ND_UNARY(LeakyRELU, 1, return x < C(0) ? p[0] * x : x;)
ND_UNARY(LeakyRELUDerivative, 1, return x >= C(0) ? C(1) : p[0];)
ND_UNARY(RELU, 1, return x < p[0] ? p[0] : x;)
ND_UNARY(Step, 1, return x > p[0] ? C(1) : C(0);)
ND_UNARY(OneMinus, 0, return C(1) - x;)
ND_UNARY(SpecialDerivative, 0, return x * (C(1) - x);)
ND_UNARY(CompareAndSetT, 4,
         int r = condition(x, p[0], p[2], (int) p[3]);
         return r > 0 ? p[1] : x;)
ND_UNARY(ReplaceNans, 1, return isnanv(x) ? p[0] : x;)
ND_UNARY(StabilizeFP16, 0, return x <= C(0) ? C(0.001) : x;)
ND_UNARY(Cube, 0, return x * x * x;)
ND_UNARY(CubeDerivative, 0, return C(3) * x * x;)
ND_UNARY(HardSigmoid, 0, return minv(C(1), maxv(C(0), C(0.2f) * x + C(0.5f)));)
ND_UNARY(HardSigmoidDerivative, 0, return (x < C(-2.5f) || x > C(2.5f)) ? C(0) : C(0.2f);)
ND_UNARY(RationalTanh, 0,
         C d = (C(2) / C(3)) * x;
         C d2 = d * d; C t = sgn(d) * (C(1) - (C(1) / (C(1) + absv(d) + d2 + C(1.41645f) * (d2 * d2))));
         return C(1.7159f) * t;)
ND_UNARY(RationalTanhDerivative, 0,
         C d = (C(2) / C(3)) * x;
         C d2 = d * d; C a = C(1) + absv(d) + d2 + C(1.41645f) * (d2 * d2);
         C t = (C(1) + sgn(d) * (C(2) * d + C(4) * C(1.41645f) * (d2 * d))) / (a * a);
         return C(1.7159f) * (C(2) / C(3)) * t;)
ND_UNARY(LogX, 1, return log(x) / log(p[0]);)
ND_UNARY(Not, 1, return x == p[0] ? C(1) : C(0);)
ND_UNARY(RectifiedTanh, 0, return maxv(C(0), tanhv(x));)
ND_UNARY(RectifiedTanhDerivative, 0, if (x > C(0)) { C t = tanhv(x); return C(1) - t * t; } return C(0);)
ND_UNARY(Sinh, 0, return sinh(x);)
ND_UNARY(Cosh, 0, return cosh(x);)
ND_UNARY(Tan, 0, return tan(x);)
ND_UNARY(TanDerivative, 0, C c = cos(x); return C(1) / (c * c);)
ND_UNARY(SELU, 0,
         return x > C(0) ? C(ND_SELU_LAMBDA) * x
                         : C(ND_SELU_LAMBDA) * (C(ND_SELU_ALPHA) * expv(x) - C(ND_SELU_ALPHA));)
ND_UNARY(SELUDerivative, 0,
         return x > C(0) ? C(ND_SELU_LAMBDA) : C(ND_SELU_ALPHA) * C(ND_SELU_LAMBDA) * expv(x);)
ND_UNARY(MatchConditionT, 3,
         int r = condition(x, p[0], p[1], (int) p[2]);
         return r < 0 ? x : C(r);)
ND_UNARY(ClipByValue, 2, return x > p[1] ? p[1] : (x < p[0] ? p[0] : x);)
ND_UNARY(Swish, 0, return x * sigmoid(x);)
ND_UNARY(SwishDerivative, 0,
         C ex = pow(C(ND_E), x);
         C e1 = C(double(ex) + 1.); return C((double(ex) * (double(x) + double(ex) + 1.)) / double(e1 * e1));)
ND_UNARY(RSqrt, 0, return C(1) / sqrt(x);)
ND_UNARY(Log1p, 0, return log(C(1) + x);)
ND_UNARY(Erf, 0, return erf(x);)
ND_UNARY(IsInf, 0, return isinfv(x) ? C(1) : C(0);)
ND_UNARY(IsNan, 0, return isnanv(x) ? C(1) : C(0);)
ND_UNARY(IsFinite, 0, return isfinite(x) ? C(1) : C(0);)
ND_UNARY(ACosh, 0, return acosh(x);)
ND_UNARY(ACoshDerivative, 0, return C(1) / (sqrt(x - C(1)) * sqrt(x + C(1)));)
ND_UNARY(ASinh, 0, return log(sqrt(x * x + C(1)) + x);)
ND_UNARY(ASinhDerivative, 0, return C(1) / sqrt(x * x + C(1));)
ND_UNARY(SinhDerivative, 0, return cosh(x);)
ND_UNARY(Rint, 0, return rint(x);)
ND_UNARY(LogSigmoid, 0, return log(sigmoid(x));)
ND_UNARY(LogSigmoidDerivative, 0, C ex = pow(C(ND_E), x); return C(1) / (ex + C(1));)
ND_UNARY(Erfc, 0, return erfc(x);)
ND_UNARY(Expm1, 0, return expv(x) - C(1);)
ND_UNARY(PowDerivativeT, 1, return p[0] * pow(x, p[0] - C(1));)
ND_UNARY(ATanh, 0, return atanh(x);)
ND_UNARY(Reciprocal, 0, return C(1) / x;)
ND_UNARY(Sqr, 0, return x * x;)
ND_UNARY(RELU6, 1, C r = x < p[0] ? p[0] : x; return r < C(6) ? r : C(6);)

// opNum -> functor. Composite transforms (Col2Im 36, Im2col 37, SoftMax 38, SoftMaxDerivative
// 39, LogSoftMax 40, IsMax 41, Histogram 48, Reverse 70, Pooling2D 71) and the two
// non-reproducible dropouts (43, 44: host rand()/device clock in the reference) are not
// elementwise functors and are reported as unsupported by the dispatcher.
#define ND_TRANSFORM_TABLE(X)                                                                     \
    X(0, Abs) X(1, Ceiling) X(2, Cosine) X(3, Exp) X(4, Floor) X(5, Log) X(6, Neg) X(7, PowT)     \
    X(8, Round) X(9, SetRange) X(10, Sigmoid) X(11, Sign) X(12, Sin) X(13, SoftPlus) X(14, Sqrt)  \
    X(15, Tanh) X(16, ACos) X(17, ASin) X(18, ATan) X(19, HardTanh) X(20, SoftSign) X(21, ELU)    \
    X(22, ELUDerivative) X(23, TanhDerivative) X(24, TimesOneMinus) X(25, HardTanhDerivative)     \
    X(26, Ones) X(27, Identity) X(28, Stabilize) X(29, SigmoidDerivative)                         \
    X(30, SoftSignDerivative) X(31, LeakyRELU) X(32, LeakyRELUDerivative) X(33, RELU) X(34, Step) \
    X(35, OneMinus) X(42, SpecialDerivative) X(45, CompareAndSetT) X(46, ReplaceNans)             \
    X(47, StabilizeFP16) X(49, Cube) X(50, CubeDerivative) X(51, HardSigmoid)                     \
    X(52, HardSigmoidDerivative) X(53, RationalTanh) X(54, RationalTanhDerivative) X(55, LogX)    \
    X(59, Not) X(61, RectifiedTanh) X(62, RectifiedTanhDerivative) X(63, Sinh) X(64, Cosh)        \
    X(65, Tan) X(66, TanDerivative) X(67, SELU) X(68, SELUDerivative) X(72, MatchConditionT)      \
    X(73, ClipByValue) X(74, Swish) X(75, SwishDerivative) X(76, RSqrt) X(77, Log1p) X(78, Erf)   \
    X(79, IsInf) X(80, IsNan) X(81, IsFinite) X(82, ACosh) X(83, ACoshDerivative) X(84, ASinh)    \
    X(85, ASinhDerivative) X(86, SinhDerivative) X(87, Rint) X(88, LogSigmoid)                    \
    X(89, LogSigmoidDerivative) X(90, Erfc) X(91, Expm1) X(92, PowDerivativeT) X(93, ATanh)       \
    X(94, Reciprocal) X(95, Sqr) X(96, RELU6)

// =============================================================================================
// Binary functors: z = f(x, y, p). Used by pairwise (y = second array), scalar (y = the
// scalar) and broadcast (y = vector element; the reference calls the parameter-less overload
// there, which for the ops below computes the same thing except AMax/AMin, see B* variants).
// =============================================================================================
#define ND_BINARY(Name, NP, ...)                                                  \
    struct Name {                                                                 \
        static constexpr int kParams = NP;                                        \
        template <class C> ND_D static C f(C x, C y, const C *p) { __VA_ARGS__ }  \
    };

ND_BINARY(Add, 0, return x + y;)
ND_BINARY(Subtract, 0, return x - y;)
ND_BINARY(Multiply, 0, return x * y;)
ND_BINARY(Divide, 0, return x / y;)
ND_BINARY(ReverseDivide, 0, return y / x;)
ND_BINARY(ReverseSubtract, 0, return y - x;)
ND_BINARY(Copy, 0, return y;)
ND_BINARY(EqualTo, 0, return C(x == y);)
ND_BINARY(NotEqualTo, 0, return C(x != y);)
ND_BINARY(GreaterThan, 0, return C(x > y);)
ND_BINARY(GreaterThanOrEqual, 0, return C(x >= y);)
ND_BINARY(LessThan, 0, return C(x < y);)
ND_BINARY(LessThanOrEqual, 0, return C(x <= y);)
ND_BINARY(Max, 0, return maxv(x, y);)
ND_BINARY(Min, 0, return minv(x, y);)
ND_BINARY(BAMax, 0, return absv(x) > absv(y) ? x : y;)   // broadcast form keeps the sign (ops.h 2-arg op)
ND_BINARY(BAMin, 0, return absv(x) < absv(y) ? x : y;)
ND_BINARY(SquaredSubtract, 0, C d = x - y; return d * d;)
ND_BINARY(FloorMod, 0,
          C m = fmod(x, y);
          return ((x < C(0)) == (y < C(0))) ? m : fmod(m + y, y);)
ND_BINARY(FloorDiv, 0, return floor(x / y);)
ND_BINARY(ReverseMod, 0, int b = (int) x; return b == 0 ? C(0) : C((int) y % b);)
ND_BINARY(SafeDivide, 0, return y == C(0) ? C(0) : x / y;)
ND_BINARY(Mod, 0, int b = (int) y; return b == 0 ? C(0) : C((int) x % b);)
ND_BINARY(TruncateDiv, 0, int b = (int) y; return b == 0 ? C(0) : C((int) x / b);)
ND_BINARY(Remainder, 0, return remainder(x, y);)
ND_BINARY(FMod, 0, return fmod(x, y);)
ND_BINARY(PowB, 0, return pow(x, y);)
ND_BINARY(Epsilon, 0, return absv(x - y) <= C(ND_MIN_EPS) ? C(1) : C(0);)
ND_BINARY(Axpy, 1, return p[0] * x + y;)
ND_BINARY(CompareAndSetB, 4,
          int mode = (int) p[3];
          // the reference tests y, except that modes 12 and 13 test x (ops.h:3722-3737)
          C probe = (mode == 12 || mode == 13) ? x : y;
          int r = condition(probe, p[0], p[2], mode);
          return r > 0 ? y : x;)
ND_BINARY(CompareAndReplace, 4,
          int r = condition(x, p[0], p[2], (int) p[3]);
          return r > 0 ? y : x;)
ND_BINARY(And, 1, return (x != p[0] && y != p[0]) ? C(1) : C(0);)
ND_BINARY(Or, 1, return (x != p[0] || y != p[0]) ? C(1) : C(0);)
ND_BINARY(Xor, 1, return ((x == p[0] && y != p[0]) || (x != p[0] && y == p[0])) ? C(1) : C(0);)
ND_BINARY(Atan2, 0, return atan2(y, x);)
ND_BINARY(RelativeError, 0, return rel_err(x, y);)
ND_BINARY(BinaryRelativeError, 1, return rel_err(x, y) > p[0] ? C(1) : C(0);)
ND_BINARY(BinaryMinimumAbsoluteRelativeError, 2,
          return rel_err(x, y) > p[0] ? (absv(x - y) < p[1] ? C(0) : C(1)) : C(0);)
ND_BINARY(PowDerivativeB, 0, return y * pow(x, y - C(1));)
ND_BINARY(LogPoisonLoss, 0, return expv(y) - x * y;)
ND_BINARY(LogPoisonLossFull, 0,
          return expv(y) - x * y + (x * log(x) - x + C(0.5) * log(C(2.0 * 3.14159265358979323846) * x));)

#define ND_PAIRWISE_TABLE(X)                                                                       \
    X(0, Add) X(1, Copy) X(2, Divide) X(3, EqualTo) X(4, GreaterThan) X(5, LessThan)               \
    X(6, Multiply) X(7, PowB) X(8, ReverseSubtract) X(9, Subtract) X(10, Epsilon)                  \
    X(11, GreaterThanOrEqual) X(12, LessThanOrEqual) X(13, Max) X(14, Min) X(15, NotEqualTo)       \
    X(16, Copy) X(17, Axpy) X(18, ReverseDivide) X(45, CompareAndSetB) X(46, CompareAndReplace)    \
    X(56, And) X(57, Or) X(58, Xor) X(59, Remainder) X(60, FMod) X(69, Atan2) X(19, TruncateDiv)   \
    X(20, FloorDiv) X(21, FloorMod) X(22, SquaredSubtract) X(23, ReverseMod) X(24, SafeDivide)     \
    X(25, Mod) X(26, RelativeError) X(27, BinaryRelativeError)                                     \
    X(28, BinaryMinimumAbsoluteRelativeError) X(92, PowDerivativeB) X(93, LogPoisonLoss)           \
    X(94, LogPoisonLossFull)

#define ND_SCALAR_TABLE(X)                                                                         \
    X(0, Add) X(1, Subtract) X(2, Multiply) X(3, Divide) X(4, ReverseDivide) X(5, ReverseSubtract) \
    X(6, Max) X(7, LessThan) X(8, GreaterThan) X(9, EqualTo) X(10, LessThanOrEqual)                \
    X(11, NotEqualTo) X(12, Min) X(13, Copy) X(14, Mod) X(15, ReverseMod)                          \
    X(16, GreaterThanOrEqual) X(17, Remainder) X(18, FMod) X(19, TruncateDiv) X(20, FloorDiv)      \
    X(21, FloorMod) X(22, SquaredSubtract) X(23, SafeDivide)

#define ND_BROADCAST_TABLE(X)                                                                      \
    X(0, Add) X(1, Subtract) X(2, Multiply) X(3, Divide) X(4, ReverseDivide) X(5, ReverseSubtract) \
    X(6, Copy) X(7, EqualTo) X(8, GreaterThan) X(9, GreaterThanOrEqual) X(10, LessThan)            \
    X(11, LessThanOrEqual) X(12, NotEqualTo) X(13, Min) X(14, Max) X(15, BAMin) X(16, BAMax)       \
    X(17, SquaredSubtract) X(18, FloorMod) X(19, FloorDiv) X(20, ReverseMod) X(21, SafeDivide)     \
    X(22, Mod) X(23, TruncateDiv)

// =============================================================================================
// Reductions: out = post(fold(combine, map(x_i)), n)      (REDUCE_OPS, legacy_ops.h:195-221)
// The reference folds sequentially with update(acc, op(x)) starting from startingValue; the
// formulations below are the associative equivalents (identity + map + combine), so partial
// results of warps and blocks can be merged in any fixed tree order.
// =============================================================================================
#define ND_REDUCE(Name, NP, IDENT, MAP, COMB, POST)                                   \
    struct Name {                                                                     \
        static constexpr int kParams = NP;                                            \
        template <class C> ND_D static C identity() { return IDENT; }                 \
        template <class C> ND_D static C map(C x, const C *p) { MAP }                 \
        template <class C> ND_D static C combine(C a, C b) { COMB }                   \
        template <class C> ND_D static C post(C r, LL n, const C *p) { POST }         \
    };

#define ND_INF(C) (sizeof(C) == 8 ? C(CUDART_INF) : C(CUDART_INF_F))

ND_REDUCE(RMean, 0, C(0), return x;, return a + b;, return r / C((int) n);)
ND_REDUCE(RSum, 0, C(0), return x;, return a + b;, return r;)
ND_REDUCE(RMax, 0, -ND_INF(C), return x;, return maxv(a, b);, return r;)
ND_REDUCE(RMin, 0, ND_INF(C), return x;, return minv(a, b);, return r;)
ND_REDUCE(RNorm1, 0, C(0), return absv(x);, return a + b;, return r;)
ND_REDUCE(RNorm2, 0, C(0), return x * x;, return a + b;, return sqrt(r);)
ND_REDUCE(RNormMax, 0, C(0), return absv(x);, return maxv(a, b);, return r;)
ND_REDUCE(RProd, 0, C(1), return x;, return a * b;, return r;)
ND_REDUCE(RVariance, 2, C(0), C d = x - p[0]; return d * d;, return a + b;,
          return (r - ((p[1] * p[1]) / C((int) n))) / C(n - 1);)
ND_REDUCE(RStandardDeviation, 2, C(0), C d = x - p[0]; return d * d;, return a + b;,
          return sqrt((r - ((p[1] * p[1]) / C((int) n))) / C(n - 1));)
ND_REDUCE(RASum, 0, C(0), return absv(x);, return a + b;, return absv(r);)
ND_REDUCE(RMatchCondition, 3, C(0), int c = condition(x, p[0], p[1], (int) p[2]); return c < 0 ? x : C(c);,
          return a + b;, return r;)
ND_REDUCE(RAMax, 0, C(0), return absv(x);, return maxv(a, b);, return absv(r);)
ND_REDUCE(RAMin, 0, ND_INF(C), return absv(x);, return minv(a, b);, return absv(r);)
ND_REDUCE(RAMean, 0, C(0), return absv(x);, return a + b;, return absv(r) / C((int) n);)
ND_REDUCE(REntropy, 0, C(0), return x * log(x);, return a + b;, return r;)
ND_REDUCE(RLogEntropy, 0, C(0), return log(x * x);, return a + b;, return r;)
ND_REDUCE(RShannonEntropy, 0, C(0), C s = x * x; return s * log(s);, return a + b;, return -r;)
ND_REDUCE(RAny, 0, C(0), return x;, return a + b;, return r > C(0) ? C(1) : C(0);)
ND_REDUCE(RAll, 0, C(1), return x;, return a * b;, return r > C(0) ? C(1) : C(0);)
ND_REDUCE(RCountNonZero, 0, C(0), return x == C(0) ? C(0) : C(1);, return a + b;, return r;)
ND_REDUCE(RNormFrobenius, 0, C(0), C v = absv(x); return v * v;, return a + b;, return sqrt(r);)
ND_REDUCE(RNormP, 1, C(0), return pow(absv(x), p[0]);, return a + b;, return pow(r, C(1) / p[0]);)
ND_REDUCE(RSquaredNorm, 0, C(0), return x * x;, return a + b;, return r;)
ND_REDUCE(RCountZero, 0, C(0), return x == C(0) ? C(1) : C(0);, return a + b;, return r;)
#define ND_REDUCE_TABLE(X)                                                                          \
    X(0, RMean) X(1, RSum) X(3, RMax) X(4, RMin) X(5, RNorm1) X(6, RNorm2) X(7, RNormMax)           \
    X(8, RProd) X(9, RStandardDeviation) X(10, RVariance) X(11, RASum) X(12, RMatchCondition)       \
    X(13, RAMax) X(14, RAMin) X(15, RAMean) X(16, REntropy) X(17, RLogEntropy)                      \
    X(18, RShannonEntropy) X(20, RAny) X(21, RAll) X(22, RCountNonZero)           \
    X(23, RNormFrobenius) X(24, RNormP) X(25, RSquaredNorm) X(26, RCountZero)

}  // namespace fn
}  // namespace nd4jb200
