/*
 * TEST INFRASTRUCTURE ONLY -- never linked into or called from the product library.
 *
 * Plain-C restatement of the reference's CPU algorithms for the legacy op families, written as
 * opNum switches over dense float32 / float64 data. oracle/port.py gathers strided operands into
 * dense TAD matrices (using its own restatement of the shapeInfo / TAD decoding) and scatters
 * results back, so everything here sees unit-stride rows.
 *
 * Parity status: pinned. tests/test_oracle.py checks every function below against the
 * reference's own CPU build (oracle/_ref, compiled from the reference sources) on seeded inputs
 * and against the golden vectors under tests/golden/ that were generated from that build.
 *
 * Build: gcc -O2 -fPIC -shared -ffp-contract=off -o _port.so port.c -lm   (oracle/port.py does it)
 * -ffp-contract=off keeps a*b+c as two roundings, like the reference's x86-64 baseline build.
 *
 * Sequential order matters for floating-point folds: the reference accumulates each TAD left to
 * right in T (include/loops/cpu/reduce.cpp:147-166), and so do these loops.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

typedef long long LL;

/* ---- shared predicate: MatchCondition / CompareAndSet / CompareAndReplace modes
 *      (include/ops/ops.h:1534-1602) ---------------------------------------------------------- */
static int cond_d(double v, double cmp, double eps, int mode) {
    switch (mode) {
        case 0: return fabs(v - cmp) <= eps;
        case 1: return fabs(v - cmp) > eps;
        case 2: return v < cmp;
        case 3: return v > cmp;
        case 4: return v <= cmp;
        case 5: return v >= cmp;
        case 6: return fabs(v) < cmp;
        case 7: return fabs(v) > cmp;
        case 8: return isinf(v);
        case 9: return isnan(v);
        case 10: return v == cmp;
        case 11: return v != cmp;
        case 12: return fabs(v) >= cmp;
        case 13: return fabs(v) <= cmp;
        default: return -1;
    }
}

#define SELU_ALPHA 1.6732632423543772848170429916717
#define SELU_LAMBDA 1.0507009873554804934193349852946
#define CUTOFF (-3.79297773665f)

/* ---- transform family, float32 (formulas: include/ops/ops.h:723-1845; math through libm as in
 *      include/templatemath.h:528-990) ---------------------------------------------------------- */
static float sigmoidf_(float x) { return 1.0f / (1.0f + expf(-x)); }
static float sgnf_(float x) { return x < 0.0f ? -1.0f : (x > 0.0f ? 1.0f : 0.0f); }

static float transform_f32(int op, float x, const float *p) {
    switch (op) {
        case 0: return fabsf(x);
        case 1: return ceilf(x);
        case 2: return cosf(x);
        case 3: return expf(x);
        case 4: return floorf(x);
        case 5: return logf(x);
        case 6: return -x;
        case 7: return powf(x, p[0]);
        case 8: return roundf(x);
        case 9: {
            float lo = p[0], hi = p[1];
            if (x >= lo && x <= hi) return x;
            if (lo == 0.0f && hi == 1.0f) { float v = 1.0f / (1.0f + expf(-x)); return floorf(v * (hi - lo)) + lo; }
            return floorf(x * (hi - lo)) + lo;
        }
        case 10: return sigmoidf_(x);
        case 11: return (float) ((x > 0.0f) - (x < 0.0f));
        case 12: return sinf(x);
        case 13: return logf(1.0f + expf(x));
        case 14: return sqrtf(x);
        case 15: return tanhf(x);
        case 16: return acosf(x);
        case 17: return asinf(x);
        case 18: return atanf(x);
        case 19: return x < -1.0f ? -1.0f : (x > 1.0f ? 1.0f : x);
        case 20: return x / (1.0f + fabsf(x));
        case 21: return x >= 0.0f ? x : expf(x) - 1.0f;
        case 22: return x >= 0.0f ? 1.0f : expf(x);
        case 23: { float t = tanhf(x); return 1.0f - t * t; }
        case 24: return x * (1.0f - x);
        case 25: return (x >= -1.0f && x <= 1.0f) ? 1.0f : 0.0f;
        case 26: return 1.0f;
        case 27: return x;
        case 28: {
            float k = p[0];
            if (x * k > -CUTOFF) return -CUTOFF / k;
            if (x * k < CUTOFF) return CUTOFF / k;
            return x;
        }
        case 29: { float s = sigmoidf_(x); return s * (1.0f - s); }
        case 30: { float y = 1.0f + fabsf(x); return 1.0f / (y * y); }
        case 31: return x < 0.0f ? p[0] * x : x;
        case 32: return x >= 0.0f ? 1.0f : p[0];
        case 33: return x < p[0] ? p[0] : x;
        case 34: return x > p[0] ? 1.0f : 0.0f;
        case 35: return 1.0f - x;
        case 42: return x * (1.0f - x);
        case 45: return cond_d(x, p[0], p[2], (int) p[3]) > 0 ? p[1] : x;
        case 46: return isnan(x) ? p[0] : x;
        case 47: return x <= 0.0f ? 0.001f : x;
        case 49: return x * x * x;
        case 50: return 3.0f * (x * x);   /* the reference build (associative-math) squares first */
        case 51: { float v = 0.2f * x + 0.5f; v = v > 0.0f ? v : 0.0f; return v < 1.0f ? v : 1.0f; }
        case 52: return (x < -2.5f || x > 2.5f) ? 0.0f : 0.2f;
        case 53: {
            float d = (2.0f / 3.0f) * x;
            float t = sgnf_(d) * (1.0f - (1.0f / (1.0f + fabsf(d) + powf(d, 2.0f) + 1.41645f * powf(d, 4.0f))));
            return 1.7159f * t;
        }
        case 54: {
            float d = (2.0f / 3.0f) * x;
            float a = 1.0f + fabsf(d) + powf(d, 2.0f) + 1.41645f * powf(d, 4.0f);
            float t = (1.0f + sgnf_(d) * (2.0f * d + 4.0f * 1.41645f * powf(d, 3.0f))) / (a * a);
            return 1.7159f * (2.0f / 3.0f) * t;
        }
        case 55: return logf(x) / logf(p[0]);
        case 59: return x == p[0] ? 1.0f : 0.0f;
        case 61: { float t = tanhf(x); return t > 0.0f ? t : 0.0f; }
        case 62: { if (x > 0.0f) { float t = tanhf(x); return 1.0f - t * t; } return 0.0f; }
        case 63: return sinhf(x);
        case 64: return coshf(x);
        case 65: return tanf(x);
        case 66: return 1.0f / powf(cosf(x), 2.0f);
        case 67: return x > 0.0f ? (float) SELU_LAMBDA * x
                                 : (float) SELU_LAMBDA * ((float) SELU_ALPHA * expf(x) - (float) SELU_ALPHA);
        case 68: return x > 0.0f ? (float) SELU_LAMBDA : (float) SELU_ALPHA * (float) SELU_LAMBDA * expf(x);
        case 72: { int c = cond_d(x, p[0], p[1], (int) p[2]); return c < 0 ? x : (float) c; }
        case 73: return x > p[1] ? p[1] : (x < p[0] ? p[0] : x);
        case 74: return x * sigmoidf_(x);
        case 75: {
            float ex = powf((float) M_E, x);
            return (float) ((ex * (x + ex + 1.)) / powf((float) (ex + 1.), 2.0f));
        }
        case 76: return 1.0f / sqrtf(x);
        case 77: return logf(1 + x);
        case 78: return erff(x);
        case 79: return isinf(x) ? 1.0f : 0.0f;
        case 80: return isnan(x) ? 1.0f : 0.0f;
        case 81: return isfinite(x) ? 1.0f : 0.0f;
        case 82: return acoshf(x);
        case 83: return 1.0f / (sqrtf(x - 1.0f) * sqrtf(x + 1.0f));
        case 84: return logf(sqrtf(powf(x, 2.0f) + 1.0f) + x);
        case 85: return 1.0f / sqrtf(powf(x, 2.0f) + 1.0f);
        case 86: return coshf(x);
        case 87: return rintf(x);
        case 88: return logf(sigmoidf_(x));
        case 89: { float ex = powf((float) M_E, x); return 1.0f / (ex + 1.0f); }
        case 90: return erfcf(x);
        case 91: return expf(x) - 1.0f;
        case 92: return p[0] * powf(x, p[0] - 1.0f);
        case 93: return atanhf(x);
        case 94: return 1.0f / x;
        case 95: return powf(x, 2.0f);
        case 96: { float r = x < p[0] ? p[0] : x; return r < 6.0f ? r : 6.0f; }
        default: return NAN;
    }
}

void port_transform_f32(int op, const float *x, float *z, LL n, const float *p) {
    for (LL i = 0; i < n; i++) z[i] = transform_f32(op, x[i], p);
}

/* ---- binary functors, float32. table: 0 pairwise, 1 scalar, 2 broadcast numbering
 *      (include/loops/legacy_ops.h:20-44, 153-177, 243-283); formulas include/ops/ops.h:77-720 - */
enum { B_ADD, B_SUB, B_MUL, B_DIV, B_RDIV, B_RSUB, B_COPY, B_EQ, B_NE, B_GT, B_GE, B_LT, B_LE, B_MAX, B_MIN,
       B_AMAXS, B_AMINS, B_SQSUB, B_FLOORMOD, B_FLOORDIV, B_RMOD, B_SAFEDIV, B_MOD, B_TRUNCDIV, B_REM, B_FMOD,
       B_POW, B_EPS, B_AXPY, B_CAS, B_CAR, B_AND, B_OR, B_XOR, B_ATAN2, B_RE, B_BRE, B_BMARE, B_POWD, B_LPL, B_LPLF,
       B_NONE };

static int binary_code(int table, int op) {
    static const int pairwise[][2] = {
        {0, B_ADD}, {1, B_COPY}, {2, B_DIV}, {3, B_EQ}, {4, B_GT}, {5, B_LT}, {6, B_MUL}, {7, B_POW}, {8, B_RSUB},
        {9, B_SUB}, {10, B_EPS}, {11, B_GE}, {12, B_LE}, {13, B_MAX}, {14, B_MIN}, {15, B_NE}, {16, B_COPY},
        {17, B_AXPY}, {18, B_RDIV}, {45, B_CAS}, {46, B_CAR}, {56, B_AND}, {57, B_OR}, {58, B_XOR}, {59, B_REM},
        {60, B_FMOD}, {69, B_ATAN2}, {19, B_TRUNCDIV}, {20, B_FLOORDIV}, {21, B_FLOORMOD}, {22, B_SQSUB},
        {23, B_RMOD}, {24, B_SAFEDIV}, {25, B_MOD}, {26, B_RE}, {27, B_BRE}, {28, B_BMARE}, {92, B_POWD},
        {93, B_LPL}, {94, B_LPLF}, {-1, B_NONE}};
    static const int scalar[] = {B_ADD, B_SUB, B_MUL, B_DIV, B_RDIV, B_RSUB, B_MAX, B_LT, B_GT, B_EQ, B_LE, B_NE, B_MIN,
                                 B_COPY, B_MOD, B_RMOD, B_GE, B_REM, B_FMOD, B_TRUNCDIV, B_FLOORDIV, B_FLOORMOD,
                                 B_SQSUB, B_SAFEDIV};
    static const int broadcast[] = {B_ADD, B_SUB, B_MUL, B_DIV, B_RDIV, B_RSUB, B_COPY, B_EQ, B_GT, B_GE, B_LT, B_LE,
                                    B_NE, B_MIN, B_MAX, B_AMINS, B_AMAXS, B_SQSUB, B_FLOORMOD, B_FLOORDIV, B_RMOD,
                                    B_SAFEDIV, B_MOD, B_TRUNCDIV};
    if (table == 0) { for (int i = 0; pairwise[i][0] >= 0; i++) if (pairwise[i][0] == op) return pairwise[i][1]; return B_NONE; }
    if (table == 1) return (op >= 0 && op < 24) ? scalar[op] : B_NONE;
    return (op >= 0 && op < 24) ? broadcast[op] : B_NONE;
}

static float re_f32(float a, float b) { if (a == 0.0f && b == 0.0f) return 0.0f; return fabsf(a - b) / (fabsf(a) + fabsf(b)); }

static float binary_f32(int code, float x, float y, const float *p) {
    switch (code) {
        case B_ADD: return x + y;
        case B_SUB: return x - y;
        case B_MUL: return x * y;
        case B_DIV: return x / y;
        case B_RDIV: return y / x;
        case B_RSUB: return y - x;
        case B_COPY: return y;
        case B_EQ: return x == y;
        case B_NE: return x != y;
        case B_GT: return x > y;
        case B_GE: return x >= y;
        case B_LT: return x < y;
        case B_LE: return x <= y;
        case B_MAX: return x > y ? x : y;
        case B_MIN: return x < y ? x : y;
        case B_AMAXS: return fabsf(x) > fabsf(y) ? x : y;
        case B_AMINS: return fabsf(x) < fabsf(y) ? x : y;
        case B_SQSUB: return powf(x - y, 2.0f);
        case B_FLOORMOD: { float m = fmodf(x, y); return ((x < 0.0f) == (y < 0.0f)) ? m : fmodf(m + y, y); }
        case B_FLOORDIV: return floorf(x / y);
        case B_RMOD: return (float) ((int) y % (int) x);
        case B_SAFEDIV: return y == 0.0f ? 0.0f : x / y;
        case B_MOD: return (float) ((int) x % (int) y);
        case B_TRUNCDIV: return (float) ((int) x / (int) y);
        case B_REM: return remainderf(x, y);
        case B_FMOD: return fmodf(x, y);
        case B_POW: return powf(x, y);
        case B_EPS: return fabsf(x - y) <= (float) 1e-12 ? 1.0f : 0.0f;
        case B_AXPY: return p[0] * x + y;
        case B_CAS: { int mode = (int) p[3]; float probe = (mode == 12 || mode == 13) ? x : y;
                      return cond_d(probe, p[0], p[2], mode) > 0 ? y : x; }
        case B_CAR: return cond_d(x, p[0], p[2], (int) p[3]) > 0 ? y : x;
        case B_AND: return (x != p[0] && y != p[0]) ? 1.0f : 0.0f;
        case B_OR: return (x != p[0] || y != p[0]) ? 1.0f : 0.0f;
        case B_XOR: return ((x == p[0] && y != p[0]) || (x != p[0] && y == p[0])) ? 1.0f : 0.0f;
        case B_ATAN2: return atan2f(y, x);
        case B_RE: return re_f32(x, y);
        case B_BRE: return re_f32(x, y) > p[0] ? 1.0f : 0.0f;
        case B_BMARE: return re_f32(x, y) > p[0] ? (fabsf(x - y) < p[1] ? 0.0f : 1.0f) : 0.0f;
        case B_POWD: return y * powf(x, y - 1.0f);
        case B_LPL: return expf(y) - x * y;
        case B_LPLF: return expf(y) - x * y + (x * logf(x) - x + 0.5f * logf((float) (2.0 * 3.14159265358979323846) * x));
        default: return NAN;
    }
}

/* z[i] = f(x[i], y[i * ystep]); ystep 0 applies one value to every element (scalar family) */
int port_binary_f32(int table, int op, const float *x, const float *y, LL ystep, float *z, LL n, const float *p) {
    int code = binary_code(table, op);
    if (code == B_NONE) return 1;
    for (LL i = 0; i < n; i++) z[i] = binary_f32(code, x[i], y[i * ystep], p);
    return 0;
}

/* ---- reduce family, float32: rows of a dense [tads, len] matrix folded left to right in float
 *      (include/loops/cpu/reduce.cpp:147-166; functors include/ops/ops.h:1846-2565) ----------- */
int port_reduce_f32(int op, const float *x, LL tads, LL len, float *z, const float *p) {
    for (LL r = 0; r < tads; r++) {
        const float *t = x + r * len;
        float acc;
        LL n = len;
        switch (op) {
            case 0: case 1: case 5: case 6: case 11: case 15: case 16: case 17: case 18: case 20: case 22: case 23:
            case 24: case 25: case 26: case 9: case 10: case 12: case 19: {
                float mx = 0.0f;
                if (op == 19) { mx = t[0]; for (LL j = 0; j < n; j++) mx = t[j] > mx ? t[j] : mx; }
                acc = 0.0f;
                for (LL j = 0; j < n; j++) {
                    float v = t[j], m;
                    switch (op) {
                        case 5: case 11: case 15: m = fabsf(v); break;
                        case 6: case 25: m = v * v; break;
                        case 23: { float a = fabsf(v); m = a * a; break; }
                        case 16: m = v * logf(v); break;
                        case 17: m = logf(powf(v, 2.0f)); break;
                        case 18: m = powf(v, 2.0f) * logf(powf(v, 2.0f)); break;
                        case 22: m = v == 0.0f ? 0.0f : 1.0f; break;
                        case 26: m = v == 0.0f ? 1.0f : 0.0f; break;
                        case 24: m = powf(fabsf(v), p[0]); break;
                        case 9: case 10: { float d = v - p[0]; m = d * d; break; }
                        case 12: { int c = cond_d(v, p[0], p[1], (int) p[2]); m = c < 0 ? v : (float) c; break; }
                        case 19: m = expf(v - mx); break;
                        default: m = v;
                    }
                    acc = (op == 11 || op == 15) ? fabsf(m) + fabsf(acc) : m + acc;
                }
                if (op == 0) acc = acc / (int) n;
                else if (op == 6 || op == 23) acc = sqrtf(acc);
                else if (op == 11) acc = fabsf(acc);
                else if (op == 15) acc = fabsf(acc) / (int) n;
                else if (op == 18) acc = -acc;
                else if (op == 20) acc = acc > 0.0f ? 1.0f : 0.0f;
                else if (op == 24) acc = powf(acc, 1.0f / p[0]);
                else if (op == 10 || op == 9) {
                    acc = (acc - (powf(p[1], 2.0f) / (int) n)) / (n - 1);
                    if (op == 9) acc = sqrtf(acc);
                } else if (op == 19) acc = mx + logf(acc);
                break;
            }
            case 3: acc = t[0]; for (LL j = 0; j < n; j++) acc = t[j] > acc ? t[j] : acc; break;
            case 4: acc = t[0]; for (LL j = 0; j < n; j++) acc = t[j] < acc ? t[j] : acc; break;
            case 7: acc = 0.0f; for (LL j = 0; j < n; j++) acc = fabsf(acc) > fabsf(t[j]) ? fabsf(acc) : fabsf(t[j]); break;
            case 13: acc = t[0]; for (LL j = 0; j < n; j++) acc = fabsf(t[j]) > fabsf(acc) ? fabsf(t[j]) : fabsf(acc); acc = fabsf(acc); break;
            case 14: acc = t[0]; for (LL j = 0; j < n; j++) acc = fabsf(t[j]) < fabsf(acc) ? fabsf(t[j]) : fabsf(acc); acc = fabsf(acc); break;
            case 8: acc = 1.0f; for (LL j = 0; j < n; j++) acc = t[j] * acc; break;
            case 21: acc = 1.0f; for (LL j = 0; j < n; j++) acc = t[j] * acc; acc = acc > 0.0f ? 1.0f : 0.0f; break;
            default: return 1;
        }
        z[r] = acc;
    }
    return 0;
}

/* ---- index reduce, float32: strict comparisons scanned in order, so the first extreme wins
 *      (include/loops/cpu/indexreduce.cpp:208-224; include/ops/ops.h:2992-3470) -------------- */
int port_index_reduce_f32(int op, const float *x, LL tads, LL len, float *z, const float *p) {
    for (LL r = 0; r < tads; r++) {
        const float *t = x + r * len;
        LL idx = (op >= 4) ? -1 : 0;
        float best = op == 0 ? (float) -1e37 : (op == 2 ? (float) 1e-37 : (float) 1e37);
        for (LL j = 0; j < len; j++) {
            float v = t[j];
            if (op == 0) { if (v > best) { best = v; idx = j; } }
            else if (op == 1) { if (v < best) { best = v; idx = j; } }
            else if (op == 2) { if (fabsf(v) > fabsf(best)) { best = v; idx = j; } }
            else if (op == 3) { if (fabsf(v) < fabsf(best)) { best = v; idx = j; } }
            else if (op == 4 || op == 5) {
                int c = cond_d(v, p[0], p[1], (int) p[2]);
                float res = c < 0 ? v : (float) c;
                if (res == 0.0f) continue;
                if (idx < 0) idx = j;
                else if (op == 4 && idx > j) idx = j;
                else if (op == 5 && idx < j) idx = j;
            } else return 1;
        }
        z[r] = (float) idx;
    }
    return 0;
}

/* ---- summary stats: per-element Chan merge of (n, mean, M2) in double
 *      (include/loops/summarystatsreduce.h:221-257; getValue include/ops/ops.h:3471-3518) ---- */
int port_summary_stats_f32(int op, const float *x, LL tads, LL len, float *z, int biasCorrected) {
    if (op != 0 && op != 1) return 1;
    for (LL r = 0; r < tads; r++) {
        const float *t = x + r * len;
        double n = 0, mean = 0, m2 = 0;
        for (LL j = 0; j < len; j++) {
            double yn = 1, ymean = t[j];
            if (n == 0) { n = 1; mean = ymean; m2 = 0; continue; }
            double nn = n + yn, delta = ymean - mean;
            double nm = mean + delta * yn / nn;
            m2 = m2 + 0.0 + delta * delta * n * yn / nn;
            mean = nm; n = nn;
        }
        double var = n <= 1.0 ? 0.0 : m2 / n;
        if (biasCorrected) {
            double vb = n <= 1.0 ? 0.0 : m2 / (n - 1.0);
            if (!(vb < 0.0)) var = vb;
        }
        z[r] = (float) (op == 1 ? sqrt(var) : var);
    }
    return 0;
}

/* ---- reduce3, float32: row r of x against row r of y (ystep = len) or against one shared row
 *      (ystep = 0); accumulators and the two auxiliary sums live in float and restart per row
 *      (include/loops/reduce3.h:1236-1262; include/ops/ops.h:2567-2990) ---------------------- */
int port_reduce3_f32(int op, const float *x, const float *y, LL ystep, LL tads, LL len, float *z, float eps) {
    for (LL r = 0; r < tads; r++) {
        const float *a = x + r * len, *b = y + r * ystep;
        float acc = 0.0f, e0 = 0.0f, e1 = 0.0f;
        for (LL j = 0; j < len; j++) {
            float u = a[j], v = b[j];
            switch (op) {
                case 0: acc = acc + fabsf(u - v); break;
                case 1: { float d = u - v; acc = d * d + acc; break; }
                case 2: case 5: e0 += u * u; e1 += v * v; acc = acc + u * v; break;
                case 3: acc = u * v + acc; break;
                case 4: {
                    float diff = fabsf(u - v);
                    float m = fabsf(u) > fabsf(v) ? fabsf(u) : fabsf(v);
                    acc = ((diff <= eps || diff <= m * eps) ? 0.0f : 1.0f) + acc;
                    break;
                }
                case 6: e0 += u < v ? u : v; e1 += u > v ? u : v; break;
                case 7: acc = acc + (u == v ? 0.0f : 1.0f); break;
                default: return 1;
            }
        }
        if (op == 1) acc = sqrtf(acc);
        else if (op == 2) acc = acc / (sqrtf(e0) * sqrtf(e1));
        else if (op == 5) acc = 1.0f - acc / (sqrtf(e0) * sqrtf(e1));
        else if (op == 6) acc = 1.0f - e0 / e1;
        else if (op == 7) acc = acc / (float) len;
        z[r] = acc;
    }
    return 0;
}

/* ---- random family (include/helpers/helper_generator.h) --------------------------------------- */
typedef struct {
    LL size, position, generation, seed, amplifier;
    uint64_t *table;
} PortRng;

static uint64_t finalise(uint64_t x) {                       /* :244-250 */
    uint64_t z = x + 0x9E3779B97F4A7C15ULL;
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ULL;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBULL;
    return z ^ (z >> 31);
}
static uint64_t rotl(uint64_t x, int k) { return (x << k) | (x >> (64 - k)); }

void port_rng_fill(PortRng *g) {                             /* :575-621 */
    uint64_t s0 = finalise((uint64_t) g->seed), s1 = finalise((uint64_t) (g->seed * 119 + 3));
    for (LL i = 0; i < g->size; i++) {
        g->table[i] = s0 + s1;
        uint64_t t = s1 ^ s0;
        s0 = rotl(s0, 55) ^ t ^ (t << 14);
        s1 = rotl(t, 36);
    }
}
static uint64_t shift(uint64_t x, uint64_t y) {              /* :238-242 */
    if (y != 0 && x > UINT64_MAX / y) return x / y + 11;
    return x * y + 11;
}
static uint64_t mix(uint64_t s0) {                           /* :222-232 */
    uint64_t s1 = s0 % 2147483647ULL + 11;
    s1 ^= s0;
    return (rotl(s0, 55) ^ s1 ^ (s1 << 14)) + rotl(s1, 36);
}
uint64_t port_rng_element(const PortRng *g, LL e) {          /* :185-220 */
    LL p = g->position + e, gen = g->generation;
    if (p >= g->size) { gen += p / g->size; p = p % g->size; }
    uint64_t r = g->table[p];
    int touched = 0;
    if (gen != g->generation) { r = shift(r, (uint64_t) gen); touched = 1; }
    if (g->generation > 1) { r = shift(r, (uint64_t) g->generation); touched = 1; }
    if (g->amplifier != g->seed) { r = shift(r, (uint64_t) g->amplifier); touched = 1; }
    if (touched) r = mix(finalise(r));
    return r;
}
void port_rng_rewind(PortRng *g, LL n) {                     /* :322-334 */
    LL pos = g->position + n;
    if (pos > g->size) { g->generation += pos / g->size; pos = pos % g->size; }
    else if (pos == g->size) { g->generation++; pos = 0; }
    g->position = pos;
}
static float unit_f32(const PortRng *g, LL e) { return (float) port_rng_element(g, e) / 18446744073709551616.0f; }
static float range_f32(const PortRng *g, LL e, float from, float to) { return from + unit_f32(g, e) * (to - from); }

/* arity 0: z only, 1: x, 2: x and y (include/ops/random_ops.h:36-196, special_random_ops.h:333-396) */
int port_random_f32(int op, int arity, const PortRng *g, const float *x, const float *y, int yIsZ, float *z, LL n,
                    const float *p) {
    if (op == 6 || op == 10) {
        if (arity != 2) { for (LL e = 0; e < n; e++) z[e] = arity == 0 ? -1.0f : -2.0f; return 0; }
        const float twoPi = (float) (2.0 * 3.14159265358979323846);
        for (LL e = 0; e < n; e += 2) {
            float u0 = range_f32(g, e, 1e-5f, 1.0f), u1 = range_f32(g, e + 1, 1e-5f, 1.0f);
            float rad = sqrtf(-2.0f * logf(u0));
            float n0 = rad * cosf(twoPi * u1), n1 = rad * sinf(twoPi * u1);
            float m0 = yIsZ ? p[0] : y[e];
            z[e] = n0 * p[1] + m0;
            if (op == 10) z[e] = expf(z[e]);
            if (e + 1 < n) {
                float m1 = yIsZ ? p[0] : y[e + 1];
                z[e + 1] = n1 * p[1] + m1;
                if (op == 10) z[e + 1] = expf(z[e + 1]);
            }
        }
        return 0;
    }
    for (LL e = 0; e < n; e++) {
        float v = arity == 0 ? -1.0f : (arity == 1 ? -2.0f : -3.0f);
        switch (op) {
            case 0: if (arity == 0) v = range_f32(g, e, p[0], p[1]); break;
            case 1: if (arity == 1) v = unit_f32(g, e) >= p[0] ? 0.0f : x[e]; break;
            case 2: if (arity == 1) v = unit_f32(g, e) >= p[0] ? 0.0f : x[e] / p[0]; break;
            case 3: if (arity == 2) v = unit_f32(g, e) <= p[0] ? y[e] : x[e]; break;
            case 4: if (arity == 0) { float s = (float) e / ((float) n - 1.0f); v = p[0] * (1.0f - s) + s * p[1]; } break;
            case 7: if (arity == 0) v = p[0] >= unit_f32(g, e) ? 1.0f : 0.0f;
                    else if (arity == 1) v = x[e] >= unit_f32(g, e) ? 1.0f : 0.0f;
                    break;
            case 12: if (arity == 1) v = unit_f32(g, e) >= p[0] ? p[1] * p[3] + p[2] : p[1] * x[e] + p[2]; break;
            case 13: if (arity == 0) { float u = range_f32(g, e, 1.175494e-38f, 1.0f); v = 1.0f - powf((float) M_E, -(p[0] * u)); }
                     else if (arity == 1) v = x[e] <= 0.0f ? 0.0f : 1.0f - powf((float) M_E, -(p[0] * x[e]));
                     break;
            default: return 1;
        }
        z[e] = v;
    }
    return 0;
}
