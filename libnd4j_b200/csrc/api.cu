// C ABI of the backend (declared in include/nd4j_b200.h): argument validation, host-side
// shape/TAD decoding and hand-off to the per-type dispatchers. No compute happens on the host.
#include "../../include/nd4j_b200.h"
#include "dispatch.h"
#include <cmath>
#include <cstring>
#include <sstream>
#include <vector>

using namespace nd4jb200;

namespace {

#define BY_DTYPE(dtype, fname, ...)                                                      \
    ((dtype) == kF32 ? fname##_f32(__VA_ARGS__)                                          \
     : (dtype) == kF64 ? fname##_f64(__VA_ARGS__)                                        \
     : (dtype) == kF16 ? fname##_f16(__VA_ARGS__)                                        \
                       : bad_arg("dtype must be 0 (float), 1 (double) or 2 (half)"))

inline cudaStream_t as_stream(void *s) { return static_cast<cudaStream_t>(s); }
inline size_t dtype_size(int dtype) { return dtype == kF64 ? 8 : (dtype == kF16 ? 2 : 4); }

Status need(const void *p, const char *name) {
    if (p == nullptr) return bad_arg(std::string(name) + " is null");
    return kOk;
}

Status check_dtype(int dtype) {
    if (dtype != kF32 && dtype != kF64 && dtype != kF16) return bad_arg("dtype must be 0 (float), 1 (double) or 2 (half)");
    return kOk;
}

// Reads a device scalar of the call's element type back through the pinned slot.
Status fetch_scalar(cudaStream_t st, int dtype, const void *dev, void *hostSlot, double *out) {
    ND_CUDA(cudaMemcpyAsync(hostSlot, dev, dtype_size(dtype), cudaMemcpyDeviceToHost, st));
    ND_CUDA(cudaStreamSynchronize(st));
    if (dtype == kF32) *out = *static_cast<float *>(hostSlot);
    else if (dtype == kF64) *out = *static_cast<double *>(hostSlot);
    else *out = __half2float(*static_cast<__half *>(hostSlot));
    return kOk;
}

// Scratch large enough for the partial states of any single-TAD (whole array) reduction:
// at most kNumSMs * kMaxRowThreadsPerSm segments of the largest state (32 bytes), plus the result slot and
// counter region.
constexpr long long kMaxRowThreadsPerSm = 4096;
constexpr size_t kScalarWorkspace = 256 + kCounterSlots * sizeof(unsigned) + 32 * (size_t) kNumSMs * kMaxRowThreadsPerSm + 4096;

bool same_shape(const ShapeDesc &a, const ShapeDesc &b) {
    if (a.rank != b.rank) return false;
    for (int i = 0; i < a.rank; i++) if (a.shape[i] != b.shape[i]) return false;
    return true;
}

// Fills mode / strides / views of an elementwise call over operands that are iterated by one
// shared linear index. Operands listed as null are ignored.
Status setup_linear(const ShapeDesc *x, const ShapeDesc *y, const ShapeDesc *z, const void *px, const void *py,
                    const void *pz, EwArgs *a) {
    const ShapeDesc *ops[3] = {x, y, z};
    bool linear = true, dense = true;
    char order = 0;
    for (auto d : ops) {
        if (!d) continue;
        if (d->ews < 1) linear = false;
        if (d->ews != 1) dense = false;
        if (order == 0) order = d->order;
        else if (d->order != order && d->rank > 1) linear = false;   // rank<=1 arrays read the same in both orders
    }
    if (linear && x && y && !same_shape(*x, *y) && x->ews != y->ews) linear = false;
    a->sx = x ? x->ews : 0; a->sy = y ? y->ews : 0; a->sz = z ? z->ews : 0;
    if (linear && dense && aligned16(px) && (!y || aligned16(py)) && aligned16(pz)) { a->mode = 0; return kOk; }
    if (linear) { a->mode = 1; return kOk; }
    a->mode = 2;
    if (x) ND_TRY(coord_view(*x, &a->vx));
    if (y) ND_TRY(coord_view(*y, &a->vy)); else a->vy = a->vx;
    if (z) ND_TRY(coord_view(*z, &a->vz));
    return kOk;
}

struct ReduceSetup {
    ShapeDesc x, y, z;
    ReduceCall call;
    bool scalarResult = false;
};

// Common front half of the four reduction families.
Status setup_reduction(const void *x, const Nd4jLong *xShapeInfo, const void *y, const Nd4jLong *yShapeInfo,
                       const Nd4jLong *zShapeInfo, const int *dimension, int dimensionLength, bool forceWhole,
                       ReduceSetup *s) {
    ND_TRY(need(x, "x"));
    ND_TRY(parse_shape(xShapeInfo, "xShapeInfo", &s->x));
    LL zLen = -1;
    if (zShapeInfo) { ND_TRY(parse_shape(zShapeInfo, "zShapeInfo", &s->z)); zLen = s->z.length; }
    ND_TRY(make_tad_plan(s->x, dimension, dimensionLength, &s->call.xPlan));
    if (y) ND_TRY(parse_shape(yShapeInfo, "yShapeInfo", &s->y));
    // reduce3 with a short x: x is one TAD that meets every TAD of y
    const bool xIsOneTad = y && s->x.length < s->y.length && zLen != 1 && !forceWhole;
    // a single result means "whole array", whatever the dimension list says
    // (include/loops/cpu/reduce.cpp:108-111, include/loops/cpu/indexreduce.cpp:135-138)
    if (!xIsOneTad && (forceWhole || zLen == 1 || s->call.xPlan.numTads == 1))
        ND_TRY(make_tad_plan(s->x, nullptr, 0, &s->call.xPlan));
    s->scalarResult = s->call.xPlan.whole && !xIsOneTad;
    if (zLen >= 0 && !forceWhole && !xIsOneTad && zLen != s->call.xPlan.numTads) {
        std::ostringstream os;
        os << "result holds " << zLen << " elements but the dimension list yields " << s->call.xPlan.numTads << " TADs";
        return bad_arg(os.str());
    }
    s->call.x = x;
    s->call.finishLen = s->call.xPlan.tadLen;
    if (y) {
        TadPlan &xp = s->call.xPlan, &yp = s->call.yPlan;
        if (s->scalarResult) {
            if (s->x.length != s->y.length) return bad_arg("reduce3 over whole arrays needs x and y of equal length");
            ND_TRY(make_tad_plan(s->y, nullptr, 0, &yp));
            // operands are walked linearly only when both allow it in the same order
            // (include/loops/reduce3.h:862-884); otherwise element i is the i-th c-order coordinate
            bool lin = s->x.ews >= 1 && s->y.ews >= 1 && (s->x.order == s->y.order || (s->x.rank <= 1 && s->y.rank <= 1));
            if (!lin) { ND_TRY(coord_view(s->x, &xp.inner)); ND_TRY(coord_view(s->y, &yp.inner)); }
        } else if (s->y.length == s->x.length) {
            ND_TRY(make_tad_plan(s->y, dimension, dimensionLength, &yp));
            if (yp.numTads != xp.numTads || yp.tadLen != xp.tadLen) return bad_arg("x and y split into different TADs");
        } else if (s->y.length == xp.tadLen) {
            // one y TAD against every x TAD
            ND_TRY(make_tad_plan(s->y, nullptr, 0, &yp));
            yp.numTads = xp.numTads;
        } else {
            ND_TRY(make_tad_plan(s->y, dimension, dimensionLength, &yp));
            if (s->x.length != yp.tadLen) return bad_arg("x and y lengths are incompatible for reduce3");
            // one x TAD against every y TAD
            ND_TRY(make_tad_plan(s->x, nullptr, 0, &xp));
            xp.numTads = yp.numTads;
            s->call.finishLen = xp.tadLen;
            if (zLen >= 0 && zLen != yp.numTads) return bad_arg("result length does not match the number of y TADs");
        }
        s->call.y = y;
    }
    return kOk;
}

struct RandomState {
    LL size;
    unsigned long long *hostTable;
    unsigned long long *devTable;
    bool ownsHost, ownsDev;
    LL seed, generation, position, amplifier;
};

unsigned long long splitmix_finalise(unsigned long long x) {
    unsigned long long z = x + 0x9E3779B97F4A7C15ull;
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    return z ^ (z >> 31);
}

// Table fill: xoroshiro128+ seeded with finalise(seed) and finalise(seed*119+3), run
// sequentially (include/helpers/helper_generator.h:575-621). It runs once per (re)seed.
void fill_table(RandomState *s) {
    unsigned long long s0 = splitmix_finalise((unsigned long long) s->seed);
    unsigned long long s1 = splitmix_finalise((unsigned long long) (s->seed * 119 + 3));
    for (LL i = 0; i < s->size; i++) {
        s->hostTable[i] = s0 + s1;
        unsigned long long t = s1 ^ s0;
        s0 = ((s0 << 55) | (s0 >> 9)) ^ t ^ (t << 14);
        s1 = (t << 36) | (t >> 28);
    }
}

Status upload_table(RandomState *s, cudaStream_t st) {
    ND_CUDA(cudaMemcpyAsync(s->devTable, s->hostTable, sizeof(unsigned long long) * s->size, cudaMemcpyHostToDevice, st));
    ND_CUDA(cudaStreamSynchronize(st));
    return kOk;
}

void rewind_state(RandomState *s, LL n) {
    // RandomBuffer::rewindH (include/helpers/helper_generator.h:322-334)
    LL pos = s->position + n;
    if (pos > s->size) { s->generation += pos / s->size; pos = pos % s->size; }
    else if (pos == s->size) { s->generation++; pos = 0; }
    s->position = pos;
}

// f-order coordinate view: the random loops decode strided outputs with ind2sub
// (include/loops/cpu/random.cpp:64-66, 125-126, 175), i.e. first axis fastest.
Status forder_view(const ShapeDesc &d, View *out) {
    LL shp[kMaxRank], str[kMaxRank];
    for (int i = 0; i < d.rank; i++) { shp[i] = d.shape[d.rank - 1 - i]; str[i] = d.stride[d.rank - 1 - i]; }
    return collapse_view(d.rank, shp, str, out);
}

Status random_common(void *stream, int dtype, int opNum, int arity, RandomState *s, const void *x,
                     const ShapeDesc *xd, const void *y, const ShapeDesc *yd, void *z, const ShapeDesc *zd,
                     const void *extra, LL first, LL count, LL length) {
    RngArgs a;
    a.g.table = s->devTable; a.g.size = s->size; a.g.position = s->position;
    a.g.generation = s->generation; a.g.seed = s->seed; a.g.amplifier = s->amplifier;
    a.g.thrGeneration = s->generation ? 0xffffffffffffffffull / (unsigned long long) s->generation : 0ull;
    a.g.thrAmplifier = s->amplifier ? 0xffffffffffffffffull / (unsigned long long) s->amplifier : 0ull;
    a.chunk = 0;
    a.x = x; a.y = y; a.z = z; a.extra = extra;
    a.first = first; a.count = count; a.length = length;
    a.sx = a.sy = a.sz = 1; a.mode = 0; a.yIsZ = (y == z);
    a.vx.rank = a.vy.rank = a.vz.rank = 0;
    const bool gaussian = (opNum == 6 || opNum == 10) && arity == 2;
    if (zd) {
        bool linear = zd->ews >= 1 && (arity < 1 || gaussian || xd->ews >= 1) && (arity < 2 || yd->ews >= 1);
        bool dense = zd->ews == 1 && (arity < 1 || gaussian || xd->ews == 1) && (arity < 2 || yd->ews == 1);
        a.sz = zd->ews; a.sx = xd ? xd->ews : 1; a.sy = yd ? yd->ews : 1;
        if (dense) a.mode = 0;
        else if (linear) a.mode = 1;
        else {
            if (gaussian) return unsupported("the Gaussian family addresses z and y by elementWiseStride only");
            a.mode = 2;
            ND_TRY(forder_view(*zd, &a.vz));
            if (arity >= 1) ND_TRY(forder_view(*xd, &a.vx));
            if (arity == 2) ND_TRY(forder_view(*yd, &a.vy));
        }
    }
    if (a.mode == 0 && !(aligned16(z) && (arity < 1 || gaussian || aligned16(x)) && (arity < 2 || gaussian || aligned16(y)))) {
        a.mode = 1;
    }
    if (gaussian && (first & 1)) return bad_arg("the Gaussian family pairs elements (2k, 2k+1): `first` must be even");
    a.aux = nullptr; a.auxLen = 0;
    if ((opNum == 5 || opNum == 8 || opNum == 9 || opNum == 11) && arity == 2) {
        // Choice / Binomial / BinomialEx / TruncatedNormal: whole calls on operands addressed by elementWiseStride
        if (!zd || first != 0 || count != length)
            return unsupported("Choice, the binomial ops and TruncatedNormal are served for whole calls only");
        if (zd->ews < 1 || xd->ews < 1 || yd->ews < 1)
            return unsupported("Choice, the binomial ops and TruncatedNormal address their operands by elementWiseStride (>= 1)");
        a.mode = 1;
        if (opNum == 11 && a.yIsZ) {
            // with one mean for all elements the acceptance test |mean| + |result| <= 2 |stddev| can never hold once
            // |mean| >= 2 |stddev|: the reference would not return (special_random_ops.h:779-798)
            ND_TRY(need(extra, "extraArguments"));
            unsigned char raw[16] = {0};
            const size_t es = dtype == kF64 ? 8 : (dtype == kF32 ? 4 : 2);
            ND_CUDA(cudaMemcpyAsync(raw, extra, 2 * es, cudaMemcpyDeviceToHost, as_stream(stream)));
            ND_CUDA(cudaStreamSynchronize(as_stream(stream)));
            double mean, sd;
            if (dtype == kF64) { mean = reinterpret_cast<double *>(raw)[0]; sd = reinterpret_cast<double *>(raw)[1]; }
            else if (dtype == kF32) { mean = reinterpret_cast<float *>(raw)[0]; sd = reinterpret_cast<float *>(raw)[1]; }
            else { mean = __half2float(reinterpret_cast<__half *>(raw)[0]); sd = __half2float(reinterpret_cast<__half *>(raw)[1]); }
            if (!(std::fabs(mean) < 2 * std::fabs(sd)))
                return bad_arg("TruncatedNormal: |mean| must be below 2 |stddev|, otherwise no sample is ever accepted");
        }
        if (opNum == 5) {
            const size_t es = dtype == kF64 ? 8 : (dtype == kF32 ? 4 : 2);
            void *ws = nullptr;
            // the sums go behind the result slot and the arrival counters of the reductions, which
            // must stay zero between launches
            const size_t skip = 256 + kCounterSlots * sizeof(unsigned);
            ND_TRY(workspace(as_stream(stream), skip + es * (size_t) yd->length, &ws, nullptr));
            a.aux = static_cast<char *>(ws) + skip;
            a.auxLen = yd->length;
        }
    }
    // special ops exist only in the three-operand form; the other arities of the reference fall
    // through to the functor defaults (-1 / -2), include/loops/cpu/random.cpp:86-185
    int op = opNum;
    if ((opNum == 6 || opNum == 10 || opNum == 5 || opNum == 8 || opNum == 9 || opNum == 11) && arity != 2) op = 100;
    return BY_DTYPE(dtype, random, op, arity, a, as_stream(stream));
}

}  // namespace

#pragma GCC visibility push(default)
extern "C" {

const char *nd4jb200_last_error(void) { return last_error(); }
unsigned long long nd4jb200_launch_count(void) { return g_launches.load(std::memory_order_relaxed); }

int nd4jb200_set_tuning(int key, long long value) {
    if (key < 0 || key >= kTuneCount || value < (key == kTuneOverlapLaunch ? 0 : 1) || (key == kTuneMaxCluster && value > 8) ||
        (key == kTuneRowThreadsPerSm && value > kMaxRowThreadsPerSm) ||
        ((key == kTuneColCtasPerSm || key == kTuneRowCtasPerSm) && value > 64)) {
        set_error("nd4jb200_set_tuning: unknown key or value out of range");
        return kBadArgument;
    }
    g_tuning[key] = value;
    return kOk;
}

// ---------------------------------------------------------------------------------------------
int nd4jb200_exec_reduce(void *stream, int dtype, int opNum, const void *x, const Nd4jLong *xShapeInfo,
                         const void *extraParams, void *z, const Nd4jLong *zShapeInfo, const int *dimension,
                         int dimensionLength) {
    ND_TRY(check_dtype(dtype));
    ND_TRY(need(z, "z"));
    ReduceSetup s;
    ND_TRY(setup_reduction(x, xShapeInfo, nullptr, nullptr, zShapeInfo, dimension, dimensionLength, false, &s));
    if (s.x.length == 0) return kOk;
    s.call.extra = extraParams; s.call.z = z;
    return BY_DTYPE(dtype, reduce, opNum, s.call, as_stream(stream));
}

int nd4jb200_exec_reduce_scalar(void *stream, int dtype, int opNum, const void *x, const Nd4jLong *xShapeInfo,
                                const void *extraParams, double *result) {
    ND_TRY(check_dtype(dtype));
    ND_TRY(need(result, "result"));
    ReduceSetup s;
    ND_TRY(setup_reduction(x, xShapeInfo, nullptr, nullptr, nullptr, nullptr, 0, true, &s));
    void *ws, *slot;
    ND_TRY(workspace(as_stream(stream), kScalarWorkspace, &ws, &slot));
    s.call.extra = extraParams; s.call.z = ws;
    ND_TRY(BY_DTYPE(dtype, reduce, opNum, s.call, as_stream(stream)));
    return fetch_scalar(as_stream(stream), dtype, ws, slot, result);
}

int nd4jb200_exec_index_reduce(void *stream, int dtype, int opNum, const void *x, const Nd4jLong *xShapeInfo,
                               const void *extraParams, void *z, const Nd4jLong *zShapeInfo, const int *dimension,
                               int dimensionLength) {
    ND_TRY(check_dtype(dtype));
    ND_TRY(need(z, "z"));
    ReduceSetup s;
    ND_TRY(setup_reduction(x, xShapeInfo, nullptr, nullptr, zShapeInfo, dimension, dimensionLength, false, &s));
    if (s.x.length == 0) return kOk;
    s.call.extra = extraParams; s.call.z = z;
    return BY_DTYPE(dtype, index_reduce, opNum, s.call, as_stream(stream));
}

int nd4jb200_exec_index_reduce_scalar(void *stream, int dtype, int opNum, const void *x, const Nd4jLong *xShapeInfo,
                                      const void *extraParams, double *result) {
    ND_TRY(check_dtype(dtype));
    ND_TRY(need(result, "result"));
    ReduceSetup s;
    ND_TRY(setup_reduction(x, xShapeInfo, nullptr, nullptr, nullptr, nullptr, 0, true, &s));
    void *ws, *slot;
    ND_TRY(workspace(as_stream(stream), kScalarWorkspace, &ws, &slot));
    s.call.extra = extraParams; s.call.z = ws;
    ND_TRY(BY_DTYPE(dtype, index_reduce, opNum, s.call, as_stream(stream)));
    return fetch_scalar(as_stream(stream), dtype, ws, slot, result);
}

int nd4jb200_exec_summary_stats(void *stream, int dtype, int opNum, const void *x, const Nd4jLong *xShapeInfo,
                                const void *extraParams, void *z, const Nd4jLong *zShapeInfo, const int *dimension,
                                int dimensionLength, int biasCorrected) {
    ND_TRY(check_dtype(dtype));
    ND_TRY(need(z, "z"));
    ReduceSetup s;
    ND_TRY(setup_reduction(x, xShapeInfo, nullptr, nullptr, zShapeInfo, dimension, dimensionLength, false, &s));
    if (s.x.length == 0) return kOk;
    s.call.extra = extraParams; s.call.z = z;
    if (biasCorrected) s.call.finishLen |= (1LL << 62);
    return BY_DTYPE(dtype, summary_stats, opNum, s.call, as_stream(stream));
}

int nd4jb200_exec_summary_stats_scalar(void *stream, int dtype, int opNum, const void *x, const Nd4jLong *xShapeInfo,
                                       const void *extraParams, int biasCorrected, double *result) {
    ND_TRY(check_dtype(dtype));
    ND_TRY(need(result, "result"));
    ReduceSetup s;
    ND_TRY(setup_reduction(x, xShapeInfo, nullptr, nullptr, nullptr, nullptr, 0, true, &s));
    void *ws, *slot;
    ND_TRY(workspace(as_stream(stream), kScalarWorkspace, &ws, &slot));
    s.call.extra = extraParams; s.call.z = ws;
    if (biasCorrected) s.call.finishLen |= (1LL << 62);
    ND_TRY(BY_DTYPE(dtype, summary_stats, opNum, s.call, as_stream(stream)));
    return fetch_scalar(as_stream(stream), dtype, ws, slot, result);
}

int nd4jb200_exec_reduce3(void *stream, int dtype, int opNum, const void *x, const Nd4jLong *xShapeInfo,
                          const void *extraParams, const void *y, const Nd4jLong *yShapeInfo, void *z,
                          const Nd4jLong *zShapeInfo, const int *dimension, int dimensionLength) {
    ND_TRY(check_dtype(dtype));
    ND_TRY(need(z, "z"));
    ND_TRY(need(y, "y"));
    ReduceSetup s;
    ND_TRY(setup_reduction(x, xShapeInfo, y, yShapeInfo, zShapeInfo, dimension, dimensionLength, false, &s));
    if (s.x.length == 0) return kOk;
    // along a dimension the reference hands the functors zeroed parameters (eps = 0 for
    // EqualsWithEps, include/loops/reduce3.h:1101); only the whole-array form forwards
    // extraParams[0] (include/loops/reduce3.h:853-857)
    s.call.extra = s.scalarResult ? extraParams : nullptr;
    s.call.z = z;
    return BY_DTYPE(dtype, reduce3, opNum, s.call, as_stream(stream));
}

int nd4jb200_exec_reduce3_all(void *stream, int dtype, int opNum, const void *x, const Nd4jLong *xShapeInfo,
                              const void *extraParams, const void *y, const Nd4jLong *yShapeInfo, void *z,
                              const Nd4jLong *zShapeInfo, const int *dimension, int dimensionLength) {
    (void) extraParams;   // the reference hands the functors a zeroed parameter block here (reduce3.h:957-962)
    ND_TRY(check_dtype(dtype));
    ND_TRY(need(x, "x")); ND_TRY(need(y, "y")); ND_TRY(need(z, "z"));
    ShapeDesc xd, yd, zd;
    ND_TRY(parse_shape(xShapeInfo, "xShapeInfo", &xd));
    ND_TRY(parse_shape(yShapeInfo, "yShapeInfo", &yd));
    ND_TRY(parse_shape(zShapeInfo, "zShapeInfo", &zd));
    ReduceCall c;
    ND_TRY(make_tad_plan(xd, dimension, dimensionLength, &c.xPlan));
    ND_TRY(make_tad_plan(yd, dimension, dimensionLength, &c.yPlan));
    if (c.xPlan.tadLen != c.yPlan.tadLen) return bad_arg("reduce3 all-pairs: the TADs of x and y differ in length");
    if (zd.length != c.xPlan.numTads * c.yPlan.numTads) return bad_arg("reduce3 all-pairs: result must hold xTads * yTads elements");
    if (zd.ews != 1) return unsupported("reduce3 all-pairs: the result must be dense (the reference writes result[r * yTads + g])");
    // inside a TAD both operands are walked in c-order; the reference pairs element f of x with
    // element f of y in each TAD's own order, which is the same pairing unless the orders differ
    if (c.xPlan.inner.rank > 1 && xd.order != yd.order)
        return unsupported("reduce3 all-pairs: multi-axis TADs of arrays with different orders");
    if (xd.length == 0 || yd.length == 0) return kOk;
    c.x = x; c.y = y; c.extra = nullptr; c.z = z;
    c.finishLen = c.xPlan.tadLen;
    return BY_DTYPE(dtype, reduce3_all, opNum, c, as_stream(stream));
}

int nd4jb200_exec_reduce3_scalar(void *stream, int dtype, int opNum, const void *x, const Nd4jLong *xShapeInfo,
                                 const void *extraParams, const void *y, const Nd4jLong *yShapeInfo, double *result) {
    ND_TRY(check_dtype(dtype));
    ND_TRY(need(result, "result"));
    ND_TRY(need(y, "y"));
    ReduceSetup s;
    ND_TRY(setup_reduction(x, xShapeInfo, y, yShapeInfo, nullptr, nullptr, 0, true, &s));
    void *ws, *slot;
    ND_TRY(workspace(as_stream(stream), kScalarWorkspace, &ws, &slot));
    s.call.extra = extraParams; s.call.z = ws;
    ND_TRY(BY_DTYPE(dtype, reduce3, opNum, s.call, as_stream(stream)));
    return fetch_scalar(as_stream(stream), dtype, ws, slot, result);
}

// ---------------------------------------------------------------------------------------------
int nd4jb200_exec_transform(void *stream, int dtype, int opNum, const void *x, const Nd4jLong *xShapeInfo, void *z,
                            const Nd4jLong *zShapeInfo, const void *extraParams) {
    ND_TRY(check_dtype(dtype));
    ND_TRY(need(x, "x")); ND_TRY(need(z, "z"));
    ShapeDesc xd, zd;
    ND_TRY(parse_shape(xShapeInfo, "xShapeInfo", &xd));
    ND_TRY(parse_shape(zShapeInfo, "zShapeInfo", &zd));
    if (opNum == 36 || opNum == 37 || opNum == 48 || opNum == 70 || opNum == 71)
        return run_special_transform(dtype, opNum, x, xd, z, zd, extraParams, as_stream(stream));
    if (xd.length != zd.length) return bad_arg("transform: x and z hold different numbers of elements");
    if (opNum == 41) {
        // IsMax: extraParams = {dimensionLength, dimension...} as element-type values on the device; absent, 0 or
        // {1, MAX_DIMENSION} mean the whole array (include/ops/special_ops.h:2199-2203)
        if (xd.length != zd.length) return bad_arg("IsMax: x and z hold different numbers of elements");
        int dims[kMaxRank];
        int ndims = 0;
        if (extraParams) {
            unsigned char raw[8 * (kMaxRank + 1)] = {0};
            const size_t es = dtype_size(dtype);
            ND_CUDA(cudaMemcpyAsync(raw, extraParams, es, cudaMemcpyDeviceToHost, as_stream(stream)));
            ND_CUDA(cudaStreamSynchronize(as_stream(stream)));
            auto value = [&](int k) -> double {
                if (dtype == kF64) return reinterpret_cast<double *>(raw)[k];
                if (dtype == kF32) return reinterpret_cast<float *>(raw)[k];
                return __half2float(reinterpret_cast<__half *>(raw)[k]);
            };
            ndims = (int) value(0);
            if (ndims < 0 || ndims > xd.rank) return bad_arg("IsMax: extraParams[0] is not a valid dimension count");
            if (ndims > 0) {
                ND_CUDA(cudaMemcpyAsync(raw, extraParams, es * (ndims + 1), cudaMemcpyDeviceToHost, as_stream(stream)));
                ND_CUDA(cudaStreamSynchronize(as_stream(stream)));
                for (int k = 0; k < ndims; k++) dims[k] = (int) value(k + 1);
                if (ndims == 1 && dims[0] == 0x7fffffff) ndims = 0;
            }
        }
        ReduceCall c;
        ND_TRY(make_tad_plan(xd, ndims ? dims : nullptr, ndims, &c.xPlan));
        TadPlan zPlan;
        ND_TRY(make_tad_plan(zd, ndims ? dims : nullptr, ndims, &zPlan));
        if (zPlan.numTads != c.xPlan.numTads || zPlan.tadLen != c.xPlan.tadLen) return bad_arg("IsMax: x and z split into different TADs");
        // TADs over several axes are scanned by the reference's raw iterator, whose order is the first TAD axis
        // fastest whatever the array's order (special_ops.h:2383-2420): ties resolve in that order
        if (ndims > 1) {
            int axes[kMaxRank];
            int n = 0;
            for (int ax = 0; ax < xd.rank; ax++) {              // the listed axes, ascending and unique
                bool listed = false;
                for (int k = 0; k < ndims; k++) listed = listed || dims[k] == ax || dims[k] + xd.rank == ax;
                if (listed) axes[n++] = ax;
            }
            LL shp[kMaxRank], sx[kMaxRank], sz[kMaxRank];
            for (int k = 0; k < n; k++) {
                const int ax = axes[n - 1 - k];                   // first listed axis last = fastest
                shp[k] = xd.shape[ax]; sx[k] = xd.stride[ax]; sz[k] = zd.stride[ax];
            }
            ND_TRY(collapse_view(n, shp, sx, &c.xPlan.inner));
            ND_TRY(collapse_view(n, shp, sz, &zPlan.inner));
        } else if (c.xPlan.whole) {
            // whole-array calls walk x and z by linear index, like the reference's doAll
            if (xd.ews < 1 && xd.rank > 1) ND_TRY(coord_view(xd, &c.xPlan.inner));
            if (zd.ews < 1 && zd.rank > 1) ND_TRY(coord_view(zd, &zPlan.inner));
        }
        // the positions go behind everything a split reduction may use of the workspace
        void *ws = nullptr;
        ND_TRY(workspace(as_stream(stream), kScalarWorkspace + sizeof(LL) * (size_t) c.xPlan.numTads, &ws, nullptr));
        LL *positions = reinterpret_cast<LL *>(static_cast<char *>(ws) + kScalarWorkspace);
        // exact 64-bit positions: the element type cannot hold them (half beyond 2048, float beyond 2^24)
        c.x = x; c.extra = nullptr; c.z = positions; c.zIndex = positions; c.finishLen = c.xPlan.tadLen;
        ND_TRY(BY_DTYPE(dtype, index_reduce, 0, c, as_stream(stream)));
        IsMaxArgs m;
        m.index = positions; m.z = z; m.numTads = zPlan.numTads; m.tadLen = zPlan.tadLen;
        m.zOuter = zPlan.outer; m.zInner = zPlan.inner;
        return BY_DTYPE(dtype, ismax_mark, m, as_stream(stream));
    }
    if (opNum == 38 || opNum == 39 || opNum == 40) {
        // SoftMax / SoftMaxDerivative / LogSoftMax: row-wise on matrices, whole-array on vectors; other
        // ranks are left untouched by the reference (include/ops/special_ops.h:1484-1570, 1640-1730, 1808-1940)
        if (xd.rank != 2 || zd.rank != 2) return unsupported("the softmax family is defined for matrices and vectors (rank 2)");
        for (int i = 0; i < 2; i++) if (xd.shape[i] != zd.shape[i]) return bad_arg("softmax: x and z differ in shape");
        SoftmaxArgs sa;
        sa.x = x; sa.z = z;
        const bool vector = xd.shape[0] == 1 || xd.shape[1] == 1;
        if (vector) {
            const int ax = xd.shape[0] == 1 ? 1 : 0;
            sa.rows = 1; sa.cols = xd.length;
            sa.xRow = 0; sa.zRow = 0; sa.xCol = xd.stride[ax]; sa.zCol = zd.stride[ax];
        } else {
            sa.rows = xd.shape[0]; sa.cols = xd.shape[1];
            sa.xRow = xd.stride[0]; sa.xCol = xd.stride[1]; sa.zRow = zd.stride[0]; sa.zCol = zd.stride[1];
        }
        return BY_DTYPE(dtype, softmax, opNum - 38, sa, as_stream(stream));
    }
    EwArgs a;
    a.x = x; a.y = nullptr; a.z = z; a.extra = extraParams; a.n = xd.length; a.scalar = 0;
    ND_TRY(setup_linear(&xd, nullptr, &zd, x, nullptr, z, &a));
    return BY_DTYPE(dtype, transform, opNum, a, as_stream(stream));
}

int nd4jb200_exec_transform_strided(void *stream, int dtype, int opNum, const void *x, Nd4jLong xStride, void *z,
                                    Nd4jLong zStride, const void *extraParams, Nd4jLong n) {
    ND_TRY(check_dtype(dtype));
    ND_TRY(need(x, "x")); ND_TRY(need(z, "z"));
    EwArgs a;
    a.x = x; a.y = nullptr; a.z = z; a.extra = extraParams; a.n = n; a.scalar = 0;
    a.sx = xStride; a.sy = 0; a.sz = zStride;
    a.mode = (xStride == 1 && zStride == 1 && aligned16(x) && aligned16(z)) ? 0 : 1;
    return BY_DTYPE(dtype, transform, opNum, a, as_stream(stream));
}

int nd4jb200_exec_pairwise(void *stream, int dtype, int opNum, const void *x, const Nd4jLong *xShapeInfo,
                           const void *y, const Nd4jLong *yShapeInfo, void *z, const Nd4jLong *zShapeInfo,
                           const void *extraParams) {
    ND_TRY(check_dtype(dtype));
    ND_TRY(need(x, "x")); ND_TRY(need(y, "y")); ND_TRY(need(z, "z"));
    ShapeDesc xd, yd, zd;
    ND_TRY(parse_shape(xShapeInfo, "xShapeInfo", &xd));
    ND_TRY(parse_shape(yShapeInfo, "yShapeInfo", &yd));
    ND_TRY(parse_shape(zShapeInfo, "zShapeInfo", &zd));
    EwArgs a;
    a.x = x; a.y = y; a.z = z; a.extra = extraParams; a.n = xd.length; a.scalar = 0;
    if (yd.length == 1 && xd.length != 1) {
        // y is a single value applied to every x (include/loops/pairwise_transform.h:168-202)
        if (xd.length != zd.length) return bad_arg("pairwise: x and z hold different numbers of elements");
        ND_TRY(setup_linear(&xd, nullptr, &zd, x, nullptr, z, &a));
        if (a.mode == 0) a.mode = 1;
        a.sy = 0;
        a.vy.rank = 0;
        for (int i = 0; i < kDevRank; i++) { a.vy.shape[i] = 1; a.vy.stride[i] = 0; }
    } else {
        if (xd.length != yd.length || xd.length != zd.length) return bad_arg("pairwise: x, y and z hold different numbers of elements");
        ND_TRY(setup_linear(&xd, &yd, &zd, x, y, z, &a));
    }
    return BY_DTYPE(dtype, pairwise, opNum, a, as_stream(stream));
}

int nd4jb200_exec_pairwise_indexed(void *stream, int dtype, int opNum, const void *x, const Nd4jLong *xShapeInfo,
                                   const void *y, void *z, const void *extraParams, const Nd4jLong *xIndexes,
                                   const Nd4jLong *yIndexes, const Nd4jLong *zIndexes) {
    ND_TRY(check_dtype(dtype));
    ND_TRY(need(x, "x")); ND_TRY(need(y, "y")); ND_TRY(need(z, "z"));
    ND_TRY(need(xIndexes, "xIndexes")); ND_TRY(need(yIndexes, "yIndexes")); ND_TRY(need(zIndexes, "resultIndexes"));
    ShapeDesc xd;
    ND_TRY(parse_shape(xShapeInfo, "xShapeInfo", &xd));
    EwArgs a;
    a.x = x; a.y = y; a.z = z; a.extra = extraParams; a.n = xd.length; a.scalar = 0;
    a.mode = 3; a.sx = a.sy = a.sz = 0;
    a.vx.rank = a.vy.rank = a.vz.rank = 0;
    a.ix = xIndexes; a.iy = yIndexes; a.iz = zIndexes;
    return BY_DTYPE(dtype, pairwise, opNum, a, as_stream(stream));
}

int nd4jb200_exec_scalar_indexed(void *stream, int dtype, int opNum, const void *x, const Nd4jLong *xShapeInfo, void *z,
                                 double scalar, const void *extraParams, const Nd4jLong *xIndexes,
                                 const Nd4jLong *zIndexes) {
    ND_TRY(check_dtype(dtype));
    ND_TRY(need(x, "x")); ND_TRY(need(z, "z"));
    ND_TRY(need(xIndexes, "xIndexes")); ND_TRY(need(zIndexes, "resultIndexes"));
    ShapeDesc xd;
    ND_TRY(parse_shape(xShapeInfo, "xShapeInfo", &xd));
    EwArgs a;
    a.x = x; a.y = nullptr; a.z = z; a.extra = extraParams; a.n = xd.length; a.scalar = scalar;
    a.mode = 3; a.sx = a.sy = a.sz = 0;
    a.vx.rank = a.vy.rank = a.vz.rank = 0;
    a.ix = xIndexes; a.iy = nullptr; a.iz = zIndexes;
    return BY_DTYPE(dtype, scalar, opNum, a, as_stream(stream));
}

int nd4jb200_exec_pairwise_strided(void *stream, int dtype, int opNum, const void *x, Nd4jLong xStride, const void *y,
                                   Nd4jLong yStride, void *z, Nd4jLong zStride, const void *extraParams, Nd4jLong n) {
    ND_TRY(check_dtype(dtype));
    ND_TRY(need(x, "x")); ND_TRY(need(y, "y")); ND_TRY(need(z, "z"));
    EwArgs a;
    a.x = x; a.y = y; a.z = z; a.extra = extraParams; a.n = n; a.scalar = 0;
    a.sx = xStride; a.sy = yStride; a.sz = zStride;
    a.mode = (xStride == 1 && yStride == 1 && zStride == 1 && aligned16(x) && aligned16(y) && aligned16(z)) ? 0 : 1;
    return BY_DTYPE(dtype, pairwise, opNum, a, as_stream(stream));
}

int nd4jb200_exec_scalar(void *stream, int dtype, int opNum, const void *x, const Nd4jLong *xShapeInfo, void *z,
                         const Nd4jLong *zShapeInfo, double scalar, const void *extraParams) {
    ND_TRY(check_dtype(dtype));
    ND_TRY(need(x, "x")); ND_TRY(need(z, "z"));
    ShapeDesc xd, zd;
    ND_TRY(parse_shape(xShapeInfo, "xShapeInfo", &xd));
    ND_TRY(parse_shape(zShapeInfo, "zShapeInfo", &zd));
    if (xd.length != zd.length) return bad_arg("scalar: x and z hold different numbers of elements");
    EwArgs a;
    a.x = x; a.y = nullptr; a.z = z; a.extra = extraParams; a.n = xd.length; a.scalar = scalar;
    ND_TRY(setup_linear(&xd, nullptr, &zd, x, nullptr, z, &a));
    return BY_DTYPE(dtype, scalar, opNum, a, as_stream(stream));
}

int nd4jb200_exec_scalar_strided(void *stream, int dtype, int opNum, const void *x, Nd4jLong xStride, void *z,
                                 Nd4jLong zStride, double scalar, const void *extraParams, Nd4jLong n) {
    ND_TRY(check_dtype(dtype));
    ND_TRY(need(x, "x")); ND_TRY(need(z, "z"));
    EwArgs a;
    a.x = x; a.y = nullptr; a.z = z; a.extra = extraParams; a.n = n; a.scalar = scalar;
    a.sx = xStride; a.sy = 0; a.sz = zStride;
    a.mode = (xStride == 1 && zStride == 1 && aligned16(x) && aligned16(z)) ? 0 : 1;
    return BY_DTYPE(dtype, scalar, opNum, a, as_stream(stream));
}

static Status setup_tad_pair(int dtype, const void *x, const Nd4jLong *xShapeInfo, void *z, const Nd4jLong *zShapeInfo,
                             const int *dimension, int dimensionLength, BcArgs *a, ShapeDesc *xd, ShapeDesc *zd) {
    ND_TRY(parse_shape(xShapeInfo, "xShapeInfo", xd));
    ND_TRY(parse_shape(zShapeInfo, "zShapeInfo", zd));
    if (xd->length != zd->length) return bad_arg("x and z hold different numbers of elements");
    TadPlan xp, zp;
    ND_TRY(make_tad_plan(*xd, dimension, dimensionLength, &xp));
    ND_TRY(make_tad_plan(*zd, dimension, dimensionLength, &zp));
    if (xp.whole) { ND_TRY(coord_view(*xd, &xp.inner)); }
    if (zp.whole) { ND_TRY(coord_view(*zd, &zp.inner)); }
    if (xp.numTads != zp.numTads || xp.tadLen != zp.tadLen) return bad_arg("x and z split into different TADs");
    a->x = x; a->z = z;
    a->numTads = xp.numTads; a->tadLen = xp.tadLen;
    a->xOuter = xp.outer; a->xInner = xp.inner; a->zOuter = zp.outer; a->zInner = zp.inner;
    a->rowsPerBlock = 1;
    const LL V = 16 / (LL) dtype_size(dtype);
    auto unit = [](const View &v) { return v.rank == 0 || (v.rank == 1 && v.stride[0] == 1); };
    bool rows = unit(a->xInner) && unit(a->zInner) && a->xOuter.rank <= 1 && a->zOuter.rank <= 1 &&
                a->tadLen % V == 0 && aligned16(x) && aligned16(z) &&
                view_strides_multiple_of(a->xOuter, V) && view_strides_multiple_of(a->zOuter, V);
    a->mode = rows ? 0 : 1;
    return kOk;
}

int nd4jb200_exec_broadcast(void *stream, int dtype, int opNum, const void *x, const Nd4jLong *xShapeInfo,
                            const void *y, const Nd4jLong *yShapeInfo, void *z, const Nd4jLong *zShapeInfo,
                            const int *dimension, int dimensionLength) {
    ND_TRY(check_dtype(dtype));
    ND_TRY(need(x, "x")); ND_TRY(need(y, "y")); ND_TRY(need(z, "z"));
    ND_TRY(need(dimension, "dimension"));
    BcArgs a;
    ShapeDesc xd, zd, yd;
    ND_TRY(setup_tad_pair(dtype, x, xShapeInfo, z, zShapeInfo, dimension, dimensionLength, &a, &xd, &zd));
    ND_TRY(parse_shape(yShapeInfo, "yShapeInfo", &yd));
    if (yd.length != a.tadLen) {
        std::ostringstream os;
        os << "broadcast: y holds " << yd.length << " elements but a TAD along the given dimension holds " << a.tadLen;
        return bad_arg(os.str());
    }
    a.y = y; a.extra = nullptr;
    ND_TRY(coord_view(yd, &a.yView));
    if (!(a.yView.rank == 0 || (a.yView.rank == 1 && a.yView.stride[0] == 1)) || !aligned16(y)) a.mode = 1;
    return BY_DTYPE(dtype, broadcast, opNum, a, as_stream(stream));
}

int nd4jb200_exec_scalar_along_dimension(void *stream, int dtype, int opNum, const void *x, const Nd4jLong *xShapeInfo,
                                         const void *extraParams, void *z, const Nd4jLong *zShapeInfo,
                                         const void *scalars, const int *dimension, int dimensionLength) {
    ND_TRY(check_dtype(dtype));
    ND_TRY(need(x, "x")); ND_TRY(need(scalars, "scalars")); ND_TRY(need(z, "z"));
    ND_TRY(need(dimension, "dimension"));
    BcArgs a;
    ShapeDesc xd, zd;
    ND_TRY(setup_tad_pair(dtype, x, xShapeInfo, z, zShapeInfo, dimension, dimensionLength, &a, &xd, &zd));
    a.y = scalars; a.extra = extraParams;
    a.yView.rank = 0;
    return BY_DTYPE(dtype, scalar_tad, opNum, a, as_stream(stream));
}

// ---------------------------------------------------------------------------------------------
// Fused chains. exec_chain: z = pairwise(transform(broadcast(x, b)), y) in one pass (fused_engine.cuh) when the
// broadcast and pairwise ops are light ops; otherwise the three steps run as separate launches through z.
int nd4jb200_exec_chain(void *stream, int dtype, int broadcastOp, const void *x, const Nd4jLong *xShapeInfo,
                        const void *b, const Nd4jLong *bShapeInfo, const int *dimension, int dimensionLength,
                        int transformOp, const void *transformExtra, int pairwiseOp, const void *y,
                        const Nd4jLong *yShapeInfo, const void *pairwiseExtra, void *z, const Nd4jLong *zShapeInfo) {
    ND_TRY(check_dtype(dtype));
    ND_TRY(need(x, "x")); ND_TRY(need(b, "b")); ND_TRY(need(y, "y")); ND_TRY(need(z, "z"));
    ND_TRY(need(dimension, "dimension"));
    const int bc = light_of_broadcast(broadcastOp), pw = light_of_pairwise(pairwiseOp);
    const bool composite = transformOp == 36 || transformOp == 37 || transformOp == 38 || transformOp == 39 ||
                           transformOp == 40 || transformOp == 41 || transformOp == 48 || transformOp == 70 ||
                           transformOp == 71;
    if (bc == kLightNone || pw == kLightNone || composite) {
        if (z == y) return unsupported("exec_chain: with these ops the steps run as separate launches through z, which "
                                       "must then not alias y");
        ND_TRY((Status) nd4jb200_exec_broadcast(stream, dtype, broadcastOp, x, xShapeInfo, b, bShapeInfo, z, zShapeInfo,
                                                dimension, dimensionLength));
        ND_TRY((Status) nd4jb200_exec_transform(stream, dtype, transformOp, z, zShapeInfo, z, zShapeInfo, transformExtra));
        return nd4jb200_exec_pairwise(stream, dtype, pairwiseOp, z, zShapeInfo, y, yShapeInfo, z, zShapeInfo, pairwiseExtra);
    }
    ShapeDesc xd, yd, zd, bd;
    ND_TRY(parse_shape(xShapeInfo, "xShapeInfo", &xd));
    ND_TRY(parse_shape(yShapeInfo, "yShapeInfo", &yd));
    ND_TRY(parse_shape(zShapeInfo, "zShapeInfo", &zd));
    ND_TRY(parse_shape(bShapeInfo, "bShapeInfo", &bd));
    // the pairwise step pairs by coordinates, which is what the separate launches do for arrays of one shape
    if (!same_shape(xd, yd) || !same_shape(xd, zd)) return bad_arg("exec_chain: x, y and z must have the same shape");
    TadPlan xp, yp, zp;
    ND_TRY(make_tad_plan(xd, dimension, dimensionLength, &xp));
    ND_TRY(make_tad_plan(yd, dimension, dimensionLength, &yp));
    ND_TRY(make_tad_plan(zd, dimension, dimensionLength, &zp));
    if (xp.whole) { ND_TRY(coord_view(xd, &xp.inner)); ND_TRY(coord_view(yd, &yp.inner)); ND_TRY(coord_view(zd, &zp.inner)); }
    if (bd.length != xp.tadLen) {
        std::ostringstream os;
        os << "exec_chain: b holds " << bd.length << " elements but a TAD along the given dimension holds " << xp.tadLen;
        return bad_arg(os.str());
    }
    if (xd.length == 0) return kOk;
    ChainArgs a;
    a.x = x; a.b = b; a.y = y; a.z = z; a.trExtra = transformExtra;
    a.numTads = xp.numTads; a.tadLen = xp.tadLen;
    a.xOuter = xp.outer; a.xInner = xp.inner; a.yOuter = yp.outer; a.yInner = yp.inner;
    a.zOuter = zp.outer; a.zInner = zp.inner;
    ND_TRY(coord_view(bd, &a.bView));
    a.bcCode = bc; a.pwCode = pw; a.rowsPerBlock = 1;
    const LL V = 16 / (LL) dtype_size(dtype);
    auto unit = [](const View &v) { return v.rank == 0 || (v.rank == 1 && v.stride[0] == 1); };
    auto rowsOf = [&](const View &inner, const View &outer, const void *ptr) {
        return unit(inner) && outer.rank <= 1 && aligned16(ptr) && view_strides_multiple_of(outer, V);
    };
    const bool rows = rowsOf(a.xInner, a.xOuter, x) && rowsOf(a.yInner, a.yOuter, y) && rowsOf(a.zInner, a.zOuter, z) &&
                      a.tadLen % V == 0 && unit(a.bView) && aligned16(b);
    a.mode = rows ? 0 : 1;
    return BY_DTYPE(dtype, chain, transformOp, a, as_stream(stream));
}

// The reference's meta-op hook (blas/NativeOps.h:2564-2785): opTypeA 2 = a pairwise op on (x, y) with extraA,
// followed by opTypeB 0 = a scalar op with scalarB (include/loops/cuda/grid_shaped.cu:159-211; no other type
// pair has an implementation there). One launch when the scalar op is a light op, two otherwise.
static Status meta_pair(void *stream, int dtype, int opTypeA, int opNumA, int opTypeB, int opNumB, EwArgs &a,
                        const Nd4jLong *zShapeInfo, Nd4jLong zStride, double scalarB, const void *extraB) {
    if (opTypeA != 2 || opTypeB != 0)
        return unsupported("execMetaPredicate: only a pairwise op (type 2) followed by a scalar op (type 0) is defined");
    const int post = light_of_scalar(opNumB);
    if (post != kLightNone) {
        a.postCode = post; a.postScalar = scalarB;
        return BY_DTYPE(dtype, pairwise_post, opNumA, a, as_stream(stream));
    }
    ND_TRY(BY_DTYPE(dtype, pairwise, opNumA, a, as_stream(stream)));
    if (zShapeInfo) return (Status) nd4jb200_exec_scalar(stream, dtype, opNumB, a.z, zShapeInfo, a.z, zShapeInfo, scalarB, extraB);
    return (Status) nd4jb200_exec_scalar_strided(stream, dtype, opNumB, a.z, zStride, a.z, zStride, scalarB, extraB, a.n);
}

int nd4jb200_exec_meta_predicate_shape(void *stream, int dtype, int opTypeA, int opNumA, int opTypeB, int opNumB,
                                       const void *x, const Nd4jLong *xShapeInfo, const void *y,
                                       const Nd4jLong *yShapeInfo, void *z, const Nd4jLong *zShapeInfo,
                                       const void *extraA, const void *extraB, double scalarA, double scalarB) {
    (void) scalarA;
    ND_TRY(check_dtype(dtype));
    ND_TRY(need(x, "x")); ND_TRY(need(y, "y")); ND_TRY(need(z, "z"));
    ShapeDesc xd, yd, zd;
    ND_TRY(parse_shape(xShapeInfo, "xShapeInfo", &xd));
    ND_TRY(parse_shape(yShapeInfo, "yShapeInfo", &yd));
    ND_TRY(parse_shape(zShapeInfo, "zShapeInfo", &zd));
    if (xd.length != yd.length || xd.length != zd.length) return bad_arg("execMetaPredicateShape: x, y and z hold different numbers of elements");
    EwArgs a;
    a.x = x; a.y = y; a.z = z; a.extra = extraA; a.n = xd.length; a.scalar = 0;
    ND_TRY(setup_linear(&xd, &yd, &zd, x, y, z, &a));
    return meta_pair(stream, dtype, opTypeA, opNumA, opTypeB, opNumB, a, zShapeInfo, 0, scalarB, extraB);
}

int nd4jb200_exec_meta_predicate_strided(void *stream, int dtype, int opTypeA, int opNumA, int opTypeB, int opNumB,
                                         Nd4jLong n, const void *x, Nd4jLong xStride, const void *y, Nd4jLong yStride,
                                         void *z, Nd4jLong zStride, const void *extraA, const void *extraB,
                                         double scalarA, double scalarB) {
    (void) scalarA;
    ND_TRY(check_dtype(dtype));
    ND_TRY(need(x, "x")); ND_TRY(need(y, "y")); ND_TRY(need(z, "z"));
    EwArgs a;
    a.x = x; a.y = y; a.z = z; a.extra = extraA; a.n = n; a.scalar = 0;
    a.sx = xStride; a.sy = yStride; a.sz = zStride;
    a.mode = (xStride == 1 && yStride == 1 && zStride == 1 && aligned16(x) && aligned16(y) && aligned16(z)) ? 0 : 1;
    return meta_pair(stream, dtype, opTypeA, opNumA, opTypeB, opNumB, a, nullptr, zStride, scalarB, extraB);
}

// ---------------------------------------------------------------------------------------------
Nd4jPointer nd4jb200_init_random(void *stream, Nd4jLong seed, Nd4jLong bufferSize, void *hostTable, void *deviceTable) {
    if (bufferSize <= 0) { bad_arg("initRandom: bufferSize must be positive"); return nullptr; }
    RandomState *s = new RandomState();
    s->size = bufferSize;
    s->seed = seed; s->amplifier = seed; s->generation = 1; s->position = 0;
    s->ownsHost = hostTable == nullptr; s->ownsDev = deviceTable == nullptr;
    s->hostTable = static_cast<unsigned long long *>(hostTable);
    s->devTable = static_cast<unsigned long long *>(deviceTable);
    if (s->ownsHost) s->hostTable = static_cast<unsigned long long *>(malloc(sizeof(unsigned long long) * bufferSize));
    if (s->ownsDev) {
        cudaError_t e = cudaMalloc(&s->devTable, sizeof(unsigned long long) * bufferSize);
        if (e != cudaSuccess) { cuda_fail(e, "cudaMalloc(random table)"); if (s->ownsHost) free(s->hostTable); delete s; return nullptr; }
    }
    fill_table(s);
    if (upload_table(s, as_stream(stream)) != kOk) { nd4jb200_destroy_random(s); return nullptr; }
    return s;
}

int nd4jb200_refresh_buffer(void *stream, Nd4jLong seed, Nd4jPointer state) {
    ND_TRY(need(state, "state"));
    RandomState *s = static_cast<RandomState *>(state);
    // setSeed resets amplifier and generation; the offset goes back to 0 (blas/cpu/NativeOps.cpp:2887-2894)
    s->seed = seed; s->amplifier = seed; s->generation = 1; s->position = 0;
    fill_table(s);
    return upload_table(s, as_stream(stream));
}

int nd4jb200_reseed_buffer(Nd4jLong seed, Nd4jPointer state) {
    ND_TRY(need(state, "state"));
    static_cast<RandomState *>(state)->amplifier = seed;   // RandomBuffer::reSeed (helper_generator.h:181-183)
    return kOk;
}

int nd4jb200_destroy_random(Nd4jPointer state) {
    if (!state) return kOk;
    RandomState *s = static_cast<RandomState *>(state);
    if (s->ownsDev && s->devTable) cudaFree(s->devTable);
    if (s->ownsHost && s->hostTable) free(s->hostTable);
    delete s;
    return kOk;
}

int nd4jb200_exec_random(void *stream, int dtype, int opNum, Nd4jPointer state, void *z, const Nd4jLong *zShapeInfo,
                         const void *extraArguments) {
    ND_TRY(check_dtype(dtype));
    ND_TRY(need(state, "state")); ND_TRY(need(z, "z"));
    ShapeDesc zd;
    ND_TRY(parse_shape(zShapeInfo, "zShapeInfo", &zd));
    RandomState *s = static_cast<RandomState *>(state);
    ND_TRY(random_common(stream, dtype, opNum, 0, s, nullptr, nullptr, nullptr, nullptr, z, &zd, extraArguments, 0,
                         zd.length, zd.length));
    rewind_state(s, zd.length);
    return kOk;
}

int nd4jb200_exec_random_x(void *stream, int dtype, int opNum, Nd4jPointer state, const void *x,
                           const Nd4jLong *xShapeInfo, void *z, const Nd4jLong *zShapeInfo, const void *extraArguments) {
    ND_TRY(check_dtype(dtype));
    ND_TRY(need(state, "state")); ND_TRY(need(x, "x")); ND_TRY(need(z, "z"));
    ShapeDesc xd, zd;
    ND_TRY(parse_shape(xShapeInfo, "xShapeInfo", &xd));
    ND_TRY(parse_shape(zShapeInfo, "zShapeInfo", &zd));
    if (xd.length < zd.length) return bad_arg("execRandom: x holds fewer elements than z");
    RandomState *s = static_cast<RandomState *>(state);
    ND_TRY(random_common(stream, dtype, opNum, 1, s, x, &xd, nullptr, nullptr, z, &zd, extraArguments, 0, zd.length, zd.length));
    rewind_state(s, zd.length);
    return kOk;
}

int nd4jb200_exec_random_xy(void *stream, int dtype, int opNum, Nd4jPointer state, const void *x,
                            const Nd4jLong *xShapeInfo, const void *y, const Nd4jLong *yShapeInfo, void *z,
                            const Nd4jLong *zShapeInfo, const void *extraArguments) {
    ND_TRY(check_dtype(dtype));
    ND_TRY(need(state, "state")); ND_TRY(need(x, "x")); ND_TRY(need(y, "y")); ND_TRY(need(z, "z"));
    ShapeDesc xd, yd, zd;
    ND_TRY(parse_shape(xShapeInfo, "xShapeInfo", &xd));
    ND_TRY(parse_shape(yShapeInfo, "yShapeInfo", &yd));
    ND_TRY(parse_shape(zShapeInfo, "zShapeInfo", &zd));
    // Choice reads x and y by choice index and Binomial reads y by trial index: their lengths are unrelated to z's
    const bool tableOperands = opNum == 5 || opNum == 8;
    if (!tableOperands && (xd.length < zd.length || yd.length < zd.length))
        return bad_arg("execRandom: x or y holds fewer elements than z");
    if (opNum == 5 && xd.length < yd.length) return bad_arg("Choice: x holds fewer values than y holds probabilities");
    RandomState *s = static_cast<RandomState *>(state);
    ND_TRY(random_common(stream, dtype, opNum, 2, s, x, &xd, y, &yd, z, &zd, extraArguments, 0, zd.length, zd.length));
    LL advance = zd.length;
    if (opNum == 8 || opNum == 9) {
        // the binomial ops consume zLength * trials draws (special_random_ops.h:523-524); trials is
        // extraArguments[0], which lives on the device
        ND_TRY(need(extraArguments, "extraArguments"));
        double trials = 0;
        unsigned char raw[8] = {0};
        const size_t es = dtype == kF64 ? 8 : (dtype == kF32 ? 4 : 2);
        ND_CUDA(cudaMemcpyAsync(raw, extraArguments, es, cudaMemcpyDeviceToHost, as_stream(stream)));
        ND_CUDA(cudaStreamSynchronize(as_stream(stream)));
        if (dtype == kF64) trials = *reinterpret_cast<double *>(raw);
        else if (dtype == kF32) trials = *reinterpret_cast<float *>(raw);
        else trials = __half2float(*reinterpret_cast<__half *>(raw));
        const int t = (int) trials;
        advance = t > 0 ? zd.length * (LL) t : 0;
    }
    rewind_state(s, advance);
    return kOk;
}

int nd4jb200_exec_random_range(void *stream, int dtype, int opNum, int arity, Nd4jPointer state, const void *x,
                               const void *y, void *z, const void *extraArguments, Nd4jLong first, Nd4jLong count,
                               Nd4jLong length) {
    ND_TRY(check_dtype(dtype));
    ND_TRY(need(state, "state")); ND_TRY(need(z, "z"));
    if (arity < 0 || arity > 2) return bad_arg("arity must be 0, 1 or 2");
    if (arity >= 1) ND_TRY(need(x, "x"));
    if (arity == 2) ND_TRY(need(y, "y"));
    if (first < 0 || count < 0 || first + count > length) return bad_arg("range [first, first+count) must lie inside [0, length)");
    RandomState *s = static_cast<RandomState *>(state);
    return random_common(stream, dtype, opNum, arity, s, x, nullptr, y, nullptr, z, nullptr, extraArguments, first, count, length);
}

int nd4jb200_rng_rewind(Nd4jPointer state, Nd4jLong count) {
    ND_TRY(need(state, "state"));
    rewind_state(static_cast<RandomState *>(state), count);
    return kOk;
}

int nd4jb200_rng_get_state(Nd4jPointer state, Nd4jLong words[5]) {
    ND_TRY(need(state, "state"));
    RandomState *s = static_cast<RandomState *>(state);
    words[0] = s->seed; words[1] = s->position; words[2] = s->generation; words[3] = s->amplifier; words[4] = s->size;
    return kOk;
}

int nd4jb200_rng_set_state(Nd4jPointer state, const Nd4jLong words[4]) {
    ND_TRY(need(state, "state"));
    RandomState *s = static_cast<RandomState *>(state);
    if (words[1] < 0 || words[1] >= s->size) return bad_arg("currentPosition must lie inside the table");
    s->seed = words[0]; s->position = words[1]; s->generation = words[2]; s->amplifier = words[3];
    return kOk;
}

void *nd4jb200_rng_device_table(Nd4jPointer state) { return state ? static_cast<RandomState *>(state)->devTable : nullptr; }

// ---------------------------------------------------------------------------------------------
int nd4jb200_tad_only_shape_info(const Nd4jLong *xShapeInfo, const int *dimension, int dimensionLength,
                                 Nd4jLong *target, Nd4jLong *offsets) {
    return tad_only_shape_info(xShapeInfo, dimension, dimensionLength, target, offsets, nullptr);
}

int nd4jb200_dims_from_tad(const Nd4jLong *xShapeInfo, const Nd4jLong *tadShapeInfo, int *dimension) {
    ShapeDesc x, t;
    if (parse_shape(xShapeInfo, "xShapeInfo", &x) != kOk || parse_shape(tadShapeInfo, "tadShapeInfo", &t) != kOk) return -1;
    return dims_from_tad_info(x, t, dimension);
}

Nd4jLong nd4jb200_tad_count(const Nd4jLong *xShapeInfo, const int *dimension, int dimensionLength) {
    LL n = -1;
    if (tad_only_shape_info(xShapeInfo, dimension, dimensionLength, nullptr, nullptr, &n) != kOk) return -1;
    return n;
}

// ---------------------------------------------------------------------------------------------
int nd4jb200_get_available_devices(void) { int n = 0; if (cudaGetDeviceCount(&n) != cudaSuccess) return 0; return n; }
int nd4jb200_set_device(int device) { ND_CUDA(cudaSetDevice(device)); return kOk; }
int nd4jb200_get_device(void) { int d = -1; cudaGetDevice(&d); return d; }
Nd4jPointer nd4jb200_malloc_device(Nd4jLong bytes) {
    void *p = nullptr;
    cudaError_t e = cudaMalloc(&p, bytes > 0 ? (size_t) bytes : 1);
    if (e != cudaSuccess) { cuda_fail(e, "cudaMalloc"); return nullptr; }
    return p;
}
int nd4jb200_free_device(Nd4jPointer p) { ND_CUDA(cudaFree(p)); return kOk; }
Nd4jPointer nd4jb200_malloc_host(Nd4jLong bytes) {
    void *p = nullptr;
    cudaError_t e = cudaMallocHost(&p, bytes > 0 ? (size_t) bytes : 1);
    if (e != cudaSuccess) { cuda_fail(e, "cudaMallocHost"); return nullptr; }
    return p;
}
int nd4jb200_free_host(Nd4jPointer p) { ND_CUDA(cudaFreeHost(p)); return kOk; }
Nd4jPointer nd4jb200_create_stream(void) {
    cudaStream_t s = nullptr;
    cudaError_t e = cudaStreamCreateWithFlags(&s, cudaStreamNonBlocking);
    if (e != cudaSuccess) { cuda_fail(e, "cudaStreamCreate"); return nullptr; }
    return s;
}
int nd4jb200_destroy_stream(Nd4jPointer stream) { ND_CUDA(cudaStreamDestroy(as_stream(stream))); return kOk; }
int nd4jb200_stream_synchronize(Nd4jPointer stream) { ND_CUDA(cudaStreamSynchronize(as_stream(stream))); return kOk; }
Nd4jPointer nd4jb200_create_event(void) {
    cudaEvent_t e = nullptr;
    cudaError_t r = cudaEventCreate(&e);
    if (r != cudaSuccess) { cuda_fail(r, "cudaEventCreate"); return nullptr; }
    return e;
}
int nd4jb200_register_event(Nd4jPointer event, Nd4jPointer stream) {
    ND_CUDA(cudaEventRecord(static_cast<cudaEvent_t>(event), as_stream(stream)));
    return kOk;
}
int nd4jb200_event_synchronize(Nd4jPointer event) { ND_CUDA(cudaEventSynchronize(static_cast<cudaEvent_t>(event))); return kOk; }
int nd4jb200_destroy_event(Nd4jPointer event) { ND_CUDA(cudaEventDestroy(static_cast<cudaEvent_t>(event))); return kOk; }
int nd4jb200_event_elapsed_ms(Nd4jPointer start, Nd4jPointer stop, float *ms) {
    ND_CUDA(cudaEventElapsedTime(ms, static_cast<cudaEvent_t>(start), static_cast<cudaEvent_t>(stop)));
    return kOk;
}
static cudaMemcpyKind copy_kind(int flags) {
    switch (flags) {
        case 0: return cudaMemcpyHostToHost;
        case 1: return cudaMemcpyHostToDevice;
        case 2: return cudaMemcpyDeviceToHost;
        case 3: return cudaMemcpyDeviceToDevice;
        default: return cudaMemcpyDefault;
    }
}
int nd4jb200_memcpy_async(Nd4jPointer dst, Nd4jPointer src, Nd4jLong bytes, int flags, Nd4jPointer stream) {
    ND_CUDA(cudaMemcpyAsync(dst, src, (size_t) bytes, copy_kind(flags), as_stream(stream)));
    return kOk;
}
int nd4jb200_memcpy(Nd4jPointer dst, Nd4jPointer src, Nd4jLong bytes, int flags) {
    ND_CUDA(cudaMemcpy(dst, src, (size_t) bytes, copy_kind(flags)));
    return kOk;
}
int nd4jb200_memset_async(Nd4jPointer dst, int value, Nd4jLong bytes, Nd4jPointer stream) {
    ND_CUDA(cudaMemsetAsync(dst, value, (size_t) bytes, as_stream(stream)));
    return kOk;
}
static int with_device(int device, Nd4jLong *freeB, Nd4jLong *totalB) {
    int prev = 0;
    ND_CUDA(cudaGetDevice(&prev));
    ND_CUDA(cudaSetDevice(device));
    size_t f = 0, t = 0;
    cudaError_t e = cudaMemGetInfo(&f, &t);
    cudaSetDevice(prev);
    if (e != cudaSuccess) return cuda_fail(e, "cudaMemGetInfo");
    *freeB = (Nd4jLong) f; *totalB = (Nd4jLong) t;
    return kOk;
}
Nd4jLong nd4jb200_device_free_memory(int device) { Nd4jLong f = 0, t = 0; return with_device(device, &f, &t) == kOk ? f : -1; }
Nd4jLong nd4jb200_device_total_memory(int device) { Nd4jLong f = 0, t = 0; return with_device(device, &f, &t) == kOk ? t : -1; }
int nd4jb200_device_major(int device) {
    int v = 0; if (cudaDeviceGetAttribute(&v, cudaDevAttrComputeCapabilityMajor, device) != cudaSuccess) return -1; return v;
}
int nd4jb200_device_minor(int device) {
    int v = 0; if (cudaDeviceGetAttribute(&v, cudaDevAttrComputeCapabilityMinor, device) != cudaSuccess) return -1; return v;
}
const char *nd4jb200_device_name(int device) {
    static thread_local cudaDeviceProp prop;
    if (cudaGetDeviceProperties(&prop, device) != cudaSuccess) return "";
    return prop.name;
}

}  // extern "C"
#pragma GCC visibility pop
