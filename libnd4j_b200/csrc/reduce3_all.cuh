// reduce3 "all pairs": z[r * yTads + g] = reduce3(TAD r of x, TAD g of y) for every pair of TADs
// (NativeOps::execReduce3All*, blas/NativeOps.h:314-360; reference loop include/loops/reduce3.h:919-990).
//
// The work is xTads * yTads * tadLen pair operations over (xTads + yTads) * tadLen elements, so
// unlike the other reductions it is arithmetic-bound once both TAD counts exceed a few dozen. A CTA
// of 256 threads owns a 64 x 64 tile of results: it stages 16 elements of 64 x-TADs and 64 y-TADs
// in shared memory per step and every thread folds them into its 4 x 4 accumulator states, so each
// staged element is reused 64 times from shared memory and 4 times from registers. The functors
// are arbitrary (|x - y|, min/max, equality tests, products), so this is plain FP32/FP64 pipe work.
#pragma once
#include "policies.cuh"
#include "runtime.h"
#include "reduce_launch.cuh"

namespace nd4jb200 {

constexpr int kAllTile = 64;    // TADs of x (and of y) per CTA
constexpr int kAllStep = 16;    // elements of every TAD staged per step
constexpr int kAllThreads = 256;

struct AllArgs {
    const void *x, *y, *extra;
    void *z;
    LL xTads, yTads, tadLen;
    View xOuter, xInner, yOuter, yInner;
    LL finishLen;
};

template <class T, class P>
__global__ void __launch_bounds__(kAllThreads) k_reduce3_all(const AllArgs a) {
    grid_dependency_sync();
    typedef typename Elem<T>::C C;
    typedef typename P::State State;
    __shared__ C xs[kAllStep][kAllTile + 1];
    __shared__ C ys[kAllStep][kAllTile + 1];
    C p[P::kParams ? P::kParams : 1];
    load_params<T, P::kParams>(static_cast<const T *>(a.extra), p);
    const T *ax = static_cast<const T *>(a.x);
    const T *ay = static_cast<const T *>(a.y);
    T *az = static_cast<T *>(a.z);

    const LL r0 = (LL) blockIdx.y * kAllTile, g0 = (LL) blockIdx.x * kAllTile;
    // compute mapping: thread (ty, tx) owns result rows ty + 16 i and columns tx + 16 j
    const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
    // staging mapping: thread loads element `le` of the step for TADs lt, lt + 16, lt + 32, lt + 48
    const int le = threadIdx.x & (kAllStep - 1), lt = threadIdx.x / kAllStep;
    LL xBase[4], yBase[4];
#pragma unroll
    for (int q = 0; q < 4; q++) {
        const LL r = r0 + lt + 16 * q, g = g0 + lt + 16 * q;
        xBase[q] = r < a.xTads ? view_offset(a.xOuter, r) : -1;
        yBase[q] = g < a.yTads ? view_offset(a.yOuter, g) : -1;
    }
    const bool xLin = a.xInner.rank <= 1, yLin = a.yInner.rank <= 1;
    const LL sx = a.xInner.rank ? a.xInner.stride[0] : 0, sy = a.yInner.rank ? a.yInner.stride[0] : 0;

    State s[4][4];
#pragma unroll
    for (int i = 0; i < 4; i++)
#pragma unroll
        for (int j = 0; j < 4; j++) P::init(s[i][j]);

    for (LL k0 = 0; k0 < a.tadLen; k0 += kAllStep) {
        const LL f = k0 + le;
        const bool in = f < a.tadLen;
        const LL xo = in ? (xLin ? f * sx : view_offset(a.xInner, f)) : 0;
        const LL yo = in ? (yLin ? f * sy : view_offset(a.yInner, f)) : 0;
        // positions past the TAD's end (and TADs past the last one) are staged as x = y = 0, which
        // every reduce3 functor maps to a contribution of 0
#pragma unroll
        for (int q = 0; q < 4; q++) {
            xs[le][lt + 16 * q] = (in && xBase[q] >= 0) ? Elem<T>::load(ax + xBase[q] + xo) : C(0);
            ys[le][lt + 16 * q] = (in && yBase[q] >= 0) ? Elem<T>::load(ay + yBase[q] + yo) : C(0);
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < kAllStep; kk++) {
            C xr[4], yr[4];
#pragma unroll
            for (int i = 0; i < 4; i++) { xr[i] = xs[kk][ty + 16 * i]; yr[i] = ys[kk][tx + 16 * i]; }
#pragma unroll
            for (int i = 0; i < 4; i++)
#pragma unroll
                for (int j = 0; j < 4; j++) P::accum(s[i][j], xr[i], yr[j], 0, p);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; i++) {
        const LL r = r0 + ty + 16 * i;
#pragma unroll
        for (int j = 0; j < 4; j++) {
            const LL g = g0 + tx + 16 * j;
            if (r < a.xTads && g < a.yTads) az[r * a.yTads + g] = Elem<T>::from_c(P::finish(s[i][j], a.finishLen, p));
        }
    }
}

template <class T, class P>
Status run_reduce3_all(const ReduceCall &c, cudaStream_t stream) {
    if (c.xPlan.numTads <= 0 || c.yPlan.numTads <= 0) return kOk;
    AllArgs a;
    a.x = c.x; a.y = c.y; a.extra = c.extra; a.z = c.z;
    a.xTads = c.xPlan.numTads; a.yTads = c.yPlan.numTads; a.tadLen = c.xPlan.tadLen;
    a.xOuter = c.xPlan.outer; a.xInner = c.xPlan.inner;
    a.yOuter = c.yPlan.outer; a.yInner = c.yPlan.inner;
    a.finishLen = c.finishLen;
    const LL gx = ceil_div(a.yTads, kAllTile), gy = ceil_div(a.xTads, kAllTile);
    if (gy > 65535) return unsupported("reduce3 all-pairs: more than 65535 * 64 TADs in x");
    launch_kernel(k_reduce3_all<T, P>, dim3((unsigned) gx, (unsigned) gy), dim3(kAllThreads), stream, a);
    ND_CUDA(cudaGetLastError());
    return kOk;
}

}  // namespace nd4jb200
