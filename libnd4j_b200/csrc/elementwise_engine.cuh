// Elementwise engine: transform (unary), pairwise (binary), scalar (binary with a by-value
// operand), broadcast (TAD element vs vector element) and scalar-along-dimension (TAD vs one
// scalar per TAD). All of them stream their operands through HBM exactly once.
//
// Memory patterns:
//   dense    every operand is one unit-stride run and 16-byte aligned: 128-bit loads/stores,
//            four packs in flight per thread, grid sized to a multiple of the SM count.
//   strided  every operand walks linearly with its own element stride (ews path of the reference).
//   views    general rank-N strided operands: linear c-order index -> per-operand offset.
//   indexed  element i of every operand sits at an offset read from that operand's index array
//            (the xIndexes / yIndexes / resultIndexes overloads): a gather / scatter.
// In-place calls (z aliasing x or y) are legal: each element is read and written by the same
// thread and inputs are fetched with ordinary (coherent) loads.
#pragma once
#include "device_utils.cuh"
#include "light_ops.cuh"
#include "runtime.h"

namespace nd4jb200 {

struct EwArgs {
    const void *x;
    const void *y;
    void *z;
    const void *extra;
    LL n;
    double scalar;
    int mode;          // 0 dense, 1 strided, 2 views, 3 indexed
    LL sx, sy, sz;
    View vx, vy, vz;
    const LL *ix = nullptr, *iy = nullptr, *iz = nullptr;   // indexed: device arrays of n offsets per operand
    // POST kernels only: z = light_apply(postCode, f(x, y), postScalar), the pairwise-then-scalar pair of the
    // reference's meta-op hook (include/ops/meta_ops.h:13-52)
    int postCode = kLightNone;
    double postScalar = 0;
};

constexpr int kEwBlock = 256;
constexpr int kEwIlp = 4;

// ARITY 1: z = f(x, p);  2: z = f(x, y[i], p);  3: z = f(x, scalar, p)
template <class Op, int ARITY, class C> ND_D C ew_apply(C x, C y, C sc, const C *p) {
    if constexpr (ARITY == 1) return Op::template f<C>(x, p);
    else if constexpr (ARITY == 2) return Op::template f<C>(x, y, p);
    else return Op::template f<C>(x, sc, p);
}
// The optional second step of a POST kernel; the first step's result goes through the element type as if it
// had been stored by one launch and loaded by the next.
template <class T, bool POST, class C> ND_D C ew_post(const EwArgs &a, C r) {
    if constexpr (POST) return light_apply<C>(a.postCode, through_memory<T>(r), C(a.postScalar));
    else return r;
}
// Functors that keep a table in shared memory declare kPrepare and a prepare() every thread of the CTA calls.
template <class Op, class = void> struct HasPrepare { static constexpr bool value = false; };
template <class Op> struct HasPrepare<Op, decltype((void) Op::kPrepare)> { static constexpr bool value = true; };

template <class T, class Op, int ARITY, bool POST = false>
__global__ void __launch_bounds__(kEwBlock) k_elementwise(const EwArgs a) {
    grid_dependency_sync();
    if constexpr (HasPrepare<Op>::value) Op::prepare();
    typedef typename Elem<T>::C C;
    constexpr int V = Elem<T>::kVec;
    const T *ax = static_cast<const T *>(a.x);
    const T *ay = static_cast<const T *>(a.y);
    T *az = static_cast<T *>(a.z);
    C p[Op::kParams ? Op::kParams : 1];
    load_params<T, Op::kParams>(static_cast<const T *>(a.extra), p);
    const C sc = C(a.scalar);
    const LL tid = (LL) blockIdx.x * kEwBlock + threadIdx.x;
    const LL nthreads = (LL) gridDim.x * kEwBlock;

    if (a.mode == 0) {
        const LL npacks = a.n / V;
        for (LL base = tid; base < npacks; base += nthreads * kEwIlp) {
            Pack<T> xv[kEwIlp], yv[kEwIlp];
#pragma unroll
            for (int u = 0; u < kEwIlp; u++) {
                LL i = base + u * nthreads;
                if (i < npacks) {
                    xv[u] = load_pack_rw(ax + i * V);
                    if (ARITY == 2) yv[u] = load_pack_rw(ay + i * V);
                }
            }
            if constexpr (POST) {
                // both steps tile-wide, so that the second op is selected once per tile and not per element
                C t[kEwIlp * V], sv[kEwIlp * V];
#pragma unroll
                for (int u = 0; u < kEwIlp; u++)
#pragma unroll
                    for (int k = 0; k < V; k++) {
                        const bool live = base + u * nthreads < npacks;
                        C xc = live ? Elem<T>::to_c(xv[u].v[k]) : C(1);
                        C yc = (ARITY == 2 && live) ? Elem<T>::to_c(yv[u].v[k]) : C(1);
                        t[u * V + k] = through_memory<T>(ew_apply<Op, ARITY, C>(xc, yc, sc, p));
                        sv[u * V + k] = C(a.postScalar);
                    }
                light_apply_tile<C, kEwIlp * V>(a.postCode, t, sv);
#pragma unroll
                for (int u = 0; u < kEwIlp; u++) {
                    LL i = base + u * nthreads;
                    if (i < npacks) {
                        Pack<T> r;
#pragma unroll
                        for (int k = 0; k < V; k++) r.v[k] = Elem<T>::from_c(t[u * V + k]);
                        store_pack(az + i * V, r);
                    }
                }
            } else {
#pragma unroll
                for (int u = 0; u < kEwIlp; u++) {
                    LL i = base + u * nthreads;
                    if (i < npacks) {
                        Pack<T> r;
#pragma unroll
                        for (int k = 0; k < V; k++) {
                            C yc = ARITY == 2 ? Elem<T>::to_c(yv[u].v[k]) : C(0);
                            r.v[k] = Elem<T>::from_c(ew_apply<Op, ARITY, C>(Elem<T>::to_c(xv[u].v[k]), yc, sc, p));
                        }
                        store_pack(az + i * V, r);
                    }
                }
            }
        }
        // ragged tail shorter than one pack
        const LL i = npacks * V + tid;
        if (i < a.n) {
            C yc = ARITY == 2 ? Elem<T>::load(ay + i) : C(0);
            Elem<T>::store(az + i, ew_post<T, POST, C>(a, ew_apply<Op, ARITY, C>(Elem<T>::load(ax + i), yc, sc, p)));
        }
    } else {
        for (LL i = tid; i < a.n; i += nthreads) {
            LL ox, oy = 0, oz;
            if (a.mode == 1) { ox = i * a.sx; oz = i * a.sz; if (ARITY == 2) oy = i * a.sy; }
            else if (a.mode == 3) { ox = __ldg(a.ix + i); oz = __ldg(a.iz + i); if (ARITY == 2) oy = __ldg(a.iy + i); }
            else {
                ox = view_offset(a.vx, i); oz = view_offset(a.vz, i);
                if (ARITY == 2) oy = view_offset(a.vy, i);
            }
            C yc = ARITY == 2 ? Elem<T>::load(ay + oy) : C(0);
            Elem<T>::store(az + oz, ew_post<T, POST, C>(a, ew_apply<Op, ARITY, C>(Elem<T>::load(ax + ox), yc, sc, p)));
        }
    }
}

template <class T, class Op, int ARITY, bool POST = false>
Status run_elementwise(EwArgs a, cudaStream_t stream) {
    constexpr int V = Elem<T>::kVec;
    if (a.n <= 0) return kOk;
    LL work = a.mode == 0 ? ceil_div(a.n, V * kEwIlp) : a.n;
    LL blocks = ceil_div(work, kEwBlock);
    const LL cap = (LL) kNumSMs * 16;
    if (blocks > cap) blocks = cap;
    if (blocks < 1) blocks = 1;
    launch_kernel(k_elementwise<T, Op, ARITY, POST>, dim3((unsigned) blocks), dim3(kEwBlock), stream, a);
    ND_CUDA(cudaGetLastError());
    return kOk;
}

// ---- broadcast / scalar-along-dimension -------------------------------------------------------
struct BcArgs {
    const void *x;
    const void *y;     // broadcast: vector indexed by the position inside a TAD; per-TAD: one value per TAD
    void *z;
    const void *extra;
    LL numTads, tadLen;
    View xOuter, xInner, zOuter, zInner, yView;
    int mode;          // 0 row tiles (dense TADs), 1 general
    LL rowsPerBlock;
};

// PER_TAD false: z_tad[f] = f(x_tad[f], y[f]);  true: z_tad[f] = f(x_tad[f], y[r], p)
template <class T, class Op, bool PER_TAD>
__global__ void __launch_bounds__(kEwBlock) k_broadcast(const BcArgs a) {
    grid_dependency_sync();
    typedef typename Elem<T>::C C;
    constexpr int V = Elem<T>::kVec;
    const T *ax = static_cast<const T *>(a.x);
    const T *ay = static_cast<const T *>(a.y);
    T *az = static_cast<T *>(a.z);
    C p[Op::kParams ? Op::kParams : 1];
    load_params<T, Op::kParams>(static_cast<const T *>(a.extra), p);

    if (a.mode == 0) {
        // a thread owns one 16-byte column group and keeps its slice of y in registers while it
        // walks down the rows of its tile
        const LL col = ((LL) blockIdx.x * kEwBlock + threadIdx.x) * V;
        if (col >= a.tadLen) return;
        const LL xs = a.xOuter.rank ? a.xOuter.stride[0] : 0;
        const LL zs = a.zOuter.rank ? a.zOuter.stride[0] : 0;
        Pack<T> yv;
        if (!PER_TAD) yv = load_pack_rw(ay + col);
        LL r = (LL) blockIdx.y * a.rowsPerBlock;
        LL rEnd = r + a.rowsPerBlock;
        if (rEnd > a.numTads) rEnd = a.numTads;
        for (; r < rEnd; r += kEwIlp) {
            Pack<T> xv[kEwIlp];
#pragma unroll
            for (int u = 0; u < kEwIlp; u++)
                if (r + u < rEnd) xv[u] = load_pack_rw(ax + (r + u) * xs + col);
#pragma unroll
            for (int u = 0; u < kEwIlp; u++) {
                if (r + u < rEnd) {
                    C ys = PER_TAD ? Elem<T>::load(ay + (r + u)) : C(0);
                    Pack<T> o;
#pragma unroll
                    for (int k = 0; k < V; k++)
                        o.v[k] = Elem<T>::from_c(Op::template f<C>(Elem<T>::to_c(xv[u].v[k]),
                                                                  PER_TAD ? ys : Elem<T>::to_c(yv.v[k]), p));
                    store_pack(az + (r + u) * zs + col, o);
                }
            }
        }
    } else {
        const LL total = a.numTads * a.tadLen;
        const LL nthreads = (LL) gridDim.x * kEwBlock;
        for (LL i = (LL) blockIdx.x * kEwBlock + threadIdx.x; i < total; i += nthreads) {
            const LL r = i / a.tadLen;
            const LL f = i - r * a.tadLen;
            const LL ox = view_offset(a.xOuter, r) + view_offset(a.xInner, f);
            const LL oz = view_offset(a.zOuter, r) + view_offset(a.zInner, f);
            const LL oy = PER_TAD ? r : view_offset(a.yView, f);
            C out = Op::template f<C>(Elem<T>::load(ax + ox), Elem<T>::load(ay + oy), p);
            Elem<T>::store(az + oz, out);
        }
    }
}

template <class T, class Op, bool PER_TAD>
Status run_broadcast(BcArgs a, cudaStream_t stream) {
    constexpr int V = Elem<T>::kVec;
    if (a.numTads <= 0 || a.tadLen <= 0) return kOk;
    if (a.mode == 0) {
        const LL colBlocks = ceil_div(ceil_div(a.tadLen, V), kEwBlock);
        LL rowChunks = ceil_div((LL) kNumSMs * 16, colBlocks);
        if (rowChunks > a.numTads) rowChunks = a.numTads;
        if (rowChunks > 65535) rowChunks = 65535;
        a.rowsPerBlock = ceil_div(a.numTads, rowChunks);
        rowChunks = ceil_div(a.numTads, a.rowsPerBlock);
        dim3 grid((unsigned) colBlocks, (unsigned) rowChunks);
        launch_kernel(k_broadcast<T, Op, PER_TAD>, grid, dim3(kEwBlock), stream, a);
    } else {
        LL blocks = ceil_div(a.numTads * a.tadLen, kEwBlock);
        const LL cap = (LL) kNumSMs * 16;
        if (blocks > cap) blocks = cap;
        launch_kernel(k_broadcast<T, Op, PER_TAD>, dim3((unsigned) blocks), dim3(kEwBlock), stream, a);
    }
    ND_CUDA(cudaGetLastError());
    return kOk;
}

}  // namespace nd4jb200
