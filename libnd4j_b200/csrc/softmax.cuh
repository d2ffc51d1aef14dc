// Row softmax family: the "special" transforms SoftMax (38), SoftMaxDerivative (39) and LogSoftMax
// (40) on matrices and vectors (include/ops/special_ops.h:1422-1940).
//
// The reference composes them from five to seven passes of the other families -- row max (reduce),
// subtract (broadcast), Exp (transform), row sum (reduce), divide (broadcast), then Log or y(1-y)
// -- each a full read and write of the matrix (special_ops.h:1490-1516). Here a row is read once,
// kept in registers (up to 1024 elements per warp, 8192 per CTA) or, for longer or unaligned rows, re-read
// from L1/L2 (a warp per row in two sweeps; a CTA per row in three sweeps when there are only a few very
// long rows), and written once. The arithmetic per element is the reference's:
//   e = exp(x - max);  y = e / sum(e);  SoftMax: y;  LogSoftMax: log(y);  Derivative: y * (1 - y)
// Two things differ from the reference's passes: the order of the row sum (a tree instead of its
// sequential / OpenMP-chunked loop) and the last bits of exp (library exp, multiply by 1/sum), so
// results agree to the tolerance of a sum reduction (1e-5 relative in float), not to 2 ulp.
#pragma once
#include "functors.cuh"
#include "device_utils.cuh"
#include "runtime.h"

namespace nd4jb200 {

struct SoftmaxArgs {
    const void *x;
    void *z;
    LL rows, cols;
    LL xRow, xCol, zRow, zCol;     // element strides of a row start and of a column step
};

constexpr int kSmBlock = 256;

// `inv` is 1 / sum, rounded once per row: e * inv is within one ulp of e / sum (the reference's own
// build is free to make the same substitution, it is compiled with reciprocal math).
template <class T, int KIND, class C> ND_D C softmax_finish(C e, C inv) {
    const C y = Elem<T>::to_c(Elem<T>::from_c(e * inv));     // the quotient is stored before Log / y(1-y) read it
    if (KIND == 0) return y;
    if (KIND == 1) return y * (C(1) - y);
    return log(y);
}

// exp(x - max) with the CUDA library's expf / exp (2 / 1 ulp): a third of the instructions of the
// correctly-rounded-class exp of the Exp transform, and far inside this family's tolerance.
ND_D float softmax_exp(float x) { return expf(x); }
ND_D double softmax_exp(double x) { return exp(x); }

template <class C> ND_D C warp_max(C v) {
    for (int m = 16; m > 0; m >>= 1) { C o = __shfl_xor_sync(0xffffffffu, v, m); v = o > v ? o : v; }
    return v;
}
template <class C> ND_D C warp_sum(C v) {
    for (int m = 16; m > 0; m >>= 1) v += __shfl_xor_sync(0xffffffffu, v, m);
    return v;
}

// A row cached in registers by G threads (one warp, or the whole CTA), K values per thread: thread t
// holds columns t, t + G, ...; rows of up to G * K elements are read once and written once. Max and
// sum are reduced by shuffles inside a warp and, for G = 256, across the CTA's warps through shared
// memory (every thread folds the eight warp results in the same order).
template <class C> ND_D C block_combine(C v, C *slots, bool isMax) {
    const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
    __syncthreads();                    // the slots may still be read from the previous reduction
    if (lane == 0) slots[w] = v;
    __syncthreads();
    C r = slots[0];
#pragma unroll
    for (int k = 1; k < kSmBlock / 32; k++) r = isMax ? (slots[k] > r ? slots[k] : r) : r + slots[k];
    return r;
}

template <class T, int KIND, int G, int K>
__global__ void __launch_bounds__(kSmBlock, 4) k_softmax_cached(const SoftmaxArgs a) {
    grid_dependency_sync();
    typedef typename Elem<T>::C C;
    const T *ax = static_cast<const T *>(a.x);
    T *az = static_cast<T *>(a.z);
    __shared__ C slots[kSmBlock / 32];
    constexpr int kRowsPerBlock = kSmBlock / G;
    const int t = threadIdx.x % G;
    const int cols = (int) a.cols;       // at most G * K
    const LL stride = (LL) gridDim.x * kRowsPerBlock;
    // with G = 256 the row index is uniform over the CTA, so the barriers inside are reached by all
    for (LL r = (LL) blockIdx.x * kRowsPerBlock + threadIdx.x / G; r < a.rows; r += stride) {
        const T *xr = ax + r * a.xRow;
        T *zr = az + r * a.zRow;
        C v[K];
        C mx = -ND_INF(C);
#pragma unroll
        for (int k = 0; k < K; k++) {
            const int c = t + G * k;
            v[k] = c < cols ? Elem<T>::load(xr + c * a.xCol) : -ND_INF(C);
            mx = v[k] > mx ? v[k] : mx;
        }
        mx = warp_max(mx);
        if (G > 32) mx = block_combine(mx, slots, true);
        C sum = C(0);
#pragma unroll
        for (int k = 0; k < K; k++) {
            const int c = t + G * k;
            // intermediate results are stored in the element type by the reference (half rows round here)
            v[k] = c < cols ? Elem<T>::to_c(Elem<T>::from_c(softmax_exp(Elem<T>::to_c(Elem<T>::from_c(v[k] - mx))))) : C(0);
            sum += v[k];
        }
        sum = warp_sum(sum);
        if (G > 32) sum = block_combine(sum, slots, false);
        const C inv = C(1) / Elem<T>::to_c(Elem<T>::from_c(sum));
#pragma unroll
        for (int k = 0; k < K; k++) {
            const int c = t + G * k;
            if (c < cols) Elem<T>::store(zr + c * a.zCol, softmax_finish<T, KIND, C>(v[k], inv));
        }
    }
}

// The same with 16-byte packs and up to 32 values (16 doubles) per thread: rows of up to 1024 elements per
// warp (G = 32) or 8192 per CTA (G = 256) are read once, kept in registers, and need one exp per element
// instead of the two of the sweeping kernels. Needs unit column strides and 16-byte aligned rows.
template <class C> struct SmRegs {
    static constexpr int kVals = sizeof(C) == 8 ? 16 : 32;
    static constexpr int kCtas = sizeof(C) == 8 ? 2 : 4;      // resident CTAs per SM the register budget is set for
};

template <class T, int KIND, int G>
__global__ void __launch_bounds__(kSmBlock, SmRegs<typename Elem<T>::C>::kCtas) k_softmax_regs(const SoftmaxArgs a) {
    grid_dependency_sync();
    typedef typename Elem<T>::C C;
    constexpr int V = Elem<T>::kVec;
    constexpr int NP = SmRegs<C>::kVals / V;
    const T *ax = static_cast<const T *>(a.x);
    T *az = static_cast<T *>(a.z);
    __shared__ C slots[kSmBlock / 32];
    constexpr int kRowsPerBlock = kSmBlock / G;
    const int t = threadIdx.x % G;
    const int packs = (int) (a.cols / V);      // at most G * NP
    const LL stride = (LL) gridDim.x * kRowsPerBlock;
    for (LL r = (LL) blockIdx.x * kRowsPerBlock + threadIdx.x / G; r < a.rows; r += stride) {
        const T *xr = ax + r * a.xRow;
        T *zr = az + r * a.zRow;
        C v[NP][V];
        C mx = -ND_INF(C);
#pragma unroll
        for (int j = 0; j < NP; j++) {
            const int p = t + G * j;
            if (p < packs) {
                const Pack<T> pk = load_pack_rw(xr + (LL) p * V);
#pragma unroll
                for (int k = 0; k < V; k++) { v[j][k] = Elem<T>::to_c(pk.v[k]); mx = v[j][k] > mx ? v[j][k] : mx; }
            }
        }
        mx = warp_max(mx);
        if (G > 32) mx = block_combine(mx, slots, true);
        C sum = C(0);
#pragma unroll
        for (int j = 0; j < NP; j++) {
            if (t + G * j < packs) {
#pragma unroll
                for (int k = 0; k < V; k++) {
                    v[j][k] = Elem<T>::to_c(Elem<T>::from_c(softmax_exp(Elem<T>::to_c(Elem<T>::from_c(v[j][k] - mx)))));
                    sum += v[j][k];
                }
            }
        }
        sum = warp_sum(sum);
        if (G > 32) sum = block_combine(sum, slots, false);
        const C inv = C(1) / Elem<T>::to_c(Elem<T>::from_c(sum));
#pragma unroll
        for (int j = 0; j < NP; j++) {
            const int p = t + G * j;
            if (p < packs) {
                Pack<T> o;
#pragma unroll
                for (int k = 0; k < V; k++) o.v[k] = Elem<T>::from_c(softmax_finish<T, KIND, C>(v[j][k], inv));
                store_pack(zr + (LL) p * V, o);
            }
        }
    }
}

// One warp per row, two sweeps, nothing cached: the first sweep carries a running maximum m and the
// sum of exp(x - m), rescaled whenever the maximum moves ("online" softmax); the second re-reads the
// row, which the first left in L1/L2, and writes the results. Warps never wait for each other, so a
// CTA keeps eight independent rows in flight. VEC: unit column strides and 16-byte aligned rows.
template <class T, int KIND, bool VEC>
__global__ void __launch_bounds__(kSmBlock) k_softmax_online(const SoftmaxArgs a) {
    grid_dependency_sync();
    typedef typename Elem<T>::C C;
    constexpr int V = Elem<T>::kVec;
    const T *ax = static_cast<const T *>(a.x);
    T *az = static_cast<T *>(a.z);
    const int lane = threadIdx.x & 31;
    const LL warps = (LL) gridDim.x * (kSmBlock / 32);
    for (LL r = (LL) blockIdx.x * (kSmBlock / 32) + (threadIdx.x >> 5); r < a.rows; r += warps) {
        const T *xr = ax + r * a.xRow;
        T *zr = az + r * a.zRow;
        C m = -ND_INF(C), s = C(0);
        if (VEC) {
            for (LL c = (LL) lane * V; c < a.cols; c += 32 * V) {
                const Pack<T> pk = load_pack_rw(xr + c);
                C xv[V];
                C mp = -ND_INF(C);
#pragma unroll
                for (int k = 0; k < V; k++) { xv[k] = Elem<T>::to_c(pk.v[k]); mp = xv[k] > mp ? xv[k] : mp; }
                if (mp > m) { s *= softmax_exp(m - mp); m = mp; }
#pragma unroll
                for (int k = 0; k < V; k++) s += softmax_exp(Elem<T>::to_c(Elem<T>::from_c(xv[k] - m)));
            }
        } else {
            for (LL c = lane; c < a.cols; c += 32) {
                const C xv = Elem<T>::load(xr + c * a.xCol);
                if (xv > m) { s *= softmax_exp(m - xv); m = xv; }
                s += softmax_exp(Elem<T>::to_c(Elem<T>::from_c(xv - m)));
            }
        }
        // butterfly over the lanes' (m, s) pairs; equal maxima (also two empty lanes at -inf) need no rescale
        for (int off = 16; off > 0; off >>= 1) {
            const C mo = __shfl_xor_sync(0xffffffffu, m, off), so = __shfl_xor_sync(0xffffffffu, s, off);
            const C mn = mo > m ? mo : m;
            const C fa = m == mn ? C(1) : softmax_exp(m - mn), fb = mo == mn ? C(1) : softmax_exp(mo - mn);
            s = s * fa + so * fb;
            m = mn;
        }
        const C inv = C(1) / Elem<T>::to_c(Elem<T>::from_c(s));
        if (VEC) {
            for (LL c = (LL) lane * V; c < a.cols; c += 32 * V) {
                const Pack<T> pk = load_pack_rw(xr + c);
                Pack<T> o;
#pragma unroll
                for (int k = 0; k < V; k++) {
                    const C e = Elem<T>::to_c(Elem<T>::from_c(softmax_exp(Elem<T>::to_c(Elem<T>::from_c(Elem<T>::to_c(pk.v[k]) - m)))));
                    o.v[k] = Elem<T>::from_c(softmax_finish<T, KIND, C>(e, inv));
                }
                store_pack(zr + c, o);
            }
        } else {
            for (LL c = lane; c < a.cols; c += 32) {
                const C e = Elem<T>::to_c(Elem<T>::from_c(softmax_exp(Elem<T>::to_c(Elem<T>::from_c(Elem<T>::load(xr + c * a.xCol) - m)))));
                Elem<T>::store(zr + c * a.zCol, softmax_finish<T, KIND, C>(e, inv));
            }
        }
    }
}

// One CTA per row for long rows: three sweeps (max, sum of exp, write); the second and third
// re-read the row, which a row of this size leaves in L2.
template <class T, int KIND>
__global__ void __launch_bounds__(kSmBlock) k_softmax_block(const SoftmaxArgs a) {
    grid_dependency_sync();
    typedef typename Elem<T>::C C;
    const T *ax = static_cast<const T *>(a.x);
    T *az = static_cast<T *>(a.z);
    __shared__ C part[kSmBlock / 32];
    __shared__ C bcast;
    const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
    for (LL r = blockIdx.x; r < a.rows; r += gridDim.x) {
        const T *xr = ax + r * a.xRow;
        T *zr = az + r * a.zRow;
        C mx = -ND_INF(C);
        for (LL c = threadIdx.x; c < a.cols; c += kSmBlock) { C v = Elem<T>::load(xr + c * a.xCol); mx = v > mx ? v : mx; }
        mx = warp_max(mx);
        if (lane == 0) part[w] = mx;
        __syncthreads();
        if (threadIdx.x == 0) { C m = part[0]; for (int k = 1; k < kSmBlock / 32; k++) m = part[k] > m ? part[k] : m; bcast = m; }
        __syncthreads();
        mx = bcast;
        C sum = C(0);
        for (LL c = threadIdx.x; c < a.cols; c += kSmBlock)
            sum += Elem<T>::to_c(Elem<T>::from_c(softmax_exp(Elem<T>::to_c(Elem<T>::from_c(Elem<T>::load(xr + c * a.xCol) - mx)))));
        sum = warp_sum(sum);
        __syncthreads();
        if (lane == 0) part[w] = sum;
        __syncthreads();
        if (threadIdx.x == 0) { C s = part[0]; for (int k = 1; k < kSmBlock / 32; k++) s += part[k]; bcast = Elem<T>::to_c(Elem<T>::from_c(s)); }
        __syncthreads();
        const C inv = C(1) / bcast;
        for (LL c = threadIdx.x; c < a.cols; c += kSmBlock) {
            const C e = Elem<T>::to_c(Elem<T>::from_c(softmax_exp(Elem<T>::to_c(Elem<T>::from_c(Elem<T>::load(xr + c * a.xCol) - mx)))));
            Elem<T>::store(zr + c * a.zCol, softmax_finish<T, KIND, C>(e, inv));
        }
        __syncthreads();
    }
}

template <class T, int KIND>
Status run_softmax(const SoftmaxArgs &a, cudaStream_t stream) {
    if (a.rows <= 0 || a.cols <= 0) return kOk;
    const LL cap = (LL) kNumSMs * 16;
    constexpr int V = Elem<T>::kVec;
    if (a.cols <= 128 || a.rows >= (LL) kNumSMs * 8 || a.cols <= 8192) {
        // a warp per row: short rows cached in registers, the rest in two sweeps
        LL blocks = ceil_div(a.rows, kSmBlock / 32);
        if (blocks > cap) blocks = cap;
        const dim3 grid((unsigned) blocks), block(kSmBlock);
        const bool vec = a.xCol == 1 && a.zCol == 1 && a.cols % V == 0 && a.xRow % V == 0 && a.zRow % V == 0 &&
                         aligned16(a.x) && aligned16(a.z);
        constexpr LL kVals = SmRegs<typename Elem<T>::C>::kVals;
        if (a.cols <= 128) launch_kernel(k_softmax_cached<T, KIND, 32, 4>, grid, block, stream, a);
        else if (vec && a.cols <= 32 * kVals) launch_kernel(k_softmax_regs<T, KIND, 32>, grid, block, stream, a);
        else if (vec && a.cols <= kSmBlock * kVals && a.rows >= kNumSMs) {
            LL ctas = a.rows < cap ? a.rows : cap;
            launch_kernel(k_softmax_regs<T, KIND, 256>, dim3((unsigned) ctas), block, stream, a);
        } else if (vec) launch_kernel(k_softmax_online<T, KIND, true>, grid, block, stream, a);
        else launch_kernel(k_softmax_online<T, KIND, false>, grid, block, stream, a);
    } else {
        LL blocks = a.rows;
        if (blocks > cap) blocks = cap;
        launch_kernel(k_softmax_block<T, KIND>, dim3((unsigned) blocks), dim3(kSmBlock), stream, a);
    }
    ND_CUDA(cudaGetLastError());
    return kOk;
}

// ---- IsMax (special transform 41; include/ops/special_ops.h:1945-2400) ---------------------------------
// z = 1 at the position of the maximum of every TAD (the first one among equals, which is what the reference's
// strict "currMax < x" scan keeps), 0 elsewhere. The positions come from the IndexMax reduction of the
// indexreduce family; this kernel only writes the marks: element j of TAD r gets (j == index[r]).
struct IsMaxArgs {
    const LL *index;     // one exact position per TAD
    void *z;
    LL numTads, tadLen;
    View zOuter, zInner;
};

template <class T>
__global__ void __launch_bounds__(kSmBlock) k_ismax_mark(const IsMaxArgs a) {
    grid_dependency_sync();
    typedef typename Elem<T>::C C;
    T *az = static_cast<T *>(a.z);
    const LL total = a.numTads * a.tadLen;
    const LL nthreads = (LL) gridDim.x * kSmBlock;
    for (LL i = (LL) blockIdx.x * kSmBlock + threadIdx.x; i < total; i += nthreads) {
        const LL r = i / a.tadLen, j = i - r * a.tadLen;
        const LL hit = __ldg(a.index + r);
        Elem<T>::store(az + view_offset(a.zOuter, r) + view_offset(a.zInner, j), j == hit ? C(1) : C(0));
    }
}

template <class T>
Status run_ismax_mark(const IsMaxArgs &a, cudaStream_t stream) {
    const LL total = a.numTads * a.tadLen;
    if (total <= 0) return kOk;
    LL blocks = ceil_div(total, kSmBlock);
    const LL cap = (LL) kNumSMs * 16;
    if (blocks > cap) blocks = cap;
    launch_kernel(k_ismax_mark<T>, dim3((unsigned) blocks), dim3(kSmBlock), stream, a);
    ND_CUDA(cudaGetLastError());
    return kOk;
}

}  // namespace nd4jb200
