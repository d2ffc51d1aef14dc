// Row softmax family: the "special" transforms SoftMax (38), SoftMaxDerivative (39) and LogSoftMax
// (40) on matrices and vectors (include/ops/special_ops.h:1422-1940).
//
// The reference composes them from five to seven passes of the other families -- row max (reduce),
// subtract (broadcast), Exp (transform), row sum (reduce), divide (broadcast), then Log or y(1-y)
// -- each a full read and write of the matrix (special_ops.h:1490-1516). Here a row is read once,
// kept in registers (rows up to 1024 elements: one warp per row) or re-read from L2 (longer rows:
// one CTA per row), and written once. The arithmetic per element is the reference's:
//   e = exp(x - max);  y = e / sum(e);  SoftMax: y;  LogSoftMax: log(y);  Derivative: y * (1 - y)
// with the Exp and Log of the transform family. Only the order of the row sum differs (a tree
// instead of the reference's sequential / OpenMP-chunked loop), so results agree to the
// tolerance of a sum reduction.
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

constexpr int kSmWarpCols = 1024;  // longest row a warp keeps in registers (32 per lane)
constexpr int kSmBlock = 256;

template <class T, int KIND, class C> ND_D C softmax_finish(C e, C sum) {
    const C y = Elem<T>::to_c(Elem<T>::from_c(e / sum));     // the quotient is stored before Log / y(1-y) read it
    if (KIND == 0) return y;
    if (KIND == 1) return y * (C(1) - y);
    return log(y);
}

template <class C> ND_D C warp_max(C v) {
    for (int m = 16; m > 0; m >>= 1) { C o = __shfl_xor_sync(0xffffffffu, v, m); v = o > v ? o : v; }
    return v;
}
template <class C> ND_D C warp_sum(C v) {
    for (int m = 16; m > 0; m >>= 1) v += __shfl_xor_sync(0xffffffffu, v, m);
    return v;
}

// One warp per row, the row cached in registers: lane l holds columns l, l + 32, ...
template <class T, int KIND>
__global__ void __launch_bounds__(kSmBlock) k_softmax_warp(const SoftmaxArgs a) {
    grid_dependency_sync();
    typedef typename Elem<T>::C C;
    constexpr int K = kSmWarpCols / 32;
    const T *ax = static_cast<const T *>(a.x);
    T *az = static_cast<T *>(a.z);
    const int lane = threadIdx.x & 31;
    const LL warps = (LL) gridDim.x * (kSmBlock / 32);
    for (LL r = (LL) blockIdx.x * (kSmBlock / 32) + (threadIdx.x >> 5); r < a.rows; r += warps) {
        const T *xr = ax + r * a.xRow;
        T *zr = az + r * a.zRow;
        C v[K];
        C mx = -ND_INF(C);
#pragma unroll
        for (int k = 0; k < K; k++) {
            const LL c = lane + 32 * k;
            v[k] = c < a.cols ? Elem<T>::load(xr + c * a.xCol) : -ND_INF(C);
            mx = v[k] > mx ? v[k] : mx;
        }
        mx = warp_max(mx);
        C sum = C(0);
#pragma unroll
        for (int k = 0; k < K; k++) {
            const LL c = lane + 32 * k;
            // intermediate results are stored in the element type by the reference (half rows round here)
            v[k] = c < a.cols ? Elem<T>::to_c(Elem<T>::from_c(fn::expv(Elem<T>::to_c(Elem<T>::from_c(v[k] - mx))))) : C(0);
            sum += v[k];
        }
        sum = Elem<T>::to_c(Elem<T>::from_c(warp_sum(sum)));
#pragma unroll
        for (int k = 0; k < K; k++) {
            const LL c = lane + 32 * k;
            if (c < a.cols) Elem<T>::store(zr + c * a.zCol, softmax_finish<T, KIND, C>(v[k], sum));
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
            sum += Elem<T>::to_c(Elem<T>::from_c(fn::expv(Elem<T>::to_c(Elem<T>::from_c(Elem<T>::load(xr + c * a.xCol) - mx)))));
        sum = warp_sum(sum);
        __syncthreads();
        if (lane == 0) part[w] = sum;
        __syncthreads();
        if (threadIdx.x == 0) { C s = part[0]; for (int k = 1; k < kSmBlock / 32; k++) s += part[k]; bcast = Elem<T>::to_c(Elem<T>::from_c(s)); }
        __syncthreads();
        sum = bcast;
        for (LL c = threadIdx.x; c < a.cols; c += kSmBlock) {
            const C e = Elem<T>::to_c(Elem<T>::from_c(fn::expv(Elem<T>::to_c(Elem<T>::from_c(Elem<T>::load(xr + c * a.xCol) - mx)))));
            Elem<T>::store(zr + c * a.zCol, softmax_finish<T, KIND, C>(e, sum));
        }
        __syncthreads();
    }
}

template <class T, int KIND>
Status run_softmax(const SoftmaxArgs &a, cudaStream_t stream) {
    if (a.rows <= 0 || a.cols <= 0) return kOk;
    if (a.cols <= kSmWarpCols) {
        LL blocks = ceil_div(a.rows, kSmBlock / 32);
        const LL cap = (LL) kNumSMs * 16;
        if (blocks > cap) blocks = cap;
        launch_kernel(k_softmax_warp<T, KIND>, dim3((unsigned) blocks), dim3(kSmBlock), stream, a);
    } else {
        LL blocks = a.rows;
        const LL cap = (LL) kNumSMs * 8;
        if (blocks > cap) blocks = cap;
        launch_kernel(k_softmax_block<T, KIND>, dim3((unsigned) blocks), dim3(kSmBlock), stream, a);
    }
    ND_CUDA(cudaGetLastError());
    return kOk;
}

}  // namespace nd4jb200
