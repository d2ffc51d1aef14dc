// Fused execution of the elementwise chain  z = pairwise( transform( broadcast(x, b) ), y ):
// one pass that reads x and y once and writes z once, with the broadcast vector in registers, instead of three
// launches that move the array through HBM seven times (2 + 2 + 3 array-sized streams). The reference's own
// fusion hook covers pairwise followed by scalar only (include/ops/meta_ops.h:13-52,
// include/loops/cuda/grid_shaped.cu:114-124); that pair is served by the POST form of k_elementwise.
//
// The broadcast and pairwise steps take one of the run-time selectable light ops (light_ops.cuh); the
// transform in the middle is a template parameter, so every functor of the transform table can sit there.
// Every intermediate goes through the element type exactly as if it had been stored and reloaded
// (through_memory), which makes the result bit-identical to the three separate launches.
#pragma once
#include "elementwise_engine.cuh"
#include "light_ops.cuh"

namespace nd4jb200 {

struct ChainArgs {
    const void *x;       // array whose TADs meet the vector b
    const void *b;       // broadcast vector, one value per position inside a TAD
    const void *y;       // second operand of the pairwise step, same shape as x
    void *z;
    const void *trExtra; // extra parameters of the transform, or null
    LL numTads, tadLen;
    View xOuter, xInner, yOuter, yInner, zOuter, zInner, bView;
    int bcCode, pwCode;  // LightOp codes
    int mode;            // 0 row tiles (dense TADs), 1 general
    LL rowsPerBlock;
};

template <class T, class Tr>
__global__ void __launch_bounds__(kEwBlock) k_chain(const ChainArgs a) {
    grid_dependency_sync();
    if constexpr (HasPrepare<Tr>::value) Tr::prepare();
    typedef typename Elem<T>::C C;
    constexpr int V = Elem<T>::kVec;
    const T *ax = static_cast<const T *>(a.x);
    const T *ab = static_cast<const T *>(a.b);
    const T *ay = static_cast<const T *>(a.y);
    T *az = static_cast<T *>(a.z);
    C p[Tr::kParams ? Tr::kParams : 1];
    load_params<T, Tr::kParams>(static_cast<const T *>(a.trExtra), p);
    const int bc = a.bcCode, pw = a.pwCode;

    if (a.mode == 0) {
        // a thread owns one 16-byte column group, keeps its slice of b in registers and walks down a tile of rows
        const LL col = ((LL) blockIdx.x * kEwBlock + threadIdx.x) * V;
        if (col >= a.tadLen) return;
        const LL xs = a.xOuter.rank ? a.xOuter.stride[0] : 0;
        const LL ys = a.yOuter.rank ? a.yOuter.stride[0] : 0;
        const LL zs = a.zOuter.rank ? a.zOuter.stride[0] : 0;
        const Pack<T> bv = load_pack_rw(ab + col);
        LL r = (LL) blockIdx.y * a.rowsPerBlock;
        LL rEnd = r + a.rowsPerBlock;
        if (rEnd > a.numTads) rEnd = a.numTads;
        for (; r < rEnd; r += kEwIlp) {
            Pack<T> xv[kEwIlp], yv[kEwIlp];
#pragma unroll
            for (int u = 0; u < kEwIlp; u++)
                if (r + u < rEnd) {
                    xv[u] = load_pack_rw(ax + (r + u) * xs + col);
                    yv[u] = load_pack_rw(ay + (r + u) * ys + col);
                } else {
                    xv[u] = Pack<T>(); yv[u] = Pack<T>();
                }
            // the three steps run tile-wide (rows past the end compute on zeros and are not stored), each
            // intermediate going through the element type as a store and a load between launches would make it
            C t[kEwIlp * V], o[kEwIlp * V];
#pragma unroll
            for (int u = 0; u < kEwIlp; u++)
#pragma unroll
                for (int k = 0; k < V; k++) { t[u * V + k] = Elem<T>::to_c(xv[u].v[k]); o[u * V + k] = Elem<T>::to_c(bv.v[k]); }
            light_apply_tile<C, kEwIlp * V>(bc, t, o);
#pragma unroll
            for (int i = 0; i < kEwIlp * V; i++) t[i] = through_memory<T>(Tr::template f<C>(through_memory<T>(t[i]), p));
#pragma unroll
            for (int u = 0; u < kEwIlp; u++)
#pragma unroll
                for (int k = 0; k < V; k++) o[u * V + k] = Elem<T>::to_c(yv[u].v[k]);
            light_apply_tile<C, kEwIlp * V>(pw, t, o);
#pragma unroll
            for (int u = 0; u < kEwIlp; u++) {
                if (r + u < rEnd) {
                    Pack<T> w;
#pragma unroll
                    for (int k = 0; k < V; k++) w.v[k] = Elem<T>::from_c(t[u * V + k]);
                    store_pack(az + (r + u) * zs + col, w);
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
            const LL oy = view_offset(a.yOuter, r) + view_offset(a.yInner, f);
            const LL oz = view_offset(a.zOuter, r) + view_offset(a.zInner, f);
            C t = through_memory<T>(light_apply<C>(bc, Elem<T>::load(ax + ox), Elem<T>::load(ab + view_offset(a.bView, f))));
            t = through_memory<T>(Tr::template f<C>(t, p));
            Elem<T>::store(az + oz, light_apply<C>(pw, t, Elem<T>::load(ay + oy)));
        }
    }
}

template <class T, class Tr>
Status run_chain(ChainArgs a, cudaStream_t stream) {
    constexpr int V = Elem<T>::kVec;
    if (a.numTads <= 0 || a.tadLen <= 0) return kOk;
    if (a.mode == 0) {
        const LL colBlocks = ceil_div(ceil_div(a.tadLen, V), kEwBlock);
        LL rowChunks = ceil_div((LL) kNumSMs * 16, colBlocks);
        if (rowChunks > a.numTads) rowChunks = a.numTads;
        if (rowChunks > 65535) rowChunks = 65535;
        a.rowsPerBlock = ceil_div(a.numTads, rowChunks);
        rowChunks = ceil_div(a.numTads, a.rowsPerBlock);
        launch_kernel(k_chain<T, Tr>, dim3((unsigned) colBlocks, (unsigned) rowChunks), dim3(kEwBlock), stream, a);
    } else {
        LL blocks = ceil_div(a.numTads * a.tadLen, kEwBlock);
        const LL cap = (LL) kNumSMs * 16;
        if (blocks > cap) blocks = cap;
        launch_kernel(k_chain<T, Tr>, dim3((unsigned) blocks), dim3(kEwBlock), stream, a);
    }
    ND_CUDA(cudaGetLastError());
    return kOk;
}

}  // namespace nd4jb200
