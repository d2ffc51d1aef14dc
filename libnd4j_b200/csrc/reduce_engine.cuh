// Reduction engine shared by the reduce, reduce3, indexreduce and summarystats families.
//
// A reduction call is "for every TAD r: z[r] = finish(fold(elements of TAD r))". The host
// plan (shape_host.h) describes the TADs as two views: `outer` maps r to the TAD's base offset
// and `inner` maps an element index j (c-order inside the TAD) to an offset from that base.
// Two memory patterns get their own kernels so that global loads stay coalesced:
//
//   along-TAD  (k_reduce_tads): consecutive elements of one TAD are (close to) adjacent in
//              memory. A group of g threads (1..32 lanes of a warp, or a whole 256-thread CTA)
//              walks one TAD segment with 128-bit loads when alignment allows, 128 bytes in
//              flight per thread.
//   across-TAD (k_reduce_cols): consecutive TADs are adjacent in memory and a TAD's own
//              elements are far apart (column reductions of row-major arrays, row reductions of
//              f-order views). 32 lanes read neighbouring TADs per row (vector loads when the
//              rows are aligned); 8 row-lanes per CTA and `splits` CTAs share the rows of one
//              TAD tile.
//
// A TAD may be cut into `splits` segments handled by different groups/CTAs; each writes its
// partial state to a scratch array. The partials of a TAD are merged in an order fixed by the
// segment numbers, either by the group that completes the TAD last (arrival counters; nobody
// waits on anybody: a group that is not last simply leaves) or by the separate k_reduce_finalize
// launch. All merges (lanes, warps, segments) happen in an order fixed by indices, never by
// arrival, so a call is bit-reproducible run to run.
//
// Policy concept (see policies.cuh):
//   typedef State;  static constexpr int kInputs (1|2), kParams, kColBytes;
//   init(State&);  accum(State&, C x, C y, LL j, const C* p);  merge(State&, const State&);
//   accum_many<N>(State&, const C (&x)[N], const C (&y)[N], LL j0, LL jstep, const C* p)
//       folds N elements with indices j0, j0 + jstep, ... (ascending) in one go;
//   C finish(const State&, LL n, const C* p);
#pragma once
#include <cooperative_groups.h>
#include "device_utils.cuh"

namespace nd4jb200 {

struct ReduceArgs {
    const void *x;
    const void *y;       // second operand (reduce3) or null
    const void *extra;   // device extra parameters or null
    void *z;             // one result per TAD, written densely
    void *partials;      // scratch for split TADs: State[numTads * splits]
    unsigned *counters;  // one zeroed arrival counter per TAD (along-TAD) or TAD tile (across-TAD): when set,
                         // the group that completes a TAD last merges its partials inside the same launch
                         // and re-zeroes the counter; when null the partials are left for k_reduce_finalize
    LL numTads;
    LL tadLen;
    View xOuter, xInner;
    View yOuter, yInner;
    int group;           // threads cooperating on one TAD segment (along-TAD kernel)
    int splits;          // segments per TAD whose partial states meet in global memory
    int cluster;         // across-TAD kernel: CTAs per thread-block cluster (1 = none). gridDim.y = splits * cluster;
                         // the segments of one cluster are merged through distributed shared memory first
    LL partTadStride;    // partial state of (TAD r, segment k) lives at partials[r * partTadStride + k * partSplitStride]
    LL partSplitStride;
    int mode;            // along-TAD: 0 = unit-stride inner + 128-bit loads, 1 = rank-1 inner, 2 = general inner view
    LL colLo;            // across-TAD: extent of the contiguous outer axis
    LL colStrideX, colStrideY;   // across-TAD: element stride between consecutive elements of a TAD
    View xOuterHi, yOuterHi;     // across-TAD: outer view without its contiguous axis
    LL finishLen;        // n handed to finish() (tadLen)
    LL *zIndex;          // index reductions only: when set, the winning position of TAD r is written here as an
                         // exact 64-bit integer instead of into z in the element type (half cannot hold
                         // positions above 2048 exactly, float none above 2^24)
    void *zState;        // when set, the raw accumulator state of TAD r is stored at zState[r] (sizeof(State) bytes
                         // each) instead of a finished result: partial results that a later step merges with the
                         // states of other shards (k_merge_states)
};

constexpr int kBlock = 256;

// Partial states written by other SMs during this launch are read through L2.
template <class S> ND_D S load_state_cg(const S *p) {
    S r;
    const unsigned *src = reinterpret_cast<const unsigned *>(p);
    unsigned *dst = reinterpret_cast<unsigned *>(&r);
#pragma unroll
    for (int w = 0; w < (int) (sizeof(S) / 4); w++) dst[w] = __ldcg(src + w);
    return r;
}

template <class T, class P, int N>
ND_D void fold_pack(typename P::State &s, const Pack<T> &xv, const Pack<T> &yv, LL j0,
                    const typename Elem<T>::C *p) {
    typedef typename Elem<T>::C C;
    C xa[N], ya[N];
#pragma unroll
    for (int k = 0; k < N; k++) {
        xa[k] = Elem<T>::to_c(xv.v[k]);
        ya[k] = P::kInputs == 2 ? Elem<T>::to_c(yv.v[k]) : C(0);
    }
    P::template accum_many<N>(s, xa, ya, j0, 1, p);
}

// One result per TAD. Policies whose state carries a position (`State::i`, marked by kIndexResult) can deliver
// it exactly through ReduceArgs::zIndex.
template <class P, class = void> struct HasIndexResult { static constexpr bool value = false; };
template <class P> struct HasIndexResult<P, decltype((void) P::kIndexResult)> { static constexpr bool value = true; };
template <class T, class P>
ND_D void write_result(const ReduceArgs &a, LL r, const typename P::State &s, const typename Elem<T>::C *p) {
    if (a.zState) { static_cast<typename P::State *>(a.zState)[r] = s; return; }
    if constexpr (HasIndexResult<P>::value) {
        if (a.zIndex) { a.zIndex[r] = s.i; return; }
    }
    static_cast<T *>(a.z)[r] = Elem<T>::from_c(P::finish(s, a.finishLen, p));
}

// Policies that can fold a whole tile of packs at once declare kTile (see pol::IndexExtreme).
template <class P, class = void> struct HasTile { static constexpr bool value = false; };
template <class P> struct HasTile<P, decltype((void) P::kTile)> { static constexpr bool value = true; };

// CTAs per SM the along-TAD kernel is compiled for. An allowance of 64 registers lets the compiler keep
// all loads of a trip in flight; a policy may name another allowance for half precision (kHalfRowCtas).
template <class T, class P, class = void> struct RowBudget { static constexpr int v = 4; };
template <class P> struct RowBudget<__half, P, decltype((void) P::kHalfRowCtas)> { static constexpr int v = P::kHalfRowCtas; };

// W consecutive elements (W * sizeof(T) is 2, 4, 8 or 16 bytes) moved as one transaction.
template <class T, int W> struct alignas(W * sizeof(T)) Vec {
    T v[W];
};
template <class T, int W> ND_D Vec<T, W> load_vec(const T *p) {
    Vec<T, W> r;
    constexpr int B = W * (int) sizeof(T);
    if (B == 16) *reinterpret_cast<uint4 *>(&r) = __ldg(reinterpret_cast<const uint4 *>(p));
    else if (B == 8) *reinterpret_cast<uint2 *>(&r) = __ldg(reinterpret_cast<const uint2 *>(p));
    else if (B == 4) *reinterpret_cast<unsigned *>(&r) = __ldg(reinterpret_cast<const unsigned *>(p));
    else *reinterpret_cast<unsigned short *>(&r) = __ldg(reinterpret_cast<const unsigned short *>(p));
    return r;
}

template <class T, class P>
__global__ void __launch_bounds__(kBlock, RowBudget<T, P>::v) k_reduce_tads(const ReduceArgs a) {
    grid_dependency_sync();
    typedef typename Elem<T>::C C;
    typedef typename P::State State;
    constexpr int V = Elem<T>::kVec;
    C p[P::kParams ? P::kParams : 1];
    load_params<T, P::kParams>(static_cast<const T *>(a.extra), p);
    const T *ax = static_cast<const T *>(a.x);
    const T *ay = static_cast<const T *>(a.y);

    const int g = a.group;
    const int groupsPerBlock = kBlock / g;
    const int lane = threadIdx.x % g;
    const LL totalSegs = a.numTads * a.splits;
    // segments start on a vector boundary so the 128-bit path stays aligned
    LL segLenAligned = a.tadLen;
    if (a.splits > 1) {
        const LL segLen = (a.tadLen + a.splits - 1) / a.splits;
        segLenAligned = (segLen + V - 1) / V * V;
    }

    __shared__ State warpStates[kBlock / 32];
    __shared__ int lastFlag;

    for (LL seg = (LL) blockIdx.x * groupsPerBlock + threadIdx.x / g; ; seg += (LL) gridDim.x * groupsPerBlock) {
        // a warp- or CTA-wide group leaves as a whole (seg is uniform across it)
        bool active = seg < totalSegs;
        if (g < 32) {
            // sub-warp groups: lanes of finished groups stay in the loop for the shuffles
            if (__all_sync(0xffffffffu, !active)) break;
        } else if (!active) break;

        State s;
        P::init(s);
        LL r = seg, sp = 0;
        if (active) {
            if (a.splits > 1) {     // the 64-bit division is only paid by split TADs
                r = seg / a.splits;
                sp = seg - r * a.splits;
            }
            const LL j0 = sp * segLenAligned;
            LL j1 = j0 + segLenAligned;
            if (j1 > a.tadLen) j1 = a.tadLen;
            const T *xb = ax + view_offset(a.xOuter, r);
            const T *yb = P::kInputs == 2 ? ay + view_offset(a.yOuter, r) : nullptr;
            if (a.mode == 0) {
                LL j = j0 + (LL) lane * V;
                const LL step = (LL) g * V;
                // U packs per operand are requested before any dependent arithmetic, so that every
                // lane keeps 128 bytes in flight (8 x 16 with one operand, 2 x 4 x 16 with two)
                constexpr int U = P::kInputs == 2 ? 4 : 8;
                for (; j + (U - 1) * step < j1; j += U * step) {
                    Pack<T> xv[U], yv[U];
#pragma unroll
                    for (int u = 0; u < U; u++) {
                        xv[u] = load_pack(xb + j + u * step);
                        if (P::kInputs == 2) yv[u] = load_pack(yb + j + u * step);
                    }
                    if constexpr (HasTile<P>::value) {
                        C xa[U * V];
#pragma unroll
                        for (int u = 0; u < U; u++)
#pragma unroll
                            for (int k = 0; k < V; k++) xa[u * V + k] = Elem<T>::to_c(xv[u].v[k]);
                        P::template accum_tile<U, V>(s, xa, j, (int) step, p);
                    } else {
#pragma unroll
                        for (int u = 0; u < U; u++) fold_pack<T, P, V>(s, xv[u], yv[u], j + u * step, p);
                    }
                }
                if (j < j1) {
                    // last, partial trip of the segment: the loads are still issued together; packs
                    // beyond the segment re-read the trip's first pack and are not folded
                    Pack<T> xv[U], yv[U];
#pragma unroll
                    for (int u = 0; u < U; u++) {
                        const LL ju = j + u * step < j1 ? j + u * step : j;
                        xv[u] = load_pack(xb + ju);
                        if (P::kInputs == 2) yv[u] = load_pack(yb + ju);
                    }
#pragma unroll
                    for (int u = 0; u < U; u++)
                        if (j + u * step < j1) fold_pack<T, P, V>(s, xv[u], yv[u], j + u * step, p);
                }
            } else if (a.mode == 1) {
                const LL sx = a.xInner.rank ? a.xInner.stride[0] : 0;
                const LL sy = (P::kInputs == 2 && a.yInner.rank) ? a.yInner.stride[0] : 0;
#pragma unroll 4
                for (LL j = j0 + lane; j < j1; j += g) {
                    C xv = Elem<T>::load(xb + j * sx);
                    C yv = P::kInputs == 2 ? Elem<T>::load(yb + j * sy) : C(0);
                    P::accum(s, xv, yv, j, p);
                }
            } else {
                for (LL j = j0 + lane; j < j1; j += g) {
                    C xv = Elem<T>::load(xb + view_offset(a.xInner, j));
                    C yv = P::kInputs == 2 ? Elem<T>::load(yb + view_offset(a.yInner, j)) : C(0);
                    P::accum(s, xv, yv, j, p);
                }
            }
        }

        if (g > 1) group_merge<P>(s, g < 32 ? g : 32);
        if (g == kBlock) {
            const int w = threadIdx.x >> 5;
            if ((threadIdx.x & 31) == 0) warpStates[w] = s;
            __syncthreads();
            if (threadIdx.x == 0) {
                s = warpStates[0];
                for (int k = 1; k < kBlock / 32; k++) P::merge(s, warpStates[k]);
            }
            __syncthreads();
        }
        if (a.splits == 1) {
            if (active && lane == 0) write_result<T, P>(a, r, s, p);
            continue;
        }
        State *parts = reinterpret_cast<State *>(a.partials);
        if (a.counters == nullptr) {
            if (active && lane == 0) parts[seg] = s;
            continue;
        }
        // publish the partial, then find out whether this group completed the TAD
        int last = 0;
        if (active && lane == 0) {
            parts[seg] = s;
            __threadfence();
            last = atomicAdd(&a.counters[r], 1u) == (unsigned) (a.splits - 1);
            if (last) a.counters[r] = 0u;
        }
        if (g == kBlock) {
            if (threadIdx.x == 0) lastFlag = last;
            __syncthreads();
            last = lastFlag;
        } else if (g > 1) {
            last = __shfl_sync(0xffffffffu, last, (threadIdx.x & 31) / g * g);
        }
        State m;
        P::init(m);
        if (last) {
            __threadfence();
            for (int k = lane; k < a.splits; k += g) P::merge(m, load_state_cg(parts + r * a.partTadStride + k));
        }
        if (g > 1) group_merge<P>(m, g < 32 ? g : 32);
        if (g == kBlock) {
            const int w = threadIdx.x >> 5;
            if ((threadIdx.x & 31) == 0) warpStates[w] = m;
            __syncthreads();
            if (threadIdx.x == 0) {
                m = warpStates[0];
                for (int k = 1; k < kBlock / 32; k++) P::merge(m, warpStates[k]);
            }
            __syncthreads();
        }
        if (last && lane == 0) write_result<T, P>(a, r, m, p);
    }
}

// blockDim = (32, 8). blockIdx.x enumerates (hi, tile of 32 * W consecutive TADs); blockIdx.y is
// the row split. W = 1, or a vector width chosen by the launcher when the TAD bases allow aligned
// vector loads: a thread then owns W neighbouring TADs and a warp reads 32 * W contiguous elements
// per row. R rows per operand are in flight per thread.
constexpr int kColRows = 8;

// bytes one lane loads per row: the policy's kColBytes, or its kHalfColBytes for half precision when it names one
template <class T, class P, class = void> struct ColBytes { static constexpr int v = P::kColBytes; };
template <class P> struct ColBytes<__half, P, decltype((void) P::kHalfColBytes)> { static constexpr int v = P::kHalfColBytes; };

// rows in flight per thread: 128 bytes over all operands, at most 8 rows
template <class T, class P> struct ColUnroll {
    static constexpr int kLane = ColBytes<T, P>::v < (int) sizeof(T) ? (int) sizeof(T) : ColBytes<T, P>::v;
    static constexpr int kFull = 128 / (kLane * P::kInputs);
    static constexpr int v = kFull > 8 ? 8 : kFull;
};

// Epilogue shared by the across-TAD kernels. The CTA's 8 row-lanes are merged through shared
// memory in one round: thread t of the CTA then owns TAD t of the tile (32 * W TADs), so partial
// states and results are written with consecutive threads on consecutive TADs. Partials of the
// across-TAD kernels are laid out [split][TAD] for that reason (a.partTadStride == 1).
// `rows` is shared memory for 8 * 32 * W states, `lastFlag` one shared int.
template <class T, class P, int W>
ND_D void cols_finish(const ReduceArgs &a, const typename P::State (&s)[W], typename P::State *rowsFlat, int *lastFlag,
                      LL hi, LL tile, const typename Elem<T>::C *p) {
    typedef typename P::State State;
    constexpr int kTile = 32 * W;
    State (*rows)[kTile] = reinterpret_cast<State (*)[kTile]>(rowsFlat);
    State *parts = reinterpret_cast<State *>(a.partials);
#pragma unroll
    for (int w = 0; w < W; w++) rows[threadIdx.y][threadIdx.x * W + w] = s[w];
    __syncthreads();
    const int t = threadIdx.y * 32 + threadIdx.x;
    const LL tlo = tile * kTile + t;
    const bool owner = t < kTile && tlo < a.colLo;
    const LL tr = hi * a.colLo + tlo;
    State m;
    P::init(m);
    if (owner) {
        m = rows[0][t];
#pragma unroll
        for (int k = 1; k < kColRows; k++) P::merge(m, rows[k][t]);
    }
    if (a.cluster > 1) {
        // The CTAs of a cluster hold consecutive row segments of the same TAD tile. Each leaves its
        // merged states in its own shared memory; rank 0 folds them in rank order through distributed
        // shared memory, so these segments never travel through global memory, fences or atomics.
        // Both cluster barriers are reached by every thread of every CTA of the cluster.
        namespace cg = cooperative_groups;
        cg::cluster_group cl = cg::this_cluster();
        __syncthreads();                       // every owner has read rows[*][t]
        if (owner) rowsFlat[t] = m;
        cl.sync();
        const unsigned rank = cl.block_rank();
        if (rank == 0 && owner) {
            for (unsigned q = 1; q < (unsigned) a.cluster; q++) {
                const State *remote = cl.map_shared_rank(rowsFlat, q);
                P::merge(m, remote[t]);
            }
        }
        cl.sync();                             // remote shared memory stays valid until rank 0 has read it
        if (rank != 0) return;
    }
    if (owner) {
        if (a.splits == 1) write_result<T, P>(a, tr, m, p);
        else parts[(LL) (blockIdx.y / a.cluster) * a.partSplitStride + tr] = m;
    }
    if (a.splits == 1 || a.counters == nullptr) return;
    // the CTA that completes this TAD tile last merges the tile's partials (nobody waits)
    __threadfence();
    __syncthreads();
    if (t == 0) {
        const int last = atomicAdd(&a.counters[blockIdx.x], 1u) == (unsigned) (a.splits - 1);
        if (last) a.counters[blockIdx.x] = 0u;
        *lastFlag = last;
    }
    __syncthreads();
    if (!*lastFlag) return;
    __threadfence();
    // row-lane y folds segments y, y + 8, ... (ascending) of every TAD of the tile, then the
    // owners fold the 8 row-lane results in ascending order
    for (int c = threadIdx.x; c < kTile; c += 32) {
        State m;
        P::init(m);
        const LL clo = tile * kTile + c;
        if (clo < a.colLo) {
            const State *src = parts + hi * a.colLo + clo;
            int k = threadIdx.y;
            for (; k + 3 * kColRows < a.splits; k += 4 * kColRows) {
                State q0 = load_state_cg(src + (LL) k * a.partSplitStride);
                State q1 = load_state_cg(src + (LL) (k + kColRows) * a.partSplitStride);
                State q2 = load_state_cg(src + (LL) (k + 2 * kColRows) * a.partSplitStride);
                State q3 = load_state_cg(src + (LL) (k + 3 * kColRows) * a.partSplitStride);
                P::merge(m, q0); P::merge(m, q1); P::merge(m, q2); P::merge(m, q3);
            }
            for (; k < a.splits; k += kColRows) P::merge(m, load_state_cg(src + (LL) k * a.partSplitStride));
        }
        rows[threadIdx.y][c] = m;
    }
    __syncthreads();
    if (owner) {
        State m = rows[0][t];
#pragma unroll
        for (int k = 1; k < kColRows; k++) P::merge(m, rows[k][t]);
        write_result<T, P>(a, tr, m, p);
    }
}

template <class T, class P, int W>
__global__ void __launch_bounds__(32 * kColRows, 4) k_reduce_cols(const ReduceArgs a) {
    grid_dependency_sync();
    typedef typename Elem<T>::C C;
    typedef typename P::State State;
    constexpr int R = ColUnroll<T, P>::v;
    C p[P::kParams ? P::kParams : 1];
    load_params<T, P::kParams>(static_cast<const T *>(a.extra), p);
    const T *ax = static_cast<const T *>(a.x);
    const T *ay = static_cast<const T *>(a.y);

    const LL tilesPerHi = (a.colLo + 32 * W - 1) / (32 * W);
    const LL hi = blockIdx.x / tilesPerHi;
    const LL tile = blockIdx.x - hi * tilesPerHi;
    const LL lo = (tile * 32 + threadIdx.x) * W;
    const bool active = lo < a.colLo;          // colLo is a multiple of W on the vector path
    const LL r = hi * a.colLo + lo;

    State s[W];
#pragma unroll
    for (int w = 0; w < W; w++) P::init(s[w]);
    if (active) {
        const T *xb = ax + view_offset(a.xOuterHi, hi) + lo;
        const T *yb = P::kInputs == 2 ? ay + view_offset(a.yOuterHi, hi) + lo : nullptr;
        const LL step = (LL) gridDim.y * kColRows;
        LL j = (LL) blockIdx.y * kColRows + threadIdx.y;
        for (; j + (R - 1) * step < a.tadLen; j += R * step) {
            Vec<T, W> xv[R], yv[R];
#pragma unroll
            for (int u = 0; u < R; u++) {
                xv[u] = load_vec<T, W>(xb + (j + u * step) * a.colStrideX);
                if (P::kInputs == 2) yv[u] = load_vec<T, W>(yb + (j + u * step) * a.colStrideY);
            }
#pragma unroll
            for (int w = 0; w < W; w++) {
                C xa[R], ya[R];
#pragma unroll
                for (int u = 0; u < R; u++) {
                    xa[u] = Elem<T>::to_c(xv[u].v[w]);
                    ya[u] = P::kInputs == 2 ? Elem<T>::to_c(yv[u].v[w]) : C(0);
                }
                P::template accum_many<R>(s[w], xa, ya, j, step, p);
            }
        }
        if (j < a.tadLen) {
            // last, partial trip: the loads are still issued together; rows beyond the TAD re-read
            // the trip's first row and are not folded
            Vec<T, W> xv[R], yv[R];
#pragma unroll
            for (int u = 0; u < R; u++) {
                const LL ju = j + u * step < a.tadLen ? j + u * step : j;
                xv[u] = load_vec<T, W>(xb + ju * a.colStrideX);
                if (P::kInputs == 2) yv[u] = load_vec<T, W>(yb + ju * a.colStrideY);
            }
#pragma unroll
            for (int u = 0; u < R; u++) {
                if (j + u * step < a.tadLen) {
#pragma unroll
                    for (int w = 0; w < W; w++)
                        P::accum(s[w], Elem<T>::to_c(xv[u].v[w]), P::kInputs == 2 ? Elem<T>::to_c(yv[u].v[w]) : C(0),
                                 j + u * step, p);
                }
            }
        }
    }
    __shared__ State rows[kColRows * 32 * W];
    __shared__ int lastFlag;
    cols_finish<T, P, W>(a, s, rows, &lastFlag, hi, tile, p);
}

// Separate merge pass for calls whose partials were not merged inside the reduction launch.
// Layout [TAD][segment] (partSplitStride == 1): one warp per TAD, lane l folds segments l, l + 32,
// ... in ascending order, then the 32 lane results are merged by the fixed butterfly.
// Layout [segment][TAD] (partTadStride == 1): one thread per TAD folds its segments in ascending
// order, four loads in flight. Both read the scratch coalesced.
template <class T, class P>
__global__ void __launch_bounds__(kBlock) k_reduce_finalize(const ReduceArgs a) {
    grid_dependency_sync();
    typedef typename Elem<T>::C C;
    typedef typename P::State State;
    C p[P::kParams ? P::kParams : 1];
    load_params<T, P::kParams>(static_cast<const T *>(a.extra), p);
    const State *parts = reinterpret_cast<const State *>(a.partials);
    if (a.partSplitStride != 1) {
        for (LL r = (LL) blockIdx.x * kBlock + threadIdx.x; r < a.numTads; r += (LL) gridDim.x * kBlock) {
            State s;
            P::init(s);
            const State *src = parts + r * a.partTadStride;
            int k = 0;
            for (; k + 3 < a.splits; k += 4) {
                State q0 = src[(LL) k * a.partSplitStride], q1 = src[(LL) (k + 1) * a.partSplitStride];
                State q2 = src[(LL) (k + 2) * a.partSplitStride], q3 = src[(LL) (k + 3) * a.partSplitStride];
                P::merge(s, q0); P::merge(s, q1); P::merge(s, q2); P::merge(s, q3);
            }
            for (; k < a.splits; k++) P::merge(s, src[(LL) k * a.partSplitStride]);
            write_result<T, P>(a, r, s, p);
        }
        return;
    }
    const int lane = threadIdx.x & 31;
    const LL warpsTotal = (LL) gridDim.x * (kBlock / 32);
    for (LL r = (LL) blockIdx.x * (kBlock / 32) + (threadIdx.x >> 5); r < a.numTads; r += warpsTotal) {
        State s;
        P::init(s);
        for (int k = lane; k < a.splits; k += 32) P::merge(s, parts[r * a.partTadStride + k]);
        group_merge<P>(s, 32);
        if (lane == 0) write_result<T, P>(a, r, s, p);
    }
}

// Folds `count` accumulator states in index order and writes the finished result: the combine step of a
// reduction whose shards were reduced separately (by other launches, or on other GPUs and gathered here).
// The order is fixed by position in `states`, so the result depends on how the array was cut into shards
// but not on which process reduced which shard.
template <class T, class P>
__global__ void k_merge_states(const void *states, int count, LL finishLen, const void *extra, void *z) {
    grid_dependency_sync();
    typedef typename Elem<T>::C C;
    typedef typename P::State State;
    if (blockIdx.x != 0 || threadIdx.x != 0) return;
    C p[P::kParams ? P::kParams : 1];
    load_params<T, P::kParams>(static_cast<const T *>(extra), p);
    const State *st = static_cast<const State *>(states);
    State m = st[0];
    for (int i = 1; i < count; i++) { State o = st[i]; P::merge(m, o); }
    static_cast<T *>(z)[0] = Elem<T>::from_c(P::finish(m, finishLen, p));
}

}  // namespace nd4jb200
