// Host side of the reduction engine: picks the memory pattern, the group width and the number
// of segments per TAD, obtains scratch for split TADs and launches the kernels.
#pragma once
#include "reduce_engine.cuh"
#include "runtime.h"

namespace nd4jb200 {

struct ReduceCall {
    const void *x = nullptr;
    const void *y = nullptr;
    const void *extra = nullptr;
    void *z = nullptr;           // device results, numTads elements; may be the workspace for scalar calls
    TadPlan xPlan;
    TadPlan yPlan;               // only when y != nullptr
    bool yBroadcast = false;     // y (or x) is a single TAD reused for every TAD of the other operand
    LL finishLen = 0;            // n handed to the policy's finish()
    LL *zIndex = nullptr;        // index reductions: exact 64-bit positions go here instead of into z
    void *zState = nullptr;      // raw accumulator states (one per TAD) go here instead of finished results into z
    LL fixedSegment = 0;         // > 0: dense TADs are cut into segments of this many elements, each reduced by one
                                 // CTA, and merged by the finalize launch, whatever the number of TADs in the call,
                                 // so that the bits of a TAD's result depend on that TAD alone
};

struct MergeCall {
    const void *states;          // device: `count` accumulator states of the op's policy, in combine order
    int count;
    LL finishLen;
    const void *extra;
    void *z;                     // device: one element of the call's type
};

// Workspace layout: [256-byte result slot][kCounterSlots arrival counters][partial states]. The
// counter region is never used for anything else; the workspace is zero-filled when it is
// allocated and every launch re-zeroes the counters it used. Merging inside the launch pays off
// when a TAD has few segments, or when there are only a few TADs worked on by whole CTAs (whole-array
// reductions); with many segments of many TADs only a few CTAs would do all the merging, so those
// cases (and calls that need more counters than the region holds) leave the partials to the separate,
// fully parallel finalize launch.
template <class State>
Status split_scratch(cudaStream_t stream, ReduceArgs &a, size_t counters) {
    const size_t counterBytes = kCounterSlots * sizeof(unsigned);
    void *ws = nullptr;
    ND_TRY(workspace(stream, 256 + counterBytes + sizeof(State) * (size_t) a.numTads * a.splits, &ws, nullptr));
    // a handful of TADs that each take whole CTAs (whole-array reductions): the last CTA of a TAD folds all of
    // its segments with 256 threads, however many there are
    const bool fewWide = a.group == kBlock && a.numTads <= 8;
    a.counters = ((a.splits <= g_tuning[kTuneMaxInKernelMerge] || fewWide) && counters <= kCounterSlots)
                     ? reinterpret_cast<unsigned *>(static_cast<char *>(ws) + 256) : nullptr;
    a.partials = static_cast<char *>(ws) + 256 + counterBytes;
    return kOk;
}


template <class T, class P>
Status run_reduction(const ReduceCall &c, cudaStream_t stream) {
    typedef typename P::State State;
    constexpr int V = Elem<T>::kVec;
    // enough resident threads to cover HBM latency on every SM
    const LL kTargetThreads = (LL) kNumSMs * g_tuning[kTuneRowThreadsPerSm];
    const bool two = P::kInputs == 2;
    if (c.xPlan.numTads <= 0 || c.xPlan.tadLen < 0) return kOk;

    ReduceArgs a;
    a.x = c.x; a.y = c.y; a.extra = c.extra; a.z = c.z;
    a.partials = nullptr;
    a.counters = nullptr;
    a.numTads = c.xPlan.numTads;
    a.tadLen = c.xPlan.tadLen;
    a.xOuter = c.xPlan.outer; a.xInner = c.xPlan.inner;
    a.yOuter = two ? c.yPlan.outer : c.xPlan.outer;
    a.yInner = two ? c.yPlan.inner : c.xPlan.inner;
    a.finishLen = c.finishLen;
    a.zIndex = c.zIndex;
    a.zState = c.zState;
    a.splits = 1; a.cluster = 1; a.group = 32; a.mode = 2;
    a.partTadStride = 1; a.partSplitStride = 1;
    a.colLo = 0; a.colStrideX = 0; a.colStrideY = 0;
    a.xOuterHi = a.xOuter; a.yOuterHi = a.yOuter;

    const View &xi = a.xInner, &yi = a.yInner, &xo = a.xOuter, &yo = a.yOuter;
    const bool xUnit = xi.rank == 0 || (xi.rank == 1 && xi.stride[0] == 1);
    const bool yUnit = !two || yi.rank == 0 || (yi.rank == 1 && yi.stride[0] == 1);
    const bool rank1 = xi.rank <= 1 && (!two || yi.rank <= 1);

    // across-TAD pattern: strided walk inside a TAD, neighbouring TADs adjacent in memory
    bool cols = !xUnit && xi.rank == 1 && xo.rank >= 1 && xo.stride[xo.rank - 1] == 1 && xo.shape[xo.rank - 1] >= 16;
    if (cols && two) {
        cols = yi.rank == 1 && yo.rank == xo.rank && yo.stride[yo.rank - 1] == 1;
        for (int d = 0; cols && d < xo.rank; d++) cols = yo.shape[d] == xo.shape[d];
    }

    if (cols) {
        a.colLo = xo.shape[xo.rank - 1];
        a.colStrideX = xi.stride[0];
        a.colStrideY = two ? yi.stride[0] : 0;
        a.xOuterHi = xo; a.xOuterHi.rank = xo.rank - 1;
        a.yOuterHi = yo; a.yOuterHi.rank = yo.rank - 1;
        const LL hiCount = a.numTads / a.colLo;
        // vector loads across neighbouring TADs need every TAD row to start on a vector boundary
        constexpr int W = ColBytes<T, P>::v / (int) sizeof(T) > 0 ? ColBytes<T, P>::v / (int) sizeof(T) : 1;
        constexpr size_t WB = (size_t) W * sizeof(T);
        bool vec = W > 1 && a.colLo % W == 0 && reinterpret_cast<uintptr_t>(a.x) % WB == 0 && a.colStrideX % W == 0 &&
                   view_strides_multiple_of(a.xOuterHi, W);
        if (two) vec = vec && reinterpret_cast<uintptr_t>(a.y) % WB == 0 && a.colStrideY % W == 0 &&
                       view_strides_multiple_of(a.yOuterHi, W);
        const LL tiles = hiCount * ceil_div(a.colLo, 32 * (vec ? W : 1));
        LL splits = ceil_div((LL) kNumSMs * g_tuning[kTuneColCtasPerSm], tiles);
        const LL maxSplits = a.tadLen / (kColRows * 2 * ColUnroll<T, P>::v);   // at least two unrolled trips per thread
        if (splits > maxSplits) splits = maxSplits;
        if (splits < 1) splits = 1;
        if (splits > 4096) splits = 4096;
        // Segments of a TAD tile are grouped into thread-block clusters of 2, 4 or 8 CTAs that merge
        // through distributed shared memory; only one partial state per cluster reaches global memory.
        LL cluster = 1;
        LL maxCluster = g_tuning[kTuneMaxCluster] < 8 ? g_tuning[kTuneMaxCluster] : 8;
        // Clusters of 4 by default (with 28 segments per tile, seven clusters of 4 beat four of 8: Variance over
        // dimension 0 of [65536,1024] 0.053 against 0.059 ms), but where one cluster of 8 holds all segments of a
        // tile nothing passes through global memory and no arrival counter is needed (Sum over dimension 0 of
        // [8192,4096]: 0.0225 against 0.0249 ms).
        if (maxCluster == 4 && splits > 4 && splits <= 8) maxCluster = 8;
        while (cluster < splits && cluster * 2 <= maxCluster && cluster * 2 <= maxSplits) cluster *= 2;
        LL groups = ceil_div(splits, cluster);
        while (groups > 1 && groups * cluster > maxSplits) groups--;
        if (cluster == 1) groups = splits;
        a.cluster = (int) cluster;
        a.splits = (int) groups;
        a.partTadStride = 1; a.partSplitStride = a.numTads;
        if (a.splits > 1) ND_TRY(split_scratch<State>(stream, a, (size_t) tiles));
        dim3 grid((unsigned) tiles, (unsigned) (groups * cluster)), block(32, kColRows);
        if (cluster > 1) {
            if (vec) launch_kernel_clustered(k_reduce_cols<T, P, W>, grid, block, (unsigned) cluster, stream, a);
            else launch_kernel_clustered(k_reduce_cols<T, P, 1>, grid, block, (unsigned) cluster, stream, a);
        } else if (vec) launch_kernel(k_reduce_cols<T, P, W>, grid, block, stream, a);
        else launch_kernel(k_reduce_cols<T, P, 1>, grid, block, stream, a);
    } else {
        if (xUnit && yUnit) {
            bool vec = a.tadLen % V == 0 && aligned16(a.x) && view_strides_multiple_of(xo, V);
            if (two) vec = vec && aligned16(a.y) && view_strides_multiple_of(yo, V);
            a.mode = vec ? 0 : 1;
        } else {
            a.mode = rank1 ? 1 : 2;
        }
        const LL perLane = a.mode == 0 ? V : 1;
        // a warp per TAD needs no barrier; a whole CTA per TAD only pays off for long TADs or when
        // there are too few TADs to fill the machine with warps
        const LL tadBytes = a.tadLen * (LL) sizeof(T);
        if (tadBytes > 262144 || (tadBytes >= 8192 && a.numTads < 4096)) a.group = kBlock;
        else {
            int g = 1;
            while (g < 32 && (LL) g * perLane * 4 < a.tadLen) g <<= 1;
            a.group = g;
        }
        // few, long TADs: cut each into segments so that every SM has work
        LL groups = a.numTads;
        LL splits = 1;
        // whole CTAs per TAD (few, long TADs) stream best with twice as many threads resident
        const LL target = a.group == kBlock ? 2 * kTargetThreads : kTargetThreads;
        if (groups * a.group < target) {
            splits = ceil_div(target, groups * a.group);
            const LL maxSplits = a.tadLen / ((LL) a.group * perLane * 8);
            if (splits > maxSplits) splits = maxSplits;
            if (splits < 1) splits = 1;
        }
        // One very long TAD (whole-array reductions): segments of 2^17 elements handed out to a capped grid of
        // CTAs balance the tail better than one large segment per resident CTA (2^31 floats: 1.16 ms against 1.34 ms)
        LL fixedSegment = c.fixedSegment;
        if (fixedSegment == 0 && a.numTads == 1 && a.group == kBlock && a.tadLen >= (1LL << 22)) fixedSegment = 1 << 17;
        if (fixedSegment > 0) {
            a.group = kBlock;
            splits = ceil_div(a.tadLen, fixedSegment);
            if (splits < 1) splits = 1;
        }
        a.splits = (int) splits;
        a.partTadStride = a.splits; a.partSplitStride = 1;
        if (a.splits > 1) ND_TRY(split_scratch<State>(stream, a, (size_t) a.numTads));
        if (fixedSegment > 0) a.counters = nullptr;
        const LL totalSegs = a.numTads * a.splits;
        LL blocks = ceil_div(totalSegs, kBlock / a.group);
        // the grid is capped so that CTAs loop over several TADs instead of being launched once per handful of
        // TADs (measured: IMax 0.91 -> 0.95 at 16 per SM; half-precision reduce3 0.70 -> 0.75 at 8 per SM)
        const LL cap = (LL) kNumSMs * (sizeof(T) == 2 && g_tuning[kTuneRowCtasPerSm] > 8 ? 8 : g_tuning[kTuneRowCtasPerSm]);
        if (blocks > cap) blocks = cap;
        launch_kernel(k_reduce_tads<T, P>, dim3((unsigned) blocks), dim3(kBlock), stream, a);
    }
    if (a.splits > 1 && a.counters == nullptr) {
        LL blocks = a.partSplitStride == 1 ? ceil_div(a.numTads, kBlock / 32)    // one warp per TAD
                                           : ceil_div(a.numTads, kBlock);         // one thread per TAD
        if (blocks > kNumSMs * 16) blocks = kNumSMs * 16;
        launch_kernel(k_reduce_finalize<T, P>, dim3((unsigned) blocks), dim3(kBlock), stream, a);
    }
    ND_CUDA(cudaGetLastError());
    return kOk;
}

template <class T, class P>
Status run_merge_states(const MergeCall &m, cudaStream_t stream) {
    if (m.count <= 0) return bad_arg("no states to merge");
    launch_kernel(k_merge_states<T, P>, dim3(1), dim3(32), stream, m.states, m.count, m.finishLen, m.extra, m.z);
    ND_CUDA(cudaGetLastError());
    return kOk;
}

}  // namespace nd4jb200
