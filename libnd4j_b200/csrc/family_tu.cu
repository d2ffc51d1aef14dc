// One translation unit per (family, element type): instantiates that family's kernels for every
// opNum of the reference's table and exposes a switch-based dispatcher.
//   ND_DTYPE:  0 float, 1 double, 2 half
//   ND_FAMILY: 0 transform, 1 binary (pairwise, scalar, broadcast, scalar-along-dimension),
//              2 reduce, 3 reduce3 + indexreduce + summarystats, 4 random, 5 composites (reduce3 over all TAD pairs, row softmax family),
//              6 fused elementwise (broadcast -> transform -> pairwise chain, pairwise -> scalar pair)
#include "dispatch.h"
#include "functors.cuh"
#include "policies.cuh"

#if ND_DTYPE == 0
#define ND_T float
#define ND_S(name) name##_f32
#elif ND_DTYPE == 1
#define ND_T double
#define ND_S(name) name##_f64
#else
#define ND_T __half
#define ND_S(name) name##_f16
#endif

namespace nd4jb200 {

typedef Elem<ND_T>::C CT;

#if ND_FAMILY == 0
Status ND_S(transform)(int opNum, const EwArgs &a, cudaStream_t st) {
    switch (opNum) {
#define X(num, Name) case num: return run_elementwise<ND_T, fn::Name, 1>(a, st);
        ND_TRANSFORM_TABLE(X)
#undef X
        case 36: case 37: case 48: case 70: case 71:
            return unsupported("transform opNum " + std::to_string(opNum) +
                               " is a whole-array (special) transform: it is served for shaped calls, not for strided or indexed ones");
        case 43: case 44:
            return unsupported("transform DropOut/DropOutInverted draw from rand()/clock in the reference and are "
                               "not reproducible; use the random family (execRandom opNum 1/2)");
        default: return unknown_op("transform", opNum);
    }
}
#elif ND_FAMILY == 1
Status ND_S(pairwise)(int opNum, const EwArgs &a, cudaStream_t st) {
    switch (opNum) {
#define X(num, Name) case num: return run_elementwise<ND_T, fn::Name, 2>(a, st);
        ND_PAIRWISE_TABLE(X)
#undef X
        default: return unknown_op("pairwise transform", opNum);
    }
}
Status ND_S(scalar)(int opNum, const EwArgs &a, cudaStream_t st) {
    switch (opNum) {
#define X(num, Name) case num: return run_elementwise<ND_T, fn::Name, 3>(a, st);
        ND_SCALAR_TABLE(X)
#undef X
        default: return unknown_op("scalar", opNum);
    }
}
Status ND_S(broadcast)(int opNum, const BcArgs &a, cudaStream_t st) {
    switch (opNum) {
#define X(num, Name) case num: return run_broadcast<ND_T, fn::Name, false>(a, st);
        ND_BROADCAST_TABLE(X)
#undef X
        default: return unknown_op("broadcast", opNum);
    }
}
Status ND_S(scalar_tad)(int opNum, const BcArgs &a, cudaStream_t st) {
    switch (opNum) {
#define X(num, Name) case num: return run_broadcast<ND_T, fn::Name, true>(a, st);
        ND_SCALAR_TABLE(X)
#undef X
        default: return unknown_op("scalar along dimension", opNum);
    }
}
#elif ND_FAMILY == 2
Status ND_S(reduce)(int opNum, const ReduceCall &c, cudaStream_t st) {
    switch (opNum) {
#define X(num, Name) case num: return run_reduction<ND_T, pol::Reduce<fn::Name, CT> >(c, st);
        ND_REDUCE_TABLE(X)
#undef X
        case 19: return run_reduction<ND_T, pol::LogSumExp<CT> >(c, st);
        default: return unknown_op("reduce", opNum);
    }
}
Status ND_S(reduce_merge)(int opNum, const MergeCall &m, cudaStream_t st) {
    switch (opNum) {
#define X(num, Name) case num: return run_merge_states<ND_T, pol::Reduce<fn::Name, CT> >(m, st);
        ND_REDUCE_TABLE(X)
#undef X
        case 19: return run_merge_states<ND_T, pol::LogSumExp<CT> >(m, st);
        default: return unknown_op("reduce", opNum);
    }
}
int ND_S(reduce_state_bytes)(int opNum) {
    switch (opNum) {
#define X(num, Name) case num: return (int) sizeof(pol::Reduce<fn::Name, CT>::State);
        ND_REDUCE_TABLE(X)
#undef X
        case 19: return (int) sizeof(pol::LogSumExp<CT>::State);
        default: return 0;
    }
}
#elif ND_FAMILY == 3
Status ND_S(reduce3)(int opNum, const ReduceCall &c, cudaStream_t st) {
    switch (opNum) {
        case 0: return run_reduction<ND_T, pol::Reduce3<0, CT> >(c, st);
        case 1: return run_reduction<ND_T, pol::Reduce3<1, CT> >(c, st);
        case 2: return run_reduction<ND_T, pol::Reduce3<2, CT> >(c, st);
        case 3: return run_reduction<ND_T, pol::Reduce3<3, CT> >(c, st);
        case 4: return run_reduction<ND_T, pol::Reduce3<4, CT> >(c, st);
        case 5: return run_reduction<ND_T, pol::Reduce3<5, CT> >(c, st);
        case 6: return run_reduction<ND_T, pol::Reduce3<6, CT> >(c, st);
        case 7: return run_reduction<ND_T, pol::Reduce3<7, CT> >(c, st);
        default: return unknown_op("reduce3", opNum);
    }
}
Status ND_S(index_reduce)(int opNum, const ReduceCall &c, cudaStream_t st) {
    switch (opNum) {
        case 0: return run_reduction<ND_T, pol::IndexExtreme<0, CT> >(c, st);
        case 1: return run_reduction<ND_T, pol::IndexExtreme<1, CT> >(c, st);
        case 2: return run_reduction<ND_T, pol::IndexExtreme<2, CT> >(c, st);
        case 3: return run_reduction<ND_T, pol::IndexExtreme<3, CT> >(c, st);
        case 4: return run_reduction<ND_T, pol::IndexMatch<4, CT> >(c, st);
        case 5: return run_reduction<ND_T, pol::IndexMatch<5, CT> >(c, st);
        default: return unknown_op("index reduce", opNum);
    }
}
Status ND_S(summary_stats)(int opNum, const ReduceCall &c, cudaStream_t st) {
    switch (opNum) {
        case 0: return run_reduction<ND_T, pol::Stats<0, CT> >(c, st);
        case 1: return run_reduction<ND_T, pol::Stats<1, CT> >(c, st);
        default: return unknown_op("summary stats", opNum);
    }
}
#elif ND_FAMILY == 5
Status ND_S(reduce3_all)(int opNum, const ReduceCall &c, cudaStream_t st) {
    switch (opNum) {
        case 0: return run_reduce3_all<ND_T, pol::Reduce3<0, CT> >(c, st);
        case 1: return run_reduce3_all<ND_T, pol::Reduce3<1, CT> >(c, st);
        case 2: return run_reduce3_all<ND_T, pol::Reduce3<2, CT> >(c, st);
        case 3: return run_reduce3_all<ND_T, pol::Reduce3<3, CT> >(c, st);
        case 4: return run_reduce3_all<ND_T, pol::Reduce3<4, CT> >(c, st);
        case 5: return run_reduce3_all<ND_T, pol::Reduce3<5, CT> >(c, st);
        case 6: return run_reduce3_all<ND_T, pol::Reduce3<6, CT> >(c, st);
        case 7: return run_reduce3_all<ND_T, pol::Reduce3<7, CT> >(c, st);
        default: return unknown_op("reduce3", opNum);
    }
}
// kind: 0 SoftMax, 1 SoftMaxDerivative, 2 LogSoftMax
Status ND_S(softmax)(int kind, const SoftmaxArgs &a, cudaStream_t st) {
    if (kind == 0) return run_softmax<ND_T, 0>(a, st);
    if (kind == 1) return run_softmax<ND_T, 1>(a, st);
    return run_softmax<ND_T, 2>(a, st);
}
Status ND_S(ismax_mark)(const IsMaxArgs &a, cudaStream_t st) { return run_ismax_mark<ND_T>(a, st); }
#elif ND_FAMILY == 6
Status ND_S(chain)(int transformOp, const ChainArgs &a, cudaStream_t st) {
    switch (transformOp) {
#define X(num, Name) case num: return run_chain<ND_T, fn::Name>(a, st);
        ND_TRANSFORM_TABLE(X)
#undef X
        default: return unknown_op("transform", transformOp);
    }
}
Status ND_S(pairwise_post)(int opNum, const EwArgs &a, cudaStream_t st) {
    switch (opNum) {
#define X(num, Name) case num: return run_elementwise<ND_T, fn::Name, 2, true>(a, st);
        ND_PAIRWISE_TABLE(X)
#undef X
        default: return unknown_op("pairwise transform", opNum);
    }
}
#elif ND_FAMILY == 4
// Dense launches give every CTA one contiguous chunk of indices (a multiple of `quantum`), enough
// CTAs to fill the machine a few times over, so that the per-thread cursor set-up is amortised.
static void plan_chunks(LL count, LL quantum, LL *chunk, LL *blocks) {
    LL want = (LL) kNumSMs * 16;
    LL maxBlocks = ceil_div(count, quantum);
    if (want > maxBlocks) want = maxBlocks;
    if (want < 1) want = 1;
    *chunk = ceil_div(ceil_div(count, want), quantum) * quantum;
    *blocks = ceil_div(count, *chunk);
}
template <int OP, int ARITY>
static Status launch_random(RngArgs a, cudaStream_t st) {
    if (a.count <= 0) return kOk;
    constexpr int V = Elem<ND_T>::kVec;
    LL blocks;
    if (a.mode == 0) plan_chunks(a.count, (LL) kRngBlock * V, &a.chunk, &blocks);
    else {
        blocks = ceil_div(a.count, kRngBlock);
        const LL cap = (LL) kNumSMs * 32;
        if (blocks > cap) blocks = cap;
    }
    launch_kernel(k_random<ND_T, OP, ARITY>, dim3((unsigned) blocks), dim3(kRngBlock), st, a);
    ND_CUDA(cudaGetLastError());
    return kOk;
}
template <bool LOGNORMAL>
static Status launch_gaussian(RngArgs a, cudaStream_t st) {
    if (a.count <= 0) return kOk;
    LL blocks;
    plan_chunks(a.count, 2 * (LL) kRngBlock, &a.chunk, &blocks);
    launch_kernel(k_random_gaussian<ND_T, LOGNORMAL>, dim3((unsigned) blocks), dim3(kRngBlock), st, a);
    ND_CUDA(cudaGetLastError());
    return kOk;
}
static LL special_blocks(LL count) {
    LL blocks = ceil_div(count, kRngBlock);
    const LL cap = (LL) kNumSMs * 32;
    return blocks > cap ? cap : blocks;
}
template <int OP>
static Status by_arity(int arity, const RngArgs &a, cudaStream_t st) {
    if (arity == 0) return launch_random<OP, 0>(a, st);
    if (arity == 1) return launch_random<OP, 1>(a, st);
    return launch_random<OP, 2>(a, st);
}
Status ND_S(random)(int opNum, int arity, const RngArgs &a, cudaStream_t st) {
    switch (opNum) {
        case 0: return by_arity<0>(arity, a, st);
        case 1: return by_arity<1>(arity, a, st);
        case 2: return by_arity<2>(arity, a, st);
        case 3: return by_arity<3>(arity, a, st);
        case 4: return by_arity<4>(arity, a, st);
        case 7: return by_arity<7>(arity, a, st);
        case 12: return by_arity<12>(arity, a, st);
        case 13: return by_arity<13>(arity, a, st);
        case 100: return by_arity<100>(arity, a, st);
        case 6: return launch_gaussian<false>(a, st);    // reached only in the three-operand form
        case 10: return launch_gaussian<true>(a, st);
        case 5: {
            if (a.count <= 0) return kOk;
            // running sums first (one thread, the reference's summation order), then the draws
            launch_kernel(k_choice_sums<ND_T>, dim3(1), dim3(32), st, static_cast<const ND_T *>(a.y), a.sy, a.auxLen,
                          static_cast<ND_T *>(const_cast<void *>(a.aux)));
            launch_kernel(k_random_choice<ND_T>, dim3((unsigned) special_blocks(a.count)), dim3(kRngBlock), st, a);
            ND_CUDA(cudaGetLastError());
            return kOk;
        }
        case 8: case 9: {
            if (a.count <= 0) return kOk;
            if (opNum == 8) launch_kernel(k_random_binomial<ND_T, false>, dim3((unsigned) special_blocks(a.count)), dim3(kRngBlock), st, a);
            else launch_kernel(k_random_binomial<ND_T, true>, dim3((unsigned) special_blocks(a.count)), dim3(kRngBlock), st, a);
            ND_CUDA(cudaGetLastError());
            return kOk;
        }
        case 11: {
            if (a.count <= 0) return kOk;
            launch_kernel(k_random_truncated_normal<ND_T>, dim3((unsigned) special_blocks(a.count - a.count / 2)), dim3(kRngBlock), st, a);
            ND_CUDA(cudaGetLastError());
            return kOk;
        }
        default: return unknown_op("random", opNum);
    }
}
#endif

}  // namespace nd4jb200
