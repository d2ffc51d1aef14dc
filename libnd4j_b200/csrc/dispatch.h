// Per-element-type dispatch entry points. Each (family, element type) pair is compiled in its
// own translation unit (family_tu.cu with -DND_FAMILY / -DND_DTYPE) so the build parallelises.
#pragma once
#include "elementwise_engine.cuh"
#include "reduce_launch.cuh"
#include "rng_engine.cuh"
#include "reduce3_all.cuh"
#include "softmax.cuh"
#include "fused_engine.cuh"

namespace nd4jb200 {

#define ND_DECLARE_DISPATCH(S)                                                         \
    Status transform_##S(int opNum, const EwArgs &a, cudaStream_t st);                 \
    Status pairwise_##S(int opNum, const EwArgs &a, cudaStream_t st);                  \
    Status pairwise_post_##S(int opNum, const EwArgs &a, cudaStream_t st);             \
    Status chain_##S(int transformOp, const ChainArgs &a, cudaStream_t st);            \
    Status scalar_##S(int opNum, const EwArgs &a, cudaStream_t st);                    \
    Status broadcast_##S(int opNum, const BcArgs &a, cudaStream_t st);                 \
    Status scalar_tad_##S(int opNum, const BcArgs &a, cudaStream_t st);                \
    Status reduce_##S(int opNum, const ReduceCall &c, cudaStream_t st);                \
    Status reduce_merge_##S(int opNum, const MergeCall &m, cudaStream_t st);           \
    int reduce_state_bytes_##S(int opNum);                                             \
    Status reduce3_##S(int opNum, const ReduceCall &c, cudaStream_t st);               \
    Status reduce3_all_##S(int opNum, const ReduceCall &c, cudaStream_t st);           \
    Status softmax_##S(int kind, const SoftmaxArgs &a, cudaStream_t st);               \
    Status ismax_mark_##S(const IsMaxArgs &a, cudaStream_t st);                        \
    Status index_reduce_##S(int opNum, const ReduceCall &c, cudaStream_t st);          \
    Status summary_stats_##S(int opNum, const ReduceCall &c, cudaStream_t st);         \
    Status random_##S(int opNum, int arity, const RngArgs &a, cudaStream_t st);

ND_DECLARE_DISPATCH(f32)
ND_DECLARE_DISPATCH(f64)
ND_DECLARE_DISPATCH(f16)

}  // namespace nd4jb200
