// Shared host/device definitions for the sm_100a legacy-op backend.
//
// The backend serves the exec* families of the reference's NativeOps interface
// (blas/NativeOps.h): reduce, indexreduce, reduce3, summarystats, transform, pairwise
// transform, broadcast, scalar and random. Every entry point takes caller-owned device
// buffers plus HOST copies of the shapeInfo descriptors; all index arithmetic is decoded on
// the host into small POD "views" that are passed to the kernels by value.
#pragma once
#include <cstdint>
#include <cstddef>

#if defined(__CUDACC__)
#define ND_HD __host__ __device__
#define ND_D __device__ __forceinline__
#else
#define ND_HD
#define ND_D inline
#endif

namespace nd4jb200 {

typedef long long LL;

// Element types of the three exec*{Float,Double,Half} flavours (blas/NativeOps.h).
enum DType : int { kF32 = 0, kF64 = 1, kF16 = 2 };

constexpr int kMaxRank = 32;  // MAX_RANK of the reference (include/helpers/shape.h:23)
constexpr int kDevRank = 8;   // maximum rank of a view after unit-dim removal and axis merging
constexpr int kMaxDimension = 0x7fffffff;  // "whole array" marker in dimension[] (shape.h:21)

// A strided view iterated in c-order: linear index -> element offset. Unit axes are dropped
// and adjacent axes that walk memory uniformly are merged, so most arrays arrive as rank 1 or 2.
struct View {
    int rank;
    LL shape[kDevRank];
    LL stride[kDevRank];
};

ND_HD inline LL view_offset(const View &v, LL idx) {
    // c-order decomposition, innermost axis last.
    LL off = 0;
#pragma unroll 1
    for (int d = v.rank - 1; d > 0; --d) {
        LL q = idx / v.shape[d];
        LL r = idx - q * v.shape[d];
        off += r * v.stride[d];
        idx = q;
    }
    if (v.rank > 0) off += idx * v.stride[0];
    return off;
}

// Status codes returned by every C-ABI entry point.
enum Status : int {
    kOk = 0,
    kBadArgument = 1,     // null pointer, malformed shapeInfo, mismatching lengths
    kUnknownOp = 2,       // opNum not in the reference's op table for the family
    kUnsupported = 3,     // recognised but not served by this backend (message says what)
    kCudaError = 4,       // CUDA runtime failure (message carries cudaGetErrorString)
    kTooLarge = 5         // exceeds a fixed capacity (message names it)
};

}  // namespace nd4jb200
