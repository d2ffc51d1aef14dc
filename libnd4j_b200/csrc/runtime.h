// Host-side runtime shared by the launchers: CUDA error capture, the per-stream scratch
// workspace and the launch-geometry helpers.
#pragma once
#include <cuda_runtime.h>
#include <cuda_fp16.h>
#include <atomic>
#include <string>
#include "common.h"
#include "shape_host.h"

namespace nd4jb200 {

Status cuda_fail(cudaError_t e, const char *where);
#define ND_CUDA(call)                                                  \
    do {                                                               \
        cudaError_t e__ = (call);                                      \
        if (e__ != cudaSuccess) return cuda_fail(e__, #call);          \
    } while (0)
#define ND_TRY(call)                                                   \
    do {                                                               \
        Status s__ = (call);                                           \
        if (s__ != kOk) return s__;                                    \
    } while (0)

// Scratch memory owned by the library, one block per (device, stream) so that calls on
// different streams never share it. The block only ever grows; an outgrown block is kept until
// release_workspaces(), so pointers into it stay valid for work already queued.
// `hostSlot`, when requested, is a 64-byte pinned buffer used to bring scalar results back.
Status workspace(cudaStream_t stream, size_t bytes, void **dev, void **hostSlot);
// Layout of a workspace block: [256-byte result slot][kCounterSlots arrival counters, always left zero]
// [scratch: partial states, index lists]. Only the part from kWorkspaceScratch on is free for a call to use.
constexpr size_t kCounterSlots = 65536;
constexpr size_t kWorkspaceScratch = 256 + kCounterSlots * sizeof(unsigned);
void release_workspaces();

// Host-to-device copy of a small list (pointer tables, swap lists) that does not stall the caller: the bytes are
// copied into a pinned staging buffer owned by the library (a ring of four per device and stream, each guarded by
// an event) and sent from there with a truly asynchronous copy. A copy straight from pageable memory is ordered
// behind the stream's earlier work and keeps the calling thread blocked until it has run, which serialises the
// host-side preparation of call k + 1 with the kernel of call k.
Status staged_upload(cudaStream_t stream, void *dev, const void *host, size_t bytes);
// The same in two steps, for callers that build the list in place: staging_begin hands out a pinned buffer of at
// least `bytes` (and the slot to commit), staging_commit sends its first `bytes` bytes to `dev`.
Status staging_begin(cudaStream_t stream, size_t bytes, void **host, int *slot);
Status staging_commit(cudaStream_t stream, int slot, void *dev, size_t bytes);

// Counts kernel launches issued by this library since load (read by the benchmark).
extern std::atomic<unsigned long long> g_launches;
inline void count_launch(int n = 1) { g_launches.fetch_add((unsigned long long) n, std::memory_order_relaxed); }

// Launch heuristics that may be overridden at run time (nd4jb200_set_tuning); defaults in runtime.cu.
enum Tuning { kTuneColCtasPerSm = 0, kTuneRowThreadsPerSm = 1, kTuneMaxInKernelMerge = 2, kTuneOverlapLaunch = 3, kTuneMaxCluster = 4, kTuneRowCtasPerSm = 5, kTuneCount = 6 };
extern long long g_tuning[kTuneCount];

// Every kernel of the library starts with grid_dependency_sync() (device_utils.cuh): it lets the
// next kernel of the stream be scheduled while this one drains and then waits for the previous
// kernel's memory operations. Launching with programmatic stream serialisation turns that on, so
// that launch latency and the kernel prologue overlap the predecessor's tail; ordering of all
// global memory accesses between consecutive kernels stays that of a plain stream.
template <class... KArgs, class... Args>
inline void launch_kernel(void (*kernel)(KArgs...), dim3 grid, dim3 block, cudaStream_t stream, Args &&...args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = 0;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = g_tuning[kTuneOverlapLaunch] ? 1 : 0;
    cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);   // errors surface in cudaGetLastError()
    count_launch();
}

// Same, with the CTAs of gridDim.y grouped into thread-block clusters of `clusterY` (<= 8, the portable limit).
template <class... KArgs, class... Args>
inline void launch_kernel_clustered(void (*kernel)(KArgs...), dim3 grid, dim3 block, unsigned clusterY, cudaStream_t stream,
                                    Args &&...args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = 0;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 1;
    attr[0].val.clusterDim.y = clusterY;
    attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = g_tuning[kTuneOverlapLaunch] ? 2 : 1;
    cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
    count_launch();
}

// The whole-array ("special") transforms Col2Im 36, Im2col 37, Histogram 48, Reverse 70, Pooling2D 71
// (special_transforms.cu); extraParams is a device pointer to element-type values.
struct ShapeDesc;
Status run_special_transform(int dtype, int opNum, const void *x, const ShapeDesc &xd, void *z, const ShapeDesc &zd,
                             const void *extraParams, cudaStream_t stream);

Status bad_arg(const std::string &msg);
Status unsupported(const std::string &msg);
Status unknown_op(const char *family, int opNum);

inline bool aligned16(const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }
inline bool view_strides_multiple_of(const View &v, LL m) {
    for (int i = 0; i < v.rank; i++) if (v.stride[i] % m != 0) return false;
    return true;
}
inline LL ceil_div(LL a, LL b) { return (a + b - 1) / b; }

}  // namespace nd4jb200
