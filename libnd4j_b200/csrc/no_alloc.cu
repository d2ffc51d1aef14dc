// Whole-array reduction for callers that must not allocate.
//
// Some hosts of this library run where device allocation is off the table: inside a memory pool
// whose owner has handed every byte of the device to its own arena (nd4j's workspaces do that),
// in a real-time loop that forbids calls which may synchronise the device, or in a process that
// was started with no allocation rights on the GPU it was given. The regular scalar reduction
// (nd4jb200_exec_reduce_scalar) keeps partial accumulator states in a per-stream workspace that
// it obtains with cudaMalloc / cudaMallocHost on first use. The entry point below does the same
// arithmetic without calling any allocator: its partial states live in the fixed device array
// `g_scratch`, which is part of the library image, and the result goes to a device location the
// caller supplies.
//
// Limits and rules that follow from the fixed array:
//   * the input is cut into segments of at most kSegment elements, one partial state each; the
//     array holds kMaxSegments states, so inputs longer than kSegment * kMaxSegments elements
//     (2^27) are refused with ND4JB200_ETOOLARGE before anything is launched;
//   * every GPU that loads the library carries the array (64 KiB) until the process exits;
//   * all calls on one device share the array. Every slot a call reads has been written by that
//     same call first, so nothing needs to be zeroed between calls, but two calls that are in
//     flight at the same time on one device (different streams or threads) would overwrite each
//     other's partial states: callers must order such calls themselves;
//   * the first call on each device looks up the array's device address (cudaGetSymbolAddress:
//     the name `g_scratch` in host code is only a host-side handle, not an address a kernel can
//     use). That first call should be made before any stream capture begins.
#include "../../include/nd4j_b200.h"
#include "functors.cuh"
#include "policies.cuh"
#include "reduce_engine.cuh"
#include "runtime.h"
#include <mutex>
#include <sstream>

using namespace nd4jb200;

namespace {

constexpr LL kSegment = 65536;            // elements per partial state
constexpr int kMaxSegments = 2048;        // states the array can hold
constexpr size_t kStateBytes = 32;        // largest accumulator state of the reduce family
constexpr size_t kScratchBytes = kMaxSegments * kStateBytes;   // 64 KiB

static __device__ __align__(256) unsigned char g_scratch[kScratchBytes];

constexpr int kMaxDevices = 64;
std::mutex g_mu;
void *g_scratchAddress[kMaxDevices] = {nullptr};

// Device address of g_scratch on the current device, looked up once per device.
Status scratch_address(void **out) {
    int device = 0;
    ND_CUDA(cudaGetDevice(&device));
    if (device < 0 || device >= kMaxDevices) return bad_arg("device ordinal outside the supported range");
    std::lock_guard<std::mutex> lock(g_mu);
    if (g_scratchAddress[device] == nullptr) {
        void *ptr = nullptr;
        ND_CUDA(cudaGetSymbolAddress((void **) &ptr, g_scratch));
        g_scratchAddress[device] = ptr;
    }
    *out = g_scratchAddress[device];
    return kOk;
}

template <class T, class P>
Status launch(ReduceArgs a, cudaStream_t stream) {
    static_assert(sizeof(typename P::State) <= kStateBytes, "state does not fit a scratch slot");
    if (a.splits == 1) {
        launch_kernel(k_reduce_tads<T, P>, dim3(1), dim3(kBlock), stream, a);
    } else {
        launch_kernel(k_reduce_tads<T, P>, dim3((unsigned) a.splits), dim3(kBlock), stream, a);
        launch_kernel(k_reduce_finalize<T, P>, dim3(1), dim3(kBlock), stream, a);
    }
    ND_CUDA(cudaGetLastError());
    return kOk;
}

template <class T>
Status dispatch(int opNum, const ReduceArgs &a, cudaStream_t stream) {
    typedef typename Elem<T>::C C;
    switch (opNum) {
#define X(num, Name) case num: return launch<T, pol::Reduce<fn::Name, C> >(a, stream);
        ND_REDUCE_TABLE(X)
#undef X
        case 19: return launch<T, pol::LogSumExp<C> >(a, stream);
        default: return unknown_op("reduce", opNum);
    }
}

}  // namespace

#pragma GCC visibility push(default)
extern "C" int nd4jb200_exec_reduce_scalar_noalloc(void *stream, int dtype, int opNum, const void *x,
                                                   const Nd4jLong *xShapeInfo, const void *extraParams, void *z) {
    if (x == nullptr) return bad_arg("x is null");
    if (z == nullptr) return bad_arg("z is null");
    ShapeDesc xd;
    ND_TRY(parse_shape(xShapeInfo, "xShapeInfo", &xd));
    if (xd.length <= 0) return bad_arg("the array is empty");
    const LL segments = ceil_div(xd.length, kSegment);
    if (segments > kMaxSegments) {
        std::ostringstream os;
        os << "array of " << xd.length << " elements needs " << segments << " partial states; the built-in scratch holds "
           << kMaxSegments << " (at most " << kSegment * kMaxSegments << " elements). Use nd4jb200_exec_reduce_scalar instead";
        set_error(os.str());
        return kTooLarge;
    }
    TadPlan plan;
    ND_TRY(make_tad_plan(xd, nullptr, 0, &plan));
    void *scratch = nullptr;
    ND_TRY(scratch_address(&scratch));

    ReduceArgs a;
    a.x = x; a.y = nullptr; a.extra = extraParams; a.z = z;
    a.partials = scratch;
    a.counters = nullptr;   // partials are merged by the separate finalize launch
    a.numTads = 1;
    a.tadLen = xd.length;
    a.xOuter = plan.outer; a.xInner = plan.inner;
    a.yOuter = plan.outer; a.yInner = plan.inner;
    a.group = kBlock;
    a.splits = (int) segments;
    a.partTadStride = a.splits; a.partSplitStride = 1;
    a.cluster = 1;
    a.colLo = 0; a.colStrideX = 0; a.colStrideY = 0;
    a.xOuterHi = plan.outer; a.yOuterHi = plan.outer;
    a.finishLen = xd.length;
    a.zIndex = nullptr;
    a.zState = nullptr;
    const size_t es = dtype == kF64 ? 8 : (dtype == kF16 ? 2 : 4);
    const LL V = 16 / (LL) es;
    const bool unit = plan.inner.rank == 0 || (plan.inner.rank == 1 && plan.inner.stride[0] == 1);
    if (unit && xd.length % V == 0 && aligned16(x)) a.mode = 0;
    else a.mode = plan.inner.rank <= 1 ? 1 : 2;

    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (dtype == kF32) return dispatch<float>(opNum, a, st);
    if (dtype == kF64) return dispatch<double>(opNum, a, st);
    if (dtype == kF16) return dispatch<__half>(opNum, a, st);
    return bad_arg("dtype must be 0 (float), 1 (double) or 2 (half)");
}
#pragma GCC visibility pop
