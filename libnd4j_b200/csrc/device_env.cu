// Device-environment members of the boundary that the exec* families do not need themselves but that callers
// of the reference's CUDA build resolve from the same library: peer-access control
// (blas/NativeOps.h:2047-2058; blas/cuda/NativeOps.cu:3854-3938) and the constant-memory staging area
// (blas/NativeOps.h:1836-1846; blas/cuda/NativeOps.cu:87, 4793-4834).
#include "../../include/nd4j_b200.h"
#include "runtime.h"

using namespace nd4jb200;

namespace {

// Same size as the reference's deviceConstantMemory: callers place shapeInfo descriptors here and pass the
// resulting device addresses as *ShapeInfo arguments.
__constant__ char g_constantSpace[49152];

bool g_p2pSupported = false;
bool g_p2pAllowed = false;

// Runs f(x, y, canAccess) for every ordered pair of distinct devices, with device x current, and restores the
// caller's device afterwards.
template <class F> Status for_each_peer_pair(F f) {
    int cur = 0, n = 0;
    ND_CUDA(cudaGetDevice(&cur));
    ND_CUDA(cudaGetDeviceCount(&n));
    Status result = kOk;
    for (int x = 0; x < n && result == kOk; x++) {
        if (cudaSetDevice(x) != cudaSuccess) { result = cuda_fail(cudaGetLastError(), "cudaSetDevice"); break; }
        for (int y = 0; y < n; y++) {
            if (x == y) continue;
            int can = 0;
            if (cudaDeviceCanAccessPeer(&can, x, y) != cudaSuccess) { cudaGetLastError(); can = 0; }
            f(x, y, can != 0);
        }
    }
    cudaSetDevice(cur);
    return result;
}

}  // namespace

#pragma GCC visibility push(default)
extern "C" {

int nd4jb200_check_p2p(void) {
    int n = 0;
    ND_CUDA(cudaGetDeviceCount(&n));
    // one device: everything lives on it, which the reference reports as "supported"
    bool all = true;
    if (n > 1) ND_TRY(for_each_peer_pair([&](int, int, bool can) { all = all && can; }));
    g_p2pSupported = all;
    return kOk;
}

int nd4jb200_is_p2p_available(void) { return g_p2pSupported ? 1 : 0; }

int nd4jb200_enable_p2p(int enable) {
    const bool want = enable != 0;
    if (want == g_p2pAllowed) return kOk;
    ND_TRY(for_each_peer_pair([&](int, int y, bool can) {
        if (!can) return;
        // "already enabled" / "not enabled" are not failures of the request
        if (want) cudaDeviceEnablePeerAccess(y, 0); else cudaDeviceDisablePeerAccess(y);
        cudaGetLastError();
    }));
    g_p2pAllowed = want;
    return kOk;
}

int nd4jb200_memcpy_constant_async(Nd4jLong offset, const void *src, Nd4jLong bytes, int flags, void *stream) {
    if (offset < 0 || bytes < 0 || offset + bytes > (Nd4jLong) sizeof(g_constantSpace))
        return bad_arg("memcpyConstantAsync: the range leaves the 49152-byte constant space");
    if (bytes == 0) return kOk;
    if (!src) return bad_arg("memcpyConstantAsync: src is null");
    const cudaMemcpyKind kind = flags == 3 ? cudaMemcpyDeviceToDevice : cudaMemcpyHostToDevice;
    ND_CUDA(cudaMemcpyToSymbolAsync(g_constantSpace, src, (size_t) bytes, (size_t) offset, kind,
                                    static_cast<cudaStream_t>(stream)));
    return kOk;
}

void *nd4jb200_get_constant_space(void) {
    void *p = nullptr;
    cudaError_t e = cudaGetSymbolAddress(&p, g_constantSpace);
    if (e != cudaSuccess) { cuda_fail(e, "cudaGetSymbolAddress(constant space)"); return nullptr; }
    return p;
}

}  // extern "C"
#pragma GCC visibility pop
