// Host-side runtime: error capture and the per-stream scratch workspace.
#include "runtime.h"
#include <map>
#include <mutex>
#include <sstream>
#include <vector>

namespace nd4jb200 {

std::atomic<unsigned long long> g_launches{0};
long long g_tuning[kTuneCount] = {3, 1024, 32, 1, 4, 16};

Status cuda_fail(cudaError_t e, const char *where) {
    std::ostringstream os;
    os << "CUDA error " << (int) e << " (" << cudaGetErrorString(e) << ") at " << where;
    set_error(os.str());
    return kCudaError;
}
Status bad_arg(const std::string &msg) { set_error(msg); return kBadArgument; }
Status unsupported(const std::string &msg) { set_error(msg); return kUnsupported; }
Status unknown_op(const char *family, int opNum) {
    std::ostringstream os;
    os << "unknown " << family << " opNum " << opNum;
    set_error(os.str());
    return kUnknownOp;
}

namespace {
struct Block { void *dev = nullptr; size_t cap = 0; void *host = nullptr; };
std::mutex g_mu;
std::map<std::pair<int, cudaStream_t>, Block> g_blocks;
// Blocks that were outgrown. They stay allocated until release_workspaces(): a caller may have handed out
// pointers into one (result slots, position lists) that launches still queued on the stream will use, and a
// block grows by half each time, so everything retired together is smaller than twice the live block.
std::vector<void *> g_retired;
}  // namespace

Status workspace(cudaStream_t stream, size_t bytes, void **dev, void **hostSlot) {
    int device = 0;
    ND_CUDA(cudaGetDevice(&device));
    std::lock_guard<std::mutex> lock(g_mu);
    Block &b = g_blocks[std::make_pair(device, stream)];
    if (bytes > b.cap) {
        size_t want = bytes < (size_t(4) << 20) ? (size_t(4) << 20) : bytes + bytes / 2;
        if (b.dev) {
            g_retired.push_back(b.dev);
            b.dev = nullptr; b.cap = 0;
        }
        ND_CUDA(cudaMalloc(&b.dev, want));
        // arrival counters live in this block and must start at zero. The fill is ordered on the stream the
        // block belongs to, i.e. in front of the launch that asked for it: a fill on the legacy default stream
        // would not be ordered against a non-blocking stream.
        ND_CUDA(cudaMemsetAsync(b.dev, 0, want, stream));
        b.cap = want;
    }
    if (hostSlot && !b.host) ND_CUDA(cudaMallocHost(&b.host, 64));
    if (dev) *dev = b.dev;
    if (hostSlot) *hostSlot = b.host;
    return kOk;
}

void release_workspaces() {
    std::lock_guard<std::mutex> lock(g_mu);
    for (auto &kv : g_blocks) {
        if (kv.second.dev) cudaFree(kv.second.dev);
        if (kv.second.host) cudaFreeHost(kv.second.host);
    }
    g_blocks.clear();
    for (void *p : g_retired) cudaFree(p);
    g_retired.clear();
}

}  // namespace nd4jb200
