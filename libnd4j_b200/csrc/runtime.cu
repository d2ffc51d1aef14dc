// Host-side runtime: error capture and the per-stream scratch workspace.
#include "runtime.h"
#include <cstring>
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

namespace {
struct Staging {
    void *buf[4] = {nullptr, nullptr, nullptr, nullptr};
    size_t cap[4] = {0, 0, 0, 0};
    cudaEvent_t done[4] = {nullptr, nullptr, nullptr, nullptr};
    int next = 0;
};
std::map<std::pair<int, cudaStream_t>, Staging> g_staging;
}  // namespace

Status staging_begin(cudaStream_t stream, size_t bytes, void **host, int *slot) {
    int device = 0;
    ND_CUDA(cudaGetDevice(&device));
    std::lock_guard<std::mutex> lock(g_mu);
    Staging &s = g_staging[std::make_pair(device, stream)];
    const int k = s.next;
    s.next = (s.next + 1) % 4;
    if (s.done[k]) ND_CUDA(cudaEventSynchronize(s.done[k]));          // the copy that last used this buffer has left it
    else ND_CUDA(cudaEventCreateWithFlags(&s.done[k], cudaEventDisableTiming));
    if (bytes > s.cap[k]) {
        if (s.buf[k]) ND_CUDA(cudaFreeHost(s.buf[k]));
        s.buf[k] = nullptr; s.cap[k] = 0;
        const size_t want = bytes < (size_t(1) << 20) ? (size_t(1) << 20) : bytes + bytes / 2;
        ND_CUDA(cudaMallocHost(&s.buf[k], want));
        s.cap[k] = want;
    }
    *host = s.buf[k];
    *slot = k;
    return kOk;
}

Status staging_commit(cudaStream_t stream, int slot, void *dev, size_t bytes) {
    int device = 0;
    ND_CUDA(cudaGetDevice(&device));
    std::lock_guard<std::mutex> lock(g_mu);
    Staging &s = g_staging[std::make_pair(device, stream)];
    if (bytes) ND_CUDA(cudaMemcpyAsync(dev, s.buf[slot], bytes, cudaMemcpyHostToDevice, stream));
    ND_CUDA(cudaEventRecord(s.done[slot], stream));
    return kOk;
}

Status staged_upload(cudaStream_t stream, void *dev, const void *host, size_t bytes) {
    if (bytes == 0) return kOk;
    void *pinned = nullptr;
    int slot = 0;
    ND_TRY(staging_begin(stream, bytes, &pinned, &slot));
    memcpy(pinned, host, bytes);
    return staging_commit(stream, slot, dev, bytes);
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
    for (auto &kv : g_staging)
        for (int k = 0; k < 4; k++) {
            if (kv.second.buf[k]) cudaFreeHost(kv.second.buf[k]);
            if (kv.second.done[k]) cudaEventDestroy(kv.second.done[k]);
        }
    g_staging.clear();
}

}  // namespace nd4jb200
