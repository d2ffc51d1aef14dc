// Multi-GPU layer: one process per GPU, one NCCL communicator per process, created from a unique id the caller
// distributes. It serves the one exchange step this path has -- combining per-GPU partials of a whole-array
// reduction -- and the across-GPU forms of average / accumulate. Everything is issued on the caller's stream;
// nothing here synchronises with the host unless the caller asks for the value.
//
// The reference combines per-device buffers by letting one kernel read peer memory
// (blas/cuda/NativeOps.cu:4884-4968 averageFloat / accumulateFloat, include/loops/special_kernels.h:711-821).
// Here no kernel reads another GPU's memory: partial accumulator states travel through ncclAllGather and are
// folded in shard order by every rank, parameter vectors through ncclAllReduce.
//
// NCCL is resolved at run time (dlopen of libnccl.so.2, which is the copy already loaded when the process also
// runs torch.distributed) so that single-GPU users need no NCCL at all.
#include "../../include/nd4j_b200.h"
#include "dispatch.h"
#include <cstring>
#include <dlfcn.h>
#include <nccl.h>
#include <mutex>
#include <sstream>

using namespace nd4jb200;

namespace {

struct NcclApi {
    void *handle = nullptr;
    ncclResult_t (*GetUniqueId)(ncclUniqueId *) = nullptr;
    ncclResult_t (*CommInitRank)(ncclComm_t *, int, ncclUniqueId, int) = nullptr;
    ncclResult_t (*CommDestroy)(ncclComm_t) = nullptr;
    ncclResult_t (*AllGather)(const void *, void *, size_t, ncclDataType_t, ncclComm_t, cudaStream_t) = nullptr;
    ncclResult_t (*AllReduce)(const void *, void *, size_t, ncclDataType_t, ncclRedOp_t, ncclComm_t, cudaStream_t) = nullptr;
    const char *(*GetErrorString)(ncclResult_t) = nullptr;
};

constexpr int kMaxShardsPerRank = 64;
constexpr int kStateSlot = 32;          // bytes reserved per accumulator state (the largest policy state)
// Every shard is cut into segments of this many elements, whatever the number of shards a rank holds: the bits
// of a shard's state then depend on the shard alone, and so does the combined value on the shard grid alone.
constexpr LL kShardSegment = 1 << 17;

struct Comm {
    bool ready = false;
    int rank = 0, world = 1, device = 0;
    ncclComm_t nccl = nullptr;
    char *send = nullptr;               // kMaxShardsPerRank states of this rank
    char *recv = nullptr;               // world * kMaxShardsPerRank states, rank-major
    void *hostSlot = nullptr;           // pinned, for callers that want the value on the host
};

std::mutex g_mu;
NcclApi g_api;
Comm g_comm;

Status load_nccl() {
    if (g_api.handle) return kOk;
    const char *names[] = {"libnccl.so.2", "libnccl.so"};
    void *h = nullptr;
    for (const char *n : names) { h = dlopen(n, RTLD_NOW | RTLD_GLOBAL); if (h) break; }
    if (!h) { set_error(std::string("NCCL is not available: ") + dlerror()); return kUnsupported; }
#define ND_SYM(field, name)                                                                       \
    g_api.field = reinterpret_cast<decltype(g_api.field)>(dlsym(h, name));                         \
    if (!g_api.field) { set_error(std::string("NCCL lacks ") + name); dlclose(h); return kUnsupported; }
    ND_SYM(GetUniqueId, "ncclGetUniqueId")
    ND_SYM(CommInitRank, "ncclCommInitRank")
    ND_SYM(CommDestroy, "ncclCommDestroy")
    ND_SYM(AllGather, "ncclAllGather")
    ND_SYM(AllReduce, "ncclAllReduce")
    ND_SYM(GetErrorString, "ncclGetErrorString")
#undef ND_SYM
    g_api.handle = h;
    return kOk;
}

Status nccl_fail(ncclResult_t r, const char *where) {
    std::ostringstream os;
    os << "NCCL error " << (int) r << " (" << (g_api.GetErrorString ? g_api.GetErrorString(r) : "?") << ") at " << where;
    set_error(os.str());
    return kCudaError;
}
#define ND_NCCL(call)                                                    \
    do {                                                                 \
        ncclResult_t r__ = (call);                                       \
        if (r__ != ncclSuccess) return nccl_fail(r__, #call);            \
    } while (0)

Status need_comm() {
    if (!g_comm.ready) return bad_arg("no communicator: call nd4jb200_comm_init first");
    int device = -1;
    ND_CUDA(cudaGetDevice(&device));
    if (device != g_comm.device) return bad_arg("the communicator belongs to another device than the current one");
    return kOk;
}

ncclDataType_t nccl_type(int dtype) { return dtype == kF64 ? ncclDouble : (dtype == kF16 ? ncclHalf : ncclFloat); }
size_t elem_bytes(int dtype) { return dtype == kF64 ? 8 : (dtype == kF16 ? 2 : 4); }

}  // namespace

#pragma GCC visibility push(default)
extern "C" {

int nd4jb200_comm_unique_id(void *id128) {
    if (!id128) return bad_arg("id128 is null");
    std::lock_guard<std::mutex> lock(g_mu);
    ND_TRY(load_nccl());
    static_assert(sizeof(ncclUniqueId) == 128, "ncclUniqueId is 128 bytes");
    ND_NCCL(g_api.GetUniqueId(static_cast<ncclUniqueId *>(id128)));
    return kOk;
}

int nd4jb200_comm_init(const void *id128, int rank, int world) {
    if (world < 1 || rank < 0 || rank >= world) return bad_arg("comm_init: rank must lie in [0, world)");
    std::lock_guard<std::mutex> lock(g_mu);
    if (g_comm.ready) return bad_arg("comm_init: a communicator already exists in this process");
    Comm c;
    c.rank = rank; c.world = world;
    ND_CUDA(cudaGetDevice(&c.device));
    if (world > 1) {
        if (!id128) return bad_arg("comm_init: id128 is null");
        ND_TRY(load_nccl());
        ncclUniqueId id;
        memcpy(&id, id128, sizeof(id));
        ND_NCCL(g_api.CommInitRank(&c.nccl, world, id, rank));
    }
    ND_CUDA(cudaMalloc(&c.send, (size_t) kMaxShardsPerRank * kStateSlot));
    ND_CUDA(cudaMalloc(&c.recv, (size_t) world * kMaxShardsPerRank * kStateSlot + 64));   // + a result slot
    ND_CUDA(cudaMallocHost(&c.hostSlot, 64));
    c.ready = true;
    g_comm = c;
    return kOk;
}

int nd4jb200_comm_destroy(void) {
    std::lock_guard<std::mutex> lock(g_mu);
    if (!g_comm.ready) return kOk;
    if (g_comm.nccl) g_api.CommDestroy(g_comm.nccl);
    cudaFree(g_comm.send); cudaFree(g_comm.recv); cudaFreeHost(g_comm.hostSlot);
    g_comm = Comm();
    return kOk;
}

int nd4jb200_comm_rank(void) { return g_comm.ready ? g_comm.rank : -1; }
int nd4jb200_comm_world(void) { return g_comm.ready ? g_comm.world : 0; }

int nd4jb200_exec_reduce_scalar_sharded(void *stream, int dtype, int opNum, const void *x, Nd4jLong localLength,
                                        const void *extraParams, int shardsPerRank, Nd4jLong totalLength, void *z,
                                        double *result) {
    ND_TRY(need_comm());
    if (dtype != kF32 && dtype != kF64 && dtype != kF16) return bad_arg("dtype must be 0 (float), 1 (double) or 2 (half)");
    if (!x) return bad_arg("x is null");
    if (!z && !result) return bad_arg("z and result are both null: nowhere to put the value");
    if (shardsPerRank < 1 || shardsPerRank > kMaxShardsPerRank) return bad_arg("shardsPerRank must lie in [1, 64]");
    if (localLength <= 0 || localLength % shardsPerRank != 0) return bad_arg("localLength must be a positive multiple of shardsPerRank");
    if (totalLength < localLength) return bad_arg("totalLength is smaller than this rank's shard");
    const int stateBytes = dtype == kF32 ? reduce_state_bytes_f32(opNum) : dtype == kF64 ? reduce_state_bytes_f64(opNum) : reduce_state_bytes_f16(opNum);
    if (stateBytes <= 0) return unknown_op("reduce", opNum);
    if (stateBytes > kStateSlot) { set_error("accumulator state exceeds the exchange slot"); return kTooLarge; }
    const cudaStream_t st = static_cast<cudaStream_t>(stream);

    // local step: this rank's array as shardsPerRank equal, contiguous shards, one accumulator state each
    ReduceCall c;
    const LL shardLen = localLength / shardsPerRank;
    c.x = x; c.extra = extraParams; c.z = g_comm.send; c.zState = g_comm.send;
    c.finishLen = shardLen;
    c.fixedSegment = kShardSegment;
    TadPlan &p = c.xPlan;
    p.numTads = shardsPerRank; p.tadLen = shardLen; p.whole = false; p.ndims = 0;
    LL len1[1] = {shardLen}, one[1] = {1}, cnt[1] = {shardsPerRank}, step[1] = {shardLen};
    ND_TRY(collapse_view(1, len1, one, &p.inner));
    ND_TRY(collapse_view(1, cnt, step, &p.outer));
    ND_TRY(dtype == kF32 ? reduce_f32(opNum, c, st) : dtype == kF64 ? reduce_f64(opNum, c, st) : reduce_f16(opNum, c, st));

    // exchange: every rank receives every rank's states, rank-major, i.e. in global shard order
    const void *states = g_comm.send;
    if (g_comm.world > 1) {
        ND_NCCL(g_api.AllGather(g_comm.send, g_comm.recv, (size_t) shardsPerRank * stateBytes, ncclChar, g_comm.nccl, st));
        states = g_comm.recv;
    }
    // combine: the same fixed-order fold on every rank
    MergeCall m;
    m.states = states; m.count = g_comm.world * shardsPerRank; m.finishLen = totalLength; m.extra = extraParams;
    void *out = z ? z : static_cast<void *>(g_comm.recv + (size_t) g_comm.world * kMaxShardsPerRank * kStateSlot);
    m.z = out;
    ND_TRY(dtype == kF32 ? reduce_merge_f32(opNum, m, st) : dtype == kF64 ? reduce_merge_f64(opNum, m, st) : reduce_merge_f16(opNum, m, st));
    if (result) {
        ND_CUDA(cudaMemcpyAsync(g_comm.hostSlot, out, elem_bytes(dtype), cudaMemcpyDeviceToHost, st));
        ND_CUDA(cudaStreamSynchronize(st));
        if (dtype == kF32) *result = *static_cast<float *>(g_comm.hostSlot);
        else if (dtype == kF64) *result = *static_cast<double *>(g_comm.hostSlot);
        else *result = __half2float(*static_cast<__half *>(g_comm.hostSlot));
    }
    return kOk;
}

int nd4jb200_accumulate_across(void *stream, int dtype, const void *x, void *z, Nd4jLong length) {
    ND_TRY(need_comm());
    if (!x || !z) return bad_arg("accumulate: null argument");
    if (length <= 0) return kOk;
    const cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (g_comm.world == 1) {
        if (x != z) ND_CUDA(cudaMemcpyAsync(z, x, (size_t) length * elem_bytes(dtype), cudaMemcpyDeviceToDevice, st));
        return kOk;
    }
    ND_NCCL(g_api.AllReduce(x, z, (size_t) length, nccl_type(dtype), ncclSum, g_comm.nccl, st));
    return kOk;
}

int nd4jb200_average_across(void *stream, int dtype, void *x, void *z, Nd4jLong length, int propagate) {
    ND_TRY(need_comm());
    if (!x) return bad_arg("average: x is null");
    if (length <= 0) return kOk;
    void *out = z ? z : x;
    const cudaStream_t st = static_cast<cudaStream_t>(stream);
    // every term is divided by the number of arrays before it is added, as the reference's loop does
    // (include/ops/impl/specials.cpp:392-400)
    ND_TRY((Status) nd4jb200_exec_scalar_strided(stream, dtype, 3, x, 1, out, 1, (double) g_comm.world, nullptr, length));
    if (g_comm.world > 1)
        ND_NCCL(g_api.AllReduce(out, out, (size_t) length, nccl_type(dtype), ncclSum, g_comm.nccl, st));
    if (propagate && out != x)
        ND_CUDA(cudaMemcpyAsync(x, out, (size_t) length * elem_bytes(dtype), cudaMemcpyDeviceToDevice, st));
    return kOk;
}

}  // extern "C"
#pragma GCC visibility pop
