// A plain C++ caller of the exported NativeOps members, the way nd4j's JavaCPP-generated JNI calls them in
// the reference's CUDA build: data, shapeInfo and dimension arguments are device pointers, extraPointers[0]
// carries the host copy of xShapeInfo and extraPointers[1] the stream (blas/cuda/NativeOps.cu:2107-2118).
// No CUDA header and no torch: memory and streams come from the same NativeOps object.
//   g++ -std=c++11 -I include tests/native/drop_in.cpp -L libnd4j_b200 -lnd4jb200 -Wl,-rpath,$PWD/libnd4j_b200
#include "NativeOps.h"
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <vector>

static NativeOps ops;
static Nd4jPointer stream;

template <class T> static T *to_device(const std::vector<T> &h) {
    T *d = static_cast<T *>(ops.mallocDevice((Nd4jLong) (h.size() * sizeof(T)), nullptr, 0));
    if (!d) { std::printf("mallocDevice failed\n"); std::exit(2); }
    ops.memcpyAsync(d, const_cast<T *>(h.data()), (Nd4jLong) (h.size() * sizeof(T)), 1, stream);
    return d;
}
template <class T> static std::vector<T> to_host(const T *d, size_t n) {
    std::vector<T> h(n);
    ops.memcpyAsync(h.data(), const_cast<T *>(d), (Nd4jLong) (n * sizeof(T)), 2, stream);
    ops.streamSynchronize(stream);
    return h;
}
static std::vector<Nd4jLong> info2(Nd4jLong r, Nd4jLong c) { return {2, r, c, c, 1, 0, 1, 99}; }
static void expect(bool ok, const char *what) {
    if (!ok) { std::printf("FAILED: %s\n", what); std::exit(1); }
}

int main() {
    ops.initializeDevicesAndFunctions();
    stream = ops.createStream();
    const Nd4jLong rows = 64, cols = 96;
    std::vector<float> x(rows * cols), y(rows * cols), b(cols);
    for (Nd4jLong i = 0; i < rows * cols; i++) { x[i] = (float) ((i * 37) % 101) / 50.0f - 1.0f; y[i] = (float) ((i * 11) % 13) - 6.0f; }
    for (Nd4jLong j = 0; j < cols; j++) b[j] = 0.25f * (float) j;
    std::vector<Nd4jLong> xi = info2(rows, cols), bi = info2(1, cols), zi = info2(rows, 1);
    std::vector<int> dim = {1};
    float *dx = to_device(x), *dy = to_device(y), *db = to_device(b);
    Nd4jLong *dxi = to_device(xi), *dbi = to_device(bi), *dzi = to_device(zi);
    int *ddim = to_device(dim);
    float *t1 = static_cast<float *>(ops.mallocDevice(rows * cols * 4, nullptr, 0));
    float *t2 = static_cast<float *>(ops.mallocDevice(rows * cols * 4, nullptr, 0));
    float *t3 = static_cast<float *>(ops.mallocDevice(rows * cols * 4, nullptr, 0));
    float *dsum = static_cast<float *>(ops.mallocDevice(rows * 4, nullptr, 0));
    float *dimax = static_cast<float *>(ops.mallocDevice(rows * 4, nullptr, 0));

    // extraPointers as the CUDA build expects them: [0] host xShapeInfo, [1] stream, [7]/[8] host y / z shapeInfo,
    // [9] host TAD shapeInfo (with [10]/[11] its device copy and the device TAD offsets, which this backend does
    // not need). With these slots filled no call below may read metadata back from the device.
    std::vector<Nd4jLong> tadInfo(8), tadOffsets(rows);
    ops.tadOnlyShapeInfo(xi.data(), dim.data(), 1, tadInfo.data(), tadOffsets.data());
    Nd4jPointer extras[16] = {nullptr};
    extras[0] = xi.data(); extras[1] = stream; extras[7] = bi.data(); extras[8] = xi.data(); extras[9] = tadInfo.data();
    const unsigned long long readsBefore = nd4jb200_metadata_reads();
    ops.execBroadcastFloat(extras, 0, dx, dxi, db, dbi, t1, dxi, ddim, 1);                    // x + b along dimension 1
    extras[7] = nullptr;
    ops.execTransformFloat(extras, 15, t1, dxi, t2, dxi, nullptr);                             // tanh
    extras[7] = xi.data();
    ops.execPairwiseTransformFloat(extras, 6, t2, dxi, dy, dxi, t3, dxi, nullptr);             // * y
    extras[8] = zi.data();
    ops.execReduceFloat(extras, 1, t3, dxi, nullptr, dsum, dzi, ddim, 1);                       // row sums
    ops.execIndexReduceFloat(extras, 0, t3, dxi, nullptr, dimax, dzi, ddim, 1);                 // row argmax
    const float total = ops.execReduceScalarFloat(extras, 1, t3, dxi, nullptr);                 // whole-array sum
    expect(nd4jb200_metadata_reads() == readsBefore, "no device reads of metadata when the host slots are filled");

    std::vector<float> g3 = to_host(t3, rows * cols), gsum = to_host(dsum, rows), gimax = to_host(dimax, rows);
    double all = 0;
    for (Nd4jLong r = 0; r < rows; r++) {
        double s = 0, mag = 0;
        Nd4jLong best = 0;
        for (Nd4jLong c = 0; c < cols; c++) {
            const float want = std::tanh(x[r * cols + c] + b[c]) * y[r * cols + c];
            expect(std::fabs(g3[r * cols + c] - want) <= 4e-7f * std::fabs(y[r * cols + c]) + 1e-12f, "chain element");
            s += g3[r * cols + c]; mag += std::fabs(g3[r * cols + c]);
            if (g3[r * cols + c] > g3[r * cols + best]) best = c;
        }
        expect(std::fabs(gsum[r] - s) <= 1e-5 * mag, "row sum");
        expect((Nd4jLong) gimax[r] == best, "row argmax (first index among equals)");
        all += s;
    }
    expect(std::fabs(total - all) <= 1e-4 * rows * cols, "whole-array sum");

    // no host copies in extraPointers, and the same device buffers reused with other contents: the dimension
    // buffer now says {0} and the result descriptor [1, cols]; nothing may be remembered from the calls above
    {
        std::vector<int> dim0 = {0};
        std::vector<Nd4jLong> ci = info2(1, cols);
        ops.memcpyAsync(ddim, dim0.data(), 4, 1, stream);
        ops.memcpyAsync(dzi, ci.data(), (Nd4jLong) (ci.size() * sizeof(Nd4jLong)), 1, stream);
        ops.streamSynchronize(stream);
        float *dcol = static_cast<float *>(ops.mallocDevice(cols * 4, nullptr, 0));
        Nd4jPointer bare[16] = {nullptr};
        bare[1] = stream;
        ops.execReduceFloat(bare, 1, t3, dxi, nullptr, dcol, dzi, ddim, 1);
        expect(nd4jb200_metadata_reads() > readsBefore, "without host slots the descriptors are read from the device");
        std::vector<float> gcol = to_host(dcol, cols);
        for (Nd4jLong c = 0; c < cols; c++) {
            double s = 0, mag = 0;
            for (Nd4jLong r = 0; r < rows; r++) { s += g3[r * cols + c]; mag += std::fabs(g3[r * cols + c]); }
            expect(std::fabs(gcol[c] - s) <= 1e-5 * mag + 1e-12, "column sum after the buffers were reused");
        }
        ops.freeDevice(dcol, nullptr);
        // restore what the rest of the program expects
        ops.memcpyAsync(ddim, dim.data(), 4, 1, stream);
        ops.memcpyAsync(dzi, zi.data(), (Nd4jLong) (zi.size() * sizeof(Nd4jLong)), 1, stream);
        ops.streamSynchronize(stream);
    }

    // the constant-memory staging area: a descriptor placed there is a valid device shapeInfo argument
    {
        char *space = static_cast<char *>(ops.getConstantSpace());
        expect(space != nullptr, "constant space address");
        ops.memcpyConstantAsync(256, xi.data(), (Nd4jLong) (xi.size() * sizeof(Nd4jLong)), 1, stream);
        Nd4jPointer bare[16] = {nullptr};
        bare[1] = stream;
        ops.execTransformFloat(bare, 0, t3, reinterpret_cast<Nd4jLong *>(space + 256), t2, reinterpret_cast<Nd4jLong *>(space + 256), nullptr);   // abs
        std::vector<float> ga = to_host(t2, rows * cols);
        for (Nd4jLong i = 0; i < rows * cols; i++) expect(ga[i] == std::fabs(g3[i]), "transform with shapeInfo in constant space");
        ops.checkP2P();
        expect(ops.getAvailableDevices() > 1 || ops.isP2PAvailable(), "one device counts as peer-capable");
        ops.enableP2P(true);
        ops.enableP2P(false);
    }

    // random: two identical states give identical draws, and the state advances
    Nd4jPointer rngExtras[2] = {nullptr, stream};
    Nd4jPointer s1 = ops.initRandom(rngExtras, 119, 100000, nullptr), s2 = ops.initRandom(rngExtras, 119, 100000, nullptr);
    std::vector<Nd4jLong> ui = info2(1, 4096);
    std::vector<float> range = {0.0f, 1.0f};
    float *du1 = static_cast<float *>(ops.mallocDevice(4096 * 4, nullptr, 0)), *du2 = static_cast<float *>(ops.mallocDevice(4096 * 4, nullptr, 0));
    float *drange = to_device(range);
    Nd4jPointer re[16] = {nullptr};
    re[0] = ui.data(); re[1] = stream; re[8] = ui.data();
    Nd4jLong *dui = to_device(ui);
    ops.execRandomFloat(re, 0, s1, du1, dui, drange);
    ops.execRandomFloat(re, 0, s2, du2, dui, drange);
    std::vector<float> u1 = to_host(du1, 4096), u2 = to_host(du2, 4096);
    for (int i = 0; i < 4096; i++) expect(u1[i] == u2[i] && u1[i] >= 0.0f && u1[i] <= 1.0f, "uniform draws");
    ops.execRandomFloat(re, 0, s1, du1, dui, drange);
    std::vector<float> u3 = to_host(du1, 4096);
    int same = 0;
    for (int i = 0; i < 4096; i++) same += u3[i] == u1[i];
    expect(same < 8, "second call continues the sequence");
    ops.destroyRandom(s1); ops.destroyRandom(s2);

    // an unknown op number is an exception, not a crash, and the context stays usable
    bool threw = false;
    try { ops.execTransformFloat(extras, 57, t1, dxi, t2, dxi, nullptr); } catch (const std::exception &) { threw = true; }
    expect(threw, "unknown opNum raises");
    extras[8] = xi.data();
    ops.execTransformFloat(extras, 0, t1, dxi, t2, dxi, nullptr);
    ops.streamSynchronize(stream);
    std::printf("drop-in ok: %lld x %lld chain, reductions, rng through the mangled NativeOps members\n", (long long) rows, (long long) cols);
    return 0;
}
