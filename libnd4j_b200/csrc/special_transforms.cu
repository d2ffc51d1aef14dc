// The transforms of the reference's op table that are not elementwise functors but whole-array routines
// ("special" transforms, include/ops/special_ops.h): Col2Im (36), Im2col (37), Histogram (48), Reverse (70) and
// Pooling2D (71). They are reached through execTransform* like every other transform
// (include/loops/cpu/transform.cpp:30-60 hands ops with requiresSpecial to Op::execSpecial). The softmax family
// and IsMax (38-41) live in softmax.cuh and api.cu.
//
// All five are data movement plus a few operations per element, so each kernel is laid out for the memory system.
// In the three image kernels a CTA works on one or a few (batch, channel[, kernel row, kernel column]) planes and
// a thread produces a run of 16 bytes of consecutive plane positions (one 128-bit store where the plane is dense
// and aligned). The index arithmetic of a run is shared by its positions (a run that stays inside one image row
// tests and addresses the row once) and is 32-bit inside a plane; the loop over the kernel taps runs inside the
// thread, so the decomposition of a thread's index is paid once for all taps. The geometry that the reference keeps in
// extraParams (kernel, stride, padding, dilation as element-type values in device memory) is read by the kernels
// themselves, so no call waits for a device-to-host copy.
#include "../../include/nd4j_b200.h"
#include "device_utils.cuh"
#include "runtime.h"
#include "shape_host.h"

namespace nd4jb200 {

namespace {

// A plane is split over threadIdx.x (runs of V positions) and several planes share a CTA through threadIdx.y when
// a plane has fewer runs than the CTA has threads.
struct PlaneGrid {
    int tx, ty;          // blockDim
    unsigned gx, gy;     // gridDim: planes / ty, chunks of runs
};

// Runs per thread that the grid is sized for (a thread loops over every gridDim.y-th chunk of runs). 4 was
// measured: no gain for Im2col and Pooling2D, Col2Im 0.079 against 0.075 ms.
constexpr int kRunsPerThread = 1;

inline PlaneGrid plane_grid(LL planes, LL positions, int v) {
    const LL runs = ceil_div(ceil_div(positions, (LL) v), (LL) kRunsPerThread);      // per thread: kRunsPerThread of them
    PlaneGrid g;
    // the CTA width (a multiple of a warp) that leaves the fewest idle threads in a plane's last chunk; ties go to
    // the wider CTA
    g.tx = 32;
    LL idle = -1;
    for (int tx = 32; tx <= 256; tx += 32) {
        const LL waste = ceil_div(runs, (LL) tx) * tx - runs;
        if (idle < 0 || waste <= idle) { idle = waste; g.tx = tx; }
        if (tx >= runs) break;
    }
    g.ty = 256 / g.tx;
    // One short-lived thread per run and plane: fewer, longer-lived CTAs that walk the planes with the grid's stride
    // were slower (Im2col 0.098 against 0.084 ms), the hardware keeps more independent loads in flight this way.
    g.gx = (unsigned) ceil_div(planes, (LL) g.ty);
    const LL chunks = ceil_div(runs, (LL) g.tx);
    g.gy = (unsigned) (chunks < 65535 ? chunks : 65535);        // the kernels loop over what a larger plane leaves
    return g;
}

// extraParams are the same few words for every CTA: read through the read-only path so that they stay in L1
template <class T> ND_D T param(const T *extra, int i) { return __ldg(extra + i); }
template <> ND_D __half param(const __half *extra, int i) { return __ushort_as_half(__ldg(reinterpret_cast<const unsigned short *>(extra) + i)); }
template <class T> ND_D int param_int(const T *extra, int i) { return (int) Elem<T>::to_c(param(extra, i)); }

// What a kernel needs to place the positions of one result plane. Offsets inside a plane fit 32 bits (checked by
// the host).
struct PlaneOut {
    int sRow, sCol;      // strides of the plane's two axes
    int width;           // positions per row
    int positions;
    int dense;           // position p lies at offset p and runs may be stored as one 128-bit word
};

// Stores vals[0 .. V) at the positions p0 .. p0 + V of a plane, as far as they exist.
template <class T, int V>
ND_D void store_run(T *__restrict__ plane, const PlaneOut &o, int p0, const T (&vals)[V]) {
    if (p0 >= o.positions) return;
    if (o.dense && p0 + V <= o.positions) {
        Pack<T> pk;
#pragma unroll
        for (int j = 0; j < V; j++) pk.v[j] = vals[j];
        store_pack(plane + p0, pk);
        return;
    }
    int row = p0 / o.width, col = p0 - row * o.width;
#pragma unroll
    for (int j = 0; j < V; j++) {
        if (p0 + j < o.positions) plane[o.dense ? p0 + j : row * o.sRow + col * o.sCol] = vals[j];
        if (++col == o.width) { col = 0; row++; }
    }
}

// ---- Im2col (37): z[b, c, kr, kc, oh, ow] = x[b, c, oh * sH - pH + kr * dH, ow * sW - pW + kc * dW] or the padding
// value (special_ops.h:414-640). extraParams = {kH, kW, sH, sW, pH, pW, dH, dW, sameMode, padValue}; the padding
// value is the one the reference's CUDA build uses (its CPU build always pads with zero). A thread owns one run
// of positions of the (oh, ow) plane and writes it for every kernel tap, so an image element is fetched from
// DRAM once and then found in L1 by the taps that follow.
struct Im2colArgs {
    const void *x, *extra;
    void *z;
    unsigned planes;            // bS * iC
    int iC, iH, iW, kH, kW;
    LL xs[2], zs[4];            // strides of the outer axes
    int xRow, xCol;             // strides of x's image axes
    PlaneOut out;               // z's last two axes
};

constexpr int kMaxSpanTaps = 7;

// One run of V result positions for every tap of the kernel, through a span per kernel row. SW (the stride along
// the row, 1 or 2) is a template constant so that the span's registers can be addressed.
template <class T, int SW>
ND_D void im2col_span(const T *__restrict__ in, T *__restrict__ out, const Im2colArgs &a, int top, int left, int dH, T pad, int p0) {
    constexpr int V = Elem<T>::kVec, SPAN = (V - 1) * SW + kMaxSpanTaps;
    const int need = (V - 1) * SW + a.kW;
    for (int kr = 0; kr < a.kH; kr++) {
        const int ih = top + kr * dH;
        const bool rowInside = (unsigned) ih < (unsigned) a.iH;
        const T *row = in + ih * a.xRow + left;
        T span[SPAN];
#pragma unroll
        for (int t = 0; t < SPAN; t++) {
            const bool ok = rowInside && t < need && (unsigned) (left + t) < (unsigned) a.iW;
            span[t] = ok ? row[t] : pad;
        }
        T *dst = out + kr * a.zs[2] + p0;
#pragma unroll
        for (int kc = 0; kc < kMaxSpanTaps; kc++) {
            if (kc < a.kW) {
                Pack<T> pk;
#pragma unroll
                for (int j = 0; j < V; j++) pk.v[j] = span[kc + j * SW];
                store_pack(dst + kc * a.zs[3], pk);
            }
        }
    }
}

template <class T>
__global__ void __launch_bounds__(256, 4) k_im2col(const Im2colArgs a) {
    grid_dependency_sync();
    constexpr int V = Elem<T>::kVec;
    const T *extra = static_cast<const T *>(a.extra);
    const int sH = param_int(extra, 2), sW = param_int(extra, 3), pH = param_int(extra, 4), pW = param_int(extra, 5);
    const int dH = param_int(extra, 6), dW = param_int(extra, 7);
    const T pad = param(extra, 9);
    const unsigned plane = blockIdx.x * blockDim.y + threadIdx.y;
    if (plane >= a.planes) return;
    const unsigned c = plane % a.iC, b = plane / a.iC;
    const T *__restrict__ in = static_cast<const T *>(a.x) + b * a.xs[0] + c * a.xs[1];
    T *__restrict__ out = static_cast<T *>(a.z) + b * a.zs[0] + c * a.zs[1];
    // a thread takes every stride-th run of the plane, so that what it derives once (the geometry, the plane) serves
    // several runs
    auto run = [&](const int p0) {
        const int oh0 = p0 / a.out.width, ow0 = p0 - oh0 * a.out.width;
        const bool oneRow = ow0 + V <= a.out.width;           // the run stays in one row of the plane (it then also
                                                              // lies wholly inside the plane)
        // Interior: the run stays in one row and every tap of every position lies inside the image. Then nothing is
        // tested per element, and a tap is a few loads at a fixed step and one store.
        const int top = oh0 * sH - pH, left = ow0 * sW - pW;
        // Stride 1 or 2 and unit dilation along contiguous image rows (the usual convolutions): the kW taps of a
        // kernel row read overlapping pieces of one span of (V - 1) * sW + kW image elements, so the span is loaded
        // once per kernel row (elements outside the image become the padding value) and every tap's run is cut out
        // of it in registers. The choice is the same for all threads of a warp, so no warp runs two forms of the loop.
        if ((sW == 1 || sW == 2) && dW == 1 && a.xCol == 1 && a.kW <= kMaxSpanTaps && a.out.dense &&
            __all_sync(__activemask(), oneRow)) {
            if (sW == 1) im2col_span<T, 1>(in, out, a, top, left, dH, pad, p0);
            else im2col_span<T, 2>(in, out, a, top, left, dH, pad, p0);
            return;
        }
        const bool interior = oneRow && a.out.dense && top >= 0 && top + (a.kH - 1) * dH < a.iH && left >= 0 &&
                              left + (V - 1) * sW + (a.kW - 1) * dW < a.iW && dH >= 0 && dW >= 0 && sW >= 0;
        if (__all_sync(__activemask(), interior)) {            // taken by whole warps only: no warp runs both forms
            const int step = sW * a.xCol;
            for (int kr = 0; kr < a.kH; kr++) {
                const T *row = in + (top + kr * dH) * a.xRow + left * a.xCol;
                T *dst = out + kr * a.zs[2] + p0;
#pragma unroll 3
                for (int kc = 0; kc < a.kW; kc++) {
                    const T *src = row + kc * dW * a.xCol;
                    Pack<T> pk;
#pragma unroll
                    for (int j = 0; j < V; j++) pk.v[j] = src[j * step];
                    store_pack(dst + kc * a.zs[3], pk);
                }
            }
            return;
        }
        for (int kr = 0; kr < a.kH; kr++) {
            const int ih0 = kr * dH - pH + oh0 * sH;
#pragma unroll 3
            for (int kc = 0; kc < a.kW; kc++) {
                T vals[V];
                if (oneRow) {
                    const bool rowInside = (unsigned) ih0 < (unsigned) a.iH;
                    const T *row = in + ih0 * a.xRow;
                    int iw = kc * dW - pW + ow0 * sW;
#pragma unroll
                    for (int j = 0; j < V; j++, iw += sW)
                        vals[j] = rowInside && (unsigned) iw < (unsigned) a.iW ? row[iw * a.xCol] : pad;
                } else {
                    int oh = oh0, ow = ow0;
#pragma unroll
                    for (int j = 0; j < V; j++) {
                        const int ih = kr * dH - pH + oh * sH, iw = kc * dW - pW + ow * sW;
                        const bool inside = p0 + j < a.out.positions && (unsigned) ih < (unsigned) a.iH && (unsigned) iw < (unsigned) a.iW;
                        vals[j] = inside ? in[ih * a.xRow + iw * a.xCol] : pad;
                        if (++ow == a.out.width) { ow = 0; oh++; }
                    }
                }
                store_run<T, V>(out + kr * a.zs[2] + kc * a.zs[3], a.out, p0, vals);
            }
        }
    };
    for (int p0 = (blockIdx.y * blockDim.x + threadIdx.x) * V; p0 < a.out.positions; p0 += gridDim.y * blockDim.x * V) run(p0);
}

// ---- Col2Im (36): z[b, c, h, w] = sum of x[b, c, kr, kc, oh, ow] over the (kr, kc, oh, ow) that im2col reads (h, w)
// for (special_ops.h:891-1120). extraParams = {sH, sW, pH, pW, iH, iW, dH, dW}. The reference adds into the zeroed
// image with kr outermost and kc next, so for one image element the order of the additions is (kr, kc) ascending;
// the gather below adds in that order and is therefore identical bit for bit, without atomics. (The reference
// zeroes the first `length` elements of the result buffer whatever its strides; here every element of the result,
// dense or not, ends as its sum.)
struct Col2imArgs {
    const void *x, *extra;
    void *z;
    unsigned planes;            // bS * iC
    int iC, kH, kW, oH, oW;
    LL xs[4], zs[2];            // strides of the outer axes (x: batch, channel, kernel row, kernel column)
    int xRow, xCol;             // strides of x's last two axes
    PlaneOut out;               // z's last two axes (the image)
};

template <class T>
__global__ void __launch_bounds__(256, 4) k_col2im(const Col2imArgs a) {
    grid_dependency_sync();
    typedef typename Elem<T>::C C;
    constexpr int V = Elem<T>::kVec;
    const T *extra = static_cast<const T *>(a.extra);
    const int sH = param_int(extra, 0), sW = param_int(extra, 1), pH = param_int(extra, 2), pW = param_int(extra, 3);
    const int dH = param_int(extra, 6), dW = param_int(extra, 7);
    const unsigned plane = blockIdx.x * blockDim.y + threadIdx.y;
    if (plane >= a.planes) return;
    const unsigned c = plane % a.iC, b = plane / a.iC;
    const T *__restrict__ in = static_cast<const T *>(a.x) + b * a.xs[0] + c * a.xs[1];
    T *__restrict__ out = static_cast<T *>(a.z) + b * a.zs[0] + c * a.zs[1];
    // a thread takes every stride-th run of the plane, so that what it derives once (the geometry, the plane) serves
    // several runs
    auto run = [&](const int p0) {
        const int h0 = p0 / a.out.width, w0 = p0 - h0 * a.out.width;
        C sum[V];
#pragma unroll
        for (int j = 0; j < V; j++) sum[j] = 0;
        if (sH == 1 && sW == 1 && a.kH == 3 && a.kW == 3 && __all_sync(__activemask(), w0 + V <= a.out.width)) {
            // the 3 x 3 kernel with unit strides (chosen per warp): all nine taps' loads - none depends on another -
            // are issued before the first addition (the general loop below keeps one kernel row's loads in flight:
            // 0.070 against 0.061 ms); the additions keep the reference's order
            C v[3][3][V];
#pragma unroll
            for (int kr = 0; kr < 3; kr++) {
                const int oh = h0 + pH - kr * dH;
                const bool rowOk = (unsigned) oh < (unsigned) a.oH;
                const T *row = in + kr * a.xs[2] + oh * a.xRow;
#pragma unroll
                for (int kc = 0; kc < 3; kc++) {
                    const int ow0 = w0 + pW - kc * dW;
#pragma unroll
                    for (int j = 0; j < V; j++)
                        v[kr][kc][j] = rowOk && (unsigned) (ow0 + j) < (unsigned) a.oW
                                           ? Elem<T>::load(row + kc * a.xs[3] + (ow0 + j) * a.xCol) : (C) 0;
                }
            }
#pragma unroll
            for (int kr = 0; kr < 3; kr++) {
                const int oh = h0 + pH - kr * dH;
                if ((unsigned) oh >= (unsigned) a.oH) continue;
#pragma unroll
                for (int kc = 0; kc < 3; kc++) {
                    const int ow0 = w0 + pW - kc * dW;
#pragma unroll
                    for (int j = 0; j < V; j++)
                        if ((unsigned) (ow0 + j) < (unsigned) a.oW) sum[j] += v[kr][kc][j];
                }
            }
        } else if (w0 + V <= a.out.width && sH == 1 && sW == 1) {
            // unit strides and a run inside one image row: one row test per kernel row, no divisions
            for (int kr = 0; kr < a.kH; kr++) {
                const int oh = h0 + pH - kr * dH;
                if ((unsigned) oh >= (unsigned) a.oH) continue;
                const T *row = in + kr * a.xs[2] + oh * a.xRow;
#pragma unroll 3
                for (int kc = 0; kc < a.kW; kc++) {
                    const T *tap = row + kc * a.xs[3];
                    const int ow0 = w0 + pW - kc * dW;
#pragma unroll
                    for (int j = 0; j < V; j++)
                        if ((unsigned) (ow0 + j) < (unsigned) a.oW) sum[j] += Elem<T>::load(tap + (ow0 + j) * a.xCol);
                }
            }
        } else {
            for (int kr = 0; kr < a.kH; kr++) {
                for (int kc = 0; kc < a.kW; kc++) {
                    const T *tap = in + kr * a.xs[2] + kc * a.xs[3];
                    int h = h0, w = w0;
#pragma unroll
                    for (int j = 0; j < V; j++) {
                        const int hh = h + pH - kr * dH, ww = w + pW - kc * dW;
                        const int oh = hh / sH, ow = ww / sW;
                        const bool hit = p0 + j < a.out.positions && hh >= 0 && ww >= 0 && oh * sH == hh && ow * sW == ww &&
                                         oh < a.oH && ow < a.oW;
                        if (hit) sum[j] += Elem<T>::load(tap + oh * a.xRow + ow * a.xCol);
                        if (++w == a.out.width) { w = 0; h++; }
                    }
                }
            }
        }
        T vals[V];
#pragma unroll
        for (int j = 0; j < V; j++) vals[j] = Elem<T>::from_c(sum[j]);
        store_run<T, V>(out, a.out, p0, vals);
    };
    for (int p0 = (blockIdx.y * blockDim.x + threadIdx.x) * V; p0 < a.out.positions; p0 += gridDim.y * blockDim.x * V) run(p0);
}

// ---- Pooling2D (71): max (mode 0), average (1) or p-norm (2) over the dilated window of every output position
// (special_ops.h:31-330). extraParams = {kH, kW, sH, sW, pH, pW, dH, dW, -, mode, extra0}; extra0 is the divisor
// rule of the average (0: positions inside the image, 1: kH * kW) or the p of the p-norm. The reference clips the
// window to the image by whole dilation steps, which leaves exactly the taps that lie inside the image, visited
// row by row; the loop below visits the same taps in the same order. A c-order result is written densely behind
// the (batch, channel) base, an f-order one through its last two strides (special_ops.h:321-325).
struct PoolArgs {
    const void *x, *extra;
    void *z;
    unsigned planes;            // bS * iC
    int iC, iH, iW;
    LL xs[2], zs[2];
    int xRow, xCol;
    PlaneOut out;
};

ND_D int ceil_div_int(int a, int b) { return a > 0 ? (a + b - 1) / b : -((-a) / b); }   // ceil(a / b) for b > 0

// Pooling over a span: with unit dilation along contiguous image rows the windows of a run of V result positions
// lie in one span of (V - 1) * SW + kW image elements per image row. The span is loaded once per row - as 128-bit
// words when it starts on a 16-byte boundary and the words stay inside the row, else element by element, an
// element outside the image becoming a value that cannot win (max) or zero (sum) - and the windows are cut out of
// it in registers. SW (1 or 2) is a template constant so that the registers can be addressed.
constexpr int kMaxPoolTaps = 4;

template <class T, int SW, class C>
ND_D void pool_span_rows(const T *__restrict__ in, int xRow, int iH, int iW, int top, int left, int kH, int kW, int dH,
                         int mode, C neutral, C (&acc)[Elem<T>::kVec]) {
    constexpr int V = Elem<T>::kVec, SPAN = (V - 1) * SW + kMaxPoolTaps, WORDS = (SPAN + V - 1) / V;
    const int need = (V - 1) * SW + kW;
    const bool words = left >= 0 && left + (need + V - 1) / V * V <= iW && (reinterpret_cast<uintptr_t>(in + left) & 15) == 0 &&
                       (xRow * (int) sizeof(T)) % 16 == 0;
    const bool wide = __all_sync(__activemask(), words);
    if (V <= 4 && kH == 2 && wide && need <= 2 * V) {
        // the usual two-row window over an aligned span of at most two words: both rows' words are loaded before
        // either is used
        const int k0 = top, k1 = top + dH;
        const bool in0 = (unsigned) k0 < (unsigned) iH, in1 = (unsigned) k1 < (unsigned) iH;
        const T *r0 = in + k0 * xRow + left, *r1 = in + k1 * xRow + left;
        Pack<T> p[2][2];
        if (in0) { p[0][0] = load_pack(r0); if (need > V) p[0][1] = load_pack(r0 + V); }
        if (in1) { p[1][0] = load_pack(r1); if (need > V) p[1][1] = load_pack(r1 + V); }
#pragma unroll
        for (int i = 0; i < 2; i++) {
            if (!(i == 0 ? in0 : in1)) continue;
#pragma unroll
            for (int k = 0; k < kMaxPoolTaps; k++) {
                if (k < kW) {
#pragma unroll
                    for (int j = 0; j < V; j++) {
                        const int t = j * SW + k;
                        if (t < 2 * V) {
                            const C v = Elem<T>::to_c(p[i][t / V].v[t % V]);
                            if (mode == 0) { if (v > acc[j]) acc[j] = v; }
                            else acc[j] += v;
                        }
                    }
                }
            }
        }
        return;
    }
    for (int i = 0; i < kH; i++) {
        const int ky = top + i * dH;
        const bool rowInside = (unsigned) ky < (unsigned) iH;
        const T *row = in + ky * xRow + left;
        C span[WORDS * V];
        if (wide) {
#pragma unroll
            for (int w = 0; w < WORDS; w++) {
                Pack<T> pk;
                if (rowInside && w * V < need) pk = load_pack(row + w * V);
#pragma unroll
                for (int j = 0; j < V; j++) span[w * V + j] = rowInside && w * V < need ? Elem<T>::to_c(pk.v[j]) : neutral;
            }
        } else {
#pragma unroll
            for (int t = 0; t < SPAN; t++) {
                const bool ok = rowInside && t < need && (unsigned) (left + t) < (unsigned) iW;
                span[t] = ok ? Elem<T>::load(row + t) : neutral;
            }
        }
#pragma unroll
        for (int k = 0; k < kMaxPoolTaps; k++) {
            if (k < kW) {
#pragma unroll
                for (int j = 0; j < V; j++) {
                    const C v = span[j * SW + k];
                    if (mode == 0) { if (v > acc[j]) acc[j] = v; }
                    else acc[j] += v;
                }
            }
        }
    }
}

template <class T>
__global__ void __launch_bounds__(256, 4) k_pooling2d(const PoolArgs a) {
    grid_dependency_sync();
    typedef typename Elem<T>::C C;
    constexpr int V = Elem<T>::kVec;
    const T *extra = static_cast<const T *>(a.extra);
    const int kH = param_int(extra, 0), kW = param_int(extra, 1), sH = param_int(extra, 2), sW = param_int(extra, 3);
    const int pH = param_int(extra, 4), pW = param_int(extra, 5), dH = param_int(extra, 6), dW = param_int(extra, 7);
    const int mode = param_int(extra, 9);
    const C extra0 = Elem<T>::to_c(param(extra, 10));
    const C lowest = Elem<T>::to_c(Elem<T>::from_c((C) -1e37));        // -MAX_FLOAT in the element type
    // Taps beyond the image (plus its padding) cannot lie inside it, so the loops over a window stop there: the
    // window's size comes from device memory, and a wild value must not turn into a launch that never ends.
    const int tapRows = min(kH, a.iH + max(pH, 0) + 1), tapCols = min(kW, a.iW + max(pW, 0) + 1);
    const unsigned plane = blockIdx.x * blockDim.y + threadIdx.y;
    if (plane >= a.planes) return;
    const unsigned c = plane % a.iC, b = plane / a.iC;
    const T *__restrict__ in = static_cast<const T *>(a.x) + b * a.xs[0] + c * a.xs[1];
    T *__restrict__ out = static_cast<T *>(a.z) + b * a.zs[0] + c * a.zs[1];
    // a thread takes every stride-th run of the plane, so that what it derives once (the geometry, the plane) serves
    // several runs
    auto run = [&](const int p0) {
        const int yy0 = p0 / a.out.width, xx0 = p0 - yy0 * a.out.width;
        if (mode == 2) {
            // p-norm: one position at a time (the power's code, unrolled over a run's positions, would set the register
            // count of the whole kernel)
#pragma unroll 1
            for (int p = p0; p < p0 + V && p < a.out.positions; p++) {
                const int yy = p / a.out.width, xx = p - yy * a.out.width;
                C acc = 0;
                for (int i = 0; i < tapRows; i++) {
                    for (int k = 0; k < tapCols; k++) {
                        const int ky = yy * sH - pH + i * dH, kx = xx * sW - pW + k * dW;
                        if ((unsigned) ky < (unsigned) a.iH && (unsigned) kx < (unsigned) a.iW)
                            acc += pow(fabs(Elem<T>::load(in + ky * a.xRow + kx * a.xCol)), extra0);
                    }
                }
                Elem<T>::store(out + (a.out.dense ? p : yy * a.out.sRow + xx * a.out.sCol), pow(acc, (C) 1 / extra0));
            }
            return;
        }
        // Unit dilation along contiguous image rows, stride 1 or 2, at most four taps per row: the span form. The
        // choice is the same for all threads of a warp.
        if (dW == 1 && a.xCol == 1 && (sW == 1 || sW == 2) && kW <= kMaxPoolTaps && dH >= 1 &&
            __all_sync(__activemask(), xx0 + V <= a.out.width)) {
            const int top = yy0 * sH - pH, left = xx0 * sW - pW;
            C acc[V];
#pragma unroll
            for (int j = 0; j < V; j++) acc[j] = mode == 0 ? lowest : (C) 0;
            if (sW == 1) pool_span_rows<T, 1>(in, a.xRow, a.iH, a.iW, top, left, tapRows, kW, dH, mode, acc[0], acc);
            else pool_span_rows<T, 2>(in, a.xRow, a.iH, a.iW, top, left, tapRows, kW, dH, mode, acc[0], acc);
            T vals[V];
#pragma unroll
            for (int j = 0; j < V; j++) {
                C res = acc[j];
                if (mode == 1) {
                    int divisor = 0;
                    if ((int) extra0 == 0) {
                        // the window as the reference clips it (special_ops.h:236-262)
                        int hstart = top, wstart = left + j * sW;
                        int hend = hstart + kH + (kH - 1) * (dH - 1), wend = wstart + kW;
                        if (hstart < 0) hstart += ceil_div_int(-hstart, dH) * dH;
                        if (wstart < 0) wstart = 0;
                        if (hend > a.iH) hend -= ceil_div_int(hend - a.iH, dH) * dH;
                        if (wend > a.iW) wend = a.iW;
                        divisor = ceil_div_int(hend - hstart, dH) * (wend - wstart);
                    } else if ((int) extra0 == 1) divisor = kH * kW;
                    res = res / (C) divisor;
                }
                vals[j] = Elem<T>::from_c(res);
            }
            store_run<T, V>(out, a.out, p0, vals);
            return;
        }
        // top-left tap of every position's window; a position past the plane's end gets a window wholly above the image
        int hs[V], ws[V];
        C acc[V];
        {
            int yy = yy0, xx = xx0;
#pragma unroll
            for (int j = 0; j < V; j++) {
                hs[j] = p0 + j < a.out.positions ? yy * sH - pH : -(kH * dH + 1); ws[j] = xx * sW - pW;
                acc[j] = mode == 0 ? lowest : (C) 0;
                if (++xx == a.out.width) { xx = 0; yy++; }
            }
        }
        if (xx0 + V <= a.out.width) {
            // the run stays in one row of the result: its windows share their image rows
            for (int i = 0; i < tapRows; i++) {
                const int ky = hs[0] + i * dH;
                if ((unsigned) ky >= (unsigned) a.iH) continue;
                const T *row = in + ky * a.xRow;
#pragma unroll 3
                for (int k = 0; k < tapCols; k++) {
#pragma unroll
                    for (int j = 0; j < V; j++) {
                        const int kx = ws[j] + k * dW;
                        if ((unsigned) kx < (unsigned) a.iW) {
                            const C v = Elem<T>::load(row + kx * a.xCol);
                            if (mode == 0) { if (v > acc[j]) acc[j] = v; }
                            else acc[j] += v;
                        }
                    }
                }
            }
        } else {
            for (int i = 0; i < tapRows; i++) {
                for (int k = 0; k < tapCols; k++) {
#pragma unroll
                    for (int j = 0; j < V; j++) {
                        const int ky = hs[j] + i * dH, kx = ws[j] + k * dW;
                        if ((unsigned) ky < (unsigned) a.iH && (unsigned) kx < (unsigned) a.iW) {
                            const C v = Elem<T>::load(in + ky * a.xRow + kx * a.xCol);
                            if (mode == 0) { if (v > acc[j]) acc[j] = v; }
                            else acc[j] += v;
                        }
                    }
                }
            }
        }
        T vals[V];
#pragma unroll
        for (int j = 0; j < V; j++) {
            C res = acc[j];
            if (mode == 1) {
                int divisor = 0;
                if ((int) extra0 == 0) {
                    // the window as the reference clips it (special_ops.h:236-262)
                    int hstart = hs[j], wstart = ws[j];
                    int hend = hstart + kH + (kH - 1) * (dH - 1), wend = wstart + kW + (kW - 1) * (dW - 1);
                    if (hstart < 0) hstart += ceil_div_int(-hstart, dH) * dH;
                    if (wstart < 0) wstart += ceil_div_int(-wstart, dW) * dW;
                    if (hend > a.iH) hend -= ceil_div_int(hend - a.iH, dH) * dH;
                    if (wend > a.iW) wend -= ceil_div_int(wend - a.iW, dW) * dW;
                    divisor = ceil_div_int(hend - hstart, dH) * ceil_div_int(wend - wstart, dW);
                } else if ((int) extra0 == 1) divisor = kH * kW;
                res = res / (C) divisor;
            }
            vals[j] = Elem<T>::from_c(res);
        }
        store_run<T, V>(out, a.out, p0, vals);
    };
    for (int p0 = (blockIdx.y * blockDim.x + threadIdx.x) * V; p0 < a.out.positions; p0 += gridDim.y * blockDim.x * V) run(p0);
}

// ---- Histogram (48): z[i] += number of x whose bin is i, bin = (int) ((x - min) / binSize) clamped to
// [0, numBins), binSize = (max - min) / numBins (special_ops.h:713-880). extraParams = {numBins, min, max}. x is
// read as one dense run of its length, as the reference does. Counts are integers (shared-memory counters per
// CTA, several copies of a small table so that neighbouring warps do not meet in one counter, then one global
// atomic per CTA and bin) and enter z in a second launch, so the result does not depend on scheduling.
struct HistArgs {
    const void *x, *extra;
    void *z;
    unsigned *counts;           // zLength zeroed words
    LL n, zLength;
    int copies;                 // tables per CTA (a power of two, copies * zLength <= kHistShared), 0: global counters
    int vec;                    // x may be read as 128-bit words
};

constexpr int kHistShared = 8192;                            // counters kept in shared memory

template <class T> ND_D T hist_sub(T a, T b) { return a - b; }
template <class T> ND_D T hist_div(T a, T b) { return a / b; }
// half: every operation of the reference rounds to half
template <> ND_D __half hist_sub(__half a, __half b) { return __float2half_rn(__half2float(a) - __half2float(b)); }
template <> ND_D __half hist_div(__half a, __half b) { return __float2half_rn(__half2float(a) / __half2float(b)); }
template <class T> ND_D int hist_int(T v) { return (int) v; }
template <> ND_D int hist_int(__half v) { return (int) __half2float(v); }

template <class T>
__global__ void __launch_bounds__(256) k_histogram(const HistArgs a) {
    grid_dependency_sync();
    constexpr int V = Elem<T>::kVec;
    __shared__ unsigned bins[kHistShared];
    const T *extra = static_cast<const T *>(a.extra);
    const int numBins = hist_int(extra[0]);
    const T lo = extra[1], hi = extra[2];
    const T binSize = hist_div(hist_sub(hi, lo), Elem<T>::from_c((typename Elem<T>::C) numBins));
    const int tables = a.copies * (int) a.zLength;
    for (int i = threadIdx.x; i < tables; i += blockDim.x) bins[i] = 0;
    __syncthreads();
    unsigned *mine = a.copies ? bins + ((threadIdx.x >> 5) & (a.copies - 1)) * a.zLength : a.counts;
    // the kernel is bound by instruction issue, so the clamps are two min / max instead of branches and the test
    // against the result's length is only made where numBins exceeds it (then there is nowhere to count those)
    const int last = numBins - 1;
    const bool any = numBins >= 1, fits = any && numBins <= a.zLength;
    auto count = [&](T v) {
        const int idx = max(min(hist_int(hist_div(hist_sub(v, lo), binSize)), last), 0);
        if (fits || (any && idx < a.zLength)) atomicAdd(mine + idx, 1u);
    };
    const T *__restrict__ x = static_cast<const T *>(a.x);
    const LL tid = (LL) blockIdx.x * blockDim.x + threadIdx.x, threads = (LL) gridDim.x * blockDim.x;
    if (a.vec) {
        const LL packs = a.n / V;
        LL i = tid;
        for (; i + threads < packs; i += 2 * threads) {                       // two words in flight
            const Pack<T> p = load_pack(x + i * V), q = load_pack(x + (i + threads) * V);
#pragma unroll
            for (int j = 0; j < V; j++) count(p.v[j]);
#pragma unroll
            for (int j = 0; j < V; j++) count(q.v[j]);
        }
        if (i < packs) {
            const Pack<T> p = load_pack(x + i * V);
#pragma unroll
            for (int j = 0; j < V; j++) count(p.v[j]);
        }
        for (LL e = packs * V + tid; e < a.n; e += threads) count(x[e]);
    } else {
        for (LL e = tid; e < a.n; e += threads) count(x[e]);
    }
    if (a.copies) {
        __syncthreads();
        for (int i = threadIdx.x; i < (int) a.zLength; i += blockDim.x) {
            unsigned s = 0;
            for (int c = 0; c < a.copies; c++) s += bins[c * a.zLength + i];
            if (s) atomicAdd(a.counts + i, s);
        }
    }
}

template <class T>
__global__ void __launch_bounds__(256) k_histogram_add(const HistArgs a) {
    grid_dependency_sync();
    T *z = static_cast<T *>(a.z);
    for (LL i = (LL) blockIdx.x * blockDim.x + threadIdx.x; i < a.zLength; i += (LL) gridDim.x * blockDim.x)
        Elem<T>::store(z + i, Elem<T>::load(z + i) + (typename Elem<T>::C) a.counts[i]);
}

// ---- Reverse (70): z at linear position n - 1 - e of its own order = x at linear position e of its own order
// (special_ops.h:1178-1415). In place, arrays with an elementWiseStride swap the two halves; in place without one
// the reference copies the first half over the second and leaves the first as it is, which is kept.
struct ReverseArgs {
    const void *x;
    void *z;
    LL n, count;                // elements; loop bound (n, or n / 2 in place)
    View vx, vz;
    int swap;
};

// Any layout: four elements per thread and trip, all loads ahead of the stores.
template <class T>
__global__ void __launch_bounds__(256) k_reverse(const ReverseArgs a) {
    grid_dependency_sync();
    const T *x = static_cast<const T *>(a.x);
    T *z = static_cast<T *>(a.z);
    const LL threads = (LL) gridDim.x * blockDim.x;
    for (LL e0 = (LL) blockIdx.x * blockDim.x + threadIdx.x; e0 < a.count; e0 += 4 * threads) {
        LL from[4], to[4];
        T low[4], high[4];
#pragma unroll
        for (int u = 0; u < 4; u++) {
            const LL e = e0 + u * threads;
            const bool live = e < a.count;
            from[u] = live ? view_offset(a.vx, e) : -1;
            to[u] = live ? view_offset(a.vz, a.n - 1 - e) : -1;
            if (live) { low[u] = x[from[u]]; if (a.swap) high[u] = z[to[u]]; }
        }
#pragma unroll
        for (int u = 0; u < 4; u++) {
            if (from[u] < 0) continue;
            z[to[u]] = low[u];
            if (a.swap) z[from[u]] = high[u];
        }
    }
}

// Both arrays dense, their ends 16-byte aligned and the length a multiple of the word: 128-bit words, the elements
// of a word turned round in registers. count = words to read (all of them, or half in place, where a word and its
// mirror are exchanged; with an odd number of words the middle one is its own mirror).
template <class T>
__global__ void __launch_bounds__(256) k_reverse_words(const ReverseArgs a) {
    grid_dependency_sync();
    constexpr int V = Elem<T>::kVec;
    const T *x = static_cast<const T *>(a.x);
    T *z = static_cast<T *>(a.z);
    const LL words = a.n / V, threads = (LL) gridDim.x * blockDim.x;
    auto turned = [](const Pack<T> &p) {
        Pack<T> r;
#pragma unroll
        for (int j = 0; j < V; j++) r.v[j] = p.v[V - 1 - j];
        return r;
    };
    for (LL i0 = (LL) blockIdx.x * blockDim.x + threadIdx.x; i0 < a.count; i0 += 2 * threads) {
        const LL i1 = i0 + threads;
        const bool two = i1 < a.count;
        const Pack<T> p0 = load_pack_rw(x + i0 * V), p1 = load_pack_rw(x + (two ? i1 : i0) * V);
        Pack<T> m0, m1;
        if (a.swap) { m0 = load_pack_rw(z + (words - 1 - i0) * V); m1 = load_pack_rw(z + (words - 1 - (two ? i1 : i0)) * V); }
        store_pack(z + (words - 1 - i0) * V, turned(p0));
        if (a.swap) store_pack(z + i0 * V, turned(m0));
        if (two) {
            store_pack(z + (words - 1 - i1) * V, turned(p1));
            if (a.swap) store_pack(z + i1 * V, turned(m1));
        }
    }
}

// The last two axes of an array as a plane: dense when position p lies at offset p; 128-bit stores need every
// plane to start on a 16-byte boundary as well (the buffer and all outer strides).
template <class T>
PlaneOut plane_out(const void *base, LL rows, LL cols, LL sRow, LL sCol, const LL *outer, int nOuter) {
    PlaneOut o;
    o.sRow = (int) sRow; o.sCol = (int) sCol; o.width = (int) cols; o.positions = (int) (rows * cols);
    bool dense = sCol == 1 && (sRow == cols || rows == 1) && aligned16(base);
    for (int i = 0; i < nOuter; i++) dense = dense && outer[i] % Elem<T>::kVec == 0;
    o.dense = dense;
    return o;
}

// Offsets inside a plane are computed in 32 bits.
inline bool plane_fits(LL rows, LL cols, LL sRow, LL sCol) {
    auto mag = [](LL v) { return v < 0 ? -v : v; };
    return rows * cols < (1LL << 30) && rows * mag(sRow) + cols * mag(sCol) < (1LL << 30);
}

template <class T>
Status special_transform_typed(int opNum, const void *x, const ShapeDesc &xd, void *z, const ShapeDesc &zd, const void *extra,
                               cudaStream_t st) {
    auto strides = [](const ShapeDesc &d, LL *out) { for (int i = 0; i < d.rank; i++) out[i] = d.stride[i]; };
    auto fits_int = [](LL v) { return v >= 0 && v <= 0x7fffffffLL; };
    // shape::strideDescendingCAscendingF for a c-order array of rank > 2 (include/helpers/shape.h:3729-3751)
    auto descending_c = [](const ShapeDesc &d) {
        if (d.order != 'c') return false;
        for (int i = 1; i < d.rank; i++) if (d.stride[i - 1] <= d.stride[i]) return false;
        return true;
    };
    // When both arrays are c-order with descending strides the reference walks the six-axis array as one dense run
    // per batch entry (a unit step for Im2col's result, the last stride for Col2Im's input) instead of by its
    // strides (special_ops.h:565-600, 1010-1045); for a dense array the two are the same, for a view they are not,
    // and the reference's choice is kept.
    auto dense_behind_batch = [](const ShapeDesc &d, LL unit, LL *out) {
        out[5] = unit;
        for (int i = 4; i >= 1; i--) out[i] = out[i + 1] * d.shape[i + 1];
    };
    if (opNum != 70 && !extra) return bad_arg("transform: this op reads its geometry from extraParams");
    switch (opNum) {
        case 37: {
            if (xd.rank != 4 || zd.rank != 6) return bad_arg("Im2col: x must have rank 4 [b, c, h, w] and z rank 6 [b, c, kH, kW, oH, oW]");
            if (xd.shape[0] != zd.shape[0] || xd.shape[1] != zd.shape[1]) return bad_arg("Im2col: x and z differ in batch size or channels");
            if (zd.length == 0) return kOk;
            LL zs[6];
            strides(zd, zs);
            if (descending_c(xd) && descending_c(zd)) dense_behind_batch(zd, 1, zs);
            if (!fits_int(xd.shape[0] * xd.shape[1] * zd.shape[2] * zd.shape[3]) ||
                !plane_fits(xd.shape[2], xd.shape[3], xd.stride[2], xd.stride[3]) || !plane_fits(zd.shape[4], zd.shape[5], zs[4], zs[5])) {
                set_error("Im2col: 2^31 or more planes, or a plane that spans 2^30 or more elements"); return kTooLarge;
            }
            Im2colArgs a;
            a.x = x; a.z = z; a.extra = extra;
            a.iC = (int) xd.shape[1]; a.iH = (int) xd.shape[2]; a.iW = (int) xd.shape[3];
            a.kH = (int) zd.shape[2]; a.kW = (int) zd.shape[3];
            a.planes = (unsigned) (xd.shape[0] * xd.shape[1]);
            a.xs[0] = xd.stride[0]; a.xs[1] = xd.stride[1]; a.xRow = (int) xd.stride[2]; a.xCol = (int) xd.stride[3];
            for (int i = 0; i < 4; i++) a.zs[i] = zs[i];
            a.out = plane_out<T>(z, zd.shape[4], zd.shape[5], zs[4], zs[5], zs, 4);
            const PlaneGrid g = plane_grid(a.planes, (LL) a.out.positions, Elem<T>::kVec);
            launch_kernel(k_im2col<T>, dim3(g.gx, g.gy), dim3(g.tx, g.ty), st, a);
            break;
        }
        case 36: {
            if (xd.rank != 6 || zd.rank != 4) return bad_arg("Col2Im: x must have rank 6 [b, c, kH, kW, oH, oW] and z rank 4 [b, c, h, w]");
            if (xd.shape[0] != zd.shape[0] || xd.shape[1] != zd.shape[1]) return bad_arg("Col2Im: x and z differ in batch size or channels");
            if (zd.length == 0) return kOk;
            LL xs[6];
            strides(xd, xs);
            if (descending_c(xd) && descending_c(zd)) dense_behind_batch(xd, xd.stride[5], xs);
            if (!fits_int(zd.shape[0] * zd.shape[1]) || !plane_fits(zd.shape[2], zd.shape[3], zd.stride[2], zd.stride[3]) ||
                !plane_fits(xd.shape[4], xd.shape[5], xs[4], xs[5])) {
                set_error("Col2Im: 2^31 or more planes, or a plane that spans 2^30 or more elements"); return kTooLarge;
            }
            Col2imArgs a;
            a.x = x; a.z = z; a.extra = extra;
            a.iC = (int) zd.shape[1];
            a.kH = (int) xd.shape[2]; a.kW = (int) xd.shape[3]; a.oH = (int) xd.shape[4]; a.oW = (int) xd.shape[5];
            a.planes = (unsigned) (zd.shape[0] * zd.shape[1]);
            for (int i = 0; i < 4; i++) a.xs[i] = xs[i];
            a.xRow = (int) xs[4]; a.xCol = (int) xs[5];
            a.zs[0] = zd.stride[0]; a.zs[1] = zd.stride[1];
            a.out = plane_out<T>(z, zd.shape[2], zd.shape[3], zd.stride[2], zd.stride[3], zd.stride, 2);
            const PlaneGrid g = plane_grid(a.planes, (LL) a.out.positions, Elem<T>::kVec);
            launch_kernel(k_col2im<T>, dim3(g.gx, g.gy), dim3(g.tx, g.ty), st, a);
            break;
        }
        case 71: {
            if (xd.rank != 4 || zd.rank != 4) return bad_arg("Pooling2D: x and z must have rank 4 [b, c, h, w]");
            if (xd.shape[0] != zd.shape[0] || xd.shape[1] != zd.shape[1]) return bad_arg("Pooling2D: x and z differ in batch size or channels");
            if (zd.length == 0) return kOk;
            LL zRow = zd.stride[2], zCol = zd.stride[3];
            if (zd.order != 'f') { zCol = 1; zRow = zd.shape[3]; }          // written densely behind the plane's base
            if (!fits_int(xd.shape[0] * xd.shape[1]) || !plane_fits(xd.shape[2], xd.shape[3], xd.stride[2], xd.stride[3]) ||
                !plane_fits(zd.shape[2], zd.shape[3], zRow, zCol)) {
                set_error("Pooling2D: 2^31 or more planes, or a plane that spans 2^30 or more elements"); return kTooLarge;
            }
            PoolArgs a;
            a.x = x; a.z = z; a.extra = extra;
            a.iC = (int) xd.shape[1]; a.iH = (int) xd.shape[2]; a.iW = (int) xd.shape[3];
            a.planes = (unsigned) (xd.shape[0] * xd.shape[1]);
            a.xs[0] = xd.stride[0]; a.xs[1] = xd.stride[1]; a.xRow = (int) xd.stride[2]; a.xCol = (int) xd.stride[3];
            a.zs[0] = zd.stride[0]; a.zs[1] = zd.stride[1];
            a.out = plane_out<T>(z, zd.shape[2], zd.shape[3], zRow, zCol, zd.stride, 2);
            const PlaneGrid g = plane_grid(a.planes, (LL) a.out.positions, Elem<T>::kVec);
            launch_kernel(k_pooling2d<T>, dim3(g.gx, g.gy), dim3(g.tx, g.ty), st, a);
            break;
        }
        case 48: {
            if (xd.ews != 1) return unsupported("Histogram: x must be one dense run (the reference reads the buffer linearly)");
            if (zd.length == 0 || xd.length == 0) return kOk;
            HistArgs a;
            a.x = x; a.z = z; a.extra = extra; a.n = xd.length; a.zLength = zd.length;
            void *ws = nullptr;
            ND_TRY(workspace(st, kWorkspaceScratch + (size_t) zd.length * sizeof(unsigned), &ws, nullptr));
            a.counts = reinterpret_cast<unsigned *>(static_cast<char *>(ws) + kWorkspaceScratch);
            ND_CUDA(cudaMemsetAsync(a.counts, 0, (size_t) zd.length * sizeof(unsigned), st));
            a.copies = 0;
            if (zd.length <= kHistShared) { a.copies = 1; while (a.copies < 8 && a.copies * 2 * zd.length <= kHistShared) a.copies *= 2; }
            a.vec = aligned16(x);
            LL blocks = ceil_div(xd.length, (LL) 256 * 16);
            if (blocks > (LL) kNumSMs * 8) blocks = (LL) kNumSMs * 8;
            launch_kernel(k_histogram<T>, dim3((unsigned) blocks), dim3(256), st, a);
            LL addBlocks = ceil_div(zd.length, (LL) 256);
            if (addBlocks > (LL) kNumSMs * 8) addBlocks = (LL) kNumSMs * 8;
            launch_kernel(k_histogram_add<T>, dim3((unsigned) addBlocks), dim3(256), st, a);
            break;
        }
        case 70: {
            if (xd.length != zd.length) return bad_arg("Reverse: x and z hold different numbers of elements");
            if (xd.length == 0) return kOk;
            ReverseArgs a;
            a.x = x; a.z = z; a.n = xd.length;
            // position e of an array in its own order: e * ews, or its coordinates in that order
            auto own_order = [](const ShapeDesc &d, View *v) -> Status {
                if (d.ews >= 1 || d.order == 'c') return linear_view(d, v);
                LL shp[kMaxRank], str[kMaxRank];
                for (int i = 0; i < d.rank; i++) { shp[i] = d.shape[d.rank - 1 - i]; str[i] = d.stride[d.rank - 1 - i]; }
                return collapse_view(d.rank, shp, str, v);
            };
            ND_TRY(own_order(xd, &a.vx));
            if (x == z) {
                a.vz = a.vx;
                a.count = xd.length / 2;
                a.swap = xd.ews >= 1;
            } else {
                ND_TRY(own_order(zd, &a.vz));
                a.count = xd.length;
                a.swap = 0;
            }
            if (a.count == 0) return kOk;
            constexpr int V = Elem<T>::kVec;
            if (xd.ews == 1 && zd.ews == 1 && (x == z || xd.order == zd.order || xd.rank <= 1) && xd.length % V == 0 &&
                aligned16(x) && aligned16(z)) {
                const LL words = xd.length / V;
                a.swap = x == z;
                a.count = a.swap ? (words + 1) / 2 : words;
                LL blocks = ceil_div(a.count, (LL) 256 * 2);
                if (blocks > (LL) kNumSMs * 16) blocks = (LL) kNumSMs * 16;
                launch_kernel(k_reverse_words<T>, dim3((unsigned) blocks), dim3(256), st, a);
                break;
            }
            LL blocks = ceil_div(a.count, (LL) 256 * 4);
            if (blocks > (LL) kNumSMs * 16) blocks = (LL) kNumSMs * 16;
            launch_kernel(k_reverse<T>, dim3((unsigned) blocks), dim3(256), st, a);
            break;
        }
        default: return unknown_op("transform", opNum);
    }
    ND_CUDA(cudaGetLastError());
    return kOk;
}

}  // namespace

Status run_special_transform(int dtype, int opNum, const void *x, const ShapeDesc &xd, void *z, const ShapeDesc &zd,
                             const void *extra, cudaStream_t st) {
    if (dtype == kF32) return special_transform_typed<float>(opNum, x, xd, z, zd, extra, st);
    if (dtype == kF64) return special_transform_typed<double>(opNum, x, xd, z, zd, extra, st);
    return special_transform_typed<__half>(opNum, x, xd, z, zd, extra, st);
}

}  // namespace nd4jb200
