// The transforms of the reference's op table that are not elementwise functors but whole-array routines
// ("special" transforms, include/ops/special_ops.h): Col2Im (36), Im2col (37), Histogram (48), Reverse (70) and
// Pooling2D (71). They are reached through execTransform* like every other transform
// (include/loops/cpu/transform.cpp:30-60 hands ops with requiresSpecial to Op::execSpecial). The softmax family
// and IsMax (38-41) live in softmax.cuh and api.cu.
//
// All five are pure data movement plus a few operations per element, so each kernel is laid out for coalesced
// access along the innermost image axis: a CTA works on one or a few (batch, channel[, kernel row, kernel column])
// planes, its threads walk the plane's positions with a stride of the CTA width, and a position's (row, column)
// pair is advanced incrementally instead of being recomputed by division. The geometry that the reference keeps
// in extraParams (kernel, stride, padding, dilation as element-type values in device memory) is read by the
// kernels themselves, so no call waits for a device-to-host copy.
#include "../../include/nd4j_b200.h"
#include "device_utils.cuh"
#include "runtime.h"
#include "shape_host.h"

namespace nd4jb200 {

namespace {

// A plane is split over threadIdx.x (positions) and several planes share a CTA through threadIdx.y when a plane
// has fewer positions than the CTA has threads.
struct PlaneGrid {
    int tx, ty;          // blockDim
    unsigned gx, gy;     // gridDim: planes / ty, position chunks
    int iters;           // positions per thread
};

inline PlaneGrid plane_grid(LL planes, LL positions) {
    PlaneGrid g;
    g.tx = 32;
    while (g.tx < 256 && g.tx < positions) g.tx *= 2;
    g.ty = 256 / g.tx;
    g.iters = positions >= 256 * 8 ? 8 : (int) ceil_div(positions, (LL) g.tx);
    if (g.iters > 8) g.iters = 8;
    g.gx = (unsigned) ceil_div(planes, (LL) g.ty);
    g.gy = (unsigned) ceil_div(positions, (LL) g.tx * g.iters);
    return g;
}

template <class T> ND_D int param_int(const T *extra, int i) { return (int) Elem<T>::load(extra + i); }

// ---- Im2col (37): z[b, c, kr, kc, oh, ow] = x[b, c, oh * sH - pH + kr * dH, ow * sW - pW + kc * dW] or the padding
// value (special_ops.h:414-640). extraParams = {kH, kW, sH, sW, pH, pW, dH, dW, sameMode, padValue}.
struct Im2colArgs {
    const void *x, *extra;
    void *z;
    LL planes;                  // bS * iC * kH * kW
    int iC, iH, iW, kH, kW, oH, oW;
    LL xs[4], zs[6];
    int iters;
};

template <class T>
__global__ void __launch_bounds__(256) k_im2col(const Im2colArgs a) {
    grid_dependency_sync();
    const T *extra = static_cast<const T *>(a.extra);
    const int sH = param_int(extra, 2), sW = param_int(extra, 3), pH = param_int(extra, 4), pW = param_int(extra, 5);
    const int dH = param_int(extra, 6), dW = param_int(extra, 7);
    const T pad = extra[9];
    const LL plane = (LL) blockIdx.x * blockDim.y + threadIdx.y;
    if (plane >= a.planes) return;
    const int kc = (int) (plane % a.kW);
    LL t = plane / a.kW;
    const int kr = (int) (t % a.kH);
    t /= a.kH;
    const int c = (int) (t % a.iC);
    const LL b = t / a.iC;
    const T *in = static_cast<const T *>(a.x) + b * a.xs[0] + c * a.xs[1];
    T *out = static_cast<T *>(a.z) + b * a.zs[0] + c * a.zs[1] + kr * a.zs[2] + kc * a.zs[3];
    const int row0 = kr * dH - pH, col0 = kc * dW - pW;
    const int positions = a.oH * a.oW;
    const int stepRows = blockDim.x / a.oW, stepCols = blockDim.x % a.oW;
    int p = blockIdx.y * (blockDim.x * a.iters) + threadIdx.x;
    int oh = p / a.oW, ow = p - oh * a.oW;
    for (int it = 0; it < a.iters && p < positions; it++) {
        const int ih = row0 + oh * sH, iw = col0 + ow * sW;
        const bool inside = (unsigned) ih < (unsigned) a.iH && (unsigned) iw < (unsigned) a.iW;
        out[oh * a.zs[4] + ow * a.zs[5]] = inside ? in[ih * a.xs[2] + iw * a.xs[3]] : pad;
        p += blockDim.x; oh += stepRows; ow += stepCols;
        if (ow >= a.oW) { ow -= a.oW; oh++; }
    }
}

// ---- Col2Im (36): z[b, c, h, w] = sum of x[b, c, kr, kc, oh, ow] over the (kr, kc, oh, ow) that im2col reads (h, w)
// for (special_ops.h:891-1120). extraParams = {sH, sW, pH, pW, iH, iW, dH, dW}. The reference adds into the zeroed
// image with kr outermost and kc next, so for one image element the order of the additions is (kr, kc) ascending;
// the gather below adds in that order and is therefore identical bit for bit, without atomics.
struct Col2imArgs {
    const void *x, *extra;
    void *z;
    LL planes;                  // bS * iC
    int iC, iH, iW, kH, kW, oH, oW;
    LL xs[6], zs[4];
    int iters;
};

template <class T>
__global__ void __launch_bounds__(256) k_col2im(const Col2imArgs a) {
    grid_dependency_sync();
    typedef typename Elem<T>::C C;
    const T *extra = static_cast<const T *>(a.extra);
    const int sH = param_int(extra, 0), sW = param_int(extra, 1), pH = param_int(extra, 2), pW = param_int(extra, 3);
    const int dH = param_int(extra, 6), dW = param_int(extra, 7);
    const LL plane = (LL) blockIdx.x * blockDim.y + threadIdx.y;
    if (plane >= a.planes) return;
    const int c = (int) (plane % a.iC);
    const LL b = plane / a.iC;
    const T *in = static_cast<const T *>(a.x) + b * a.xs[0] + c * a.xs[1];
    T *out = static_cast<T *>(a.z) + b * a.zs[0] + c * a.zs[1];
    const int positions = a.iH * a.iW;
    const int stepRows = blockDim.x / a.iW, stepCols = blockDim.x % a.iW;
    int p = blockIdx.y * (blockDim.x * a.iters) + threadIdx.x;
    int h = p / a.iW, w = p - h * a.iW;
    for (int it = 0; it < a.iters && p < positions; it++) {
        C sum = 0;
        for (int kr = 0; kr < a.kH; kr++) {
            const int hh = h + pH - kr * dH;
            if (hh < 0) break;                            // decreases with kr
            const int oh = hh / sH;
            if (oh * sH != hh || oh >= a.oH) continue;
            const T *row = in + kr * a.xs[2] + oh * a.xs[4];
            for (int kc = 0; kc < a.kW; kc++) {
                const int ww = w + pW - kc * dW;
                if (ww < 0) break;
                const int ow = ww / sW;
                if (ow * sW != ww || ow >= a.oW) continue;
                sum += Elem<T>::load(row + kc * a.xs[3] + ow * a.xs[5]);
            }
        }
        Elem<T>::store(out + h * a.zs[2] + w * a.zs[3], sum);
        p += blockDim.x; h += stepRows; w += stepCols;
        if (w >= a.iW) { w -= a.iW; h++; }
    }
}

// ---- Pooling2D (71): max (mode 0), average (1) or p-norm (2) over the dilated window of every output position
// (special_ops.h:31-330). extraParams = {kH, kW, sH, sW, pH, pW, dH, dW, -, mode, extra0}; extra0 is the divisor
// rule of the average (0: positions inside the image, 1: kH * kW) or the p of the p-norm. The window is clipped to
// the image by whole dilation steps, as the reference does. A c-order result is written densely behind the
// (batch, channel) base, an f-order one through its last two strides (special_ops.h:321-325).
struct PoolArgs {
    const void *x, *extra;
    void *z;
    LL planes;                  // bS * iC
    int iC, iH, iW, oH, oW;
    LL xs[4], zs[4];
    int fOrder;
    int iters;
};

ND_D int ceil_div_pos(int a, int b) { return a > 0 ? (a + b - 1) / b : -((-a) / b); }   // ceil(a / b) for b > 0

template <class T>
__global__ void __launch_bounds__(256) k_pooling2d(const PoolArgs a) {
    grid_dependency_sync();
    typedef typename Elem<T>::C C;
    const T *extra = static_cast<const T *>(a.extra);
    const int kH = param_int(extra, 0), kW = param_int(extra, 1), sH = param_int(extra, 2), sW = param_int(extra, 3);
    const int pH = param_int(extra, 4), pW = param_int(extra, 5), dH = param_int(extra, 6), dW = param_int(extra, 7);
    const int mode = param_int(extra, 9);
    const C extra0 = Elem<T>::load(extra + 10);
    const int kHEff = kH + (kH - 1) * (dH - 1), kWEff = kW + (kW - 1) * (dW - 1);
    const LL plane = (LL) blockIdx.x * blockDim.y + threadIdx.y;
    if (plane >= a.planes) return;
    const int c = (int) (plane % a.iC);
    const LL b = plane / a.iC;
    const T *in = static_cast<const T *>(a.x) + b * a.xs[0] + c * a.xs[1];
    T *out = static_cast<T *>(a.z) + b * a.zs[0] + c * a.zs[1];
    const int positions = a.oH * a.oW;
    const int stepRows = blockDim.x / a.oW, stepCols = blockDim.x % a.oW;
    int p = blockIdx.y * (blockDim.x * a.iters) + threadIdx.x;
    int yy = p / a.oW, xx = p - yy * a.oW;
    for (int it = 0; it < a.iters && p < positions; it++) {
        int hstart = yy * sH - pH, wstart = xx * sW - pW;
        int hend = hstart + kHEff, wend = wstart + kWEff;
        if (hstart < 0) hstart += ceil_div_pos(-hstart, dH) * dH;
        if (wstart < 0) wstart += ceil_div_pos(-wstart, dW) * dW;
        if (hend > a.iH) hend -= ceil_div_pos(hend - a.iH, dH) * dH;
        if (wend > a.iW) wend -= ceil_div_pos(wend - a.iW, dW) * dW;
        C acc = mode == 0 ? (C) Elem<T>::to_c(Elem<T>::from_c((C) -1e37)) : (C) 0;   // -MAX_FLOAT in the element type
        for (int ky = hstart; ky < hend; ky += dH) {
            const T *row = in + ky * a.xs[2];
            for (int kx = wstart; kx < wend; kx += dW) {
                const C v = Elem<T>::load(row + kx * a.xs[3]);
                if (mode == 0) { if (v > acc) acc = v; }
                else if (mode == 1) acc += v;
                else acc += pow(fabs(v), extra0);
            }
        }
        if (mode == 1) {
            int divisor = 0;
            if ((int) extra0 == 0) {
                divisor = ceil_div_pos(hend - hstart, dH) * ceil_div_pos(wend - wstart, dW);
            } else if ((int) extra0 == 1) divisor = kH * kW;
            acc = acc / (C) divisor;
        } else if (mode == 2) acc = pow(acc, (C) 1 / extra0);
        const LL at = a.fOrder ? yy * a.zs[2] + xx * a.zs[3] : (LL) p;
        Elem<T>::store(out + at, acc);
        p += blockDim.x; yy += stepRows; xx += stepCols;
        if (xx >= a.oW) { xx -= a.oW; yy++; }
    }
}

// ---- Histogram (48): z[i] += number of x whose bin is i, bin = (int) ((x - min) / binSize) clamped to
// [0, numBins), binSize = (max - min) / numBins (special_ops.h:713-880). extraParams = {numBins, min, max}. x is
// read as one dense run of its length, as the reference does. Counts are integers (shared-memory counters per
// CTA, then one global atomic per CTA and bin) and enter z in a second launch, so the result does not depend
// on scheduling.
struct HistArgs {
    const void *x, *extra;
    void *z;
    unsigned *counts;           // zLength zeroed words
    LL n, zLength;
};

constexpr int kHistShared = 8192;                            // bins kept in shared memory

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
    __shared__ unsigned bins[kHistShared];
    const T *extra = static_cast<const T *>(a.extra);
    const int numBins = hist_int(extra[0]);
    const T lo = extra[1], hi = extra[2];
    const T binSize = hist_div(hist_sub(hi, lo), Elem<T>::from_c((typename Elem<T>::C) numBins));
    const bool useShared = a.zLength <= kHistShared;
    if (useShared) {
        for (LL i = threadIdx.x; i < a.zLength; i += blockDim.x) bins[i] = 0;
        __syncthreads();
    }
    const T *x = static_cast<const T *>(a.x);
    for (LL i = (LL) blockIdx.x * blockDim.x + threadIdx.x; i < a.n; i += (LL) gridDim.x * blockDim.x) {
        int idx = hist_int(hist_div(hist_sub(x[i], lo), binSize));
        if (idx < 0) idx = 0;
        else if (idx >= numBins) idx = numBins - 1;
        if (idx < 0 || idx >= a.zLength) continue;            // numBins beyond the result: nowhere to count
        if (useShared) atomicAdd(&bins[idx], 1u);
        else atomicAdd(a.counts + idx, 1u);
    }
    if (useShared) {
        __syncthreads();
        for (LL i = threadIdx.x; i < a.zLength; i += blockDim.x)
            if (bins[i]) atomicAdd(a.counts + i, bins[i]);
    }
}

template <class T>
__global__ void __launch_bounds__(256) k_histogram_add(const HistArgs a) {
    grid_dependency_sync();
    T *z = static_cast<T *>(a.z);
    for (LL i = (LL) blockIdx.x * blockDim.x + threadIdx.x; i < a.zLength; i += (LL) gridDim.x * blockDim.x) {
        Elem<T>::store(z + i, Elem<T>::load(z + i) + (typename Elem<T>::C) a.counts[i]);
    }
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

template <class T>
__global__ void __launch_bounds__(256) k_reverse(const ReverseArgs a) {
    grid_dependency_sync();
    const T *x = static_cast<const T *>(a.x);
    T *z = static_cast<T *>(a.z);
    for (LL e = (LL) blockIdx.x * blockDim.x + threadIdx.x; e < a.count; e += (LL) gridDim.x * blockDim.x) {
        const LL from = view_offset(a.vx, e), to = view_offset(a.vz, a.n - 1 - e);
        if (a.swap) {
            const T lowV = z[from], highV = z[to];
            z[from] = highV; z[to] = lowV;
        } else {
            z[to] = x[from];
        }
    }
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
            if (!fits_int(zd.shape[4] * zd.shape[5]) || !fits_int(xd.shape[2] * xd.shape[3])) { set_error("Im2col: an image plane of 2^31 or more positions"); return kTooLarge; }
            Im2colArgs a;
            a.x = x; a.z = z; a.extra = extra;
            a.iC = (int) xd.shape[1]; a.iH = (int) xd.shape[2]; a.iW = (int) xd.shape[3];
            a.kH = (int) zd.shape[2]; a.kW = (int) zd.shape[3]; a.oH = (int) zd.shape[4]; a.oW = (int) zd.shape[5];
            a.planes = xd.shape[0] * xd.shape[1] * zd.shape[2] * zd.shape[3];
            strides(xd, a.xs); strides(zd, a.zs);
            if (descending_c(xd) && descending_c(zd)) dense_behind_batch(zd, 1, a.zs);
            const PlaneGrid g = plane_grid(a.planes, (LL) a.oH * a.oW);
            a.iters = g.iters;
            launch_kernel(k_im2col<T>, dim3(g.gx, g.gy), dim3(g.tx, g.ty), st, a);
            break;
        }
        case 36: {
            if (xd.rank != 6 || zd.rank != 4) return bad_arg("Col2Im: x must have rank 6 [b, c, kH, kW, oH, oW] and z rank 4 [b, c, h, w]");
            if (xd.shape[0] != zd.shape[0] || xd.shape[1] != zd.shape[1]) return bad_arg("Col2Im: x and z differ in batch size or channels");
            if (zd.length == 0) return kOk;
            if (!fits_int(zd.shape[2] * zd.shape[3]) || !fits_int(xd.shape[4] * xd.shape[5])) { set_error("Col2Im: an image plane of 2^31 or more positions"); return kTooLarge; }
            Col2imArgs a;
            a.x = x; a.z = z; a.extra = extra;
            a.iC = (int) zd.shape[1]; a.iH = (int) zd.shape[2]; a.iW = (int) zd.shape[3];
            a.kH = (int) xd.shape[2]; a.kW = (int) xd.shape[3]; a.oH = (int) xd.shape[4]; a.oW = (int) xd.shape[5];
            a.planes = zd.shape[0] * zd.shape[1];
            strides(xd, a.xs); strides(zd, a.zs);
            if (descending_c(xd) && descending_c(zd)) dense_behind_batch(xd, xd.stride[5], a.xs);
            const PlaneGrid g = plane_grid(a.planes, (LL) a.iH * a.iW);
            a.iters = g.iters;
            launch_kernel(k_col2im<T>, dim3(g.gx, g.gy), dim3(g.tx, g.ty), st, a);
            break;
        }
        case 71: {
            if (xd.rank != 4 || zd.rank != 4) return bad_arg("Pooling2D: x and z must have rank 4 [b, c, h, w]");
            if (xd.shape[0] != zd.shape[0] || xd.shape[1] != zd.shape[1]) return bad_arg("Pooling2D: x and z differ in batch size or channels");
            if (zd.length == 0) return kOk;
            if (!fits_int(zd.shape[2] * zd.shape[3]) || !fits_int(xd.shape[2] * xd.shape[3])) { set_error("Pooling2D: an image plane of 2^31 or more positions"); return kTooLarge; }
            PoolArgs a;
            a.x = x; a.z = z; a.extra = extra;
            a.iC = (int) xd.shape[1]; a.iH = (int) xd.shape[2]; a.iW = (int) xd.shape[3];
            a.oH = (int) zd.shape[2]; a.oW = (int) zd.shape[3];
            a.planes = xd.shape[0] * xd.shape[1];
            a.fOrder = zd.order == 'f';
            strides(xd, a.xs); strides(zd, a.zs);
            const PlaneGrid g = plane_grid(a.planes, (LL) a.oH * a.oW);
            a.iters = g.iters;
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
