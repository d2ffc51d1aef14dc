// Device helpers shared by all kernels: element-type traits, 128-bit vector access, and
// warp/block merging of small POD accumulator states.
#pragma once
#include <cuda_runtime.h>
#include <cuda_fp16.h>
#include "common.h"

namespace nd4jb200 {

constexpr int kNumSMs = 148;  // B200: two dies of 74 SMs

template <class T> struct Elem;
template <> struct Elem<float> {
    typedef float C;
    static constexpr int kVec = 4;
    ND_D static float load(const float *p) { return *p; }
    ND_D static void store(float *p, float v) { *p = v; }
    ND_D static float to_c(float v) { return v; }
    ND_D static float from_c(float v) { return v; }
};
template <> struct Elem<double> {
    typedef double C;
    static constexpr int kVec = 2;
    ND_D static double load(const double *p) { return *p; }
    ND_D static void store(double *p, double v) { *p = v; }
    ND_D static double to_c(double v) { return v; }
    ND_D static double from_c(double v) { return v; }
};
template <> struct Elem<__half> {
    typedef float C;  // half data is widened to float, computed, and rounded to nearest-even once
    static constexpr int kVec = 8;
    ND_D static float load(const __half *p) { return __half2float(*p); }
    ND_D static void store(__half *p, float v) { *p = __float2half_rn(v); }
    ND_D static float to_c(__half v) { return __half2float(v); }
    ND_D static __half from_c(float v) { return __float2half_rn(v); }
};

// 16 bytes of T moved as one transaction.
template <class T> struct alignas(16) Pack {
    T v[Elem<T>::kVec];
};
template <class T> ND_D Pack<T> load_pack(const T *p) {
    Pack<T> r;
    *reinterpret_cast<uint4 *>(&r) = __ldg(reinterpret_cast<const uint4 *>(p));
    return r;
}
template <class T> ND_D Pack<T> load_pack_rw(const T *p) {
    // plain load: the buffer may be written by this kernel (in-place ops)
    Pack<T> r;
    *reinterpret_cast<uint4 *>(&r) = *reinterpret_cast<const uint4 *>(p);
    return r;
}
template <class T> ND_D void store_pack(T *p, const Pack<T> &r) {
    *reinterpret_cast<uint4 *>(p) = *reinterpret_cast<const uint4 *>(&r);
}

template <class T, int N> ND_D void load_params(const T *extra, typename Elem<T>::C *p) {
#pragma unroll
    for (int k = 0; k < N; k++) p[k] = extra ? Elem<T>::load(extra + k) : typename Elem<T>::C(0);
}

// Exchange an arbitrary POD state between lanes, 32 bits at a time.
template <class S> ND_D S shfl_xor_state(const S &s, int mask) {
    static_assert(sizeof(S) % 4 == 0, "state must be a multiple of 4 bytes");
    S r;
    const unsigned *src = reinterpret_cast<const unsigned *>(&s);
    unsigned *dst = reinterpret_cast<unsigned *>(&r);
#pragma unroll
    for (int w = 0; w < (int) (sizeof(S) / 4); w++) dst[w] = __shfl_xor_sync(0xffffffffu, src[w], mask);
    return r;
}

// First statement of every kernel: allow the stream's next kernel to be scheduled early, then wait
// until the previous kernel has completed and its memory operations are visible. Both are no-ops
// for a kernel launched without programmatic stream serialisation.
ND_D void grid_dependency_sync() {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
}

// Butterfly merge across `width` adjacent lanes (width a power of two <= 32). Every lane of the
// group ends with the same merged state; the merge order is fixed by the lane ids, so results
// do not depend on scheduling.
template <class P, class S> ND_D void group_merge(S &s, int width) {
    for (int m = width >> 1; m > 0; m >>= 1) {
        S o = shfl_xor_state(s, m);
        // keep the lower lane's state on the left so that non-commutative ties resolve identically
        if ((threadIdx.x & m) == 0) { P::merge(s, o); } else { S t = o; P::merge(t, s); s = t; }
    }
}

}  // namespace nd4jb200
