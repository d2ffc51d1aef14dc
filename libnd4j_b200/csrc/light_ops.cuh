// Binary ops cheap enough to be selected by a run-time code inside a fused kernel (a warp-uniform switch of
// one or two instructions per case), and the mapping from the reference's op numbers
// (include/loops/legacy_ops.h) onto those codes. Each case is the same expression as the functor of that name
// in functors.cuh, so a fused kernel rounds exactly like the separate launches it replaces.
#pragma once
#include "device_utils.cuh"

namespace nd4jb200 {

enum LightOp : int {
    kLightNone = -1,
    kLightAdd = 0, kLightSubtract, kLightMultiply, kLightDivide, kLightReverseDivide, kLightReverseSubtract,
    kLightCopy, kLightMax, kLightMin, kLightSquaredSubtract, kLightEqualTo, kLightNotEqualTo, kLightGreaterThan,
    kLightGreaterThanOrEqual, kLightLessThan, kLightLessThanOrEqual
};

template <class C> ND_D C light_apply(int code, C x, C y) {
    switch (code) {
        case kLightAdd: return x + y;
        case kLightSubtract: return x - y;
        case kLightMultiply: return x * y;
        case kLightDivide: return x / y;
        case kLightReverseDivide: return y / x;
        case kLightReverseSubtract: return y - x;
        case kLightCopy: return y;
        case kLightMax: return x > y ? x : y;
        case kLightMin: return x < y ? x : y;
        case kLightSquaredSubtract: { const C d = x - y; return d * d; }
        case kLightEqualTo: return C(x == y);
        case kLightNotEqualTo: return C(x != y);
        case kLightGreaterThan: return C(x > y);
        case kLightGreaterThanOrEqual: return C(x >= y);
        case kLightLessThan: return C(x < y);
        default: return C(x <= y);
    }
}

// t[i] = op(t[i], y[i]) for a register tile: the op is selected once per tile, outside the element loop, so the
// selection costs a few instructions per N elements instead of per element.
template <class C, int N> ND_D void light_apply_tile(int code, C (&t)[N], const C (&y)[N]) {
#define ND_LIGHT_CASE(CODE, EXPR)                                         \
    case CODE: {                                                          \
        _Pragma("unroll") for (int i = 0; i < N; i++) {                   \
            const C a = t[i], b = y[i];                                   \
            t[i] = (EXPR);                                                \
        }                                                                 \
    } break;
    switch (code) {
        ND_LIGHT_CASE(kLightAdd, a + b)
        ND_LIGHT_CASE(kLightSubtract, a - b)
        ND_LIGHT_CASE(kLightMultiply, a * b)
        ND_LIGHT_CASE(kLightDivide, a / b)
        ND_LIGHT_CASE(kLightReverseDivide, b / a)
        ND_LIGHT_CASE(kLightReverseSubtract, b - a)
        ND_LIGHT_CASE(kLightCopy, b)
        ND_LIGHT_CASE(kLightMax, a > b ? a : b)
        ND_LIGHT_CASE(kLightMin, a < b ? a : b)
        ND_LIGHT_CASE(kLightSquaredSubtract, (a - b) * (a - b))
        ND_LIGHT_CASE(kLightEqualTo, C(a == b))
        ND_LIGHT_CASE(kLightNotEqualTo, C(a != b))
        ND_LIGHT_CASE(kLightGreaterThan, C(a > b))
        ND_LIGHT_CASE(kLightGreaterThanOrEqual, C(a >= b))
        ND_LIGHT_CASE(kLightLessThan, C(a < b))
        default: {
            _Pragma("unroll") for (int i = 0; i < N; i++) t[i] = C(t[i] <= y[i]);
        } break;
    }
#undef ND_LIGHT_CASE
}

// BROADCAST_OPS / PAIRWISE_TRANSFORM_OPS / SCALAR_OPS number -> light code, or kLightNone.
inline int light_of_broadcast(int opNum) {
    static const int map[] = {kLightAdd, kLightSubtract, kLightMultiply, kLightDivide, kLightReverseDivide,
                              kLightReverseSubtract, kLightCopy, kLightEqualTo, kLightGreaterThan,
                              kLightGreaterThanOrEqual, kLightLessThan, kLightLessThanOrEqual, kLightNotEqualTo,
                              kLightMin, kLightMax, kLightNone, kLightNone, kLightSquaredSubtract};
    return opNum >= 0 && opNum < (int) (sizeof(map) / sizeof(map[0])) ? map[opNum] : kLightNone;
}
inline int light_of_pairwise(int opNum) {
    switch (opNum) {
        case 0: return kLightAdd;
        case 1: case 16: return kLightCopy;
        case 2: return kLightDivide;
        case 3: return kLightEqualTo;
        case 4: return kLightGreaterThan;
        case 5: return kLightLessThan;
        case 6: return kLightMultiply;
        case 8: return kLightReverseSubtract;
        case 9: return kLightSubtract;
        case 11: return kLightGreaterThanOrEqual;
        case 12: return kLightLessThanOrEqual;
        case 13: return kLightMax;
        case 14: return kLightMin;
        case 15: return kLightNotEqualTo;
        case 18: return kLightReverseDivide;
        case 22: return kLightSquaredSubtract;
        default: return kLightNone;
    }
}
inline int light_of_scalar(int opNum) {
    static const int map[] = {kLightAdd, kLightSubtract, kLightMultiply, kLightDivide, kLightReverseDivide,
                              kLightReverseSubtract, kLightMax, kLightLessThan, kLightGreaterThan, kLightEqualTo,
                              kLightLessThanOrEqual, kLightNotEqualTo, kLightMin, kLightCopy, kLightNone, kLightNone,
                              kLightGreaterThanOrEqual, kLightNone, kLightNone, kLightNone, kLightNone, kLightNone,
                              kLightSquaredSubtract};
    return opNum >= 0 && opNum < (int) (sizeof(map) / sizeof(map[0])) ? map[opNum] : kLightNone;
}

// A value as the separate launches would hand it on: stored in the element type and loaded again.
template <class T> ND_D typename Elem<T>::C through_memory(typename Elem<T>::C v) { return Elem<T>::to_c(Elem<T>::from_c(v)); }

}  // namespace nd4jb200
