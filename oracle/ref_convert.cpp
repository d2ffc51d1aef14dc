// TEST INFRASTRUCTURE ONLY -- never linked into or called from the product library.
//
// The reference defines NativeOps::convertTypes in a header (include/loops/type_conversions.h:696-880);
// this translation unit instantiates it, with the reference's saturating integer wrappers from
// include/types/impl/, and exposes it to the parity tests.
#include <NativeOps.h>
#include <loops/type_conversions.h>

extern "C" void ref_convertTypes(int srcType, void *x, long long n, int dstType, void *z) {
    NativeOps ops;
    ops.convertTypes(nullptr, srcType, x, n, dstType, z);
}
