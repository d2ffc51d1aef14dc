// Host-side decoding of the reference's shapeInfo descriptors and of tensors-along-dimension
// (TADs). Layout of a shapeInfo buffer (include/helpers/shape.h:2558-2617 of the reference):
//   [rank, shape[0..rank), stride[0..rank), offset, elementWiseStride, order]   (2*rank+4 longs)
// Nothing here touches the GPU: the result of decoding is a small POD plan that the kernel
// launchers pass by value.
#pragma once
#include <string>
#include "common.h"

namespace nd4jb200 {

struct ShapeDesc {
    int rank;
    LL shape[kMaxRank];
    LL stride[kMaxRank];
    LL offset;
    LL ews;      // elementWiseStride slot; >= 1 means "walk the buffer linearly in `order`"
    char order;  // 'c' or 'f'
    LL length;
};

// Thread-local message describing the last non-zero Status.
void set_error(const std::string &msg);
const char *last_error();

Status parse_shape(const LL *info, const char *what, ShapeDesc *out);

// View over the whole array in the iteration order the reference's loops use for a
// "linear index": i*ews when ews >= 1, otherwise c-order coordinates (ind2subC + getOffset).
Status linear_view(const ShapeDesc &d, View *out);
// View over the whole array by c-order coordinates regardless of ews.
Status coord_view(const ShapeDesc &d, View *out);
// Collapse (shape, stride) lists given in c-order significance into a View.
Status collapse_view(int n, const LL *shape, const LL *stride, View *out);

// True when the array is one dense run of `length` elements (ews == 1).
inline bool is_dense(const ShapeDesc &d) { return d.ews == 1; }

struct TadPlan {
    LL numTads;
    LL tadLen;
    View inner;  // element j of a TAD (c-order over the TAD's own axes) -> offset from TAD base
    View outer;  // TAD index r (c-order over the remaining axes) -> TAD base offset
    int ndims;   // normalised dimension list (ascending, unique)
    int dims[kMaxRank];
    bool whole;  // the dimension list covers the whole array (scalar reduction)
};

// Normalises `dimension` (negative values count from the back, duplicates dropped, sorted) and
// builds the plan. dimension == {kMaxDimension}, dimensionLength == rank or a null/empty list
// mean "whole array" (include/loops/cpu/reduce.cpp:108-111, include/helpers/TAD.h:723-725).
Status make_tad_plan(const ShapeDesc &x, const int *dimension, int dimensionLength, TadPlan *out);

// Equivalent of NativeOps::tadOnlyShapeInfo (blas/cpu/NativeOps.cpp:2022-2032): writes the
// TAD's own shapeInfo to `target` (room for 2*rank+4 longs) and the numTads base offsets to
// `offsets`. Either output may be null.
Status tad_only_shape_info(const LL *xShapeInfo, const int *dimension, int dimensionLength,
                           LL *target, LL *offsets, LL *numTadsOut);

// Recovers a dimension list from the array's shapeInfo and the shapeInfo of its TADs (what callers of the
// reference's CUDA build keep on the host next to the device copies): every non-unit TAD axis is matched to
// the array axis with the same extent and stride, in ascending order. Unit axes do not change any offset and
// are left out, except when the TAD is a single element (then the array's unit axes are the list). Returns the
// number of dimensions written to `dims` (room for kMaxRank), 0 when the TAD is the whole array, and -1 when
// the descriptors do not determine the list (the caller then has to obtain it another way).
int dims_from_tad_info(const ShapeDesc &x, const ShapeDesc &tad, int *dims);

// 'c'/'f'/'a' classification of a (shape, stride) pair, as written into permuted and sliced
// shapeInfos by the reference (include/helpers/shape.h:2195-2236).
char stride_order(int rank, const LL *shape, const LL *stride);

}  // namespace nd4jb200
