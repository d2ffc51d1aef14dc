// Host-side shapeInfo / TAD decoding. See shape_host.h for the contract.
#include "shape_host.h"
#include <algorithm>
#include <cstring>
#include <sstream>

namespace nd4jb200 {

static thread_local std::string g_last_error;

void set_error(const std::string &msg) { g_last_error = msg; }
const char *last_error() { return g_last_error.c_str(); }

Status parse_shape(const LL *info, const char *what, ShapeDesc *out) {
    if (info == nullptr) {
        set_error(std::string(what) + ": shapeInfo is null");
        return kBadArgument;
    }
    LL rank = info[0];
    if (rank < 0 || rank > kMaxRank) {
        std::ostringstream os;
        os << what << ": rank " << rank << " outside [0, " << kMaxRank << "]";
        set_error(os.str());
        return kBadArgument;
    }
    out->rank = (int) rank;
    out->length = 1;
    for (int i = 0; i < out->rank; i++) {
        out->shape[i] = info[1 + i];
        out->stride[i] = info[1 + rank + i];
        if (out->shape[i] < 0) {
            std::ostringstream os;
            os << what << ": negative extent " << out->shape[i] << " on axis " << i;
            set_error(os.str());
            return kBadArgument;
        }
        out->length *= out->shape[i];
    }
    out->offset = info[2 * rank + 1];
    out->ews = info[2 * rank + 2];
    LL order = info[2 * rank + 3];
    out->order = (order == 'f') ? 'f' : 'c';
    return kOk;
}

Status collapse_view(int n, const LL *shape, const LL *stride, View *out) {
    LL s[kMaxRank], t[kMaxRank];
    int m = 0;
    for (int i = 0; i < n; i++) {
        if (shape[i] == 1) continue;  // a unit axis contributes nothing (shape.h getOffset skips them too)
        if (m > 0 && t[m - 1] == shape[i] * stride[i]) {
            s[m - 1] *= shape[i];  // outer axis continues exactly where the inner one wraps
            t[m - 1] = stride[i];
        } else {
            s[m] = shape[i];
            t[m] = stride[i];
            m++;
        }
    }
    if (m > kDevRank) {
        std::ostringstream os;
        os << "view needs " << m << " independent axes after merging; this backend carries at most " << kDevRank;
        set_error(os.str());
        return kTooLarge;
    }
    out->rank = m;
    for (int i = 0; i < kDevRank; i++) {
        out->shape[i] = i < m ? s[i] : 1;
        out->stride[i] = i < m ? t[i] : 0;
    }
    return kOk;
}

Status coord_view(const ShapeDesc &d, View *out) { return collapse_view(d.rank, d.shape, d.stride, out); }

Status linear_view(const ShapeDesc &d, View *out) {
    if (d.ews >= 1) {
        LL shape[1] = {d.length};
        LL stride[1] = {d.ews};
        return collapse_view(1, shape, stride, out);
    }
    return coord_view(d, out);
}

char stride_order(int rank, const LL *shape, const LL *stride) {
    bool c = true, f = true;
    LL sd = 1;
    for (int i = rank - 1; i >= 0; --i) {
        if (stride[i] != sd) { c = false; break; }
        if (shape[i] == 0) break;
        sd *= shape[i];
    }
    sd = 1;
    for (int i = 0; i < rank; ++i) {
        if (stride[i] != sd) f = false;
        if (shape[i] == 0) break;
        sd *= shape[i];
    }
    if (f && c) return 'a';
    if (f) return 'f';
    return 'c';
}

Status make_tad_plan(const ShapeDesc &x, const int *dimension, int dimensionLength, TadPlan *out) {
    bool isDim[kMaxRank] = {false};
    bool whole = (dimension == nullptr || dimensionLength <= 0 ||
                  (dimensionLength == 1 && dimension[0] == kMaxDimension));
    int nd = 0;
    if (!whole) {
        for (int i = 0; i < dimensionLength; i++) {
            int d = dimension[i];
            if (d < 0) d += x.rank;
            if (d < 0 || d >= x.rank) {
                std::ostringstream os;
                os << "dimension[" << i << "] = " << dimension[i] << " is not an axis of a rank-" << x.rank << " array";
                set_error(os.str());
                return kBadArgument;
            }
            if (!isDim[d]) { isDim[d] = true; nd++; }
        }
        if (nd == x.rank) whole = true;
    }
    out->whole = whole;
    out->ndims = 0;
    if (whole) {
        out->numTads = 1;
        out->tadLen = x.length;
        for (int i = 0; i < x.rank; i++) out->dims[out->ndims++] = i;
        Status st = linear_view(x, &out->inner);
        if (st != kOk) return st;
        return collapse_view(0, nullptr, nullptr, &out->outer);
    }
    LL is[kMaxRank], it[kMaxRank], os_[kMaxRank], ot[kMaxRank];
    int ni = 0, no = 0;
    out->tadLen = 1;
    out->numTads = 1;
    for (int i = 0; i < x.rank; i++) {
        if (isDim[i]) {
            out->dims[out->ndims++] = i;
            is[ni] = x.shape[i]; it[ni] = x.stride[i]; ni++;
            out->tadLen *= x.shape[i];
        } else {
            os_[no] = x.shape[i]; ot[no] = x.stride[i]; no++;
            out->numTads *= x.shape[i];
        }
    }
    Status st = collapse_view(ni, is, it, &out->inner);
    if (st != kOk) return st;
    return collapse_view(no, os_, ot, &out->outer);
}

int dims_from_tad_info(const ShapeDesc &x, const ShapeDesc &tad, int *dims) {
    if (tad.length == x.length) return 0;                 // one TAD: the whole array
    if (tad.length <= 0 || x.length % tad.length != 0) return -1;
    bool used[kMaxRank] = {false};
    int n = 0;
    if (tad.length == 1) {
        for (int i = 0; i < x.rank; i++) if (x.shape[i] == 1) dims[n++] = i;
        return n > 0 ? n : -1;
    }
    int from = 0;
    for (int t = 0; t < tad.rank; t++) {
        if (tad.shape[t] == 1) continue;
        int hit = -1;
        // TAD axes keep the array's axis order, so look behind the previous match first
        for (int pass = 0; pass < 2 && hit < 0; pass++)
            for (int i = pass == 0 ? from : 0; i < (pass == 0 ? x.rank : from); i++)
                if (!used[i] && x.shape[i] == tad.shape[t] && x.stride[i] == tad.stride[t]) { hit = i; break; }
        if (hit < 0) return -1;
        used[hit] = true;
        from = hit + 1;
    }
    LL len = 1;
    for (int i = 0; i < x.rank; i++) if (used[i]) { dims[n++] = i; len *= x.shape[i]; }
    return len == tad.length ? n : -1;
}

static void write_info(LL *target, int rank, const LL *shape, const LL *stride, LL offset, LL ews, char order) {
    target[0] = rank;
    for (int i = 0; i < rank; i++) { target[1 + i] = shape[i]; target[1 + rank + i] = stride[i]; }
    target[2 * rank + 1] = offset;
    target[2 * rank + 2] = ews;
    target[2 * rank + 3] = order;
}

Status tad_only_shape_info(const LL *xShapeInfo, const int *dimension, int dimensionLength,
                           LL *target, LL *offsets, LL *numTadsOut) {
    ShapeDesc x;
    Status st = parse_shape(xShapeInfo, "tadOnlyShapeInfo: x", &x);
    if (st != kOk) return st;
    TadPlan plan;
    st = make_tad_plan(x, dimension, dimensionLength, &plan);
    if (st != kOk) return st;
    if (numTadsOut) *numTadsOut = plan.numTads;

    if (target) {
        bool scalarArray = x.rank == 0 || x.length == 1;
        bool maxDim = dimensionLength == 1 && dimension != nullptr && dimension[0] == kMaxDimension;
        if (scalarArray || maxDim) {
            // rank-1 single-element descriptor, as createScalarShapeInfo-based paths report it
            LL one[1] = {1};
            write_info(target, 1, one, one, 0, 1, 'c');
        } else if (plan.whole) {
            // the TAD is the array itself: the descriptor is handed back unchanged
            std::memcpy(target, xShapeInfo, sizeof(LL) * (2 * x.rank + 4));
        } else if (plan.ndims == 1) {
            int d = plan.dims[0];
            if (x.shape[d] == 1) {
                LL one[1] = {1};
                write_info(target, 1, one, one, 0, 1, 'c');
            } else {
                // a single axis is always reported as a [1, n] row with strides [1, s]
                LL shp[2] = {1, x.shape[d]};
                LL str[2] = {1, x.stride[d]};
                write_info(target, 2, shp, str, 0, x.stride[d], stride_order(2, shp, str));
            }
        } else {
            LL shp[kMaxRank], str[kMaxRank];
            for (int i = 0; i < plan.ndims; i++) { shp[i] = x.shape[plan.dims[i]]; str[i] = x.stride[plan.dims[i]]; }
            // several axes: shape/stride of those axes in ascending order, no linear stride
            write_info(target, plan.ndims, shp, str, 0, -1, stride_order(plan.ndims, shp, str));
        }
    }
    if (offsets) {
        // base offsets enumerate the remaining axes in c-order (TAD.h tad2Sub uses ind2subC)
        LL os_[kMaxRank], ot[kMaxRank], idx[kMaxRank];
        int no = 0;
        bool isDim[kMaxRank] = {false};
        for (int i = 0; i < plan.ndims; i++) isDim[plan.dims[i]] = true;
        for (int i = 0; i < x.rank; i++) if (!isDim[i]) { os_[no] = x.shape[i]; ot[no] = x.stride[i]; idx[no] = 0; no++; }
        LL off = 0;
        for (LL r = 0; r < plan.numTads; r++) {
            offsets[r] = off;
            for (int a = no - 1; a >= 0; --a) {  // odometer increment
                idx[a]++; off += ot[a];
                if (idx[a] < os_[a]) break;
                off -= ot[a] * os_[a]; idx[a] = 0;
            }
        }
    }
    return kOk;
}

}  // namespace nd4jb200
