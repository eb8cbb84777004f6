// Host-side planning for the reductions: recognise the contiguous [O, R, I] structure
// behind the reference's fold formulas, otherwise fall back to the literal scatter.
// Metadata layouts (crates/maidenx_tensor/src/ops/reduction.rs:722-744):
//   sum/mean/max/min: [dims(n) | strides(n) | red_len(r) | red_stride(r) | offset]
//   sum_to_shape:     [in_dims(n) | in_strides(n) | out_dims(n) | offset]
#include <cstring>

#include "reduction.cuh"

namespace mx {

namespace {
bool contiguous(size_t nd, const size_t* dims, const size_t* strides) {
    // size-1 dims are ignored (crates/maidenx_cpu/src/utils.rs:2-12)
    size_t acc = 1;
    for (size_t d = nd; d-- > 0;) {
        if (dims[d] > 1 && strides[d] != acc) return false;
        acc *= dims[d];
    }
    return true;
}
}  // namespace

void red_plan_dims(RedPlan& pl, size_t n, size_t nd, size_t nr, const size_t* hm) {
    std::memset(&pl, 0, sizeof(pl));
    const size_t* dims = hm;
    const size_t* strides = hm + nd;
    const size_t* rl = hm + 2 * nd;
    const size_t* rs = hm + 2 * nd + nr;
    pl.off = hm[2 * nd + 2 * nr];
    u64 out = n, factor = 1;
    for (size_t k = 0; k < nr; k++) {
        if (rl[k] == 0) {
            pl.kind = n == 0 ? RP_EMPTY : RP_ERROR;
            return;
        }
        out /= rl[k];
        factor *= rl[k];
    }
    pl.out_count = out;
    pl.factor = factor;
    if (n == 0 || out == 0) {
        pl.kind = RP_EMPTY;
        return;
    }
    const bool cont = contiguous(nd, dims, strides);
    if (cont && nr == 0) {
        pl.kind = RP_COLS;
        pl.O = 1;
        pl.R = 1;
        pl.I = n;
        return;
    }
    if (cont && nr == 1) {
        u64 l = rl[0], s = rs[0];
        if (s == 0) {  // the reference's contiguous branch divides by this stride
            pl.kind = RP_ERROR;
            return;
        }
        if (n % (l * s) == 0) {
            pl.O = n / (l * s);
            pl.R = l;
            pl.I = s;
            pl.kind = s == 1 ? RP_ROWS : RP_COLS;
            return;
        }
    }
    if (nd > (size_t)kRedMaxDims || nr > (size_t)kRedMaxDims) {
        pl.kind = RP_ERROR;
        return;
    }
    if (cont)
        for (size_t k = 0; k < nr; k++)
            if (rs[k] == 0) {
                pl.kind = RP_ERROR;
                return;
            }
    RedGenParams& g = pl.gen;
    g.mode = 0;
    g.n = n;
    g.nd = (int)nd;
    g.nr = (int)nr;
    g.contiguous = cont ? 1 : 0;
    for (size_t d = 0; d < nd; d++) {
        g.dims[d] = dims[d];
        g.strides[d] = strides[d];
        if (!cont && dims[d] == 0) {
            pl.kind = RP_ERROR;
            return;
        }
    }
    for (size_t k = 0; k < nr; k++) {
        g.red_len[k] = rl[k];
        g.red_stride[k] = rs[k];
    }
    g.off = pl.off;
    pl.kind = RP_GENERIC;
}

void red_plan_shape(RedPlan& pl, size_t n, size_t nd, const size_t* hm) {
    std::memset(&pl, 0, sizeof(pl));
    const size_t* idims = hm;
    const size_t* ist = hm + nd;
    const size_t* odims = hm + 2 * nd;
    pl.off = hm[3 * nd];
    pl.factor = 1;
    u64 out = 1, in = 1;
    for (size_t d = 0; d < nd; d++) {
        out *= odims[d];
        in *= idims[d];
    }
    pl.out_count = out;
    if (out == 0) {
        pl.kind = RP_EMPTY;
        return;
    }
    for (size_t d = 0; d < nd; d++)
        if (n != 0 && (idims[d] == 0 || idims[d] / odims[d] == 0)) {  // reduction factor 0: division by zero in the reference
            pl.kind = RP_ERROR;
            return;
        }
    const bool cont = contiguous(nd, idims, ist);
    if (n != 0 && cont && in == n) {
        // classify dims: keep (out == in) / reduce (out == 1); size-1 dims are neutral
        bool simple = true;
        int kinds[64];
        u64 sizes[64];
        int m = 0;
        for (size_t d = 0; d < nd && simple; d++) {
            if (idims[d] == 1 && odims[d] == 1) continue;
            int kind;
            if (odims[d] == idims[d]) kind = 0;
            else if (odims[d] == 1) kind = 1;
            else {
                simple = false;
                break;
            }
            if (m > 0 && kinds[m - 1] == kind) sizes[m - 1] *= idims[d];
            else if (m < 64) {
                kinds[m] = kind;
                sizes[m] = idims[d];
                m++;
            } else simple = false;
        }
        if (simple) {
            if (m == 0 || (m == 1 && kinds[0] == 0)) {  // nothing folded: copy
                pl.kind = RP_COLS;
                pl.O = 1;
                pl.R = 1;
                pl.I = n;
                return;
            }
            if (m == 1) {  // [R]
                pl.kind = RP_ROWS;
                pl.O = 1;
                pl.R = sizes[0];
                pl.I = 1;
                return;
            }
            if (m == 2 && kinds[0] == 0) {  // [K, R]
                pl.kind = RP_ROWS;
                pl.O = sizes[0];
                pl.R = sizes[1];
                pl.I = 1;
                return;
            }
            if (m == 2) {  // [R, K]
                pl.kind = RP_COLS;
                pl.O = 1;
                pl.R = sizes[0];
                pl.I = sizes[1];
                return;
            }
            if (m == 3 && kinds[0] == 0) {  // [K, R, K]
                pl.kind = RP_COLS;
                pl.O = sizes[0];
                pl.R = sizes[1];
                pl.I = sizes[2];
                return;
            }
        }
    }
    if (nd > (size_t)kRedMaxDims) {
        pl.kind = RP_ERROR;
        return;
    }
    RedGenParams& g = pl.gen;
    g.mode = 1;
    g.n = n;
    g.nd = (int)nd;
    g.contiguous = cont ? 1 : 0;
    for (size_t d = 0; d < nd; d++) {
        g.dims[d] = idims[d];
        g.strides[d] = ist[d];
        g.out_dims[d] = odims[d];
    }
    g.off = pl.off;
    pl.kind = RP_GENERIC;
}

}  // namespace mx

// Host-only view of the reduction planner (see mx_debug_elementwise_plan): returns the RedPlanKind
// (0 empty, 1 rows, 2 cols, 3 generic scatter, 4 error) and the recognised [O, R, I] structure.
// sum_to_shape != 0 reads metadata as [in_dims | in_strides | out_dims | offset] and ignores num_red_dims.
extern "C" int mx_debug_reduce_plan(size_t num_els, size_t num_dims, size_t num_red_dims, const size_t* host_metadata, int sum_to_shape,
                                    size_t* outer, size_t* reduced, size_t* inner) {
    mx::RedPlan pl;
    if (sum_to_shape) mx::red_plan_shape(pl, num_els, num_dims, host_metadata);
    else mx::red_plan_dims(pl, num_els, num_dims, num_red_dims, host_metadata);
    if (outer) *outer = pl.O;
    if (reduced) *reduced = pl.R;
    if (inner) *inner = pl.I;
    return pl.kind;
}
