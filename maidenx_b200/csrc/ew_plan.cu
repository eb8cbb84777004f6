// Host-side layout canonicalisation and kernel selection for the elementwise engine.
// Metadata layouts (built by the reference's tensor layer):
//   binary / in-place: [dims(n) | lhs_strides(n) | rhs_strides(n) | lhs_off, rhs_off]
//                      crates/maidenx_tensor/src/ops/binary.rs:754-769
//   unary:             [dims(n) | strides(n) | off]
//                      crates/maidenx_tensor/src/ops/unary.rs:1308-1320
// A NULL metadata pointer means contiguous operands with zero offsets
// (crates/maidenx_cuda/kernels/ops/binary.cu:20-25).
#include <algorithm>
#include <cstring>

#include "elementwise.cuh"

namespace mx {

namespace {
constexpr int kRawMax = 32;

inline bool aligned_to(const void* base, int64_t off_elems, size_t elem, size_t bytes) {
    return ((uintptr_t)base + (uintptr_t)(off_elems * (int64_t)elem)) % bytes == 0;
}
}  // namespace

void ew_make_plan(EwPlan& pl, size_t num_els, size_t num_dims, const size_t* hm, int nin, bool inplace, size_t in_size,
                  size_t out_size, const void* out, const void* a, const void* b) {
    std::memset(&pl, 0, sizeof(pl));
    pl.nin = nin;
    pl.n = num_els;
    if (num_els == 0) {
        pl.kind = EW_EMPTY;
        return;
    }
    if (num_dims > (size_t)kRawMax) {
        pl.kind = EW_ERROR;
        return;
    }
    // ---- raw dims / strides --------------------------------------------------------
    uint64_t dim[kRawMax];
    int64_t st[3][kRawMax];
    int nd = 0;
    if (!hm) {
        nd = 1;
        dim[0] = num_els;
        st[0][0] = st[1][0] = st[2][0] = 1;
    } else {
        nd = (int)num_dims;
        uint64_t prod = 1;
        for (int d = 0; d < nd; d++) {
            dim[d] = hm[d];
            st[1][d] = (int64_t)hm[nd + d];
            st[2][d] = nin == 2 ? (int64_t)hm[2 * nd + d] : 0;
            prod *= dim[d];
        }
        if (prod != num_els) {  // metadata and element count disagree
            pl.kind = EW_ERROR;
            return;
        }
        if (nin == 2) {
            pl.off[1] = (int64_t)hm[3 * nd];
            pl.off[2] = (int64_t)hm[3 * nd + 1];
        } else {
            pl.off[1] = (int64_t)hm[2 * nd];
        }
        if (inplace) {
            for (int d = 0; d < nd; d++) st[0][d] = st[1][d];
            pl.off[0] = pl.off[1];
        } else {
            int64_t acc = 1;
            for (int d = nd - 1; d >= 0; d--) {
                st[0][d] = acc;
                acc *= (int64_t)dim[d];
            }
        }
    }
    const void* ptr[3] = {out, a, b};
    const size_t esz[3] = {out_size, in_size, in_size};
    const int nop = nin + 1;

    // ---- drop size-1 dims ----------------------------------------------------------
    {
        int w = 0;
        for (int d = 0; d < nd; d++)
            if (dim[d] != 1) {
                dim[w] = dim[d];
                for (int k = 0; k < 3; k++) st[k][w] = st[k][d];
                w++;
            }
        nd = w;
    }
    bool serial = false;
    if (inplace && nd > 0) {
        // The output is the lhs view: order dims by its strides so the kernels' "last dim
        // is the output's fastest" convention holds, and make sure the view does not
        // overlap itself.
        int order[kRawMax];
        for (int d = 0; d < nd; d++) order[d] = d;
        std::stable_sort(order, order + nd, [&](int x, int y) { return st[0][x] > st[0][y]; });
        bool ok = true;
        for (int i = 0; i < nd; i++) {
            int d = order[i];
            if (st[0][d] <= 0) ok = false;
            if (i + 1 < nd && st[0][d] < st[0][order[i + 1]] * (int64_t)dim[order[i + 1]]) ok = false;
        }
        if (!ok) {
            serial = true;
        } else {
            uint64_t nd_dim[kRawMax];
            int64_t nst[3][kRawMax];
            for (int i = 0; i < nd; i++) {
                nd_dim[i] = dim[order[i]];
                for (int k = 0; k < 3; k++) nst[k][i] = st[k][order[i]];
            }
            std::memcpy(dim, nd_dim, sizeof(uint64_t) * nd);
            for (int k = 0; k < 3; k++) std::memcpy(st[k], nst[k], sizeof(int64_t) * nd);
        }
    }
    auto store = [&](int n_dims) {
        pl.nd = n_dims;
        for (int d = 0; d < n_dims; d++) {
            pl.dim[d] = (uint32_t)dim[d];
            for (int k = 0; k < 3; k++) pl.st[k][d] = st[k][d];
        }
    };
    auto fits_generic = [&](int n_dims) {
        if (n_dims > kMaxDims) return false;
        for (int d = 0; d < n_dims; d++)
            if (dim[d] > 0xFFFFFFFFull) return false;
        return true;
    };
    if (serial) {
        if (!fits_generic(nd)) {
            pl.kind = EW_ERROR;
            return;
        }
        store(nd);
        pl.kind = EW_SERIAL;
        return;
    }
    // keep an unmerged copy for the >= 2^32-element fallback
    uint64_t dim_raw[kRawMax];
    int64_t st_raw[3][kRawMax];
    int nd_raw = nd;
    std::memcpy(dim_raw, dim, sizeof(dim));
    std::memcpy(st_raw, st, sizeof(st));

    // ---- merge adjacent dims -------------------------------------------------------
    if (nd > 1) {
        int w = nd - 1;  // write cursor, building from the back
        for (int d = nd - 2; d >= 0; d--) {
            bool can = true;
            for (int k = 0; k < nop; k++)
                if (st[k][d] != st[k][w] * (int64_t)dim[w]) can = false;
            if (can) {
                dim[w] *= dim[d];
            } else {
                w--;
                dim[w] = dim[d];
                for (int k = 0; k < 3; k++) st[k][w] = st[k][d];
            }
        }
        int shift = w;
        nd -= shift;
        for (int d = 0; d < nd; d++) {
            dim[d] = dim[d + shift];
            for (int k = 0; k < 3; k++) st[k][d] = st[k][d + shift];
        }
    }
    if (nd == 0) {  // scalar
        nd = 1;
        dim[0] = 1;
        st[0][0] = 1;
        st[1][0] = st[2][0] = 0;
    }
    const int vec = (int)(16 / in_size);
    const int q = nd - 1;
    auto unit_or_zero = [&](int k) { return st[k][q] == 0 || st[k][q] == 1; };
    bool inputs_direct = unit_or_zero(1) && (nin == 1 || unit_or_zero(2));

    // ---- flat ------------------------------------------------------------------------
    if (nd == 1 && st[0][0] == 1 && inputs_direct) {
        bool ok = aligned_to(ptr[0], pl.off[0], esz[0], vec * esz[0]);
        for (int k = 1; k < nop; k++)
            if (st[k][0] == 1 && !aligned_to(ptr[k], pl.off[k], esz[k], 16)) ok = false;
        // every operand element-aligned (always true for typed pointers handed over by a sane caller): misaligned
        // flat operands take the shifted form of the flat kernel instead of the per-element gather
        bool elem_ok = true;
        for (int k = 0; k < nop; k++)
            if (!aligned_to(ptr[k], pl.off[k], esz[k], esz[k])) elem_ok = false;
        if (ok || elem_ok) {
            pl.nd = 1;
            pl.dim[0] = (uint32_t)std::min<uint64_t>(dim[0], 0xFFFFFFFFull);
            for (int k = 0; k < 3; k++) pl.st[k][0] = st[k][0];
            pl.kind = ok ? EW_FLAT : EW_FLAT_SHIFT;
            pl.vec = true;
            return;
        }
    }
    // ---- everything below indexes with 32-bit logical coordinates ---------------------
    if (num_els > 0xFFFFFFFFull || !fits_generic(nd)) {
        std::memcpy(dim, dim_raw, sizeof(dim));
        std::memcpy(st, st_raw, sizeof(st));
        nd = nd_raw;
        if (!fits_generic(nd)) {
            pl.kind = EW_ERROR;
            return;
        }
        store(nd);
        pl.kind = EW_GENERIC;
        return;
    }
    store(nd);
    // ---- row -------------------------------------------------------------------------
    if (st[0][q] == 1 && inputs_direct && dim[q] % vec == 0) {
        bool ok = true;
        for (int k = 0; k < nop; k++) {
            if (st[k][q] != 1) continue;
            if (!aligned_to(ptr[k], pl.off[k], esz[k], vec * esz[k])) ok = false;
            for (int d = 0; d < q; d++)
                if (st[k][d] % vec != 0) ok = false;
        }
        if (ok) {
            pl.kind = EW_ROW;
            pl.vec = true;
            return;
        }
    }
    // ---- tile ------------------------------------------------------------------------
    if (st[0][q] == 1 && !inputs_direct && nd >= 2) {
        int p = -1;
        bool ok = true;
        for (int k = 1; k < nop; k++) {
            pl.transposed[k] = false;
            if (unit_or_zero(k)) continue;
            int pk = -1;
            for (int d = 0; d < q; d++)
                if (st[k][d] == 1) pk = d;
            if (pk < 0 || (p >= 0 && pk != p)) ok = false;
            p = pk;
            pl.transposed[k] = true;
        }
        if (ok && p >= 0 && dim[p] >= 8 && dim[q] >= 8) {
            const int tile = in_size == 8 ? 32 : 64;
            uint64_t blocks = ((dim[p] + tile - 1) / tile) * ((dim[q] + tile - 1) / tile);
            for (int d = 0; d < nd; d++)
                if (d != p && d != q) blocks *= dim[d];
            if (blocks < 0x7FFFFFFFull) {
                bool v = dim[p] % vec == 0 && dim[q] % vec == 0;
                for (int k = 0; k < nop && v; k++) {
                    int unit = pl.transposed[k] ? p : q;
                    if (k != 0 && !pl.transposed[k] && st[k][q] == 0) continue;  // scalar loads only
                    if (!aligned_to(ptr[k], pl.off[k], esz[k], vec * esz[k])) v = false;
                    for (int d = 0; d < nd; d++)
                        if (d != unit && st[k][d] % vec != 0) v = false;
                }
                pl.kind = EW_TILE;
                pl.p = p;
                pl.vec = v;
                return;
            }
        }
    }
    pl.kind = EW_GENERIC;
}

void ew_fill_row_params(const EwPlan& pl, int vec, EwRowParams& P) {
    const int q = pl.nd - 1;
    P.nd_outer = q;
    P.total_vecs = (uint32_t)(pl.n / vec);
    P.qv = pl.dim[q] / vec;
    P.chunks_per_row = (P.qv + kEwThreads * kEwUnroll - 1) / (kEwThreads * kEwUnroll);
    P.qv_div.init(P.qv);
    P.chunk_div.init(P.chunks_per_row);
    for (int d = 0; d < q; d++) {
        P.outer_div[d].init(pl.dim[d]);
        for (int k = 0; k < 3; k++) P.st[k][d] = pl.st[k][d];
    }
    for (int k = 0; k < 3; k++) P.sq[k] = (int)pl.st[k][q];
}

void ew_fill_tile_params(const EwPlan& pl, int tile, EwTileParams& P, uint32_t& blocks) {
    const int q = pl.nd - 1, p = pl.p;
    P.P = pl.dim[p];
    P.Q = pl.dim[q];
    P.tiles_p = (P.P + tile - 1) / tile;
    P.tiles_q = (P.Q + tile - 1) / tile;
    P.tiles_q_div.init(P.tiles_q);
    P.tiles_p_div.init(P.tiles_p);
    P.nd_batch = 0;
    uint64_t nb = 1;
    for (int d = 0; d < pl.nd; d++) {
        if (d == p || d == q) continue;
        P.batch_div[P.nd_batch].init(pl.dim[d]);
        for (int k = 0; k < 3; k++) P.st_batch[k][P.nd_batch] = pl.st[k][d];
        P.nd_batch++;
        nb *= pl.dim[d];
    }
    for (int k = 0; k < 3; k++) {
        P.st_p[k] = pl.st[k][p];
        P.st_q[k] = pl.st[k][q];
        P.transposed[k] = pl.transposed[k] ? 1 : 0;
    }
    P.smem_slot[0] = 0;
    P.smem_slot[1] = 0;
    P.smem_slot[2] = pl.transposed[1] ? 1 : 0;
    blocks = (uint32_t)(nb * P.tiles_p * P.tiles_q);
}

void ew_fill_gen_params(const EwPlan& pl, EwGenParams& P) {
    P.nd = pl.nd;
    P.n = pl.n;
    for (int d = 0; d < pl.nd; d++) {
        P.dim[d] = pl.dim[d];
        P.div[d].init(pl.dim[d]);
        for (int k = 0; k < 3; k++) P.st[k][d] = pl.st[k][d];
    }
}

}  // namespace mx

// Host-only view of the planner for tests that run without a GPU: which kernel class a call would take.
// metadata is HOST memory in the layout of the op family (binary: [dims | lhs strides | rhs strides | offsets],
// unary: [dims | strides | offset]); returns the EwKind (0 empty, 1 flat, 2 row, 3 tile, 4 generic,
// 5 serial, 6 error, 7 flat with shifted loads) and writes the merged rank, the vector flag and the tile's transposed-operand mask.
extern "C" int mx_debug_elementwise_plan(size_t num_els, size_t num_dims, const size_t* host_metadata, int num_inputs, int inplace,
                                         size_t elem_size, size_t out_elem_size, const void* out, const void* a, const void* b, int* merged_rank,
                                         int* vector_ok, int* transposed_mask) {
    mx::EwPlan pl;
    mx::ew_make_plan(pl, num_els, num_dims, host_metadata, num_inputs, inplace != 0, elem_size, out_elem_size, out, a, b);
    if (merged_rank) *merged_rank = pl.nd;
    if (vector_ok) *vector_ok = pl.vec ? 1 : 0;
    if (transposed_mask) *transposed_mask = pl.kind == mx::EW_TILE ? ((pl.transposed[1] ? 1 : 0) | (pl.transposed[2] ? 2 : 0)) : 0;
    return pl.kind;
}
