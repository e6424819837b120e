// The per-thread walks down a 4-column strip (see bc_taps.cuh for the scheme).
//
// `Rows` is any callable a -> indexable row of the integral image (row a of a padded
// (h+1) x (w+1) plane, wherever it lives: global memory, shared memory, a host array).
#pragma once
#include "bc_taps.cuh"

namespace bc {

// Forward gather for rows [p0, p1) of one strip.  emit(p, o) receives the 4 output values of
// row p (already multiplied by the box's scale).
template <typename T, class Rows, class Emit>
BC_HD void walk_forward(const Rows &rows, const BoxTapsT<T> &t, const StripCols &sc, int p0, int p1,
                        int h, Emit &&emit)
{
    RowDT<T> a = load_row_d(rows(clampi(p0 + t.lo_r - 1, 0, h)), sc, t);
    RowDT<T> c = load_row_d(rows(clampi(p0 + t.hi_r, 0, h)), sc, t);
    for (int p = p0; p < p1; ++p) {
        const RowDT<T> b = load_row_d(rows(clampi(p + t.lo_r, 0, h)), sc, t);
        const RowDT<T> d = load_row_d(rows(clampi(p + t.hi_r + 1, 0, h)), sc, t);
        T o[kStrip];
#pragma unroll
        for (int k = 0; k < kStrip; ++k)
            o[k] = combine_rows(a.d[k], b.d[k], c.d[k], d.d[k], t.f_lo_r, t.f_hi_r) * t.scale;
        emit(p, o);
        a = b;
        c = d;
    }
}

// Backward walk over integral(grad_output plane) with the mirrored box `t`.
//   xval(p, k)   -> input value at row p, column q0+k of the strip (0 outside the plane)
//   gin(p, k)    -> reference to the grad-input accumulator of that pixel
// Adds this filter's contribution to the accumulators and to the five sums.
template <typename T, class Rows, class XVal, class GinRef>
BC_HD void walk_backward(const Rows &rows, const BoxTapsT<T> &t, const StripCols &sc, int p0, int p1,
                         int h, XVal &&xval, GinRef &&gin, ParamSumsT<T> &sums)
{
    RowDET<T> a = load_row_de(rows(clampi(p0 + t.lo_r - 1, 0, h)), sc, t);
    RowDET<T> c = load_row_de(rows(clampi(p0 + t.hi_r, 0, h)), sc, t);
    for (int p = p0; p < p1; ++p) {
        const RowDET<T> b = load_row_de(rows(clampi(p + t.lo_r, 0, h)), sc, t);
        const RowDET<T> d = load_row_de(rows(clampi(p + t.hi_r + 1, 0, h)), sc, t);
#pragma unroll
        for (int k = 0; k < kStrip; ++k) {
            const T top = b.d[k] - a.d[k];
            const T bot = d.d[k] - c.d[k];
            const T g = (c.d[k] - b.d[k]) + t.f_hi_r * bot + t.f_lo_r * top;
            const T sl = combine_rows(a.e_lo[k], b.e_lo[k], c.e_lo[k], d.e_lo[k], t.f_lo_r, t.f_hi_r);
            const T sr = combine_rows(a.e_hi[k], b.e_hi[k], c.e_hi[k], d.e_hi[k], t.f_lo_r, t.f_hi_r);
            const T xv = xval(p, k);
            sums.s_out += xv * g;
            sums.s_top += xv * top;
            sums.s_bot += xv * bot;
            sums.s_left += xv * sl;
            sums.s_right += xv * sr;
            gin(p, k) += g * t.scale;
        }
        a = b;
        c = d;
    }
}

}  // namespace bc
