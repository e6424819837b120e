// Box descriptors and the per-thread "column walk" that every gather kernel is built from.
//
// A box filter with fractional borders is a tensor product: per axis the box touches four
// integral-image taps {lo-1, lo, hi, hi+1} (clamped to the plane) with weights
// {-f_lo, -(1-f_lo), (1-f_hi), f_hi}.  Written that way the reference's main area, its four
// fractional edge strips and its four corner pixels (src/box_convolution.cpp:157-248) are the
// sixteen cross terms, and the reference's corner guards are implied by the clamping: whenever
// a guard fails the two taps of that axis clamp to the same index and the term is zero.
//
// A thread owns a strip of 4 adjacent columns and walks down its rows.  Going from row p to
// p+1 the taps {lo-1, hi} of p+1 are the taps {lo, hi+1} of p, so each step loads only two
// new tap rows and carries the other two in registers; within a tap row the 4 columns share
// their taps (lo of column q is lo-1 of column q+1), so a tap row costs 10 loads for 4 columns.
//
// Everything here is __host__ __device__ so that the arithmetic can also be exercised on a CPU
// by the unit tests.
#pragma once
#include <math.h>

#if defined(__CUDACC__)
#define BC_HD __host__ __device__ __forceinline__
#else
#define BC_HD inline
#endif

namespace bc {

constexpr int kStrip = 4;  // columns per thread

// Scalar type: float on the benchmarked path; double instantiates the general (global-memory)
// kernels for the reference's float64 use (gradient checks).
BC_HD float bc_ceil(float v) { return ceilf(v); }
BC_HD double bc_ceil(double v) { return ceil(v); }
BC_HD float bc_floor(float v) { return floorf(v); }
BC_HD double bc_floor(double v) { return floor(v); }

// Integer tap offsets (relative to the pixel) and fractional weights of one box, plus the
// normalisation factor applied to the gathered value.
template <typename T>
struct BoxTapsT {
    int lo_r, hi_r, lo_c, hi_c;     // rows: taps lo_r-1, lo_r, hi_r, hi_r+1; columns likewise
    T f_lo_r, f_hi_r, f_lo_c, f_hi_c;
    T scale;                        // 1/area when normalising, else 1
};
using BoxTaps = BoxTapsT<float>;

BC_HD int clampi(int v, int lo, int hi) { return v < lo ? lo : (v > hi ? hi : v); }

// Reciprocal of the box area (or of one side), src/box_convolution.cpp:765-793.  In rounded
// mode the box is first shrunk to whole pixels.
template <typename T>
BC_HD T inv_area(T xmin, T xmax, T ymin, T ymax, bool exact, bool use_x, bool use_y)
{
    if (!exact) { xmin = bc_ceil(xmin); ymin = bc_ceil(ymin); xmax = bc_floor(xmax); ymax = bc_floor(ymax); }
    T a = T(1);
    if (use_x) { T len = xmax - xmin; len += T(1); a *= len; }
    if (use_y) { T len = ymax - ymin; len += T(1); a *= len; }
    return T(1) / a;
}

// Forward split, src/box_convolution.cpp:14-40.  Rounded mode keeps the integer taps and drops
// the fractions (src/box_convolution_cuda_forward.cu:28-70).
template <typename T>
BC_HD BoxTapsT<T> taps_forward(T xmin, T xmax, T ymin, T ymax, bool normalize, bool exact)
{
    BoxTapsT<T> t;
    T v;
    v = bc_ceil(xmin);  t.lo_r = (int)v;      t.f_lo_r = v - xmin;
    v = bc_ceil(ymin);  t.lo_c = (int)v;      t.f_lo_c = v - ymin;
    v = bc_floor(xmax); t.hi_r = (int)v + 1;  t.f_hi_r = xmax - v;
    v = bc_floor(ymax); t.hi_c = (int)v + 1;  t.f_hi_c = ymax - v;
    if (!exact) t.f_lo_r = t.f_lo_c = t.f_hi_r = t.f_hi_c = T(0);
    t.scale = normalize ? inv_area(xmin, xmax, ymin, ymax, exact, true, true) : T(1);
    return t;
}

// Split of the mirrored box [-max, -min] that grad-input gathers with over the integral image
// of grad_output, src/box_convolution.cpp:43-69.
template <typename T>
BC_HD BoxTapsT<T> taps_mirrored(T xmin, T xmax, T ymin, T ymax, bool normalize, bool exact)
{
    BoxTapsT<T> t;
    T v;
    v = bc_ceil(-xmax);          t.lo_r = (int)v;  t.f_lo_r = v + xmax;
    v = bc_ceil(-ymax);          t.lo_c = (int)v;  t.f_lo_c = v + ymax;
    v = bc_floor(-xmin) + T(1);  t.hi_r = (int)v;  t.f_hi_r = -xmin + T(1) - v;
    v = bc_floor(-ymin) + T(1);  t.hi_c = (int)v;  t.f_hi_c = -ymin + T(1) - v;
    if (!exact) t.f_lo_r = t.f_lo_c = t.f_hi_r = t.f_hi_c = T(0);
    t.scale = normalize ? inv_area(xmin, xmax, ymin, ymax, exact, true, true) : T(1);
    return t;
}

// The ten clamped column indices a 4-column strip starting at column q0 reads in every tap row.
struct StripCols {
    int lo[kStrip + 1];   // columns q0+lo_c-1 .. q0+lo_c+3, clamped to [0, w]
    int hi[kStrip + 1];   // columns q0+hi_c   .. q0+hi_c+4, clamped to [0, w]
};

template <typename T>
BC_HD StripCols strip_cols(const BoxTapsT<T> &t, int q0, int w)
{
    StripCols s;
#pragma unroll
    for (int m = 0; m <= kStrip; ++m) {
        s.lo[m] = clampi(q0 + t.lo_c - 1 + m, 0, w);
        s.hi[m] = clampi(q0 + t.hi_c + m, 0, w);
    }
    return s;
}

// Column-combined value of one tap row for the 4 columns of a strip:
//   D[c] = (1-f_hi) I[hi(c)] + f_hi I[hi(c)+1] - (1-f_lo) I[lo(c)] - f_lo I[lo(c)-1]
// i.e. the fractional-width box sum of everything above that integral row.
template <typename T>
struct RowDT {
    T d[kStrip];
};
using RowD = RowDT<float>;

// Same, plus the one-column strips just outside the box on either side (needed by the
// parameter gradients): e_lo[c] = I[lo(c)] - I[lo(c)-1], e_hi[c] = I[hi(c)+1] - I[hi(c)].
template <typename T>
struct RowDET {
    T d[kStrip], e_lo[kStrip], e_hi[kStrip];
};
using RowDE = RowDET<float>;

template <typename T, class RowPtr>
BC_HD RowDT<T> load_row_d(RowPtr row, const StripCols &s, const BoxTapsT<T> &t)
{
    T vl[kStrip + 1], vh[kStrip + 1];
#pragma unroll
    for (int m = 0; m <= kStrip; ++m) { vl[m] = row[s.lo[m]]; vh[m] = row[s.hi[m]]; }
    RowDT<T> r;
    const T wh = T(1) - t.f_hi_c, wl = T(1) - t.f_lo_c;
#pragma unroll
    for (int c = 0; c < kStrip; ++c)
        r.d[c] = wh * vh[c] + t.f_hi_c * vh[c + 1] - wl * vl[c + 1] - t.f_lo_c * vl[c];
    return r;
}

template <typename T, class RowPtr>
BC_HD RowDET<T> load_row_de(RowPtr row, const StripCols &s, const BoxTapsT<T> &t)
{
    T vl[kStrip + 1], vh[kStrip + 1];
#pragma unroll
    for (int m = 0; m <= kStrip; ++m) { vl[m] = row[s.lo[m]]; vh[m] = row[s.hi[m]]; }
    RowDET<T> r;
    const T wh = T(1) - t.f_hi_c, wl = T(1) - t.f_lo_c;
#pragma unroll
    for (int c = 0; c < kStrip; ++c) {
        r.d[c] = wh * vh[c] + t.f_hi_c * vh[c + 1] - wl * vl[c + 1] - t.f_lo_c * vl[c];
        r.e_lo[c] = vl[c + 1] - vl[c];
        r.e_hi[c] = vh[c + 1] - vh[c];
    }
    return r;
}

// Row combination of the four tap rows {A = lo-1, B = lo, Cc = hi, Dd = hi+1}:
//   (C - B) + f_hi (D - C) + f_lo (B - A)
template <typename T>
BC_HD T combine_rows(T a, T b, T c, T d, T f_lo, T f_hi)
{
    return (c - b) + f_hi * (d - c) + f_lo * (b - a);
}

// The five per-(plane, filter) sums the parameter gradients are finished from.  With G the
// grad_output plane, X the input plane and the mirrored box gathered over integral(G):
//   s_out  = sum X * gather            ( = sum G * un-normalised forward output )
//   s_top  = sum X * (row strip just outside the lo-row side)   -> d/d x_max
//   s_bot  = sum X * (row strip just outside the hi-row side)   -> d/d x_min
//   s_left = sum X * (column strip outside the lo-column side)  -> d/d y_max
//   s_right= sum X * (column strip outside the hi-column side)  -> d/d y_min
// (the mirrored box's lo side is the original box's max side).
template <typename T>
struct ParamSumsT {
    T s_out, s_top, s_bot, s_left, s_right;
};
using ParamSums = ParamSumsT<float>;
constexpr int kNumSums = 5;

// Final parameter gradients from the five sums, src/box_convolution_interface.cpp:343-391:
// integrand sums times 1/area, plus (when normalising) the derivative of 1/area times
// sum(grad_output * output), times the reparametrization factor.
template <typename T>
BC_HD void finish_param_grads(const ParamSumsT<T> &s, T xmin, T xmax, T ymin, T ymax,
                              bool normalize, bool exact, T rep_h, T rep_w, T g[4])
{
    T ia = T(1), second_x = T(0), second_y = T(0);
    if (normalize) {
        ia = inv_area(xmin, xmax, ymin, ymax, exact, true, true);
        const T go_out = s.s_out * ia;   // sum(grad_output * output)
        second_x = go_out * inv_area(xmin, xmax, ymin, ymax, exact, true, false);
        second_y = go_out * inv_area(xmin, xmax, ymin, ymax, exact, false, true);
    }
    g[0] = (-s.s_bot * ia + second_x) * rep_h;    // x_min
    g[1] = (s.s_top * ia - second_x) * rep_h;     // x_max
    g[2] = (-s.s_right * ia + second_y) * rep_w;  // y_min
    g[3] = (s.s_left * ia - second_y) * rep_w;    // y_max
}

}  // namespace bc
