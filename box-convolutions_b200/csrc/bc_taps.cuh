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

// Integer tap offsets (relative to the pixel) and fractional weights of one box, plus the
// normalisation factor applied to the gathered value.
struct BoxTaps {
    int lo_r, hi_r, lo_c, hi_c;     // rows: taps lo_r-1, lo_r, hi_r, hi_r+1; columns likewise
    float f_lo_r, f_hi_r, f_lo_c, f_hi_c;
    float scale;                    // 1/area when normalising, else 1
};

BC_HD int clampi(int v, int lo, int hi) { return v < lo ? lo : (v > hi ? hi : v); }

// Reciprocal of the box area (or of one side), src/box_convolution.cpp:765-793.  In rounded
// mode the box is first shrunk to whole pixels.
BC_HD float inv_area(float xmin, float xmax, float ymin, float ymax, bool exact, bool use_x, bool use_y)
{
    if (!exact) { xmin = ceilf(xmin); ymin = ceilf(ymin); xmax = floorf(xmax); ymax = floorf(ymax); }
    float a = 1.0f;
    if (use_x) { float len = xmax - xmin; len += 1.0f; a *= len; }
    if (use_y) { float len = ymax - ymin; len += 1.0f; a *= len; }
    return 1.0f / a;
}

// Forward split, src/box_convolution.cpp:14-40.  Rounded mode keeps the integer taps and drops
// the fractions (src/box_convolution_cuda_forward.cu:28-70).
BC_HD BoxTaps taps_forward(float xmin, float xmax, float ymin, float ymax, bool normalize, bool exact)
{
    BoxTaps t;
    float v;
    v = ceilf(xmin);  t.lo_r = (int)v;      t.f_lo_r = v - xmin;
    v = ceilf(ymin);  t.lo_c = (int)v;      t.f_lo_c = v - ymin;
    v = floorf(xmax); t.hi_r = (int)v + 1;  t.f_hi_r = xmax - v;
    v = floorf(ymax); t.hi_c = (int)v + 1;  t.f_hi_c = ymax - v;
    if (!exact) t.f_lo_r = t.f_lo_c = t.f_hi_r = t.f_hi_c = 0.0f;
    t.scale = normalize ? inv_area(xmin, xmax, ymin, ymax, exact, true, true) : 1.0f;
    return t;
}

// Split of the mirrored box [-max, -min] that grad-input gathers with over the integral image
// of grad_output, src/box_convolution.cpp:43-69.
BC_HD BoxTaps taps_mirrored(float xmin, float xmax, float ymin, float ymax, bool normalize, bool exact)
{
    BoxTaps t;
    float v;
    v = ceilf(-xmax);         t.lo_r = (int)v;  t.f_lo_r = v + xmax;
    v = ceilf(-ymax);         t.lo_c = (int)v;  t.f_lo_c = v + ymax;
    v = floorf(-xmin) + 1.0f; t.hi_r = (int)v;  t.f_hi_r = -xmin + 1.0f - v;
    v = floorf(-ymin) + 1.0f; t.hi_c = (int)v;  t.f_hi_c = -ymin + 1.0f - v;
    if (!exact) t.f_lo_r = t.f_lo_c = t.f_hi_r = t.f_hi_c = 0.0f;
    t.scale = normalize ? inv_area(xmin, xmax, ymin, ymax, exact, true, true) : 1.0f;
    return t;
}

// The ten clamped column indices a 4-column strip starting at column q0 reads in every tap row.
struct StripCols {
    int lo[kStrip + 1];   // columns q0+lo_c-1 .. q0+lo_c+3, clamped to [0, w]
    int hi[kStrip + 1];   // columns q0+hi_c   .. q0+hi_c+4, clamped to [0, w]
};

BC_HD StripCols strip_cols(const BoxTaps &t, int q0, int w)
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
struct RowD {
    float d[kStrip];
};

// Same, plus the one-column strips just outside the box on either side (needed by the
// parameter gradients): e_lo[c] = I[lo(c)] - I[lo(c)-1], e_hi[c] = I[hi(c)+1] - I[hi(c)].
struct RowDE {
    float d[kStrip], e_lo[kStrip], e_hi[kStrip];
};

template <class RowPtr>
BC_HD RowD load_row_d(RowPtr row, const StripCols &s, const BoxTaps &t)
{
    float vl[kStrip + 1], vh[kStrip + 1];
#pragma unroll
    for (int m = 0; m <= kStrip; ++m) { vl[m] = row[s.lo[m]]; vh[m] = row[s.hi[m]]; }
    RowD r;
    const float wh = 1.0f - t.f_hi_c, wl = 1.0f - t.f_lo_c;
#pragma unroll
    for (int c = 0; c < kStrip; ++c)
        r.d[c] = wh * vh[c] + t.f_hi_c * vh[c + 1] - wl * vl[c + 1] - t.f_lo_c * vl[c];
    return r;
}

template <class RowPtr>
BC_HD RowDE load_row_de(RowPtr row, const StripCols &s, const BoxTaps &t)
{
    float vl[kStrip + 1], vh[kStrip + 1];
#pragma unroll
    for (int m = 0; m <= kStrip; ++m) { vl[m] = row[s.lo[m]]; vh[m] = row[s.hi[m]]; }
    RowDE r;
    const float wh = 1.0f - t.f_hi_c, wl = 1.0f - t.f_lo_c;
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
BC_HD float combine_rows(float a, float b, float c, float d, float f_lo, float f_hi)
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
struct ParamSums {
    float s_out, s_top, s_bot, s_left, s_right;
};
constexpr int kNumSums = 5;

// Final parameter gradients from the five sums, src/box_convolution_interface.cpp:343-391:
// integrand sums times 1/area, plus (when normalising) the derivative of 1/area times
// sum(grad_output * output), times the reparametrization factor.
BC_HD void finish_param_grads(const ParamSums &s, float xmin, float xmax, float ymin, float ymax,
                              bool normalize, bool exact, float rep_h, float rep_w, float g[4])
{
    float ia = 1.0f, second_x = 0.0f, second_y = 0.0f;
    if (normalize) {
        ia = inv_area(xmin, xmax, ymin, ymax, exact, true, true);
        const float go_out = s.s_out * ia;   // sum(grad_output * output)
        second_x = go_out * inv_area(xmin, xmax, ymin, ymax, exact, true, false);
        second_y = go_out * inv_area(xmin, xmax, ymin, ymax, exact, false, true);
    }
    g[0] = (-s.s_bot * ia + second_x) * rep_h;    // x_min
    g[1] = (s.s_top * ia - second_x) * rep_h;     // x_max
    g[2] = (-s.s_right * ia + second_y) * rep_w;  // y_min
    g[3] = (s.s_left * ia - second_y) * rep_w;    // y_max
}

}  // namespace bc
