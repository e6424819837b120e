/*
 * CPU restatement of the box-convolution hot path, in plain C.
 *
 * TEST INFRASTRUCTURE ONLY: this file is the checker that the parity tests, the smoke check
 * and the CPU-baseline leg of the benchmark compare the CUDA library against.  The product
 * library never links, loads or calls it.
 *
 * Parity status: PINNED.  The reference project holds no golden vectors for this path; the
 * pin is the reference's own CPU extension compiled from its sources (oracle/build_ref.py)
 * and the fixtures under tests/golden/ that were generated with it
 * (tests/golden/make_golden.py).  Forward, grad-input and the integral image agree with that
 * build bit for bit; parameter gradients agree to fp32 summation-order noise because the
 * reference finishes them with ATen tree reductions, restated here as double sums.
 *
 * Conventions (same as the reference): the "x" axis is rows/height, "y" is columns/width.
 * An integral image I of an h x w plane has (h+1) x (w+1) entries, row 0 and column 0 zero,
 * I[a][b] = sum of in[p][q] over p < a, q < b.  Box parameters are in actual pixels, one
 * (x_min, x_max, y_min, y_max) per (input plane c, filter f), index k = c*F + f.
 *
 * Each function names the reference source (path within its project : lines) it follows.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

static inline int clampi(int v, int lo, int hi) { return v < lo ? lo : (v > hi ? hi : v); }

/* Zero-padded inclusive 2-D prefix sum.  src/integral_image.cpp:8-39: the running sum along a
 * row is kept in double (ATen's acc_type of float on the CPU), added to the fp32 entry above
 * and rounded to fp32 on store. */
void orc_integral_image(const float *in, float *out, int64_t planes, int h, int w)
{
    const int pw = w + 1;
    for (int64_t p = 0; p < planes; ++p) {
        const float *src = in + p * (int64_t)h * w;
        float *dst = out + p * (int64_t)(h + 1) * pw;
        memset(dst, 0, sizeof(float) * pw);
        for (int r = 0; r < h; ++r) {
            float *cur = dst + (int64_t)(r + 1) * pw;
            const float *above = dst + (int64_t)r * pw;
            double run = 0.0;
            cur[0] = 0.0f;
            for (int c = 0; c < w; ++c) {
                run += src[(int64_t)r * w + c];
                cur[c + 1] = (float)(run + above[c + 1]);
            }
        }
    }
}

typedef struct {
    int xmin_i, xmax_i, ymin_i, ymax_i;
    float xmin_f, xmax_f, ymin_f, ymax_f;
} split_t;

/* src/box_convolution.cpp:14-40 -- split used by the forward gather. */
static split_t split_forward(float xmin, float xmax, float ymin, float ymax)
{
    split_t s;
    float t;
    t = ceilf(xmin);  s.xmin_f = t - xmin;  s.xmin_i = (int)t;
    t = ceilf(ymin);  s.ymin_f = t - ymin;  s.ymin_i = (int)t;
    t = floorf(xmax); s.xmax_f = xmax - t;  s.xmax_i = (int)t + 1;
    t = floorf(ymax); s.ymax_f = ymax - t;  s.ymax_i = (int)t + 1;
    return s;
}

/* src/box_convolution.cpp:43-69 -- split of the mirrored box [-max, -min] used for grad-input. */
static split_t split_grad_input(float xmin, float xmax, float ymin, float ymax)
{
    split_t s;
    float t;
    t = ceilf(-xmax);       s.xmin_f = t + xmax;          s.xmin_i = (int)t;
    t = ceilf(-ymax);       s.ymin_f = t + ymax;          s.ymin_i = (int)t;
    t = floorf(-xmin) + 1;  s.xmax_f = -xmin + 1 - t;     s.xmax_i = (int)t;
    t = floorf(-ymin) + 1;  s.ymax_f = -ymin + 1 - t;     s.ymax_i = (int)t;
    return s;
}

/* src/box_convolution.cpp:72-98 -- split used for the parameter gradients. */
static split_t split_grad_params(float xmin, float xmax, float ymin, float ymax)
{
    split_t s;
    float t;
    t = ceilf(xmin - 1);  s.xmin_f = t - xmin + 1;  s.xmin_i = (int)t;
    t = ceilf(ymin - 1);  s.ymin_f = t - ymin + 1;  s.ymin_i = (int)t;
    t = floorf(xmax);     s.xmax_f = xmax - t;      s.xmax_i = (int)t;
    t = floorf(ymax);     s.ymax_f = ymax - t;      s.ymax_i = (int)t;
    return s;
}

/* src/box_convolution.cpp:765-793 -- reciprocal of the box area (or of one side length).
 * In rounded mode the box is first shrunk to whole pixels. */
static float inv_area(float xmin, float xmax, float ymin, float ymax, int exact, int use_x, int use_y)
{
    float a = 1.0f;
    if (!exact) { xmin = ceilf(xmin); ymin = ceilf(ymin); xmax = floorf(xmax); ymax = floorf(ymax); }
    if (use_x) { float len = xmax - xmin; len += 1; a *= len; }
    if (use_y) { float len = ymax - ymin; len += 1; a *= len; }
    return 1.0f / a;
}

#define AT(I, pitch, r, c) ((I)[(int64_t)(r) * (pitch) + (c)])

/* One output value of the gather shared by forward and grad-input in the reference's forward
 * formulation.  src/box_convolution.cpp:157-254 (term order kept, so results are bit-equal). */
static inline float gather_forward(const float *I, int h, int w, int x, int y, const split_t *s, int exact)
{
    const int pw = w + 1;
    const int t = clampi(x + s->xmin_i, 0, h), b = clampi(x + s->xmax_i, 0, h);
    const int l = clampi(y + s->ymin_i, 0, w), r = clampi(y + s->ymax_i, 0, w);
    float v = AT(I, pw, b, r) - AT(I, pw, t, r) - AT(I, pw, b, l) + AT(I, pw, t, l);
    if (!exact) return v;

    const int bA = clampi(x + s->xmax_i + 1, 0, h), rA = clampi(y + s->ymax_i + 1, 0, w);
    const int tA = clampi(x + s->xmin_i - 1, 0, h), lA = clampi(y + s->ymin_i - 1, 0, w);
    /* one-pixel-thick strips beyond each edge, weighted by the fractional parts */
    v += (AT(I, pw, bA, r) - AT(I, pw, b, r) - AT(I, pw, bA, l) + AT(I, pw, b, l)) * s->xmax_f;
    v += (AT(I, pw, b, rA) - AT(I, pw, b, r) - AT(I, pw, t, rA) + AT(I, pw, t, r)) * s->ymax_f;
    v += (AT(I, pw, t, r) - AT(I, pw, tA, r) - AT(I, pw, t, l) + AT(I, pw, tA, l)) * s->xmin_f;
    v += (AT(I, pw, b, l) - AT(I, pw, b, lA) - AT(I, pw, t, l) + AT(I, pw, t, lA)) * s->ymin_f;
    /* single corner pixels; guards look at the unclamped coordinates */
    const int xb = x + s->xmax_i, xt = x + s->xmin_i, yr = y + s->ymax_i, yl = y + s->ymin_i;
    if (!(xb >= h || yr >= w || xb < 0 || yr < 0))
        v += s->xmax_f * s->ymax_f *
             (AT(I, pw, b + 1, r + 1) - AT(I, pw, b, r + 1) - AT(I, pw, b + 1, r) + AT(I, pw, b, r));
    if (!(xt > h || yr >= w || xt <= 0 || yr < 0))
        v += s->xmin_f * s->ymax_f *
             (AT(I, pw, t, r + 1) - AT(I, pw, t - 1, r + 1) - AT(I, pw, t, r) + AT(I, pw, t - 1, r));
    if (!(xb >= h || yl > w || xb < 0 || yl <= 0))
        v += s->xmax_f * s->ymin_f *
             (AT(I, pw, b + 1, l) - AT(I, pw, b, l) - AT(I, pw, b + 1, l - 1) + AT(I, pw, b, l - 1));
    if (!(xt > h || yl > w || xt <= 0 || yl <= 0))
        v += s->xmin_f * s->ymin_f *
             (AT(I, pw, t, l) - AT(I, pw, t - 1, l) - AT(I, pw, t, l - 1) + AT(I, pw, t - 1, l - 1));
    return v;
}

/* box_convolution_forward: src/box_convolution_interface.cpp:13-139 driving
 * src/box_convolution.cpp:100-261.  integ is (N, C, h+1, w+1); out is (N, C, F, h, w). */
void orc_box_convolution_forward(const float *integ, const float *x_min, const float *x_max,
                                 const float *y_min, const float *y_max, float *out,
                                 int N, int C, int F, int h, int w, int normalize, int exact)
{
    const int64_t ipl = (int64_t)(h + 1) * (w + 1), opl = (int64_t)h * w;
    for (int n = 0; n < N; ++n)
        for (int c = 0; c < C; ++c) {
            const float *I = integ + ((int64_t)n * C + c) * ipl;
            for (int f = 0; f < F; ++f) {
                const int k = c * F + f;
                split_t s = split_forward(x_min[k], x_max[k], y_min[k], y_max[k]);
                const float scale = normalize ? inv_area(x_min[k], x_max[k], y_min[k], y_max[k], exact, 1, 1) : 1.0f;
                float *o = out + (((int64_t)n * C + c) * F + f) * opl;
                for (int x = 0; x < h; ++x)
                    for (int y = 0; y < w; ++y)
                        o[(int64_t)x * w + y] = gather_forward(I, h, w, x, y, &s, exact) * scale;
            }
        }
}

/* One value of the mirrored-box gather over integral(grad_output).
 * src/box_convolution.cpp:334-449 (its own clamping of the advanced taps and corner guards). */
static inline float gather_grad_input(const float *G, int h, int w, int x, int y, const split_t *s, int exact)
{
    const int pw = w + 1;
    const int xt = x + s->xmin_i, xb = x + s->xmax_i, yl = y + s->ymin_i, yr = y + s->ymax_i;
    const int t = clampi(xt, 0, h), b = clampi(xb, 0, h), l = clampi(yl, 0, w), r = clampi(yr, 0, w);
    float v = AT(G, pw, b, r) - AT(G, pw, t, r) - AT(G, pw, b, l) + AT(G, pw, t, l);
    if (!exact) return v;

    const int tA = xt - 1 < h ? clampi(t - 1, 0, h) : t;
    const int bA = xb >= 0 ? clampi(b + 1, 0, h) : b;
    const int lA = yl - 1 < w ? clampi(l - 1, 0, w) : l;
    const int rA = yr >= 0 ? clampi(r + 1, 0, w) : r;
    v += (AT(G, pw, bA, r) - AT(G, pw, b, r) - AT(G, pw, bA, l) + AT(G, pw, b, l)) * s->xmax_f;
    v += (AT(G, pw, b, rA) - AT(G, pw, b, r) - AT(G, pw, t, rA) + AT(G, pw, t, r)) * s->ymax_f;
    v += (AT(G, pw, t, r) - AT(G, pw, tA, r) - AT(G, pw, t, l) + AT(G, pw, tA, l)) * s->xmin_f;
    v += (AT(G, pw, b, l) - AT(G, pw, b, lA) - AT(G, pw, t, l) + AT(G, pw, t, lA)) * s->ymin_f;

    float corner;
    corner = (xb >= h || yr >= w || xb < 0 || yr < 0 || b == bA || r == rA) ? 0.0f :
             (AT(G, pw, b + 1, r + 1) - AT(G, pw, b, r + 1) - AT(G, pw, b + 1, r) + AT(G, pw, b, r));
    v += s->xmax_f * s->ymax_f * corner;
    corner = (xt > h || yr >= w || xt <= 0 || yr < 0 || t == tA || r == rA) ? 0.0f :
             (AT(G, pw, tA + 1, r + 1) - AT(G, pw, tA + 1, r) - AT(G, pw, tA, r + 1) + AT(G, pw, tA, r));
    v += s->xmin_f * s->ymax_f * corner;
    corner = (xb >= h || yl > w || xb < 0 || yl <= 0 || b == bA || l == lA) ? 0.0f :
             (AT(G, pw, b + 1, lA + 1) - AT(G, pw, b, lA + 1) - AT(G, pw, b + 1, lA) + AT(G, pw, b, lA));
    v += s->xmax_f * s->ymin_f * corner;
    corner = (xt > h || yl > w || xt <= 0 || yl <= 0 || t == tA || l == lA) ? 0.0f :
             (AT(G, pw, tA + 1, lA + 1) - AT(G, pw, tA + 1, lA) - AT(G, pw, tA, lA + 1) + AT(G, pw, tA, lA));
    v += s->xmin_f * s->ymin_f * corner;
    return v;
}

/* Per-pixel integrand of d(un-normalised box sum)/d(parameter), src/box_convolution.cpp:524-709.
 * x and y are the reference's 1-based pixel coordinates. which: 0 xMin, 1 xMax, 2 yMin, 3 yMax
 * (src/box_convolution.h:3). */
static inline float pixel1(const float *I, int pw, int cx, int cy)
{
    return AT(I, pw, cx + 1, cy + 1) - AT(I, pw, cx, cy + 1) - AT(I, pw, cx + 1, cy) + AT(I, pw, cx, cy);
}

static inline float param_integrand(const float *I, int h, int w, int x, int y, const split_t *s,
                                    int exact, int which)
{
    const int pw = w + 1;
    const int xi = x + s->xmin_i, xa = x + s->xmax_i, yi = y + s->ymin_i, ya = y + s->ymax_i;
    float d = 0.0f;
    if (which == 0 || which == 1) {
        /* a one-row strip: the image row just above the box (xMin) or just below it (xMax) */
        const int row_hi = which == 0 ? xi : xa + 1;     /* integral rows row_hi-1 .. row_hi */
        if (exact) {
            const int edge_ok = which == 0 ? !(xi < 1) : !(xa >= h);
            const int cx = clampi(row_hi - 1, 0, h - 1);
            const int okl = !(yi < 1) & !(yi > w) & edge_ok;
            const float left = okl * pixel1(I, pw, cx, clampi(yi - 1, 0, w - 1));
            const int okr = !(ya < 0) & !(ya >= w) & edge_ok;
            const float right = okr * pixel1(I, pw, cx, clampi(ya, 0, w - 1));
            d += right * s->ymax_f;
            d += left * s->ymin_f;
        }
        d += AT(I, pw, clampi(row_hi, 0, h), clampi(ya, 0, w));
        d -= AT(I, pw, clampi(row_hi - 1, 0, h), clampi(ya, 0, w));
        d -= AT(I, pw, clampi(row_hi, 0, h), clampi(yi, 0, w));
        d += AT(I, pw, clampi(row_hi - 1, 0, h), clampi(yi, 0, w));
        if (which == 0) { d *= (float)((xi >= 1) & (xi <= h)); return -d; }
        d *= (float)((xa >= 0) & (xa < h));
        return d;
    } else {
        /* a one-column strip left of the box (yMin) or right of it (yMax) */
        const int col_hi = which == 2 ? yi : ya + 1;
        if (exact) {
            const int edge_ok = which == 2 ? !(yi < 1) : !(ya >= w);
            const int cy = clampi(col_hi - 1, 0, w - 1);
            const int okt = edge_ok & !(xi < 1) & !(xi > h);
            const float top = okt * pixel1(I, pw, clampi(xi - 1, 0, h - 1), cy);
            const int okb = edge_ok & !(xa < 0) & !(xa >= h);
            const float bottom = okb * pixel1(I, pw, clampi(xa, 0, h - 1), cy);
            d += top * s->xmin_f;
            d += bottom * s->xmax_f;
        }
        d += AT(I, pw, clampi(xa, 0, h), clampi(col_hi, 0, w));
        d -= AT(I, pw, clampi(xa, 0, h), clampi(col_hi - 1, 0, w));
        d -= AT(I, pw, clampi(xi, 0, h), clampi(col_hi, 0, w));
        d += AT(I, pw, clampi(xi, 0, h), clampi(col_hi - 1, 0, w));
        if (which == 2) { d *= (float)((yi >= 1) & (yi <= w)); return -d; }
        d *= (float)((ya >= 0) & (ya < w));
        return d;
    }
}

/* box_convolution_backward: src/box_convolution_interface.cpp:141-395.
 *   integ        (N, C, h+1, w+1)   integral image of the input
 *   grad_output  (N, C, F, h, w)
 *   output       (N, C, F, h, w)    forward result; read only when normalize (may be NULL otherwise)
 *   grad_input   (N, C, h, w)       written when need_mask bit 0 is set
 *   grad_params  4 arrays of C*F    written when need_mask bits 1..4 are set (xMin, xMax, yMin, yMax)
 * The reference finishes the reductions with ATen sum kernels in fp32; here products are rounded
 * to fp32 exactly as the reference's mul_ does and then summed in double, and the remaining
 * scalar steps are carried out in fp32 in the reference's order. */
void orc_box_convolution_backward(const float *integ, const float *x_min, const float *x_max,
                                  const float *y_min, const float *y_max, const float *grad_output,
                                  const float *output, float rep_h, float rep_w,
                                  int N, int C, int F, int h, int w, int normalize, int exact,
                                  int need_mask, float *grad_input, float *const *grad_params)
{
    const int64_t ipl = (int64_t)(h + 1) * (w + 1), opl = (int64_t)h * w;

    if (need_mask & 1) {
        /* interface.cpp:198-275 -- integrate grad_output per (n,c,f) plane, gather with the
         * mirrored box, then sum over the filters (tmpArray.sum(2)) */
        float *gint = (float *)malloc(sizeof(float) * ipl);
        double *acc = (double *)malloc(sizeof(double) * opl);
        for (int n = 0; n < N; ++n)
            for (int c = 0; c < C; ++c) {
                for (int64_t i = 0; i < opl; ++i) acc[i] = 0.0;
                for (int f = 0; f < F; ++f) {
                    const int k = c * F + f;
                    const float *g = grad_output + (((int64_t)n * C + c) * F + f) * opl;
                    orc_integral_image(g, gint, 1, h, w);
                    split_t s = split_grad_input(x_min[k], x_max[k], y_min[k], y_max[k]);
                    const float scale = normalize ? inv_area(x_min[k], x_max[k], y_min[k], y_max[k], exact, 1, 1) : 1.0f;
                    for (int x = 0; x < h; ++x)
                        for (int y = 0; y < w; ++y)
                            acc[(int64_t)x * w + y] += (double)(gather_grad_input(gint, h, w, x, y, &s, exact) * scale);
                }
                float *gi = grad_input + ((int64_t)n * C + c) * opl;
                for (int64_t i = 0; i < opl; ++i) gi[i] = (float)acc[i];
            }
        free(gint);
        free(acc);
    }

    if (!(need_mask & 0x1e)) return;

    /* interface.cpp:277-392 */
    double *sum_param = (double *)calloc((size_t)4 * C * F, sizeof(double));
    double *sum_go_out = (double *)calloc((size_t)C * F, sizeof(double));
    for (int n = 0; n < N; ++n)
        for (int c = 0; c < C; ++c) {
            const float *I = integ + ((int64_t)n * C + c) * ipl;
            for (int f = 0; f < F; ++f) {
                const int k = c * F + f;
                split_t s = split_grad_params(x_min[k], x_max[k], y_min[k], y_max[k]);
                const int64_t off = (((int64_t)n * C + c) * F + f) * opl;
                const float *g = grad_output + off;
                for (int which = 0; which < 4; ++which) {
                    if (!(need_mask & (2 << which))) continue;
                    double acc = 0.0;
                    for (int x = 1; x <= h; ++x)
                        for (int y = 1; y <= w; ++y) {
                            const float v = param_integrand(I, h, w, x, y, &s, exact, which) *
                                            g[(int64_t)(x - 1) * w + (y - 1)];
                            acc += (double)v;
                        }
                    sum_param[(int64_t)which * C * F + k] += acc;
                }
                if (normalize) {
                    const float *o = output + off;
                    double acc = 0.0;
                    for (int64_t i = 0; i < opl; ++i) acc += (double)(g[i] * o[i]);
                    sum_go_out[k] += acc;
                }
            }
        }

    for (int which = 0; which < 4; ++which) {
        if (!(need_mask & (2 << which))) continue;
        const int is_x = which < 2;
        for (int k = 0; k < C * F; ++k) {
            float gp = (float)sum_param[(int64_t)which * C * F + k];
            if (normalize) {
                gp *= inv_area(x_min[k], x_max[k], y_min[k], y_max[k], exact, 1, 1);           /* :348-350 */
                const float inv_len = inv_area(x_min[k], x_max[k], y_min[k], y_max[k], exact, is_x, !is_x);
                const float sign = (which == 1 || which == 3) ? -1.0f : 1.0f;                 /* :376-377 */
                gp += sign * ((float)sum_go_out[k] * inv_len);
            }
            gp *= is_x ? rep_h : rep_w;                                                       /* :383-391 */
            grad_params[which][k] = gp;
        }
    }
    free(sum_param);
    free(sum_go_out);
}

/* clip_parameters: src/box_convolution_interface.cpp:397-415 + src/box_convolution.cpp:729-763.
 * In place, on the stored (reparametrized) values, arithmetic in double. */
static void clip_pair(float *pmin, float *pmax, int count, double rep, double min_size, double max_size)
{
    const double inv = 1.0 / rep;
    const double lo = -(max_size + 1) * inv, hi = (max_size - 1) * inv;
    for (int i = 0; i < count; ++i) {
        double a = (double)pmin[i], b = (double)pmax[i];
        a = a > hi ? hi : a; a = a < lo ? lo : a;
        b = b > hi ? hi : b; b = b < lo ? lo : b;
        if (a + (min_size - 0.9999) * inv > b) {
            const float mean = (float)(0.5 * (a + b));   /* the reference rounds the mean to scalar_t */
            a = mean - 0.5 * (min_size - 0.9999) * inv;
            b = mean + 0.5 * (min_size - 0.9999) * inv;
        }
        pmin[i] = (float)a;
        pmax[i] = (float)b;
    }
}

void orc_clip_parameters(float *x_min, float *x_max, float *y_min, float *y_max, int count,
                         double rep_h, double rep_w, double max_h, double max_w, int exact)
{
    const float min_size = exact ? 1.001f : 2.001f;      /* interface.cpp:405-406 (floats) */
    clip_pair(x_min, x_max, count, rep_h, (double)min_size, max_h);
    clip_pair(y_min, y_max, count, rep_w, (double)min_size, max_w);
}
