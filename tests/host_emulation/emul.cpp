// Host build of the strip-walk arithmetic (csrc/bc_taps.cuh, csrc/bc_walk.cuh) so that the unit
// tests can check it against the oracle on a machine without a GPU.  This is a test harness:
// it is compiled by tests/test_walk_host.py only and is not part of the shipped library.
#include <cstdint>
#include <vector>

#include "bc_walk.cuh"

using namespace bc;

extern "C" void emu_forward(const float *integ, const float *xmin, const float *xmax,
                            const float *ymin, const float *ymax, float *out, int N, int C, int F,
                            int h, int w, int normalize, int exact, int rows_per_thread)
{
    const int64_t ipl = (int64_t)(h + 1) * (w + 1), opl = (int64_t)h * w;
    for (int64_t nc = 0; nc < (int64_t)N * C; ++nc)
        for (int f = 0; f < F; ++f) {
            const int k = (int)(nc % C) * F + f;
            const BoxTaps t = taps_forward(xmin[k], xmax[k], ymin[k], ymax[k], normalize, exact);
            const float *I = integ + nc * ipl;
            float *o = out + (nc * F + f) * opl;
            auto rows = [&](int a) { return I + (int64_t)a * (w + 1); };
            for (int q0 = 0; q0 < w; q0 += kStrip) {
                const StripCols sc = strip_cols(t, q0, w);
                for (int p0 = 0; p0 < h; p0 += rows_per_thread) {
                    const int p1 = p0 + rows_per_thread < h ? p0 + rows_per_thread : h;
                    walk_forward(rows, t, sc, p0, p1, h, [&](int p, const float *v) {
                        for (int m = 0; m < kStrip; ++m)
                            if (q0 + m < w) o[(int64_t)p * w + q0 + m] = v[m];
                    });
                }
            }
        }
}

extern "C" void emu_backward(const float *x, const float *gint, const float *xmin,
                             const float *xmax, const float *ymin, const float *ymax, float rep_h,
                             float rep_w, int N, int C, int F, int h, int w, int normalize,
                             int exact, int rows_per_thread, float *grad_input, float *grad_params)
{
    // gint: integral images of the grad_output planes, (N, C, F, h+1, w+1)
    const int64_t ipl = (int64_t)(h + 1) * (w + 1), opl = (int64_t)h * w;
    std::vector<double> acc((size_t)C * F * kNumSums, 0.0);
    for (int64_t i = 0; i < (int64_t)N * C * opl; ++i) grad_input[i] = 0.0f;
    for (int64_t nc = 0; nc < (int64_t)N * C; ++nc)
        for (int f = 0; f < F; ++f) {
            const int k = (int)(nc % C) * F + f;
            const BoxTaps t = taps_mirrored(xmin[k], xmax[k], ymin[k], ymax[k], normalize, exact);
            const float *G = gint + (nc * F + f) * ipl;
            const float *xp = x + nc * opl;
            float *gi = grad_input + nc * opl;
            auto rows = [&](int a) { return G + (int64_t)a * (w + 1); };
            for (int q0 = 0; q0 < w; q0 += kStrip) {
                const StripCols sc = strip_cols(t, q0, w);
                for (int p0 = 0; p0 < h; p0 += rows_per_thread) {
                    const int p1 = p0 + rows_per_thread < h ? p0 + rows_per_thread : h;
                    ParamSums s = {0, 0, 0, 0, 0};
                    float dump;
                    walk_backward(
                        rows, t, sc, p0, p1, h,
                        [&](int p, int m) { return q0 + m < w ? xp[(int64_t)p * w + q0 + m] : 0.0f; },
                        [&](int p, int m) -> float & {
                            dump = 0.0f;
                            return q0 + m < w ? gi[(int64_t)p * w + q0 + m] : dump;
                        },
                        s);
                    double *a = &acc[(size_t)k * kNumSums];
                    a[0] += s.s_out; a[1] += s.s_top; a[2] += s.s_bot; a[3] += s.s_left; a[4] += s.s_right;
                }
            }
        }
    for (int k = 0; k < C * F; ++k) {
        const double *a = &acc[(size_t)k * kNumSums];
        ParamSums s = {(float)a[0], (float)a[1], (float)a[2], (float)a[3], (float)a[4]};
        float g[4];
        finish_param_grads(s, xmin[k], xmax[k], ymin[k], ymax[k], normalize, exact, rep_h, rep_w, g);
        for (int j = 0; j < 4; ++j) grad_params[(size_t)j * C * F + k] = g[j];
    }
}
