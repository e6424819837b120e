// Shared-memory-resident kernels for planes small enough to keep on chip (the 1/8-frame ENet
// shape, 64 x 128, is the design point).  HBM traffic is the compulsory minimum: the forward
// reads the input once and writes the output once; the backward reads the input and grad_output
// once and writes grad_input once.  No integral image ever goes to global memory.
//
// Forward : one CTA per (plane, group of filters).  The plane's integral image is built in shared
//           memory, then every thread walks its 4-column x 8-row strip (bc_walk.cuh scheme) for
//           each filter of the group and writes 128-bit rows of the output.
// Backward: one CTA per plane.  The input plane stays in shared memory; for each filter the
//           grad_output plane is integrated in shared memory and gathered with the mirrored box.
//           Grad-input accumulates in registers over the filters; the five sums that finish the
//           parameter gradients are reduced per CTA and left for finish_param_grads_kernel.
//
// Thread layout (same for building the integral image and for gathering): a warp owns a tile of
// 32 x 32 pixels; lane = 8 column groups (cg, 4 columns each) x 4 row groups (rg, 8 rows each).
//
// Shared-memory layout of the integral image: row a (0..h) starts at a*pitch + a/8 floats and
// holds [4 zeros | I[a][0..w] | 4 copies of I[a][w]].
//   * the padding turns the clamping of the five adjacent column taps of a strip into a clamp of
//     the window start, so a tap row is read with two base addresses and immediate offsets;
//   * the a/8 skew puts the four row groups of a warp (tap rows 8 apart) into the four bank
//     residues modulo 4 while the eight column groups are 4 floats apart: 32 lanes, 32 banks.
//
// Integral image construction: each thread loads its 8 x 4 block (128-bit loads), scans it in
// registers, the 8 column-group lanes scan row totals with shuffles, warps of the same tile row
// exchange row totals through shared memory; the same again down the columns.  The block is then
// stored with the layout above (conflict-free).
#include "bc_common.cuh"

namespace bc {

namespace {

constexpr int kR = 8;            // rows per strip
constexpr int kTile = 32;        // a warp covers kTile x kTile pixels
constexpr int kPad = 4;          // padding columns on either side of an integral-image row
constexpr int kMaxTiles = 32;
constexpr int kMaxSmem = 200 * 1024;

__host__ __device__ inline int layout_pitch(int w) { return w + 1 + 2 * kPad; }
__host__ __device__ inline int layout_floats(int h, int w) { return (((h + 1) * layout_pitch(w) + (h >> 3) + 4) + 3) & ~3; }
__device__ __forceinline__ int row_offset(int a, int k8) { return (a * k8) >> 3; }   // k8 = 8*pitch + 1

inline int warp_tiles(int h, int w) { return ((w + kTile - 1) / kTile) * ((h + kTile - 1) / kTile); }

__device__ __forceinline__ float warp_sum(float v)
{
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) v += __shfl_xor_sync(0xffffffffu, v, d);
    return v;
}

struct TilePos {
    int p0, q0, rt, ct;
    bool valid;
};

__device__ __forceinline__ TilePos tile_pos(int wt, int ntiles, int col_tiles, int cg, int rg)
{
    TilePos t;
    t.valid = wt < ntiles;
    t.rt = wt / col_tiles;
    t.ct = wt - t.rt * col_tiles;
    t.p0 = t.rt * kTile + rg * kR;
    t.q0 = t.ct * kTile + cg * kStrip;
    return t;
}

// Builds the padded, skewed integral image of one h x w plane (global memory) in shared memory.
// sRow / sCol: scratch for the totals exchanged between warps (kMaxTiles*32 floats each).
// All threads of the CTA must call it; it ends with a barrier.
template <int T>
__device__ __forceinline__ void build_integral(const float *__restrict__ src, float *sI, float *sRow,
                                               float *sCol, int h, int w, bool vec4)
{
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, nwarps = blockDim.x >> 5;
    const int cg = lane & 7, rg = lane >> 3;
    const int col_tiles = (w + kTile - 1) / kTile, row_tiles = (h + kTile - 1) / kTile;
    const int ntiles = col_tiles * row_tiles;
    const int pitch = layout_pitch(w), k8 = 8 * pitch + 1;

    float v[T][kR][kStrip];
    TilePos tp[T];

    // ---- load
#pragma unroll
    for (int k = 0; k < T; ++k) {
        tp[k] = tile_pos(warp + k * nwarps, ntiles, col_tiles, cg, rg);
#pragma unroll
        for (int i = 0; i < kR; ++i) {
            const int p = tp[k].p0 + i;
            const bool in = tp[k].valid && p < h && tp[k].q0 < w;
            if (vec4) {
                const float4 t = in ? __ldg(reinterpret_cast<const float4 *>(src + p * w + tp[k].q0))
                                    : make_float4(0.f, 0.f, 0.f, 0.f);
                v[k][i][0] = t.x; v[k][i][1] = t.y; v[k][i][2] = t.z; v[k][i][3] = t.w;
            } else {
#pragma unroll
                for (int m = 0; m < kStrip; ++m)
                    v[k][i][m] = (in && tp[k].q0 + m < w) ? __ldg(src + p * w + tp[k].q0 + m) : 0.0f;
            }
        }
    }
    for (int c = tid; c < pitch; c += blockDim.x) sI[c] = 0.0f;          // row 0 with its padding

    // ---- along rows: in-thread, across the 8 column-group lanes, across the warps of a tile row
#pragma unroll
    for (int k = 0; k < T; ++k) {
#pragma unroll
        for (int i = 0; i < kR; ++i) {
            v[k][i][1] += v[k][i][0]; v[k][i][2] += v[k][i][1]; v[k][i][3] += v[k][i][2];
            const float own = v[k][i][3];
            float incl = own;
#pragma unroll
            for (int d = 1; d < 8; d <<= 1) {
                const float u = __shfl_up_sync(0xffffffffu, incl, d, 8);
                if (cg >= d) incl += u;
            }
            const float e = incl - own;
#pragma unroll
            for (int m = 0; m < kStrip; ++m) v[k][i][m] += e;
            if (cg == 7 && tp[k].valid) sRow[(tp[k].ct * row_tiles + tp[k].rt) * kTile + rg * kR + i] = incl;
        }
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < T; ++k) {
        if (tp[k].valid) {
            for (int c2 = 0; c2 < tp[k].ct; ++c2) {
                const float4 *s = reinterpret_cast<const float4 *>(sRow + (c2 * row_tiles + tp[k].rt) * kTile + rg * kR);
                const float4 a = s[0], b = s[1];
                const float add[kR] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
#pragma unroll
                for (int i = 0; i < kR; ++i)
#pragma unroll
                    for (int m = 0; m < kStrip; ++m) v[k][i][m] += add[i];
            }
        }
    }

    // ---- down columns: in-thread, across the 4 row-group lanes, across the warps of a tile column
#pragma unroll
    for (int k = 0; k < T; ++k) {
#pragma unroll
        for (int i = 1; i < kR; ++i)
#pragma unroll
            for (int m = 0; m < kStrip; ++m) v[k][i][m] += v[k][i - 1][m];
        float tot[kStrip];
#pragma unroll
        for (int m = 0; m < kStrip; ++m) {
            const float own = v[k][kR - 1][m];
            float incl = own;
            float u = __shfl_up_sync(0xffffffffu, incl, 8);
            if (rg >= 1) incl += u;
            u = __shfl_up_sync(0xffffffffu, incl, 16);
            if (rg >= 2) incl += u;
            const float e = incl - own;
#pragma unroll
            for (int i = 0; i < kR; ++i) v[k][i][m] += e;
            tot[m] = incl;
        }
        if (rg == 3 && tp[k].valid)
            *reinterpret_cast<float4 *>(sCol + (tp[k].rt * col_tiles + tp[k].ct) * kTile + cg * kStrip) =
                make_float4(tot[0], tot[1], tot[2], tot[3]);
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < T; ++k) {
        if (tp[k].valid) {
            for (int r2 = 0; r2 < tp[k].rt; ++r2) {
                const float4 a = *reinterpret_cast<const float4 *>(sCol + (r2 * col_tiles + tp[k].ct) * kTile + cg * kStrip);
#pragma unroll
                for (int i = 0; i < kR; ++i) {
                    v[k][i][0] += a.x; v[k][i][1] += a.y; v[k][i][2] += a.z; v[k][i][3] += a.w;
                }
            }
        }
    }

    // ---- store rows 1..h with their padding
#pragma unroll
    for (int k = 0; k < T; ++k) {
        if (tp[k].valid && tp[k].q0 < w) {
            const int q0 = tp[k].q0;
#pragma unroll
            for (int i = 0; i < kR; ++i) {
                const int a = tp[k].p0 + i + 1;
                if (a <= h) {
                    float *row = sI + row_offset(a, k8) + kPad;
                    // columns q0+1 .. q0+4; past the plane's last column the running value is
                    // I[a][w], which is exactly what the right-hand padding has to hold
#pragma unroll
                    for (int m = 0; m < kStrip; ++m) row[q0 + 1 + m] = v[k][i][m];
                    if (q0 + kStrip >= w) {
#pragma unroll
                        for (int m = 0; m < kPad; ++m)
                            if (q0 + kStrip + 1 + m <= w + kPad) row[q0 + kStrip + 1 + m] = v[k][i][kStrip - 1];
                    }
                    if (q0 == 0) {
#pragma unroll
                        for (int m = -kPad; m <= 0; ++m) row[m] = 0.0f;
                    }
                }
            }
        }
    }
    __syncthreads();
}

// Column window starts of a strip (clamped: see the layout note on top).
__device__ __forceinline__ void window_bases(const BoxTaps &t, int q0, int w, int &bl, int &bh)
{
    bl = clampi(q0 + t.lo_c - 1, -kPad, w);
    bh = clampi(q0 + t.hi_c, -kPad, w);
}

struct TapRow {      // column-combined value of one tap row, per column of the strip
    float d[kStrip];
};
struct TapRowE {     // ... plus the one-column strips outside the box on either side
    float d[kStrip], e_lo[kStrip], e_hi[kStrip];
};

__device__ __forceinline__ TapRow load_tap_row(const float *sIp, int a, int k8, int bl, int bh, float wl,
                                               float fl, float wh, float fh)
{
    const float *r = sIp + row_offset(a, k8);
    const float *pl = r + bl, *ph = r + bh;
    float vl[kStrip + 1], vh[kStrip + 1];
#pragma unroll
    for (int m = 0; m <= kStrip; ++m) { vl[m] = pl[m]; vh[m] = ph[m]; }
    TapRow o;
#pragma unroll
    for (int m = 0; m < kStrip; ++m) o.d[m] = wh * vh[m] + fh * vh[m + 1] - wl * vl[m + 1] - fl * vl[m];
    return o;
}

__device__ __forceinline__ TapRowE load_tap_row_e(const float *sIp, int a, int k8, int bl, int bh, float wl,
                                                  float fl, float wh, float fh)
{
    const float *r = sIp + row_offset(a, k8);
    const float *pl = r + bl, *ph = r + bh;
    float vl[kStrip + 1], vh[kStrip + 1];
#pragma unroll
    for (int m = 0; m <= kStrip; ++m) { vl[m] = pl[m]; vh[m] = ph[m]; }
    TapRowE o;
#pragma unroll
    for (int m = 0; m < kStrip; ++m) {
        o.d[m] = wh * vh[m] + fh * vh[m + 1] - wl * vl[m + 1] - fl * vl[m];
        o.e_lo[m] = vl[m + 1] - vl[m];
        o.e_hi[m] = vh[m + 1] - vh[m];
    }
    return o;
}

template <int T>
__global__ void __launch_bounds__(256)
forward_plane_kernel(const float *__restrict__ x, BoxParams bp, float *__restrict__ out, int C, int F,
                     int h, int w, int fsplit, bool normalize, bool exact, bool vec4)
{
    extern __shared__ float4 smem4[];
    float *sI = reinterpret_cast<float *>(smem4);
    __shared__ __align__(16) float sRow[kMaxTiles * kTile];
    __shared__ __align__(16) float sCol[kMaxTiles * kTile];

    const int64_t nc = blockIdx.x / fsplit;
    const int part = blockIdx.x % fsplit;
    const int c = (int)(nc % C);
    const int f_begin = (F * part) / fsplit, f_end = (F * (part + 1)) / fsplit;

    build_integral<T>(x + nc * (int64_t)h * w, sI, sRow, sCol, h, w, vec4);

    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
    const int cg = lane & 7, rg = lane >> 3;
    const int col_tiles = (w + kTile - 1) / kTile, row_tiles = (h + kTile - 1) / kTile;
    const int ntiles = col_tiles * row_tiles;
    const int k8 = 8 * layout_pitch(w) + 1;
    const float *sIp = sI + kPad;

    for (int f = f_begin; f < f_end; ++f) {
        const Box box = load_box(bp, c * F + f);
        const BoxTaps t = taps_forward(box.xmin, box.xmax, box.ymin, box.ymax, normalize, exact);
        const float wl = 1.0f - t.f_lo_c, wh = 1.0f - t.f_hi_c;
        float *o = out + (nc * F + f) * (int64_t)h * w;
#pragma unroll
        for (int k = 0; k < T; ++k) {
            const TilePos tp = tile_pos(warp + k * nwarps, ntiles, col_tiles, cg, rg);
            if (!tp.valid || tp.q0 >= w || tp.p0 >= h) continue;
            int bl, bh;
            window_bases(t, tp.q0, w, bl, bh);
            TapRow ra = load_tap_row(sIp, clampi(tp.p0 + t.lo_r - 1, 0, h), k8, bl, bh, wl, t.f_lo_c, wh, t.f_hi_c);
            TapRow rc = load_tap_row(sIp, clampi(tp.p0 + t.hi_r, 0, h), k8, bl, bh, wl, t.f_lo_c, wh, t.f_hi_c);
#pragma unroll
            for (int i = 0; i < kR; ++i) {
                const int p = tp.p0 + i;
                if (p < h) {
                    const TapRow rb = load_tap_row(sIp, clampi(p + t.lo_r, 0, h), k8, bl, bh, wl, t.f_lo_c, wh, t.f_hi_c);
                    const TapRow rd = load_tap_row(sIp, clampi(p + t.hi_r + 1, 0, h), k8, bl, bh, wl, t.f_lo_c, wh, t.f_hi_c);
                    float v[kStrip];
#pragma unroll
                    for (int m = 0; m < kStrip; ++m)
                        v[m] = combine_rows(ra.d[m], rb.d[m], rc.d[m], rd.d[m], t.f_lo_r, t.f_hi_r) * t.scale;
                    float *dst = o + p * w + tp.q0;
                    if (vec4) {
                        *reinterpret_cast<float4 *>(dst) = make_float4(v[0], v[1], v[2], v[3]);
                    } else {
#pragma unroll
                        for (int m = 0; m < kStrip; ++m)
                            if (tp.q0 + m < w) dst[m] = v[m];
                    }
                    ra = rb;
                    rc = rd;
                }
            }
        }
    }
}

// T = warp tiles per warp: grad-input accumulators are registers, so the number of strips a
// thread owns is a compile-time constant.
template <int T, bool NEED_PARAMS>
__global__ void __launch_bounds__(512)
backward_plane_kernel(const float *__restrict__ x, const float *__restrict__ grad_output, BoxParams bp,
                      float *__restrict__ grad_input, float *__restrict__ partials, int N, int C, int F,
                      int h, int w, bool normalize, bool exact, bool vec4, bool write_gin)
{
    extern __shared__ float4 smem4[];
    float *sI = reinterpret_cast<float *>(smem4);          // integral(grad_output plane)
    float *sX = sI + layout_floats(h, w);                  // the input plane, pitch w
    __shared__ __align__(16) float sRow[kMaxTiles * kTile];
    __shared__ __align__(16) float sCol[kMaxTiles * kTile];
    __shared__ float red[16][kNumSums];

    const int64_t nc = blockIdx.x;
    const int c = (int)(nc % C), n = (int)(nc / C);
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, nwarps = blockDim.x >> 5;
    const int cg = lane & 7, rg = lane >> 3;
    const int col_tiles = (w + kTile - 1) / kTile, row_tiles = (h + kTile - 1) / kTile;
    const int ntiles = col_tiles * row_tiles;
    const int k8 = 8 * layout_pitch(w) + 1;
    const float *sIp = sI + kPad;
    const int npix = h * w;

    if (NEED_PARAMS) {
        const float *xp = x + nc * (int64_t)npix;
        if (vec4) {
            for (int i = tid; i < (npix >> 2); i += blockDim.x)
                reinterpret_cast<float4 *>(sX)[i] = __ldg(reinterpret_cast<const float4 *>(xp) + i);
        } else {
            for (int i = tid; i < npix; i += blockDim.x) sX[i] = __ldg(xp + i);
        }
    }

    float gin[T][kR][kStrip];
#pragma unroll
    for (int k = 0; k < T; ++k)
#pragma unroll
        for (int i = 0; i < kR; ++i)
#pragma unroll
            for (int m = 0; m < kStrip; ++m) gin[k][i][m] = 0.0f;

    for (int f = 0; f < F; ++f) {
        // (the barrier that ends the previous iteration protects sI, sRow, sCol)
        const float *gplane = grad_output + (nc * F + f) * (int64_t)npix;
        build_integral<T>(gplane, sI, sRow, sCol, h, w, vec4);
        if (f + 1 < F && cg == 0) {
            // pull the next grad_output plane towards L2 while this one is gathered
#pragma unroll
            for (int k = 0; k < T; ++k) {
                const TilePos tp = tile_pos(warp + k * nwarps, ntiles, col_tiles, cg, rg);
#pragma unroll
                for (int i = 0; i < kR; ++i)
                    if (tp.valid && tp.p0 + i < h && tp.q0 < w)
                        asm volatile("prefetch.global.L2 [%0];" ::"l"(gplane + npix + (tp.p0 + i) * w + tp.q0));
            }
        }

        const Box box = load_box(bp, c * F + f);
        const BoxTaps t = taps_mirrored(box.xmin, box.xmax, box.ymin, box.ymax, normalize, exact);
        const float wl = 1.0f - t.f_lo_c, wh = 1.0f - t.f_hi_c;
        ParamSums sums = {0.f, 0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int k = 0; k < T; ++k) {
            const TilePos tp = tile_pos(warp + k * nwarps, ntiles, col_tiles, cg, rg);
            if (tp.valid && tp.q0 < w && tp.p0 < h) {
                int bl, bh;
                window_bases(t, tp.q0, w, bl, bh);
                if (NEED_PARAMS) {
                    TapRowE ra = load_tap_row_e(sIp, clampi(tp.p0 + t.lo_r - 1, 0, h), k8, bl, bh, wl, t.f_lo_c, wh, t.f_hi_c);
                    TapRowE rc = load_tap_row_e(sIp, clampi(tp.p0 + t.hi_r, 0, h), k8, bl, bh, wl, t.f_lo_c, wh, t.f_hi_c);
#pragma unroll
                    for (int i = 0; i < kR; ++i) {
                        const int p = tp.p0 + i;
                        if (p < h) {
                            const TapRowE rb = load_tap_row_e(sIp, clampi(p + t.lo_r, 0, h), k8, bl, bh, wl, t.f_lo_c, wh, t.f_hi_c);
                            const TapRowE rd = load_tap_row_e(sIp, clampi(p + t.hi_r + 1, 0, h), k8, bl, bh, wl, t.f_lo_c, wh, t.f_hi_c);
                            float xv[kStrip];
                            if (vec4) {
                                const float4 v = *reinterpret_cast<const float4 *>(sX + p * w + tp.q0);
                                xv[0] = v.x; xv[1] = v.y; xv[2] = v.z; xv[3] = v.w;
                            } else {
#pragma unroll
                                for (int m = 0; m < kStrip; ++m) xv[m] = tp.q0 + m < w ? sX[p * w + tp.q0 + m] : 0.0f;
                            }
#pragma unroll
                            for (int m = 0; m < kStrip; ++m) {
                                const float top = rb.d[m] - ra.d[m];
                                const float bot = rd.d[m] - rc.d[m];
                                const float g = (rc.d[m] - rb.d[m]) + t.f_hi_r * bot + t.f_lo_r * top;
                                const float sl = combine_rows(ra.e_lo[m], rb.e_lo[m], rc.e_lo[m], rd.e_lo[m], t.f_lo_r, t.f_hi_r);
                                const float sr = combine_rows(ra.e_hi[m], rb.e_hi[m], rc.e_hi[m], rd.e_hi[m], t.f_lo_r, t.f_hi_r);
                                sums.s_out += xv[m] * g;
                                sums.s_top += xv[m] * top;
                                sums.s_bot += xv[m] * bot;
                                sums.s_left += xv[m] * sl;
                                sums.s_right += xv[m] * sr;
                                gin[k][i][m] += g * t.scale;
                            }
                            ra = rb;
                            rc = rd;
                        }
                    }
                } else {
                    TapRow ra = load_tap_row(sIp, clampi(tp.p0 + t.lo_r - 1, 0, h), k8, bl, bh, wl, t.f_lo_c, wh, t.f_hi_c);
                    TapRow rc = load_tap_row(sIp, clampi(tp.p0 + t.hi_r, 0, h), k8, bl, bh, wl, t.f_lo_c, wh, t.f_hi_c);
#pragma unroll
                    for (int i = 0; i < kR; ++i) {
                        const int p = tp.p0 + i;
                        if (p < h) {
                            const TapRow rb = load_tap_row(sIp, clampi(p + t.lo_r, 0, h), k8, bl, bh, wl, t.f_lo_c, wh, t.f_hi_c);
                            const TapRow rd = load_tap_row(sIp, clampi(p + t.hi_r + 1, 0, h), k8, bl, bh, wl, t.f_lo_c, wh, t.f_hi_c);
#pragma unroll
                            for (int m = 0; m < kStrip; ++m)
                                gin[k][i][m] += combine_rows(ra.d[m], rb.d[m], rc.d[m], rd.d[m], t.f_lo_r, t.f_hi_r) * t.scale;
                            ra = rb;
                            rc = rd;
                        }
                    }
                }
            }
        }
        if (NEED_PARAMS) {
            float v[kNumSums] = {sums.s_out, sums.s_top, sums.s_bot, sums.s_left, sums.s_right};
#pragma unroll
            for (int j = 0; j < kNumSums; ++j) v[j] = warp_sum(v[j]);
            if (lane == 0) {
#pragma unroll
                for (int j = 0; j < kNumSums; ++j) red[warp][j] = v[j];
            }
        }
        __syncthreads();      // gathers of this filter are done: sI may be rebuilt; red[] is complete
        if (NEED_PARAMS && tid < kNumSums) {
            float s = 0.0f;
            for (int g = 0; g < nwarps; ++g) s += red[g][tid];
            partials[((int64_t)(c * F + f) * N + n) * kNumSums + tid] = s;
        }
        // red[] is next written after the barriers inside the next build_integral
    }

    if (write_gin) {
        float *gi = grad_input + nc * (int64_t)npix;
#pragma unroll
        for (int k = 0; k < T; ++k) {
            const TilePos tp = tile_pos(warp + k * nwarps, ntiles, col_tiles, cg, rg);
            if (tp.valid && tp.q0 < w) {
#pragma unroll
                for (int i = 0; i < kR; ++i) {
                    const int p = tp.p0 + i;
                    if (p < h) {
                        float *dst = gi + p * w + tp.q0;
                        if (vec4) {
                            *reinterpret_cast<float4 *>(dst) = make_float4(gin[k][i][0], gin[k][i][1], gin[k][i][2], gin[k][i][3]);
                        } else {
#pragma unroll
                            for (int m = 0; m < kStrip; ++m)
                                if (tp.q0 + m < w) dst[m] = gin[k][i][m];
                        }
                    }
                }
            }
        }
    }
}

template <class K>
int opt_in_smem(K kernel, size_t bytes)
{
    if (bytes <= 36 * 1024) return BC_OK;     // static scratch included, this stays under the 48 KB default
    if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes) != cudaSuccess)
        return check_launch("shared memory opt-in");
    return BC_OK;
}

}  // namespace

bool plane_path_fits_forward(int h, int w)
{
    return (size_t)layout_floats(h, w) * sizeof(float) <= kMaxSmem && warp_tiles(h, w) <= kMaxTiles;
}

bool plane_path_fits_backward(int h, int w)
{
    const size_t bytes = ((size_t)layout_floats(h, w) + (size_t)h * w) * sizeof(float);
    return bytes <= kMaxSmem && warp_tiles(h, w) <= kMaxTiles;
}

int launch_forward_plane(const float *x, const BoxParams &bp, float *out, int N, int C, int F, int h,
                         int w, bool normalize, bool exact, cudaStream_t s)
{
    const int64_t planes = (int64_t)N * C;
    // split the filters of a plane over several CTAs while there are too few planes to balance
    // 148 SMs; every part rebuilds the integral image (cheap next to the gathers, and the second
    // read of the plane comes from L2)
    int fsplit = 1;
    while (fsplit < F && planes * fsplit < 148 * 12 && F % (fsplit * 2) == 0) fsplit *= 2;
    if (planes * fsplit > 0x7fffffffLL) return BC_ERR_BAD_SHAPE;
    const size_t smem = (size_t)layout_floats(h, w) * sizeof(float);
    const int tiles = warp_tiles(h, w);
    const int T = tiles > 16 ? 4 : (tiles > 8 ? 2 : 1);
    const int warps = (tiles + T - 1) / T;
    auto kern = T == 1 ? forward_plane_kernel<1> : (T == 2 ? forward_plane_kernel<2> : forward_plane_kernel<4>);
    int st = opt_in_smem(kern, smem);
    if (st != BC_OK) return st;
    const bool vec4 = (w % 4 == 0) && ((reinterpret_cast<uintptr_t>(x) & 15) == 0) &&
                      ((reinterpret_cast<uintptr_t>(out) & 15) == 0);
    {
        LaunchScope scope(KID_FORWARD_PLANE, s);
        kern<<<(unsigned)(planes * fsplit), warps * 32, smem, s>>>(x, bp, out, C, F, h, w, fsplit, normalize,
                                                                    exact, vec4);
    }
    return check_launch("forward_plane");
}

int launch_backward_plane(const float *x, const float *grad_output, const BoxParams &bp, float rep_h,
                          float rep_w, int N, int C, int F, int h, int w, bool normalize, bool exact,
                          int need_mask, float *grad_input, float *grad_params, float *partials,
                          cudaStream_t s)
{
    const int64_t planes = (int64_t)N * C;
    if (planes > 0x7fffffffLL) return BC_ERR_BAD_SHAPE;
    const bool need_params = (need_mask & (BC_NEED_ALL & ~BC_NEED_INPUT)) != 0;
    const bool write_gin = (need_mask & BC_NEED_INPUT) != 0;
    const size_t smem = ((size_t)layout_floats(h, w) + (need_params ? (size_t)h * w : 0)) * sizeof(float);
    const int tiles = warp_tiles(h, w);
    const int T = tiles > 8 ? 2 : 1;
    const int warps = (tiles + T - 1) / T;
    const bool vec4 = (w % 4 == 0) && ((reinterpret_cast<uintptr_t>(x) & 15) == 0) &&
                      ((reinterpret_cast<uintptr_t>(grad_output) & 15) == 0) &&
                      (!write_gin || (reinterpret_cast<uintptr_t>(grad_input) & 15) == 0);
    auto kern = T == 1 ? (need_params ? backward_plane_kernel<1, true> : backward_plane_kernel<1, false>)
                       : (need_params ? backward_plane_kernel<2, true> : backward_plane_kernel<2, false>);
    int st = opt_in_smem(kern, smem);
    if (st != BC_OK) return st;
    {
        LaunchScope scope(KID_BACKWARD_PLANE, s);
        kern<<<(unsigned)planes, warps * 32, smem, s>>>(x, grad_output, bp, grad_input, partials, N, C, F, h,
                                                       w, normalize, exact, vec4, write_gin);
    }
    st = check_launch("backward_plane");
    if (st != BC_OK || !need_params) return st;
    return launch_finish_param_grads(partials, bp, C * F, N, normalize, exact, rep_h, rep_w, need_mask,
                                     grad_params, s);
}

}  // namespace bc
