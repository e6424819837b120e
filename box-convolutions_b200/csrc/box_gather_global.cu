// Gather kernels that read integral images from global memory (through L1/L2).  They work for
// every plane size and are the path for planes too large to keep in shared memory; the
// shared-memory-resident kernels for small planes are in box_plane_smem.cu.
//
// Work decomposition: a block of 128 threads covers a tile of 128 columns x 32 rows of one
// plane; warp = one row group, lane = one 4-column strip, each thread walks 8 rows
// (bc_walk.cuh).  Forward: one block per (plane, filter, tile).  Backward: one block per
// (plane, tile); the block loops over the filters so that grad-input is accumulated in
// registers and written once, and leaves five partial sums per filter that the finishing kernel
// turns into the parameter gradients (no atomics: a fixed summation order, bit-reproducible).
#include "bc_common.cuh"
#include "bc_walk.cuh"

namespace bc {

namespace {

constexpr int kRowsPerThread = 8;
constexpr int kRowGroups = 4;
constexpr int kThreads = 32 * kRowGroups;
constexpr int kTileCols = 32 * kStrip;                    // 128
constexpr int kTileRows = kRowGroups * kRowsPerThread;    // 32

struct GlobalRows {
    const float *base;
    int pitch;
    __device__ __forceinline__ const float *operator()(int a) const { return base + (int64_t)a * pitch; }
};

__global__ void __launch_bounds__(kThreads)
forward_global_kernel(const float *__restrict__ integ, BoxParams bp, float *__restrict__ out, int C,
                      int F, int h, int w, int row_tiles, int col_tiles, bool normalize, bool exact)
{
    int64_t b = blockIdx.x;
    const int ct = (int)(b % col_tiles); b /= col_tiles;
    const int rt = (int)(b % row_tiles); b /= row_tiles;
    const int f = (int)(b % F);
    const int64_t nc = b / F;
    const int c = (int)(nc % C);

    const int lane = threadIdx.x & 31, rg = threadIdx.x >> 5;
    const int q0 = ct * kTileCols + lane * kStrip;
    const int p0 = rt * kTileRows + rg * kRowsPerThread;
    if (q0 >= w || p0 >= h) return;
    const int p1 = min(p0 + kRowsPerThread, h);

    const Box box = load_box(bp, c * F + f);
    const BoxTaps t = taps_forward(box.xmin, box.xmax, box.ymin, box.ymax, normalize, exact);
    const StripCols sc = strip_cols(t, q0, w);
    const GlobalRows rows{integ + nc * (int64_t)(h + 1) * (w + 1), w + 1};
    float *o = out + (nc * F + f) * (int64_t)h * w;
    const bool vec = (w % kStrip == 0) && ((reinterpret_cast<uintptr_t>(out) & 15) == 0);

    walk_forward(rows, t, sc, p0, p1, h, [&](int p, const float *v) {
        float *dst = o + (int64_t)p * w + q0;
        if (vec) {
            *reinterpret_cast<float4 *>(dst) = make_float4(v[0], v[1], v[2], v[3]);
        } else {
#pragma unroll
            for (int m = 0; m < kStrip; ++m)
                if (q0 + m < w) dst[m] = v[m];
        }
    });
}

__device__ __forceinline__ float warp_sum(float v)
{
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) v += __shfl_xor_sync(0xffffffffu, v, d);
    return v;
}

// x value of a pixel rebuilt from the input's integral image (used only when the caller has
// no copy of the input itself, as through the reference's four-function interface).
__device__ __forceinline__ float pixel_from_integral(const float *I, int pitch, int p, int q)
{
    const float *r0 = I + (int64_t)p * pitch + q;
    const float *r1 = r0 + pitch;
    return __ldg(r1 + 1) - __ldg(r0 + 1) - __ldg(r1) + __ldg(r0);
}

template <bool NEED_PARAMS>
__global__ void __launch_bounds__(kThreads)
backward_global_kernel(const float *__restrict__ x, const float *__restrict__ x_integ,
                       const float *__restrict__ go_integ, BoxParams bp, float *__restrict__ grad_input,
                       float *__restrict__ partials, int N, int C, int F, int h, int w, int row_tiles,
                       int col_tiles, bool normalize, bool exact, bool write_gin)
{
    __shared__ float red[kRowGroups][kNumSums];

    int64_t b = blockIdx.x;
    const int ct = (int)(b % col_tiles); b /= col_tiles;
    const int rt = (int)(b % row_tiles);
    const int64_t nc = b / row_tiles;
    const int c = (int)(nc % C);
    const int n = (int)(nc / C);
    const int tile = rt * col_tiles + ct;
    const int tiles = row_tiles * col_tiles;

    const int lane = threadIdx.x & 31, rg = threadIdx.x >> 5;
    const int q0 = ct * kTileCols + lane * kStrip;
    const int p0 = rt * kTileRows + rg * kRowsPerThread;
    const bool active = q0 < w && p0 < h;
    const int p1 = min(p0 + kRowsPerThread, h);
    const int ipitch = w + 1;
    const int64_t ipl = (int64_t)(h + 1) * ipitch;

    float gin[kRowsPerThread][kStrip];
#pragma unroll
    for (int i = 0; i < kRowsPerThread; ++i)
#pragma unroll
        for (int m = 0; m < kStrip; ++m) gin[i][m] = 0.0f;

    const float *xp = x ? x + nc * (int64_t)h * w : nullptr;
    const float *xi = x_integ ? x_integ + nc * ipl : nullptr;

    for (int f = 0; f < F; ++f) {
        ParamSums sums = {0.f, 0.f, 0.f, 0.f, 0.f};
        if (active) {
            const Box box = load_box(bp, c * F + f);
            const BoxTaps t = taps_mirrored(box.xmin, box.xmax, box.ymin, box.ymax, normalize, exact);
            const StripCols sc = strip_cols(t, q0, w);
            const GlobalRows rows{go_integ + (nc * F + f) * ipl, ipitch};
            if (NEED_PARAMS) {
                // the walk is unrolled by hand over a register tile: row index relative to p0
                RowDE ra = load_row_de(rows(clampi(p0 + t.lo_r - 1, 0, h)), sc, t);
                RowDE rc = load_row_de(rows(clampi(p0 + t.hi_r, 0, h)), sc, t);
#pragma unroll
                for (int i = 0; i < kRowsPerThread; ++i) {
                    const int p = p0 + i;
                    if (p < p1) {
                        const RowDE rb = load_row_de(rows(clampi(p + t.lo_r, 0, h)), sc, t);
                        const RowDE rd = load_row_de(rows(clampi(p + t.hi_r + 1, 0, h)), sc, t);
#pragma unroll
                        for (int m = 0; m < kStrip; ++m) {
                            const float top = rb.d[m] - ra.d[m];
                            const float bot = rd.d[m] - rc.d[m];
                            const float g = (rc.d[m] - rb.d[m]) + t.f_hi_r * bot + t.f_lo_r * top;
                            const float sl = combine_rows(ra.e_lo[m], rb.e_lo[m], rc.e_lo[m], rd.e_lo[m], t.f_lo_r, t.f_hi_r);
                            const float sr = combine_rows(ra.e_hi[m], rb.e_hi[m], rc.e_hi[m], rd.e_hi[m], t.f_lo_r, t.f_hi_r);
                            float xv = 0.0f;
                            if (q0 + m < w)
                                xv = xp ? __ldg(xp + (int64_t)p * w + q0 + m) : pixel_from_integral(xi, ipitch, p, q0 + m);
                            sums.s_out += xv * g;
                            sums.s_top += xv * top;
                            sums.s_bot += xv * bot;
                            sums.s_left += xv * sl;
                            sums.s_right += xv * sr;
                            gin[i][m] += g * t.scale;
                        }
                        ra = rb;
                        rc = rd;
                    }
                }
            } else {
                RowD ra = load_row_d(rows(clampi(p0 + t.lo_r - 1, 0, h)), sc, t);
                RowD rc = load_row_d(rows(clampi(p0 + t.hi_r, 0, h)), sc, t);
#pragma unroll
                for (int i = 0; i < kRowsPerThread; ++i) {
                    const int p = p0 + i;
                    if (p < p1) {
                        const RowD rb = load_row_d(rows(clampi(p + t.lo_r, 0, h)), sc, t);
                        const RowD rd = load_row_d(rows(clampi(p + t.hi_r + 1, 0, h)), sc, t);
#pragma unroll
                        for (int m = 0; m < kStrip; ++m)
                            gin[i][m] += combine_rows(ra.d[m], rb.d[m], rc.d[m], rd.d[m], t.f_lo_r, t.f_hi_r) * t.scale;
                        ra = rb;
                        rc = rd;
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
                for (int j = 0; j < kNumSums; ++j) red[rg][j] = v[j];
            }
            __syncthreads();
            if (threadIdx.x < kNumSums) {
                float s = 0.0f;
#pragma unroll
                for (int g = 0; g < kRowGroups; ++g) s += red[g][threadIdx.x];
                const int64_t slot = ((int64_t)(c * F + f) * N + n) * tiles + tile;
                partials[slot * kNumSums + threadIdx.x] = s;
            }
            __syncthreads();
        }
    }

    if (write_gin && active) {
        float *gi = grad_input + nc * (int64_t)h * w;
        const bool vec = (w % kStrip == 0) && ((reinterpret_cast<uintptr_t>(grad_input) & 15) == 0);
#pragma unroll
        for (int i = 0; i < kRowsPerThread; ++i) {
            const int p = p0 + i;
            if (p < p1) {
                float *dst = gi + (int64_t)p * w + q0;
                if (vec) {
                    *reinterpret_cast<float4 *>(dst) = make_float4(gin[i][0], gin[i][1], gin[i][2], gin[i][3]);
                } else {
#pragma unroll
                    for (int m = 0; m < kStrip; ++m)
                        if (q0 + m < w) dst[m] = gin[i][m];
                }
            }
        }
    }
}

}  // namespace

// One warp per (plane c, filter f): sums the per-(sample, tile) partials in a fixed order and
// finishes the four gradients.  grad_params is (4, C, F).
__global__ void finish_param_grads_kernel(const float *__restrict__ partials, BoxParams bp, int count,
                                          int per_box, bool normalize, bool exact, float rep_h,
                                          float rep_w, int need_mask, float *__restrict__ grad_params)
{
    const int k = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    const int lane = threadIdx.x & 31;
    if (k >= count) return;
    const float *src = partials + (int64_t)k * per_box * kNumSums;
    float acc[kNumSums] = {0.f, 0.f, 0.f, 0.f, 0.f};
    for (int i = lane; i < per_box; i += 32) {
#pragma unroll
        for (int j = 0; j < kNumSums; ++j) acc[j] += src[(int64_t)i * kNumSums + j];
    }
#pragma unroll
    for (int j = 0; j < kNumSums; ++j) acc[j] = warp_sum(acc[j]);
    if (lane == 0) {
        const Box box = load_box(bp, k);
        const ParamSums s = {acc[0], acc[1], acc[2], acc[3], acc[4]};
        float g[4];
        finish_param_grads(s, box.xmin, box.xmax, box.ymin, box.ymax, normalize, exact, rep_h, rep_w, g);
#pragma unroll
        for (int j = 0; j < 4; ++j)
            if (need_mask & (BC_NEED_X_MIN << j)) grad_params[(int64_t)j * count + k] = g[j];
    }
}

int launch_finish_param_grads(const float *partials, const BoxParams &bp, int count, int per_box,
                              bool normalize, bool exact, float rep_h, float rep_w, int need_mask,
                              float *grad_params, cudaStream_t s)
{
    const int warps_per_block = 4;
    const int blocks = (count + warps_per_block - 1) / warps_per_block;
    {
        LaunchScope scope(KID_FINISH_PARAM_GRADS, s);
        finish_param_grads_kernel<<<blocks, warps_per_block * 32, 0, s>>>(
            partials, bp, count, per_box, normalize, exact, rep_h, rep_w, need_mask, grad_params);
    }
    return check_launch("finish_param_grads");
}

static inline int ceil_div(int a, int b) { return (a + b - 1) / b; }

int launch_forward_global(const float *integ, const BoxParams &bp, float *out, int N, int C, int F,
                          int h, int w, bool normalize, bool exact, cudaStream_t s)
{
    const int row_tiles = ceil_div(h, kTileRows), col_tiles = ceil_div(w, kTileCols);
    const int64_t blocks = (int64_t)N * C * F * row_tiles * col_tiles;
    if (blocks == 0) return BC_OK;
    if (blocks > 0x7fffffffLL) return BC_ERR_BAD_SHAPE;
    {
        LaunchScope scope(KID_FORWARD_GLOBAL, s);
        forward_global_kernel<<<(unsigned)blocks, kThreads, 0, s>>>(integ, bp, out, C, F, h, w, row_tiles,
                                                                     col_tiles, normalize, exact);
    }
    return check_launch("forward_global");
}

size_t backward_partials_bytes(int N, int C, int F, int h, int w)
{
    const size_t tiles = (size_t)ceil_div(h, kTileRows) * ceil_div(w, kTileCols);
    return (size_t)C * F * N * tiles * kNumSums * sizeof(float);
}

int launch_backward_global(const float *x, const float *x_integ, const float *go_integ,
                           const BoxParams &bp, float rep_h, float rep_w, int N, int C, int F,
                           int h, int w, bool normalize, bool exact, int need_mask,
                           float *grad_input, float *grad_params, float *partials, cudaStream_t s)
{
    const int row_tiles = ceil_div(h, kTileRows), col_tiles = ceil_div(w, kTileCols);
    const int64_t blocks = (int64_t)N * C * row_tiles * col_tiles;
    if (blocks == 0) return BC_OK;
    if (blocks > 0x7fffffffLL) return BC_ERR_BAD_SHAPE;
    const bool need_params = (need_mask & (BC_NEED_ALL & ~BC_NEED_INPUT)) != 0;
    const bool write_gin = (need_mask & BC_NEED_INPUT) != 0;
    {
    LaunchScope scope(KID_BACKWARD_GLOBAL, s);
    if (need_params) {
        backward_global_kernel<true><<<(unsigned)blocks, kThreads, 0, s>>>(
            x, x_integ, go_integ, bp, grad_input, partials, N, C, F, h, w, row_tiles, col_tiles,
            normalize, exact, write_gin);
    } else {
        backward_global_kernel<false><<<(unsigned)blocks, kThreads, 0, s>>>(
            x, x_integ, go_integ, bp, grad_input, partials, N, C, F, h, w, row_tiles, col_tiles,
            normalize, exact, write_gin);
    }
    }
    int st = check_launch("backward_global");
    if (st != BC_OK || !need_params) return st;
    return launch_finish_param_grads(partials, bp, C * F, N * row_tiles * col_tiles, normalize, exact,
                                     rep_h, rep_w, need_mask, grad_params, s);
}

}  // namespace bc
