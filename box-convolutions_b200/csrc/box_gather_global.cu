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

template <typename T>
struct GlobalRows {
    const T *base;
    int pitch;
    __device__ __forceinline__ const T *operator()(int a) const { return base + (int64_t)a * pitch; }
};

// 4 adjacent values: one 128-bit store for float (when aligned), plain stores otherwise
template <typename T>
__device__ __forceinline__ void store_strip(T *dst, const T *v, int q0, int w, bool vec)
{
#pragma unroll
    for (int m = 0; m < kStrip; ++m)
        if (q0 + m < w) dst[m] = v[m];
}
template <>
__device__ __forceinline__ void store_strip<float>(float *dst, const float *v, int q0, int w, bool vec)
{
    if (vec) {
        *reinterpret_cast<float4 *>(dst) = make_float4(v[0], v[1], v[2], v[3]);
    } else {
#pragma unroll
        for (int m = 0; m < kStrip; ++m)
            if (q0 + m < w) dst[m] = v[m];
    }
}

template <typename T>
__global__ void __launch_bounds__(kThreads)
forward_global_kernel(const T *__restrict__ integ, BoxParamsT<T> bp, T *__restrict__ out, int C,
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

    const BoxT<T> box = load_box(bp, c * F + f);
    const BoxTapsT<T> t = taps_forward(box.xmin, box.xmax, box.ymin, box.ymax, normalize, exact);
    const StripCols sc = strip_cols(t, q0, w);
    const GlobalRows<T> rows{integ + nc * (int64_t)(h + 1) * (w + 1), w + 1};
    T *o = out + (nc * F + f) * (int64_t)h * w;
    const bool vec = (w % kStrip == 0) && ((reinterpret_cast<uintptr_t>(out) & 15) == 0);

    walk_forward(rows, t, sc, p0, p1, h, [&](int p, const T *v) {
        store_strip(o + (int64_t)p * w + q0, v, q0, w, vec);
    });
}

// Forward with the inference steps around the gather (float): the input ReLU has already gone
// into the integral image; here the per-channel affine, the residual and the output ReLU.
__global__ void __launch_bounds__(kThreads)
forward_global_fused_kernel(const float *__restrict__ integ, BoxParams bp, Fusion fu, float *out,
                            int C, int F, int h, int w, int row_tiles, int col_tiles, bool normalize, bool exact)
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
    const GlobalRows<float> rows{integ + nc * (int64_t)(h + 1) * (w + 1), w + 1};
    const int64_t plane = (nc * F + f) * (int64_t)h * w;
    const float mul = fu.scale ? __ldg(fu.scale + c * F + f) : 1.0f;
    const float add = fu.shift ? __ldg(fu.shift + c * F + f) : 0.0f;
    const bool vec = (w % kStrip == 0) && ((reinterpret_cast<uintptr_t>(out) & 15) == 0);

    walk_forward(rows, t, sc, p0, p1, h, [&](int p, const float *v) {
        const int64_t off = plane + (int64_t)p * w + q0;
        float r[kStrip];
#pragma unroll
        for (int m = 0; m < kStrip; ++m) {
            r[m] = v[m] * mul + add;
            if (fu.residual && q0 + m < w) r[m] += fu.residual[off + m];   // plain load: may alias `out`
            if (fu.output_relu) r[m] = fmaxf(r[m], 0.0f);
        }
        store_strip(out + off, r, q0, w, vec);
    });
}

template <typename T>
__device__ __forceinline__ T warp_sum(T v)
{
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) v += __shfl_xor_sync(0xffffffffu, v, d);
    return v;
}

// x value of a pixel rebuilt from the input's integral image (used only when the caller has
// no copy of the input itself, as through the reference's four-function interface).
template <typename T>
__device__ __forceinline__ T pixel_from_integral(const T *I, int pitch, int p, int q)
{
    const T *r0 = I + (int64_t)p * pitch + q;
    const T *r1 = r0 + pitch;
    return __ldg(r1 + 1) - __ldg(r0 + 1) - __ldg(r1) + __ldg(r0);
}

template <typename T, bool NEED_PARAMS>
__global__ void __launch_bounds__(kThreads)
backward_global_kernel(const T *__restrict__ x, const T *__restrict__ x_integ,
                       const T *__restrict__ go_integ, BoxParamsT<T> bp, T *__restrict__ grad_input,
                       T *__restrict__ partials, int N, int C, int F, int h, int w, int row_tiles,
                       int col_tiles, bool normalize, bool exact, bool write_gin)
{
    __shared__ T red[kRowGroups][kNumSums];

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

    T gin[kRowsPerThread][kStrip];
#pragma unroll
    for (int i = 0; i < kRowsPerThread; ++i)
#pragma unroll
        for (int m = 0; m < kStrip; ++m) gin[i][m] = T(0);

    const T *xp = x ? x + nc * (int64_t)h * w : nullptr;
    const T *xi = x_integ ? x_integ + nc * ipl : nullptr;

    for (int f = 0; f < F; ++f) {
        ParamSumsT<T> sums = {T(0), T(0), T(0), T(0), T(0)};
        if (active) {
            const BoxT<T> box = load_box(bp, c * F + f);
            const BoxTapsT<T> t = taps_mirrored(box.xmin, box.xmax, box.ymin, box.ymax, normalize, exact);
            const StripCols sc = strip_cols(t, q0, w);
            const GlobalRows<T> rows{go_integ + (nc * F + f) * ipl, ipitch};
            if (NEED_PARAMS) {
                // the walk is unrolled by hand over a register tile: row index relative to p0
                RowDET<T> ra = load_row_de(rows(clampi(p0 + t.lo_r - 1, 0, h)), sc, t);
                RowDET<T> rc = load_row_de(rows(clampi(p0 + t.hi_r, 0, h)), sc, t);
#pragma unroll
                for (int i = 0; i < kRowsPerThread; ++i) {
                    const int p = p0 + i;
                    if (p < p1) {
                        const RowDET<T> rb = load_row_de(rows(clampi(p + t.lo_r, 0, h)), sc, t);
                        const RowDET<T> rd = load_row_de(rows(clampi(p + t.hi_r + 1, 0, h)), sc, t);
#pragma unroll
                        for (int m = 0; m < kStrip; ++m) {
                            const T top = rb.d[m] - ra.d[m];
                            const T bot = rd.d[m] - rc.d[m];
                            const T g = (rc.d[m] - rb.d[m]) + t.f_hi_r * bot + t.f_lo_r * top;
                            const T sl = combine_rows(ra.e_lo[m], rb.e_lo[m], rc.e_lo[m], rd.e_lo[m], t.f_lo_r, t.f_hi_r);
                            const T sr = combine_rows(ra.e_hi[m], rb.e_hi[m], rc.e_hi[m], rd.e_hi[m], t.f_lo_r, t.f_hi_r);
                            T xv = T(0);
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
                RowDT<T> ra = load_row_d(rows(clampi(p0 + t.lo_r - 1, 0, h)), sc, t);
                RowDT<T> rc = load_row_d(rows(clampi(p0 + t.hi_r, 0, h)), sc, t);
#pragma unroll
                for (int i = 0; i < kRowsPerThread; ++i) {
                    const int p = p0 + i;
                    if (p < p1) {
                        const RowDT<T> rb = load_row_d(rows(clampi(p + t.lo_r, 0, h)), sc, t);
                        const RowDT<T> rd = load_row_d(rows(clampi(p + t.hi_r + 1, 0, h)), sc, t);
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
            T v[kNumSums] = {sums.s_out, sums.s_top, sums.s_bot, sums.s_left, sums.s_right};
#pragma unroll
            for (int j = 0; j < kNumSums; ++j) v[j] = warp_sum(v[j]);
            if (lane == 0) {
#pragma unroll
                for (int j = 0; j < kNumSums; ++j) red[rg][j] = v[j];
            }
            __syncthreads();
            if (threadIdx.x < kNumSums) {
                T s = T(0);
#pragma unroll
                for (int g = 0; g < kRowGroups; ++g) s += red[g][threadIdx.x];
                const int64_t slot = ((int64_t)(c * F + f) * N + n) * tiles + tile;
                partials[slot * kNumSums + threadIdx.x] = s;
            }
            __syncthreads();
        }
    }

    if (write_gin && active) {
        T *gi = grad_input + nc * (int64_t)h * w;
        const bool vec = (w % kStrip == 0) && ((reinterpret_cast<uintptr_t>(grad_input) & 15) == 0);
#pragma unroll
        for (int i = 0; i < kRowsPerThread; ++i) {
            const int p = p0 + i;
            if (p < p1) store_strip(gi + (int64_t)p * w + q0, gin[i], q0, w, vec);
        }
    }
}

}  // namespace

// One warp per (plane c, filter f): sums the per-(sample, tile) partials in a fixed order and
// finishes the four gradients.  grad_params is (4, C, F).
template <typename T>
__global__ void finish_param_grads_kernel(const T *__restrict__ partials, BoxParamsT<T> bp, int count,
                                          int per_box, bool normalize, bool exact, T rep_h, T rep_w,
                                          int need_mask, T *__restrict__ grad_params)
{
    grid_dependency_wait();
    const int k = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    const int lane = threadIdx.x & 31;
    if (k >= count) return;
    const T *src = partials + (int64_t)k * per_box * kNumSums;
    T acc[kNumSums] = {T(0), T(0), T(0), T(0), T(0)};
    for (int i = lane; i < per_box; i += 32) {
#pragma unroll
        for (int j = 0; j < kNumSums; ++j) acc[j] += src[(int64_t)i * kNumSums + j];
    }
#pragma unroll
    for (int j = 0; j < kNumSums; ++j) acc[j] = warp_sum(acc[j]);
    if (lane == 0) {
        const BoxT<T> box = load_box(bp, k);
        const ParamSumsT<T> s = {acc[0], acc[1], acc[2], acc[3], acc[4]};
        T g[4];
        finish_param_grads(s, box.xmin, box.xmax, box.ymin, box.ymax, normalize, exact, rep_h, rep_w, g);
#pragma unroll
        for (int j = 0; j < 4; ++j)
            if (need_mask & (BC_NEED_X_MIN << j)) grad_params[(int64_t)j * count + k] = g[j];
    }
}

template <typename T>
int launch_finish_param_grads(const T *partials, const BoxParamsT<T> &bp, int count, int per_box,
                              bool normalize, bool exact, T rep_h, T rep_w, int need_mask,
                              T *grad_params, cudaStream_t s)
{
    const int warps_per_block = 4;
    const int blocks = (count + warps_per_block - 1) / warps_per_block;
    {
        LaunchScope scope(KID_FINISH_PARAM_GRADS, s);
        if (cudaError_t e = launch_overlapped(finish_param_grads_kernel<T>, (unsigned)blocks, warps_per_block * 32, 0, s,
                                              partials, bp, count, per_box, normalize, exact, rep_h, rep_w, need_mask,
                                              grad_params))
            return cuda_failed(e, "finish_param_grads");
    }
    return check_launch("finish_param_grads");
}

static inline int ceil_div(int a, int b) { return (a + b - 1) / b; }

template <typename T>
int launch_forward_global(const T *integ, const BoxParamsT<T> &bp, T *out, int N, int C, int F,
                          int h, int w, bool normalize, bool exact, cudaStream_t s)
{
    const int row_tiles = ceil_div(h, kTileRows), col_tiles = ceil_div(w, kTileCols);
    const int64_t blocks = (int64_t)N * C * F * row_tiles * col_tiles;
    if (blocks == 0) return BC_OK;
    if (blocks > 0x7fffffffLL) return BC_ERR_BAD_SHAPE;
    {
        LaunchScope scope(KID_FORWARD_GLOBAL, s);
        forward_global_kernel<T><<<(unsigned)blocks, kThreads, 0, s>>>(integ, bp, out, C, F, h, w, row_tiles,
                                                                        col_tiles, normalize, exact);
    }
    return check_launch("forward_global");
}

int launch_forward_global_fused(const float *integ, const BoxParams &bp, const Fusion &fu, float *out, int N,
                                int C, int F, int h, int w, bool normalize, bool exact, cudaStream_t s)
{
    const int row_tiles = ceil_div(h, kTileRows), col_tiles = ceil_div(w, kTileCols);
    const int64_t blocks = (int64_t)N * C * F * row_tiles * col_tiles;
    if (blocks == 0) return BC_OK;
    if (blocks > 0x7fffffffLL) return BC_ERR_BAD_SHAPE;
    {
        LaunchScope scope(KID_FORWARD_GLOBAL, s);
        forward_global_fused_kernel<<<(unsigned)blocks, kThreads, 0, s>>>(integ, bp, fu, out, C, F, h, w, row_tiles,
                                                                         col_tiles, normalize, exact);
    }
    return check_launch("forward_global (fused)");
}

size_t backward_partials_bytes(int N, int C, int F, int h, int w, size_t elem_size)
{
    const size_t tiles = (size_t)ceil_div(h, kTileRows) * ceil_div(w, kTileCols);
    return (size_t)C * F * N * tiles * kNumSums * elem_size;
}

template <typename T>
int launch_backward_global(const T *x, const T *x_integ, const T *go_integ, const BoxParamsT<T> &bp,
                           T rep_h, T rep_w, int N, int C, int F, int h, int w, bool normalize,
                           bool exact, int need_mask, T *grad_input, T *grad_params, T *partials,
                           cudaStream_t s)
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
            backward_global_kernel<T, true><<<(unsigned)blocks, kThreads, 0, s>>>(
                x, x_integ, go_integ, bp, grad_input, partials, N, C, F, h, w, row_tiles, col_tiles,
                normalize, exact, write_gin);
        } else {
            backward_global_kernel<T, false><<<(unsigned)blocks, kThreads, 0, s>>>(
                x, x_integ, go_integ, bp, grad_input, partials, N, C, F, h, w, row_tiles, col_tiles,
                normalize, exact, write_gin);
        }
    }
    int st = check_launch("backward_global");
    if (st != BC_OK || !need_params) return st;
    return launch_finish_param_grads<T>(partials, bp, C * F, N * row_tiles * col_tiles, normalize, exact,
                                        rep_h, rep_w, need_mask, grad_params, s);
}

// the two instantiations of the general path
template int launch_finish_param_grads<float>(const float *, const BoxParamsT<float> &, int, int, bool, bool, float, float, int, float *, cudaStream_t);
template int launch_finish_param_grads<double>(const double *, const BoxParamsT<double> &, int, int, bool, bool, double, double, int, double *, cudaStream_t);
template int launch_forward_global<float>(const float *, const BoxParamsT<float> &, float *, int, int, int, int, int, bool, bool, cudaStream_t);
template int launch_forward_global<double>(const double *, const BoxParamsT<double> &, double *, int, int, int, int, int, bool, bool, cudaStream_t);
template int launch_backward_global<float>(const float *, const float *, const float *, const BoxParamsT<float> &, float, float, int, int, int, int, int, bool, bool, int, float *, float *, float *, cudaStream_t);
template int launch_backward_global<double>(const double *, const double *, const double *, const BoxParamsT<double> &, double, double, int, int, int, int, int, bool, bool, int, double *, double *, double *, cudaStream_t);

}  // namespace bc
