// Forward and backward gathers for planes too large to keep in shared memory whole.  A CTA owns a
// band of 32 pixel columns over the full height of a plane and gathers from integral images that
// live in global memory (written by integral_image_kernel, partly still in L2).
//
// A walk reads two windows per tap row: one around column q+lo_c on the low side of the box and one
// around q+hi_c on its high side.  For a band of 32 pixel columns the low windows of all its
// pixels fall into 33 adjacent columns of the integral image and the high windows into another
// 33, whatever the box.  The CTA copies these two column bands (all h+1 rows, 40 columns each:
// the start rounded down to a multiple of 4) into shared memory and gathers from there, so every
// tap crosses from L2 once per band.  Gathering straight from global memory in 32 x 128 tiles, as
// the general kernels do, needs four tile-sized rectangles of the integral image per tile and is
// limited by that traffic (measured: three tile shapes and addressing schemes, 189-206 us on
// 8 x 16 planes of 256 x 512 with 4 filters; the general kernel 192 us).
//
// The integral images are in the padded row layout [4 zeros | I[a][0..w] | copies of I[a][w]] with
// a pitch that is a multiple of 4 floats (launch_integral_image_f32 with band_lpad()/band_rpad()):
// clamping a tap's column to the plane becomes a clamp of the window start, and a band is made of
// 16-byte aligned row segments that 16-byte asynchronous copies (cp.async.cg) move without touching
// registers.
//
// Thread layout: one thread per pixel column, a warp = 32 adjacent columns x 32 rows, warp i of a
// CTA takes rows 32i .. 32i+31.  The 32 lanes of a warp read 32 adjacent floats of a row: no bank
// conflicts whatever the window offset, so the rectangles are dense (40 floats per row).
//
// Forward : one CTA per (plane, filter, band); FUSED adds the inference steps.
// Backward: one CTA per (plane, band); it loops over the filters (integral images of the grad_output
//           planes, mirrored boxes); the thread's 32 input values and its 32 grad-input
//           accumulators stay in registers; five partial sums per (plane, filter, band).
#include "bc_common.cuh"
#include "bc_smem_walk.cuh"

namespace bc {

namespace {

constexpr int kBand = 32;                  // pixel columns per CTA
constexpr int kRows = 32;                  // rows per thread
constexpr int kRectCols = 40;              // columns of a staged band (33 needed + alignment slack)
constexpr int kRectPitch4 = kRectCols * 4; // bytes per staged row
constexpr int kLPad = 4;                   // zeros in front of every integral-image row
constexpr size_t kBandMaxSmem = 200 * 1024;

__host__ __device__ inline int band_pitch(int w) { return (kLPad + w + 1 + (kRectCols - 1) + 3) & ~3; }
__host__ __device__ inline uint32_t rect_bytes(int h) { return (uint32_t)(h + 1) * kRectPitch4; }

__device__ __forceinline__ void copy_async16(uint32_t dst, const float *src)
{
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src));
}
__device__ __forceinline__ void copy_async_wait_all()
{
    asm volatile("cp.async.commit_group;\n cp.async.wait_group 0;" ::: "memory");
}

// Where the two bands of a CTA start: plane column of the first window of the band, clamped like
// every window start, and rounded down to a multiple of 4 (all of it may lie in the padding).
struct BandStart {
    int lo4, hi4;
};
__device__ __forceinline__ int clamp_start(int c, int w) { return min(max(c, -kLPad), w); }
__device__ __forceinline__ BandStart band_start(const BoxTaps &t, int qb, int w)
{
    BandStart s;
    s.lo4 = clamp_start(qb + t.lo_c - 1, w) & ~3;       // two's complement: rounds -1..-4 down to -4
    s.hi4 = clamp_start(qb + t.hi_c, w) & ~3;
    return s;
}

// Copies plane columns [lo4, lo4+40) and [hi4, hi4+40) of rows 0..h of one padded integral image
// (pitch floats per row, `plane` points at its first float) to the rectangles at sL32 and
// sL32 + rect_bytes(h).  The caller waits (copy_async_wait_all) and synchronises the CTA.
__device__ __forceinline__ void stage_bands(const float *__restrict__ plane, int pitch, int h, const BandStart &bs,
                                            uint32_t sL32)
{
    const float *srcL = plane + kLPad + bs.lo4, *srcH = plane + kLPad + bs.hi4;
    const uint32_t sH32 = sL32 + rect_bytes(h);
    const int n = (h + 1) * (kRectCols / 4);
    for (int i = threadIdx.x; i < n; i += blockDim.x) {
        const int row = i / (kRectCols / 4), v = i - row * (kRectCols / 4);
        const int64_t g = (int64_t)row * pitch + v * 4;
        copy_async16(sL32 + (uint32_t)(i * 16), srcL + g);
        copy_async16(sH32 + (uint32_t)(i * 16), srcH + g);
    }
}

// Shared addresses of a thread's two windows in row 0 of the rectangles.
struct ColWalk {
    uint32_t lo, hi;
    int h;
};
__device__ __forceinline__ ColWalk col_walk(const BoxTaps &t, const BandStart &bs, int q, int w, int h, uint32_t sL32)
{
    ColWalk c;
    c.lo = sL32 + (uint32_t)((clamp_start(q + t.lo_c - 1, w) - bs.lo4) * 4);
    c.hi = sL32 + rect_bytes(h) + (uint32_t)((clamp_start(q + t.hi_c, w) - bs.hi4) * 4);
    c.h = h;
    return c;
}

// The four taps of tap rows a_lo (low halves) and a_hi (high halves) of one pixel column:
// l0, l1 = window on the low side of the box, h0, h1 = window on its high side.
__device__ __forceinline__ void load_taps4(const ColWalk &cw, int a_lo, int a_hi, f2_t &l0, f2_t &l1, f2_t &h0, f2_t &h1)
{
    const uint32_t o0 = (uint32_t)(min(max(a_lo, 0), cw.h) * kRectPitch4);
    const uint32_t o1 = (uint32_t)(min(max(a_hi, 0), cw.h) * kRectPitch4);
    l0 = pack2(lds<0>(cw.lo + o0), lds<0>(cw.lo + o1));
    l1 = pack2(lds<4>(cw.lo + o0), lds<4>(cw.lo + o1));
    h0 = pack2(lds<0>(cw.hi + o0), lds<0>(cw.hi + o1));
    h1 = pack2(lds<4>(cw.hi + o0), lds<4>(cw.hi + o1));
}

template <bool FUSED>
__global__ void __launch_bounds__(1024)
forward_band_kernel(const float *__restrict__ integ, BoxParams bp, Fusion fu, float *out, int C, int F, int h,
                    int w, int bands, bool normalize, bool exact)
{
    extern __shared__ float4 smem4[];
    const uint32_t sL32 = smem_u32(smem4);
    int64_t b = blockIdx.x;
    const int band = (int)(b % bands); b /= bands;
    const int f = (int)(b % F);
    const int64_t nc = b / F;
    const int c = (int)(nc % C);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int qb = band * kBand, q = qb + lane, p0 = warp * kRows;
    const int pitch = band_pitch(w);

    const Box box = load_box(bp, c * F + f);
    const BoxTaps t = taps_forward(box.xmin, box.xmax, box.ymin, box.ymax, normalize, exact);
    const BandStart bs = band_start(t, qb, w);
    stage_bands(integ + nc * (int64_t)(h + 1) * pitch, pitch, h, bs, sL32);
    copy_async_wait_all();
    __syncthreads();
    if (q >= w || p0 >= h) return;

    const ColWalk cw = col_walk(t, bs, q, w, h, sL32);
    const ColW2 k = col_weights(t);
    // scale * ((C - B) + f_hi (D - C) + f_lo (B - A)) with (A, C) and (B, D) as packed pairs
    const float sfl = t.scale * t.f_lo_r, sfh = t.scale * t.f_hi_r;
    float mul = 1.0f, add = 0.0f;
    if (FUSED) {
        if (fu.scale) mul = __ldg(fu.scale + c * F + f);
        if (fu.shift) add = __ldg(fu.shift + c * F + f);
    }
    int64_t off = (nc * F + f) * (int64_t)h * w + (int64_t)p0 * w + q;
    const int p1 = min(p0 + kRows, h);

    f2_t l0, l1, h0, h1;
    load_taps4(cw, p0 + t.lo_r - 1, p0 + t.hi_r, l0, l1, h0, h1);
    f2_t prev = fma2(k.nfl, l0, fma2(k.nwl, l1, fma2(k.fh, h1, mul2(k.wh, h0))));       // (d of row lo-1, d of row hi)
#pragma unroll 4
    for (int p = p0; p < p1; ++p) {
        load_taps4(cw, p + t.lo_r, p + t.hi_r + 1, l0, l1, h0, h1);
        const f2_t cur = fma2(k.nfl, l0, fma2(k.nwl, l1, fma2(k.fh, h1, mul2(k.wh, h0))));   // (row lo, row hi+1)
        float bb, dd, aa, cc, top, bot;
        unpack2(cur, bb, dd);
        unpack2(prev, aa, cc);
        unpack2(sub2(cur, prev), top, bot);
        float v = (cc - bb) * t.scale + sfh * bot + sfl * top;
        (void)aa; (void)dd;
        if (FUSED) {
            v = v * mul + add;
            if (fu.residual) v += fu.residual[off];       // plain load: may alias `out`
            if (fu.output_relu) v = fmaxf(v, 0.0f);
        }
        out[off] = v;
        off += w;
        prev = cur;
    }
}

template <bool NEED_PARAMS>
__global__ void __launch_bounds__(512)
backward_band_kernel(const float *__restrict__ x, const float *__restrict__ go_integ, BoxParams bp,
                     float *__restrict__ grad_input, float *__restrict__ partials, int N, int C, int F,
                     int h, int w, int bands, bool normalize, bool exact, bool write_gin)
{
    extern __shared__ float4 smem4[];
    const uint32_t sL32 = smem_u32(smem4);
    __shared__ __align__(16) float sTaps[kMaxFilters * kTapWords];
    __shared__ float red[16][kNumSums];

    const int64_t nc = blockIdx.x / bands;
    const int band = blockIdx.x % bands;
    const int c = (int)(nc % C), n = (int)(nc / C);
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, nwarps = blockDim.x >> 5;
    const int qb = band * kBand, q = qb + lane, p0 = warp * kRows;
    const bool active = q < w && p0 < h;
    const int pitch = band_pitch(w);
    const int64_t ipl = (int64_t)(h + 1) * pitch;

    if (tid < F) {
        const Box box = load_box(bp, c * F + tid);
        store_taps(sTaps + tid * kTapWords, taps_mirrored(box.xmin, box.xmax, box.ymin, box.ymax, normalize, exact));
    }

    // the thread's column of the input plane and its grad-input accumulators
    float xv[kRows], gin[kRows];
#pragma unroll
    for (int i = 0; i < kRows; ++i) {
        gin[i] = 0.0f;
        xv[i] = (NEED_PARAMS && active && p0 + i < h) ? __ldg(x + nc * (int64_t)h * w + (int64_t)(p0 + i) * w + q) : 0.0f;
    }
    __syncthreads();

    for (int f = 0; f < F; ++f) {
        const BoxTaps t = load_taps(sTaps + f * kTapWords);
        const BandStart bs = band_start(t, qb, w);
        // (the barrier that ends the previous iteration protects the rectangles and red[])
        stage_bands(go_integ + (nc * F + f) * ipl, pitch, h, bs, sL32);
        copy_async_wait_all();
        __syncthreads();

        float s_out = 0.f;
        f2_t topbot2 = pack2(0.f, 0.f);
        f2_t leftP = pack2(0.f, 0.f), leftQ = pack2(0.f, 0.f), rightP = pack2(0.f, 0.f), rightQ = pack2(0.f, 0.f);
        if (active) {
            const ColWalk cw = col_walk(t, bs, q, w, h, sL32);
            const ColW2 k = col_weights(t);
            f2_t l0, l1, h0, h1;
            load_taps4(cw, p0 + t.lo_r - 1, p0 + t.hi_r, l0, l1, h0, h1);
            // e_lo = l1 - l0, e_hi = h1 - h0, d = (h0 - l1) + f_hi e_hi + f_lo e_lo
            f2_t pel = sub2(l1, l0), peh = sub2(h1, h0);
            f2_t pd = fma2(k.fl, pel, fma2(k.fh, peh, sub2(h0, l1)));
#pragma unroll
            for (int i = 0; i < kRows; ++i) {
                const int p = p0 + i;
                if (p < h) {
                    load_taps4(cw, p + t.lo_r, p + t.hi_r + 1, l0, l1, h0, h1);
                    const f2_t cel = sub2(l1, l0), ceh = sub2(h1, h0);
                    const f2_t cd = fma2(k.fl, cel, fma2(k.fh, ceh, sub2(h0, l1)));
                    float lo_new, hi_new, lo_old, hi_old, top, bot;
                    const f2_t dd = sub2(cd, pd);
                    unpack2(cd, lo_new, hi_new);
                    unpack2(pd, lo_old, hi_old);
                    unpack2(dd, top, bot);
                    const float gg = (hi_old - lo_new) + t.f_hi_r * bot + t.f_lo_r * top;
                    (void)hi_new; (void)lo_old;
                    gin[i] += gg * t.scale;
                    if (NEED_PARAMS) {
                        const f2_t xx = pack2(xv[i], xv[i]);
                        topbot2 = fma2(xx, dd, topbot2);
                        s_out += xv[i] * gg;
                        leftP = fma2(xx, pel, leftP);
                        leftQ = fma2(xx, cel, leftQ);
                        rightP = fma2(xx, peh, rightP);
                        rightQ = fma2(xx, ceh, rightQ);
                    }
                    pd = cd; pel = cel; peh = ceh;
                }
            }
        }
        if (NEED_PARAMS) {
            float tb_top, tb_bot, la, lc, lb, ld, ra, rc, rb, rd;
            unpack2(topbot2, tb_top, tb_bot);
            unpack2(leftP, la, lc);
            unpack2(leftQ, lb, ld);
            unpack2(rightP, ra, rc);
            unpack2(rightQ, rb, rd);
            float v[kNumSums] = {s_out, tb_top, tb_bot,
                                 combine_rows(la, lb, lc, ld, t.f_lo_r, t.f_hi_r),
                                 combine_rows(ra, rb, rc, rd, t.f_lo_r, t.f_hi_r)};
#pragma unroll
            for (int j = 0; j < kNumSums; ++j) v[j] = warp_sum(v[j]);
            if (lane == 0) {
#pragma unroll
                for (int j = 0; j < kNumSums; ++j) red[warp][j] = v[j];
            }
        }
        __syncthreads();      // gathers of this filter are done: the rectangles may be refilled; red[] is complete
        if (NEED_PARAMS && tid < kNumSums) {
            float s = 0.0f;
            for (int j = 0; j < nwarps; ++j) s += red[j][tid];
            partials[(((int64_t)(c * F + f) * N + n) * bands + band) * kNumSums + tid] = s;
        }
        // red[] is written again only after the barrier that follows the next staging
    }

    if (write_gin && active) {
        float *dst = grad_input + nc * (int64_t)h * w + (int64_t)p0 * w + q;
#pragma unroll
        for (int i = 0; i < kRows; ++i)
            if (p0 + i < h) dst[(int64_t)i * w] = gin[i];
    }
}

inline int band_count(int w) { return (w + kBand - 1) / kBand; }
inline int band_threads(int h) { return 32 * ((h + kRows - 1) / kRows); }
inline size_t band_smem_bytes(int h) { return 2 * (size_t)rect_bytes(h); }

template <class K>
int band_opt_in(K kernel, size_t bytes)
{
    if (bytes <= 40 * 1024) return BC_OK;
    if (cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes))
        return cuda_failed(e, "shared memory opt-in");
    return BC_OK;
}

}  // namespace

int band_lpad() { return kLPad; }
int band_rpad(int w) { return band_pitch(w) - kLPad - (w + 1); }
size_t band_integral_floats(int64_t planes, int h, int w) { return (size_t)planes * (size_t)(h + 1) * (size_t)band_pitch(w); }

bool band_path_fits_forward(int h, int w)
{
    return h >= 1 && w >= 1 && band_threads(h) <= 1024 && band_smem_bytes(h) <= kBandMaxSmem;
}

bool band_path_fits_backward(int F, int h, int w)
{
    return h >= 1 && w >= 1 && F <= kMaxFilters && band_threads(h) <= 512 && band_smem_bytes(h) <= kBandMaxSmem;
}

// Partial sums the band backward leaves per (plane, filter): one set per sample and band.
size_t band_partials_bytes(int N, int C, int F, int w)
{
    return (size_t)C * F * N * band_count(w) * kNumSums * sizeof(float);
}

int launch_forward_band(const float *integ_padded, const BoxParams &bp, const Fusion *fu, float *out, int N, int C,
                        int F, int h, int w, bool normalize, bool exact, cudaStream_t s)
{
    const int bands = band_count(w);
    const int64_t blocks = (int64_t)N * C * F * bands;
    if (blocks == 0) return BC_OK;
    if (blocks > 0x7fffffffLL) return BC_ERR_BAD_SHAPE;
    void (*kern)(const float *, BoxParams, Fusion, float *, int, int, int, int, int, bool, bool) =
        fu ? forward_band_kernel<true> : forward_band_kernel<false>;
    const size_t smem = band_smem_bytes(h);
    int st = band_opt_in(kern, smem);
    if (st != BC_OK) return st;
    const Fusion none{0, nullptr, nullptr, nullptr, 0};
    {
        LaunchScope scope(KID_FORWARD_BAND, s);
        kern<<<(unsigned)blocks, band_threads(h), smem, s>>>(integ_padded, bp, fu ? *fu : none, out, C, F, h, w, bands,
                                                             normalize, exact);
    }
    return check_launch("forward_band");
}

int launch_backward_band(const float *x, const float *go_integ_padded, const BoxParams &bp, float rep_h, float rep_w,
                         int N, int C, int F, int h, int w, bool normalize, bool exact, int need_mask,
                         float *grad_input, float *grad_params, float *partials, cudaStream_t s)
{
    const int bands = band_count(w);
    const int64_t blocks = (int64_t)N * C * bands;
    if (blocks == 0) return BC_OK;
    if (blocks > 0x7fffffffLL) return BC_ERR_BAD_SHAPE;
    const bool need_params = (need_mask & (BC_NEED_ALL & ~BC_NEED_INPUT)) != 0;
    const bool write_gin = (need_mask & BC_NEED_INPUT) != 0;
    void (*kern)(const float *, const float *, BoxParams, float *, float *, int, int, int, int, int, int, bool, bool, bool) =
        need_params ? backward_band_kernel<true> : backward_band_kernel<false>;
    const size_t smem = band_smem_bytes(h);
    int st = band_opt_in(kern, smem);
    if (st != BC_OK) return st;
    {
        LaunchScope scope(KID_BACKWARD_BAND, s);
        kern<<<(unsigned)blocks, band_threads(h), smem, s>>>(x, go_integ_padded, bp, grad_input, partials, N, C, F, h, w,
                                                             bands, normalize, exact, write_gin);
    }
    st = check_launch("backward_band");
    if (st != BC_OK || !need_params) return st;
    return launch_finish_param_grads<float>(partials, bp, C * F, N * bands, normalize, exact, rep_h, rep_w,
                                            need_mask, grad_params, s);
}

}  // namespace bc
