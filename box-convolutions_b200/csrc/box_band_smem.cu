// Backward gather for planes too large to keep in shared memory whole: a CTA owns a band of 32
// pixel columns over the full height of a plane and gathers from integral images that live in
// global memory (written by integral_image_kernel, partly still in L2).
//
// A strip walk reads two windows per tap row: one around column q+lo_c on the low side of the box
// and one around q+hi_c on its high side.  For a band of 32 output columns the low windows of
// all its pixels fall into 33 adjacent columns of the integral image and the high windows into
// another 33, whatever the box.  The CTA copies these two column bands (all h+1 rows) into shared
// memory with coalesced loads, clamping the column index of every element to the plane while it
// does so, and then walks exactly like the whole-plane kernels (box_plane_smem.cu): every tap is
// read from global memory once per band instead of four times per 32x128 tile through L1 with
// 16-byte-strided lanes, which is what the general kernels (box_gather_global.cu) do.
//
// One CTA per (plane, band); it loops over the filters (integral images of the grad_output planes,
// mirrored boxes), grad-input accumulates in registers, the input is read from global memory with
// 128-bit loads, and five partial sums are left per (plane, filter, band).
//
// The forward pass of such planes stays with forward_global_kernel: one gather per staged band does
// not pay for the staging (measured on 256 x 512 planes: 230 us staged against 188 us direct),
// the backward pass with its heavier walk does (305 us against 432 us).
//
// Thread layout as in box_plane_smem.cu: warp = 32 x 32 pixels, lane = 8 column groups x 4 row
// groups; warp i of a CTA takes rows 32i .. 32i+31 of the band.  Shared-memory rows have a pitch
// of 33 floats plus one float of skew every 8 rows, so the 32 lanes of a warp hit 32 banks.
#include "bc_common.cuh"
#include "bc_smem_walk.cuh"

namespace bc {

namespace {

constexpr int kR = 8;                      // rows per strip
constexpr int kTile = 32;                  // rows per warp
constexpr int kBand = 32;                  // output columns per CTA
constexpr int kBandPitch4 = (kBand + 1) * 4;
constexpr size_t kBandMaxSmem = 200 * 1024;

__host__ __device__ inline int rect_floats(int h) { return (((h + 1) * (kBand + 1) + (h >> 3) + 1) + 3) & ~3; }

__device__ __forceinline__ int clampc(int v, int hi) { return min(max(v, 0), hi); }

// Asynchronous 4-byte copy global -> shared (no register in between, so a thread can have all
// the copies of a staging pass in flight at once).
__device__ __forceinline__ void copy_async4(uint32_t dst, const float *src)
{
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(dst), "l"(src));
}
__device__ __forceinline__ void copy_async_wait_all()
{
    asm volatile("cp.async.commit_group;\n cp.async.wait_group 0;" ::: "memory");
}

// Copies columns cL .. cL+32 and cH .. cH+32 (each clamped to [0, w]) of rows 0..h of the integral
// image I (pitch w+1) into the two rectangles at sL32 and sL32 + rect_bytes.  Row a of a rectangle
// starts at a*33 + a/8 floats.  A warp copies a row at a time (coalesced), then every thread one
// element of the 33rd column.  The caller waits (copy_async_wait_all) and synchronises the CTA.
__device__ __forceinline__ void stage_bands(const float *__restrict__ I, int h, int w, int cL, int cH,
                                            uint32_t sL32, uint32_t rect_bytes)
{
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
    const int ipitch = w + 1;
    const int gl = clampc(cL + lane, w), gh = clampc(cH + lane, w);
    if ((nwarps & 7) == 0) {
        // a warp's rows are a multiple of 8 apart, so the skew grows by a constant too: source
        // pointers and destination advance by fixed steps
        const float *pl = I + (int64_t)warp * ipitch + gl;
        const float *ph = I + (int64_t)warp * ipitch + gh;
        uint32_t so = sL32 + (uint32_t)(warp * kBandPitch4 + ((warp >> 3) << 2) + lane * 4);
        const int64_t gstep = (int64_t)nwarps * ipitch;
        const uint32_t sstep = (uint32_t)(nwarps * kBandPitch4 + ((nwarps >> 3) << 2));
        const int n = warp <= h ? (h - warp) / nwarps + 1 : 0;
#pragma unroll 4
        for (int k = 0; k < n; ++k) {
            copy_async4(so, pl);
            copy_async4(so + rect_bytes, ph);
            pl += gstep; ph += gstep; so += sstep;
        }
    } else {
        for (int a = warp; a <= h; a += nwarps) {
            const float *row = I + (int64_t)a * ipitch;
            const uint32_t so = sL32 + (uint32_t)(a * kBandPitch4 + ((a >> 3) << 2) + lane * 4);
            copy_async4(so, row + gl);
            copy_async4(so + rect_bytes, row + gh);
        }
    }
    const int gl32 = clampc(cL + kBand, w), gh32 = clampc(cH + kBand, w);
    for (int r = threadIdx.x; r <= h; r += blockDim.x) {
        const float *row = I + (int64_t)r * ipitch;
        const uint32_t so = sL32 + (uint32_t)(r * kBandPitch4 + ((r >> 3) << 2) + kBand * 4);
        copy_async4(so, row + gl32);
        copy_async4(so + rect_bytes, row + gh32);
    }
}

__device__ __forceinline__ Walk band_walk(uint32_t sL32, uint32_t rect_bytes, int cg, int h)
{
    Walk o;
    o.lo = sL32 + cg * kStrip * 4;
    o.dhi = rect_bytes;
    o.pitch4 = kBandPitch4;
    o.h = h;
    return o;
}

template <bool FAST, bool NEED_PARAMS>
__global__ void __launch_bounds__(512)
backward_band_kernel(const float *__restrict__ x, const float *__restrict__ go_integ, BoxParams bp,
                     float *__restrict__ grad_input, float *__restrict__ partials, int N, int C, int F,
                     int h, int w, int bands, bool normalize, bool exact, bool write_gin)
{
    extern __shared__ float4 smem4[];
    const uint32_t sL32 = smem_u32(smem4);
    const uint32_t rect_bytes = (uint32_t)rect_floats(h) * 4u;
    __shared__ __align__(16) float sTaps[kMaxFilters * kTapWords];
    __shared__ float red[16][kNumSums];

    const int64_t nc = blockIdx.x / bands;
    const int band = blockIdx.x % bands;
    const int c = (int)(nc % C), n = (int)(nc / C);
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, nwarps = blockDim.x >> 5;
    const int cg = lane & 7, rg = lane >> 3;
    const int qb = band * kBand;
    const int p0 = warp * kTile + rg * kR, q0 = qb + cg * kStrip;
    const bool active = p0 < h && q0 < w;
    const int64_t ipl = (int64_t)(h + 1) * (w + 1);

    if (tid < F) {
        const Box box = load_box(bp, c * F + tid);
        store_taps(sTaps + tid * kTapWords, taps_mirrored(box.xmin, box.xmax, box.ymin, box.ymax, normalize, exact));
    }
    __syncthreads();

    float gin[kR][kStrip];
#pragma unroll
    for (int i = 0; i < kR; ++i)
#pragma unroll
        for (int m = 0; m < kStrip; ++m) gin[i][m] = 0.0f;
    const float *xp = x + nc * (int64_t)h * w + (int64_t)p0 * w + q0;
    const Walk wk = band_walk(sL32, rect_bytes, cg, h);

    for (int f = 0; f < F; ++f) {
        const BoxTaps t = load_taps(sTaps + f * kTapWords);
        // (the barrier that ends the previous iteration protects the rectangles and red[])
        stage_bands(go_integ + (nc * F + f) * ipl, h, w, qb + t.lo_c - 1, qb + t.hi_c, sL32, rect_bytes);
        copy_async_wait_all();
        __syncthreads();

        const ColW2 cw = col_weights(t);
        // sums over the strip of x times the column-strip values of the four tap rows, kept per
        // tap-row pair: *P = (row lo-1, row hi), *Q = (row lo, row hi+1); combined after the walk
        float s_out = 0.f;
        f2_t topbot2 = pack2(0.f, 0.f);
        f2_t leftP = pack2(0.f, 0.f), leftQ = pack2(0.f, 0.f), rightP = pack2(0.f, 0.f), rightQ = pack2(0.f, 0.f);
        if (active) {
            if (NEED_PARAMS) {
                f2_t pd[kStrip], pel[kStrip], peh[kStrip];
                load_pair_e(wk, p0 + t.lo_r - 1, p0 + t.hi_r, cw, pd, pel, peh);
#pragma unroll
                for (int i = 0; i < kR; ++i) {
                    const int p = p0 + i;
                    if (FAST || p < h) {
                        float xv[kStrip];
                        if (FAST) {
                            const float4 v = __ldg(reinterpret_cast<const float4 *>(xp + (int64_t)i * w));
                            xv[0] = v.x; xv[1] = v.y; xv[2] = v.z; xv[3] = v.w;
                        } else {
#pragma unroll
                            for (int m = 0; m < kStrip; ++m) xv[m] = q0 + m < w ? __ldg(xp + (int64_t)i * w + m) : 0.0f;
                        }
                        f2_t cd[kStrip], cel[kStrip], ceh[kStrip];
                        load_pair_e(wk, p + t.lo_r, p + t.hi_r + 1, cw, cd, cel, ceh);
#pragma unroll
                        for (int m = 0; m < kStrip; ++m) {
                            const f2_t xx = pack2(xv[m], xv[m]);
                            float lo_new, hi_new, lo_old, hi_old, top, bot;
                            const f2_t dd = sub2(cd[m], pd[m]);
                            unpack2(cd[m], lo_new, hi_new);
                            unpack2(pd[m], lo_old, hi_old);
                            unpack2(dd, top, bot);
                            const float gg = (hi_old - lo_new) + t.f_hi_r * bot + t.f_lo_r * top;
                            topbot2 = fma2(xx, dd, topbot2);
                            s_out += xv[m] * gg;
                            gin[i][m] += gg * t.scale;
                            // e_lo / e_hi: the two column strips
                            leftP = fma2(xx, pel[m], leftP);
                            leftQ = fma2(xx, cel[m], leftQ);
                            rightP = fma2(xx, peh[m], rightP);
                            rightQ = fma2(xx, ceh[m], rightQ);
                            pd[m] = cd[m]; pel[m] = cel[m]; peh[m] = ceh[m];
                        }
                    }
                }
            } else {
                f2_t prev[kStrip];
                load_pair(wk, p0 + t.lo_r - 1, p0 + t.hi_r, cw, prev);
#pragma unroll
                for (int i = 0; i < kR; ++i) {
                    const int p = p0 + i;
                    if (FAST || p < h) {
                        f2_t cur[kStrip];
                        load_pair(wk, p + t.lo_r, p + t.hi_r + 1, cw, cur);
#pragma unroll
                        for (int m = 0; m < kStrip; ++m) {
                            float bb, dd, aa, cc, top, bot;
                            unpack2(cur[m], bb, dd);
                            unpack2(prev[m], aa, cc);
                            unpack2(sub2(cur[m], prev[m]), top, bot);
                            gin[i][m] += ((cc - bb) + t.f_hi_r * bot + t.f_lo_r * top) * t.scale;
                            (void)aa; (void)dd;
                            prev[m] = cur[m];
                        }
                    }
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
        float *dst = grad_input + nc * (int64_t)h * w + (int64_t)p0 * w + q0;
#pragma unroll
        for (int i = 0; i < kR; ++i) {
            if (FAST) {
                *reinterpret_cast<float4 *>(dst + (int64_t)i * w) = make_float4(gin[i][0], gin[i][1], gin[i][2], gin[i][3]);
            } else if (p0 + i < h) {
#pragma unroll
                for (int m = 0; m < kStrip; ++m)
                    if (q0 + m < w) dst[(int64_t)i * w + m] = gin[i][m];
            }
        }
    }
}

inline bool aligned16(const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }
inline int band_count(int w) { return (w + kBand - 1) / kBand; }
inline int band_threads(int h) { return 32 * ((h + kTile - 1) / kTile); }
inline size_t band_smem_bytes(int h) { return 2 * (size_t)rect_floats(h) * sizeof(float); }

template <class K>
int band_opt_in(K kernel, size_t bytes)
{
    if (bytes <= 40 * 1024) return BC_OK;
    if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes) != cudaSuccess)
        return check_launch("shared memory opt-in");
    return BC_OK;
}

}  // namespace

bool band_path_fits_backward(int F, int h, int w)
{
    return h >= 1 && w >= 1 && F <= kMaxFilters && band_threads(h) <= 512 && band_smem_bytes(h) <= kBandMaxSmem;
}

// Partial sums the band backward leaves per (plane, filter): one set per sample and band.
size_t band_partials_bytes(int N, int C, int F, int w)
{
    return (size_t)C * F * N * band_count(w) * kNumSums * sizeof(float);
}

int launch_backward_band(const float *x, const float *go_integ, const BoxParams &bp, float rep_h, float rep_w,
                         int N, int C, int F, int h, int w, bool normalize, bool exact, int need_mask,
                         float *grad_input, float *grad_params, float *partials, cudaStream_t s)
{
    const int bands = band_count(w);
    const int64_t blocks = (int64_t)N * C * bands;
    if (blocks == 0) return BC_OK;
    if (blocks > 0x7fffffffLL) return BC_ERR_BAD_SHAPE;
    const bool need_params = (need_mask & (BC_NEED_ALL & ~BC_NEED_INPUT)) != 0;
    const bool write_gin = (need_mask & BC_NEED_INPUT) != 0;
    const bool fast = (h % kR == 0) && (w % kStrip == 0) && aligned16(x) && (!write_gin || aligned16(grad_input));
    void (*kern)(const float *, const float *, BoxParams, float *, float *, int, int, int, int, int, int, bool, bool, bool);
    if (fast) kern = need_params ? backward_band_kernel<true, true> : backward_band_kernel<true, false>;
    else kern = need_params ? backward_band_kernel<false, true> : backward_band_kernel<false, false>;
    const size_t smem = band_smem_bytes(h);
    int st = band_opt_in(kern, smem);
    if (st != BC_OK) return st;
    {
        LaunchScope scope(KID_BACKWARD_BAND, s);
        kern<<<(unsigned)blocks, band_threads(h), smem, s>>>(x, go_integ, bp, grad_input, partials, N, C, F, h, w,
                                                             bands, normalize, exact, write_gin);
    }
    st = check_launch("backward_band");
    if (st != BC_OK || !need_params) return st;
    return launch_finish_param_grads<float>(partials, bp, C * F, N * bands, normalize, exact, rep_h, rep_w,
                                            need_mask, grad_params, s);
}

}  // namespace bc
