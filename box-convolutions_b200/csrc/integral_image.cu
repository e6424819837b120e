// Zero-padded 2-D inclusive prefix sum, one pass over HBM: every input element is read once and
// every output element written once (the reference does two column scans and two cuBLAS
// transposes, src/integral_image_cuda.cu:67-118).
//
// One CTA walks down one plane in tiles of `tile_rows` rows.
//   1. row pass   -- each warp takes rows of the tile; a lane loads 4 adjacent values (one
//                    128-bit load), sums them, the warp scans the lane totals with shuffles and a
//                    running carry joins the 128-column segments of a long row.  Results go to
//                    shared memory already in the output's (w+1)-pitch layout, zero column included.
//   2. column pass-- one thread per column adds the carry left by the tiles above and walks down
//                    the tile's rows (bank-conflict free: adjacent lanes, adjacent columns).
//   3. store pass -- the tile's rows are one contiguous range of the output.  Rows of w+1 floats
//                    are not 16-byte aligned, so the tile is placed in shared memory at the same
//                    offset modulo 16 bytes as its destination; the range is then written with
//                    128-bit stores apart from at most 3 scalar elements at either end.
#include "bc_common.cuh"

namespace bc {

namespace {

constexpr int kMaxThreads = 256;

__device__ __forceinline__ float warp_inclusive_scan(float v, int lane)
{
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
        const float u = __shfl_up_sync(0xffffffffu, v, d);
        if (lane >= d) v += u;
    }
    return v;
}

constexpr int kBatch = 8;      // 128-bit loads a lane keeps in flight: 8 x 32 lanes x 16 B = one 1024-float row

// Loads kBatch consecutive 128-column segments of a row, starting at segment seg0.
__device__ __forceinline__ float4 relu4(float4 v)
{
    return make_float4(fmaxf(v.x, 0.f), fmaxf(v.y, 0.f), fmaxf(v.z, 0.f), fmaxf(v.w, 0.f));
}

__device__ __forceinline__ void load_segments(const float4 *row4, int n4, int seg0, int lane, float4 (&buf)[kBatch])
{
#pragma unroll
    for (int k = 0; k < kBatch; ++k) {
        const int j = (seg0 + k) * 32 + lane;
        buf[k] = j < n4 ? __ldg(row4 + j) : make_float4(0.f, 0.f, 0.f, 0.f);
    }
}

// Prefix-sums the loaded segments along the row (carry `running` joins segments and batches) and
// writes them to the tile row at columns c+1.
// (the optional ReLU is applied here, where the values are consumed, so that the loads of the
// next tile stay in flight untouched)
__device__ __forceinline__ void scan_segments(const float4 (&buf)[kBatch], int n4, int seg0, int lane, int w,
                                              float *trow, float &running, bool relu)
{
#pragma unroll
    for (int k = 0; k < kBatch; ++k) {
        if ((seg0 + k) * 32 < n4) {
            float4 v = relu ? relu4(buf[k]) : buf[k];
            v.y += v.x; v.z += v.y; v.w += v.z;
            const float incl = warp_inclusive_scan(v.w, lane);
            const float add = running + (incl - v.w);
            running += __shfl_sync(0xffffffffu, incl, 31);
            const int c = ((seg0 + k) * 32 + lane) << 2;
            if (c < w) {
                trow[c + 1] = v.x + add; trow[c + 2] = v.y + add;
                trow[c + 3] = v.z + add; trow[c + 4] = v.w + add;
            }
        }
    }
}

// Halves of the register batch, for rows of at most 512 floats: a warp then keeps two rows in flight.
__device__ __forceinline__ void load_half(const float4 *row4, int n4, int lane, float4 (&buf)[kBatch], int k0)
{
#pragma unroll
    for (int k = 0; k < kBatch / 2; ++k) {
        const int j = k * 32 + lane;
        buf[k0 + k] = j < n4 ? __ldg(row4 + j) : make_float4(0.f, 0.f, 0.f, 0.f);
    }
}
__device__ __forceinline__ void scan_half(const float4 (&buf)[kBatch], int k0, int n4, int lane, int w, float *trow,
                                          float &running, bool relu)
{
#pragma unroll
    for (int k = 0; k < kBatch / 2; ++k) {
        if (k * 32 < n4) {
            float4 v = relu ? relu4(buf[k0 + k]) : buf[k0 + k];
            v.y += v.x; v.z += v.y; v.w += v.z;
            const float incl = warp_inclusive_scan(v.w, lane);
            const float add = running + (incl - v.w);
            running += __shfl_sync(0xffffffffu, incl, 31);
            const int c = (k * 32 + lane) << 2;
            if (c < w) {
                trow[c + 1] = v.x + add; trow[c + 2] = v.y + add;
                trow[c + 3] = v.z + add; trow[c + 4] = v.w + add;
            }
        }
    }
}

// PIPELINED (rows of 512..1024 floats, one row per warp; TWO: rows of 256..512 floats, two rows per warp): a lane keeps a whole row of 128-bit loads
// in flight and the next tile's row is fetched while the current tile is scanned down its columns
// and stored, so a CTA always has a full tile of loads outstanding.  Otherwise (short rows, many
// planes) the kernel stays small in registers and relies on many resident CTAs.
// BIG: 512 threads per CTA, for launches of at most one CTA per SM (twice the loads in flight)
template <bool VEC4, bool PIPELINED, bool BIG = false, bool TWO = false>
__global__ void __launch_bounds__(BIG ? 2 * kMaxThreads : kMaxThreads)
integral_image_kernel(const float *__restrict__ in, float *__restrict__ out, int plane_h, int w, int tile_rows, bool relu,
                      int band_rows, int nbands, int lpad, int rpad)
{
    // With padding every output row is written as [lpad zeros | 0, prefix sums | rpad copies of the
    // row's last value], the layout the column-band kernels copy their bands from (the copies
    // take part in the column pass like ordinary columns, so they end up as copies of I[a][w]).
    extern __shared__ float4 smem4[];
    float *tile = reinterpret_cast<float *>(smem4);           // tile_rows*pw + 4 floats
    const int pw = lpad + w + 1 + rpad;
    float *carry = tile + ((tile_rows * pw + 4 + 3) & ~3);    // w + rpad floats

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int kThreads = blockDim.x, kWarps = blockDim.x >> 5;
    // a CTA integrates rows [band*band_rows, +h) of its plane on their own (nbands = 1: the whole
    // plane); with more bands two small kernels afterwards add what lies above each band
    const int64_t plane = blockIdx.x / nbands;
    const int band = blockIdx.x % nbands;
    const int h = min(band_rows, plane_h - band * band_rows);
    const float *src = in + plane * (int64_t)plane_h * w + (int64_t)band * band_rows * w;
    float *dst = out + plane * (int64_t)(plane_h + 1) * pw + (int64_t)band * band_rows * pw;
    const int n4 = w >> 2;
    float4 pre[kBatch];      // dead in the instantiations that are not PIPELINED
    if (PIPELINED && TWO) {
#pragma unroll
        for (int rr = 0; rr < 2; ++rr)
            if (2 * warp + rr < tile_rows && 2 * warp + rr < h)
                load_half(reinterpret_cast<const float4 *>(src + (int64_t)(2 * warp + rr) * w), n4, lane, pre, rr * (kBatch / 2));
    } else if (PIPELINED && warp < tile_rows && warp < h) {
        load_segments(reinterpret_cast<const float4 *>(src + (int64_t)warp * w), n4, 0, lane, pre);
    }

    for (int c = tid; c < w + rpad; c += kThreads) carry[c] = 0.0f;
    if (band == 0)
        for (int c = tid; c < pw; c += kThreads) dst[c] = 0.0f;   // the zero row on top

    for (int r0 = 0; r0 < h; r0 += tile_rows) {
        const int rows = min(tile_rows, h - r0);
        float *gdst = dst + (int64_t)(r0 + 1) * pw;           // where this tile's rows go
        const int mis = (int)((reinterpret_cast<uintptr_t>(gdst) >> 2) & 3);
        float *t = tile + mis;

        // ---- 1. row pass
        if (PIPELINED && TWO) {
#pragma unroll
            for (int rr = 0; rr < 2; ++rr) {
                const int i = 2 * warp + rr;
                if (i < rows) {
                    float *trow = t + i * pw + lpad;
                    if (lane == 0) trow[0] = 0.0f;
                    float running = 0.0f;
                    scan_half(pre, rr * (kBatch / 2), n4, lane, w, trow, running, relu);
                    if (lane < lpad) trow[-1 - lane] = 0.0f;
                    for (int j = lane; j < rpad; j += 32) trow[w + 1 + j] = running;
                }
                const int rn = r0 + tile_rows + i;
                if (i < tile_rows && rn < h)
                    load_half(reinterpret_cast<const float4 *>(src + (int64_t)rn * w), n4, lane, pre, rr * (kBatch / 2));
            }
        } else if (PIPELINED) {
            if (warp < rows) {
                float *trow = t + warp * pw + lpad;
                if (lane == 0) trow[0] = 0.0f;
                float running = 0.0f;
                scan_segments(pre, n4, 0, lane, w, trow, running, relu);
                if (lane < lpad) trow[-1 - lane] = 0.0f;
                for (int j = lane; j < rpad; j += 32) trow[w + 1 + j] = running;
            }
            const int rn = r0 + tile_rows + warp;
            if (warp < tile_rows && rn < h)
                load_segments(reinterpret_cast<const float4 *>(src + (int64_t)rn * w), n4, 0, lane, pre);
        } else {
            for (int i = warp; i < rows; i += kWarps) {
                const float *row = src + (int64_t)(r0 + i) * w;
                float *trow = t + i * pw + lpad;
                if (lane == 0) trow[0] = 0.0f;
                float running = 0.0f;
                if (VEC4) {
                    const float4 *row4 = reinterpret_cast<const float4 *>(row);
                    float4 nxt = lane < n4 ? __ldg(row4 + lane) : make_float4(0.f, 0.f, 0.f, 0.f);
                    for (int c4 = 0; c4 < n4; c4 += 32) {
                        float4 v = relu ? relu4(nxt) : nxt;
                        const int j = c4 + 32 + lane;
                        if (c4 + 32 < n4) nxt = j < n4 ? __ldg(row4 + j) : make_float4(0.f, 0.f, 0.f, 0.f);
                        v.y += v.x; v.z += v.y; v.w += v.z;
                        const float incl = warp_inclusive_scan(v.w, lane);
                        const float add = running + (incl - v.w);
                        running += __shfl_sync(0xffffffffu, incl, 31);
                        const int c = (c4 + lane) << 2;
                        if (c < w) {
                            trow[c + 1] = v.x + add; trow[c + 2] = v.y + add;
                            trow[c + 3] = v.z + add; trow[c + 4] = v.w + add;
                        }
                    }
                } else {
                    for (int c0 = 0; c0 < w; c0 += 32) {
                        const int c = c0 + lane;
                        float v = c < w ? __ldg(row + c) : 0.0f;
                        if (relu) v = fmaxf(v, 0.0f);
                        const float incl = warp_inclusive_scan(v, lane);
                        if (c < w) trow[c + 1] = incl + running;
                        running += __shfl_sync(0xffffffffu, incl, 31);
                    }
                }
                if (lane < lpad) trow[-1 - lane] = 0.0f;
                for (int j = lane; j < rpad; j += 32) trow[w + 1 + j] = running;
            }
        }
        __syncthreads();

        // ---- 2. column pass (8 rows at a time in registers so that the loads overlap)
        for (int c = tid; c < w + rpad; c += kThreads) {
            float run = carry[c];
            float *col = t + lpad + c + 1;
            int i = 0;
            for (; i + 8 <= rows; i += 8) {
                float v[8];
#pragma unroll
                for (int k = 0; k < 8; ++k) v[k] = col[(i + k) * pw];
#pragma unroll
                for (int k = 0; k < 8; ++k) {
                    run += v[k];
                    col[(i + k) * pw] = run;
                }
            }
            for (; i < rows; ++i) {
                run += col[i * pw];
                col[i * pw] = run;
            }
            carry[c] = run;
        }
        __syncthreads();

        // ---- 3. store pass: elements [mis, mis+n) of `tile` go to gdst[-mis ...]
        const int n = rows * pw;
        const int end = mis + n;
        float *gal = gdst - mis;                               // 16-byte aligned
        for (int s = tid * 4; s < end; s += kThreads * 4) {
            if (s >= mis && s + 4 <= end) {
                *reinterpret_cast<float4 *>(gal + s) = *reinterpret_cast<const float4 *>(tile + s);
            } else {
#pragma unroll
                for (int m = 0; m < 4; ++m)
                    if (s + m >= mis && s + m < end) gal[s + m] = tile[s + m];
            }
        }
        __syncthreads();
    }
}

// float64 planes (gradient checks, not a benchmarked path): the same three passes with scalar
// 8-byte accesses, which are already full 256-byte requests per warp.
__global__ void __launch_bounds__(kMaxThreads)
integral_image_f64_kernel(const double *__restrict__ in, double *__restrict__ out, int h, int w, int tile_rows)
{
    extern __shared__ double tile64[];                         // tile_rows*(w+1) + w doubles
    const int pw = w + 1;
    double *carry = tile64 + tile_rows * pw;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int kThreads = blockDim.x, kWarps = blockDim.x >> 5;
    const int64_t plane = blockIdx.x;
    const double *src = in + plane * (int64_t)h * w;
    double *dst = out + plane * (int64_t)(h + 1) * pw;

    for (int c = tid; c < w; c += kThreads) carry[c] = 0.0;
    for (int c = tid; c < pw; c += kThreads) dst[c] = 0.0;

    for (int r0 = 0; r0 < h; r0 += tile_rows) {
        const int rows = min(tile_rows, h - r0);
        for (int i = warp; i < rows; i += kWarps) {
            const double *row = src + (int64_t)(r0 + i) * w;
            double *trow = tile64 + i * pw;
            if (lane == 0) trow[0] = 0.0;
            double running = 0.0;
            for (int c0 = 0; c0 < w; c0 += 32) {
                const int c = c0 + lane;
                double v = c < w ? __ldg(row + c) : 0.0;
#pragma unroll
                for (int d = 1; d < 32; d <<= 1) {
                    const double u = __shfl_up_sync(0xffffffffu, v, d);
                    if (lane >= d) v += u;
                }
                if (c < w) trow[c + 1] = v + running;
                running += __shfl_sync(0xffffffffu, v, 31);
            }
        }
        __syncthreads();
        for (int c = tid; c < w; c += kThreads) {
            double run = carry[c];
            double *col = tile64 + c + 1;
            for (int i = 0; i < rows; ++i) {
                run += col[i * pw];
                col[i * pw] = run;
            }
            carry[c] = run;
        }
        __syncthreads();
        double *gdst = dst + (int64_t)(r0 + 1) * pw;
        const int n = rows * pw;
        for (int s = tid; s < n; s += kThreads) gdst[s] = tile64[s];
        __syncthreads();
    }
}

// After the bands of a plane have been integrated separately: the last row of band b' (row
// (b'+1)*band_rows of the output) holds that band's column totals.  This kernel adds the totals of
// all bands above to every row of a band except its own last row, which other CTAs are reading;
// the last rows are finished afterwards by band_last_rows_kernel.  The final band has no readers
// and is updated whole.
__global__ void __launch_bounds__(256)
band_add_above_kernel(float *__restrict__ out, int plane_h, int pw, int c0, int ncols, int band_rows, int nbands,
                      int col_chunks)
{
    // columns c0 .. c0+ncols-1 of rows of pitch pw (everything to the left of c0 is zero)
    int b = blockIdx.x;
    const int chunk = b % col_chunks; b /= col_chunks;
    const int band = 1 + b % (nbands - 1);
    const int64_t plane = b / (nbands - 1);
    const int c = c0 + chunk * 256 + threadIdx.x;
    if (c >= c0 + ncols) return;
    float *base = out + plane * (int64_t)(plane_h + 1) * pw + c;
    float above = 0.0f;
    for (int k = 1; k <= band; ++k) above += base[(int64_t)k * band_rows * pw];
    const int r0 = band * band_rows + 1;
    const int r1 = band == nbands - 1 ? plane_h + 1 : (band + 1) * band_rows;    // exclusive
    int r = r0;
    for (; r + 8 <= r1; r += 8) {
        float v[8];
#pragma unroll
        for (int k = 0; k < 8; ++k) v[k] = base[(int64_t)(r + k) * pw];
#pragma unroll
        for (int k = 0; k < 8; ++k) base[(int64_t)(r + k) * pw] = v[k] + above;
    }
    for (; r < r1; ++r) base[(int64_t)r * pw] += above;
}

// Running sum down the last rows of bands 0 .. nbands-2, one thread per (plane, column).
__global__ void band_last_rows_kernel(float *__restrict__ out, int64_t planes, int plane_h, int pw, int c0, int ncols,
                                      int band_rows, int nbands)
{
    const int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x;
    if (i >= planes * ncols) return;
    const int64_t plane = i / ncols;
    const int c = c0 + (int)(i - plane * ncols);
    float *base = out + plane * (int64_t)(plane_h + 1) * pw + c;
    const int64_t stride = (int64_t)band_rows * pw;
    float run = 0.0f;
    // 16 rows at a time: the loads are independent of one another, only the sums are a chain
    for (int k0 = 1; k0 < nbands; k0 += 16) {
        float v[16];
#pragma unroll
        for (int j = 0; j < 16; ++j) v[j] = k0 + j < nbands ? base[(k0 + j) * stride] : 0.0f;
#pragma unroll
        for (int j = 0; j < 16; ++j) {
            if (k0 + j < nbands) base[(k0 + j) * stride] = v[j] + run;
            run += v[j];
        }
    }
}

}  // namespace

// Shared memory a CTA needs for tiles of `tile_rows` rows.
static size_t tile_smem_bytes(int tile_rows, int w, int lpad, int rpad)
{
    return ((size_t)((tile_rows * (lpad + w + 1 + rpad) + 4 + 3) & ~3) + (size_t)(w + rpad)) * sizeof(float);
}

template <>
int launch_integral_image<double>(const double *in, double *out, int64_t planes, int h, int w, cudaStream_t s)
{
    if (planes == 0) return BC_OK;
    if (planes > 0x7fffffffLL) return BC_ERR_BAD_SHAPE;
    const int pw = w + 1;
    int tile_rows = 4500 / pw;
    if (tile_rows < 1) tile_rows = 1;
    if (tile_rows > h) tile_rows = h > 0 ? h : 1;
    const size_t smem = ((size_t)tile_rows * pw + (size_t)w) * sizeof(double);
    if (smem > 200 * 1024) return BC_ERR_UNSUPPORTED;
    if (smem > 48 * 1024) {
        if (cudaError_t e = cudaFuncSetAttribute(integral_image_f64_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 (int)smem))
        return cuda_failed(e, "integral_image (f64): shared memory opt-in");
    }
    {
        LaunchScope scope(KID_INTEGRAL, s);
        integral_image_f64_kernel<<<(unsigned)planes, kMaxThreads, smem, s>>>(in, out, h, w, tile_rows);
    }
    return check_launch("integral_image (f64)");
}

template <>
int launch_integral_image<float>(const float *in, float *out, int64_t planes, int h, int w, cudaStream_t s)
{
    return launch_integral_image_f32(in, out, planes, h, w, false, s, 0, 0);
}

int launch_integral_image_f32(const float *in, float *out, int64_t planes, int h, int w, bool relu_in, cudaStream_t s,
                              int lpad, int rpad)
{
    if (planes == 0) return BC_OK;
    if (planes > 0x7fffffffLL) return BC_ERR_BAD_SHAPE;
    const int pw = lpad + w + 1 + rpad;
    const bool vec4 = (w % 4 == 0) && ((reinterpret_cast<uintptr_t>(in) & 15) == 0);
    // A few tall planes (at most 64) cannot fill the GPU with one CTA each (a CTA walks down its plane tile by
    // tile): cut every plane into bands of rows that are integrated side by side, then add what
    // lies above each band (two more small launches over data that is still in L2).
    int band_rows = h, nbands = 1;
    if (planes <= 64 && h >= 64 && w >= 1) {
        const int want = (int)((2 * 148 + planes - 1) / planes);          // bands per plane for ~2 CTAs per SM
        int rows = (h + want - 1) / want;
        rows = ((rows < 16 ? 16 : rows) + 7) & ~7;
        if (rows < h) {
            band_rows = rows;
            nbands = (h + rows - 1) / rows;
        }
    }
    // rows per tile: about 36 KB of shared memory, never more than a band has
    int tile_rows = 9000 / pw;
    // with at most one CTA per SM a CTA of twice the size keeps twice the loads in flight
    const int threads = planes * nbands <= 148 ? 2 * kMaxThreads : kMaxThreads;
    const bool two = vec4 && w >= 256 && w <= 64 * kBatch && band_rows >= 4 * (threads / 32);      // two rows per warp
    const bool pipelined = two || (vec4 && w >= 512 && w <= 128 * kBatch && band_rows >= 2 * (threads / 32));
    if (pipelined) tile_rows = (two ? 2 : 1) * (threads / 32);
    if (tile_rows < 1) tile_rows = 1;
    if (tile_rows > band_rows) tile_rows = band_rows > 0 ? band_rows : 1;
    const size_t smem = tile_smem_bytes(tile_rows, w, lpad, rpad);
    if (smem > 200 * 1024) return BC_ERR_UNSUPPORTED;
    void (*kern)(const float *, float *, int, int, int, bool, int, int, int, int);
    if (threads > kMaxThreads)
        kern = two ? integral_image_kernel<true, true, true, true>
                   : (pipelined ? integral_image_kernel<true, true, true>
                                : (vec4 ? integral_image_kernel<true, false, true> : integral_image_kernel<false, false, true>));
    else
        kern = two ? integral_image_kernel<true, true, false, true>
                   : (pipelined ? integral_image_kernel<true, true>
                                : (vec4 ? integral_image_kernel<true, false> : integral_image_kernel<false, false>));
    if (smem > 48 * 1024) {
        if (cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem))
        return cuda_failed(e, "integral_image: shared memory opt-in");
    }
    {
        LaunchScope scope(KID_INTEGRAL, s);
        kern<<<(unsigned)(planes * nbands), threads, smem, s>>>(in, out, h, w, tile_rows, relu_in, band_rows, nbands, lpad, rpad);
    }
    int st = check_launch("integral_image");
    if (st != BC_OK || nbands == 1) return st;
    const int c0 = lpad + 1, ncols = w + rpad;
    const int col_chunks = (ncols + 255) / 256;
    {
        LaunchScope scope(KID_INTEGRAL_BANDS, s);
        band_add_above_kernel<<<(unsigned)(planes * (nbands - 1) * col_chunks), 256, 0, s>>>(out, h, pw, c0, ncols, band_rows,
                                                                                           nbands, col_chunks);
    }
    st = check_launch("integral_image (bands)");
    if (st != BC_OK || nbands == 2) return st;       // two bands: the only last row with readers is band 0's, already final
    {
        LaunchScope scope(KID_INTEGRAL_BANDS, s);
        band_last_rows_kernel<<<(unsigned)((planes * ncols + 255) / 256), 256, 0, s>>>(out, planes, h, pw, c0, ncols, band_rows, nbands);
    }
    return check_launch("integral_image (band rows)");
}

}  // namespace bc
