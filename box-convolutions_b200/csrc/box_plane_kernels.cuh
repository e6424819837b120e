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
//
// The kernels are instantiated twice: FAST for planes whose height is a multiple of 8 and width
// a multiple of 4 with aligned tensors (no per-row guards, one vector access per strip row), and
// a guarded version for everything else.
//
// This file holds the kernels and their launchers as templates over the storage type of the big
// tensors (Io<> below); box_plane_smem.cu instantiates them for float, box_plane_half.cu for
// __half and __nv_bfloat16.  What limits these kernels is the shared-memory data pipe: every
// output value takes about five 4-byte words from the integral image in shared memory, against
// four bytes of HBM traffic.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "bc_common.cuh"
#include "bc_smem_walk.cuh"

namespace bc {

namespace {

constexpr int kR = 8;            // rows per strip
constexpr int kTile = 32;        // a warp covers kTile x kTile pixels
constexpr int kPad = 4;          // padding columns on either side of an integral-image row
constexpr int kMaxTiles = 32;
constexpr int kMaxSmem = 200 * 1024;

__host__ __device__ inline int layout_pitch(int w) { return w + 1 + 2 * kPad; }
__host__ __device__ inline int layout_floats(int h, int w) { return (((h + 1) * layout_pitch(w) + (h >> 3) + 4) + 3) & ~3; }

inline int warp_tiles(int h, int w) { return ((w + kTile - 1) / kTile) * ((h + kTile - 1) / kTile); }

struct Geometry {
    int h, w, col_tiles, row_tiles, ntiles, pitch4;
};

__device__ __forceinline__ Geometry geometry(int h, int w)
{
    Geometry g;
    g.h = h; g.w = w;
    g.col_tiles = (w + kTile - 1) / kTile;
    g.row_tiles = (h + kTile - 1) / kTile;
    g.ntiles = g.col_tiles * g.row_tiles;
    g.pitch4 = layout_pitch(w) * 4;
    return g;
}

// Everything a thread needs to know about one of its strips; computed once per kernel.
struct Strip {
    int p0, q0, rt, ct;
    int pix;              // p0*w + q0: offset of the strip's first pixel in a plane
    uint32_t store;       // shared address of column q0 of integral row p0+1
    bool tile;            // the warp tile exists
    bool active;          // ... and this strip has pixels inside the plane
};

__device__ __forceinline__ Strip make_strip(const Geometry &g, uint32_t sI32, int wt, int cg, int rg)
{
    Strip t;
    t.rt = wt / g.col_tiles;
    t.ct = wt - t.rt * g.col_tiles;
    t.p0 = t.rt * kTile + rg * kR;
    t.q0 = t.ct * kTile + cg * kStrip;
    t.pix = t.p0 * g.w + t.q0;
    t.tile = wt < g.ntiles;
    t.active = t.tile && t.p0 < g.h && t.q0 < g.w;
    const int a = t.p0 + 1;
    t.store = sI32 + (kPad + t.q0) * 4 + a * g.pitch4 + ((a >> 3) << 2);
    return t;
}

// Zeroes what never changes in the integral image: row 0 and the left-hand padding (and column
// 0) of every row.  Followed by the barriers inside the build.
__device__ __forceinline__ void init_integral_padding(float *sI, const Geometry &g)
{
    const int pitch = g.pitch4 >> 2;
    for (int c = threadIdx.x; c < pitch; c += blockDim.x) sI[c] = 0.0f;
    for (int i = threadIdx.x; i < g.h * (kPad + 1); i += blockDim.x) {
        const int a = 1 + i / (kPad + 1), c = i - (a - 1) * (kPad + 1);
        sI[a * pitch + (a >> 3) + c] = 0.0f;
    }
}

// ---- asynchronous bulk copies (TMA, no tensor map) global -> shared, completion on an mbarrier.
// Every wait is bounded: when the limit expires the kernel counts the event in g_wait_timeouts
// and carries on, so a lost copy shows up as a reported error instead of a hung GPU.
static __device__ int g_wait_timeouts = 0;      // one counter per translation unit that includes this file
constexpr long long kWaitLimitCycles = 2000000000LL;      // about a second

__device__ __forceinline__ void mbar_init(uint32_t mbar, uint32_t count)
{
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(mbar), "r"(count) : "memory");
}
__device__ __forceinline__ void fence_mbar_init() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }
__device__ __forceinline__ void fence_proxy_async() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void bulk_load(uint32_t dst, const void *src, uint32_t bytes, uint32_t mbar)
{
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(mbar), "r"(bytes) : "memory");
    asm volatile("cp.async.bulk.shared::cta.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(dst), "l"(src), "r"(bytes), "r"(mbar) : "memory");
}
// Hint that `bytes` (a multiple of 16) at `src` (16-byte aligned) will be copied soon: brings them into L2.
__device__ __forceinline__ void bulk_prefetch_l2(const void *src, uint32_t bytes)
{
    asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(src), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_wait(uint32_t mbar, uint32_t parity)
{
    const long long t0 = clock64();
    for (;;) {
        uint32_t done;
        asm volatile("{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n"
                     " selp.u32 %0, 1, 0, p;\n}"
                     : "=r"(done) : "r"(mbar), "r"(parity), "r"(2000u) : "memory");
        if (done) return true;
        if (clock64() - t0 > kWaitLimitCycles) return false;
    }
}

// ---- storage types of the big tensors --------------------------------------------------------
// The kernels are instantiated for float, __half and __nv_bfloat16 input / grad_output / output /
// grad_input tensors.  Narrow types are converted as they are loaded and rounded to nearest as they
// are stored; the integral images, every accumulator and the parameter gradients stay float.
// load4 / store4 move the 4 values of one strip row with one instruction (16 or 8 bytes).
template <typename IO>
struct Io;

template <>
struct Io<float> {
    static constexpr int kVecBytes = 16;
    static __device__ __forceinline__ float4 load4(const float *p) { return __ldg(reinterpret_cast<const float4 *>(p)); }
    static __device__ __forceinline__ float load1(const float *p) { return __ldg(p); }
    static __device__ __forceinline__ void store4(float *p, float a, float b, float c, float d)
    {
        *reinterpret_cast<float4 *>(p) = make_float4(a, b, c, d);
    }
    static __device__ __forceinline__ void store1(float *p, float v) { *p = v; }
    static __device__ __forceinline__ float4 lds4(uint32_t a) { return lds128(a); }
};

__device__ __forceinline__ uint2 lds64(uint32_t a)
{
    uint2 v;
    asm volatile("ld.shared.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "r"(a));
    return v;
}

template <>
struct Io<__half> {
    static constexpr int kVecBytes = 8;
    static __device__ __forceinline__ float4 widen(uint2 r)
    {
        const float2 a = __half22float2(*reinterpret_cast<const __half2 *>(&r.x));
        const float2 b = __half22float2(*reinterpret_cast<const __half2 *>(&r.y));
        return make_float4(a.x, a.y, b.x, b.y);
    }
    static __device__ __forceinline__ float4 load4(const __half *p) { return widen(__ldg(reinterpret_cast<const uint2 *>(p))); }
    static __device__ __forceinline__ float load1(const __half *p) { return __half2float(__ldg(p)); }
    static __device__ __forceinline__ void store4(__half *p, float a, float b, float c, float d)
    {
        const __half2 lo = __floats2half2_rn(a, b), hi = __floats2half2_rn(c, d);
        uint2 r;
        r.x = *reinterpret_cast<const uint32_t *>(&lo);
        r.y = *reinterpret_cast<const uint32_t *>(&hi);
        *reinterpret_cast<uint2 *>(p) = r;
    }
    static __device__ __forceinline__ void store1(__half *p, float v) { *p = __float2half_rn(v); }
    static __device__ __forceinline__ float4 lds4(uint32_t a) { return widen(lds64(a)); }
};

template <>
struct Io<__nv_bfloat16> {
    static constexpr int kVecBytes = 8;
    static __device__ __forceinline__ float4 widen(uint2 r)
    {
        const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162 *>(&r.x));
        const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162 *>(&r.y));
        return make_float4(a.x, a.y, b.x, b.y);
    }
    static __device__ __forceinline__ float4 load4(const __nv_bfloat16 *p) { return widen(__ldg(reinterpret_cast<const uint2 *>(p))); }
    static __device__ __forceinline__ float load1(const __nv_bfloat16 *p) { return __bfloat162float(__ldg(p)); }
    static __device__ __forceinline__ void store4(__nv_bfloat16 *p, float a, float b, float c, float d)
    {
        const __nv_bfloat162 lo = __floats2bfloat162_rn(a, b), hi = __floats2bfloat162_rn(c, d);
        uint2 r;
        r.x = *reinterpret_cast<const uint32_t *>(&lo);
        r.y = *reinterpret_cast<const uint32_t *>(&hi);
        *reinterpret_cast<uint2 *>(p) = r;
    }
    static __device__ __forceinline__ void store1(__nv_bfloat16 *p, float v) { *p = __float2bfloat16_rn(v); }
    static __device__ __forceinline__ float4 lds4(uint32_t a) { return widen(lds64(a)); }
};

template <typename IO>
struct IsFloat { static constexpr bool value = false; };
template <>
struct IsFloat<float> { static constexpr bool value = true; };

// Register block of a strip while the integral image is being built.
template <int T>
struct Blocks {
    float v[T][kR][kStrip];
    float carry[T][kR];
};

// Build, part 1: fetch every strip's 8 x 4 block (from the staged copy of the plane in shared
// memory when STAGED, else from global memory), prefix it along rows inside the thread and across
// the 8 column-group lanes, publish the tile's row totals.  Ends with a barrier, after which the
// staged plane is no longer needed.
template <typename IO, int T, bool FAST, bool STAGED, bool MAYBE_RELU = false>
__device__ __forceinline__ void build_rows(Blocks<T> &b, const Strip (&st)[T], const IO *__restrict__ src,
                                           uint32_t sG32, float *sRow, const Geometry &g, int cg, int rg,
                                           bool relu = false)
{
#pragma unroll
    for (int k = 0; k < T; ++k) {
#pragma unroll
        for (int i = 0; i < kR; ++i) {
            if (STAGED) {
                const float4 t = st[k].active ? Io<IO>::lds4(sG32 + (st[k].pix + i * g.w) * (uint32_t)sizeof(IO))
                                              : make_float4(0.f, 0.f, 0.f, 0.f);
                b.v[k][i][0] = t.x; b.v[k][i][1] = t.y; b.v[k][i][2] = t.z; b.v[k][i][3] = t.w;
            } else if (FAST) {
                const float4 t = st[k].active ? Io<IO>::load4(src + st[k].pix + i * g.w) : make_float4(0.f, 0.f, 0.f, 0.f);
                b.v[k][i][0] = t.x; b.v[k][i][1] = t.y; b.v[k][i][2] = t.z; b.v[k][i][3] = t.w;
            } else {
                const bool in = st[k].active && st[k].p0 + i < g.h;
#pragma unroll
                for (int m = 0; m < kStrip; ++m)
                    b.v[k][i][m] = (in && st[k].q0 + m < g.w) ? Io<IO>::load1(src + st[k].pix + i * g.w + m) : 0.0f;
            }
        }
    }
    if (MAYBE_RELU && relu) {
#pragma unroll
        for (int k = 0; k < T; ++k)
#pragma unroll
            for (int i = 0; i < kR; ++i)
#pragma unroll
                for (int m = 0; m < kStrip; ++m) b.v[k][i][m] = fmaxf(b.v[k][i][m], 0.0f);
    }
#pragma unroll
    for (int k = 0; k < T; ++k) {
        float tot[kR];
#pragma unroll
        for (int i = 0; i < kR; ++i) {
            b.v[k][i][1] += b.v[k][i][0]; b.v[k][i][2] += b.v[k][i][1]; b.v[k][i][3] += b.v[k][i][2];
            const float own = b.v[k][i][3];
            float incl = own;
#pragma unroll
            for (int d = 1; d < 8; d <<= 1) {
                const float u = __shfl_up_sync(0xffffffffu, incl, d, 8);
                incl += cg >= d ? u : 0.0f;
            }
            b.carry[k][i] = incl - own;
            tot[i] = incl;
        }
        if (cg == 7 && st[k].tile) {
            float4 *dst = reinterpret_cast<float4 *>(sRow + (st[k].ct * g.row_tiles + st[k].rt) * kTile + rg * kR);
            dst[0] = make_float4(tot[0], tot[1], tot[2], tot[3]);
            dst[1] = make_float4(tot[4], tot[5], tot[6], tot[7]);
        }
    }
    __syncthreads();
}

// Build, part 2: row totals of the tiles to the left, prefix down the columns (thread, the 4
// row-group lanes, tiles above), store rows p0+1 .. p0+8 with the right-hand padding.  Ends with
// a barrier: the integral image is complete.
template <int T, bool FAST>
__device__ __forceinline__ void build_columns(Blocks<T> &b, const Strip (&st)[T], float *sRow, float *sCol,
                                              const Geometry &g, int cg, int rg)
{
    float ccarry[T][kStrip];
#pragma unroll
    for (int k = 0; k < T; ++k) {
        if (st[k].tile) {
            for (int c2 = 0; c2 < st[k].ct; ++c2) {
                const float4 *s = reinterpret_cast<const float4 *>(sRow + (c2 * g.row_tiles + st[k].rt) * kTile + rg * kR);
                const float4 x = s[0], y = s[1];
                b.carry[k][0] += x.x; b.carry[k][1] += x.y; b.carry[k][2] += x.z; b.carry[k][3] += x.w;
                b.carry[k][4] += y.x; b.carry[k][5] += y.y; b.carry[k][6] += y.z; b.carry[k][7] += y.w;
            }
        }
        // apply the row carry and run the in-thread column prefix in the same sweep
#pragma unroll
        for (int m = 0; m < kStrip; ++m) b.v[k][0][m] += b.carry[k][0];
#pragma unroll
        for (int i = 1; i < kR; ++i)
#pragma unroll
            for (int m = 0; m < kStrip; ++m) b.v[k][i][m] += b.carry[k][i] + b.v[k][i - 1][m];

        float tot[kStrip];
#pragma unroll
        for (int m = 0; m < kStrip; ++m) {
            const float own = b.v[k][kR - 1][m];
            float incl = own;
            float u = __shfl_up_sync(0xffffffffu, incl, 8);
            incl += rg >= 1 ? u : 0.0f;
            u = __shfl_up_sync(0xffffffffu, incl, 16);
            incl += rg >= 2 ? u : 0.0f;
            ccarry[k][m] = incl - own;
            tot[m] = incl;
        }
        if (rg == 3 && st[k].tile)
            *reinterpret_cast<float4 *>(sCol + (st[k].rt * g.col_tiles + st[k].ct) * kTile + cg * kStrip) =
                make_float4(tot[0], tot[1], tot[2], tot[3]);
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < T; ++k) {
        if (st[k].tile) {
            for (int r2 = 0; r2 < st[k].rt; ++r2) {
                const float4 x = *reinterpret_cast<const float4 *>(sCol + (r2 * g.col_tiles + st[k].ct) * kTile + cg * kStrip);
                ccarry[k][0] += x.x; ccarry[k][1] += x.y; ccarry[k][2] += x.z; ccarry[k][3] += x.w;
            }
        }
        if (st[k].active) {
            const bool last = st[k].q0 + kStrip >= g.w;
            const int npad = g.w - st[k].q0;      // padding columns still to fill (1..4) when `last`
#pragma unroll
            for (int i = 0; i < kR; ++i) {
                if (FAST || st[k].p0 + i < g.h) {
                    // p0 is a multiple of 8, so only the last of the 8 rows moves to the next skew
                    const uint32_t ra = st[k].store + i * g.pitch4 + (i == kR - 1 ? 4 : 0);
                    const float x0 = b.v[k][i][0] + ccarry[k][0], x1 = b.v[k][i][1] + ccarry[k][1];
                    const float x2 = b.v[k][i][2] + ccarry[k][2], x3 = b.v[k][i][3] + ccarry[k][3];
                    // past the plane's last column the running value is I[a][w], which is exactly
                    // what the right-hand padding has to hold
                    sts<4>(ra, x0); sts<8>(ra, x1); sts<12>(ra, x2); sts<16>(ra, x3);
                    if (last) {
                        sts<20>(ra, x3);
                        if (npad > 1) sts<24>(ra, x3);
                        if (npad > 2) sts<28>(ra, x3);
                        if (npad > 3) sts<32>(ra, x3);
                    }
                }
            }
        }
    }
    __syncthreads();
}

__device__ __forceinline__ Walk make_walk(uint32_t sI32, const BoxTaps &t, int q0, const Geometry &g)
{
    const int bl = min(max(q0 + t.lo_c - 1, -kPad), g.w);
    const int bh = min(max(q0 + t.hi_c, -kPad), g.w);
    Walk o;
    o.lo = sI32 + (kPad + bl) * 4;
    o.dhi = (uint32_t)((bh - bl) * 4);
    o.pitch4 = g.pitch4;
    o.h = g.h;
    return o;
}

// FUSED: the inference steps of `Fusion` around the gather (the output may then alias the residual,
// so it is not declared restrict).
template <typename IO, int T, bool FAST, bool FUSED = false>
__global__ void __launch_bounds__(T == 1 ? 256 : 512, T == 1 ? 4 : 1)
forward_plane_kernel(const IO *__restrict__ x, BoxParams bp, IO *out, int C, int F,
                     int h, int w, int fsplit, bool normalize, bool exact, Fusion fu)
{
    extern __shared__ float4 smem4[];
    float *sI = reinterpret_cast<float *>(smem4);
    const Geometry g = geometry(h, w);
    float *sRow = sI + layout_floats(h, w);
    float *sCol = sRow + g.ntiles * kTile;
    __shared__ __align__(16) float sTaps[kMaxFilters * kTapWords];
    grid_dependency_release();

    const int64_t nc = blockIdx.x / fsplit;
    const int part = blockIdx.x % fsplit;
    const int c = (int)(nc % C);
    const int f_begin = (F * part) / fsplit, f_end = (F * (part + 1)) / fsplit;
    const uint32_t sI32 = smem_u32(sI);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
    const int cg = lane & 7, rg = lane >> 3;

    // a hint only: the plane on its way to L2 while this CTA still waits for the kernel in front
    if (FAST && IsFloat<IO>::value && threadIdx.x == 0 && part == 0)
        bulk_prefetch_l2(x + nc * (int64_t)h * w, (uint32_t)(h * w) * 4u);
    Strip st[T];
#pragma unroll
    for (int k = 0; k < T; ++k) st[k] = make_strip(g, sI32, warp + k * nwarps, cg, rg);
    init_integral_padding(sI, g);

    // everything above touches registers and shared memory only (and hints); from here on the parameters and
    // the input are read, which the kernel in front of this one in the stream may have written
    grid_dependency_wait();
    if ((int)threadIdx.x < f_end - f_begin) {
        const Box box = load_box(bp, c * F + f_begin + threadIdx.x);
        store_taps(sTaps + threadIdx.x * kTapWords,
                   taps_forward(box.xmin, box.xmax, box.ymin, box.ymax, normalize, exact));
    }
    {
        Blocks<T> blk;
        build_rows<IO, T, FAST, false, FUSED>(blk, st, x + nc * (int64_t)h * w, 0u, sRow, g, cg, rg, FUSED && fu.input_relu);
        build_columns<T, FAST>(blk, st, sRow, sCol, g, cg, rg);
    }

    for (int f = f_begin; f < f_end; ++f) {
        const BoxTaps t = load_taps(sTaps + (f - f_begin) * kTapWords);
        const ColW2 cw = col_weights(t);
        const float sfl = t.scale * t.f_lo_r, sfh = t.scale * t.f_hi_r;
        IO *o = out + (nc * F + f) * (int64_t)h * w;
        float mul = 1.0f, add = 0.0f;
        if (FUSED) {
            if (fu.scale) mul = __ldg(fu.scale + c * F + f);
            if (fu.shift) add = __ldg(fu.shift + c * F + f);
        }
#pragma unroll
        for (int k = 0; k < T; ++k) {
            if (!st[k].active) continue;
            const Walk wk = make_walk(sI32, t, st[k].q0, g);
            f2_t prev[kStrip];                 // (d of row lo-1, d of row hi) of the current pixel row
            load_pair(wk, st[k].p0 + t.lo_r - 1, st[k].p0 + t.hi_r, cw, prev);
            IO *dst = o + st[k].pix;
            const float *res = (FUSED && fu.residual) ? fu.residual + (nc * F + f) * (int64_t)h * w + st[k].pix : nullptr;
#pragma unroll
            for (int i = 0; i < kR; ++i) {
                const int p = st[k].p0 + i;
                if (FAST || p < h) {
                    f2_t cur[kStrip];          // (d of row lo, d of row hi+1)
                    load_pair(wk, p + t.lo_r, p + t.hi_r + 1, cw, cur);
                    float v[kStrip];
#pragma unroll
                    for (int m = 0; m < kStrip; ++m) {
                        // (C - B) + f_hi (D - C) + f_lo (B - A), times scale
                        float b, dd, a, cc, top, bot;
                        unpack2(cur[m], b, dd);
                        unpack2(prev[m], a, cc);
                        unpack2(sub2(cur[m], prev[m]), top, bot);
                        v[m] = (cc - b) * t.scale + sfh * bot + sfl * top;
                        (void)a; (void)dd;
                        prev[m] = cur[m];
                    }
                    if (FUSED) {
#pragma unroll
                        for (int m = 0; m < kStrip; ++m) v[m] = v[m] * mul + add;
                        if (res) {
                            if (FAST) {
                                const float4 r = *reinterpret_cast<const float4 *>(res);
                                v[0] += r.x; v[1] += r.y; v[2] += r.z; v[3] += r.w;
                            } else {
#pragma unroll
                                for (int m = 0; m < kStrip; ++m)
                                    if (st[k].q0 + m < w) v[m] += res[m];
                            }
                            res += w;
                        }
                        if (fu.output_relu) {
#pragma unroll
                            for (int m = 0; m < kStrip; ++m) v[m] = fmaxf(v[m], 0.0f);
                        }
                    }
                    if (FAST) {
                        Io<IO>::store4(dst, v[0], v[1], v[2], v[3]);
                    } else {
#pragma unroll
                        for (int m = 0; m < kStrip; ++m)
                            if (st[k].q0 + m < w) Io<IO>::store1(dst + m, v[m]);
                    }
                    dst += w;
                }
            }
        }
    }
}

// T = warp tiles per warp: grad-input accumulators are registers, so the number of strips a
// thread owns is a compile-time constant.
// STAGED: the input plane and each grad_output plane arrive in shared memory by asynchronous bulk
// copies (one instruction per plane, issued by one thread); the copy of the next grad_output
// plane runs while the current one is gathered.
// XSMEM: the input plane is kept in shared memory (else its values are read from global memory
// as they are needed, which lets planes of up to ~48 000 pixels use this kernel).
// The input plane in shared memory is float whatever IO is: float planes arrive by a bulk copy when
// STAGED, narrow ones are converted by the threads as they are copied in.
template <typename IO, int T, bool FAST, bool STAGED, bool NEED_PARAMS, bool XSMEM = true>
__global__ void __launch_bounds__(512)
backward_plane_kernel(const IO *__restrict__ x, const IO *__restrict__ grad_output, BoxParams bp,
                      IO *__restrict__ grad_input, float *__restrict__ partials, int N, int C, int F,
                      int h, int w, bool normalize, bool exact, bool write_gin)
{
    extern __shared__ float4 smem4[];
    const Geometry g = geometry(h, w);
    const int npix = h * w;
    float *sI = reinterpret_cast<float *>(smem4);          // integral(grad_output plane)
    float *sRow = sI + layout_floats(h, w);
    float *sCol = sRow + g.ntiles * kTile;
    float *sX = sCol + g.ntiles * kTile;                   // the input plane, pitch w (NEED_PARAMS)
    float *sG = sX + (NEED_PARAMS && XSMEM ? npix : 0);    // staged grad_output plane, as stored (STAGED)
    constexpr bool X_BY_COPY = STAGED && IsFloat<IO>::value;
    __shared__ __align__(16) float sTaps[kMaxFilters * kTapWords];
    __shared__ float red[16][kNumSums];
    __shared__ __align__(8) unsigned long long mbar[2];
    grid_dependency_release();

    const int64_t nc = blockIdx.x;
    const int c = (int)(nc % C), n = (int)(nc / C);
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, nwarps = blockDim.x >> 5;
    const int cg = lane & 7, rg = lane >> 3;
    const uint32_t sI32 = smem_u32(sI), sX32 = smem_u32(sX), sG32 = smem_u32(sG);
    const uint32_t mbarX = smem_u32(&mbar[0]), mbarG = smem_u32(&mbar[1]);
    const IO *gbase = grad_output + nc * F * (int64_t)npix;
    const uint32_t plane_bytes = (uint32_t)npix * (uint32_t)sizeof(IO);
    bool timed_out = false;

    Strip st[T];
#pragma unroll
    for (int k = 0; k < T; ++k) st[k] = make_strip(g, sI32, warp + k * nwarps, cg, rg);

    // The first copies are started as early as possible, by a thread of the second warp (when there is
    // one) so that they do not queue behind the box arithmetic of the first warp's threads.  That thread
    // initialises the barriers itself and so needs no CTA barrier before it uses them; the other
    // threads first wait on them after the __syncthreads() below.
    const int starter = blockDim.x > 32 ? 32 : 0;
    if (STAGED && tid == starter) {
        mbar_init(mbarX, 1);
        mbar_init(mbarG, 1);
        fence_mbar_init();
        // While this CTA waits for the kernel in front of it, its first planes can already travel to L2
        // (a hint: if that kernel is still writing them, L2 receives its writes as well).
        bulk_prefetch_l2(gbase, plane_bytes);
        if (NEED_PARAMS && X_BY_COPY) bulk_prefetch_l2(x + nc * (int64_t)npix, plane_bytes);
        grid_dependency_wait();      // grad_output and the input may come from the kernel in front
        bulk_load(sG32, gbase, plane_bytes, mbarG);
        if (NEED_PARAMS && X_BY_COPY) bulk_load(sX32, x + nc * (int64_t)npix, plane_bytes, mbarX);
        if (F > 1) bulk_prefetch_l2(gbase + (int64_t)npix, plane_bytes);
    }
    init_integral_padding(sI, g);

    // registers and shared memory only up to here; now global memory that the kernel in front of
    // this one in the stream may still be using
    grid_dependency_wait();
    if (tid < F) {
        const Box box = load_box(bp, c * F + tid);
        store_taps(sTaps + tid * kTapWords, taps_mirrored(box.xmin, box.xmax, box.ymin, box.ymax, normalize, exact));
    }
    if (STAGED) __syncthreads();                           // barriers initialised before anyone waits
    if (!X_BY_COPY && NEED_PARAMS && XSMEM) {
        // (read by the first gather, which follows the barriers of the first build)
        const IO *xp = x + nc * (int64_t)npix;
        if (FAST) {
            for (int i = tid; i < (npix >> 2); i += blockDim.x)
                reinterpret_cast<float4 *>(sX)[i] = Io<IO>::load4(xp + 4 * i);
        } else {
            for (int i = tid; i < npix; i += blockDim.x) sX[i] = Io<IO>::load1(xp + i);
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
        {
            Blocks<T> blk;
            if (STAGED) timed_out |= !mbar_wait(mbarG, f & 1);
            build_rows<IO, T, FAST, STAGED>(blk, st, gbase + f * (int64_t)npix, sG32, sRow, g, cg, rg);
            if (STAGED && tid == 0 && f + 1 < F) {
                // every thread has taken its block out of the staging buffer (barrier above)
                fence_proxy_async();
                bulk_load(sG32, gbase + (f + 1) * (int64_t)npix, plane_bytes, mbarG);
                // the plane after that one on its way to L2 already (about 1 % on 256-sample batches)
                if (f + 2 < F) bulk_prefetch_l2(gbase + (f + 2) * (int64_t)npix, plane_bytes);
            }
            build_columns<T, FAST>(blk, st, sRow, sCol, g, cg, rg);
        }
        if (!STAGED && f + 1 < F && cg == 0) {
            // pull the next grad_output plane towards L2 while this one is gathered
#pragma unroll
            for (int k = 0; k < T; ++k)
#pragma unroll
                for (int i = 0; i < kR; ++i)
                    if (st[k].active && st[k].p0 + i < h)
                        asm volatile("prefetch.global.L2 [%0];" ::"l"(gbase + (f + 1) * (int64_t)npix + st[k].pix + i * w));
        }
        if (X_BY_COPY && NEED_PARAMS && f == 0) timed_out |= !mbar_wait(mbarX, 0);

        const BoxTaps t = load_taps(sTaps + f * kTapWords);
        const ColW2 cw = col_weights(t);
        // accumulators of this filter: see ParamSums.  The strip sums are kept per tap-row pair and
        // combined after the walk: sum x*(C-B) in *1, (sum x*(B-A), sum x*(D-C)) in *2.
        // sums over the strip of x times the column-strip values of the four tap rows, kept per
        // tap-row pair: *P = (row lo-1, row hi), *Q = (row lo, row hi+1); combined after the walk
        float s_out = 0.f;
        f2_t topbot2 = pack2(0.f, 0.f);
        f2_t leftP = pack2(0.f, 0.f), leftQ = pack2(0.f, 0.f), rightP = pack2(0.f, 0.f), rightQ = pack2(0.f, 0.f);
#pragma unroll
        for (int k = 0; k < T; ++k) {
            if (st[k].active) {
                const Walk wk = make_walk(sI32, t, st[k].q0, g);
                if (NEED_PARAMS) {
                    f2_t pd[kStrip], pel[kStrip], peh[kStrip];
                    load_pair_e(wk, st[k].p0 + t.lo_r - 1, st[k].p0 + t.hi_r, cw, pd, pel, peh);
                    uint32_t xa = sX32 + st[k].pix * 4;
                    const IO *xg = x + nc * (int64_t)npix + st[k].pix;         // used when !XSMEM
#pragma unroll
                    for (int i = 0; i < kR; ++i) {
                        const int p = st[k].p0 + i;
                        if (FAST || p < h) {
                            f2_t cd[kStrip], cel[kStrip], ceh[kStrip];
                            load_pair_e(wk, p + t.lo_r, p + t.hi_r + 1, cw, cd, cel, ceh);
                            float xv[kStrip];
                            if (FAST) {
                                const float4 v = XSMEM ? lds128(xa) : Io<IO>::load4(xg);
                                xv[0] = v.x; xv[1] = v.y; xv[2] = v.z; xv[3] = v.w;
                            } else {
#pragma unroll
                                for (int m = 0; m < kStrip; ++m)
                                    xv[m] = st[k].q0 + m < w ? (XSMEM ? sX[p * w + st[k].q0 + m] : Io<IO>::load1(xg + m)) : 0.0f;
                            }
                            xa += w * 4;
                            xg += w;
#pragma unroll
                            for (int m = 0; m < kStrip; ++m) {
                                const f2_t xx = pack2(xv[m], xv[m]);
                                float lo_new, hi_new, lo_old, hi_old, top, bot;
                                // d: gather value and the two row strips
                                const f2_t dd = sub2(cd[m], pd[m]);
                                unpack2(cd[m], lo_new, hi_new);
                                unpack2(pd[m], lo_old, hi_old);
                                unpack2(dd, top, bot);
                                const float gg = (hi_old - lo_new) + t.f_hi_r * bot + t.f_lo_r * top;
                                topbot2 = fma2(xx, dd, topbot2);
                                s_out += xv[m] * gg;
                                gin[k][i][m] += gg * t.scale;
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
                    load_pair(wk, st[k].p0 + t.lo_r - 1, st[k].p0 + t.hi_r, cw, prev);
#pragma unroll
                    for (int i = 0; i < kR; ++i) {
                        const int p = st[k].p0 + i;
                        if (FAST || p < h) {
                            f2_t cur[kStrip];
                            load_pair(wk, p + t.lo_r, p + t.hi_r + 1, cw, cur);
#pragma unroll
                            for (int m = 0; m < kStrip; ++m) {
                                float b, dd, a, cc, top, bot;
                                unpack2(cur[m], b, dd);
                                unpack2(prev[m], a, cc);
                                unpack2(sub2(cur[m], prev[m]), top, bot);
                                gin[k][i][m] += ((cc - b) + t.f_hi_r * bot + t.f_lo_r * top) * t.scale;
                                (void)a; (void)dd;
                                prev[m] = cur[m];
                            }
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
        __syncthreads();      // gathers of this filter are done: sI may be rebuilt; red[] is complete
        if (NEED_PARAMS && tid < kNumSums) {
            float s = 0.0f;
            for (int j = 0; j < nwarps; ++j) s += red[j][tid];
            partials[((int64_t)(c * F + f) * N + n) * kNumSums + tid] = s;
        }
        // red[] is next written after the barriers inside the next build
    }
    if (STAGED && timed_out && lane == 0) atomicAdd(&g_wait_timeouts, 1);

    if (write_gin) {
        IO *gi = grad_input + nc * (int64_t)npix;
#pragma unroll
        for (int k = 0; k < T; ++k) {
            if (st[k].active) {
                IO *dst = gi + st[k].pix;
#pragma unroll
                for (int i = 0; i < kR; ++i) {
                    if (FAST) {
                        Io<IO>::store4(dst + i * w, gin[k][i][0], gin[k][i][1], gin[k][i][2], gin[k][i][3]);
                    } else if (st[k].p0 + i < h) {
#pragma unroll
                        for (int m = 0; m < kStrip; ++m)
                            if (st[k].q0 + m < w) Io<IO>::store1(dst + i * w + m, gin[k][i][m]);
                    }
                }
            }
        }
    }
}

template <class K>
int opt_in_smem(K kernel, size_t bytes)
{
    if (bytes <= 34 * 1024) return BC_OK;     // static scratch included, this stays under the 48 KB default
    if (cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes))
        return cuda_failed(e, "shared memory opt-in");
    return BC_OK;
}

inline bool aligned_to(const void *p, int bytes) { return (reinterpret_cast<uintptr_t>(p) & (uintptr_t)(bytes - 1)) == 0; }

inline size_t plane_forward_smem_bytes(int h, int w)
{
    return ((size_t)layout_floats(h, w) + 2 * (size_t)warp_tiles(h, w) * kTile) * sizeof(float);
}

// io_bytes: element size of the staged grad_output plane
inline size_t plane_backward_smem_bytes(int h, int w, bool need_params, bool staged, size_t io_bytes)
{
    return plane_forward_smem_bytes(h, w) + (need_params ? (size_t)h * w * sizeof(float) : 0) +
           (staged ? (size_t)h * w * io_bytes : 0);
}

inline bool plane_fits_forward(int F, int h, int w)
{
    return F <= kMaxFilters && warp_tiles(h, w) <= kMaxTiles && plane_forward_smem_bytes(h, w) <= kMaxSmem;
}

inline bool plane_fits_backward(int F, int h, int w)
{
    return F <= kMaxFilters && warp_tiles(h, w) <= kMaxTiles && plane_backward_smem_bytes(h, w, false, false, 4) <= kMaxSmem;
}

// `fu` (inference steps around the gather) exists for float tensors only.
template <typename IO>
int launch_forward_plane_t(const IO *x, const BoxParams &bp, const Fusion *fu, IO *out, int N, int C, int F, int h,
                           int w, bool normalize, bool exact, cudaStream_t s)
{
    const int64_t planes = (int64_t)N * C;
    // Split the filters of a plane over two CTAs when there are too few planes to balance 148 SMs
    // (each part rebuilds the integral image; the second read of the plane comes from L2).
    int fsplit = 1;
    if (F % 2 == 0 && planes < 148 * 6) fsplit = 2;
    while (fsplit < F && F % (fsplit * 2) == 0 && planes * fsplit * 2 <= 148 * 2) fsplit *= 2;   // tiny batches: fill the SMs
    if (planes * fsplit > 0x7fffffffLL) return BC_ERR_BAD_SHAPE;
    const size_t smem = plane_forward_smem_bytes(h, w);
    const int tiles = warp_tiles(h, w);
    // one tile per warp up to 8 tiles, two beyond (up to 16 warps: a CTA of a large plane has the SM to itself)
    const int T = tiles > 8 ? 2 : 1;
    const int warps = (tiles + T - 1) / T;
    const int vec = Io<IO>::kVecBytes;
    const bool fast = (h % kR == 0) && (w % kStrip == 0) && aligned_to(x, vec) && aligned_to(out, vec) &&
                      (!fu || !fu->residual || aligned_to(fu->residual, 16));
    void (*kern)(const IO *, BoxParams, IO *, int, int, int, int, int, bool, bool, Fusion);
    if (fu && IsFloat<IO>::value) {
        if (fast) kern = T == 1 ? forward_plane_kernel<IO, 1, true, IsFloat<IO>::value> : forward_plane_kernel<IO, 2, true, IsFloat<IO>::value>;
        else kern = T == 1 ? forward_plane_kernel<IO, 1, false, IsFloat<IO>::value> : forward_plane_kernel<IO, 2, false, IsFloat<IO>::value>;
    } else if (fu) {
        return BC_ERR_UNSUPPORTED;
    } else {
        if (fast) kern = T == 1 ? forward_plane_kernel<IO, 1, true> : forward_plane_kernel<IO, 2, true>;
        else kern = T == 1 ? forward_plane_kernel<IO, 1, false> : forward_plane_kernel<IO, 2, false>;
    }
    int st = opt_in_smem(kern, smem);
    if (st != BC_OK) return st;
    const Fusion none{0, nullptr, nullptr, nullptr, 0};
    {
        LaunchScope scope(KID_FORWARD_PLANE, s);
        if (cudaError_t e = launch_overlapped(kern, (unsigned)(planes * fsplit), warps * 32, smem, s, x, bp, out, C, F, h, w,
                                              fsplit, normalize, exact, fu ? *fu : none))
            return cuda_failed(e, "forward_plane");
    }
    return check_launch("forward_plane");
}

template <typename IO>
int launch_backward_plane_t(const IO *x, const IO *grad_output, const BoxParams &bp, float rep_h, float rep_w, int N,
                            int C, int F, int h, int w, bool normalize, bool exact, int need_mask, IO *grad_input,
                            float *grad_params, float *partials, cudaStream_t s)
{
    const int64_t planes = (int64_t)N * C;
    if (planes > 0x7fffffffLL) return BC_ERR_BAD_SHAPE;
    const bool need_params = (need_mask & (BC_NEED_ALL & ~BC_NEED_INPUT)) != 0;
    const bool write_gin = (need_mask & BC_NEED_INPUT) != 0;
    const int tiles = warp_tiles(h, w);
    const int T = tiles > 8 ? 2 : 1;
    const int warps = (tiles + T - 1) / T;
    const int vec = Io<IO>::kVecBytes;
    const size_t io = sizeof(IO);
    const bool fast = (h % kR == 0) && (w % kStrip == 0) && aligned_to(x, vec) && aligned_to(grad_output, vec) &&
                      (!write_gin || aligned_to(grad_input, vec));
    // bulk copies need 16-byte aligned planes of a multiple of 16 bytes and room for the staging buffer;
    // staging must not cost a resident CTA (two fit below ~112 KB each)
    // the input plane joins the integral image in shared memory when both fit
    const bool xsmem = !need_params || plane_backward_smem_bytes(h, w, true, false, io) <= kMaxSmem;
    const size_t with_staging = plane_backward_smem_bytes(h, w, need_params, true, io);
    const size_t two_ctas = 112 * 1024;
    const bool staged = fast && T == 1 && xsmem && with_staging <= kMaxSmem && aligned_to(grad_output, 16) &&
                        aligned_to(x, 16) && ((size_t)h * w * io) % 16 == 0 &&
                        (with_staging <= two_ctas || plane_backward_smem_bytes(h, w, need_params, false, io) > two_ctas);
    const size_t smem = plane_backward_smem_bytes(h, w, need_params && xsmem, staged, io);
    void (*kern)(const IO *, const IO *, BoxParams, IO *, float *, int, int, int, int, int, bool, bool, bool);
    if (!xsmem) {
        if (fast) kern = T == 1 ? backward_plane_kernel<IO, 1, true, false, true, false> : backward_plane_kernel<IO, 2, true, false, true, false>;
        else kern = T == 1 ? backward_plane_kernel<IO, 1, false, false, true, false> : backward_plane_kernel<IO, 2, false, false, true, false>;
    } else if (staged) {
        kern = need_params ? backward_plane_kernel<IO, 1, true, true, true> : backward_plane_kernel<IO, 1, true, true, false>;
    } else if (fast) {
        kern = T == 1 ? (need_params ? backward_plane_kernel<IO, 1, true, false, true> : backward_plane_kernel<IO, 1, true, false, false>)
                      : (need_params ? backward_plane_kernel<IO, 2, true, false, true> : backward_plane_kernel<IO, 2, true, false, false>);
    } else {
        kern = T == 1 ? (need_params ? backward_plane_kernel<IO, 1, false, false, true> : backward_plane_kernel<IO, 1, false, false, false>)
                      : (need_params ? backward_plane_kernel<IO, 2, false, false, true> : backward_plane_kernel<IO, 2, false, false, false>);
    }
    int st = opt_in_smem(kern, smem);
    if (st != BC_OK) return st;
    {
        LaunchScope scope(KID_BACKWARD_PLANE, s);
        if (cudaError_t e = launch_overlapped(kern, (unsigned)planes, warps * 32, smem, s, x, grad_output, bp, grad_input,
                                              partials, N, C, F, h, w, normalize, exact, write_gin))
            return cuda_failed(e, "backward_plane");
    }
    st = check_launch("backward_plane");
    if (st != BC_OK || !need_params) return st;
    return launch_finish_param_grads<float>(partials, bp, C * F, N, normalize, exact, rep_h, rep_w, need_mask,
                                            grad_params, s);
}

// Bounded waits that expired in the kernels of this translation unit (synchronises).
inline int read_wait_timeouts_here(int *count)
{
    if (cudaError_t e = cudaMemcpyFromSymbol(count, g_wait_timeouts, sizeof(int))) return cuda_failed(e, "read_wait_timeouts");
    return BC_OK;
}

}  // namespace

}  // namespace bc
