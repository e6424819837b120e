// Device helpers shared by the kernels that gather from an integral image held in shared memory
// (box_plane_smem.cu: whole planes; box_band_smem.cu: column bands of large planes): explicit
// 32-bit shared-memory accesses, packed fp32 arithmetic, the per-CTA table of boxes and the
// tap-row loads of a strip walk.
#pragma once
#include "bc_common.cuh"

namespace bc {

constexpr int kMaxFilters = 32;
constexpr int kTapWords = 12;

// Shared memory is addressed with 32-bit window addresses and explicit ld/st.shared so that the
// five adjacent taps of a window cost one address computation and five immediate offsets.
__device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }
template <int OFF>
__device__ __forceinline__ float lds(uint32_t a)
{
    float v;
    asm volatile("ld.shared.f32 %0, [%1+%2];" : "=f"(v) : "r"(a), "n"(OFF));
    return v;
}
template <int OFF>
__device__ __forceinline__ void sts(uint32_t a, float v)
{
    asm volatile("st.shared.f32 [%0+%1], %2;" ::"r"(a), "n"(OFF), "f"(v));
}
__device__ __forceinline__ float4 lds128(uint32_t a)
{
    float4 v;
    asm volatile("ld.shared.v4.f32 {%0,%1,%2,%3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(a));
    return v;
}
// Two floats in one 64-bit register for the packed fp32 pipe of sm_100 (add/sub/mul/fma.f32x2):
// one issue slot does the arithmetic of two lanes.  .x is the low half.
typedef unsigned long long f2_t;
__device__ __forceinline__ f2_t pack2(float lo, float hi)
{
    f2_t r;
    asm("mov.b64 %0, {%1,%2};" : "=l"(r) : "f"(lo), "f"(hi));
    return r;
}
__device__ __forceinline__ void unpack2(f2_t v, float &lo, float &hi)
{
    asm("mov.b64 {%0,%1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}
__device__ __forceinline__ f2_t fma2(f2_t a, f2_t b, f2_t c)
{
    f2_t r;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(r) : "l"(a), "l"(b), "l"(c));
    return r;
}
__device__ __forceinline__ f2_t mul2(f2_t a, f2_t b)
{
    f2_t r;
    asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
    return r;
}
__device__ __forceinline__ f2_t sub2(f2_t a, f2_t b)
{
    f2_t r;
    asm("sub.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
    return r;
}

__device__ __forceinline__ float warp_sum(float v)
{
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) v += __shfl_xor_sync(0xffffffffu, v, d);
    return v;
}

// Per-CTA table of the boxes this CTA works with (shared memory, filled once before the first
// barrier): integer tap offsets, fractions and scale of BoxTaps, padded to three 16-byte words.
__device__ __forceinline__ void store_taps(float *tab, const BoxTaps &t)
{
    int *ti = reinterpret_cast<int *>(tab);
    ti[0] = t.lo_r; ti[1] = t.hi_r; ti[2] = t.lo_c; ti[3] = t.hi_c;
    tab[4] = t.f_lo_r; tab[5] = t.f_hi_r; tab[6] = t.f_lo_c; tab[7] = t.f_hi_c;
    tab[8] = t.scale; tab[9] = 0.f; tab[10] = 0.f; tab[11] = 0.f;
}

__device__ __forceinline__ BoxTaps load_taps(const float *tab)
{
    const float4 a = *reinterpret_cast<const float4 *>(tab);
    const float4 b = *reinterpret_cast<const float4 *>(tab + 4);
    BoxTaps t;
    t.lo_r = __float_as_int(a.x); t.hi_r = __float_as_int(a.y);
    t.lo_c = __float_as_int(a.z); t.hi_c = __float_as_int(a.w);
    t.f_lo_r = b.x; t.f_hi_r = b.y; t.f_lo_c = b.z; t.f_hi_c = b.w;
    t.scale = tab[8];
    return t;
}

// Address arithmetic of a strip walk.  Tap rows are read in (lo, hi) pairs: the row on the lo
// side of the box and the row on its hi side are fetched together and their values kept as the
// two halves of packed registers, so the column combination runs on the f32x2 pipe.
struct Walk {
    uint32_t lo;      // address of the lo-side window (column clamp(q0+lo_c-1)) in row 0, no skew
    uint32_t dhi;     // byte distance from the lo window to the hi window
    int pitch4, h;
};

__device__ __forceinline__ uint32_t tap_addr(const Walk &wk, int a)
{
    a = min(max(a, 0), wk.h);
    return wk.lo + (uint32_t)(a * wk.pitch4) + (uint32_t)((a >> 3) << 2);
}

struct ColW2 {        // column weights of a box, each broadcast to both halves
    f2_t wh, fh, nwl, nfl, fl;
};

__device__ __forceinline__ ColW2 col_weights(const BoxTaps &t)
{
    ColW2 c;
    c.wh = pack2(1.0f - t.f_hi_c, 1.0f - t.f_hi_c);
    c.fh = pack2(t.f_hi_c, t.f_hi_c);
    c.nwl = pack2(t.f_lo_c - 1.0f, t.f_lo_c - 1.0f);
    c.nfl = pack2(-t.f_lo_c, -t.f_lo_c);
    c.fl = pack2(t.f_lo_c, t.f_lo_c);
    return c;
}

// Column-combined values d[m] of the tap rows a_lo (low halves) and a_hi (high halves):
//   d = (1-f_hi) h[m] + f_hi h[m+1] - (1-f_lo) l[m+1] - f_lo l[m]
__device__ __forceinline__ void load_pair(const Walk &wk, int a_lo, int a_hi, const ColW2 &cw, f2_t d[kStrip])
{
    const uint32_t al0 = tap_addr(wk, a_lo), ah0 = al0 + wk.dhi;
    const uint32_t al1 = tap_addr(wk, a_hi), ah1 = al1 + wk.dhi;
    const f2_t l0 = pack2(lds<0>(al0), lds<0>(al1)), l1 = pack2(lds<4>(al0), lds<4>(al1));
    const f2_t l2 = pack2(lds<8>(al0), lds<8>(al1)), l3 = pack2(lds<12>(al0), lds<12>(al1));
    const f2_t l4 = pack2(lds<16>(al0), lds<16>(al1));
    const f2_t h0 = pack2(lds<0>(ah0), lds<0>(ah1)), h1 = pack2(lds<4>(ah0), lds<4>(ah1));
    const f2_t h2 = pack2(lds<8>(ah0), lds<8>(ah1)), h3 = pack2(lds<12>(ah0), lds<12>(ah1));
    const f2_t h4 = pack2(lds<16>(ah0), lds<16>(ah1));
    d[0] = fma2(cw.nfl, l0, fma2(cw.nwl, l1, fma2(cw.fh, h1, mul2(cw.wh, h0))));
    d[1] = fma2(cw.nfl, l1, fma2(cw.nwl, l2, fma2(cw.fh, h2, mul2(cw.wh, h1))));
    d[2] = fma2(cw.nfl, l2, fma2(cw.nwl, l3, fma2(cw.fh, h3, mul2(cw.wh, h2))));
    d[3] = fma2(cw.nfl, l3, fma2(cw.nwl, l4, fma2(cw.fh, h4, mul2(cw.wh, h3))));
}

// Same plus the one-column strips outside the box: e_lo[m] = l[m+1]-l[m], e_hi[m] = h[m+1]-h[m],
// and d = (h[m] - l[m+1]) + f_hi e_hi[m] + f_lo e_lo[m].
__device__ __forceinline__ void load_pair_e(const Walk &wk, int a_lo, int a_hi, const ColW2 &cw, f2_t d[kStrip],
                                            f2_t el[kStrip], f2_t eh[kStrip])
{
    const uint32_t al0 = tap_addr(wk, a_lo), ah0 = al0 + wk.dhi;
    const uint32_t al1 = tap_addr(wk, a_hi), ah1 = al1 + wk.dhi;
    f2_t l[kStrip + 1], hh[kStrip + 1];
    l[0] = pack2(lds<0>(al0), lds<0>(al1)); l[1] = pack2(lds<4>(al0), lds<4>(al1));
    l[2] = pack2(lds<8>(al0), lds<8>(al1)); l[3] = pack2(lds<12>(al0), lds<12>(al1));
    l[4] = pack2(lds<16>(al0), lds<16>(al1));
    hh[0] = pack2(lds<0>(ah0), lds<0>(ah1)); hh[1] = pack2(lds<4>(ah0), lds<4>(ah1));
    hh[2] = pack2(lds<8>(ah0), lds<8>(ah1)); hh[3] = pack2(lds<12>(ah0), lds<12>(ah1));
    hh[4] = pack2(lds<16>(ah0), lds<16>(ah1));
#pragma unroll
    for (int m = 0; m < kStrip; ++m) {
        el[m] = sub2(l[m + 1], l[m]);
        eh[m] = sub2(hh[m + 1], hh[m]);
        d[m] = fma2(cw.fl, el[m], fma2(cw.fh, eh[m], sub2(hh[m], l[m + 1])));
    }
}

}  // namespace bc
