// Pieces shared by the tcgen05 kernels: the sampling plan of a tile, the swizzled shared-memory tile
// layout the producers write, tensor-map creation, layout staging kernels.
#pragma once

#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <type_traits>

#include "common.cuh"
#include "kernels.h"
#include "sm100_ptx.cuh"

namespace tvdcn_b200 {

template <int DIM>
inline Geo<DIM> geo_from_host(const GeoHost &h) {
    Geo<DIM> g;
    g.B = h.B; g.Cs = h.Cs; g.Cd = h.Cd; g.groups = h.groups; g.og = h.og; g.mg = h.mg; g.K = h.K;
    g.S = h.S; g.P = h.P;
    g.csg = h.Cs / h.groups;
    g.cdg = h.Cd / h.groups;
    g.cs_per_og = h.og > 0 ? h.Cs / h.og : h.Cs;
    g.cs_per_mg = h.mg > 0 ? h.Cs / h.mg : h.Cs;
    g.BP = (long long)h.B * h.P;
    for (int a = 0; a < DIM; ++a) {
        g.img[a] = h.img[a]; g.grid[a] = h.grid[a]; g.ker[a] = h.ker[a];
        g.stride[a] = h.stride[a]; g.pad[a] = h.pad[a]; g.dil[a] = h.dil[a];
    }
    return g;
}

// How the 16-bit tensor-core operands are derived from the user's data type.
enum : int {
    TC_BF16 = 0,   // bf16 data, one MMA pass
    TC_F16 = 1,    // f16 data, one MMA pass
    TC_SPLIT = 2   // f32 data, each operand split into bf16 hi + lo, three MMA passes (hi*hi + lo*hi + hi*lo)
};

constexpr int TILE_POS = 128;       // grid positions per tile = TMEM lanes
constexpr int CHUNK_C = 64;         // channels per K chunk = one 128-byte swizzle row of 16-bit values
constexpr int A_TILE_BYTES = TILE_POS * 128;

// Byte offset of 16-byte chunk `chunk` (0..7) of row `row` inside a 128-byte-swizzled tile.
__device__ __forceinline__ uint32_t sw128_offset(int row, int chunk) {
    return (uint32_t)row * 128u + (uint32_t)((chunk ^ (row & 7)) << 4);
}

// Decoded grid position of one thread.
template <int DIM>
struct PosInfo {
    bool valid;
    int b, p;
    int base[DIM];  // grid * stride - pad per axis
};

template <int DIM>
__device__ __forceinline__ void decode_in_image(const Geo<DIM> &g, PosInfo<DIM> &pi) {
    int r = pi.p;
#pragma unroll
    for (int a = DIM - 1; a >= 0; --a) {
        const int c = r % g.grid[a];
        r /= g.grid[a];
        pi.base[a] = c * g.stride[a] - g.pad[a];
    }
}

template <int DIM>
__device__ __forceinline__ PosInfo<DIM> decode_position(const Geo<DIM> &g, long long idx) {
    PosInfo<DIM> pi;
    pi.valid = idx < g.BP;
    pi.b = pi.valid ? (int)(idx / g.P) : 0;
    pi.p = pi.valid ? (int)(idx % g.P) : 0;
    decode_in_image<DIM>(g, pi);
    return pi;
}

// ---- sampling plan ------------------------------------------------------------------------------------
// One entry per (position, corner of the 2^DIM cell): where the corner's 64-channel row starts in the
// channels-last image, in 16-byte units, and the corner's interpolation weight times the mask -- as a packed
// 16-bit pair (w, w) for 16-bit data, as f32 bits for f32 data.  Unused / out-of-bounds corners point at row 0
// with weight 0, so the producers can load unconditionally.
struct PlanEntry {
    uint32_t row16;
    uint32_t w;
};

// Offsets and mask of one (position, tap, groups): loaded early, turned into plan entries later, so that the
// global-memory latency overlaps the sampling of the previous chunk.
template <int DIM>
struct RawCoords {
    float off[DIM];
    float m;
};

template <int DIM>
__device__ __forceinline__ RawCoords<DIM> load_coords(const Geo<DIM> &g, const PosInfo<DIM> &pi,
                                                      const float *__restrict__ offset,
                                                      const float *__restrict__ mask, int tap, int ogi, int mgi) {
    RawCoords<DIM> rc;
#pragma unroll
    for (int a = 0; a < DIM; ++a)
        rc.off[a] = (offset != nullptr && pi.valid)
                        ? __ldg(offset + ((((int64_t)pi.b * g.og + ogi) * g.K + tap) * DIM + a) * (int64_t)g.P + pi.p)
                        : 0.f;
    rc.m = (mask != nullptr && pi.valid)
               ? __ldg(mask + (((int64_t)pi.b * g.mg + mgi) * g.K + tap) * (int64_t)g.P + pi.p)
               : 1.f;
    return rc;
}

template <int MODE>
__device__ __forceinline__ uint32_t encode_weight(float w) {
    if constexpr (MODE == TC_SPLIT) {
        return __float_as_uint(w);
    } else if constexpr (MODE == TC_F16) {
        const __half2 h = __float2half2_rn(w);
        return *reinterpret_cast<const uint32_t *>(&h);
    } else {
        const __nv_bfloat162 h = __float2bfloat162_rn(w);
        return *reinterpret_cast<const uint32_t *>(&h);
    }
}

// Kernel coordinates of a tap (axis 0 outermost).
template <int DIM>
__device__ __forceinline__ void tap_coords(const Geo<DIM> &g, int tap, int (&tc)[DIM]) {
    int r = tap;
#pragma unroll
    for (int a = DIM - 1; a >= 0; --a) {
        tc[a] = r % g.ker[a];
        r /= g.ker[a];
    }
}

template <int DIM, int MODE>
__device__ __forceinline__ void build_plan_at(const Geo<DIM> &g, const PosInfo<DIM> &pi, const RawCoords<DIM> &rc,
                                              bool deformable, const int (&tc)[DIM], uint32_t row_scale,
                                              PlanEntry *slot);

// Writes the NC plan entries of one position.  row_scale = Cs * element size / 16.
template <int DIM, int MODE>
__device__ __forceinline__ void build_plan(const Geo<DIM> &g, const PosInfo<DIM> &pi, const RawCoords<DIM> &rc,
                                           bool deformable, int tap, uint32_t row_scale, PlanEntry *slot) {
    int tc[DIM];
    tap_coords<DIM>(g, tap, tc);
    build_plan_at<DIM, MODE>(g, pi, rc, deformable, tc, row_scale, slot);
}

// Same, with the tap's kernel coordinates already known: the divisions by the kernel extents are a quarter of
// the instructions of a plan entry, and a planner thread makes entries back to back.
template <int DIM, int MODE>
__device__ __forceinline__ void build_plan_at(const Geo<DIM> &g, const PosInfo<DIM> &pi, const RawCoords<DIM> &rc,
                                              bool deformable, const int (&tc)[DIM], uint32_t row_scale,
                                              PlanEntry *slot) {
    constexpr int NC = 1 << DIM;
    int fl[DIM];
    float fr[DIM];
#pragma unroll
    for (int a = 0; a < DIM; ++a) {
        const int base = pi.base[a] + tc[a] * g.dil[a];
        if (deformable) {
            const float pos = (float)base + rc.off[a];
            const float f = floorf(pos);
            fl[a] = (int)f;
            fr[a] = pos - f;
        } else {
            fl[a] = base;
            fr[a] = 0.f;
        }
    }
#pragma unroll
    for (int c = 0; c < NC; ++c) {
        bool ok = pi.valid && (deformable || c == 0);
        int flat = 0;
        float w = rc.m;
#pragma unroll
        for (int a = 0; a < DIM; ++a) {
            const int bit = (c >> (DIM - 1 - a)) & 1;
            const int i = (int)((unsigned)fl[a] + (unsigned)bit);
            ok = ok && ((unsigned)i < (unsigned)g.img[a]);
            flat = flat * g.img[a] + i;
            w *= bit ? fr[a] : (1.f - fr[a]);
        }
        PlanEntry e;
        // out-of-image corners read the row of zeros that follows the staged image
        e.row16 = (uint32_t)(ok ? pi.b * g.S + flat : g.B * g.S) * row_scale;
        e.w = encode_weight<MODE>(ok ? w : 0.f);
        slot[c] = e;
    }
}

__device__ __forceinline__ void unpack8(const uint4 &v, float (&f)[8], __nv_bfloat16) {
    const uint32_t u[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        f[2 * i] = __uint_as_float(u[i] << 16);
        f[2 * i + 1] = __uint_as_float(u[i] & 0xffff0000u);
    }
}
__device__ __forceinline__ void unpack8(const uint4 &v, float (&f)[8], __half) {
    const uint32_t u[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float2 p = __half22float2(*reinterpret_cast<const __half2 *>(&u[i]));
        f[2 * i] = p.x;
        f[2 * i + 1] = p.y;
    }
}
__device__ __forceinline__ uint32_t pack2(float a, float b, __nv_bfloat16) {
    const __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
    return *reinterpret_cast<const uint32_t *>(&h);
}
__device__ __forceinline__ uint32_t pack2(float a, float b, __half) {
    const __half2 h = __floats2half2_rn(a, b);
    return *reinterpret_cast<const uint32_t *>(&h);
}

// acc (+)= w * v on packed 16-bit pairs (the blend of 16-bit data stays in its own precision: the result is
// rounded to that precision for the tensor core anyway)
template <typename T16>
__device__ __forceinline__ uint32_t fma2(uint32_t w, uint32_t v, uint32_t acc) {
    if constexpr (std::is_same<T16, __half>::value) {
        const __half2 r = __hfma2(*reinterpret_cast<const __half2 *>(&w), *reinterpret_cast<const __half2 *>(&v),
                                  *reinterpret_cast<const __half2 *>(&acc));
        return *reinterpret_cast<const uint32_t *>(&r);
    } else {
        const __nv_bfloat162 r = __hfma2(*reinterpret_cast<const __nv_bfloat162 *>(&w),
                                         *reinterpret_cast<const __nv_bfloat162 *>(&v),
                                         *reinterpret_cast<const __nv_bfloat162 *>(&acc));
        return *reinterpret_cast<const uint32_t *>(&r);
    }
}
template <typename T16>
__device__ __forceinline__ uint32_t mul2(uint32_t w, uint32_t v) {
    if constexpr (std::is_same<T16, __half>::value) {
        const __half2 r = __hmul2(*reinterpret_cast<const __half2 *>(&w), *reinterpret_cast<const __half2 *>(&v));
        return *reinterpret_cast<const uint32_t *>(&r);
    } else {
        const __nv_bfloat162 r = __hmul2(*reinterpret_cast<const __nv_bfloat162 *>(&w),
                                         *reinterpret_cast<const __nv_bfloat162 *>(&v));
        return *reinterpret_cast<const uint32_t *>(&r);
    }
}

// Samples `nvpos` virtual positions x 64 channels into 128-byte-swizzled tiles (row = position).  Virtual
// position v belongs to sub-tile v / pos_per_sub (tiles `sub_bytes` apart, each with its own first channel
// chan16[sub], in 16-byte units) and is row v % pos_per_sub of it.  plan[v * NC + c] is the entry of corner c.
// All NT threads take part; each keeps the loads of IB positions in flight together so that global-memory
// latency is overlapped.  nvpos must be a multiple of (NT / lanes-per-position) * IB.
//   MODE TC_BF16 / TC_F16: img16 is the 16-bit image, one tile `hi`; 8 lanes x 8 channels per position.
//   MODE TC_SPLIT: img16 is the f32 image, the blend is split into bf16 hi + lo; 16 lanes x 4 channels.
template <int NC, int MODE, int NT, int IB = (NC >= 8 ? 2 : 4)>
__device__ __forceinline__ void produce_tiles(uint8_t *hi, uint8_t *lo, uint32_t sub_bytes, int pos_per_sub, int nvpos,
                                              const uint4 *__restrict__ img16, const uint32_t *chan16,
                                              const PlanEntry *plan, int tid) {
    constexpr int LPP = MODE == TC_SPLIT ? 16 : 8;
    constexpr int PPI = NT / LPP;
    const int part = tid & (LPP - 1);
    const int psub = tid / LPP;
    for (int v0 = 0; v0 < nvpos; v0 += PPI * IB) {
        uint4 v[IB][NC];
        uint32_t w[IB][NC];
#pragma unroll
        for (int i = 0; i < IB; ++i) {
            const int vp = v0 + i * PPI + psub;
            const uint4 *src = img16 + chan16[(v0 + i * PPI) / pos_per_sub] + part;
            const PlanEntry *pe = plan + vp * NC;
#pragma unroll
            for (int c = 0; c < NC; ++c) {
                const PlanEntry e = pe[c];
                w[i][c] = e.w;
                v[i][c] = __ldg(src + e.row16);
            }
        }
#pragma unroll
        for (int i = 0; i < IB; ++i) {
            const int vp = v0 + i * PPI + psub;
            const int sub = (v0 + i * PPI) / pos_per_sub;
            const int pos = vp - sub * pos_per_sub;
            uint8_t *dst_hi = hi + (size_t)sub * sub_bytes;
            if constexpr (MODE != TC_SPLIT) {
                using T16 = typename std::conditional<MODE == TC_F16, __half, __nv_bfloat16>::type;
                uint4 o;
                o.x = mul2<T16>(w[i][0], v[i][0].x);
                o.y = mul2<T16>(w[i][0], v[i][0].y);
                o.z = mul2<T16>(w[i][0], v[i][0].z);
                o.w = mul2<T16>(w[i][0], v[i][0].w);
#pragma unroll
                for (int c = 1; c < NC; ++c) {
                    o.x = fma2<T16>(w[i][c], v[i][c].x, o.x);
                    o.y = fma2<T16>(w[i][c], v[i][c].y, o.y);
                    o.z = fma2<T16>(w[i][c], v[i][c].z, o.z);
                    o.w = fma2<T16>(w[i][c], v[i][c].w, o.w);
                }
                *reinterpret_cast<uint4 *>(dst_hi + sw128_offset(pos, part)) = o;
            } else {
                uint8_t *dst_lo = lo + (size_t)sub * sub_bytes;
                float acc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
                for (int c = 0; c < NC; ++c) {
                    const float wf = __uint_as_float(w[i][c]);
                    acc[0] = fmaf(wf, __uint_as_float(v[i][c].x), acc[0]);
                    acc[1] = fmaf(wf, __uint_as_float(v[i][c].y), acc[1]);
                    acc[2] = fmaf(wf, __uint_as_float(v[i][c].z), acc[2]);
                    acc[3] = fmaf(wf, __uint_as_float(v[i][c].w), acc[3]);
                }
                // hi = bf16(acc) by truncation-free rounding, lo = bf16(acc - hi)
                const uint32_t h01 = pack2(acc[0], acc[1], __nv_bfloat16());
                const uint32_t h23 = pack2(acc[2], acc[3], __nv_bfloat16());
                const float l0 = acc[0] - __uint_as_float(h01 << 16);
                const float l1 = acc[1] - __uint_as_float(h01 & 0xffff0000u);
                const float l2 = acc[2] - __uint_as_float(h23 << 16);
                const float l3 = acc[3] - __uint_as_float(h23 & 0xffff0000u);
                uint2 oh, ol;
                oh.x = h01;
                oh.y = h23;
                ol.x = pack2(l0, l1, __nv_bfloat16());
                ol.y = pack2(l2, l3, __nv_bfloat16());
                const uint32_t off = sw128_offset(pos, part >> 1) + (uint32_t)(part & 1) * 8u;
                *reinterpret_cast<uint2 *>(dst_hi + off) = oh;
                *reinterpret_cast<uint2 *>(dst_lo + off) = ol;
            }
        }
    }
}

// ---- host helpers ---------------------------------------------------------------------------------
// 16-bit tiled tensor map with 128-byte swizzle; dims innermost first.  Returns false when the driver
// entry point is unavailable or rejects the description.
bool make_tensor_map_16bit(CUtensorMap *map, const void *base, int rank, const uint64_t *dims,
                           const uint64_t *strides_bytes /* rank-1 entries */, const uint32_t *box);

}  // namespace tvdcn_b200
