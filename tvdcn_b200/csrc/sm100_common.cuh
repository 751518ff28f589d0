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

// Per-position sampling plan of one (tap, offset group, mask group): for every corner of the 2^DIM cell
// the row of the channels-last image it reads (batch * S + flat index; 0 when the corner is unused) and
// its interpolation weight times the mask (0 when the corner is out of bounds).
template <int DIM>
struct PlanView {
    int *rows;     // [1 << DIM][TILE_POS]
    float *wts;    // [1 << DIM][TILE_POS]
};

// Decoded grid position of one thread, fixed for the life of a tile.
template <int DIM>
struct PosInfo {
    bool valid;
    int b, p;
    int base[DIM];  // grid * stride - pad per axis
};

template <int DIM>
__device__ __forceinline__ PosInfo<DIM> decode_position(const Geo<DIM> &g, long long idx) {
    PosInfo<DIM> pi;
    pi.valid = idx < g.BP;
    pi.b = pi.valid ? (int)(idx / g.P) : 0;
    pi.p = pi.valid ? (int)(idx % g.P) : 0;
    int r = pi.p;
#pragma unroll
    for (int a = DIM - 1; a >= 0; --a) {
        const int c = r % g.grid[a];
        r /= g.grid[a];
        pi.base[a] = c * g.stride[a] - g.pad[a];
    }
    return pi;
}

// Fills this thread's slot of the plan.  want_deriv == false: weights are interpolation weight * mask.
template <int DIM>
__device__ __forceinline__ void fill_plan(const Geo<DIM> &g, const PosInfo<DIM> &pi, const float *__restrict__ offset,
                                          const float *__restrict__ mask, int tap, int ogi, int mgi, int slot, int pstride,
                                          PlanView<DIM> pv) {
    constexpr int NC = 1 << DIM;
    int fl[DIM];
    float fr[DIM];
    int r = tap;
    int tc[DIM];
#pragma unroll
    for (int a = DIM - 1; a >= 0; --a) {
        tc[a] = r % g.ker[a];
        r /= g.ker[a];
    }
#pragma unroll
    for (int a = 0; a < DIM; ++a) {
        const int base = pi.base[a] + tc[a] * g.dil[a];
        if (offset != nullptr && pi.valid) {
            const float o = __ldg(offset + ((((int64_t)pi.b * g.og + ogi) * g.K + tap) * DIM + a) * (int64_t)g.P + pi.p);
            const float pos = (float)base + o;
            const float f = floorf(pos);
            fl[a] = (int)f;
            fr[a] = pos - f;
        } else {
            fl[a] = base;
            fr[a] = 0.f;
        }
    }
    float m = 1.f;
    if (mask != nullptr && pi.valid) m = __ldg(mask + (((int64_t)pi.b * g.mg + mgi) * g.K + tap) * (int64_t)g.P + pi.p);
#pragma unroll
    for (int c = 0; c < NC; ++c) {
        bool ok = pi.valid && (offset != nullptr || c == 0);
        int flat = 0;
        float w = m;
#pragma unroll
        for (int a = 0; a < DIM; ++a) {
            const int bit = (c >> (DIM - 1 - a)) & 1;
            const int i = (int)((unsigned)fl[a] + (unsigned)bit);
            ok = ok && ((unsigned)i < (unsigned)g.img[a]);
            flat = flat * g.img[a] + i;
            w *= bit ? fr[a] : (1.f - fr[a]);
        }
        pv.rows[c * pstride + slot] = ok ? pi.b * g.S + flat : 0;
        pv.wts[c * pstride + slot] = ok ? w : 0.f;
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

// Samples `npos` positions x 64 channels into a 128-byte-swizzled tile (row = position).  `rows` / `wts`
// are one plan ([NC][TILE_POS], entry = position within the tile).  All NT threads take part; loads are
// issued unconditionally (unused corners point at row 0 with weight 0) and in batches of up to 16 per
// thread so that global-memory latency is overlapped instead of being paid once per corner.
//   MODE TC_BF16 / TC_F16: img_cl is 16-bit, one tile `hi`.
//   MODE TC_SPLIT: img_cl is f32, the blended value is split into bf16 hi + lo tiles.
template <int NC, int MODE, int NT>
__device__ __forceinline__ void produce_tile(uint8_t *hi, uint8_t *lo, const void *img_cl, int Cs, int chan0,
                                             const int *rows, const float *wts, int pstride, int npos, int tid) {
    constexpr int IB = NC >= 8 ? 2 : 4;  // positions per thread whose loads are in flight together
    if constexpr (MODE != TC_SPLIT) {
        using T16 = typename std::conditional<MODE == TC_F16, __half, __nv_bfloat16>::type;
        const T16 *img = reinterpret_cast<const T16 *>(img_cl) + chan0 + (tid & 7) * 8;
        constexpr int PPI = NT / 8;  // positions covered by one pass of all threads (8 lanes per position)
        const int psub = tid >> 3;
        for (int p0 = 0; p0 < npos; p0 += PPI * IB) {
            uint4 v[IB][NC];
            float w[IB][NC];
#pragma unroll
            for (int i = 0; i < IB; ++i) {
                const int pos = p0 + i * PPI + psub;
                if (pos < npos) {
#pragma unroll
                    for (int c = 0; c < NC; ++c) {
                        w[i][c] = wts[c * pstride + pos];
                        v[i][c] = __ldg(reinterpret_cast<const uint4 *>(img + (int64_t)rows[c * pstride + pos] * Cs));
                    }
                }
            }
#pragma unroll
            for (int i = 0; i < IB; ++i) {
                const int pos = p0 + i * PPI + psub;
                if (pos < npos) {
                    float acc[8];
#pragma unroll
                    for (int e = 0; e < 8; ++e) acc[e] = 0.f;
#pragma unroll
                    for (int c = 0; c < NC; ++c) {
                        float f[8];
                        unpack8(v[i][c], f, T16());
#pragma unroll
                        for (int e = 0; e < 8; ++e) acc[e] = fmaf(w[i][c], f[e], acc[e]);
                    }
                    uint4 o;
                    o.x = pack2(acc[0], acc[1], T16());
                    o.y = pack2(acc[2], acc[3], T16());
                    o.z = pack2(acc[4], acc[5], T16());
                    o.w = pack2(acc[6], acc[7], T16());
                    *reinterpret_cast<uint4 *>(hi + sw128_offset(pos, tid & 7)) = o;
                }
            }
        }
    } else {
        const int quad = tid & 15;
        const float *img = reinterpret_cast<const float *>(img_cl) + chan0 + quad * 4;
        constexpr int PPI = NT / 16;  // 16 lanes (4 channels each) per position
        const int psub = tid >> 4;
        for (int p0 = 0; p0 < npos; p0 += PPI * IB) {
            float4 v[IB][NC];
            float w[IB][NC];
#pragma unroll
            for (int i = 0; i < IB; ++i) {
                const int pos = p0 + i * PPI + psub;
                if (pos < npos) {
#pragma unroll
                    for (int c = 0; c < NC; ++c) {
                        w[i][c] = wts[c * pstride + pos];
                        v[i][c] = __ldg(reinterpret_cast<const float4 *>(img + (int64_t)rows[c * pstride + pos] * Cs));
                    }
                }
            }
#pragma unroll
            for (int i = 0; i < IB; ++i) {
                const int pos = p0 + i * PPI + psub;
                if (pos < npos) {
                    float acc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
                    for (int c = 0; c < NC; ++c) {
                        acc[0] = fmaf(w[i][c], v[i][c].x, acc[0]);
                        acc[1] = fmaf(w[i][c], v[i][c].y, acc[1]);
                        acc[2] = fmaf(w[i][c], v[i][c].z, acc[2]);
                        acc[3] = fmaf(w[i][c], v[i][c].w, acc[3]);
                    }
                    float h[4], l[4];
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        h[e] = __bfloat162float(__float2bfloat16_rn(acc[e]));
                        l[e] = acc[e] - h[e];
                    }
                    uint2 oh, ol;
                    oh.x = pack2(h[0], h[1], __nv_bfloat16());
                    oh.y = pack2(h[2], h[3], __nv_bfloat16());
                    ol.x = pack2(l[0], l[1], __nv_bfloat16());
                    ol.y = pack2(l[2], l[3], __nv_bfloat16());
                    const uint32_t off = sw128_offset(pos, quad >> 1) + (uint32_t)(quad & 1) * 8u;
                    *reinterpret_cast<uint2 *>(hi + off) = oh;
                    *reinterpret_cast<uint2 *>(lo + off) = ol;
                }
            }
        }
    }
}

// ---- host helpers ---------------------------------------------------------------------------------
// 16-bit tiled tensor map with 128-byte swizzle; dims innermost first.  Returns false when the driver
// entry point is unavailable or rejects the description.
bool make_tensor_map_16bit(CUtensorMap *map, const void *base, int rank, const uint64_t *dims,
                           const uint64_t *strides_bytes /* rank-1 entries */, const uint32_t *box);

// [B, C, S] -> [B, S, C], element size 2 or 4 bytes.
cudaError_t launch_to_channels_last(const void *src, void *dst, int B, int C, int S, int elem_bytes,
                                    cudaStream_t stream);
// [B, S, C] f32 -> [B, C, S] f32 (grad buffers coming back from channels-last accumulation).
cudaError_t launch_from_channels_last_f32(const float *src, void *dst, int dst_dtype, int B, int C, int S,
                                          cudaStream_t stream);

// weight [Cd, csg, K] (dtype: f32 / bf16 / f16) -> packed[g][tap][d'][s'] 16-bit (hi) and, in split mode, lo.
cudaError_t launch_pack_weight_ks(const void *w, int dtype, int mode, int groups, int cdg, int csg, int K, void *hi,
                                  void *lo, cudaStream_t stream);
// same source -> packed[g][tap][s'][d'] (reduction over dense channels contiguous)
cudaError_t launch_pack_weight_kd(const void *w, int dtype, int mode, int groups, int cdg, int csg, int K, void *hi,
                                  void *lo, cudaStream_t stream);

}  // namespace tvdcn_b200
