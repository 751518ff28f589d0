// Pieces shared by the tcgen05 kernels: the sampling plan of a tile, the swizzled shared-memory tile
// layout the producers write, tensor-map creation, layout staging kernels.
#pragma once

#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include "common.cuh"
#include "kernels.h"
#include "sm100_ptx.cuh"

namespace tvdcn_b200 {

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
                                          const float *__restrict__ mask, int tap, int ogi, int mgi, int slot,
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
        pv.rows[c * TILE_POS + slot] = ok ? pi.b * g.S + flat : 0;
        pv.wts[c * TILE_POS + slot] = ok ? w : 0.f;
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
