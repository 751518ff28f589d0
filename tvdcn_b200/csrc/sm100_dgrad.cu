// Tensor-core "GEMM -> scatter" kernel (tcgen05 / TMEM).
//
//   col[k | b, p] = sum_{d in group} W[d, k] * dense[b, d, p],   k = (tap, sampled channel)
// consumed straight out of tensor memory, never stored:
//   img_grad[b, s, corner]   += col * mask * corner weight                      (scatter)
//   grad_offset[b, og, tap, axis, p] += col * mask * d sample / d axis          (needs the sampled image)
//   grad_mask[b, mg, tap, p]         += col * sample                            (needs the sampled image)
//
// Replaces addmm_ + compute_grad_offset + compute_grad_mask + col2im of the reference's backward loop
// (tvdcn/csrc/ops/cuda/deform_conv2d_kernel.cpp:519-598) and addmm_ + col2im of the transposed forward
// (tvdcn/csrc/ops/cuda/deform_conv_transpose2d_kernel.cpp:333-362): the column buffer is never written.
//
// GEMM view: D[128 positions (M, TMEM lanes) x 64*nb channels of one tap (N)] over the dense channels.
//   A = dense, channels-last [B*P, Cd] 16-bit, tile [128 pos][64 d] (K-major, TMA); all reduction chunks of
//       the position tile stay resident in shared memory while the CTA walks the column blocks;
//   B = weights packed [g][tap][s'][d'] (K-major, TMA ring);
//   D = a ring of accumulators in tensor memory, so the MMA of later column blocks overlaps the epilogue.
// Epilogue: eight scatter warps (two per TMEM lane quadrant, splitting the columns) read the accumulator,
// stage it transposed in shared memory and scatter it with 16-byte vector reductions into a channels-last
// f32 image, 8 lanes per row; eight coordinate warps read the same staged tile, gather the image corners
// with 4 lanes per row and reduce one dot product <col, corner row> per corner, which gives both
// coordinate gradients.
//
// Warp roles (576 threads): warps 0-7 scatter, warps 8-15 coordinate gradients, warp 16 MMA issue + TMEM
// owner, warp 17 TMA.
#include <algorithm>
#include <type_traits>

#include "plan.h"
#include "sm100_common.cuh"

namespace tvdcn_b200 {

template <int DIM>
struct DgradParams {
    Geo<DIM> g;
    const void *img_cl;     // sampled image, channels-last (16-bit or f32); null when no coordinate gradient is wanted
    const float *offset;    // may be null
    const float *mask;      // may be null
    float *img_grad_cl;     // [B*S, Cs] f32, accumulated into; may be null
    float *goff;            // f32, accumulated into; may be null
    float *gmask;           // f32, accumulated into; may be null
    int *status;
    int nb;                 // 64-channel chunks per column block: 1 or 2
    int rc;                 // reduction chunks: cdg / 64
    int b_stages;
    int chunks_per_tap;     // csg / 64
    int g_bufs;             // staged-tile buffers per warp pair: 1 or 2
};

namespace {

constexpr int DG_PAIRS = 8;            // scatter warp + coordinate warp per (lane quadrant, column half)
constexpr int DG_MMA_WARP = 2 * DG_PAIRS;
constexpr int DG_TMA_WARP = 2 * DG_PAIRS + 1;
constexpr int DG_THREADS = (2 * DG_PAIRS + 2) * 32;
constexpr int DG_A_TILE = 128 * 128;   // [128 pos][64 d] 16-bit
constexpr int DG_TMEM_COLS = 512;

// where one corner of one position scatters to (row of the channels-last image) and with what factor
struct ScatterInfo {
    uint32_t off;   // row * Cs: element offset of the row in the channels-last image
    float scale;
};

// predicated form: no branch around the reduction
__device__ __forceinline__ void red_add_v4_if(bool p, float *addr, float a, float b, float c, float d) {
    asm volatile(
        "{\n\t"
        ".reg .pred q;\n\t"
        "setp.ne.b32 q, %5, 0;\n\t"
        "@q red.global.add.v4.f32 [%0], {%1, %2, %3, %4};\n\t"
        "}\n" ::"l"(addr), "f"(a), "f"(b), "f"(c), "f"(d), "r"((int)p)
        : "memory");
}

__device__ __forceinline__ void red_add_v4(float *addr, float a, float b, float c, float d) {
    asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(addr), "f"(a), "f"(b), "f"(c), "f"(d)
                 : "memory");
}

// <g[0..n), image row> for n channels starting at `src` (16-bit or f32 elements)
template <int N, typename TI>
struct CornerLoad;

template <int N>
struct CornerLoad<N, float> {
    float4 v[N / 4];
    __device__ __forceinline__ void load(const float *src) {
#pragma unroll
        for (int i = 0; i < N / 4; ++i) v[i] = __ldg(reinterpret_cast<const float4 *>(src) + i);
    }
    __device__ __forceinline__ float dot(const float *gv) const {
        float s = 0.f;
#pragma unroll
        for (int i = 0; i < N / 4; ++i) {
            s = fmaf(gv[4 * i], v[i].x, s);
            s = fmaf(gv[4 * i + 1], v[i].y, s);
            s = fmaf(gv[4 * i + 2], v[i].z, s);
            s = fmaf(gv[4 * i + 3], v[i].w, s);
        }
        return s;
    }
};

template <int N, typename T16>
struct CornerLoad {
    uint4 v[N / 8];
    __device__ __forceinline__ void load(const T16 *src) {
#pragma unroll
        for (int i = 0; i < N / 8; ++i) v[i] = __ldg(reinterpret_cast<const uint4 *>(src) + i);
    }
    __device__ __forceinline__ float dot(const float *gv) const {
        float s = 0.f;
#pragma unroll
        for (int i = 0; i < N / 8; ++i) {
            float f[8];
            unpack8(v[i], f, T16());
#pragma unroll
            for (int e = 0; e < 8; ++e) s = fmaf(gv[8 * i + e], f[e], s);
        }
        return s;
    }
};

// Sampling geometry of one (position, tap, offset group, mask group), kept by an epilogue thread.
template <int DIM>
struct TapGeometry {
    int fl[DIM];
    float fr[DIM];
    float mval = 1.f;
    int tap = -1, og = -1, mtap = -1, mg = -1;
};

// corner c of the 2^DIM cell: in bounds?, row of the channels-last image, interpolation weight
template <int DIM>
__device__ __forceinline__ void corner_of(const Geo<DIM> &g, const PosInfo<DIM> &pi, const TapGeometry<DIM> &tg,
                                          bool deformable, int c, bool &ok, int &rowi, float &w) {
    ok = pi.valid && (deformable || c == 0);
    int flat = 0;
    w = 1.f;
#pragma unroll
    for (int a = 0; a < DIM; ++a) {
        const int bit = (c >> (DIM - 1 - a)) & 1;
        const int i = (int)((unsigned)tg.fl[a] + (unsigned)bit);
        ok = ok && ((unsigned)i < (unsigned)g.img[a]);
        flat = flat * g.img[a] + i;
        w *= bit ? tg.fr[a] : (1.f - tg.fr[a]);
    }
    rowi = ok ? pi.b * g.S + flat : g.B * g.S;   // the row of zeros after the staged image (never scattered to: w = 0)
    if (!ok) w = 0.f;
}

template <int DIM>
__device__ __forceinline__ void load_point(const Geo<DIM> &g, const PosInfo<DIM> &pi, const float *__restrict__ offset,
                                           int tap, int ogi, TapGeometry<DIM> &tg) {
    int r = tap, tc[DIM];
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
            tg.fl[a] = (int)f;
            tg.fr[a] = pos - f;
        } else {
            tg.fl[a] = base;
            tg.fr[a] = 0.f;
        }
    }
    tg.tap = tap;
    tg.og = ogi;
}

template <int DIM>
__device__ __forceinline__ void load_mask(const Geo<DIM> &g, const PosInfo<DIM> &pi, const float *__restrict__ mask,
                                          int tap, int mgi, TapGeometry<DIM> &tg) {
    tg.mval = (mask != nullptr && pi.valid)
                  ? __ldg(mask + (((int64_t)pi.b * g.mg + mgi) * g.K + tap) * (int64_t)g.P + pi.p)
                  : 1.f;
    tg.mtap = tap;
    tg.mg = mgi;
}

// f32 data: three MMAs and twice the bytes per chunk make every role wait longer on its neighbours; sleeping between
// polls there gives 3 % (measured), for 16-bit data it costs 4 %.
template <bool BACKOFF>
__device__ __forceinline__ bool dg_wait(uint64_t *bar, uint32_t parity) {
    if constexpr (BACKOFF)
        return ptx::mbar_wait_backoff(bar, parity);
    else
        return ptx::mbar_wait(bar, parity);
}

template <int DIM, int MODE>
__global__ void __launch_bounds__(DG_THREADS, 1)
dcn_dgrad_tc_kernel(const DgradParams<DIM> P, const __grid_constant__ CUtensorMap tmap_a_hi,
                    const __grid_constant__ CUtensorMap tmap_a_lo, const __grid_constant__ CUtensorMap tmap_b_hi,
                    const __grid_constant__ CUtensorMap tmap_b_lo) {
    constexpr int NC = 1 << DIM;
    constexpr bool SPLIT = MODE == TC_SPLIT;
    constexpr int PARTS = SPLIT ? 2 : 1;
    using TI = typename std::conditional<SPLIT, float, typename std::conditional<MODE == TC_F16, __half, __nv_bfloat16>::type>::type;
    const Geo<DIM> &g = P.g;

    extern __shared__ uint8_t smem_raw[];
    // align by offset, not by integer round-trip, so that the compiler keeps these as shared-memory pointers
    uint8_t *smem = smem_raw + ((1024u - (ptx::smem_u32(smem_raw) & 1023u)) & 1023u);
    const int RC = P.rc, NB = P.nb, BS = P.b_stages;
    const int ncol = NB * 64;                       // columns per accumulator
    const int NQ = DG_TMEM_COLS / ncol;             // accumulators in the ring (8 or 4)
    const uint32_t a_bytes = (uint32_t)(RC * PARTS * DG_A_TILE);       // [rc][part]
    const uint32_t b_part_bytes = (uint32_t)(ncol * 128);
    const uint32_t b_stage_bytes = b_part_bytes * PARTS;
    uint8_t *sA = smem;
    uint8_t *sB = sA + a_bytes;
    // epilogue staging, per scatter warp: two [32 pos][32 ch] f32 tiles (double buffer shared with the paired
    // coordinate warp), scatter info [32][NC]; per coordinate warp: row offsets [32][NC] and dots [32][NC]
    float *stage_g = reinterpret_cast<float *>(sB + (size_t)BS * b_stage_bytes);          // [8][g_bufs][32*32]
    ScatterInfo *stage_c = reinterpret_cast<ScatterInfo *>(stage_g + DG_PAIRS * P.g_bufs * 1024);  // [8][32*NC]
    uint32_t *stage_r = reinterpret_cast<uint32_t *>(stage_c + DG_PAIRS * 32 * NC);         // [8][32*NC]
    float *stage_d = reinterpret_cast<float *>(stage_r + DG_PAIRS * 32 * NC);               // [8][32*NC]
    uint64_t *bars = reinterpret_cast<uint64_t *>(stage_d + DG_PAIRS * 32 * NC);
    uint64_t *a_full = bars;
    uint64_t *b_full = bars + 1;
    uint64_t *b_empty = b_full + BS;
    uint64_t *t_full = b_empty + BS;
    uint64_t *t_empty = t_full + 8;
    uint64_t *g_full = t_empty + 8;       // [8 pairs][2]: scatter warp -> coordinate warp: tile staged
    uint64_t *g_empty = g_full + 16;      // [8 pairs][2]: coordinate warp -> scatter warp: tile consumed
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(g_empty + 16);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int grp = blockIdx.y;
    const long long m0 = (long long)blockIdx.x * TILE_POS;
    // column blocks of this CTA: gridDim.z CTAs share one position tile and take equal ranges of its (tap, chunk)
    // blocks, which evens out the last wave when the tiles do not fill the SMs a whole number of times
    const int n_blocks = g.K * (P.chunks_per_tap / NB) / (int)gridDim.z;
    const int blk0 = (int)blockIdx.z * n_blocks;
    const bool want_coord = P.goff != nullptr || P.gmask != nullptr;
    const bool deformable = P.offset != nullptr;

    if (threadIdx.x == 0) {
        ptx::mbar_init(a_full, 1);
        for (int s = 0; s < BS; ++s) {
            ptx::mbar_init(&b_full[s], 1);
            ptx::mbar_init(&b_empty[s], 1);
        }
        for (int q = 0; q < 8; ++q) {
            ptx::mbar_init(&t_full[q], 1);
            ptx::mbar_init(&t_empty[q], DG_PAIRS);
        }
        for (int i = 0; i < 16; ++i) {
            ptx::mbar_init(&g_full[i], 1);
            ptx::mbar_init(&g_empty[i], SPLIT ? 1 : 2);   // 16-bit: two coordinate warps read every staged tile
        }
        ptx::fence_mbar_init();
    }
    if (warp == DG_TMA_WARP && lane == 0) {
        ptx::prefetch_tmap(&tmap_a_hi);
        ptx::prefetch_tmap(&tmap_b_hi);
        if (SPLIT) {
            ptx::prefetch_tmap(&tmap_a_lo);
            ptx::prefetch_tmap(&tmap_b_lo);
        }
    }
    if (warp == DG_MMA_WARP) {
        ptx::tmem_alloc(tmem_slot, DG_TMEM_COLS);
        ptx::tmem_relinquish();
    }
    ptx::tc_fence_before();
    __syncthreads();
    ptx::tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp < DG_PAIRS) {
        // ------------------------------------------------------------------ scatter warps
        // TMEM -> registers -> shared tile (handed to the paired coordinate warp) -> vector reductions
        const int lane_q = warp & 3, half = warp >> 2;
        const PosInfo<DIM> pi = decode_position<DIM>(g, m0 + lane_q * 32 + lane);
        TapGeometry<DIM> tg;
        ScatterInfo *cs = stage_c + warp * 32 * NC;
        const bool scatter = P.img_grad_cl != nullptr;
        int k = 0;  // chunks handled so far: selects the staging buffer
        bool ok = true;
        for (int bi = 0; bi < n_blocks && ok; ++bi) {
                const int blk = blk0 + bi;
            const int q = bi % NQ;
            const int tap = blk % g.K;
            const int cc0 = (blk / g.K) * NB;
            ok = dg_wait<SPLIT>(&t_full[q], (uint32_t)((bi / NQ) & 1));
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) {
                if (lane == 0) atomicExch(P.status, 301);
                break;
            }
            ptx::tc_fence_after();
            for (int ci = 0; ci < NB; ++ci, ++k) {
                const int chan0 = grp * g.csg + (cc0 + ci) * CHUNK_C;
                const int ch0 = chan0 + half * 32;
                const int buf = k % P.g_bufs;
                float *gs = stage_g + (warp * P.g_bufs + buf) * 1024;
                uint32_t raw[32];
                ptx::tmem_ld_32x32(tmem_base + ((uint32_t)(lane_q * 32) << 16) + (uint32_t)(q * ncol + ci * 64 + half * 32),
                                   raw);
                if (scatter) {
                    const int ogi = g.og > 0 ? chan0 / g.cs_per_og : 0;
                    const int mgi = g.mg > 0 ? chan0 / g.cs_per_mg : 0;
                    if (tap != tg.tap || ogi != tg.og) load_point<DIM>(g, pi, P.offset, tap, ogi, tg);
                    if (tap != tg.mtap || mgi != tg.mg) load_mask<DIM>(g, pi, P.mask, tap, mgi, tg);
                }
                ptx::tmem_ld_wait();
                if (ci == NB - 1) {
                    // the accumulator is in registers: hand it back to the MMA warp right away
                    ptx::tc_fence_before();
                    __syncwarp();
                    if (lane == 0) ptx::mbar_arrive(&t_empty[q]);
                }
                if (want_coord) {
                    ok = dg_wait<SPLIT>(&g_empty[warp * 2 + buf], (uint32_t)(((k / P.g_bufs) & 1) ^ 1));
                    ok = __all_sync(0xffffffffu, ok);
                    if (!ok) {
                        if (lane == 0) atomicExch(P.status, 306);
                        break;
                    }
                }
                __syncwarp();
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    float4 qv;
                    qv.x = __uint_as_float(raw[4 * i]);
                    qv.y = __uint_as_float(raw[4 * i + 1]);
                    qv.z = __uint_as_float(raw[4 * i + 2]);
                    qv.w = __uint_as_float(raw[4 * i + 3]);
                    *reinterpret_cast<float4 *>(gs + lane * 32 + ((i ^ (lane & 7)) << 2)) = qv;
                }
                if (scatter) {
#pragma unroll
                    for (int c = 0; c < NC; ++c) {
                        bool okc;
                        int rowi;
                        float w;
                        corner_of<DIM>(g, pi, tg, deformable, c, okc, rowi, w);
                        ScatterInfo si;
                        si.off = (uint32_t)rowi * (uint32_t)g.Cs;
                        si.scale = tg.mval * w;
                        cs[lane * NC + c] = si;
                    }
                }
                __syncwarp();
                if (want_coord && lane == 0) ptx::mbar_arrive(&g_full[warp * 2 + buf]);
                if (scatter) {
                    // 8 lanes cover the 128 contiguous bytes of one image row: a warp-wide vector reduction
                    // touches 4 rows (thread = position would touch 32)
                    const int quad = lane & 7;
                    float *dst0 = P.img_grad_cl + ch0 + quad * 4;
#pragma unroll 2
                    for (int it = 0; it < 8; ++it) {
                        const int pos = it * 4 + (lane >> 3);
                        const float4 qv = *reinterpret_cast<const float4 *>(gs + pos * 32 + ((quad ^ (pos & 7)) << 2));
#pragma unroll
                        for (int c = 0; c < NC; ++c) {
                            const ScatterInfo si = cs[pos * NC + c];
                            red_add_v4_if(si.scale != 0.f, dst0 + si.off, qv.x * si.scale, qv.y * si.scale, qv.z * si.scale,
                                          qv.w * si.scale);
                        }
                    }
                }
            }
        }
    } else if (warp < 2 * DG_PAIRS) {
        // ------------------------------------------------------------------ coordinate warps
        // Coordinate warp (q, sub) takes 16 of the 32 positions of lane quadrant q, all 64 channels of the chunk:
        // it reads the two 32-channel tiles that scatter warps q and q + 4 staged, gathers the image corners with
        // 8 lanes per row (a warp-wide load touches 4 rows of 128 / 256 contiguous bytes) and turns
        // <col, corner row> dot products into grad_offset / grad_mask sums kept by lanes 0-15 (one position each).
        if (want_coord && !SPLIT) {
            const int cw = warp - DG_PAIRS;
            const int lane_q = cw & 3, sub = cw >> 2;
            const int own = lane & 15;
            const PosInfo<DIM> pi = decode_position<DIM>(g, m0 + lane_q * 32 + sub * 16 + own);
            const bool mine = pi.valid && lane < 16;
            const TI *img = reinterpret_cast<const TI *>(P.img_cl);
            TapGeometry<DIM> tg;
            uint32_t *rs = stage_r + cw * 32 * NC;     // [16][NC] row offsets
            float *ds_ = stage_d + cw * 32 * NC;       // [16][NC] dot products
            float go_sum[DIM], gm_sum = 0.f;
#pragma unroll
            for (int a = 0; a < DIM; ++a) go_sum[a] = 0.f;
            auto flush_off = [&]() {
                if (P.goff != nullptr && tg.tap >= 0 && mine) {
#pragma unroll
                    for (int a = 0; a < DIM; ++a)
                        atomicAdd(P.goff + ((((int64_t)pi.b * g.og + tg.og) * g.K + tg.tap) * DIM + a) * (int64_t)g.P + pi.p,
                                  go_sum[a]);
                }
#pragma unroll
                for (int a = 0; a < DIM; ++a) go_sum[a] = 0.f;
            };
            auto flush_mask = [&]() {
                if (P.gmask != nullptr && tg.mtap >= 0 && mine)
                    atomicAdd(P.gmask + (((int64_t)pi.b * g.mg + tg.mg) * g.K + tg.mtap) * (int64_t)g.P + pi.p, gm_sum);
                gm_sum = 0.f;
            };
            const int q8 = lane & 7, p4 = lane >> 3;
            const int half = q8 >> 2;                 // which scatter warp staged this lane's 8 channels
            const int sw = lane_q + 4 * half;
            const int ci0 = 2 * (q8 & 3);             // first of its two 16-byte chunks in that warp's row
            int k = 0;
            bool ok = true;
            for (int bi = 0; bi < n_blocks && ok; ++bi) {
                const int blk = blk0 + bi;
                const int tap = blk % g.K;
                const int cc0 = (blk / g.K) * NB;
                for (int ci = 0; ci < NB; ++ci, ++k) {
                    const int chan0 = grp * g.csg + (cc0 + ci) * CHUNK_C;
                    const int ogi = g.og > 0 ? chan0 / g.cs_per_og : 0;
                    const int mgi = g.mg > 0 ? chan0 / g.cs_per_mg : 0;
                    if (tap != tg.tap || ogi != tg.og) {
                        flush_off();
                        load_point<DIM>(g, pi, P.offset, tap, ogi, tg);
                    }
                    if (tap != tg.mtap || mgi != tg.mg) {
                        flush_mask();
                        load_mask<DIM>(g, pi, P.mask, tap, mgi, tg);
                    }
                    bool okc[NC];
                    float wc[NC];
                    __syncwarp();
#pragma unroll
                    for (int c = 0; c < NC; ++c) {
                        int rowi;
                        corner_of<DIM>(g, pi, tg, deformable, c, okc[c], rowi, wc[c]);
                        if (lane < 16) rs[own * NC + c] = (uint32_t)rowi * (uint32_t)g.Cs;
                    }
                    __syncwarp();
                    const int buf = k % P.g_bufs;
                    const float *gs = stage_g + (sw * P.g_bufs + buf) * 1024;
                    // 16-bit image: lane q8 owns channels 8 q8 .. 8 q8 + 7 (16 bytes; 8 lanes = one 128-byte row).
                    // f32 image: lane q8 owns channels 4 q8 .. + 3 and 32 + 4 q8 .. + 3, so that each of its two
                    // 16-byte loads lines up with its neighbours' into a full 128-byte line.
                    auto load_corner = [&](CornerLoad<8, TI> &dst, const TI *row) {
                        if constexpr (SPLIT) {
                            dst.v[0] = __ldg(reinterpret_cast<const float4 *>(row + q8 * 4));
                            dst.v[1] = __ldg(reinterpret_cast<const float4 *>(row + 32 + q8 * 4));
                        } else {
                            dst.load(row + q8 * 8);
                        }
                    };
                    // corner loads do not depend on the staged tiles: issue them before waiting
                    constexpr int ITB = SPLIT ? 2 : 4;
                    CornerLoad<8, TI> cl[ITB][NC];
#pragma unroll
                    for (int i = 0; i < ITB; ++i) {
#pragma unroll
                        for (int c = 0; c < NC; ++c)
                            load_corner(cl[i][c], img + rs[(i * 4 + p4) * NC + c] + (uint32_t)chan0);
                    }
                    const uint32_t par = (uint32_t)((k / P.g_bufs) & 1);
                    ok = dg_wait<SPLIT>(&g_full[lane_q * 2 + buf], par) && dg_wait<SPLIT>(&g_full[(lane_q + 4) * 2 + buf], par);
                    ok = __all_sync(0xffffffffu, ok);
                    if (!ok) {
                        if (lane == 0) atomicExch(P.status, 307);
                        break;
                    }
#pragma unroll
                    for (int it0 = 0; it0 < 4; it0 += ITB) {
                        if (it0 > 0) {
#pragma unroll
                            for (int i = 0; i < ITB; ++i) {
#pragma unroll
                                for (int c = 0; c < NC; ++c)
                                    load_corner(cl[i][c], img + rs[((it0 + i) * 4 + p4) * NC + c] + (uint32_t)chan0);
                            }
                        }
#pragma unroll
                        for (int i = 0; i < ITB; ++i) {
                            const int p16 = (it0 + i) * 4 + p4;      // position within this warp's 16
                            const int row = sub * 16 + p16;          // row of the staged 32-position tiles
                            float4 g0, g1;
                            if constexpr (SPLIT) {
                                // chunk q8 of the lower and of the upper 32 channels
                                const float *lo = stage_g + (lane_q * P.g_bufs + buf) * 1024 + row * 32;
                                const float *hi = stage_g + ((lane_q + 4) * P.g_bufs + buf) * 1024 + row * 32;
                                g0 = *reinterpret_cast<const float4 *>(lo + ((q8 ^ (row & 7)) << 2));
                                g1 = *reinterpret_cast<const float4 *>(hi + ((q8 ^ (row & 7)) << 2));
                            } else {
                                // the two halves read their chunk pair in opposite order: 8 distinct banks per phase
                                const float4 ga = *reinterpret_cast<const float4 *>(gs + row * 32 + (((ci0 + half) ^ (row & 7)) << 2));
                                const float4 gb = *reinterpret_cast<const float4 *>(gs + row * 32 + (((ci0 + 1 - half) ^ (row & 7)) << 2));
                                g0 = half ? gb : ga;
                                g1 = half ? ga : gb;
                            }
                            const float gg[8] = {g0.x, g0.y, g0.z, g0.w, g1.x, g1.y, g1.z, g1.w};
#pragma unroll
                            for (int c = 0; c < NC; ++c) {
                                float d = cl[i][c].dot(gg);
                                d += __shfl_xor_sync(0xffffffffu, d, 1);
                                d += __shfl_xor_sync(0xffffffffu, d, 2);
                                d += __shfl_xor_sync(0xffffffffu, d, 4);
                                if (q8 == 0) ds_[p16 * NC + c] = d;
                            }
                        }
                    }
                    __syncwarp();
                    if (lane == 0) {   // both staged tiles are no longer needed by this warp
                        ptx::mbar_arrive(&g_empty[lane_q * 2 + buf]);
                        ptx::mbar_arrive(&g_empty[(lane_q + 4) * 2 + buf]);
                    }
                    float s_val = 0.f;
                    float dotc[NC];
#pragma unroll
                    for (int c = 0; c < NC; ++c) {
                        dotc[c] = ds_[own * NC + c];
                        s_val = fmaf(wc[c], dotc[c], s_val);
                    }
                    gm_sum += s_val;
                    if (P.goff != nullptr) {
#pragma unroll
                        for (int a = 0; a < DIM; ++a) {
                            float ds = 0.f;
#pragma unroll
                            for (int c = 0; c < NC; ++c) {
                                if (okc[c]) {
                                    float w = ((c >> (DIM - 1 - a)) & 1) ? 1.f : -1.f;
#pragma unroll
                                    for (int a2 = 0; a2 < DIM; ++a2)
                                        if (a2 != a) w *= ((c >> (DIM - 1 - a2)) & 1) ? tg.fr[a2] : (1.f - tg.fr[a2]);
                                    ds = fmaf(w, dotc[c], ds);
                                }
                            }
                            go_sum[a] = fmaf(tg.mval, ds, go_sum[a]);
                        }
                    }
                }
            }
            flush_off();
            flush_mask();
        }
        if (want_coord && SPLIT) {
            // f32 image: one coordinate warp per scatter warp, 32 positions x 32 channels, 4 lanes per position
            // (measured faster than the full-row mapping below for 256-byte rows)
            const int pair = warp - DG_PAIRS;
            const int lane_q = pair & 3, half = pair >> 2;
            const PosInfo<DIM> pi = decode_position<DIM>(g, m0 + lane_q * 32 + lane);
            const TI *img = reinterpret_cast<const TI *>(P.img_cl);
            TapGeometry<DIM> tg;
            uint32_t *rs = stage_r + pair * 32 * NC;
            float *ds_ = stage_d + pair * 32 * NC;
            float go_sum[DIM], gm_sum = 0.f;
#pragma unroll
            for (int a = 0; a < DIM; ++a) go_sum[a] = 0.f;
            auto flush_off = [&]() {
                if (P.goff != nullptr && tg.tap >= 0 && pi.valid) {
#pragma unroll
                    for (int a = 0; a < DIM; ++a)
                        atomicAdd(P.goff + ((((int64_t)pi.b * g.og + tg.og) * g.K + tg.tap) * DIM + a) * (int64_t)g.P + pi.p,
                                  go_sum[a]);
                }
#pragma unroll
                for (int a = 0; a < DIM; ++a) go_sum[a] = 0.f;
            };
            auto flush_mask = [&]() {
                if (P.gmask != nullptr && tg.mtap >= 0 && pi.valid)
                    atomicAdd(P.gmask + (((int64_t)pi.b * g.mg + tg.mg) * g.K + tg.mtap) * (int64_t)g.P + pi.p, gm_sum);
                gm_sum = 0.f;
            };
            const int q4 = lane & 3, p8 = lane >> 2;
            int k = 0;
            bool ok = true;
            for (int bi = 0; bi < n_blocks && ok; ++bi) {
                const int blk = blk0 + bi;
                const int tap = blk % g.K;
                const int cc0 = (blk / g.K) * NB;
                for (int ci = 0; ci < NB; ++ci, ++k) {
                    const int chan0 = grp * g.csg + (cc0 + ci) * CHUNK_C;
                    const int ch0 = chan0 + half * 32;
                    const int ogi = g.og > 0 ? chan0 / g.cs_per_og : 0;
                    const int mgi = g.mg > 0 ? chan0 / g.cs_per_mg : 0;
                    if (tap != tg.tap || ogi != tg.og) {
                        flush_off();
                        load_point<DIM>(g, pi, P.offset, tap, ogi, tg);
                    }
                    if (tap != tg.mtap || mgi != tg.mg) {
                        flush_mask();
                        load_mask<DIM>(g, pi, P.mask, tap, mgi, tg);
                    }
                    bool okc[NC];
                    float wc[NC];
                    __syncwarp();
#pragma unroll
                    for (int c = 0; c < NC; ++c) {
                        int rowi;
                        corner_of<DIM>(g, pi, tg, deformable, c, okc[c], rowi, wc[c]);
                        rs[lane * NC + c] = (uint32_t)rowi * (uint32_t)g.Cs;
                    }
                    __syncwarp();
                    const int buf = k % P.g_bufs;
                    const float *gs = stage_g + (pair * P.g_bufs + buf) * 1024;
                    // corner loads do not depend on the staged tile: issue them before waiting for it
                    constexpr int ITB = SPLIT ? 2 : 4;
                    CornerLoad<8, TI> cl[ITB][NC];
#pragma unroll
                    for (int i = 0; i < ITB; ++i) {
#pragma unroll
                        for (int c = 0; c < NC; ++c)
                            cl[i][c].load(img + rs[(i * 8 + p8) * NC + c] + (uint32_t)(ch0 + q4 * 8));
                    }
                    ok = dg_wait<SPLIT>(&g_full[pair * 2 + buf], (uint32_t)((k / P.g_bufs) & 1));
                    ok = __all_sync(0xffffffffu, ok);
                    if (!ok) {
                        if (lane == 0) atomicExch(P.status, 307);
                        break;
                    }
#pragma unroll
                    for (int it0 = 0; it0 < 4; it0 += ITB) {
                        if (it0 > 0) {
#pragma unroll
                            for (int i = 0; i < ITB; ++i) {
#pragma unroll
                                for (int c = 0; c < NC; ++c)
                                    cl[i][c].load(img + rs[((it0 + i) * 8 + p8) * NC + c] + (uint32_t)(ch0 + q4 * 8));
                            }
                        }
#pragma unroll
                        for (int i = 0; i < ITB; ++i) {
                            const int pos = (it0 + i) * 8 + p8;
                            const float4 g0 = *reinterpret_cast<const float4 *>(gs + pos * 32 + (((2 * q4) ^ (pos & 7)) << 2));
                            const float4 g1 = *reinterpret_cast<const float4 *>(gs + pos * 32 + (((2 * q4 + 1) ^ (pos & 7)) << 2));
                            const float gg[8] = {g0.x, g0.y, g0.z, g0.w, g1.x, g1.y, g1.z, g1.w};
#pragma unroll
                            for (int c = 0; c < NC; ++c) {
                                float d = cl[i][c].dot(gg);
                                d += __shfl_xor_sync(0xffffffffu, d, 1);
                                d += __shfl_xor_sync(0xffffffffu, d, 2);
                                if (q4 == 0) ds_[pos * NC + c] = d;
                            }
                        }
                    }
                    __syncwarp();
                    if (lane == 0) ptx::mbar_arrive(&g_empty[pair * 2 + buf]);  // staged tile no longer needed
                    float s_val = 0.f;
                    float dotc[NC];
#pragma unroll
                    for (int c = 0; c < NC; ++c) {
                        dotc[c] = ds_[lane * NC + c];
                        s_val = fmaf(wc[c], dotc[c], s_val);
                    }
                    gm_sum += s_val;
                    if (P.goff != nullptr) {
#pragma unroll
                        for (int a = 0; a < DIM; ++a) {
                            float ds = 0.f;
#pragma unroll
                            for (int c = 0; c < NC; ++c) {
                                if (okc[c]) {
                                    float w = ((c >> (DIM - 1 - a)) & 1) ? 1.f : -1.f;
#pragma unroll
                                    for (int a2 = 0; a2 < DIM; ++a2)
                                        if (a2 != a) w *= ((c >> (DIM - 1 - a2)) & 1) ? tg.fr[a2] : (1.f - tg.fr[a2]);
                                    ds = fmaf(w, dotc[c], ds);
                                }
                            }
                            go_sum[a] = fmaf(tg.mval, ds, go_sum[a]);
                        }
                    }
                }
            }
            flush_off();
            flush_mask();
        }
    } else if (warp == DG_MMA_WARP) {
        // ------------------------------------------------------------------ MMA issue
        if (lane == 0) {
            const uint32_t idesc = ptx::instr_desc_f16(MODE == TC_F16 ? 0 : 1, TILE_POS, ncol, 0, 0);
            bool ok = dg_wait<SPLIT>(a_full, 0);
            if (!ok) atomicExch(P.status, 302);
            const uint32_t a_addr = ptx::smem_u32(sA);
            int j = 0;  // running B stage counter
            for (int bi = 0; bi < n_blocks && ok; ++bi) {
                const int blk = blk0 + bi;
                const int q = bi % NQ;
                if (!dg_wait<SPLIT>(&t_empty[q], (uint32_t)(((bi / NQ) & 1) ^ 1))) {
                    atomicExch(P.status, 303);
                    ok = false;
                    break;
                }
                ptx::tc_fence_after();
                const uint32_t d_tmem = tmem_base + (uint32_t)(q * ncol);
                for (int rc = 0; rc < RC && ok; ++rc, ++j) {
                    const int s = j % BS;
                    if (!dg_wait<SPLIT>(&b_full[s], (uint32_t)((j / BS) & 1))) {
                        atomicExch(P.status, 304);
                        ok = false;
                        break;
                    }
                    ptx::tc_fence_after();
                    const uint32_t a_rc = a_addr + (uint32_t)(rc * PARTS * DG_A_TILE);
                    const uint32_t b_addr = ptx::smem_u32(sB + (size_t)s * b_stage_bytes);
#pragma unroll
                    for (int k4 = 0; k4 < 4; ++k4) {
                        const uint64_t a_hi = ptx::smem_desc_sw128(a_rc + k4 * 32, 16, 1024);
                        const uint64_t b_hi = ptx::smem_desc_sw128(b_addr + k4 * 32, 16, 1024);
                        ptx::mma_f16(d_tmem, a_hi, b_hi, idesc, (rc > 0 || k4 > 0) ? 1u : 0u);
                        if constexpr (SPLIT) {
                            const uint64_t a_lo = ptx::smem_desc_sw128(a_rc + DG_A_TILE + k4 * 32, 16, 1024);
                            const uint64_t b_lo = ptx::smem_desc_sw128(b_addr + b_part_bytes + k4 * 32, 16, 1024);
                            ptx::mma_f16(d_tmem, a_lo, b_hi, idesc, 1u);
                            ptx::mma_f16(d_tmem, a_hi, b_lo, idesc, 1u);
                        }
                    }
                    ptx::mma_commit(&b_empty[s]);
                }
                if (ok) ptx::mma_commit(&t_full[q]);
            }
        }
        __syncwarp();
    } else if (warp == DG_TMA_WARP) {
        // ------------------------------------------------------------------ TMA: dense tiles once, weight ring
        if (lane == 0) {
            ptx::mbar_arrive_expect_tx(a_full, a_bytes);
            for (int rc = 0; rc < RC; ++rc) {
                ptx::tma_load_2d(sA + (size_t)(rc * PARTS) * DG_A_TILE, &tmap_a_hi, a_full, grp * g.cdg + rc * 64, (int)m0);
                if (SPLIT)
                    ptx::tma_load_2d(sA + (size_t)(rc * PARTS + 1) * DG_A_TILE, &tmap_a_lo, a_full, grp * g.cdg + rc * 64,
                                     (int)m0);
            }
            int j = 0, issued = 0;
            bool ok = true;
            for (int bi = 0; bi < n_blocks && ok; ++bi) {
                const int blk = blk0 + bi;
                const int tap = blk % g.K;
                const int cc0 = (blk / g.K) * NB;
                for (int rc = 0; rc < RC; ++rc, ++j) {
                    const int s = j % BS;
                    if (!dg_wait<SPLIT>(&b_empty[s], (uint32_t)(((j / BS) & 1) ^ 1))) {
                        atomicExch(P.status, 305);
                        ok = false;
                        break;
                    }
                    uint8_t *dst = sB + (size_t)s * b_stage_bytes;
                    ptx::mbar_arrive_expect_tx(&b_full[s], b_stage_bytes);
                    ptx::tma_load_4d(dst, &tmap_b_hi, &b_full[s], rc * 64, cc0 * CHUNK_C, tap, grp);
                    if (SPLIT) ptx::tma_load_4d(dst + b_part_bytes, &tmap_b_lo, &b_full[s], rc * 64, cc0 * CHUNK_C, tap, grp);
                    issued = j + 1;
                }
            }
            dg_wait<SPLIT>(a_full, 0);
            if (issued > 0) {
                const int jj = issued - 1;
                dg_wait<SPLIT>(&b_full[jj % BS], (uint32_t)((jj / BS) & 1));
            }
        }
        __syncwarp();
    }

    ptx::tc_fence_before();
    __syncthreads();
    if (warp == DG_MMA_WARP) ptx::tmem_dealloc(tmem_base, DG_TMEM_COLS);
}

// [B, C, S] f32 -> [B, S, C] bf16 hi + lo
__global__ void __launch_bounds__(256) to_channels_last_split_kernel(const float *__restrict__ src,
                                                                     __nv_bfloat16 *__restrict__ hi,
                                                                     __nv_bfloat16 *__restrict__ lo, int C, int S,
                                                                     __nv_bfloat16 *__restrict__ hi_same,
                                                                     __nv_bfloat16 *__restrict__ lo_same) {
    __shared__ float tile[32][33];
    const int b = blockIdx.z;
    const int s0 = blockIdx.x * 32, c0 = blockIdx.y * 32;
    const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
    const float *in = src + (int64_t)b * C * S;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int c = c0 + ty + 8 * i, s = s0 + tx;
        if (c < C && s < S) {
            const float v = in[(int64_t)c * S + s];
            tile[ty + 8 * i][tx] = v;
            if (hi_same != nullptr) {
                const __nv_bfloat16 h = __float2bfloat16_rn(v);
                const int64_t o = (int64_t)b * C * S + (int64_t)c * S + s;
                hi_same[o] = h;
                lo_same[o] = __float2bfloat16_rn(v - __bfloat162float(h));
            }
        }
    }
    __syncthreads();
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int s = s0 + ty + 8 * i, c = c0 + tx;
        if (c < C && s < S) {
            const float v = tile[tx][ty + 8 * i];
            const __nv_bfloat16 h = __float2bfloat16_rn(v);
            const int64_t o = (int64_t)b * C * S + (int64_t)s * C + c;
            hi[o] = h;
            lo[o] = __float2bfloat16_rn(v - __bfloat162float(h));
        }
    }
}

// [B, C, S] f32 -> [B, S, C] bf16 hi + lo with 16-byte loads and 4-byte (channel pair) stores, for S a multiple of 4
// and C of 2; 64 x 64 tiles.  Even channels sit in rows 0-31 of the shared tile, odd ones in rows 32-63, so that the
// transposing reads of a channel pair per lane are free of bank conflicts.
__global__ void __launch_bounds__(256) to_channels_last_split64_kernel(const float *__restrict__ src,
                                                                       uint32_t *__restrict__ hi,
                                                                       uint32_t *__restrict__ lo, int C, int S,
                                                                       uint2 *__restrict__ hi_same,
                                                                       uint2 *__restrict__ lo_same) {
    __shared__ float tile[64 * 65];
    const int b = blockIdx.z;
    const int s0 = blockIdx.x * 64, c0 = blockIdx.y * 64;
    const float *in = src + (int64_t)b * C * S;
    const int v = threadIdx.x & 15, r = threadIdx.x >> 4;
#pragma unroll
    for (int pass = 0; pass < 4; ++pass) {
        const int cl = pass * 16 + r;
        const int c = c0 + cl, s = s0 + v * 4;
        float4 x = make_float4(0.f, 0.f, 0.f, 0.f);
        if (c < C && s < S) {
            x = __ldg(reinterpret_cast<const float4 *>(in + (int64_t)c * S + s));
            if (hi_same != nullptr) {   // the same split in the source layout, while the values are in registers
                const float f[4] = {x.x, x.y, x.z, x.w};
                uint32_t h[4], l[4];
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                    const __nv_bfloat16 hb = __float2bfloat16_rn(f[k]);
                    h[k] = __bfloat16_as_ushort(hb);
                    l[k] = __bfloat16_as_ushort(__float2bfloat16_rn(f[k] - __bfloat162float(hb)));
                }
                const int64_t o = ((int64_t)b * C * S + (int64_t)c * S + s) >> 2;
                hi_same[o] = make_uint2(h[0] | (h[1] << 16), h[2] | (h[3] << 16));
                lo_same[o] = make_uint2(l[0] | (l[1] << 16), l[2] | (l[3] << 16));
            }
        }
        float *w = tile + ((cl >> 1) + 32 * (cl & 1)) * 65 + v * 4;
        w[0] = x.x;
        w[1] = x.y;
        w[2] = x.z;
        w[3] = x.w;
    }
    __syncthreads();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int c = c0 + 2 * lane;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const int sl = warp * 8 + i;
        const int s = s0 + sl;
        if (c < C && s < S) {
            const float a = tile[lane * 65 + sl], bb = tile[(32 + lane) * 65 + sl];
            const __nv_bfloat16 ha = __float2bfloat16_rn(a), hb = __float2bfloat16_rn(bb);
            const __nv_bfloat16 la = __float2bfloat16_rn(a - __bfloat162float(ha));
            const __nv_bfloat16 lb = __float2bfloat16_rn(bb - __bfloat162float(hb));
            const int64_t o = ((int64_t)b * C * S + (int64_t)s * C + c) >> 1;
            hi[o] = (uint32_t)__bfloat16_as_ushort(ha) | ((uint32_t)__bfloat16_as_ushort(hb) << 16);
            lo[o] = (uint32_t)__bfloat16_as_ushort(la) | ((uint32_t)__bfloat16_as_ushort(lb) << 16);
        }
    }
}

// [B, S, C] f32 (+ bias[c]) -> [B, C, S] with 16-byte loads and 4-element stores, for S and C multiples of 4
template <typename TO>
__global__ void __launch_bounds__(256) from_channels_last_bias64_kernel(const float *__restrict__ src,
                                                                        const float *__restrict__ bias,
                                                                        TO *__restrict__ dst, int C, int S) {
    __shared__ float tile[64 * 65];
    const int b = blockIdx.z;
    const int s0 = blockIdx.x * 64, c0 = blockIdx.y * 64;
    const float *in = src + (int64_t)b * C * S;
    TO *out = dst + (int64_t)b * C * S;
    const int v = threadIdx.x & 15, r = threadIdx.x >> 4;
#pragma unroll
    for (int pass = 0; pass < 4; ++pass) {
        const int sl = pass * 16 + r;
        const int s = s0 + sl, c = c0 + v * 4;
        float4 x = make_float4(0.f, 0.f, 0.f, 0.f);
        if (c < C && s < S) x = __ldg(reinterpret_cast<const float4 *>(in + (int64_t)s * C + c));
        float *w = tile + sl * 65 + v * 4;
        w[0] = x.x;
        w[1] = x.y;
        w[2] = x.z;
        w[3] = x.w;
    }
    __syncthreads();
#pragma unroll
    for (int pass = 0; pass < 4; ++pass) {
        const int cl = pass * 16 + r;
        const int c = c0 + cl, s = s0 + v * 4;
        if (c < C && s < S) {
            const float bv = bias != nullptr ? __ldg(bias + c) : 0.f;
            float x[4];
#pragma unroll
            for (int k = 0; k < 4; ++k) x[k] = tile[(v * 4 + k) * 65 + cl] + bv;
            TO *o = out + (int64_t)c * S + s;
            if constexpr (sizeof(TO) == 4) {
                *reinterpret_cast<float4 *>(o) = make_float4(x[0], x[1], x[2], x[3]);
            } else {
                TO y[4];
#pragma unroll
                for (int k = 0; k < 4; ++k) store_acc(y, k, x[k]);
                *reinterpret_cast<uint2 *>(o) = *reinterpret_cast<const uint2 *>(y);
            }
        }
    }
}

// [B, S, C] f32 (+ bias[c]) -> [B, C, S] in the destination type
template <typename TO>
__global__ void __launch_bounds__(256) from_channels_last_bias_kernel(const float *__restrict__ src,
                                                                      const float *__restrict__ bias,
                                                                      TO *__restrict__ dst, int C, int S) {
    __shared__ float tile[32][33];
    const int b = blockIdx.z;
    const int s0 = blockIdx.x * 32, c0 = blockIdx.y * 32;
    const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
    const float *in = src + (int64_t)b * C * S;
    TO *out = dst + (int64_t)b * C * S;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int s = s0 + ty + 8 * i, c = c0 + tx;
        if (c < C && s < S) tile[ty + 8 * i][tx] = in[(int64_t)s * C + c];
    }
    __syncthreads();
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int c = c0 + ty + 8 * i, s = s0 + tx;
        if (c < C && s < S) {
            float v = tile[tx][ty + 8 * i];
            if (bias != nullptr) v += __ldg(bias + c);
            store_acc(out, (int64_t)c * S + s, v);
        }
    }
}

size_t dgrad_smem_bytes(int dim, int mode, int rc, int nb, int b_stages, int g_bufs) {
    const int parts = mode == TC_SPLIT ? 2 : 1;
    const int nc = 1 << dim;
    const size_t staging = (size_t)DG_PAIRS * (g_bufs * 4096 + 32 * nc * (8 + 4 + 4));  // epilogue buffers
    return 1024 + (size_t)rc * parts * DG_A_TILE + (size_t)b_stages * parts * nb * 64 * 128 + staging +
           (49 + 2 * b_stages) * 8 + 16;
}

template <int DIM, int MODE>
cudaError_t launch_dgrad_t(const DgradParams<DIM> &P, dim3 grid, const CUtensorMap *maps, cudaStream_t stream) {
    const size_t smem = dgrad_smem_bytes(DIM, MODE, P.rc, P.nb, P.b_stages, P.g_bufs);
    auto kern = dcn_dgrad_tc_kernel<DIM, MODE>;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return e;
    LaunchScope scope("dcn_dgrad_tc", stream);
    kern<<<grid, DG_THREADS, smem, stream>>>(P, maps[0], maps[1], maps[2], maps[3]);
    return cudaGetLastError();
}

}  // namespace

// Column-block width, weight-ring depth and staging depth that fit shared memory; false when nothing fits.
bool dgrad_tc_config(int dim, int mode, int cdg, int csg, int *nb, int *b_stages, int *g_bufs) {
    const int rc = cdg / 64;
    const int n_max = std::min(((csg / 64) % 2 == 0) ? 2 : 1, std::max(1, tuning_int("TVDCN_B200_DG_NB", 2)));
    for (int gb = std::min(2, std::max(1, tuning_int("TVDCN_B200_DG_GBUFS", 2))); gb >= 1; --gb)
        for (int n = n_max; n >= 1; --n)
            for (int cand = tuning_int("TVDCN_B200_DG_STAGES", 3); cand >= 2; --cand)
                if (dgrad_smem_bytes(dim, mode, rc, n, cand, gb) <= 227 * 1024) {
                    *nb = n;
                    *b_stages = cand;
                    *g_bufs = gb;
                    return true;
                }
    return false;
}

// hi_same / lo_same (both or neither): the same hi + lo split in the layout of the source, written in the same pass
cudaError_t launch_to_channels_last_split(const float *src, void *hi, void *lo, int B, int C, int S,
                                          cudaStream_t stream, void *hi_same, void *lo_same) {
    dim3 grid((S + 31) / 32, (C + 31) / 32, B);
    LaunchScope scope("to_channels_last", stream);
    const bool same_ok = hi_same == nullptr ||
                         ((reinterpret_cast<uintptr_t>(hi_same) | reinterpret_cast<uintptr_t>(lo_same)) & 7) == 0;
    if (S % 4 == 0 && C % 2 == 0 && same_ok && (reinterpret_cast<uintptr_t>(src) & 15) == 0 &&
        ((reinterpret_cast<uintptr_t>(hi) | reinterpret_cast<uintptr_t>(lo)) & 3) == 0) {
        dim3 grid64((S + 63) / 64, (C + 63) / 64, B);
        to_channels_last_split64_kernel<<<grid64, 256, 0, stream>>>(src, (uint32_t *)hi, (uint32_t *)lo, C, S,
                                                                   (uint2 *)hi_same, (uint2 *)lo_same);
    } else {
        to_channels_last_split_kernel<<<grid, 256, 0, stream>>>(src, (__nv_bfloat16 *)hi, (__nv_bfloat16 *)lo, C, S,
                                                                (__nv_bfloat16 *)hi_same, (__nv_bfloat16 *)lo_same);
    }
    return cudaGetLastError();
}

cudaError_t launch_from_channels_last_bias(const float *src, const float *bias, void *dst, int dst_dtype, int B, int C,
                                           int S, cudaStream_t stream) {
    dim3 grid((S + 31) / 32, (C + 31) / 32, B);
    LaunchScope scope("from_channels_last", stream);
    const bool wide = S % 4 == 0 && C % 4 == 0 && (reinterpret_cast<uintptr_t>(src) & 15) == 0 &&
                      (reinterpret_cast<uintptr_t>(dst) & 15) == 0;
    dim3 grid64((S + 63) / 64, (C + 63) / 64, B);
    if (dst_dtype == DT_F32 && wide)
        from_channels_last_bias64_kernel<float><<<grid64, 256, 0, stream>>>(src, bias, (float *)dst, C, S);
    else if (dst_dtype == DT_BF16 && wide)
        from_channels_last_bias64_kernel<__nv_bfloat16><<<grid64, 256, 0, stream>>>(src, bias, (__nv_bfloat16 *)dst, C, S);
    else if (dst_dtype == DT_F16 && wide)
        from_channels_last_bias64_kernel<__half><<<grid64, 256, 0, stream>>>(src, bias, (__half *)dst, C, S);
    else if (dst_dtype == DT_F32)
        from_channels_last_bias_kernel<float><<<grid, 256, 0, stream>>>(src, bias, (float *)dst, C, S);
    else if (dst_dtype == DT_BF16)
        from_channels_last_bias_kernel<__nv_bfloat16><<<grid, 256, 0, stream>>>(src, bias, (__nv_bfloat16 *)dst, C, S);
    else if (dst_dtype == DT_F16)
        from_channels_last_bias_kernel<__half><<<grid, 256, 0, stream>>>(src, bias, (__half *)dst, C, S);
    else
        return cudaErrorInvalidValue;
    return cudaGetLastError();
}

// dense_cl_*: dense tensor channels-last [B*P, Cd] 16-bit (hi / lo); w_kd_*: weights packed [g][tap][s'][d'];
// img_cl: sampled image channels-last (needed for goff / gmask); accumulation targets are f32 and
// initialised by the caller.
cudaError_t launch_gemm_scatter_tc(const GeoHost &h, int mode, const void *dense_cl_hi, const void *dense_cl_lo,
                                   const void *w_kd_hi, const void *w_kd_lo, const void *img_cl, const float *offset,
                                   const float *mask, float *img_grad_cl, float *goff, float *gmask, int *status,
                                   cudaStream_t stream) {
    const int cdg = h.Cd / h.groups, csg = h.Cs / h.groups;
    int nb = 0, bs = 0, gb = 0;
    if (!dgrad_tc_config(h.dim, mode, cdg, csg, &nb, &bs, &gb)) return cudaErrorInvalidConfiguration;
    const long long BP = (long long)h.B * h.P;
    CUtensorMap maps[4];
    {
        const uint64_t dims[2] = {(uint64_t)h.Cd, (uint64_t)BP};
        const uint64_t strides[1] = {(uint64_t)h.Cd * 2};
        const uint32_t box[2] = {64, TILE_POS};
        if (!make_tensor_map_16bit(&maps[0], dense_cl_hi, 2, dims, strides, box)) return cudaErrorInvalidValue;
        if (mode == TC_SPLIT) {
            if (!make_tensor_map_16bit(&maps[1], dense_cl_lo, 2, dims, strides, box)) return cudaErrorInvalidValue;
        } else {
            maps[1] = maps[0];
        }
    }
    {
        const uint64_t dims[4] = {(uint64_t)cdg, (uint64_t)csg, (uint64_t)h.K, (uint64_t)h.groups};
        const uint64_t strides[3] = {(uint64_t)cdg * 2, (uint64_t)cdg * csg * 2, (uint64_t)cdg * csg * h.K * 2};
        const uint32_t box[4] = {64, (uint32_t)(nb * 64), 1, 1};
        if (!make_tensor_map_16bit(&maps[2], w_kd_hi, 4, dims, strides, box)) return cudaErrorInvalidValue;
        if (mode == TC_SPLIT) {
            if (!make_tensor_map_16bit(&maps[3], w_kd_lo, 4, dims, strides, box)) return cudaErrorInvalidValue;
        } else {
            maps[3] = maps[2];
        }
    }
    // Share each position tile between `splits` CTAs (equal ranges of its column blocks) when that evens out the
    // last wave: cost of a launch ~ ceil(CTAs / SMs) / splits tile-times; a split is taken only for a gain above
    // 4 % (each extra CTA reloads the dense tile).
    const long long tiles = ((BP + TILE_POS - 1) / TILE_POS) * h.groups;
    const int n_total = h.K * ((csg / 64) / nb);
    int splits = 1;
    {
        const int forced = tuning_int("TVDCN_B200_DG_SPLITS", 0);
        double best = (double)((tiles + 147) / 148);
        for (int cand = 2; cand <= 3; ++cand) {
            if (n_total % cand != 0) continue;
            const double cost = (double)((tiles * cand + 147) / 148) / cand;
            if (cost < best * 0.96) { best = cost; splits = cand; }
        }
        if (forced > 0 && n_total % forced == 0) splits = forced;
    }
    dim3 grid((unsigned)((BP + TILE_POS - 1) / TILE_POS), (unsigned)h.groups, (unsigned)splits);
    auto run = [&](auto dimc) -> cudaError_t {
        constexpr int DIM = decltype(dimc)::value;
        DgradParams<DIM> P;
        P.g = geo_from_host<DIM>(h);
        P.img_cl = img_cl;
        P.offset = offset;
        P.mask = mask;
        P.img_grad_cl = img_grad_cl;
        P.goff = goff;
        P.gmask = gmask;
        P.status = status;
        P.nb = nb;
        P.rc = cdg / 64;
        P.b_stages = bs;
        P.chunks_per_tap = csg / CHUNK_C;
        P.g_bufs = gb;
        if (mode == TC_BF16) return launch_dgrad_t<DIM, TC_BF16>(P, grid, maps, stream);
        if (mode == TC_F16) return launch_dgrad_t<DIM, TC_F16>(P, grid, maps, stream);
        return launch_dgrad_t<DIM, TC_SPLIT>(P, grid, maps, stream);
    };
    if (h.dim == 1) return run(std::integral_constant<int, 1>());
    if (h.dim == 2) return run(std::integral_constant<int, 2>());
    if (h.dim == 3) return run(std::integral_constant<int, 3>());
    return cudaErrorInvalidValue;
}

}  // namespace tvdcn_b200
