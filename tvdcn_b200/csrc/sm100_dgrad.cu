// Tensor-core "GEMM -> scatter" kernel (tcgen05 / TMEM) with pixel-owned aggregation.
//
//   col[k | b, p] = sum_{d in group} W[d, k] * dense[b, d, p],   k = (tap, sampled channel)
// consumed straight out of tensor memory, never stored in global memory:
//   img_grad[b, s, corner]   += col * mask * corner weight                      (scatter)
//   grad_offset[b, og, tap, axis, p] += col * mask * d sample / d axis          (needs the sampled image)
//   grad_mask[b, mg, tap, p]         += col * sample                            (needs the sampled image)
//
// Replaces addmm_ + compute_grad_offset + compute_grad_mask + col2im of the reference's backward loop
// (tvdcn/csrc/ops/cuda/deform_conv2d_kernel.cpp:519-598) and addmm_ + col2im of the transposed forward
// (tvdcn/csrc/ops/cuda/deform_conv_transpose2d_kernel.cpp:333-362): the column buffer is never written.
//
// One CTA owns a tile of 128 grid positions and walks *units* = (64-channel chunk, batch of TB taps); every
// unit is two *passes* over 32-channel slabs.
//   GEMM   D[128 positions (TMEM lanes) x TB*32 columns] over the dense channels of the group.
//          A = the dense tile [128 pos][cdg], read once per CTA from the caller's [B, Cd, P] tensor (thread =
//              position, coalesced), converted to 16-bit (f32 data: bf16 hi + lo) and kept in TENSOR MEMORY for
//              the whole CTA (tcgen05.st; the MMA reads A from TMEM, so shared memory carries only B);
//          B = weights packed [g][tap][s'][d'], one TMA box {64 d', 32 s', TB taps} per reduction chunk (ring);
//          D = ring of accumulators in the TMEM columns behind A.
//   plan   Four planner warps (thread = position) turn the unit's offsets / mask into one entry per in-image
//          bilinear corner (pixel row, position, tap, weight x mask) and GROUP THE ENTRIES BY PIXEL with a
//          shared-memory hash table (integer atomics) + prefix sum.
//   store  Four warps copy each finished accumulator TMEM -> shared memory ([128 pos][TB*32] f32).
//   gather Twelve warps, 8 lanes per entry (4 channels each), walk equal spans of the pixel-grouped entry
//          list: one 16-byte shared load of the entry's column values feeds both the running sum of the
//          pixel (one red.global.add.v4.f32 per lane leaves the SM when the pixel changes, instead of one per
//          corner) and the dot product <col, image row of the pixel> that the coordinate gradients need.
//          The dots of a unit's entries are finally combined per (position, tap) by the planner threads.
//
// Warp roles (704 threads): 0-3 store, 4-15 gather, 16-19 planners, 20 MMA issue + TMEM owner, 21 TMA.
#include <algorithm>
#include <type_traits>

#include "plan.h"
#include "sm100_common.cuh"

namespace tvdcn_b200 {

template <int DIM>
struct DgradParams {
    Geo<DIM> g;
    const void *dense;      // [B, Cd, P] in the problem's data type, the caller's layout
    const void *img_cl;     // sampled image, channels-last (16-bit or f32); null when no coordinate gradient is wanted
    const float *offset;    // may be null
    const float *mask;      // may be null
    float *img_grad_cl;     // [B*S, Cs] f32, accumulated into; may be null
    float *goff;            // f32, accumulated into; may be null
    float *gmask;           // f32, accumulated into; may be null
    int *status;
    int rc;                 // reduction chunks: cdg / 64
    int tb;                 // taps per batch
    int nbatch;             // ceil(K / tb)
    int nacc;               // accumulators in the TMEM ring
    int b_stages;
    int units_per_cta;      // (csg / 64) * nbatch / gridDim.z
};

namespace {

constexpr int SC_STORE_WARPS = 4;
constexpr int SC_GATHER_WARPS = 12;
constexpr int SC_WORK_WARPS = SC_STORE_WARPS + SC_GATHER_WARPS;   // all of them load the dense tile first
constexpr int SC_PLAN_WARP0 = SC_WORK_WARPS;
constexpr int SC_PLAN_WARPS = 4;                                  // one planner thread per tile position
constexpr int SC_MMA_WARP = SC_PLAN_WARP0 + SC_PLAN_WARPS;
constexpr int SC_TMA_WARP = SC_MMA_WARP + 1;
constexpr int SC_THREADS = (SC_TMA_WARP + 1) * 32;
constexpr int SC_GROUPS = SC_GATHER_WARPS * 4;                    // 8-lane groups walking the entry list
constexpr int SC_SLAB = 32;                                       // channels per pass
constexpr int SC_HASH = 2048;                                     // slots; >= entries of one unit
constexpr uint32_t SC_NONE = 0xffffffffu;
constexpr int SC_PF = 4;                                          // entries fetched ahead by a gather group
constexpr int SC_TMEM_COLS = 512;

// most taps per batch: 128 * tb * 2^dim entries must fit the hash table
__host__ __device__ constexpr int sc_tb_max(int dim) { return dim == 1 ? 4 : (dim == 2 ? 3 : 2); }

__device__ __forceinline__ void red_add_v4(float *addr, float a, float b, float c, float d) {
    asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(addr), "f"(a), "f"(b), "f"(c), "f"(d)
                 : "memory");
}

__device__ __forceinline__ void planner_barrier() { asm volatile("bar.sync 1, 128;" ::: "memory"); }

// Sampling geometry of one (position, tap): floor and fraction per axis, mask value.
template <int DIM>
struct TapGeometry {
    int fl[DIM];
    float fr[DIM];
    float mval;
};

template <int DIM>
__device__ __forceinline__ TapGeometry<DIM> load_geometry(const Geo<DIM> &g, const PosInfo<DIM> &pi,
                                                          const float *__restrict__ offset,
                                                          const float *__restrict__ mask, int tap, int ogi, int mgi) {
    TapGeometry<DIM> tg;
    int tc[DIM];
    tap_coords<DIM>(g, tap, tc);
#pragma unroll
    for (int a = 0; a < DIM; ++a) {
        const int base = pi.base[a] + tc[a] * g.dil[a];
        if (offset != nullptr) {
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
    tg.mval = mask != nullptr ? __ldg(mask + (((int64_t)pi.b * g.mg + mgi) * g.K + tap) * (int64_t)g.P + pi.p) : 1.f;
    return tg;
}

// corner c of the 2^DIM cell: in the image?, pixel row of the channels-last image, interpolation weight
template <int DIM>
__device__ __forceinline__ void corner_of(const Geo<DIM> &g, const PosInfo<DIM> &pi, const TapGeometry<DIM> &tg,
                                          bool deformable, int c, bool &ok, uint32_t &row, float &w) {
    ok = deformable || c == 0;
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
    row = (uint32_t)(pi.b * g.S + flat);
}

// Byte offsets of the dynamic shared memory regions (after alignment to 1024).
struct ScLayout {
    uint32_t b_stage, col_buf, plan_buf, col, plan, keys, cnt, misc, bars, total;
    int n, col_stride, max_entries;
};
__host__ __device__ inline ScLayout sc_layout(int dim, int mode, int tb, int b_stages) {
    ScLayout L;
    const int parts = mode == TC_SPLIT ? 2 : 1;
    L.n = tb * SC_SLAB;
    L.col_stride = L.n + 4;                       // words; = 4 mod 32, so that the row-per-lane stores spread over the banks
    L.max_entries = TILE_POS * tb * (1 << dim);
    L.b_stage = (uint32_t)(L.n * 128 * parts);
    L.col_buf = (uint32_t)(TILE_POS * L.col_stride * 4);
    L.plan_buf = (uint32_t)(L.max_entries * 16);  // pixel row, meta, weight, dot product: 4 bytes each per entry
    uint32_t o = 0;
    o += (uint32_t)b_stages * L.b_stage;
    L.col = o;  o += 2 * L.col_buf;
    L.plan = o; o += 2 * L.plan_buf;
    L.keys = o; o += SC_HASH * 4;
    L.cnt = o;  o += SC_HASH * 4;
    L.misc = o; o += 64;                          // scan partial sums [4], wait flag, entry counts [2], TMEM slot
    L.bars = o; o += (uint32_t)(17 + 2 * b_stages) * 8;
    L.total = o;
    return L;
}

template <int DIM, int MODE>
__global__ void __launch_bounds__(SC_THREADS, 1)
dcn_dgrad_tc_kernel(const DgradParams<DIM> P, const __grid_constant__ CUtensorMap tmap_b_hi,
                    const __grid_constant__ CUtensorMap tmap_b_lo) {
    constexpr int NC = 1 << DIM;
    constexpr bool SPLIT = MODE == TC_SPLIT;
    constexpr int PARTS = SPLIT ? 2 : 1;
    constexpr int TBM = sc_tb_max(DIM);
    using T16 = typename std::conditional<MODE == TC_F16, __half, __nv_bfloat16>::type;
    const Geo<DIM> &g = P.g;

    extern __shared__ uint8_t smem_raw[];
    // align by offset, not by integer round-trip, so that the compiler keeps these as shared-memory pointers
    uint8_t *smem = smem_raw + ((1024u - (ptx::smem_u32(smem_raw) & 1023u)) & 1023u);
    const int RC = P.rc, TB = P.tb, BS = P.b_stages, NACC = P.nacc;
    const ScLayout L = sc_layout(DIM, MODE, TB, BS);
    const int N = L.n;
    const int a_cols = g.cdg / 2;                       // TMEM columns of one 16-bit copy of the dense tile
    const uint32_t acc_col0 = (uint32_t)(a_cols * PARTS);
    uint8_t *sB = smem;
    float *col = reinterpret_cast<float *>(smem + L.col);
    uint32_t *keys = reinterpret_cast<uint32_t *>(smem + L.keys);
    uint32_t *cnt = reinterpret_cast<uint32_t *>(smem + L.cnt);
    uint32_t *misc = reinterpret_cast<uint32_t *>(smem + L.misc);
    uint32_t *scan_part = misc;          // [4]
    uint32_t *wait_flag = misc + 4;
    uint32_t *n_entries = misc + 6;      // [2]
    uint32_t *tmem_slot = misc + 8;
    uint64_t *bars = reinterpret_cast<uint64_t *>(smem + L.bars);
    uint64_t *a_full = bars;
    uint64_t *b_full = bars + 1;
    uint64_t *b_empty = b_full + BS;
    uint64_t *t_full = b_empty + BS;     // [4] MMA -> store warps: accumulator complete
    uint64_t *t_empty = t_full + 4;      // [4] store warps -> MMA: accumulator read out
    uint64_t *col_full = t_empty + 4;    // [2] store warps -> gather warps
    uint64_t *col_empty = col_full + 2;  // [2] gather warps -> store warps
    uint64_t *plan_full = col_empty + 2; // [2] planners -> gather warps
    uint64_t *plan_done = plan_full + 2; // [2] gather warps -> planners
    auto plan_pix = [&](int pb) { return reinterpret_cast<uint32_t *>(smem + L.plan + (size_t)pb * L.plan_buf); };
    auto plan_meta = [&](int pb) { return plan_pix(pb) + L.max_entries; };
    auto plan_w = [&](int pb) { return reinterpret_cast<float *>(plan_pix(pb) + 2 * L.max_entries); };
    auto plan_dot = [&](int pb) { return reinterpret_cast<float *>(plan_pix(pb) + 3 * L.max_entries); };

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int grp = blockIdx.y;
    const long long m0 = (long long)blockIdx.x * TILE_POS;
    // units of this CTA: gridDim.z CTAs share one position tile and take equal ranges of its units, which evens
    // out the last wave when the tiles do not fill the SMs a whole number of times
    const int n_units = P.units_per_cta;
    const int unit0 = (int)blockIdx.z * n_units;
    const int n_pass = 2 * n_units;
    const bool want_coord = P.goff != nullptr || P.gmask != nullptr;
    const bool scatter = P.img_grad_cl != nullptr;
    const bool deformable = P.offset != nullptr;

    if (threadIdx.x == 0) {
        ptx::mbar_init(a_full, SC_WORK_WARPS);
        for (int s = 0; s < BS; ++s) {
            ptx::mbar_init(&b_full[s], 1);
            ptx::mbar_init(&b_empty[s], 1);
        }
        for (int q = 0; q < 4; ++q) {
            ptx::mbar_init(&t_full[q], 1);
            ptx::mbar_init(&t_empty[q], SC_STORE_WARPS);
        }
        for (int i = 0; i < 2; ++i) {
            ptx::mbar_init(&col_full[i], SC_STORE_WARPS);
            ptx::mbar_init(&col_empty[i], SC_GATHER_WARPS);
            ptx::mbar_init(&plan_full[i], SC_PLAN_WARPS);
            ptx::mbar_init(&plan_done[i], SC_GATHER_WARPS);
        }
        ptx::fence_mbar_init();
    }
    if (warp == SC_TMA_WARP && lane == 0) {
        ptx::prefetch_tmap(&tmap_b_hi);
        if (SPLIT) ptx::prefetch_tmap(&tmap_b_lo);
    }
    if (warp == SC_MMA_WARP) {
        ptx::tmem_alloc(tmem_slot, SC_TMEM_COLS);
        ptx::tmem_relinquish();
    }
    ptx::tc_fence_before();
    __syncthreads();
    ptx::tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp < SC_WORK_WARPS) {
        // ------------------------------------------------------------------ dense tile -> tensor memory
        // Thread = position (its TMEM lane); the 16 warps split the channels in units of 16 (8 TMEM columns).
        {
            const int q = warp & 3, part = warp >> 2;
            const PosInfo<DIM> pa = decode_position<DIM>(g, m0 + q * 32 + lane);
            const uint32_t t_lane = tmem_base + ((uint32_t)(q * 32) << 16);
            const int64_t base = ((int64_t)pa.b * g.Cd + (int64_t)grp * g.cdg) * g.P + pa.p;
            for (int u = part; u < g.cdg / 16; u += SC_WORK_WARPS / 4) {
                const int d0 = u * 16;
                uint32_t hi[8];
                if constexpr (SPLIT) {
                    const float *src = reinterpret_cast<const float *>(P.dense) + base + (int64_t)d0 * g.P;
                    float v[16];
#pragma unroll
                    for (int i = 0; i < 16; ++i) v[i] = pa.valid ? __ldg(src + (int64_t)i * g.P) : 0.f;
                    uint32_t lo[8];
#pragma unroll
                    for (int i = 0; i < 8; ++i) {
                        hi[i] = pack2(v[2 * i], v[2 * i + 1], __nv_bfloat16());
                        const float l0 = v[2 * i] - __uint_as_float(hi[i] << 16);
                        const float l1 = v[2 * i + 1] - __uint_as_float(hi[i] & 0xffff0000u);
                        lo[i] = pack2(l0, l1, __nv_bfloat16());
                    }
                    ptx::tmem_st_32x8(t_lane + (uint32_t)(d0 / 2), hi);
                    ptx::tmem_st_32x8(t_lane + (uint32_t)(a_cols + d0 / 2), lo);
                } else {
                    const uint16_t *src = reinterpret_cast<const uint16_t *>(P.dense) + base + (int64_t)d0 * g.P;
                    uint32_t v[16];
#pragma unroll
                    for (int i = 0; i < 16; ++i) v[i] = pa.valid ? (uint32_t)__ldg(src + (int64_t)i * g.P) : 0u;
#pragma unroll
                    for (int i = 0; i < 8; ++i) hi[i] = v[2 * i] | (v[2 * i + 1] << 16);
                    ptx::tmem_st_32x8(t_lane + (uint32_t)(d0 / 2), hi);
                }
            }
            ptx::tmem_st_wait();
            ptx::tc_fence_before();
            __syncwarp();
            if (lane == 0) ptx::mbar_arrive(a_full);
        }

        if (warp < SC_STORE_WARPS) {
            // -------------------------------------------------------------- store warps: TMEM -> shared
            const int q = warp;
            const int row = q * 32 + lane;
            bool ok = true;
            for (int jp = 0; jp < n_pass && ok; ++jp) {
                const int aq = jp % NACC, cb = jp & 1;
                ok = ptx::mbar_wait(&t_full[aq], (uint32_t)((jp / NACC) & 1)) &&
                     ptx::mbar_wait(&col_empty[cb], (uint32_t)(((jp >> 1) & 1) ^ 1));
                ok = __all_sync(0xffffffffu, ok);
                if (!ok) {
                    if (lane == 0) atomicExch(P.status, 301);
                    break;
                }
                ptx::tc_fence_after();
                float *dst = col + (size_t)cb * (L.col_buf / 4) + row * L.col_stride;
                const uint32_t src = tmem_base + ((uint32_t)(q * 32) << 16) + acc_col0 + (uint32_t)(aq * N);
                for (int j32 = 0; j32 < N / 32; ++j32) {
                    uint32_t raw[32];
                    ptx::tmem_ld_32x32(src + (uint32_t)(j32 * 32), raw);
                    ptx::tmem_ld_wait();
#pragma unroll
                    for (int i = 0; i < 8; ++i) {
                        float4 v;
                        v.x = __uint_as_float(raw[4 * i]);
                        v.y = __uint_as_float(raw[4 * i + 1]);
                        v.z = __uint_as_float(raw[4 * i + 2]);
                        v.w = __uint_as_float(raw[4 * i + 3]);
                        *reinterpret_cast<float4 *>(dst + j32 * 32 + i * 4) = v;
                    }
                }
                ptx::tc_fence_before();
                __syncwarp();
                if (lane == 0) {
                    ptx::mbar_arrive(&t_empty[aq]);
                    ptx::mbar_arrive(&col_full[cb]);
                }
            }
        } else {
            // -------------------------------------------------------------- gather warps
            const int gid = (warp - SC_STORE_WARPS) * 4 + (lane >> 3);
            const int l8 = lane & 7;
            using TI = typename std::conditional<SPLIT, float, T16>::type;
            const TI *img = reinterpret_cast<const TI *>(P.img_cl);
            bool ok = true;
            for (int jp = 0; jp < n_pass && ok; ++jp) {
                const int j = jp >> 1, slab = jp & 1, pb = j & 1, cb = jp & 1;
                const int unit = unit0 + j;
                const int chunk = unit / P.nbatch;
                if (slab == 0) ok = ptx::mbar_wait(&plan_full[pb], (uint32_t)((j >> 1) & 1));
                ok = ok && ptx::mbar_wait(&col_full[cb], (uint32_t)((jp >> 1) & 1));
                ok = __all_sync(0xffffffffu, ok);
                if (!ok) {
                    if (lane == 0) atomicExch(P.status, 306);
                    break;
                }
                const int n = (int)n_entries[pb];
                const int span = (n + SC_GROUPS - 1) / SC_GROUPS;
                const int e0 = gid * span;
                const int e1 = min(n, e0 + span);
                const uint32_t *p_pix = plan_pix(pb);
                const uint32_t *p_meta = plan_meta(pb);
                const float *p_w = plan_w(pb);
                float *p_dot = plan_dot(pb);
                const float4 *colb = reinterpret_cast<const float4 *>(col + (size_t)cb * (L.col_buf / 4));
                const uint32_t chan = (uint32_t)(grp * g.csg + chunk * CHUNK_C + slab * SC_SLAB + l8 * 4);
                const uint32_t Cs = (uint32_t)g.Cs;

                uint32_t e_pix[SC_PF], e_meta[SC_PF];
                float e_w[SC_PF];
                uint4 e_raw[SC_PF];   // the pixel's 4 channels of the image as loaded (converted when used)
                auto fetch = [&](int s, int e) {
                    e_pix[s] = SC_NONE;
                    e_meta[s] = 0u;
                    e_w[s] = 0.f;
                    e_raw[s] = make_uint4(0u, 0u, 0u, 0u);
                    if (e < e1) {
                        const uint32_t px = p_pix[e];
                        e_pix[s] = px;
                        e_meta[s] = p_meta[e];
                        e_w[s] = p_w[e];
                        if (want_coord) {
                            if constexpr (SPLIT) {
                                e_raw[s] = __ldg(reinterpret_cast<const uint4 *>(img + px * Cs + chan));
                            } else {
                                const uint2 r = __ldg(reinterpret_cast<const uint2 *>(img + px * Cs + chan));
                                e_raw[s].x = r.x;
                                e_raw[s].y = r.y;
                            }
                        }
                    }
                };
                auto image_values = [&](int s) -> float4 {
                    const uint4 r = e_raw[s];
                    if constexpr (SPLIT) {
                        return make_float4(__uint_as_float(r.x), __uint_as_float(r.y), __uint_as_float(r.z),
                                           __uint_as_float(r.w));
                    } else if constexpr (MODE == TC_F16) {
                        const float2 a = __half22float2(*reinterpret_cast<const __half2 *>(&r.x));
                        const float2 b = __half22float2(*reinterpret_cast<const __half2 *>(&r.y));
                        return make_float4(a.x, a.y, b.x, b.y);
                    } else {
                        return make_float4(__uint_as_float(r.x << 16), __uint_as_float(r.x & 0xffff0000u),
                                           __uint_as_float(r.y << 16), __uint_as_float(r.y & 0xffff0000u));
                    }
                };
#pragma unroll
                for (int s = 0; s < SC_PF; ++s) fetch(s, e0 + s);

                uint32_t cur = SC_NONE;
                float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
                for (int it = 0; it < span; it += SC_PF) {
#pragma unroll
                    for (int s = 0; s < SC_PF; ++s) {
                        if (it + s < span) {
                            const uint32_t px = e_pix[s];
                            if (px != cur) {
                                if (cur != SC_NONE && scatter)
                                    red_add_v4(P.img_grad_cl + cur * Cs + chan, acc.x, acc.y, acc.z, acc.w);
                                acc = make_float4(0.f, 0.f, 0.f, 0.f);
                                cur = px;
                            }
                            float d = 0.f;
                            if (px != SC_NONE) {
                                const float4 c4 = colb[(e_meta[s] & 0xffffu) + l8];
                                const float w = e_w[s];
                                acc.x = fmaf(w, c4.x, acc.x);
                                acc.y = fmaf(w, c4.y, acc.y);
                                acc.z = fmaf(w, c4.z, acc.z);
                                acc.w = fmaf(w, c4.w, acc.w);
                                const float4 iv = image_values(s);
                                d = fmaf(c4.x, iv.x, fmaf(c4.y, iv.y, fmaf(c4.z, iv.z, c4.w * iv.w)));
                            }
                            if (want_coord) {
                                d += __shfl_xor_sync(0xffffffffu, d, 1);
                                d += __shfl_xor_sync(0xffffffffu, d, 2);
                                d += __shfl_xor_sync(0xffffffffu, d, 4);
                                if (l8 == 0 && px != SC_NONE) {
                                    float *slot = p_dot + (e_meta[s] >> 16);
                                    *slot = slab == 0 ? d : *slot + d;
                                }
                            }
                            fetch(s, e0 + it + s + SC_PF);
                        }
                    }
                }
                if (cur != SC_NONE && scatter) red_add_v4(P.img_grad_cl + cur * Cs + chan, acc.x, acc.y, acc.z, acc.w);
                __syncwarp();
                if (lane == 0) {
                    ptx::mbar_arrive(&col_empty[cb]);
                    if (slab == 1) ptx::mbar_arrive(&plan_done[pb]);
                }
            }
        }
    } else if (warp < SC_MMA_WARP) {
        // ------------------------------------------------------------------ planners
        const int pt = threadIdx.x - SC_PLAN_WARP0 * 32;
        const int pw = warp - SC_PLAN_WARP0;
        const PosInfo<DIM> pi = decode_position<DIM>(g, m0 + pt);
        const uint32_t colq_row = (uint32_t)(pt * (L.col_stride / 4));

        // one thread waits, all learn the result: the named barrier must always see all 128 threads
        auto wait_all = [&](uint64_t *bar, uint32_t parity) -> bool {
            if (pt == 0) *wait_flag = ptx::mbar_wait(bar, parity) ? 1u : 0u;
            planner_barrier();
            const bool r = *wait_flag != 0u;
            planner_barrier();
            return r;
        };
        auto unit_groups = [&](int unit, int &chunk, int &t0, int &ogi, int &mgi) {
            chunk = unit / P.nbatch;
            t0 = (unit % P.nbatch) * TB;
            const int chan0 = grp * g.csg + chunk * CHUNK_C;
            ogi = g.og > 0 ? chan0 / g.cs_per_og : 0;
            mgi = g.mg > 0 ? chan0 / g.cs_per_mg : 0;
        };

        auto build = [&](int unit, int pb) {
            int chunk, t0, ogi, mgi;
            unit_groups(unit, chunk, t0, ogi, mgi);
#pragma unroll
            for (int i = 0; i < SC_HASH / 128; ++i) {
                keys[pt + 128 * i] = SC_NONE;
                cnt[pt + 128 * i] = 0u;
            }
            planner_barrier();
            // pass 1: a hash slot per distinct pixel row, a rank within the slot per entry
            uint32_t sr[TBM * NC];
#pragma unroll
            for (int t = 0; t < TBM; ++t) {
#pragma unroll
                for (int c = 0; c < NC; ++c) sr[t * NC + c] = SC_NONE;
                if (t < TB && t0 + t < g.K && pi.valid) {
                    const TapGeometry<DIM> tg = load_geometry<DIM>(g, pi, P.offset, P.mask, t0 + t, ogi, mgi);
#pragma unroll
                    for (int c = 0; c < NC; ++c) {
                        bool okc;
                        uint32_t row;
                        float w;
                        corner_of<DIM>(g, pi, tg, deformable, c, okc, row, w);
                        if (okc) {
                            uint32_t h = (row * 2654435761u) >> 21;
                            for (int probe = 0; probe < SC_HASH; ++probe) {
                                const uint32_t old = atomicCAS(&keys[h], SC_NONE, row);
                                if (old == SC_NONE || old == row) break;
                                h = (h + 1) & (SC_HASH - 1);
                            }
                            sr[t * NC + c] = (h << 16) | atomicAdd(&cnt[h], 1u);
                        }
                    }
                }
            }
            planner_barrier();
            // exclusive prefix sum of the slot counts, in place (16 slots per thread)
            {
                uint32_t v[16];
                uint32_t s = 0;
#pragma unroll
                for (int i = 0; i < 16; ++i) {
                    v[i] = cnt[pt * 16 + i];
                    s += v[i];
                }
                uint32_t inc = s;
#pragma unroll
                for (int d = 1; d < 32; d <<= 1) {
                    const uint32_t o = __shfl_up_sync(0xffffffffu, inc, d);
                    if (lane >= d) inc += o;
                }
                if (lane == 31) scan_part[pw] = inc;
                planner_barrier();
                uint32_t run = inc - s;
                for (int w = 0; w < pw; ++w) run += scan_part[w];
                if (pt == 127) n_entries[pb] = run + s;
#pragma unroll
                for (int i = 0; i < 16; ++i) {
                    cnt[pt * 16 + i] = run;
                    run += v[i];
                }
            }
            planner_barrier();
            // pass 2: write the entries to their places
            uint32_t *e_pix = plan_pix(pb);
            uint32_t *e_meta = plan_meta(pb);
            float *e_w = plan_w(pb);
#pragma unroll
            for (int t = 0; t < TBM; ++t) {
                if (t < TB && t0 + t < g.K && pi.valid) {
                    const TapGeometry<DIM> tg = load_geometry<DIM>(g, pi, P.offset, P.mask, t0 + t, ogi, mgi);
#pragma unroll
                    for (int c = 0; c < NC; ++c) {
                        bool okc;
                        uint32_t row;
                        float w;
                        corner_of<DIM>(g, pi, tg, deformable, c, okc, row, w);
                        if (okc) {
                            const uint32_t code = sr[t * NC + c];
                            const uint32_t at = cnt[code >> 16] + (code & 0xffffu);
                            e_pix[at] = row;
                            e_meta[at] = (colq_row + (uint32_t)(t * (SC_SLAB / 4))) | ((uint32_t)((pt * TB + t) * NC + c) << 16);
                            e_w[at] = w * tg.mval;
                        }
                    }
                }
            }
            planner_barrier();
            if (lane == 0) ptx::mbar_arrive(&plan_full[pb]);
        };

        // combines the dot products of a finished unit into the coordinate gradients of its (position, tap)s
        auto finalize = [&](int unit, int pb) {
            if (!want_coord || !pi.valid) return;
            int chunk, t0, ogi, mgi;
            unit_groups(unit, chunk, t0, ogi, mgi);
            const float *dots = plan_dot(pb);
#pragma unroll
            for (int t = 0; t < TBM; ++t) {
                if (t < TB && t0 + t < g.K) {
                    const int tap = t0 + t;
                    const TapGeometry<DIM> tg = load_geometry<DIM>(g, pi, P.offset, P.mask, tap, ogi, mgi);
                    float gm = 0.f, go[DIM];
#pragma unroll
                    for (int a = 0; a < DIM; ++a) go[a] = 0.f;
#pragma unroll
                    for (int c = 0; c < NC; ++c) {
                        bool okc;
                        uint32_t row;
                        float w;
                        corner_of<DIM>(g, pi, tg, deformable, c, okc, row, w);
                        if (okc) {
                            const float d = dots[(pt * TB + t) * NC + c];
                            gm = fmaf(w, d, gm);
#pragma unroll
                            for (int a = 0; a < DIM; ++a) {
                                float dw = ((c >> (DIM - 1 - a)) & 1) ? 1.f : -1.f;
#pragma unroll
                                for (int a2 = 0; a2 < DIM; ++a2)
                                    if (a2 != a) dw *= ((c >> (DIM - 1 - a2)) & 1) ? tg.fr[a2] : (1.f - tg.fr[a2]);
                                go[a] = fmaf(dw, d, go[a]);
                            }
                        }
                    }
                    if (P.goff != nullptr) {
#pragma unroll
                        for (int a = 0; a < DIM; ++a)
                            atomicAdd(P.goff + ((((int64_t)pi.b * g.og + ogi) * g.K + tap) * DIM + a) * (int64_t)g.P + pi.p,
                                      tg.mval * go[a]);
                    }
                    if (P.gmask != nullptr)
                        atomicAdd(P.gmask + (((int64_t)pi.b * g.mg + mgi) * g.K + tap) * (int64_t)g.P + pi.p, gm);
                }
            }
        };

        bool ok = true;
        for (int j = 0; j < n_units && ok; ++j) {
            const int pb = j & 1;
            if (j >= 2) {
                ok = wait_all(&plan_done[pb], (uint32_t)(((j >> 1) & 1) ^ 1));
                if (!ok) {
                    if (pt == 0) atomicExch(P.status, 307);
                    break;
                }
                finalize(unit0 + j - 2, pb);
                planner_barrier();   // the dots are read before the buffer is rebuilt
            }
            build(unit0 + j, pb);
        }
        for (int j = max(0, n_units - 2); j < n_units && ok; ++j) {
            ok = wait_all(&plan_done[j & 1], (uint32_t)((j >> 1) & 1));
            if (!ok) {
                if (pt == 0) atomicExch(P.status, 308);
                break;
            }
            finalize(unit0 + j, j & 1);
        }
    } else if (warp == SC_MMA_WARP) {
        // ------------------------------------------------------------------ MMA issue
        if (lane == 0) {
            const uint32_t idesc = ptx::instr_desc_f16(MODE == TC_F16 ? 0 : 1, TILE_POS, N, 0, 0);
            bool ok = ptx::mbar_wait(a_full, 0);
            if (!ok) atomicExch(P.status, 302);
            ptx::tc_fence_after();
            int jj = 0;  // running B stage counter
            for (int jp = 0; jp < n_pass && ok; ++jp) {
                const int aq = jp % NACC;
                if (!ptx::mbar_wait(&t_empty[aq], (uint32_t)(((jp / NACC) & 1) ^ 1))) {
                    atomicExch(P.status, 303);
                    ok = false;
                    break;
                }
                ptx::tc_fence_after();
                const uint32_t d_tmem = tmem_base + acc_col0 + (uint32_t)(aq * N);
                for (int rc = 0; rc < RC && ok; ++rc, ++jj) {
                    const int s = jj % BS;
                    if (!ptx::mbar_wait(&b_full[s], (uint32_t)((jj / BS) & 1))) {
                        atomicExch(P.status, 304);
                        ok = false;
                        break;
                    }
                    ptx::tc_fence_after();
                    const uint32_t b_addr = ptx::smem_u32(sB + (size_t)s * L.b_stage);
#pragma unroll
                    for (int k4 = 0; k4 < 4; ++k4) {
                        const uint32_t a_hi = tmem_base + (uint32_t)(rc * 32 + k4 * 8);
                        const uint64_t b_hi = ptx::smem_desc_sw128(b_addr + k4 * 32, 16, 1024);
                        ptx::mma_f16_ts(d_tmem, a_hi, b_hi, idesc, (rc > 0 || k4 > 0) ? 1u : 0u);
                        if constexpr (SPLIT) {
                            const uint64_t b_lo = ptx::smem_desc_sw128(b_addr + (uint32_t)(N * 128) + k4 * 32, 16, 1024);
                            ptx::mma_f16_ts(d_tmem, a_hi + (uint32_t)a_cols, b_hi, idesc, 1u);
                            ptx::mma_f16_ts(d_tmem, a_hi, b_lo, idesc, 1u);
                        }
                    }
                    ptx::mma_commit(&b_empty[s]);
                }
                if (ok) ptx::mma_commit(&t_full[aq]);
            }
        }
        __syncwarp();
    } else if (warp == SC_TMA_WARP) {
        // ------------------------------------------------------------------ TMA: weight ring
        if (lane == 0) {
            int jj = 0, issued = 0;
            bool ok = true;
            for (int jp = 0; jp < n_pass && ok; ++jp) {
                const int unit = unit0 + (jp >> 1);
                const int chunk = unit / P.nbatch;
                const int t0 = (unit % P.nbatch) * TB;
                const int s0 = chunk * CHUNK_C + (jp & 1) * SC_SLAB;
                for (int rc = 0; rc < RC; ++rc, ++jj) {
                    const int s = jj % BS;
                    if (!ptx::mbar_wait(&b_empty[s], (uint32_t)(((jj / BS) & 1) ^ 1))) {
                        atomicExch(P.status, 305);
                        ok = false;
                        break;
                    }
                    uint8_t *dst = sB + (size_t)s * L.b_stage;
                    ptx::mbar_arrive_expect_tx(&b_full[s], L.b_stage);
                    ptx::tma_load_4d(dst, &tmap_b_hi, &b_full[s], rc * 64, s0, t0, grp);
                    if (SPLIT) ptx::tma_load_4d(dst + N * 128, &tmap_b_lo, &b_full[s], rc * 64, s0, t0, grp);
                    issued = jj + 1;
                }
            }
            if (issued > 0) {   // no copy may still be in flight when the CTA's shared memory is released
                const int last = issued - 1;
                ptx::mbar_wait(&b_full[last % BS], (uint32_t)((last / BS) & 1));
            }
        }
        __syncwarp();
    }

    ptx::tc_fence_before();
    __syncthreads();
    if (warp == SC_MMA_WARP) ptx::tmem_dealloc(tmem_base, SC_TMEM_COLS);
}

size_t dgrad_smem_bytes(int dim, int mode, int tb, int b_stages) {
    return 1024 + sc_layout(dim, mode, tb, b_stages).total;
}

template <int DIM, int MODE>
cudaError_t launch_dgrad_t(const DgradParams<DIM> &P, dim3 grid, const CUtensorMap *maps, cudaStream_t stream) {
    const size_t smem = dgrad_smem_bytes(DIM, MODE, P.tb, P.b_stages);
    auto kern = dcn_dgrad_tc_kernel<DIM, MODE>;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return e;
    LaunchScope scope("dcn_dgrad_tc", stream);
    kern<<<grid, SC_THREADS, smem, stream>>>(P, maps[0], maps[1]);
    return cudaGetLastError();
}

}  // namespace

// Taps per batch, accumulator ring and weight-ring depth that fit tensor memory and shared memory; false when
// nothing fits (the dense tile of one group must fit tensor memory beside one accumulator).
bool dgrad_tc_config(int dim, int mode, int cdg, int K, int *tb, int *nacc, int *b_stages) {
    static const int tb_cap = tuning_int("TVDCN_B200_DG_TB", 4);
    static const int st_cap = tuning_int("TVDCN_B200_DG_STAGES", 4);
    const int a_cols = (cdg / 2) * (mode == TC_SPLIT ? 2 : 1);
    for (int cand = std::min(std::min(sc_tb_max(dim), tb_cap), K); cand >= 1; --cand) {
        // equal batches: the fewest batches of at most `cand` taps
        const int nb = (K + cand - 1) / cand;
        const int t = (K + nb - 1) / nb;
        const int n = t * SC_SLAB;
        const int acc = std::min(4, (SC_TMEM_COLS - a_cols) / n);
        if (acc < 1) continue;
        for (int st = std::min(st_cap, 4); st >= 2; --st)
            if (dgrad_smem_bytes(dim, mode, t, st) <= 227 * 1024) {
                *tb = t;
                *nacc = acc;
                *b_stages = st;
                return true;
            }
    }
    return false;
}

// dense: [B, Cd, P] in the problem's data type; w_kd_*: weights packed [g][tap][s'][d'] 16-bit (hi / lo);
// img_cl: sampled image channels-last (needed for goff / gmask); accumulation targets are f32 and initialised by
// the caller.
cudaError_t launch_gemm_scatter_tc(const GeoHost &h, int mode, const void *dense, const void *w_kd_hi,
                                   const void *w_kd_lo, const void *img_cl, const float *offset, const float *mask,
                                   float *img_grad_cl, float *goff, float *gmask, int *status, cudaStream_t stream) {
    const int cdg = h.Cd / h.groups, csg = h.Cs / h.groups;
    int tb = 0, nacc = 0, bs = 0;
    if (!dgrad_tc_config(h.dim, mode, cdg, h.K, &tb, &nacc, &bs)) return cudaErrorInvalidConfiguration;
    const int nbatch = (h.K + tb - 1) / tb;
    const long long BP = (long long)h.B * h.P;
    CUtensorMap maps[2];
    {
        const uint64_t dims[4] = {(uint64_t)cdg, (uint64_t)csg, (uint64_t)h.K, (uint64_t)h.groups};
        const uint64_t strides[3] = {(uint64_t)cdg * 2, (uint64_t)cdg * csg * 2, (uint64_t)cdg * csg * h.K * 2};
        const uint32_t box[4] = {64, (uint32_t)SC_SLAB, (uint32_t)tb, 1};
        if (!make_tensor_map_16bit(&maps[0], w_kd_hi, 4, dims, strides, box)) return cudaErrorInvalidValue;
        if (mode == TC_SPLIT) {
            if (!make_tensor_map_16bit(&maps[1], w_kd_lo, 4, dims, strides, box)) return cudaErrorInvalidValue;
        } else {
            maps[1] = maps[0];
        }
    }
    // Share each position tile between `splits` CTAs (equal ranges of its units) when that evens out the last
    // wave: cost of a launch ~ ceil(CTAs / SMs) / splits tile-times; a split is taken only for a gain above 4 %
    // (each extra CTA reloads the dense tile).
    const long long tiles = ((BP + TILE_POS - 1) / TILE_POS) * h.groups;
    const int n_units = (csg / CHUNK_C) * nbatch;
    int splits = 1;
    {
        static const int forced = tuning_int("TVDCN_B200_DG_SPLITS", 0);
        double best = (double)((tiles + 147) / 148);
        for (int cand = 2; cand <= 4; ++cand) {
            if (n_units % cand != 0) continue;
            const double cost = (double)((tiles * cand + 147) / 148) / cand;
            if (cost < best * 0.96) { best = cost; splits = cand; }
        }
        if (forced > 0 && n_units % forced == 0) splits = forced;
    }
    dim3 grid((unsigned)((BP + TILE_POS - 1) / TILE_POS), (unsigned)h.groups, (unsigned)splits);
    auto run = [&](auto dimc) -> cudaError_t {
        constexpr int DIM = decltype(dimc)::value;
        DgradParams<DIM> P;
        P.g = geo_from_host<DIM>(h);
        P.dense = dense;
        P.img_cl = img_cl;
        P.offset = offset;
        P.mask = mask;
        P.img_grad_cl = img_grad_cl;
        P.goff = goff;
        P.gmask = gmask;
        P.status = status;
        P.rc = cdg / 64;
        P.tb = tb;
        P.nbatch = nbatch;
        P.nacc = nacc;
        P.b_stages = bs;
        P.units_per_cta = n_units / splits;
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
