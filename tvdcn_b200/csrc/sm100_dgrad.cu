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
// Warp roles (768 threads): 0-3 store, 4-15 gather, 16-19 planners, 20 MMA issue + TMEM owner, 21 TMA, 22-23 idle
// (they complete the last warpgroup for the register hand-over).
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
constexpr int SC_WORK_WARPS = SC_STORE_WARPS + SC_GATHER_WARPS;
constexpr int SC_LOAD_WARPS = 16;                                 // the first 16 of them load the dense tile first
constexpr int SC_PLAN_WARP0 = SC_WORK_WARPS;
constexpr int SC_PLAN_WARPS = 4;                                  // one planner thread per tile position
constexpr int SC_MMA_WARP = SC_PLAN_WARP0 + SC_PLAN_WARPS;
constexpr int SC_TMA_WARP = SC_MMA_WARP + 1;
constexpr int SC_THREADS = (SC_TMA_WARP + 3) * 32;                // two idle warps complete the last warpgroup
static_assert(SC_THREADS == 768, "six warpgroups");
// Registers per thread after the warpgroups have rebalanced them (launch: 80 each for 6 warpgroups = 480 x 128):
// the three gather warpgroups and the planners take 96, the store warps keep 56, the MMA / TMA warpgroup 40:
// 4 x 96 + 56 + 40 = 480.
constexpr int SC_REGS_WORK = 96, SC_REGS_STORE = 56, SC_REGS_ISSUE = 40;
constexpr int SC_GROUPS = SC_GATHER_WARPS * 4;                    // 8-lane groups walking the entry list
constexpr int SC_SLAB = 32;                                       // channels per pass
constexpr int SC_PLAN_SLACK = SC_GROUPS * 4 + 16;
constexpr int SC_HASH = 2048;                                     // slots; >= entries of one unit
constexpr uint32_t SC_NONE = 0xffffffffu;
constexpr int SC_TMEM_COLS = 512;
constexpr int SC_SLEEP_NS = 32;                                   // back-off of the long waits (64 to 512 measured equal)
constexpr int SC_MAX_TAPS = 512;                                  // taps whose kernel coordinates a CTA tabulates

// most taps per batch: 128 * tb * 2^dim entries must fit the hash table
__host__ __device__ constexpr int sc_tb_max(int dim) { return dim == 1 ? 4 : (dim == 2 ? 3 : 2); }

// Predicated form: no branch around the reduction, and no "memory" clobber either -- nothing in this kernel reads
// what the reduction writes, and the shared-memory loads around it must stay free to move.
__device__ __forceinline__ void red_add_v4_if(bool p, float *addr, float a, float b, float c, float d) {
    asm volatile(
        "{\n\t"
        ".reg .pred q;\n\t"
        "setp.ne.b32 q, %5, 0;\n\t"
        "@q red.global.add.v4.f32 [%0], {%1, %2, %3, %4};\n\t"
        "}\n" ::"l"(addr), "f"(a), "f"(b), "f"(c), "f"(d), "r"((int)p));
}

// Cycle counters of one CTA in the middle of the grid, per role; compiled in only with -DTVDCN_B200_TUNING.
#ifdef TVDCN_B200_TUNING
__device__ long long g_dg_prof[64];
#define SC_CLK() clock64()
#define SC_PROF_OUT(i, v) do { if (prof_cta) g_dg_prof[i] = (v); } while (0)
#else
#define SC_CLK() 0ll
#define SC_PROF_OUT(i, v) do { (void)(v); } while (0)
#endif

__device__ __forceinline__ void planner_barrier() { asm volatile("bar.sync 1, 128;" ::: "memory"); }

// Sampling geometry of one (position, tap): floor and fraction per axis, mask value.
template <int DIM>
struct TapGeometry {
    int fl[DIM];
    float fr[DIM];
    float mval;
};

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
    uint32_t b_stage, col_buf, plan_buf, col, plan, keys, cnt, taps, misc, bars, total;
    int n, col_stride, max_entries;
};
__host__ __device__ inline ScLayout sc_layout(int dim, int mode, int tb, int b_stages) {
    ScLayout L;
    const int parts = mode == TC_SPLIT ? 2 : 1;
    L.n = tb * SC_SLAB;
    L.col_stride = L.n + 4;                       // words; = 4 mod 32, so that the row-per-lane stores spread over the banks
    L.max_entries = TILE_POS * tb * (1 << dim);
    L.b_stage = (uint32_t)(L.n * 128);             // one 16-bit part (hi or lo) of one reduction chunk
    (void)parts;
    L.col_buf = (uint32_t)(TILE_POS * L.col_stride * 4);
    // three arrays (pixel offset; col index | dot slot << 16; weight) of max_entries + SC_PLAN_SLACK words -- room for
    // the padding of the groups' spans and the read-ahead of the last group -- then one dot product per entry (+ a
    // slot for the padding entries)
    L.plan_buf = (uint32_t)(3 * (L.max_entries + SC_PLAN_SLACK) * 4 + (L.max_entries + 4) * 4);
    uint32_t o = 0;
    o += (uint32_t)b_stages * L.b_stage;
    L.col = o;  o += 2 * L.col_buf;
    L.plan = o; o += 2 * L.plan_buf;
    L.keys = o; o += SC_HASH * 4;
    L.cnt = o;  o += SC_HASH * 4;
    L.taps = o; o += SC_MAX_TAPS * 3 * 2;         // kernel coordinates of every tap (int16)
    L.misc = o; o += 64;                          // scan partial sums [4], wait flag, entry counts [2], TMEM slot
    L.bars = o; o += (uint32_t)(19 + 2 * b_stages) * 8;
    L.total = o;
    return L;
}

template <int DIM, int MODE, bool COORD>
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
    uint64_t *plan_done = plan_full + 2; // [2] gather warps -> whoever turns the unit's dots into gradients / planners
    uint64_t *fin_done = plan_done + 2;  // [2] store warps -> planners: the unit's dots have been used
    int16_t *tap_tab = reinterpret_cast<int16_t *>(smem + L.taps);
    // Entry e of the pixel-grouped list sits at word e of each array; a group's span is a multiple of four entries, so
    // that a batch of four is one 16-byte read per array (each 8-lane group is a quarter-warp phase of its own: the
    // four groups of a warp never meet in one bank access).
    const int plan_words = L.max_entries + SC_PLAN_SLACK;
    auto plan_px = [&](int pb) { return reinterpret_cast<uint32_t *>(smem + L.plan + (size_t)pb * L.plan_buf); };
    auto plan_meta = [&](int pb) { return plan_px(pb) + plan_words; };
    auto plan_w = [&](int pb) { return reinterpret_cast<float *>(plan_px(pb) + 2 * plan_words); };
    auto plan_dot = [&](int pb) { return reinterpret_cast<float *>(plan_px(pb) + 3 * plan_words); };

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int grp = blockIdx.y;
    const long long m0 = (long long)blockIdx.x * TILE_POS;
    // units of this CTA: gridDim.z CTAs share one position tile and take equal ranges of its units, which evens
    // out the last wave when the tiles do not fill the SMs a whole number of times
    const int n_units = P.units_per_cta;
    const int unit0 = (int)blockIdx.z * n_units;
    const int n_pass = 2 * n_units;
    constexpr bool want_coord = COORD;    // grad_offset and / or grad_mask are wanted
    const bool scatter = P.img_grad_cl != nullptr;
    const bool deformable = P.offset != nullptr;
    const bool prof_cta = blockIdx.x == gridDim.x / 2 && blockIdx.y == 0 && blockIdx.z == 0;
    (void)prof_cta;
    const long long clk_start = SC_CLK();

    if (threadIdx.x == 0) {
        ptx::mbar_init(a_full, SC_LOAD_WARPS);
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
            ptx::mbar_init(&fin_done[i], SC_STORE_WARPS);
        }
        ptx::fence_mbar_init();
    }
    for (int tp = threadIdx.x; tp < g.K; tp += SC_THREADS) {
        int tc[DIM];
        tap_coords<DIM>(g, tp, tc);
#pragma unroll
        for (int a = 0; a < DIM; ++a) tap_tab[tp * DIM + a] = (int16_t)tc[a];
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

    // ---- pieces shared by the planners (which build a unit's entry list) and the store warps (which turn its dot
    // products into coordinate gradients); both map thread -> position of the tile
    auto unit_groups = [&](int unit, int &t0, int &ogi, int &mgi) {
        const int chunk = unit / P.nbatch;
        t0 = (unit % P.nbatch) * TB;
        const int chan0 = grp * g.csg + chunk * CHUNK_C;
        ogi = g.og > 0 ? chan0 / g.cs_per_og : 0;
        mgi = g.mg > 0 ? chan0 / g.cs_per_mg : 0;
    };
    // offsets and mask of this position for the taps of one unit, as loaded (all loads in flight together)
    struct RawUnit {
        float off[TBM][DIM];
        float m[TBM];
    };
    auto load_unit = [&](const PosInfo<DIM> &pi, int unit, RawUnit &ru) {
        int t0, ogi, mgi;
        unit_groups(unit, t0, ogi, mgi);
#pragma unroll
        for (int t = 0; t < TBM; ++t) {
            const bool live = t < TB && t0 + t < g.K && pi.valid;
#pragma unroll
            for (int a = 0; a < DIM; ++a)
                ru.off[t][a] = (live && P.offset != nullptr)
                                   ? __ldg(P.offset + ((((int64_t)pi.b * g.og + ogi) * g.K + t0 + t) * DIM + a) * (int64_t)g.P + pi.p)
                                   : 0.f;
            ru.m[t] = (live && P.mask != nullptr)
                          ? __ldg(P.mask + (((int64_t)pi.b * g.mg + mgi) * g.K + t0 + t) * (int64_t)g.P + pi.p)
                          : 1.f;
        }
    };
    auto geometry = [&](const PosInfo<DIM> &pi, const RawUnit &ru, int t, int tap) -> TapGeometry<DIM> {
        TapGeometry<DIM> tg;
#pragma unroll
        for (int a = 0; a < DIM; ++a) {
            const int base = pi.base[a] + (int)tap_tab[tap * DIM + a] * g.dil[a];
            if (deformable) {
                const float pos = (float)base + ru.off[t][a];
                const float f = floorf(pos);
                tg.fl[a] = (int)f;
                tg.fr[a] = pos - f;
            } else {
                tg.fl[a] = base;
                tg.fr[a] = 0.f;
            }
        }
        tg.mval = ru.m[t];
        return tg;
    };

    // combines the dot products of a finished unit into the coordinate gradients of its (position, tap)s
    auto finalize = [&](const PosInfo<DIM> &pi, int pt, int unit, int pb, const RawUnit &ru) {
        if (!want_coord || !pi.valid) return;
        int t0, ogi, mgi;
        unit_groups(unit, t0, ogi, mgi);
        const float *dots = plan_dot(pb);
#pragma unroll
        for (int t = 0; t < TBM; ++t) {
            if (t < TB && t0 + t < g.K) {
                const int tap = t0 + t;
                const TapGeometry<DIM> tg = geometry(pi, ru, t, tap);
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


    // ------------------------------------------------------------------ dense tile -> tensor memory
    // Thread = position (its TMEM lane); the 16 store + gather warps split the channels in units of 16 (8 TMEM
    // columns).
    auto load_dense = [&]() {
        const int q = warp & 3, part = warp >> 2;
        const PosInfo<DIM> pa = decode_position<DIM>(g, m0 + q * 32 + lane);
        const uint32_t t_lane = tmem_base + ((uint32_t)(q * 32) << 16);
        const int64_t base = ((int64_t)pa.b * g.Cd + (int64_t)grp * g.cdg) * g.P + pa.p;
        // two units (32 loads) in flight per thread: the tile is read once from DRAM, its latency is what counts
        const int n_units_a = g.cdg / 16;
        for (int u0 = part; u0 < n_units_a; u0 += 2 * (SC_LOAD_WARPS / 4)) {
            const int u1 = u0 + SC_LOAD_WARPS / 4;
            const bool two = u1 < n_units_a;
            if constexpr (SPLIT) {
                const float *src0 = reinterpret_cast<const float *>(P.dense) + base + (int64_t)(u0 * 16) * g.P;
                const float *src1 = reinterpret_cast<const float *>(P.dense) + base + (int64_t)(u1 * 16) * g.P;
                float v[2][16];
#pragma unroll
                for (int i = 0; i < 16; ++i) v[0][i] = pa.valid ? __ldg(src0 + (int64_t)i * g.P) : 0.f;
#pragma unroll
                for (int i = 0; i < 16; ++i) v[1][i] = (pa.valid && two) ? __ldg(src1 + (int64_t)i * g.P) : 0.f;
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    if (h == 1 && !two) break;
                    const int d0 = (h == 0 ? u0 : u1) * 16;
                    uint32_t hi[8], lo[8];
#pragma unroll
                    for (int i = 0; i < 8; ++i) {
                        hi[i] = pack2(v[h][2 * i], v[h][2 * i + 1], __nv_bfloat16());
                        const float l0 = v[h][2 * i] - __uint_as_float(hi[i] << 16);
                        const float l1 = v[h][2 * i + 1] - __uint_as_float(hi[i] & 0xffff0000u);
                        lo[i] = pack2(l0, l1, __nv_bfloat16());
                    }
                    ptx::tmem_st_32x8(t_lane + (uint32_t)(d0 / 2), hi);
                    ptx::tmem_st_32x8(t_lane + (uint32_t)(a_cols + d0 / 2), lo);
                }
            } else {
                const uint16_t *src0 = reinterpret_cast<const uint16_t *>(P.dense) + base + (int64_t)(u0 * 16) * g.P;
                const uint16_t *src1 = reinterpret_cast<const uint16_t *>(P.dense) + base + (int64_t)(u1 * 16) * g.P;
                uint32_t v[2][16];
#pragma unroll
                for (int i = 0; i < 16; ++i) v[0][i] = pa.valid ? (uint32_t)__ldg(src0 + (int64_t)i * g.P) : 0u;
#pragma unroll
                for (int i = 0; i < 16; ++i) v[1][i] = (pa.valid && two) ? (uint32_t)__ldg(src1 + (int64_t)i * g.P) : 0u;
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    if (h == 1 && !two) break;
                    const int d0 = (h == 0 ? u0 : u1) * 16;
                    uint32_t hi[8];
#pragma unroll
                    for (int i = 0; i < 8; ++i) hi[i] = v[h][2 * i] | (v[h][2 * i + 1] << 16);
                    ptx::tmem_st_32x8(t_lane + (uint32_t)(d0 / 2), hi);
                }
            }
        }
        ptx::tmem_st_wait();
        ptx::tc_fence_before();
        __syncwarp();
        if (lane == 0) ptx::mbar_arrive(a_full);
        if (threadIdx.x == 0) SC_PROF_OUT(1, SC_CLK() - clk_start);
    };

    if (warp < SC_WORK_WARPS) {
        if (warp < SC_STORE_WARPS) {
            // -------------------------------------------------------------- store warps: TMEM -> shared
            load_dense();                      // with the launch allocation, before registers are handed over
            ptx::reg_dec<SC_REGS_STORE>();
            const int q = warp;
            const int row = q * 32 + lane;
            const PosInfo<DIM> pi = decode_position<DIM>(g, m0 + row);
            bool ok = true;
            long long w_tfull = 0, w_cempty = 0, t_fin = 0;
            // The gather warps finish unit j (its dot products are complete) with pass 2 j + 1; the wait for that
            // pass' staging buffer below covers it, so the unit is turned into gradients right after the next store.
            auto finish_unit = [&](int j, const RawUnit &ru) -> bool {
                const int pb = j & 1;
                bool good = ptx::mbar_wait(&plan_done[pb], (uint32_t)((j >> 1) & 1));
                good = __all_sync(0xffffffffu, good);
                if (!good) {
                    if (lane == 0) atomicExch(P.status, 308);
                    return false;
                }
                finalize(pi, row, unit0 + j, pb, ru);
                __syncwarp();
                if (lane == 0) ptx::mbar_arrive(&fin_done[pb]);
                return true;
            };
            for (int jp = 0; jp < n_pass && ok; ++jp) {
                const int aq = jp % NACC, cb = jp & 1;
                const bool fin_now = COORD && jp >= 3 && (jp & 1) == 1;   // pass jp - 2 closed unit (jp - 2) / 2
                RawUnit ru_fin;
                if (fin_now) load_unit(pi, unit0 + ((jp - 2) >> 1), ru_fin);
                long long c0 = SC_CLK();
                ok = ptx::mbar_wait(&t_full[aq], (uint32_t)((jp / NACC) & 1));
                long long c1 = SC_CLK();
                ok = ok && ptx::mbar_wait_backoff<SC_SLEEP_NS>(&col_empty[cb], (uint32_t)(((jp >> 1) & 1) ^ 1));
                w_tfull += c1 - c0;
                w_cempty += SC_CLK() - c1;
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
                if (fin_now) {
                    long long c3 = SC_CLK();
                    ok = finish_unit((jp - 2) >> 1, ru_fin);
                    t_fin += SC_CLK() - c3;
                }
            }
            if (COORD && ok) {   // the last unit
                RawUnit ru_fin;
                load_unit(pi, unit0 + n_units - 1, ru_fin);
                ok = finish_unit(n_units - 1, ru_fin);
            }
            if (threadIdx.x == 0) {
                SC_PROF_OUT(2, w_tfull);
                SC_PROF_OUT(3, w_cempty);
                SC_PROF_OUT(4, SC_CLK() - clk_start);
                SC_PROF_OUT(18, t_fin);
            }
        } else {
            // -------------------------------------------------------------- gather warps
            if (warp < SC_LOAD_WARPS) load_dense();
            ptx::reg_inc<SC_REGS_WORK>();
            // An 8-lane group walks its span of the pixel-grouped entry list four entries at a time; lane l8 owns
            // channels 4 l8 .. 4 l8 + 3 of the slab.  The next four entries (and their image rows) are fetched
            // while the current four are processed.
            const int gid = (warp - SC_STORE_WARPS) * 4 + (lane >> 3);
            const int l8 = lane & 7;
            using TI = typename std::conditional<SPLIT, float, T16>::type;
            using RAW = typename std::conditional<SPLIT, uint4, uint2>::type;
            const TI *img = reinterpret_cast<const TI *>(P.img_cl);
            const uint32_t zrow = (uint32_t)g.B * (uint32_t)g.S * (uint32_t)g.Cs;   // what padding entries point at
            bool ok = true;
            long long w_plan = 0, w_col = 0, t_loop = 0, n_ent = 0;
            for (int jp = 0; jp < n_pass && ok; ++jp) {
                const int j = jp >> 1, slab = jp & 1, pb = j & 1, cb = jp & 1;
                const int unit = unit0 + j;
                const int chunk = unit / P.nbatch;
                long long c0 = SC_CLK();
                if (slab == 0) ok = ptx::mbar_wait(&plan_full[pb], (uint32_t)((j >> 1) & 1));
                long long c1 = SC_CLK();
                ok = ok && ptx::mbar_wait(&col_full[cb], (uint32_t)((jp >> 1) & 1));
                long long c2 = SC_CLK();
                w_plan += c1 - c0;
                w_col += c2 - c1;
                ok = __all_sync(0xffffffffu, ok);
                if (!ok) {
                    if (lane == 0) atomicExch(P.status, 306);
                    break;
                }
                const int span = (int)n_entries[pb];     // entries per group, padded: a multiple of 4
                const uint4 *my_px = reinterpret_cast<const uint4 *>(plan_px(pb) + gid * span);
                const uint4 *my_meta = reinterpret_cast<const uint4 *>(plan_meta(pb) + gid * span);
                const float4 *my_w = reinterpret_cast<const float4 *>(plan_w(pb) + gid * span);
                float *p_dot = plan_dot(pb);
                const float4 *colb = reinterpret_cast<const float4 *>(col + (size_t)cb * (L.col_buf / 4)) + l8;
                const uint32_t chan = (uint32_t)(grp * g.csg + chunk * CHUNK_C + slab * SC_SLAB + l8 * 4);
                const TI *img_c = img + chan;
                float *gimg_c = P.img_grad_cl + chan;

                uint32_t cur = zrow;
                float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
                // pixel offsets of the four entries at `at`, and (for the coordinate gradients) their image rows
                auto fetch_rows = [&](uint32_t (&px)[4], RAW (&R)[4], int at) {
                    const uint4 p4 = my_px[at >> 2];
                    px[0] = p4.x; px[1] = p4.y; px[2] = p4.z; px[3] = p4.w;
                    if constexpr (COORD) {
#pragma unroll
                        for (int s = 0; s < 4; ++s) R[s] = __ldg(reinterpret_cast<const RAW *>(img_c + px[s]));
                    }
                };
                auto image_values = [&](const RAW &r) -> float4 {
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
                auto process = [&](int at, const uint32_t (&pxs)[4], const RAW (&R)[4]) {
                    const uint4 m4 = my_meta[at >> 2];
                    const float4 w4 = my_w[at >> 2];
                    const uint32_t meta[4] = {m4.x, m4.y, m4.z, m4.w};
                    const float wt[4] = {w4.x, w4.y, w4.z, w4.w};
                    float d[4];
#pragma unroll
                    for (int s = 0; s < 4; ++s) {
                        const uint32_t px = pxs[s];
                        const bool change = px != cur;
                        red_add_v4_if(change && scatter, gimg_c + cur, acc.x, acc.y, acc.z, acc.w);
                        cur = px;
                        const float4 c4 = colb[meta[s] & 0xffffu];
                        const float w = wt[s];
                        acc.x = fmaf(w, c4.x, change ? 0.f : acc.x);
                        acc.y = fmaf(w, c4.y, change ? 0.f : acc.y);
                        acc.z = fmaf(w, c4.z, change ? 0.f : acc.z);
                        acc.w = fmaf(w, c4.w, change ? 0.f : acc.w);
                        if constexpr (COORD) {
                            const float4 iv = image_values(R[s]);
                            d[s] = fmaf(c4.x, iv.x, fmaf(c4.y, iv.y, fmaf(c4.z, iv.z, c4.w * iv.w)));
                        }
                    }
                    if constexpr (COORD) {
                        // sums over the 8 lanes of the four dots at once: after the exchanges lane (b2 b1 b0) holds
                        // the dot of entry 2 b2 + b1
                        const bool h4 = (l8 & 4) != 0, h2 = (l8 & 2) != 0;
                        float k0 = h4 ? d[2] : d[0], k1 = h4 ? d[3] : d[1];
                        k0 += __shfl_xor_sync(0xffffffffu, h4 ? d[0] : d[2], 4);
                        k1 += __shfl_xor_sync(0xffffffffu, h4 ? d[1] : d[3], 4);
                        float k = h2 ? k1 : k0;
                        k += __shfl_xor_sync(0xffffffffu, h2 ? k0 : k1, 2);
                        k += __shfl_xor_sync(0xffffffffu, k, 1);
                        if ((l8 & 1) == 0) {
                            const uint32_t m = h4 ? (h2 ? meta[3] : meta[2]) : (h2 ? meta[1] : meta[0]);
                            float *slot = p_dot + (m >> 16);
                            *slot = slab == 0 ? k : *slot + k;
                        }
                    }
                };
                RAW Ra[4], Rb[4];
                uint32_t Pa[4], Pb[4];
                if (span > 0) {
                    fetch_rows(Pa, Ra, 0);
                    // The running pixel starts as the first entry's: no flush before anything was summed.  Padding
                    // entries (pixel offset zrow) only follow real ones, so inside the loop a flush never has
                    // cur == zrow; the one after the loop may.
                    cur = Pa[0];
                }
                for (int it = 0; it < span; it += 8) {
                    // the fetch one batch ahead may run up to 8 entries past the span: still inside the list's slack
                    fetch_rows(Pb, Rb, it + 4);
                    process(it, Pa, Ra);
                    if (it + 4 < span) {
                        fetch_rows(Pa, Ra, it + 8);
                        process(it + 4, Pb, Rb);
                    }
                }
                red_add_v4_if(cur != zrow && scatter, gimg_c + cur, acc.x, acc.y, acc.z, acc.w);
                __syncwarp();
                if (lane == 0) {
                    ptx::mbar_arrive(&col_empty[cb]);
                    if (slab == 1) ptx::mbar_arrive(&plan_done[pb]);
                }
                t_loop += SC_CLK() - c2;
                n_ent += span;
            }
            if (threadIdx.x == SC_STORE_WARPS * 32) {
                SC_PROF_OUT(8, w_plan);
                SC_PROF_OUT(9, w_col);
                SC_PROF_OUT(10, t_loop);
                SC_PROF_OUT(11, n_ent);
                SC_PROF_OUT(12, SC_CLK() - clk_start);
            }
        }
    } else if (warp < SC_MMA_WARP) {
        // ------------------------------------------------------------------ planners
        ptx::reg_inc<SC_REGS_WORK>();
        const int pt = threadIdx.x - SC_PLAN_WARP0 * 32;
        const int pw = warp - SC_PLAN_WARP0;
        const PosInfo<DIM> pi = decode_position<DIM>(g, m0 + pt);
        const uint32_t colq_row = (uint32_t)(pt * (L.col_stride / 4));
        const uint32_t zrow = (uint32_t)g.B * (uint32_t)g.S * (uint32_t)g.Cs;

        // one thread waits, all learn the result: the named barrier must always see all 128 threads
        auto wait_all = [&](uint64_t *bar, uint32_t parity) -> bool {
            if (pt == 0) *wait_flag = ptx::mbar_wait_backoff<SC_SLEEP_NS>(bar, parity) ? 1u : 0u;
            planner_barrier();
            const bool r = *wait_flag != 0u;
            planner_barrier();
            return r;
        };
        long long ph[6] = {0, 0, 0, 0, 0, 0};
        auto build = [&](int unit, int pb, const RawUnit &ru) {
            long long pc = SC_CLK();
            auto phase = [&](int i) { const long long now = SC_CLK(); ph[i] += now - pc; pc = now; };
            int t0, ogi, mgi;
            unit_groups(unit, t0, ogi, mgi);
            {
                uint4 *k4 = reinterpret_cast<uint4 *>(keys), *c4 = reinterpret_cast<uint4 *>(cnt);
#pragma unroll
                for (int i = 0; i < SC_HASH / 4 / 128; ++i) {
                    k4[pt + 128 * i] = make_uint4(SC_NONE, SC_NONE, SC_NONE, SC_NONE);
                    c4[pt + 128 * i] = make_uint4(0u, 0u, 0u, 0u);
                }
            }
            planner_barrier();
            phase(0);
            // pass 1: a hash slot per distinct pixel row, and the entry's rank among the entries of that row.  First
            // probe of every entry before any retry, so that the shared-memory atomics of one thread overlap.
            uint32_t rows[TBM * NC], slot[TBM * NC];
            float wts[TBM * NC];
#pragma unroll
            for (int t = 0; t < TBM; ++t) {
                const bool live = t < TB && t0 + t < g.K && pi.valid;
                const TapGeometry<DIM> tg = geometry(pi, ru, t, t0 + t);
#pragma unroll
                for (int c = 0; c < NC; ++c) {
                    bool okc;
                    uint32_t row;
                    float w;
                    corner_of<DIM>(g, pi, tg, deformable, c, okc, row, w);
                    rows[t * NC + c] = (live && okc) ? row : SC_NONE;
                    wts[t * NC + c] = w * tg.mval;
                }
            }
            uint32_t old[TBM * NC];
#pragma unroll
            for (int i = 0; i < TBM * NC; ++i) {
                slot[i] = (rows[i] * 2654435761u) >> 21;
                old[i] = rows[i] != SC_NONE ? atomicCAS(&keys[slot[i]], SC_NONE, rows[i]) : rows[i];
            }
#pragma unroll
            for (int i = 0; i < TBM * NC; ++i) {
                if (rows[i] != SC_NONE) {
                    uint32_t o = old[i];
                    for (int probe = 0; probe < SC_HASH && o != SC_NONE && o != rows[i]; ++probe) {
                        slot[i] = (slot[i] + 1) & (SC_HASH - 1);
                        o = atomicCAS(&keys[slot[i]], SC_NONE, rows[i]);
                    }
                    old[i] = atomicAdd(&cnt[slot[i]], 1u);   // from here on: the entry's rank within its pixel's run
                }
            }
            phase(1);
            planner_barrier();
            phase(2);
            // exclusive prefix sum of the slot counts, in place (16 slots per thread)
            uint32_t total;
            {
                uint32_t v[16];
                uint32_t s = 0;
                const uint4 *c4 = reinterpret_cast<const uint4 *>(cnt + pt * 16);
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const uint4 x = c4[i];
                    v[4 * i] = x.x; v[4 * i + 1] = x.y; v[4 * i + 2] = x.z; v[4 * i + 3] = x.w;
                    s += x.x + x.y + x.z + x.w;
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
                total = 0;
#pragma unroll
                for (int w = 0; w < SC_PLAN_WARPS; ++w) {
                    const uint32_t part = scan_part[w];
                    if (w < pw) run += part;
                    total += part;
                }
#pragma unroll
                for (int i = 0; i < 16; ++i) {
                    cnt[pt * 16 + i] = run;
                    run += v[i];
                }
            }
            // entries per gather group: a multiple of 4; the list is padded with entries that add nothing
            const uint32_t span = ((total + SC_GROUPS * 4 - 1) / (SC_GROUPS * 4)) * 4;
            if (pt == 0) n_entries[pb] = span;
            planner_barrier();
            phase(3);
            // pass 2: every entry goes to (start of its pixel's run) + (its rank)
            uint32_t *e_px = plan_px(pb);
            uint32_t *e_meta = plan_meta(pb);
            float *e_w = plan_w(pb);
#pragma unroll
            for (int t = 0; t < TBM; ++t) {
#pragma unroll
                for (int c = 0; c < NC; ++c) {
                    const int i = t * NC + c;
                    if (rows[i] != SC_NONE) {
                        const uint32_t at = cnt[slot[i]] + old[i];
                        e_px[at] = rows[i] * (uint32_t)g.Cs;
                        e_meta[at] = (colq_row + (uint32_t)(t * (SC_SLAB / 4))) | ((uint32_t)((pt * TB + t) * NC + c) << 16);
                        e_w[at] = wts[i];
                    }
                }
            }
            // padding entries up to the end of the last span and the words the read-ahead of the last group touches:
            // all point at the row of zeros and add nothing
            const uint32_t n_words = span * SC_GROUPS + 8;
            for (uint32_t i = total + pt; i < n_words; i += 128) {
                e_px[i] = zrow;
                e_meta[i] = (uint32_t)L.max_entries << 16;
                e_w[i] = 0.f;
            }
            phase(4);
            planner_barrier();
            phase(5);
            if (lane == 0) ptx::mbar_arrive(&plan_full[pb]);
        };

        bool ok = true;
        long long w_done = 0, t_build = 0;
        // a plan buffer is free again once its unit's dots have been used (store warps), or, without coordinate
        // gradients, once the gather warps are through with it
        uint64_t *plan_free = COORD ? fin_done : plan_done;
        RawUnit ru, ru_next;
        load_unit(pi, unit0, ru);
        ru_next = ru;
        for (int j = 0; j < n_units && ok; ++j) {
            const int pb = j & 1;
            // the next unit's offsets and mask travel while this unit is built
            if (j + 1 < n_units) load_unit(pi, unit0 + j + 1, ru_next);
            if (j >= 2) {
                long long c0 = SC_CLK();
                ok = wait_all(&plan_free[pb], (uint32_t)(((j >> 1) & 1) ^ 1));
                w_done += SC_CLK() - c0;
                if (!ok) {
                    if (pt == 0) atomicExch(P.status, 307);
                    break;
                }
            }
            long long c2 = SC_CLK();
            build(unit0 + j, pb, ru);
            t_build += SC_CLK() - c2;
            ru = ru_next;
        }
        if (pt == 0) {
            SC_PROF_OUT(16, w_done);
            SC_PROF_OUT(17, t_build);
            SC_PROF_OUT(19, SC_CLK() - clk_start);
            for (int i = 0; i < 6; ++i) SC_PROF_OUT(32 + i, ph[i]);
        }
    } else if (warp == SC_MMA_WARP) {
        // ------------------------------------------------------------------ MMA issue
        ptx::reg_dec<SC_REGS_ISSUE>();
        if (lane == 0) {
            const uint32_t idesc = ptx::instr_desc_f16(MODE == TC_F16 ? 0 : 1, TILE_POS, N, 0, 0);
            bool ok = ptx::mbar_wait(a_full, 0);
            if (!ok) atomicExch(P.status, 302);
            ptx::tc_fence_after();
            // ring position and phase are stepped, never divided: a division by the run-time ring depth per stage
            // costs this single thread more than the stage's MMAs
            int s = 0, aq = 0;
            uint32_t b_phase = 0, t_phase = 1;
            const uint64_t b_desc0 = ptx::smem_desc_sw128(ptx::smem_u32(sB), 16, 1024);
            long long w_te = 0, w_bf = 0;
            SC_PROF_OUT(24, SC_CLK() - clk_start);
            for (int jp = 0; jp < n_pass && ok; ++jp) {
                long long c0 = SC_CLK();
                const bool got = ptx::mbar_wait_backoff<SC_SLEEP_NS>(&t_empty[aq], t_phase);
                w_te += SC_CLK() - c0;
                if (!got) {
                    atomicExch(P.status, 303);
                    ok = false;
                    break;
                }
                ptx::tc_fence_after();
                const uint32_t d_tmem = tmem_base + acc_col0 + (uint32_t)(aq * N);
                // f32 data: the hi and the lo part of a weight chunk are two stages of the ring; the first feeds
                // a_hi x b_hi and a_lo x b_hi, the second a_hi x b_lo
                for (int st = 0; st < RC * PARTS && ok; ++st) {
                    const int rc = st / PARTS, part = st % PARTS;
                    long long c1 = SC_CLK();
                    const bool gotb = ptx::mbar_wait(&b_full[s], b_phase);
                    w_bf += SC_CLK() - c1;
                    if (!gotb) {
                        atomicExch(P.status, 304);
                        ok = false;
                        break;
                    }
                    // no tcgen05 fence here: the stage was filled by TMA (async proxy, like the MMA's own reads) and
                    // the fence would wait for the MMAs in flight to drain, once per stage
                    // descriptor of the stage = descriptor of stage 0 + its byte distance / 16; one K = 16 step further
                    // is 32 bytes inside the swizzled rows (+ 2), 8 TMEM columns of A
                    const uint64_t b_desc = b_desc0 + (uint64_t)((uint32_t)s * (L.b_stage >> 4));
                    const uint32_t a_hi = tmem_base + (uint32_t)(rc * 32);
                    if (part == 0) {
                        if (rc == 0)
                            ptx::mma_f16_ts(d_tmem, a_hi, b_desc, idesc, 0u);
                        else
                            ptx::mma_f16_ts_acc(d_tmem, a_hi, b_desc, idesc);
                        if constexpr (SPLIT) ptx::mma_f16_ts_acc(d_tmem, a_hi + (uint32_t)a_cols, b_desc, idesc);
#pragma unroll
                        for (int k4 = 1; k4 < 4; ++k4) {
                            ptx::mma_f16_ts_acc(d_tmem, a_hi + (uint32_t)(k4 * 8), b_desc + (uint64_t)(2 * k4), idesc);
                            if constexpr (SPLIT)
                                ptx::mma_f16_ts_acc(d_tmem, a_hi + (uint32_t)(a_cols + k4 * 8), b_desc + (uint64_t)(2 * k4), idesc);
                        }
                    } else {
#pragma unroll
                        for (int k4 = 0; k4 < 4; ++k4)
                            ptx::mma_f16_ts_acc(d_tmem, a_hi + (uint32_t)(k4 * 8), b_desc + (uint64_t)(2 * k4), idesc);
                    }
                    ptx::mma_commit(&b_empty[s]);
                    if (++s == BS) {
                        s = 0;
                        b_phase ^= 1u;
                    }
                }
                if (ok) ptx::mma_commit(&t_full[aq]);
                if (++aq == NACC) {
                    aq = 0;
                    t_phase ^= 1u;
                }
            }
            SC_PROF_OUT(25, w_te);
            SC_PROF_OUT(26, w_bf);
            SC_PROF_OUT(27, SC_CLK() - clk_start);
        }
        __syncwarp();
    } else if (warp == SC_TMA_WARP) {
        // ------------------------------------------------------------------ TMA: weight ring
        ptx::reg_dec<SC_REGS_ISSUE>();
        if (lane == 0) {
            int s = 0, last_s = -1;
            uint32_t e_phase = 1, last_phase = 0;
            bool ok = true;
            for (int jp = 0; jp < n_pass && ok; ++jp) {
                const int unit = unit0 + (jp >> 1);
                const int chunk = unit / P.nbatch;
                const int t0 = (unit % P.nbatch) * TB;
                const int s0 = chunk * CHUNK_C + (jp & 1) * SC_SLAB;
                for (int st = 0; st < RC * PARTS; ++st) {
                    const int rc = st / PARTS, part = st % PARTS;
                    if (!ptx::mbar_wait_backoff<SC_SLEEP_NS>(&b_empty[s], e_phase)) {
                        atomicExch(P.status, 305);
                        ok = false;
                        break;
                    }
                    ptx::mbar_arrive_expect_tx(&b_full[s], L.b_stage);
                    ptx::tma_load_4d(sB + (size_t)s * L.b_stage, part == 0 ? &tmap_b_hi : &tmap_b_lo, &b_full[s], rc * 64, s0,
                                     t0, grp);
                    last_s = s;
                    last_phase = e_phase ^ 1u;
                    if (++s == BS) {
                        s = 0;
                        e_phase ^= 1u;
                    }
                }
                if (!ok) break;
            }
            // no copy may still be in flight when the CTA's shared memory is released
            if (last_s >= 0) ptx::mbar_wait(&b_full[last_s], last_phase);
        }
        __syncwarp();
    } else {
        ptx::reg_dec<SC_REGS_ISSUE>();   // the two idle warps of the last warpgroup
    }

    ptx::tc_fence_before();
    __syncthreads();
    if (warp == SC_MMA_WARP) ptx::tmem_dealloc(tmem_base, SC_TMEM_COLS);
    if (threadIdx.x == 0) SC_PROF_OUT(0, SC_CLK() - clk_start);
}

size_t dgrad_smem_bytes(int dim, int mode, int tb, int b_stages) {
    return 1024 + sc_layout(dim, mode, tb, b_stages).total;
}

template <int DIM, int MODE>
cudaError_t launch_dgrad_t(const DgradParams<DIM> &P, dim3 grid, const CUtensorMap *maps, cudaStream_t stream) {
    const size_t smem = dgrad_smem_bytes(DIM, MODE, P.tb, P.b_stages);
    const bool coord = P.goff != nullptr || P.gmask != nullptr;
    auto kern = coord ? dcn_dgrad_tc_kernel<DIM, MODE, true> : dcn_dgrad_tc_kernel<DIM, MODE, false>;
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

#ifdef TVDCN_B200_TUNING
// tuning builds only: copies the cycle counters of the profiled CTA to the host
extern "C" int tvdcn_b200_tuning_read_dgrad(long long *out, int n) {
    long long host[64];
    if (cudaDeviceSynchronize() != cudaSuccess) return -1;
    if (cudaMemcpyFromSymbol(host, g_dg_prof, sizeof(host)) != cudaSuccess) return -1;
    for (int i = 0; i < n && i < 64; ++i) out[i] = host[i];
    return 0;
}
#endif

}  // namespace tvdcn_b200
