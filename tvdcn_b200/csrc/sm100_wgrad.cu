// Tensor-core weight gradient with on-the-fly sampling (tcgen05 / TMEM).
//
//   gw[d, s', tap] += sum_{b, p} dense[b, d, p] * mask * sample(img[b, s], pos(b, og(s), tap, p))
//
// Replaces the second im2col + addmm_ of the reference's backward loop
// (tvdcn/csrc/ops/cuda/deform_conv2d_kernel.cpp:600-626): the sampled columns never reach global memory.
//
// GEMM view: D[dense channel d (M) x column k = (tap, channel) (N)] += A[d x pos] * B[pos x k], reduction
// over grid positions.  One CTA owns up to 2 x 128 dense channels and up to 4 x 64 columns (the whole
// accumulator lives in tensor memory, up to 512 columns) and walks a range of 64-position chunks:
//   A = dense^T tile [128 d][64 pos]: position-contiguous in the NCHW tensor, so it is a K-major operand
//       that TMA loads directly (zero-filled past the end of an image);
//   B = sampled tile [64 pos][64 channels] per column block, written by the producer warps in the same
//       swizzled row = position layout as the forward kernel and consumed as an MN-major operand.
// Position ranges are split over CTAs; partial results are added with 16-byte vector reductions to a staged f32
// copy of gw laid out [g][tap][d][s] (a thread holds 32 consecutive s of one d), which a small kernel then turns
// into the caller's [Cd, Cs / groups, taps] tensor.
//
// Warp roles (704 threads): warps 0-15 producers + epilogue, in two groups that take alternate stages so that
// one group's gathers are in flight while the other blends and stores; warp 16 MMA issue + TMEM owner;
// warp 17 TMA; warps 18-21 planners, which run ahead and turn coordinates into plan entries.
#include <algorithm>
#include <type_traits>

#include "plan.h"
#include "sm100_common.cuh"

namespace tvdcn_b200 {

template <int DIM>
struct WgradParams {
    Geo<DIM> g;
    const void *img_cl;
    const float *offset;
    const float *mask;
    float *gw;               // staged weight gradient [g][tap][d'][s'] f32, accumulated into
    int *status;
    int stages;
    int chunks_per_tap;      // csg / 64
    int n_sub;               // 64-column blocks per CTA
    int m_tiles;             // 128-dense-channel tiles per CTA
    int chunks_per_image;    // ceil(P / 64)
    int chunks_per_split;
    int total_chunks;        // B * chunks_per_image
};

namespace {

constexpr int WG_PRODUCER_WARPS = 16;
constexpr int WG_PRODUCERS = WG_PRODUCER_WARPS * 32;
constexpr int WG_GROUPS = 2;                     // producer groups; group q samples stages i with i % 2 == q
constexpr int WG_GROUP_WARPS = WG_PRODUCER_WARPS / WG_GROUPS;
constexpr int WG_GROUP_THREADS = WG_GROUP_WARPS * 32;
constexpr int WG_PLANNER_WARPS = 4;
constexpr int WG_PLANNERS = WG_PLANNER_WARPS * 32;
constexpr int WG_PLAN_BUFS = 3;
constexpr int WG_THREADS = WG_PRODUCERS + 64 + WG_PLANNERS;
constexpr int WG_POS = 64;                       // positions per stage
constexpr int WG_A_TILE = 128 * 128;             // [128 d][64 pos] 16-bit
constexpr int WG_B_TILE = WG_POS * 128;          // [64 pos][64 ch] 16-bit

template <int DIM, int MODE>
__global__ void __launch_bounds__(WG_THREADS, 1)
dcn_wgrad_tc_kernel(const WgradParams<DIM> P, const __grid_constant__ CUtensorMap tmap_hi,
                    const __grid_constant__ CUtensorMap tmap_lo) {
    constexpr int NC = 1 << DIM;
    constexpr bool SPLIT = MODE == TC_SPLIT;
    constexpr int PARTS = SPLIT ? 2 : 1;
    const Geo<DIM> &g = P.g;

    extern __shared__ uint8_t smem_raw[];
    // align by offset, not by integer round-trip, so that the compiler keeps these as shared-memory pointers
    uint8_t *smem = smem_raw + ((1024u - (ptx::smem_u32(smem_raw) & 1023u)) & 1023u);
    const int S = P.stages;
    const int NS = P.n_sub, MT = P.m_tiles;
    const uint32_t a_stage_bytes = (uint32_t)(MT * PARTS * WG_A_TILE);   // [m][part]
    const uint32_t b_part_bytes = (uint32_t)(NS * WG_B_TILE);            // [part][sub]
    const uint32_t b_stage_bytes = b_part_bytes * PARTS;
    uint8_t *sA = smem;
    uint8_t *sB = sA + (size_t)S * a_stage_bytes;
    PlanEntry *plan = reinterpret_cast<PlanEntry *>(sB + (size_t)S * b_stage_bytes);   // [bufs][NS * 64][NC]
    uint64_t *bars = reinterpret_cast<uint64_t *>(plan + WG_PLAN_BUFS * NS * NC * WG_POS);
    uint64_t *full_s = bars;           // sampled tiles written
    uint64_t *full_d = bars + S;       // dense tiles landed
    uint64_t *empty = bars + 2 * S;
    uint64_t *accum = bars + 3 * S;
    uint64_t *plan_full = bars + 3 * S + 1;
    uint64_t *plan_empty = plan_full + WG_PLAN_BUFS;
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(plan_empty + WG_PLAN_BUFS);
    __shared__ uint32_t chan16_s[4];

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int sub_total = g.K * P.chunks_per_tap;                 // 64-column blocks per group
    const int kt0 = blockIdx.x * NS;                              // first column block of this CTA
    const int y_tiles = (g.cdg + 128 * MT - 1) / (128 * MT);
    const int grp = blockIdx.y / y_tiles;
    const int d0 = (blockIdx.y % y_tiles) * 128 * MT;             // first dense channel within the group
    const int chunk_begin = blockIdx.z * P.chunks_per_split;
    const int chunk_end = min(chunk_begin + P.chunks_per_split, P.total_chunks);
    const int n_stages = max(chunk_end - chunk_begin, 0);
    const uint32_t cols_used = (uint32_t)(MT * NS * 64);
    uint32_t ncols = 32;
    while (ncols < cols_used) ncols <<= 1;
    constexpr uint32_t ESZ = SPLIT ? 4 : 2;
    // column blocks are ordered channel chunk outermost, tap innermost: the blocks of one CTA share an
    // image slab, which stays in L1
    auto sub_chan0 = [&](int sub) {
        const int kt = kt0 + sub;
        return grp * g.csg + (kt < sub_total ? kt / g.K : 0) * CHUNK_C;
    };

    if (threadIdx.x == 0) {
        for (int s = 0; s < S; ++s) {
            ptx::mbar_init(&full_s[s], WG_GROUP_WARPS);
            ptx::mbar_init(&full_d[s], 1);
            ptx::mbar_init(&empty[s], 1);
        }
        ptx::mbar_init(accum, 1);
        for (int b = 0; b < WG_PLAN_BUFS; ++b) {
            ptx::mbar_init(&plan_full[b], WG_PLANNER_WARPS);
            ptx::mbar_init(&plan_empty[b], WG_GROUP_WARPS);
        }
        ptx::fence_mbar_init();
    }
    if (threadIdx.x < 4) chan16_s[threadIdx.x] = (uint32_t)sub_chan0(min((int)threadIdx.x, NS - 1)) * ESZ / 16u;
    if (warp == WG_PRODUCER_WARPS + 1 && lane == 0) {
        ptx::prefetch_tmap(&tmap_hi);
        if (SPLIT) ptx::prefetch_tmap(&tmap_lo);
    }
    if (warp == WG_PRODUCER_WARPS) {
        ptx::tmem_alloc(tmem_slot, ncols);
        ptx::tmem_relinquish();
    }
    ptx::tc_fence_before();
    __syncthreads();
    ptx::tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp < WG_PRODUCER_WARPS) {
        // ------------------------------------------------------------------ producers
        const int pgroup = warp / WG_GROUP_WARPS;
        const int tg = threadIdx.x % WG_GROUP_THREADS;
        const uint4 *img16 = reinterpret_cast<const uint4 *>(P.img_cl);
        bool ok = true;
        for (int i = pgroup; i < n_stages; i += WG_GROUPS) {
            const int s = i % S, r = i / S;
            const int pb = i % WG_PLAN_BUFS;
            if (ok && !ptx::mbar_wait(&plan_full[pb], (uint32_t)((i / WG_PLAN_BUFS) & 1))) {
                atomicExch(P.status, 205);
                ok = false;
            }
            if (ok && !ptx::mbar_wait(&empty[s], (uint32_t)((r & 1) ^ 1))) {
                atomicExch(P.status, 201);
                ok = false;
            }
            ok = __all_sync(0xffffffffu, ok);  // keep the warp converged for the __syncwarp below
            if (!ok) break;
            uint8_t *b_hi = sB + (size_t)s * b_stage_bytes;
            produce_tiles<NC, MODE, WG_GROUP_THREADS>(b_hi, b_hi + b_part_bytes, WG_B_TILE, WG_POS, NS * WG_POS, img16,
                                                      chan16_s, plan + pb * NS * WG_POS * NC, tg);
            ptx::fence_proxy_async_smem();
            __syncwarp();
            if (lane == 0) {
                ptx::mbar_arrive(&full_s[s]);
                ptx::mbar_arrive(&plan_empty[pb]);
            }
        }

        // ------------------------------------------------------------------ epilogue: atomics into gw
        if (n_stages > 0) {
            if (ok && !ptx::mbar_wait(accum, 0)) {
                atomicExch(P.status, 202);
                ok = false;
            }
            ok = __all_sync(0xffffffffu, ok);  // tcgen05.ld is a whole-warp instruction
            ptx::tc_fence_after();
            if (ok) {
                const int lane_q = warp & 3;
                const uint32_t lane_base = tmem_base + ((uint32_t)(lane_q * 32) << 16);
                const int blocks = MT * NS * 2;  // 32-column blocks
                for (int cb = (warp >> 2); cb < blocks; cb += WG_PRODUCER_WARPS / 4) {
                    uint32_t v[32];
                    ptx::tmem_ld_32x32(lane_base + (uint32_t)(cb * 32), v);
                    ptx::tmem_ld_wait();
                    const int m = cb / (NS * 2);
                    const int col0 = (cb % (NS * 2)) * 32;      // column within the M tile
                    const int sub = col0 / 64;
                    const int kt = kt0 + sub;
                    const int dl = d0 + m * 128 + lane_q * 32 + lane;   // dense channel within the group
                    if (kt < sub_total && dl < g.cdg) {
                        const int tap = kt % g.K;
                        const int sl0 = (kt / g.K) * CHUNK_C + (col0 % 64);
                        // staged layout [g][tap][d'][s']: this thread's 32 values are 128 contiguous bytes, added
                        // with eight 16-byte reductions (the caller's [Cd, csg, K] layout would put every value in
                        // a sector of its own)
                        float *dst = P.gw + (((int64_t)grp * g.K + tap) * g.cdg + dl) * g.csg + sl0;
#pragma unroll
                        for (int e = 0; e < 32; e += 4)
                            asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(dst + e),
                                         "f"(__uint_as_float(v[e])), "f"(__uint_as_float(v[e + 1])),
                                         "f"(__uint_as_float(v[e + 2])), "f"(__uint_as_float(v[e + 3]))
                                         : "memory");
                    }
                }
            }
        }
    } else if (warp == WG_PRODUCER_WARPS) {
        // ------------------------------------------------------------------ MMA issue
        if (lane == 0) {
            const uint32_t idesc = ptx::instr_desc_f16(MODE == TC_F16 ? 0 : 1, 128, NS * 64, 0, 1);
            bool ok = true;
            // ring position and phase are stepped and the stage's descriptors derived from those of stage 0 by an
            // addition: bookkeeping must stay cheap next to the MMAs this single thread issues
            const uint64_t a_desc0 = ptx::smem_desc_sw128(ptx::smem_u32(sA), 16, 1024);
            const uint64_t b_desc0 = ptx::smem_desc_sw128(ptx::smem_u32(sB), WG_B_TILE, 1024);
            int s = 0;
            uint32_t phase = 0;
            for (int i = 0; i < n_stages && ok; ++i) {
                if (!ptx::mbar_wait(&full_s[s], phase) || !ptx::mbar_wait(&full_d[s], phase)) {
                    atomicExch(P.status, 203);
                    ok = false;
                    break;
                }
                ptx::tc_fence_after();
                const uint64_t a_st = a_desc0 + (uint64_t)((uint32_t)s * (a_stage_bytes >> 4));
                const uint64_t b_hi0 = b_desc0 + (uint64_t)((uint32_t)s * (b_stage_bytes >> 4));
                for (int m = 0; m < MT; ++m) {
                    const uint32_t d_tmem = tmem_base + (uint32_t)(m * NS * 64);
                    const uint64_t am = a_st + (uint64_t)((uint32_t)(m * PARTS) * (WG_A_TILE >> 4));
#pragma unroll
                    for (int k4 = 0; k4 < 4; ++k4) {
                        // A: K-major rows of 64 positions (32 bytes per K step); B: MN-major, 16 positions = 16 rows
                        // of 128 bytes (2048 bytes per K step)
                        const uint64_t a_hi = am + 2 * k4;
                        const uint64_t b_hi = b_hi0 + 128 * k4;
                        ptx::mma_f16(d_tmem, a_hi, b_hi, idesc, (i > 0 || k4 > 0) ? 1u : 0u);
                        if constexpr (SPLIT) {
                            ptx::mma_f16(d_tmem, a_hi + (WG_A_TILE >> 4), b_hi, idesc, 1u);
                            ptx::mma_f16(d_tmem, a_hi, b_hi + (b_part_bytes >> 4), idesc, 1u);
                        }
                    }
                }
                ptx::mma_commit(&empty[s]);
                if (++s == S) {
                    s = 0;
                    phase ^= 1u;
                }
            }
            if (ok && n_stages > 0) ptx::mma_commit(accum);
        }
        __syncwarp();
    } else if (warp == WG_PRODUCER_WARPS + 1) {
        // ------------------------------------------------------------------ TMA: dense tiles
        if (lane == 0) {
            int issued = 0;
            for (int i = 0; i < n_stages; ++i) {
                const int s = i % S, r = i / S;
                if (!ptx::mbar_wait(&empty[s], (uint32_t)((r & 1) ^ 1))) {
                    atomicExch(P.status, 204);
                    break;
                }
                const int pc = chunk_begin + i;
                const int b = pc / P.chunks_per_image;
                const int p0 = (pc % P.chunks_per_image) * WG_POS;
                uint8_t *a_dst = sA + (size_t)s * a_stage_bytes;
                ptx::mbar_arrive_expect_tx(&full_d[s], a_stage_bytes);
                for (int m = 0; m < MT; ++m) {
                    const int dch = grp * g.cdg + d0 + m * 128;
                    ptx::tma_load_3d(a_dst + (size_t)(m * PARTS) * WG_A_TILE, &tmap_hi, &full_d[s], p0, dch, b);
                    if (SPLIT)
                        ptx::tma_load_3d(a_dst + (size_t)(m * PARTS + 1) * WG_A_TILE, &tmap_lo, &full_d[s], p0, dch, b);
                }
                issued = i + 1;
            }
            // never leave with a copy still in flight into this CTA's shared memory
            if (issued > 0) {
                const int i = issued - 1;
                ptx::mbar_wait(&full_d[i % S], (uint32_t)((i / S) & 1));
            }
        }
        __syncwarp();
    } else {
        // ------------------------------------------------------------------ planners
        // entry e = (column block e / 64, position slot e % 64) of a stage; each thread fills up to two entries
        constexpr int EPT = 4 * WG_POS / WG_PLANNERS;
        const int t = threadIdx.x - (WG_PRODUCERS + 64);
        const bool deformable = P.offset != nullptr;
        const uint32_t row_scale = (uint32_t)g.Cs * ESZ / 16u;
        int e_tap[EPT], e_og[EPT], e_mg[EPT];
        bool e_on[EPT], e_ok[EPT];
#pragma unroll
        for (int k = 0; k < EPT; ++k) {
            const int sub = (t + k * WG_PLANNERS) / WG_POS;
            const int kt = kt0 + sub;
            e_on[k] = sub < NS;
            e_ok[k] = e_on[k] && kt < sub_total;
            e_tap[k] = e_ok[k] ? kt % g.K : 0;
            const int chan0 = sub_chan0(sub);
            e_og[k] = g.og > 0 ? chan0 / g.cs_per_og : 0;
            e_mg[k] = g.mg > 0 ? chan0 / g.cs_per_mg : 0;
        }
        const int slot = t % WG_POS;
        // offsets / mask of stage i + 2 are requested while stage i is planned, so that their latency stays off
        // the critical path
        struct StageCoords {
            PosInfo<DIM> pi[EPT];
            RawCoords<DIM> rc[EPT];
        };
        auto fetch = [&](int i, StageCoords &sc) {
            const int pc = chunk_begin + i;
            const int p = (pc % P.chunks_per_image) * WG_POS + slot;
#pragma unroll
            for (int k = 0; k < EPT; ++k) {
                sc.pi[k].valid = e_ok[k] && p < g.P;
                sc.pi[k].b = pc / P.chunks_per_image;
                sc.pi[k].p = sc.pi[k].valid ? p : 0;
                decode_in_image<DIM>(g, sc.pi[k]);
                if (e_on[k]) sc.rc[k] = load_coords<DIM>(g, sc.pi[k], P.offset, P.mask, e_tap[k], e_og[k], e_mg[k]);
            }
        };
        StageCoords c0, c1, c2;
        if (n_stages > 0) fetch(0, c0);
        if (n_stages > 1) fetch(1, c1);
        for (int i = 0; i < n_stages; ++i) {
            const int pb = i % WG_PLAN_BUFS;
            if (i + 2 < n_stages) fetch(i + 2, c2);
            const StageCoords cur = c0;
            c0 = c1;
            c1 = c2;
            bool ok = ptx::mbar_wait(&plan_empty[pb], (uint32_t)(((i / WG_PLAN_BUFS) & 1) ^ 1));
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) {
                if (lane == 0) atomicExch(P.status, 206);
                break;
            }
#pragma unroll
            for (int k = 0; k < EPT; ++k) {
                if (e_on[k])
                    build_plan<DIM, MODE>(g, cur.pi[k], cur.rc[k], deformable, e_tap[k], row_scale,
                                          plan + ((pb * NS) * WG_POS + t + k * WG_PLANNERS) * NC);
            }
            __syncwarp();
            if (lane == 0) ptx::mbar_arrive(&plan_full[pb]);
        }
    }

    ptx::tc_fence_before();
    __syncthreads();
    if (warp == WG_PRODUCER_WARPS) ptx::tmem_dealloc(tmem_base, ncols);
}

size_t wgrad_smem_bytes(int dim, int mode, int n_sub, int m_tiles, int stages) {
    const int parts = mode == TC_SPLIT ? 2 : 1;
    const size_t stage = (size_t)parts * (m_tiles * WG_A_TILE + n_sub * WG_B_TILE);
    const size_t plan = (size_t)WG_PLAN_BUFS * n_sub * (1 << dim) * WG_POS * 8;
    return 1024 + stages * stage + plan + (3 * stages + 1 + 2 * WG_PLAN_BUFS) * 8 + 16;
}

template <int DIM, int MODE>
cudaError_t launch_wgrad_t(const WgradParams<DIM> &P, dim3 grid, const CUtensorMap &hi, const CUtensorMap &lo,
                           cudaStream_t stream) {
    const size_t smem = wgrad_smem_bytes(DIM, MODE, P.n_sub, P.m_tiles, P.stages);
    auto kern = dcn_wgrad_tc_kernel<DIM, MODE>;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return e;
    LaunchScope scope("dcn_wgrad_tc", stream);
    kern<<<grid, WG_THREADS, smem, stream>>>(P, hi, lo);
    return cudaGetLastError();
}

}  // namespace

// Tile shape and pipeline depth; false when the shape is not covered.
bool wgrad_tc_config(int dim, int mode, int cdg, int P, int *n_sub, int *m_tiles, int *stages) {
    if (P % 8 != 0) return false;  // the dense tensor's row pitch must be a multiple of 16 bytes for TMA
    const int mt = cdg > 128 ? 2 : 1;
    int ns = mode == TC_SPLIT ? 2 : 4;
    if (dim == 3 && mode != TC_SPLIT) ns = 4;
    int s = 0;
    static const int max_stages = tuning_int("TVDCN_B200_WG_STAGES", 2);
    for (int cand = max_stages; cand >= 2; --cand)
        if (wgrad_smem_bytes(dim, mode, ns, mt, cand) <= 227 * 1024) { s = cand; break; }
    if (s == 0) return false;
    *n_sub = ns;
    *m_tiles = mt;
    *stages = s;
    return true;
}

// dense_hi / dense_lo: the dense tensor [B, Cd, P] as 16-bit (the tensor itself for 16-bit data; bf16 hi
// and lo parts of the f32 tensor in split mode).  gw must be zero-initialised f32.
cudaError_t launch_sample_wgrad_tc(const GeoHost &h, int mode, const void *dense_hi, const void *dense_lo,
                                   const void *img_cl, const float *offset, const float *mask, float *gw,
                                   int *status, cudaStream_t stream) {
    const int cdg = h.Cd / h.groups, csg = h.Cs / h.groups;
    int ns = 0, mt = 0, st = 0;
    if (!wgrad_tc_config(h.dim, mode, cdg, h.P, &ns, &mt, &st)) return cudaErrorInvalidConfiguration;
    CUtensorMap hi, lo;
    const uint64_t dims[3] = {(uint64_t)h.P, (uint64_t)h.Cd, (uint64_t)h.B};
    const uint64_t strides[2] = {(uint64_t)h.P * 2, (uint64_t)h.P * h.Cd * 2};
    const uint32_t box[3] = {WG_POS, 128, 1};
    if (!make_tensor_map_16bit(&hi, dense_hi, 3, dims, strides, box)) return cudaErrorInvalidValue;
    if (mode == TC_SPLIT) {
        if (!make_tensor_map_16bit(&lo, dense_lo, 3, dims, strides, box)) return cudaErrorInvalidValue;
    } else {
        lo = hi;
    }
    const int sub_total = h.K * (csg / CHUNK_C);
    const int k_tiles = (sub_total + ns - 1) / ns;
    const int y_tiles = h.groups * ((cdg + 128 * mt - 1) / (128 * mt));
    const int cpi = (h.P + WG_POS - 1) / WG_POS;
    const int total = h.B * cpi;
    const int per_wave = std::max(1, 148 / std::max(1, k_tiles * y_tiles));
    int splits = per_wave;
    if (mode == TC_SPLIT) {
        // The tensor core's f32 accumulation rounds toward zero, so the error of one accumulator grows linearly
        // with the number of MMAs added into it (measured: ~4e-8 of the result per MMA).  f32 data promises
        // 1e-4: keep one CTA's chain at 56 stages (672 MMAs) by using more waves of CTAs; the partial sums
        // meet in grad_weight through round-to-nearest f32 atomics.
        const int max_stages = 56;
        int waves = 1;
        while ((total + waves * per_wave - 1) / (waves * per_wave) > max_stages) ++waves;
        splits = waves * per_wave;
    }
    splits = std::min(splits, total);
    const int per = (total + splits - 1) / splits;
    splits = (total + per - 1) / per;
    dim3 grid((unsigned)k_tiles, (unsigned)y_tiles, (unsigned)splits);
    auto run = [&](auto dimc) -> cudaError_t {
        constexpr int DIM = decltype(dimc)::value;
        WgradParams<DIM> P;
        P.g = geo_from_host<DIM>(h);
        P.img_cl = img_cl;
        P.offset = offset;
        P.mask = mask;
        P.gw = gw;
        P.status = status;
        P.stages = st;
        P.chunks_per_tap = csg / CHUNK_C;
        P.n_sub = ns;
        P.m_tiles = mt;
        P.chunks_per_image = cpi;
        P.chunks_per_split = per;
        P.total_chunks = total;
        if (mode == TC_BF16) return launch_wgrad_t<DIM, TC_BF16>(P, grid, hi, lo, stream);
        if (mode == TC_F16) return launch_wgrad_t<DIM, TC_F16>(P, grid, hi, lo, stream);
        return launch_wgrad_t<DIM, TC_SPLIT>(P, grid, hi, lo, stream);
    };
    if (h.dim == 1) return run(std::integral_constant<int, 1>());
    if (h.dim == 2) return run(std::integral_constant<int, 2>());
    if (h.dim == 3) return run(std::integral_constant<int, 3>());
    return cudaErrorInvalidValue;
}

namespace {
// staged [g][tap][d'][s'] f32 -> the caller's [Cd, csg, K] in its data type
template <typename TO>
__global__ void __launch_bounds__(256) unpack_weight_grad_kernel(const float *__restrict__ staged, TO *__restrict__ gw,
                                                                 int groups, int cdg, int csg, int K) {
    // one block per (dense channel, 64 sampled channels): reads K rows of 64 floats, writes 64 * K contiguous values
    extern __shared__ float tile[];   // [K][65]
    const int d = blockIdx.x;                // grp * cdg + dl
    const int grp = d / cdg, dl = d % cdg;
    const int s0 = blockIdx.y * 64;
    for (int i = threadIdx.x; i < K * 64; i += blockDim.x) {
        const int tap = i / 64, sl = i % 64;
        tile[tap * 65 + sl] = s0 + sl < csg ? staged[(((int64_t)grp * K + tap) * cdg + dl) * csg + s0 + sl] : 0.f;
    }
    __syncthreads();
    TO *out = gw + ((int64_t)d * csg + s0) * K;
    const int n = min(64, csg - s0) * K;
    for (int i = threadIdx.x; i < n; i += blockDim.x) store_acc(out, i, tile[(i % K) * 65 + i / K]);
}
}  // namespace

cudaError_t launch_unpack_weight_grad(const float *staged, void *gw, int dtype, int groups, int cdg, int csg, int K,
                                      cudaStream_t stream) {
    dim3 grid((unsigned)(groups * cdg), (unsigned)((csg + 63) / 64));
    const size_t smem = (size_t)K * 65 * sizeof(float);
    auto run = [&](auto kern, auto *out) -> cudaError_t {
        if (smem > 48 * 1024) {   // many taps: the tile needs the opt-in shared memory size
            cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
            if (e != cudaSuccess) return e;
        }
        LaunchScope scope("unpack_weight_grad", stream);
        kern<<<grid, 256, smem, stream>>>(staged, out, groups, cdg, csg, K);
        return cudaGetLastError();
    };
    if (dtype == DT_F32) return run(unpack_weight_grad_kernel<float>, (float *)gw);
    if (dtype == DT_BF16) return run(unpack_weight_grad_kernel<__nv_bfloat16>, (__nv_bfloat16 *)gw);
    if (dtype == DT_F16) return run(unpack_weight_grad_kernel<__half>, (__half *)gw);
    return cudaErrorInvalidValue;
}

}  // namespace tvdcn_b200
