// Tensor-core "sample -> GEMM" kernel (tcgen05 / TMEM), plus the layout staging kernels it needs.
//
//   dense[b, d, p] = bias[d] + sum_{tap, s'} W[d, s', tap] * mask * sample(img[b, s], pos(b, og(s), tap, p))
//
// It is an implicit GEMM  D[128 positions x BN dense channels] += A[128 x 64] * B[BN x 64]^T  over K chunks
// of 64 channels of one kernel tap.  The A tile (the im2col columns of the reference,
// tvdcn/csrc/ops/cuda/deform_conv2d_common_kernels.cu:138-192) is never written to global memory: sixteen
// producer warps sample a channels-last copy of the image straight into the 128-byte-swizzled shared
// memory layout the tensor core reads.  The B tile (weights packed per tap) arrives by TMA.  One thread
// issues tcgen05.mma with the accumulator in tensor memory; the producer warps then read it back
// (tcgen05.ld: lane = position) and store NCHW with the bias added, so the reference's output_buf
// transpose and bias pass (tvdcn/csrc/ops/cuda/deform_conv2d_kernel.cpp:371-380) are gone too.
//
// Warp roles (768 threads): warps 0-15 producers + epilogue, warps 16-19 planners, warp 20 MMA issue + TMEM owner,
// warp 21 TMA, warps 22-23 idle.  The planners turn sampling coordinates into plan entries a few chunks ahead.
#include <algorithm>
#include <cstdio>
#include <cstdlib>
#include <type_traits>

#include "plan.h"
#include "sm100_common.cuh"

namespace tvdcn_b200 {

template <int DIM>
struct FwdParams {
    Geo<DIM> g;
    const void *img_cl;     // [B, S, Cs] 16-bit (TC_BF16 / TC_F16) or f32 (TC_SPLIT)
    const float *offset;    // may be null
    const float *mask;      // may be null
    const float *bias;      // may be null
    void *out;              // [B, Cd, P], data type of the problem
    int *status;            // device status word (0 = ok)
    int bn;                 // dense channels per tile: 64, 128 or 256
    int stages;
    int chunks_per_tap;     // csg / 64
    int prefetch;           // planners also issue L1 prefetches of the corner rows
};

namespace {

constexpr int PRODUCER_WARPS = 16;
constexpr int PRODUCERS = PRODUCER_WARPS * 32;
// Producer groups: group q samples chunks j with j % groups == q.  Two groups for 16-bit data (three stages: one
// group's gathers are in flight while the other blends); one group of all 16 warps for f32 data, whose two stages
// would otherwise make each group wait for the MMA of its own previous chunk.
__host__ __device__ constexpr int producer_groups_of(int mode) {
#ifdef TVDCN_FWD_GROUPS_16
    return mode == TC_SPLIT ? 1 : TVDCN_FWD_GROUPS_16;
#else
    return mode == TC_SPLIT ? 1 : 2;
#endif
}
constexpr int PLANNER_WARPS = 4;                  // one planner thread per tile position
constexpr int PLAN_BUFS = 4;
// Warps: 0-15 producers (four warpgroups), 16-19 planners, 20 MMA, 21 TMA, 22-23 idle (they complete the last
// warpgroup).  The warpgroups re-divide the registers at kernel start (launch: 80 each, 6 x 80 = 480): the
// producers, who keep the gathers of several positions in flight, take FWD_REGS_PRODUCER, the planners and the
// MMA / TMA warpgroup give up what that costs: 4 x 104 + 40 + 24 = 480.
constexpr int MMA_WARP = PRODUCER_WARPS + PLANNER_WARPS;
constexpr int TMA_WARP = MMA_WARP + 1;
constexpr int FWD_THREADS = (TMA_WARP + 3) * 32;
static_assert(FWD_THREADS == 768, "six warpgroups");
constexpr int FWD_REGS_PRODUCER = 104, FWD_REGS_PLANNER = 40, FWD_REGS_ISSUE = 24;
#ifndef TVDCN_FWD_IB
#define TVDCN_FWD_IB 4
#endif
constexpr int FWD_MAX_TAPS = 512;                 // taps whose kernel coordinates a CTA tabulates (more: SIMT kernels)

template <int DIM, int MODE>
__global__ void __launch_bounds__(FWD_THREADS, 1)
dcn_fwd_tc_kernel(const FwdParams<DIM> P, const __grid_constant__ CUtensorMap tmap_hi,
                  const __grid_constant__ CUtensorMap tmap_lo) {
    constexpr int NC = 1 << DIM;
    constexpr bool SPLIT = MODE == TC_SPLIT;
    constexpr int PARTS = SPLIT ? 2 : 1;
    constexpr int PGROUPS = producer_groups_of(MODE);
    constexpr int GROUP_WARPS = PRODUCER_WARPS / PGROUPS;
    constexpr int GROUP_THREADS = GROUP_WARPS * 32;
    using T16 = typename std::conditional<MODE == TC_F16, __half, __nv_bfloat16>::type;
    const Geo<DIM> &g = P.g;

    extern __shared__ uint8_t smem_raw[];
    // align by offset, not by integer round-trip, so that the compiler keeps these as shared-memory pointers
    uint8_t *smem = smem_raw + ((1024u - (ptx::smem_u32(smem_raw) & 1023u)) & 1023u);
    const int S = P.stages;
    const int BN = P.bn;
    const uint32_t a_stage_bytes = A_TILE_BYTES * PARTS;
    const uint32_t b_part_bytes = (uint32_t)BN * 128u;
    const uint32_t b_stage_bytes = b_part_bytes * PARTS;
    uint8_t *sA = smem;
    uint8_t *sB = sA + (size_t)S * a_stage_bytes;
    PlanEntry *plan = reinterpret_cast<PlanEntry *>(sB + (size_t)S * b_stage_bytes);  // [PLAN_BUFS][128][NC]
    uint64_t *bars = reinterpret_cast<uint64_t *>(plan + PLAN_BUFS * NC * TILE_POS);
    uint64_t *full_a = bars;
    uint64_t *full_b = bars + S;
    uint64_t *empty = bars + 2 * S;
    uint64_t *accum = bars + 3 * S;
    uint64_t *plan_full = bars + 3 * S + 1;
    uint64_t *plan_empty = plan_full + PLAN_BUFS;
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(plan_empty + PLAN_BUFS);

    // kernel coordinates of every tap, so that the planners do not divide by the kernel extents per chunk
    __shared__ int16_t tap_tab[FWD_MAX_TAPS * DIM];
    for (int tp = threadIdx.x; tp < g.K; tp += FWD_THREADS) {
        int tc[DIM];
        tap_coords<DIM>(g, tp, tc);
#pragma unroll
        for (int a = 0; a < DIM; ++a) tap_tab[tp * DIM + a] = (int16_t)tc[a];
    }
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int tiles_n = g.cdg / BN;
    const int grp = blockIdx.y / tiles_n;
    const int n0 = (blockIdx.y % tiles_n) * BN;
    const long long m0 = (long long)blockIdx.x * TILE_POS;
    const int n_chunks = g.K * P.chunks_per_tap;
    // f32 data: the tensor core's f32 accumulation rounds toward zero, so the error of one accumulator grows
    // with the number of MMAs added into it.  Chunks go round-robin into NACC accumulators, which the epilogue
    // adds (round to nearest); this divides the chain length by NACC.
    // As many accumulators as keep one chain near 250 MMAs (12 per chunk), at most 4 and what 512 columns hold.
    int NACC = 1;
    if (SPLIT) {
        NACC = min(min(4, 512 / BN), (n_chunks * 12 + 249) / 250);
        NACC = NACC == 3 ? 2 : max(NACC, 1);          // the column count must be a power of two
    }
    const uint32_t ncols = (uint32_t)(NACC * BN) < 32u ? 32u : (uint32_t)(NACC * BN);

    if (threadIdx.x == 0) {
        for (int s = 0; s < S; ++s) {
            ptx::mbar_init(&full_a[s], GROUP_WARPS);
            ptx::mbar_init(&full_b[s], 1);
            ptx::mbar_init(&empty[s], 1);
        }
        ptx::mbar_init(accum, 1);
        for (int b = 0; b < PLAN_BUFS; ++b) {
            ptx::mbar_init(&plan_full[b], PLANNER_WARPS);
            ptx::mbar_init(&plan_empty[b], GROUP_WARPS);
        }
        ptx::fence_mbar_init();
    }
    if (warp == TMA_WARP && lane == 0) {
        ptx::prefetch_tmap(&tmap_hi);
        if (SPLIT) ptx::prefetch_tmap(&tmap_lo);
    }
    if (warp == MMA_WARP) {
        ptx::tmem_alloc(tmem_slot, ncols);
        ptx::tmem_relinquish();
    }
    ptx::tc_fence_before();
    __syncthreads();
    ptx::tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    constexpr uint32_t ESZ = SPLIT ? 4 : 2;
    const uint4 *img16 = reinterpret_cast<const uint4 *>(P.img_cl);
    // chunk j -> (tap, first channel): channel chunk outermost, so the taps of one 64-channel chunk sample the
    // same slab of the image, which then stays in L1 for all of them
    auto chunk_tap = [&](int j) { return j % g.K; };
    auto chunk_chan0 = [&](int j) { return grp * g.csg + (j / g.K) * CHUNK_C; };

    if (warp < PRODUCER_WARPS) {
        // ------------------------------------------------------------------ producers
        ptx::reg_inc<FWD_REGS_PRODUCER>();
        const int t = threadIdx.x;
        // position this thread stores in the epilogue (TMEM lane of its warp)
        const PosInfo<DIM> pi = decode_position<DIM>(g, m0 + (warp & 3) * 32 + lane);
        bool ok = true;
        // Two groups of producer warps take alternate chunks, so that one group's loads are in flight while the
        // other blends and stores: the load/store pipe stays busy instead of idling between phases.
        const int pgroup = warp / GROUP_WARPS;
        const int tg = t % GROUP_THREADS;
        for (int j = pgroup; j < n_chunks; j += PGROUPS) {
            const int s = j % S, r = j / S;
            const int pbuf = j % PLAN_BUFS;
            if (ok && !ptx::mbar_wait(&plan_full[pbuf], (uint32_t)((j / PLAN_BUFS) & 1))) {
                atomicExch(P.status, 105);
                ok = false;
            }
            if (ok && !ptx::mbar_wait(&empty[s], (uint32_t)((r & 1) ^ 1))) {
                atomicExch(P.status, 101);
                ok = false;
            }
            ok = __all_sync(0xffffffffu, ok);  // keep the warp converged for the __syncwarp below
            if (!ok) break;
            uint8_t *a_hi = sA + (size_t)s * a_stage_bytes;
            const uint32_t c16 = (uint32_t)chunk_chan0(j) * ESZ / 16u;
            produce_tiles<NC, MODE, GROUP_THREADS, (NC >= 8 ? 2 : TVDCN_FWD_IB)>(a_hi, a_hi + A_TILE_BYTES, 0u, TILE_POS, TILE_POS, img16, &c16,
                                                   plan + pbuf * TILE_POS * NC, tg);
            ptx::fence_proxy_async_smem();
            __syncwarp();
            if (lane == 0) {
                ptx::mbar_arrive(&full_a[s]);
                ptx::mbar_arrive(&plan_empty[pbuf]);
            }
        }

        // ------------------------------------------------------------------ epilogue
        if (ok && !ptx::mbar_wait(accum, 0)) {
            atomicExch(P.status, 102);
            ok = false;
        }
        ok = __all_sync(0xffffffffu, ok);  // tcgen05.ld is a whole-warp instruction
        ptx::tc_fence_after();
        if (ok) {
            // warps w, w + 4, w + 8, ... share TMEM lanes 32 * (w % 4) ...; they split the columns
            const uint32_t lane_base = tmem_base + ((uint32_t)((warp & 3) * 32) << 16);
            const int blocks = BN / 32;
            for (int cb = (warp >> 2); cb < blocks; cb += PRODUCER_WARPS / 4) {
                uint32_t v[32];
                ptx::tmem_ld_32x32(lane_base + (uint32_t)(cb * 32), v);
                ptx::tmem_ld_wait();
                for (int a = 1; a < NACC && a < n_chunks; ++a) {
                    uint32_t u[32];
                    ptx::tmem_ld_32x32(lane_base + (uint32_t)(a * BN + cb * 32), u);
                    ptx::tmem_ld_wait();
#pragma unroll
                    for (int e = 0; e < 32; ++e) v[e] = __float_as_uint(__uint_as_float(v[e]) + __uint_as_float(u[e]));
                }
                if (pi.valid) {
#pragma unroll
                    for (int e = 0; e < 32; ++e) {
                        const int d = grp * g.cdg + n0 + cb * 32 + e;
                        float val = __uint_as_float(v[e]);
                        if (P.bias != nullptr) val += __ldg(P.bias + d);
                        const int64_t o = ((int64_t)pi.b * g.Cd + d) * (int64_t)g.P + pi.p;
                        if constexpr (SPLIT)
                            reinterpret_cast<float *>(P.out)[o] = val;
                        else
                            store_acc(reinterpret_cast<T16 *>(P.out), o, val);
                    }
                }
            }
        }
    } else if (warp == MMA_WARP) {
        // ------------------------------------------------------------------ MMA issue
        ptx::reg_dec<FWD_REGS_ISSUE>();
        if (lane == 0) {
            const uint32_t idesc = ptx::instr_desc_f16(MODE == TC_F16 ? 0 : 1, TILE_POS, BN, 0, 0);
            bool ok = true;
            // ring position, phase and accumulator are stepped, and the descriptors of a stage derived from those of
            // stage 0 by an addition: this single thread must not spend longer on bookkeeping than on issuing MMAs
            const uint64_t a_desc0 = ptx::smem_desc_sw128(ptx::smem_u32(sA), 16, 1024);
            const uint64_t b_desc0 = ptx::smem_desc_sw128(ptx::smem_u32(sB), 16, 1024);
            int s = 0, acc_i = 0;
            uint32_t phase = 0;
            for (int j = 0; j < n_chunks && ok; ++j) {
                const bool got_b = ptx::mbar_wait(&full_a[s], phase) && ptx::mbar_wait(&full_b[s], phase);
                if (!got_b) {
                    atomicExch(P.status, 103);
                    ok = false;
                    break;
                }
                ptx::tc_fence_after();
                const uint64_t a_hi = a_desc0 + (uint64_t)((uint32_t)s * (a_stage_bytes >> 4));
                const uint64_t b_hi = b_desc0 + (uint64_t)((uint32_t)s * (b_stage_bytes >> 4));
                const uint32_t d_tmem = tmem_base + (uint32_t)(acc_i * BN);
#pragma unroll
                for (int k4 = 0; k4 < 4; ++k4) {
                    ptx::mma_f16(d_tmem, a_hi + 2 * k4, b_hi + 2 * k4, idesc, (j >= NACC || k4 > 0) ? 1u : 0u);
                    if constexpr (SPLIT) {
                        ptx::mma_f16(d_tmem, a_hi + (A_TILE_BYTES >> 4) + 2 * k4, b_hi + 2 * k4, idesc, 1u);
                        ptx::mma_f16(d_tmem, a_hi + 2 * k4, b_hi + (b_part_bytes >> 4) + 2 * k4, idesc, 1u);
                    }
                }
                ptx::mma_commit(&empty[s]);
                if (++s == S) {
                    s = 0;
                    phase ^= 1u;
                }
                if (++acc_i == NACC) acc_i = 0;
            }
            if (ok) ptx::mma_commit(accum);
        }
        __syncwarp();
    } else if (warp == TMA_WARP) {
        // ------------------------------------------------------------------ TMA: weight tiles
        ptx::reg_dec<FWD_REGS_ISSUE>();
        if (lane == 0) {
            int s = 0, tap = 0, cc = 0, last_s = -1;
            uint32_t e_phase = 1, last_phase = 0;
            for (int j = 0; j < n_chunks; ++j) {
                if (!ptx::mbar_wait(&empty[s], e_phase)) {
                    atomicExch(P.status, 104);
                    break;
                }
                uint8_t *b_dst = sB + (size_t)s * b_stage_bytes;
                ptx::mbar_arrive_expect_tx(&full_b[s], b_stage_bytes);
                ptx::tma_load_4d(b_dst, &tmap_hi, &full_b[s], cc * CHUNK_C, n0, tap, grp);
                if (SPLIT) ptx::tma_load_4d(b_dst + b_part_bytes, &tmap_lo, &full_b[s], cc * CHUNK_C, n0, tap, grp);
                last_s = s;
                last_phase = e_phase ^ 1u;
                if (++s == S) {
                    s = 0;
                    e_phase ^= 1u;
                }
                if (++tap == g.K) {   // chunk j -> (tap j % K, channel chunk j / K)
                    tap = 0;
                    ++cc;
                }
            }
            // never leave with a copy still in flight into this CTA's shared memory
            if (last_s >= 0) ptx::mbar_wait(&full_b[last_s], last_phase);
        }
        __syncwarp();
    }

    if (warp > TMA_WARP) ptx::reg_dec<FWD_REGS_ISSUE>();   // the two idle warps of the last warpgroup

    if (warp >= PRODUCER_WARPS && warp < MMA_WARP) {
        // ------------------------------------------------------------------ planners: one thread per position
        ptx::reg_dec<FWD_REGS_PLANNER>();
        // run ahead of the producers: coordinates -> plan entries, and an L1 prefetch of every corner row so
        // that the producers' gathers hit L1
        const int t = threadIdx.x - PRODUCERS;
        const PosInfo<DIM> pi = decode_position<DIM>(g, m0 + t);
        const bool deformable = P.offset != nullptr;
        const uint32_t row_scale = (uint32_t)g.Cs * ESZ / 16u;
        // offsets / mask of chunk j + 2 are requested while chunk j is planned: their latency stays off the
        // critical path (one planner thread has nothing else in flight)
        // this thread's position is fixed: its offset / mask addresses differ per chunk by a multiple of P only
        const float *off_base = (P.offset != nullptr && pi.valid)
                                    ? P.offset + (int64_t)pi.b * g.og * g.K * DIM * (int64_t)g.P + pi.p : nullptr;
        const float *mask_base = (P.mask != nullptr && pi.valid)
                                     ? P.mask + (int64_t)pi.b * g.mg * g.K * (int64_t)g.P + pi.p : nullptr;
        // (tap, channel chunk) of the chunk being planned and of the chunk whose coordinates are being requested,
        // advanced by counting: a planner thread runs one dependent instruction chain, so every division in it
        // costs the whole CTA
        struct Cursor {
            int tap, cc, ogi, mgi;
        };
        auto settle = [&](Cursor &c) {
            const int chan0 = grp * g.csg + c.cc * CHUNK_C;
            c.ogi = g.og > 0 ? chan0 / g.cs_per_og : 0;
            c.mgi = g.mg > 0 ? chan0 / g.cs_per_mg : 0;
        };
        auto advance = [&](Cursor &c) {
            if (++c.tap == g.K) {
                c.tap = 0;
                ++c.cc;
                settle(c);
            }
        };
        Cursor cur_c{0, 0, 0, 0}, fetch_c{0, 0, 0, 0};
        settle(cur_c);
        settle(fetch_c);
        auto coords_at = [&](const Cursor &c) {
            RawCoords<DIM> rc;
#pragma unroll
            for (int a = 0; a < DIM; ++a)
                rc.off[a] = off_base != nullptr ? __ldg(off_base + (int64_t)((c.ogi * g.K + c.tap) * DIM + a) * g.P) : 0.f;
            rc.m = mask_base != nullptr ? __ldg(mask_base + (int64_t)(c.mgi * g.K + c.tap) * g.P) : 1.f;
            return rc;
        };
        // Plans chunk j from `cur` and requests the coordinates of chunk j + 2 into `fill`.  The three coordinate
        // sets rotate by name (the loop below is unrolled by three), never by assignment: copying a set whose loads
        // are still in flight would wait for them and put their latency back on the critical path.
        auto step = [&](int j, const RawCoords<DIM> &cur, RawCoords<DIM> &fill) -> bool {
            const int pbuf = j % PLAN_BUFS;
            const int tap = cur_c.tap, chan0 = grp * g.csg + cur_c.cc * CHUNK_C;
            if (j + 2 < n_chunks) {
                fill = coords_at(fetch_c);
                advance(fetch_c);
            }
            advance(cur_c);
            bool ok = ptx::mbar_wait(&plan_empty[pbuf], (uint32_t)(((j / PLAN_BUFS) & 1) ^ 1));
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) {
                if (lane == 0) atomicExch(P.status, 106);
                return false;
            }
            PlanEntry *slot = plan + (pbuf * TILE_POS + t) * NC;
            int tc[DIM];
#pragma unroll
            for (int a = 0; a < DIM; ++a) tc[a] = tap_tab[tap * DIM + a];
            build_plan_at<DIM, MODE>(g, pi, cur, deformable, tc, row_scale, slot);
            if (P.prefetch) {
                const uint4 *row0 = img16 + (uint32_t)chan0 * ESZ / 16u;
#pragma unroll
                for (int c = 0; c < NC; ++c) {
                    if (slot[c].w != 0u) {
                        const uint4 *ptr = row0 + slot[c].row16;
                        asm volatile("prefetch.global.L1 [%0];" ::"l"(ptr));
                        if (SPLIT) asm volatile("prefetch.global.L1 [%0];" ::"l"(ptr + 8));
                    }
                }
            }
            __syncwarp();
            if (lane == 0) ptx::mbar_arrive(&plan_full[pbuf]);
            return true;
        };
        RawCoords<DIM> r0, r1, r2;
        if (n_chunks > 0) {
            r0 = coords_at(fetch_c);
            advance(fetch_c);
        }
        if (n_chunks > 1) {
            r1 = coords_at(fetch_c);
            advance(fetch_c);
        }
        int j = 0;
        bool ok = true;
        for (; ok && j + 2 < n_chunks; j += 3) ok = step(j, r0, r2) && step(j + 1, r1, r0) && step(j + 2, r2, r1);
        if (ok && j < n_chunks) ok = step(j, r0, r2);
        if (ok && j + 1 < n_chunks) ok = step(j + 1, r1, r0);
    }

    ptx::tc_fence_before();
    __syncthreads();
    if (warp == MMA_WARP) ptx::tmem_dealloc(tmem_base, ncols);
}

// ---- staging kernels ---------------------------------------------------------------------------------
// [B, C, S] -> [B, S, C] through a 32 x 33 shared tile; ET is an unsigned type of the element size.
template <typename ET>
__global__ void __launch_bounds__(256) to_channels_last_kernel(const ET *__restrict__ src, ET *__restrict__ dst, int C,
                                                               int S) {
    __shared__ ET tile[32][33];
    const int b = blockIdx.z;
    const int s0 = blockIdx.x * 32, c0 = blockIdx.y * 32;
    const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;  // 32 x 8
    const ET *in = src + (int64_t)b * C * S;
    ET *out = dst + (int64_t)b * C * S;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int c = c0 + ty + 8 * i, s = s0 + tx;
        if (c < C && s < S) tile[ty + 8 * i][tx] = in[(int64_t)c * S + s];
    }
    __syncthreads();
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int s = s0 + ty + 8 * i, c = c0 + tx;
        if (c < C && s < S) out[(int64_t)s * C + c] = tile[tx][ty + 8 * i];
    }
}

// 16-bit [B, C, S] -> [B, S, C] with 16-byte loads, for S and C multiples of 8 and 2.  A 64 x 64 tile is held
// as 32-bit words of two neighbouring positions; words of a channel pair sit 32 words apart and pairs 65 words
// apart, so the transposing reads (one channel pair per lane) and the writes are free of bank conflicts.
__global__ void __launch_bounds__(256) to_channels_last16_kernel(const uint16_t *__restrict__ src,
                                                                 uint16_t *__restrict__ dst, int C, int S) {
    __shared__ uint32_t tile[32 * 65];
    const int b = blockIdx.z;
    const int s0 = blockIdx.x * 64, c0 = blockIdx.y * 64;
    const uint16_t *in = src + (int64_t)b * C * S;
    uint32_t *out = reinterpret_cast<uint32_t *>(dst + (int64_t)b * C * S);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int v = lane & 7;                  // 8 positions s0 + 8 v ...
#pragma unroll
    for (int pass = 0; pass < 2; ++pass) {
        const int cl = warp * 8 + (lane >> 3) * 2 + pass;   // one parity per instruction
        const int c = c0 + cl, s = s0 + v * 8;
        uint4 x = make_uint4(0u, 0u, 0u, 0u);
        if (c < C && s < S) x = __ldg(reinterpret_cast<const uint4 *>(in + (int64_t)c * S + s));
        uint32_t *w = tile + (cl >> 1) * 65 + (cl & 1) * 32 + v * 4;
        w[0] = x.x;
        w[1] = x.y;
        w[2] = x.z;
        w[3] = x.w;
    }
    __syncthreads();
    const int c = c0 + 2 * lane;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int s2 = warp * 4 + i;
        const uint32_t a = tile[lane * 65 + s2], bb = tile[lane * 65 + 32 + s2];
        const int s = s0 + 2 * s2;
        if (c < C && s < S) {
            out[((int64_t)s * C + c) >> 1] = __byte_perm(a, bb, 0x5410);
            out[((int64_t)(s + 1) * C + c) >> 1] = __byte_perm(a, bb, 0x7632);
        }
    }
}

// 32-bit [B, C, S] -> [B, S, C] with 16-byte loads and stores, for S and C multiples of 4; 64 x 64 tiles.
__global__ void __launch_bounds__(256) to_channels_last32_kernel(const uint32_t *__restrict__ src,
                                                                 uint32_t *__restrict__ dst, int C, int S) {
    __shared__ uint32_t tile[64 * 65];
    const int b = blockIdx.z;
    const int s0 = blockIdx.x * 64, c0 = blockIdx.y * 64;
    const uint32_t *in = src + (int64_t)b * C * S;
    uint32_t *out = dst + (int64_t)b * C * S;
    const int v = threadIdx.x & 15, r = threadIdx.x >> 4;   // 16 vectors per row, 16 rows per pass
#pragma unroll
    for (int pass = 0; pass < 4; ++pass) {
        const int cl = pass * 16 + r;
        const int c = c0 + cl, s = s0 + v * 4;
        uint4 x = make_uint4(0u, 0u, 0u, 0u);
        if (c < C && s < S) x = __ldg(reinterpret_cast<const uint4 *>(in + (int64_t)c * S + s));
        uint32_t *w = tile + cl * 65 + v * 4;
        w[0] = x.x;
        w[1] = x.y;
        w[2] = x.z;
        w[3] = x.w;
    }
    __syncthreads();
#pragma unroll
    for (int pass = 0; pass < 4; ++pass) {
        const int sl = pass * 16 + r;
        const int s = s0 + sl, c = c0 + v * 4;
        if (c < C && s < S) {
            uint4 x;
            x.x = tile[(v * 4 + 0) * 65 + sl];
            x.y = tile[(v * 4 + 1) * 65 + sl];
            x.z = tile[(v * 4 + 2) * 65 + sl];
            x.w = tile[(v * 4 + 3) * 65 + sl];
            *reinterpret_cast<uint4 *>(out + (int64_t)s * C + c) = x;
        }
    }
}

// weight [Cd, csg, K] -> hi/lo [g][tap][d'][s'] (KS = true) or [g][tap][s'][d'] (KS = false)
// (the weight tensor has fewer than 2^31 elements, checked by the launcher: 32-bit index arithmetic, whose
// divisions by run-time values cost a quarter of the 64-bit ones this small kernel used to spend its time on)
template <typename TW, bool KS>
__global__ void pack_weight_kernel(const TW *__restrict__ w, int mode, int groups, int cdg, int csg, int K,
                                   uint16_t *__restrict__ hi, uint16_t *__restrict__ lo) {
    const uint32_t n = (uint32_t)groups * (uint32_t)K * (uint32_t)cdg * (uint32_t)csg;
    const uint32_t ucdg = (uint32_t)cdg, ucsg = (uint32_t)csg, uK = (uint32_t)K;
    for (uint32_t i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x) {
        uint32_t r = i;
        uint32_t dl, sl;
        if (KS) {
            sl = r % ucsg; r /= ucsg;
            dl = r % ucdg; r /= ucdg;
        } else {
            dl = r % ucdg; r /= ucdg;
            sl = r % ucsg; r /= ucsg;
        }
        const uint32_t tap = r % uK;
        const uint32_t grp = r / uK;
        const float v = to_acc(w[((grp * ucdg + dl) * ucsg + sl) * uK + tap]);
        if (mode == TC_F16) {
            const __half h = __float2half_rn(v);
            hi[i] = *reinterpret_cast<const uint16_t *>(&h);
        } else {
            const __nv_bfloat16 h = __float2bfloat16_rn(v);
            hi[i] = *reinterpret_cast<const uint16_t *>(&h);
            if (mode == TC_SPLIT) {
                const __nv_bfloat16 l = __float2bfloat16_rn(v - __bfloat162float(h));
                lo[i] = *reinterpret_cast<const uint16_t *>(&l);
            }
        }
    }
}

// same, four elements per thread
__global__ void split_f32_vec4_kernel(const float4 *__restrict__ src, uint2 *__restrict__ hi, uint2 *__restrict__ lo,
                                      int64_t n4) {
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n4; i += (int64_t)gridDim.x * blockDim.x) {
        const float4 v = __ldg(src + i);
        const float f[4] = {v.x, v.y, v.z, v.w};
        uint32_t h[4], l[4];
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const __nv_bfloat16 hb = __float2bfloat16_rn(f[k]);
            h[k] = __bfloat16_as_ushort(hb);
            l[k] = __bfloat16_as_ushort(__float2bfloat16_rn(f[k] - __bfloat162float(hb)));
        }
        hi[i] = make_uint2(h[0] | (h[1] << 16), h[2] | (h[3] << 16));
        lo[i] = make_uint2(l[0] | (l[1] << 16), l[2] | (l[3] << 16));
    }
}

template <bool KS>
cudaError_t launch_pack_weight(const void *w, int dtype, int mode, int groups, int cdg, int csg, int K, void *hi,
                               void *lo, cudaStream_t stream) {
    const int64_t n = (int64_t)groups * K * cdg * csg;
    if (n >= ((int64_t)1 << 31)) return cudaErrorInvalidValue;
    const int blocks = (int)std::min<int64_t>((n + 255) / 256, 148 * 16);
    LaunchScope scope("pack_weight", stream);
    if (dtype == DT_F32)
        pack_weight_kernel<float, KS><<<blocks, 256, 0, stream>>>((const float *)w, mode, groups, cdg, csg, K,
                                                                 (uint16_t *)hi, (uint16_t *)lo);
    else if (dtype == DT_BF16)
        pack_weight_kernel<__nv_bfloat16, KS><<<blocks, 256, 0, stream>>>((const __nv_bfloat16 *)w, mode, groups, cdg,
                                                                         csg, K, (uint16_t *)hi, (uint16_t *)lo);
    else if (dtype == DT_F16)
        pack_weight_kernel<__half, KS><<<blocks, 256, 0, stream>>>((const __half *)w, mode, groups, cdg, csg, K,
                                                                  (uint16_t *)hi, (uint16_t *)lo);
    else
        return cudaErrorInvalidValue;
    return cudaGetLastError();
}

// f32 -> bf16 hi + lo (same layout), for operands that reach the tensor core through TMA
__global__ void split_f32_kernel(const float *__restrict__ src, __nv_bfloat16 *__restrict__ hi,
                                 __nv_bfloat16 *__restrict__ lo, int64_t n) {
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
        const float v = src[i];
        const __nv_bfloat16 h = __float2bfloat16_rn(v);
        hi[i] = h;
        lo[i] = __float2bfloat16_rn(v - __bfloat162float(h));
    }
}

}  // namespace

cudaError_t launch_pack_weight_ks(const void *w, int dtype, int mode, int groups, int cdg, int csg, int K, void *hi,
                                  void *lo, cudaStream_t stream) {
    return launch_pack_weight<true>(w, dtype, mode, groups, cdg, csg, K, hi, lo, stream);
}
cudaError_t launch_pack_weight_kd(const void *w, int dtype, int mode, int groups, int cdg, int csg, int K, void *hi,
                                  void *lo, cudaStream_t stream) {
    return launch_pack_weight<false>(w, dtype, mode, groups, cdg, csg, K, hi, lo, stream);
}

cudaError_t launch_split_f32(const float *src, void *hi, void *lo, int64_t n, cudaStream_t stream) {
    LaunchScope scope("split_f32", stream);
    const bool wide = n % 4 == 0 && (reinterpret_cast<uintptr_t>(src) & 15) == 0 &&
                      ((reinterpret_cast<uintptr_t>(hi) | reinterpret_cast<uintptr_t>(lo)) & 7) == 0;
    if (wide) {
        const int blocks = (int)std::min<int64_t>((n / 4 + 255) / 256, 148 * 16);
        split_f32_vec4_kernel<<<blocks, 256, 0, stream>>>(reinterpret_cast<const float4 *>(src), (uint2 *)hi, (uint2 *)lo,
                                                          n / 4);
    } else {
        const int blocks = (int)std::min<int64_t>((n + 255) / 256, 148 * 16);
        split_f32_kernel<<<blocks, 256, 0, stream>>>(src, (__nv_bfloat16 *)hi, (__nv_bfloat16 *)lo, n);
    }
    return cudaGetLastError();
}

cudaError_t launch_to_channels_last(const void *src, void *dst, int B, int C, int S, int elem_bytes,
                                    cudaStream_t stream) {
    dim3 grid((S + 31) / 32, (C + 31) / 32, B);
    LaunchScope scope("to_channels_last", stream);
    if (elem_bytes == 2 && S % 8 == 0 && C % 2 == 0 && (reinterpret_cast<uintptr_t>(src) & 15) == 0 &&
        (reinterpret_cast<uintptr_t>(dst) & 3) == 0) {
        dim3 grid64((S + 63) / 64, (C + 63) / 64, B);
        to_channels_last16_kernel<<<grid64, 256, 0, stream>>>((const uint16_t *)src, (uint16_t *)dst, C, S);
    } else if (elem_bytes == 2)
        to_channels_last_kernel<uint16_t><<<grid, 256, 0, stream>>>((const uint16_t *)src, (uint16_t *)dst, C, S);
    else if (elem_bytes == 4 && S % 4 == 0 && C % 4 == 0 && (reinterpret_cast<uintptr_t>(src) & 15) == 0 &&
             (reinterpret_cast<uintptr_t>(dst) & 15) == 0) {
        dim3 grid64((S + 63) / 64, (C + 63) / 64, B);
        to_channels_last32_kernel<<<grid64, 256, 0, stream>>>((const uint32_t *)src, (uint32_t *)dst, C, S);
    } else if (elem_bytes == 4)
        to_channels_last_kernel<uint32_t><<<grid, 256, 0, stream>>>((const uint32_t *)src, (uint32_t *)dst, C, S);
    else
        return cudaErrorInvalidValue;
    return cudaGetLastError();
}

bool make_tensor_map_16bit(CUtensorMap *map, const void *base, int rank, const uint64_t *dims,
                           const uint64_t *strides_bytes, const uint32_t *box) {
    typedef CUresult (*EncodeFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                 const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                 CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
    static EncodeFn encode = nullptr;
    if (encode == nullptr) {
        void *fn = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres) != cudaSuccess ||
            qres != cudaDriverEntryPointSuccess || fn == nullptr)
            return false;
        encode = (EncodeFn)fn;
    }
    cuuint32_t ones[5] = {1, 1, 1, 1, 1};
    const CUresult rc = encode(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, (cuuint32_t)rank, const_cast<void *>(base),
                               (const cuuint64_t *)dims, (const cuuint64_t *)strides_bytes, (const cuuint32_t *)box,
                               ones, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                               CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return rc == CUDA_SUCCESS;
}

// Tuning knob read from the environment (experiments only; the defaults are what is measured and reported).
int tuning_int(const char *name, int fallback) {
    const char *v = getenv(name);
    if (v == nullptr || *v == 0) return fallback;
    const int x = atoi(v);
    return x > 0 ? x : fallback;
}

// ---- launcher -----------------------------------------------------------------------------------------
size_t fwd_tc_smem_bytes(int dim, int mode, int bn, int stages) {
    const int parts = mode == TC_SPLIT ? 2 : 1;
    const size_t stage = (size_t)(A_TILE_BYTES + bn * 128) * parts;
    const size_t plan = (size_t)PLAN_BUFS * (1 << dim) * TILE_POS * 8;
    return 1024 + stages * stage + plan + (3 * stages + 1 + 2 * PLAN_BUFS) * 8 + 16;
}

// statically allocated shared memory of the kernel (tap table), which counts against the same 227 KB
static size_t fwd_static_smem(int dim) { return (size_t)FWD_MAX_TAPS * dim * sizeof(int16_t) + 64; }

// Picks the dense-channel tile and the pipeline depth; returns false when the shape is not covered.
bool fwd_tc_config(int dim, int mode, int cdg, int *bn, int *stages) {
    static const int cap_split = tuning_int("TVDCN_B200_FWD_BN_SPLIT", 256);
    static const int max_stages = tuning_int("TVDCN_B200_FWD_STAGES", 3);
    const int cap = mode == TC_SPLIT ? cap_split : 256;
    // widest tile of dense channels first (the sampled tile is produced once per CTA, so a wider tile divides the
    // sampling work), then the deepest pipeline that fits
    int n = 0, s = 0;
    for (int cand_n : {256, 128, 64}) {
        if (cand_n > cap || cdg % cand_n != 0) continue;
        for (int cand = max_stages; cand >= 2; --cand)
            if (fwd_tc_smem_bytes(dim, mode, cand_n, cand) + fwd_static_smem(dim) <= 227 * 1024) { s = cand; break; }
        if (s != 0) { n = cand_n; break; }
    }
    if (n == 0) return false;
    *bn = n;
    *stages = s;
    return true;
}

template <int DIM, int MODE>
cudaError_t launch_fwd_tc_t(const GeoHost &h, const FwdParams<DIM> &P, const CUtensorMap &hi, const CUtensorMap &lo,
                            cudaStream_t stream) {
    const size_t smem = fwd_tc_smem_bytes(DIM, MODE, P.bn, P.stages);
    auto kern = dcn_fwd_tc_kernel<DIM, MODE>;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return e;
    const long long BP = (long long)h.B * h.P;
    dim3 grid((unsigned)((BP + TILE_POS - 1) / TILE_POS), (unsigned)(h.groups * ((h.Cd / h.groups) / P.bn)));
    LaunchScope scope("dcn_fwd_tc", stream);
    kern<<<grid, FWD_THREADS, smem, stream>>>(P, hi, lo);
    return cudaGetLastError();
}

// img_cl: channels-last sampled image (16-bit or f32 per mode); w_hi / w_lo: weights packed [g][tap][d'][s'].
cudaError_t launch_sample_gemm_tc(const GeoHost &h, int mode, const void *img_cl, const void *w_hi, const void *w_lo,
                                  const float *offset, const float *mask, const float *bias, void *out, int *status,
                                  cudaStream_t stream) {
    const int cdg = h.Cd / h.groups, csg = h.Cs / h.groups;
    int bn = 0, stages = 0;
    if (!fwd_tc_config(h.dim, mode, cdg, &bn, &stages)) return cudaErrorInvalidConfiguration;
    CUtensorMap hi, lo;
    const uint64_t dims[4] = {(uint64_t)csg, (uint64_t)cdg, (uint64_t)h.K, (uint64_t)h.groups};
    const uint64_t strides[3] = {(uint64_t)csg * 2, (uint64_t)csg * cdg * 2, (uint64_t)csg * cdg * h.K * 2};
    const uint32_t box[4] = {CHUNK_C, (uint32_t)bn, 1, 1};
    if (!make_tensor_map_16bit(&hi, w_hi, 4, dims, strides, box)) return cudaErrorInvalidValue;
    if (mode == TC_SPLIT) {
        if (!make_tensor_map_16bit(&lo, w_lo, 4, dims, strides, box)) return cudaErrorInvalidValue;
    } else {
        lo = hi;
    }
    auto run = [&](auto dimc) -> cudaError_t {
        constexpr int DIM = decltype(dimc)::value;
        FwdParams<DIM> P;
        P.g = geo_from_host<DIM>(h);
        P.img_cl = img_cl;
        P.offset = offset;
        P.mask = mask;
        P.bias = bias;
        P.out = out;
        P.status = status;
        P.bn = bn;
        P.stages = stages;
        P.chunks_per_tap = csg / CHUNK_C;
        static const int prefetch = tuning_int("TVDCN_B200_PREFETCH", 0);
        P.prefetch = prefetch;
        if (mode == TC_BF16) return launch_fwd_tc_t<DIM, TC_BF16>(h, P, hi, lo, stream);
        if (mode == TC_F16) return launch_fwd_tc_t<DIM, TC_F16>(h, P, hi, lo, stream);
        return launch_fwd_tc_t<DIM, TC_SPLIT>(h, P, hi, lo, stream);
    };
    if (h.dim == 1) return run(std::integral_constant<int, 1>());
    if (h.dim == 2) return run(std::integral_constant<int, 2>());
    if (h.dim == 3) return run(std::integral_constant<int, 3>());
    return cudaErrorInvalidValue;
}

}  // namespace tvdcn_b200
