// Generic SIMT kernels: any shape, any channel grouping, f32 / f64 / f16 / bf16.
//
// They are the correctness floor and the f64 path (the tensor pipe has no f64 kind); the
// tensor-core kernels take over where the shape allows.  All three are shared-memory-tiled
// GEMMs whose sampled operand is produced on the fly -- the im2col column buffer of the
// reference (tvdcn/csrc/ops/cuda/deform_conv2d_kernel.cpp:331-340) never exists in global memory.
//
//   sample_gemm   replaces  im2col + addmm_ + layout copy + bias add   (…2d_kernel.cpp:341-380)
//   gemm_scatter  replaces  addmm_ + compute_grad_offset + compute_grad_mask + col2im (…:519-598)
//   sample_wgrad  replaces  second im2col + addmm_                     (…:600-626)
#include "common.cuh"
#include "kernels.h"

namespace tvdcn_b200 {
namespace {

constexpr int BM = 64;   // tile extent along grid positions (sample_gemm, gemm_scatter) / dense channels (wgrad)
constexpr int BN = 64;   // tile extent along the other output axis
constexpr int BK = 16;   // reduction chunk
constexpr int NT = 256;  // threads per block; each owns a 4 x 4 micro tile
constexpr int PADDED = BM + 4;

template <int DIM>
Geo<DIM> make_geo(const GeoHost &h) {
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

// One masked sample of channel s at the cached point.
template <typename T, typename TA, int DIM>
__device__ __forceinline__ acc_t<T> masked_sample(const Geo<DIM> &g, const T *__restrict__ img,
                                                  const TA *__restrict__ mask, const SamplePoint<DIM, acc_t<T>> &pt,
                                                  bool deformable, int b, int s, int tap, int p) {
    using A = acc_t<T>;
    const int64_t plane = ((int64_t)b * g.Cs + s) * (int64_t)g.S;
    A val = (A)0;
    for_each_corner<DIM, A>(g, pt, deformable, -1, [&](int flat, A w) { val += w * load_acc(img, plane + flat); });
    if (mask != nullptr)
        val *= (A)load_acc(mask, (((int64_t)b * g.mg + s / g.cs_per_mg) * g.K + tap) * (int64_t)g.P + p);
    return val;
}

// ------------------------------------------------------------------------------------------
// dense[b, d, p] = bias[d] + sum_k W[d, k] * col[k | b, p],  k = tap * csg + s' (tap-major so the
// four consecutive k of one thread share a sampling point).
// grid: x = position tiles over the flattened (b, p) axis, y = groups * dense-channel tiles.
// ------------------------------------------------------------------------------------------
template <typename T, typename TA, int DIM>
__global__ void __launch_bounds__(NT)
sample_gemm_kernel(const Geo<DIM> g, const T *__restrict__ img, const T *__restrict__ weight,
                   const TA *__restrict__ offset, const TA *__restrict__ mask, const TA *__restrict__ bias,
                   T *__restrict__ out) {
    using A = acc_t<T>;
    __shared__ A As[BK][PADDED];
    __shared__ A Ws[BK][PADDED];
    const int t = threadIdx.x;
    const int tx = t % 16, ty = t / 16;
    const int64_t m0 = (int64_t)blockIdx.x * BM;
    const int tiles_n = (g.cdg + BN - 1) / BN;
    const int grp = blockIdx.y / tiles_n;
    const int n0 = (blockIdx.y % tiles_n) * BN;
    const int Ktot = g.csg * g.K;
    const bool deformable = offset != nullptr;

    const int sm = t % BM;
    const int sk = (t / BM) * 4;
    const int64_t sidx = m0 + sm;
    const bool svalid = sidx < g.BP;
    const int sb = svalid ? (int)(sidx / g.P) : 0;
    const int sp = svalid ? (int)(sidx % g.P) : 0;

    A acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = (A)0;

    SamplePoint<DIM, A> pt;
    int cached_tap = -1, cached_og = -1;

    for (int k0 = 0; k0 < Ktot; k0 += BK) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int kk = t % BK;
            const int n = t / BK + 16 * i;
            const int k = k0 + kk;
            A v = (A)0;
            if (k < Ktot && n0 + n < g.cdg) {
                const int tap = k / g.csg, sl = k % g.csg;
                v = load_acc(weight, ((int64_t)(grp * g.cdg + n0 + n) * g.csg + sl) * g.K + tap);
            }
            Ws[kk][n] = v;
        }
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int kk = sk + i;
            const int k = k0 + kk;
            A v = (A)0;
            if (svalid && k < Ktot) {
                const int tap = k / g.csg, sl = k % g.csg;
                const int s = grp * g.csg + sl;
                const int ogi = deformable ? s / g.cs_per_og : 0;
                if (tap != cached_tap || ogi != cached_og) {
                    compute_point<DIM, TA, A>(g, offset, sb, ogi, tap, sp, pt);
                    cached_tap = tap;
                    cached_og = ogi;
                }
                v = masked_sample<T, TA, DIM>(g, img, mask, pt, deformable, sb, s, tap, sp);
            }
            As[kk][sm] = v;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < BK; ++kk) {
            A a[4], w[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) a[i] = As[kk][tx * 4 + i];
#pragma unroll
            for (int j = 0; j < 4; ++j) w[j] = Ws[kk][ty * 4 + j];
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] += a[i] * w[j];
        }
        __syncthreads();
    }

#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int64_t idx = m0 + tx * 4 + i;
        if (idx >= g.BP) continue;
        const int b = (int)(idx / g.P), p = (int)(idx % g.P);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int n = n0 + ty * 4 + j;
            if (n >= g.cdg) continue;
            const int d = grp * g.cdg + n;
            A v = acc[i][j];
            if (bias != nullptr) v += (A)load_acc(bias, d);
            store_acc(out, ((int64_t)b * g.Cd + d) * (int64_t)g.P + p, v);
        }
    }
}

// ------------------------------------------------------------------------------------------
// col[k | b, p] = sum_{d in group} W[d, k] * dense[b, d, p]  (k tap-major), consumed in registers:
// scatter onto the sampled image, offset gradient, mask gradient.
// grid: x = position tiles, y = groups * k tiles.
// ------------------------------------------------------------------------------------------
template <typename T, typename TA, int DIM>
__global__ void __launch_bounds__(NT)
gemm_scatter_kernel(const Geo<DIM> g, const T *__restrict__ dense, const T *__restrict__ weight,
                    const TA *__restrict__ offset, const TA *__restrict__ mask, const T *__restrict__ img,
                    acc_t<T> *__restrict__ img_grad, acc_t<T> *__restrict__ goff, acc_t<T> *__restrict__ gmask) {
    using A = acc_t<T>;
    __shared__ A Ds[BK][PADDED];
    __shared__ A Ws[BK][PADDED];
    const int t = threadIdx.x;
    const int tx = t % 16, ty = t / 16;
    const int64_t m0 = (int64_t)blockIdx.x * BM;
    const int Ktot = g.csg * g.K;
    const int tiles_k = (Ktot + BN - 1) / BN;
    const int grp = blockIdx.y / tiles_k;
    const int kt0 = (blockIdx.y % tiles_k) * BN;
    const bool deformable = offset != nullptr;

    const int lm = t % BM;
    const int64_t lidx = m0 + lm;
    const bool lvalid = lidx < g.BP;
    const int lb = lvalid ? (int)(lidx / g.P) : 0;
    const int lp = lvalid ? (int)(lidx % g.P) : 0;

    // weight column of this thread (fixed through the reduction)
    const int wn = t % BN;
    const int wk = kt0 + wn;
    const bool wvalid = wk < Ktot;
    const int wtap = wvalid ? wk / g.csg : 0;
    const int wsl = wvalid ? wk % g.csg : 0;

    A acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = (A)0;

    for (int d0 = 0; d0 < g.cdg; d0 += BK) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int kk = t / BM + 4 * i;
            A v = (A)0;
            if (lvalid && d0 + kk < g.cdg)
                v = load_acc(dense, ((int64_t)lb * g.Cd + grp * g.cdg + d0 + kk) * (int64_t)g.P + lp);
            Ds[kk][lm] = v;
        }
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int kk = t / BN + 4 * i;
            A v = (A)0;
            if (wvalid && d0 + kk < g.cdg)
                v = load_acc(weight, ((int64_t)(grp * g.cdg + d0 + kk) * g.csg + wsl) * g.K + wtap);
            Ws[kk][wn] = v;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < BK; ++kk) {
            A a[4], w[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) a[i] = Ds[kk][tx * 4 + i];
#pragma unroll
            for (int j = 0; j < 4; ++j) w[j] = Ws[kk][ty * 4 + j];
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] += a[i] * w[j];
        }
        __syncthreads();
    }

    const bool want_coord = (goff != nullptr) || (gmask != nullptr);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int64_t idx = m0 + tx * 4 + i;
        if (idx >= g.BP) continue;
        const int b = (int)(idx / g.P), p = (int)(idx % g.P);
        SamplePoint<DIM, A> pt;
        int cached_tap = -1, cached_og = -1;
        // running sums over the channels of this thread that share (tap, group)
        A go_sum[DIM];
        A gm_sum = (A)0;
        int go_tap = -1, go_og = -1, gm_tap = -1, gm_mg = -1;
#pragma unroll
        for (int a = 0; a < DIM; ++a) go_sum[a] = (A)0;

        auto flush_off = [&]() {
            if (go_tap >= 0) {
#pragma unroll
                for (int a = 0; a < DIM; ++a)
                    atomic_add(goff + ((((int64_t)b * g.og + go_og) * g.K + go_tap) * DIM + a) * (int64_t)g.P + p,
                               go_sum[a]);
            }
#pragma unroll
            for (int a = 0; a < DIM; ++a) go_sum[a] = (A)0;
        };
        auto flush_mask = [&]() {
            if (gm_tap >= 0)
                atomic_add(gmask + (((int64_t)b * g.mg + gm_mg) * g.K + gm_tap) * (int64_t)g.P + p, gm_sum);
            gm_sum = (A)0;
        };

#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int k = kt0 + ty * 4 + j;
            if (k >= Ktot) continue;
            const int tap = k / g.csg, sl = k % g.csg;
            const int s = grp * g.csg + sl;
            const int ogi = deformable ? s / g.cs_per_og : 0;
            if (tap != cached_tap || ogi != cached_og) {
                compute_point<DIM, TA, A>(g, offset, b, ogi, tap, p, pt);
                cached_tap = tap;
                cached_og = ogi;
            }
            const int mgi = mask != nullptr ? s / g.cs_per_mg : 0;
            const A m = mask != nullptr
                            ? (A)load_acc(mask, (((int64_t)b * g.mg + mgi) * g.K + tap) * (int64_t)g.P + p)
                            : (A)1;
            const A col = acc[i][j];
            const int64_t plane = ((int64_t)b * g.Cs + s) * (int64_t)g.S;
            if (img_grad != nullptr) {
                const A cm = col * m;
                for_each_corner<DIM, A>(g, pt, deformable, -1,
                                        [&](int flat, A w) { atomic_add(img_grad + plane + flat, cm * w); });
            }
            if (want_coord) {
                if (goff != nullptr) {
                    if (tap != go_tap || ogi != go_og) {
                        flush_off();
                        go_tap = tap;
                        go_og = ogi;
                    }
#pragma unroll
                    for (int a = 0; a < DIM; ++a) {
                        A dv = (A)0;
                        for_each_corner<DIM, A>(g, pt, true, a,
                                                [&](int flat, A w) { dv += w * load_acc(img, plane + flat); });
                        go_sum[a] += col * m * dv;
                    }
                }
                if (gmask != nullptr) {
                    if (tap != gm_tap || mgi != gm_mg) {
                        flush_mask();
                        gm_tap = tap;
                        gm_mg = mgi;
                    }
                    A sv = (A)0;
                    for_each_corner<DIM, A>(g, pt, deformable, -1,
                                            [&](int flat, A w) { sv += w * load_acc(img, plane + flat); });
                    gm_sum += col * sv;
                }
            }
        }
        if (goff != nullptr) flush_off();
        if (gmask != nullptr) flush_mask();
    }
}

// ------------------------------------------------------------------------------------------
// gw[d, k] += sum_{(b, p) in split} dense[b, d, p] * col[k | b, p]
// grid: x = k tiles (tap-major), y = groups * dense-channel tiles, z = position splits.
// ------------------------------------------------------------------------------------------
template <typename T, typename TA, int DIM>
__global__ void __launch_bounds__(NT)
sample_wgrad_kernel(const Geo<DIM> g, const T *__restrict__ dense, const T *__restrict__ img,
                    const TA *__restrict__ offset, const TA *__restrict__ mask, acc_t<T> *__restrict__ gw,
                    long long pos_per_split) {
    using A = acc_t<T>;
    __shared__ A Ds[BK][PADDED];
    __shared__ A Cs[BK][PADDED];
    const int t = threadIdx.x;
    const int tx = t % 16, ty = t / 16;
    const int Ktot = g.csg * g.K;
    const int kt0 = blockIdx.x * BN;
    const int tiles_d = (g.cdg + BM - 1) / BM;
    const int grp = blockIdx.y / tiles_d;
    const int d0 = (blockIdx.y % tiles_d) * BM;
    const bool deformable = offset != nullptr;
    const long long begin = (long long)blockIdx.z * pos_per_split;
    const long long end = min(begin + pos_per_split, g.BP);

    const int lpos = t % BK;
    const int lsub = t / BK;  // 0..15

    A acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = (A)0;

    for (long long pos0 = begin; pos0 < end; pos0 += BK) {
        const long long idx = pos0 + lpos;
        const bool valid = idx < end;
        const int b = valid ? (int)(idx / g.P) : 0;
        const int p = valid ? (int)(idx % g.P) : 0;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int dd = lsub + 16 * i;
            A v = (A)0;
            if (valid && d0 + dd < g.cdg)
                v = load_acc(dense, ((int64_t)b * g.Cd + grp * g.cdg + d0 + dd) * (int64_t)g.P + p);
            Ds[lpos][dd] = v;
        }
        SamplePoint<DIM, A> pt;
        int cached_tap = -1, cached_og = -1;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int kk = lsub * 4 + i;
            const int k = kt0 + kk;
            A v = (A)0;
            if (valid && k < Ktot) {
                const int tap = k / g.csg, sl = k % g.csg;
                const int s = grp * g.csg + sl;
                const int ogi = deformable ? s / g.cs_per_og : 0;
                if (tap != cached_tap || ogi != cached_og) {
                    compute_point<DIM, TA, A>(g, offset, b, ogi, tap, p, pt);
                    cached_tap = tap;
                    cached_og = ogi;
                }
                v = masked_sample<T, TA, DIM>(g, img, mask, pt, deformable, b, s, tap, p);
            }
            Cs[lpos][kk] = v;
        }
        __syncthreads();
#pragma unroll
        for (int pp = 0; pp < BK; ++pp) {
            A a[4], c[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) a[i] = Ds[pp][ty * 4 + i];
#pragma unroll
            for (int j = 0; j < 4; ++j) c[j] = Cs[pp][tx * 4 + j];
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] += a[i] * c[j];
        }
        __syncthreads();
    }

#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int dd = d0 + ty * 4 + i;
        if (dd >= g.cdg) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int k = kt0 + tx * 4 + j;
            if (k >= Ktot) continue;
            const int tap = k / g.csg, sl = k % g.csg;
            atomic_add(gw + ((int64_t)(grp * g.cdg + dd) * g.csg + sl) * g.K + tap, acc[i][j]);
        }
    }
}

// out[c] = sum over batch and space of x[b, c, s]; one 1024-thread block per channel: warp w walks the
// images b = w, w + 32, ... and reads each contiguous row of S elements with 16-byte loads when it can.
template <typename T, typename TO>
__global__ void __launch_bounds__(1024) channel_sum_kernel(const T *__restrict__ x, int B, int C, int S,
                                                           TO *__restrict__ out) {
    using A = acc_t<T>;
    constexpr int VEC = 16 / sizeof(T);
    __shared__ A red[32];
    const int c = blockIdx.x;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const bool vec_ok = (S % VEC == 0) && ((reinterpret_cast<uintptr_t>(x) & 15) == 0);
    A sum = (A)0;
    for (int b = warp; b < B; b += 32) {
        const T *row = x + ((int64_t)b * C + c) * (int64_t)S;
        if (vec_ok) {
            const uint4 *row16 = reinterpret_cast<const uint4 *>(row);
            for (int i = lane; i < S / VEC; i += 32) {
                const uint4 v = __ldg(row16 + i);
                const T *e = reinterpret_cast<const T *>(&v);
#pragma unroll
                for (int k = 0; k < VEC; ++k) sum += to_acc(e[k]);
            }
        } else {
            for (int s2 = lane; s2 < S; s2 += 32) sum += load_acc(row, s2);
        }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
    if (lane == 0) red[warp] = sum;
    __syncthreads();
    if (warp == 0) {
        A v = red[lane];
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
        if (lane == 0) store_acc(out, c, v);
    }
}

template <typename A, typename T>
__global__ void cast_kernel(const A *__restrict__ src, T *__restrict__ dst, int64_t n) {
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x)
        store_acc(dst, i, src[i]);
}

template <typename A, typename TA>
__global__ void fill_bias_kernel(const TA *__restrict__ bias, int C, int S, int64_t n, A *__restrict__ dst) {
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
        const int c = (int)((i / S) % C);
        dst[i] = bias != nullptr ? (A)load_acc(bias, c) : (A)0;
    }
}

// ---- dispatch helpers ------------------------------------------------------------------
template <typename F>
cudaError_t dispatch_types(int dtype, int aux, F &&f) {
    if (dtype == DT_F32 && aux == DT_F32) return f((float *)nullptr, (float *)nullptr);
    if (dtype == DT_F64 && aux == DT_F64) return f((double *)nullptr, (double *)nullptr);
    if (dtype == DT_F16 && aux == DT_F16) return f((__half *)nullptr, (__half *)nullptr);
    if (dtype == DT_BF16 && aux == DT_BF16) return f((__nv_bfloat16 *)nullptr, (__nv_bfloat16 *)nullptr);
    if (dtype == DT_F16 && aux == DT_F32) return f((__half *)nullptr, (float *)nullptr);
    if (dtype == DT_BF16 && aux == DT_F32) return f((__nv_bfloat16 *)nullptr, (float *)nullptr);
    return cudaErrorInvalidValue;
}

template <typename F>
cudaError_t dispatch_dim(int dim, F &&f) {
    if (dim == 1) return f(std::integral_constant<int, 1>());
    if (dim == 2) return f(std::integral_constant<int, 2>());
    if (dim == 3) return f(std::integral_constant<int, 3>());
    return cudaErrorInvalidValue;
}

int grid_1d(int64_t n, int threads) {
    int64_t b = (n + threads - 1) / threads;
    const int64_t cap = 148 * 16;
    return (int)(b < 1 ? 1 : (b > cap ? cap : b));
}

}  // namespace

cudaError_t launch_sample_gemm(const GeoHost &h, int dtype, int aux, const void *img, const void *weight,
                               const void *offset, const void *mask, const void *bias, void *out,
                               cudaStream_t stream) {
    return dispatch_types(dtype, aux, [&](auto *tp, auto *tap) {
        using T = std::remove_pointer_t<decltype(tp)>;
        using TA = std::remove_pointer_t<decltype(tap)>;
        return dispatch_dim(h.dim, [&](auto dimc) {
            constexpr int DIM = decltype(dimc)::value;
            const Geo<DIM> g = make_geo<DIM>(h);
            dim3 grid((unsigned)((g.BP + BM - 1) / BM), (unsigned)(g.groups * ((g.cdg + BN - 1) / BN)));
            LaunchScope scope("sample_gemm", stream);
            sample_gemm_kernel<T, TA, DIM><<<grid, NT, 0, stream>>>(g, (const T *)img, (const T *)weight,
                                                                    (const TA *)offset, (const TA *)mask,
                                                                    (const TA *)bias, (T *)out);
            return cudaGetLastError();
        });
    });
}

cudaError_t launch_gemm_scatter(const GeoHost &h, int dtype, int aux, const void *dense, const void *weight,
                                const void *offset, const void *mask, const void *img, void *img_grad,
                                void *goff, void *gmask, cudaStream_t stream) {
    return dispatch_types(dtype, aux, [&](auto *tp, auto *tap) {
        using T = std::remove_pointer_t<decltype(tp)>;
        using TA = std::remove_pointer_t<decltype(tap)>;
        using A = acc_t<T>;
        return dispatch_dim(h.dim, [&](auto dimc) {
            constexpr int DIM = decltype(dimc)::value;
            const Geo<DIM> g = make_geo<DIM>(h);
            const int Ktot = g.csg * g.K;
            dim3 grid((unsigned)((g.BP + BM - 1) / BM), (unsigned)(g.groups * ((Ktot + BN - 1) / BN)));
            LaunchScope scope("gemm_scatter", stream);
            gemm_scatter_kernel<T, TA, DIM><<<grid, NT, 0, stream>>>(g, (const T *)dense, (const T *)weight,
                                                                     (const TA *)offset, (const TA *)mask,
                                                                     (const T *)img, (A *)img_grad, (A *)goff,
                                                                     (A *)gmask);
            return cudaGetLastError();
        });
    });
}

cudaError_t launch_sample_wgrad(const GeoHost &h, int dtype, int aux, const void *dense, const void *img,
                                const void *offset, const void *mask, void *gw, cudaStream_t stream) {
    return dispatch_types(dtype, aux, [&](auto *tp, auto *tap) {
        using T = std::remove_pointer_t<decltype(tp)>;
        using TA = std::remove_pointer_t<decltype(tap)>;
        using A = acc_t<T>;
        return dispatch_dim(h.dim, [&](auto dimc) {
            constexpr int DIM = decltype(dimc)::value;
            const Geo<DIM> g = make_geo<DIM>(h);
            const int Ktot = g.csg * g.K;
            const int tiles = ((Ktot + BN - 1) / BN) * g.groups * ((g.cdg + BM - 1) / BM);
            // enough position splits for about four waves of blocks, each at least 256 positions long
            long long splits = (148LL * 4 + tiles - 1) / tiles;
            const long long max_splits = (g.BP + 255) / 256;
            if (splits > max_splits) splits = max_splits;
            if (splits < 1) splits = 1;
            if (splits > 65535) splits = 65535;
            long long per = (g.BP + splits - 1) / splits;
            per = (per + BK - 1) / BK * BK;
            splits = (g.BP + per - 1) / per;
            dim3 grid((unsigned)((Ktot + BN - 1) / BN), (unsigned)(g.groups * ((g.cdg + BM - 1) / BM)),
                      (unsigned)splits);
            LaunchScope scope("sample_wgrad", stream);
            sample_wgrad_kernel<T, TA, DIM><<<grid, NT, 0, stream>>>(g, (const T *)dense, (const T *)img,
                                                                     (const TA *)offset, (const TA *)mask, (A *)gw,
                                                                     per);
            return cudaGetLastError();
        });
    });
}

cudaError_t launch_channel_sum(int dtype, int out_dtype, const void *x, int B, int C, int S, void *out,
                               cudaStream_t stream) {
    return dispatch_types(dtype, out_dtype, [&](auto *tp, auto *top) {
        using T = std::remove_pointer_t<decltype(tp)>;
        using TO = std::remove_pointer_t<decltype(top)>;
        LaunchScope scope("channel_sum", stream);
        channel_sum_kernel<T, TO><<<C, 1024, 0, stream>>>((const T *)x, B, C, S, (TO *)out);
        return cudaGetLastError();
    });
}

cudaError_t launch_cast_from_acc(int dst_dtype, const void *src, void *dst, int64_t n, cudaStream_t stream) {
    if (n <= 0) return cudaSuccess;
    const int blocks = grid_1d(n, 256);
    LaunchScope scope("cast", stream);
    if (dst_dtype == DT_F16)
        cast_kernel<float, __half><<<blocks, 256, 0, stream>>>((const float *)src, (__half *)dst, n);
    else if (dst_dtype == DT_BF16)
        cast_kernel<float, __nv_bfloat16><<<blocks, 256, 0, stream>>>((const float *)src, (__nv_bfloat16 *)dst, n);
    else
        return cudaErrorInvalidValue;
    return cudaGetLastError();
}

cudaError_t launch_fill_bias(int dtype, int aux, const void *bias, int B, int C, int S, void *dst,
                             cudaStream_t stream) {
    const int64_t n = (int64_t)B * C * S;
    if (n <= 0) return cudaSuccess;
    const int blocks = grid_1d(n, 256);
    return dispatch_types(dtype, aux, [&](auto *tp, auto *tap) {
        using T = std::remove_pointer_t<decltype(tp)>;
        using TA = std::remove_pointer_t<decltype(tap)>;
        using A = acc_t<T>;
        LaunchScope scope("fill_bias", stream);
        fill_bias_kernel<A, TA><<<blocks, 256, 0, stream>>>((const TA *)bias, C, S, n, (A *)dst);
        return cudaGetLastError();
    });
}

}  // namespace tvdcn_b200
