// Shared device-side vocabulary of the deformable-convolution kernels.
//
// Terms (the same for the convolution and the transposed convolution):
//   sampled image  tensor read or written at fractional positions; [B, Cs, *img]
//                  (conv: input / grad_input, transposed: output / grad_output)
//   dense tensor   tensor that enters the GEMM as it is, laid out on the offset grid; [B, Cd, *grid]
//                  (conv: output / grad_output, transposed: input / grad_input)
//   weight         [Cd, Cs / groups, taps] in both cases
//   column value   col[s, tap | b, p] -- exists only in registers / shared / tensor memory
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace tvdcn_b200 {

template <typename T> struct Acc { using type = float; };
template <> struct Acc<double> { using type = double; };
template <typename T> using acc_t = typename Acc<T>::type;

__device__ __forceinline__ float load_acc(const float *p, int64_t i) { return __ldg(p + i); }
__device__ __forceinline__ double load_acc(const double *p, int64_t i) { return __ldg(p + i); }
__device__ __forceinline__ float load_acc(const __half *p, int64_t i) { return __half2float(__ldg(p + i)); }
__device__ __forceinline__ float load_acc(const __nv_bfloat16 *p, int64_t i) {
    return __bfloat162float(__ldg(p + i));
}

__device__ __forceinline__ float to_acc(float v) { return v; }
__device__ __forceinline__ double to_acc(double v) { return v; }
__device__ __forceinline__ float to_acc(__half v) { return __half2float(v); }
__device__ __forceinline__ float to_acc(__nv_bfloat16 v) { return __bfloat162float(v); }

__device__ __forceinline__ void store_acc(float *p, int64_t i, float v) { p[i] = v; }
__device__ __forceinline__ void store_acc(double *p, int64_t i, double v) { p[i] = v; }
__device__ __forceinline__ void store_acc(__half *p, int64_t i, float v) { p[i] = __float2half_rn(v); }
__device__ __forceinline__ void store_acc(__nv_bfloat16 *p, int64_t i, float v) { p[i] = __float2bfloat16_rn(v); }

// Geometry of one problem, expressed in sampled-image / dense-tensor terms.
template <int DIM>
struct Geo {
    int B;          // batch
    int Cs, Cd;     // channels of the sampled image / of the dense tensor
    int groups;     // convolution groups
    int og, mg;     // offset groups (0: integer-grid sampling), mask groups (0: no mask)
    int K;          // kernel taps
    int S, P;       // spatial elements per image: sampled image, offset grid
    int csg, cdg;   // channels per convolution group
    int cs_per_og, cs_per_mg;
    long long BP;   // B * P
    int img[DIM], grid[DIM], ker[DIM], stride[DIM], pad[DIM], dil[DIM];
};

// Fractional sampling position of one (batch, offset group, tap, grid position).
template <int DIM, typename A>
struct SamplePoint {
    int fl[DIM];  // floor of the coordinate per axis
    A fr[DIM];    // fractional part per axis
};

// position = grid * stride - pad + tap * dilation + offset; offset channel order is
// ((group * taps + tap) * DIM + axis), axis 0 outermost.
template <int DIM, typename TA, typename A>
__device__ __forceinline__ void compute_point(const Geo<DIM> &g, const TA *__restrict__ offset, int b, int ogi,
                                              int tap, int p, SamplePoint<DIM, A> &sp) {
    int pc[DIM], tc[DIM];
    int r = p;
#pragma unroll
    for (int a = DIM - 1; a >= 0; --a) {
        pc[a] = r % g.grid[a];
        r /= g.grid[a];
    }
    r = tap;
#pragma unroll
    for (int a = DIM - 1; a >= 0; --a) {
        tc[a] = r % g.ker[a];
        r /= g.ker[a];
    }
#pragma unroll
    for (int a = 0; a < DIM; ++a) {
        const int base = pc[a] * g.stride[a] - g.pad[a] + tc[a] * g.dil[a];
        if (offset != nullptr) {
            const A o = load_acc(offset, ((((int64_t)b * g.og + ogi) * g.K + tap) * DIM + a) * (int64_t)g.P + p);
            const A pos = (A)base + o;
            const A f = floor(pos);
            sp.fl[a] = (int)f;
            sp.fr[a] = pos - f;
        } else {
            sp.fl[a] = base;
            sp.fr[a] = (A)0;
        }
    }
}

// Calls f(flat_index_in_image, weight) for every in-bounds corner of the 2^DIM cell around the
// point.  deriv_axis >= 0 replaces that axis' interpolation weights by (-1, +1): the derivative
// of the interpolant with respect to that coordinate.  Integer-grid sampling (deformable ==
// false) touches the floor corner only.
template <int DIM, typename A, typename F>
__device__ __forceinline__ void for_each_corner(const Geo<DIM> &g, const SamplePoint<DIM, A> &sp, bool deformable,
                                                int deriv_axis, F &&f) {
#pragma unroll
    for (int c = 0; c < (1 << DIM); ++c) {
        if (!deformable && c != 0) break;
        bool valid = true;
        int flat = 0;
        A w = (A)1;
#pragma unroll
        for (int a = 0; a < DIM; ++a) {
            const int bit = (c >> (DIM - 1 - a)) & 1;
            const int idx = (int)((unsigned)sp.fl[a] + (unsigned)bit);  // wraps, never traps, on saturated floors
            valid = valid && ((unsigned)idx < (unsigned)g.img[a]);
            flat = flat * g.img[a] + idx;
            if (a == deriv_axis)
                w *= bit ? (A)1 : (A)-1;
            else
                w *= bit ? sp.fr[a] : ((A)1 - sp.fr[a]);
        }
        if (valid) f(flat, w);
    }
}

__device__ __forceinline__ void atomic_add(float *p, float v) { atomicAdd(p, v); }
__device__ __forceinline__ void atomic_add(double *p, double v) { atomicAdd(p, v); }

}  // namespace tvdcn_b200
