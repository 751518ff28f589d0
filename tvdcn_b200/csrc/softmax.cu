// mask_softmax: softmax over the K kernel taps of each mask group, tensor viewed as
// [outer = batch * mask_groups, K, P = spatial].  Replaces the strided torch.softmax of
// tvdcn/ops/activations/mask_softmax.py:78-88 with a single-pass, coalesced kernel: one thread
// owns VEC consecutive spatial positions and walks the K taps (stride P), keeping the K x VEC
// values in registers, so every element is read once and written once with full-width accesses.
#include <type_traits>

#include "common.cuh"
#include "kernels.h"

namespace tvdcn_b200 {
namespace {

template <typename T, int VEC>
struct alignas(sizeof(T) * VEC) Pack {
    T v[VEC];
};

template <typename T, int VEC>
__device__ __forceinline__ void load_pack(const T *p, acc_t<T> (&dst)[VEC]) {
    const Pack<T, VEC> pk = *reinterpret_cast<const Pack<T, VEC> *>(p);
#pragma unroll
    for (int i = 0; i < VEC; ++i) dst[i] = to_acc(pk.v[i]);
}

template <typename T, int VEC>
__device__ __forceinline__ void store_pack(T *p, const acc_t<T> (&src)[VEC]) {
    Pack<T, VEC> pk;
#pragma unroll
    for (int i = 0; i < VEC; ++i) store_acc(pk.v, i, src[i]);
    *reinterpret_cast<Pack<T, VEC> *>(p) = pk;
}

__device__ __forceinline__ float fast_exp(float x) { return __expf(x); }
__device__ __forceinline__ double fast_exp(double x) { return exp(x); }

// KMAX >= K: taps held in registers.
template <typename T, int VEC, int KMAX>
__global__ void __launch_bounds__(256)
softmax_fwd_reg_kernel(const T *__restrict__ in, T *__restrict__ out, int64_t outer, int K, int64_t P) {
    using A = acc_t<T>;
    const int64_t pv = P / VEC;  // vectors per row
    const int64_t total = outer * pv;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total;
         i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t o = i / pv;
        const int64_t p = (i % pv) * VEC;
        const int64_t base = o * K * P + p;
        A v[KMAX][VEC];
        A mx[VEC];
#pragma unroll
        for (int e = 0; e < VEC; ++e) mx[e] = -INFINITY;
#pragma unroll
        for (int k = 0; k < KMAX; ++k) {
            if (k < K) {
                load_pack<T, VEC>(in + base + (int64_t)k * P, v[k]);
#pragma unroll
                for (int e = 0; e < VEC; ++e) mx[e] = fmax(mx[e], v[k][e]);
            }
        }
        A sum[VEC];
#pragma unroll
        for (int e = 0; e < VEC; ++e) sum[e] = (A)0;
#pragma unroll
        for (int k = 0; k < KMAX; ++k) {
            if (k < K) {
#pragma unroll
                for (int e = 0; e < VEC; ++e) {
                    v[k][e] = fast_exp(v[k][e] - mx[e]);
                    sum[e] += v[k][e];
                }
            }
        }
#pragma unroll
        for (int e = 0; e < VEC; ++e) sum[e] = (A)1 / sum[e];
#pragma unroll
        for (int k = 0; k < KMAX; ++k) {
            if (k < K) {
#pragma unroll
                for (int e = 0; e < VEC; ++e) v[k][e] *= sum[e];
                store_pack<T, VEC>(out + base + (int64_t)k * P, v[k]);
            }
        }
    }
}

// Any K: three walks over the taps (the second and third hit cache).
template <typename T, int VEC>
__global__ void __launch_bounds__(256)
softmax_fwd_loop_kernel(const T *__restrict__ in, T *__restrict__ out, int64_t outer, int K, int64_t P) {
    using A = acc_t<T>;
    const int64_t pv = P / VEC;
    const int64_t total = outer * pv;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total;
         i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t o = i / pv;
        const int64_t p = (i % pv) * VEC;
        const int64_t base = o * K * P + p;
        A mx[VEC], sum[VEC], v[VEC];
#pragma unroll
        for (int e = 0; e < VEC; ++e) { mx[e] = -INFINITY; sum[e] = (A)0; }
        for (int k = 0; k < K; ++k) {
            load_pack<T, VEC>(in + base + (int64_t)k * P, v);
#pragma unroll
            for (int e = 0; e < VEC; ++e) mx[e] = fmax(mx[e], v[e]);
        }
        for (int k = 0; k < K; ++k) {
            load_pack<T, VEC>(in + base + (int64_t)k * P, v);
#pragma unroll
            for (int e = 0; e < VEC; ++e) sum[e] += fast_exp(v[e] - mx[e]);
        }
#pragma unroll
        for (int e = 0; e < VEC; ++e) sum[e] = (A)1 / sum[e];
        for (int k = 0; k < K; ++k) {
            load_pack<T, VEC>(in + base + (int64_t)k * P, v);
#pragma unroll
            for (int e = 0; e < VEC; ++e) v[e] = fast_exp(v[e] - mx[e]) * sum[e];
            store_pack<T, VEC>(out + base + (int64_t)k * P, v);
        }
    }
}

// grad_in = y * (g - sum_k g * y); y and g are each read twice (second read hits cache).
template <typename T, int VEC>
__global__ void __launch_bounds__(256)
softmax_bwd_kernel(const T *__restrict__ gout, const T *__restrict__ y, T *__restrict__ gin, int64_t outer, int K,
                   int64_t P) {
    using A = acc_t<T>;
    const int64_t pv = P / VEC;
    const int64_t total = outer * pv;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total;
         i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t o = i / pv;
        const int64_t p = (i % pv) * VEC;
        const int64_t base = o * K * P + p;
        A dot[VEC], a[VEC], b[VEC];
#pragma unroll
        for (int e = 0; e < VEC; ++e) dot[e] = (A)0;
        for (int k = 0; k < K; ++k) {
            load_pack<T, VEC>(gout + base + (int64_t)k * P, a);
            load_pack<T, VEC>(y + base + (int64_t)k * P, b);
#pragma unroll
            for (int e = 0; e < VEC; ++e) dot[e] += a[e] * b[e];
        }
        for (int k = 0; k < K; ++k) {
            load_pack<T, VEC>(gout + base + (int64_t)k * P, a);
            load_pack<T, VEC>(y + base + (int64_t)k * P, b);
#pragma unroll
            for (int e = 0; e < VEC; ++e) a[e] = b[e] * (a[e] - dot[e]);
            store_pack<T, VEC>(gin + base + (int64_t)k * P, a);
        }
    }
}

int blocks_for(int64_t total) {
    int64_t b = (total + 255) / 256;
    const int64_t cap = 148 * 8;
    return (int)(b < 1 ? 1 : (b > cap ? cap : b));
}

bool aligned(const void *p, size_t a) { return (reinterpret_cast<uintptr_t>(p) % a) == 0; }

template <typename T, int VEC>
cudaError_t fwd_vec(int64_t outer, int K, int64_t P, const T *in, T *out, cudaStream_t stream) {
    const int64_t total = outer * (P / VEC);
    const int blocks = blocks_for(total);
    LaunchScope scope("mask_softmax_fwd", stream);
    if (K <= 8)
        softmax_fwd_reg_kernel<T, VEC, 8><<<blocks, 256, 0, stream>>>(in, out, outer, K, P);
    else if (K <= 16)
        softmax_fwd_reg_kernel<T, VEC, 16><<<blocks, 256, 0, stream>>>(in, out, outer, K, P);
    else if (K <= 32)
        softmax_fwd_reg_kernel<T, VEC, 32><<<blocks, 256, 0, stream>>>(in, out, outer, K, P);
    else
        softmax_fwd_loop_kernel<T, VEC><<<blocks, 256, 0, stream>>>(in, out, outer, K, P);
    return cudaGetLastError();
}

template <typename T>
cudaError_t fwd_t(int64_t outer, int K, int64_t P, const void *in, void *out, cudaStream_t stream) {
    constexpr int VEC = 16 / sizeof(T) > 4 ? 4 : 16 / sizeof(T);  // f32: 4, 16-bit: 4, f64: 2
    if (P % VEC == 0 && aligned(in, sizeof(T) * VEC) && aligned(out, sizeof(T) * VEC))
        return fwd_vec<T, VEC>(outer, K, P, (const T *)in, (T *)out, stream);
    return fwd_vec<T, 1>(outer, K, P, (const T *)in, (T *)out, stream);
}

template <typename T>
cudaError_t bwd_t(int64_t outer, int K, int64_t P, const void *g, const void *y, void *gi, cudaStream_t stream) {
    constexpr int VEC = 16 / sizeof(T) > 4 ? 4 : 16 / sizeof(T);
    LaunchScope scope("mask_softmax_bwd", stream);
    if (P % VEC == 0 && aligned(g, sizeof(T) * VEC) && aligned(y, sizeof(T) * VEC) &&
        aligned(gi, sizeof(T) * VEC)) {
        const int blocks = blocks_for(outer * (P / VEC));
        softmax_bwd_kernel<T, VEC><<<blocks, 256, 0, stream>>>((const T *)g, (const T *)y, (T *)gi, outer, K, P);
    } else {
        const int blocks = blocks_for(outer * P);
        softmax_bwd_kernel<T, 1><<<blocks, 256, 0, stream>>>((const T *)g, (const T *)y, (T *)gi, outer, K, P);
    }
    return cudaGetLastError();
}

}  // namespace

cudaError_t launch_mask_softmax_fwd(int dtype, int64_t outer, int K, int64_t P, const void *in, void *out,
                                    cudaStream_t stream) {
    if (outer <= 0 || P <= 0) return cudaSuccess;
    switch (dtype) {
        case DT_F32: return fwd_t<float>(outer, K, P, in, out, stream);
        case DT_F64: return fwd_t<double>(outer, K, P, in, out, stream);
        case DT_F16: return fwd_t<__half>(outer, K, P, in, out, stream);
        case DT_BF16: return fwd_t<__nv_bfloat16>(outer, K, P, in, out, stream);
    }
    return cudaErrorInvalidValue;
}

cudaError_t launch_mask_softmax_bwd(int dtype, int64_t outer, int K, int64_t P, const void *gout, const void *out,
                                    void *gin, cudaStream_t stream) {
    if (outer <= 0 || P <= 0) return cudaSuccess;
    switch (dtype) {
        case DT_F32: return bwd_t<float>(outer, K, P, gout, out, gin, stream);
        case DT_F64: return bwd_t<double>(outer, K, P, gout, out, gin, stream);
        case DT_F16: return bwd_t<__half>(outer, K, P, gout, out, gin, stream);
        case DT_BF16: return bwd_t<__nv_bfloat16>(outer, K, P, gout, out, gin, stream);
    }
    return cudaErrorInvalidValue;
}

}  // namespace tvdcn_b200
