// Layout staging kernels around the GEMM -> scatter kernel: the f32 channels-last accumulator image goes back to
// the caller's [B, C, *spatial] layout (plus bias, in the destination type).
#include <type_traits>

#include "plan.h"
#include "sm100_common.cuh"

namespace tvdcn_b200 {

namespace {

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

// f32 [B, C, S] -> bf16 hi + lo (same layout) and, in the same pass, out[c] = sum over batch and space: one
// 1024-thread block per channel, warp w walks the images b = w, w + 32, ...; S is a multiple of 4 and the three
// pointers allow 16- / 8-byte accesses.  The sum is taken in a fixed order (no atomics).
__global__ void __launch_bounds__(1024) split_f32_channel_sum_kernel(const float *__restrict__ src,
                                                                     uint2 *__restrict__ hi, uint2 *__restrict__ lo,
                                                                     int B, int C, int S, float *__restrict__ out) {
    __shared__ float red[32];
    const int c = blockIdx.x;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int s4 = S / 4;
    float sum = 0.f;
    for (int b = warp; b < B; b += 32) {
        const int64_t row = ((int64_t)b * C + c) * (int64_t)s4;
        const float4 *in = reinterpret_cast<const float4 *>(src) + row;
        for (int i = lane; i < s4; i += 32) {
            const float4 v = __ldg(in + i);
            const float f[4] = {v.x, v.y, v.z, v.w};
            uint32_t h[4], l[4];
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                const __nv_bfloat16 hb = __float2bfloat16_rn(f[k]);
                h[k] = __bfloat16_as_ushort(hb);
                l[k] = __bfloat16_as_ushort(__float2bfloat16_rn(f[k] - __bfloat162float(hb)));
                sum += f[k];
            }
            hi[row + i] = make_uint2(h[0] | (h[1] << 16), h[2] | (h[3] << 16));
            lo[row + i] = make_uint2(l[0] | (l[1] << 16), l[2] | (l[3] << 16));
        }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
    if (lane == 0) red[warp] = sum;
    __syncthreads();
    if (warp == 0) {
        float v = red[lane];
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
        if (lane == 0) out[c] = v;
    }
}

}  // namespace

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

bool can_split_f32_with_channel_sum(const float *src, const void *hi, const void *lo, int S) {
    return S % 4 == 0 && (reinterpret_cast<uintptr_t>(src) & 15) == 0 &&
           ((reinterpret_cast<uintptr_t>(hi) | reinterpret_cast<uintptr_t>(lo)) & 7) == 0;
}

cudaError_t launch_split_f32_channel_sum(const float *src, void *hi, void *lo, int B, int C, int S, float *sum_out,
                                         cudaStream_t stream) {
    if (B <= 0 || C <= 0 || S <= 0) return cudaSuccess;
    LaunchScope scope("split_f32_channel_sum", stream);
    split_f32_channel_sum_kernel<<<C, 1024, 0, stream>>>(src, (uint2 *)hi, (uint2 *)lo, B, C, S, sum_out);
    return cudaGetLastError();
}

}  // namespace tvdcn_b200
