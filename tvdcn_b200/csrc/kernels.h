// Host-side launchers of the device kernels (internal; the public surface is include/tvdcn_b200.h).
#pragma once

#include <cuda_runtime.h>
#include <stddef.h>
#include <stdint.h>

namespace tvdcn_b200 {

// Runtime-dimension geometry; converted to Geo<DIM> at launch.
struct GeoHost {
    int dim;
    int B, Cs, Cd, groups, og, mg, K, S, P;
    int img[3], grid[3], ker[3], stride[3], pad[3], dil[3];
};

enum : int { DT_F32 = 0, DT_F64 = 1, DT_F16 = 2, DT_BF16 = 3 };

inline size_t dtype_size(int dt) { return dt == DT_F64 ? 8 : (dt == DT_F32 ? 4 : 2); }
// accumulation type that goes with a data type: double for f64, float otherwise
inline int acc_dtype(int dt) { return dt == DT_F64 ? DT_F64 : DT_F32; }

void count_launch(int n = 1);

// Put one of these on the stack around a kernel launch: it counts the launch and, while kernel timing is
// switched on (tvdcn_b200_timing_enable), brackets it with CUDA events on the launching stream.
struct LaunchScope {
    LaunchScope(const char *name, cudaStream_t stream);
    ~LaunchScope();
    LaunchScope(const LaunchScope &) = delete;
    LaunchScope &operator=(const LaunchScope &) = delete;

   private:
    const char *name_;
    cudaStream_t stream_;
    cudaEvent_t start_ = nullptr;
};

// ---- generic SIMT kernels (generic.cu) -------------------------------------------------
// dense[b, d, p] = bias[d] + sum_{s', tap} W[d, s', tap] * mask * sample(img[b, s], pos)
cudaError_t launch_sample_gemm(const GeoHost &g, int dtype, int aux_dtype, const void *img, const void *weight,
                               const void *offset, const void *mask, const void *bias, void *dense_out,
                               cudaStream_t stream);

// col = W^T * dense per group, consumed in registers:
//   img_grad_acc[b, s, corners] += col * mask * corner weight          (if img_grad_acc)
//   goff_acc[b, og, tap, axis, p] += col * mask * d sample / d axis     (if goff_acc; needs img)
//   gmask_acc[b, mg, tap, p]      += col * sample(img)                  (if gmask_acc; needs img)
// The *_acc buffers have the accumulation type of dtype and must be initialised by the caller.
cudaError_t launch_gemm_scatter(const GeoHost &g, int dtype, int aux_dtype, const void *dense, const void *weight,
                                const void *offset, const void *mask, const void *img, void *img_grad_acc,
                                void *goff_acc, void *gmask_acc, cudaStream_t stream);

// gw_acc[d, s', tap] += sum_{b, p} dense[b, d, p] * mask * sample(img[b, s], pos)
cudaError_t launch_sample_wgrad(const GeoHost &g, int dtype, int aux_dtype, const void *dense, const void *img,
                                const void *offset, const void *mask, void *gw_acc, cudaStream_t stream);

// out[c] = sum_{b, s} x[b, c, s]; out has dtype out_dtype
cudaError_t launch_channel_sum(int dtype, int out_dtype, const void *x, int B, int C, int S, void *out,
                               cudaStream_t stream);

// dst[i] = (dst dtype) src[i]; src has the accumulation type of dst_dtype
cudaError_t launch_cast_from_acc(int dst_dtype, const void *src, void *dst, int64_t n, cudaStream_t stream);

// dst[b, c, s] = bias[c] (or 0 when bias == nullptr); dst has the accumulation type of dtype
cudaError_t launch_fill_bias(int dtype, int aux_dtype, const void *bias, int B, int C, int S, void *dst_acc,
                             cudaStream_t stream);

// ---- mask softmax (softmax.cu) -----------------------------------------------------------
cudaError_t launch_mask_softmax_fwd(int dtype, int64_t outer, int K, int64_t P, const void *in, void *out,
                                    cudaStream_t stream);
cudaError_t launch_mask_softmax_bwd(int dtype, int64_t outer, int K, int64_t P, const void *gout, const void *out,
                                    void *gin, cudaStream_t stream);

}  // namespace tvdcn_b200
