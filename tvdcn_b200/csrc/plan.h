// Engine choice and workspace layout of one forward / backward call (internal).
#pragma once

#include <cuda_runtime.h>
#include <stddef.h>

#include "../../include/tvdcn_b200.h"
#include "kernels.h"

namespace tvdcn_b200 {

constexpr size_t NO_BUF = (size_t)-1;

struct Plan {
    bool tensor = false;           // at least one primitive runs on the tensor-core (tcgen05) kernels
    bool tc_sg = false;            // sample -> GEMM on tensor cores
    bool tc_gs = false;            // GEMM -> scatter / coordinate gradients on tensor cores
    bool tc_sw = false;            // sampled weight gradient on tensor cores
    const char *why_not = "";      // reason the tensor-core kernels were not chosen
    size_t total = 0;              // workspace bytes
    // SIMT path: accumulation buffers for 16-bit outputs (byte offsets into the workspace)
    size_t img_acc = NO_BUF;       // sampled-image-shaped accumulator (grad_input / transposed output)
    size_t gw_acc = NO_BUF;        // f32 weight gradient: [Cd, csg, K] for the SIMT kernel, [g][tap][d'][s'] for the tensor-core one
    size_t goff_acc = NO_BUF;
    size_t gmask_acc = NO_BUF;
    // tensor path: staged copies
    size_t img_cl = NO_BUF;        // sampled image, channels-last (16-bit, or f32 in split mode)
    size_t w_pack = NO_BUF;        // weights packed [g][tap][d'][s'], 16-bit (hi part in split mode)
    size_t w_pack_lo = NO_BUF;     // low part of the split
    size_t w_pack_kd = NO_BUF;     // weights packed [g][tap][s'][d']
    size_t w_pack_kd_lo = NO_BUF;
    size_t dense_hi = NO_BUF;      // dense tensor, original layout, 16-bit hi / lo (split mode)
    size_t dense_lo = NO_BUF;
    size_t img_grad_cl = NO_BUF;   // f32 channels-last accumulator of the scatter
};

inline size_t align_up(size_t v, size_t a = 256) { return (v + a - 1) / a * a; }

Plan plan_forward(const tvdcn_problem *p);
Plan plan_backward(const tvdcn_problem *p, bool want_input, bool want_weight, bool want_offset, bool want_mask);

GeoHost make_geo_host(const tvdcn_problem *p);
int fail(int code, const char *fmt, ...);
int cuda_fail(cudaError_t e, const char *what);

// 0: bf16, 1: f16, 2: f32 split into bf16 hi + lo (the TC_* modes of the tensor-core kernels)
int tc_mode_of(int dtype);

// ---- tensor-core kernels (sm100_*.cu) -----------------------------------------------------------------
bool fwd_tc_config(int dim, int mode, int cdg, int *bn, int *stages);
cudaError_t launch_sample_gemm_tc(const GeoHost &g, int mode, const void *img_cl, const void *w_hi, const void *w_lo,
                                  const float *offset, const float *mask, const float *bias, void *out, int *status,
                                  cudaStream_t stream);
bool wgrad_tc_config(int dim, int mode, int cdg, int P, int *n_sub, int *m_tiles, int *stages);
cudaError_t launch_sample_wgrad_tc(const GeoHost &g, int mode, const void *dense_hi, const void *dense_lo,
                                   const void *img_cl, const float *offset, const float *mask, float *gw,
                                   int *status, cudaStream_t stream);
bool dgrad_tc_config(int dim, int mode, int cdg, int K, int *tb, int *nacc, int *b_stages);
cudaError_t launch_gemm_scatter_tc(const GeoHost &g, int mode, const void *dense, const void *w_kd_hi,
                                   const void *w_kd_lo, const void *img_cl, const float *offset, const float *mask,
                                   float *img_grad_cl, float *goff, float *gmask, int *status, cudaStream_t stream);
cudaError_t launch_from_channels_last_bias(const float *src, const float *bias, void *dst, int dst_dtype, int B, int C,
                                           int S, cudaStream_t stream);
cudaError_t launch_pack_weight_kd(const void *w, int dtype, int mode, int groups, int cdg, int csg, int K, void *hi,
                                  void *lo, cudaStream_t stream);
// staged weight gradient of the tensor-core kernel, [g][tap][d'][s'] f32 -> [Cd, csg, K] in the data type `dtype`
cudaError_t launch_unpack_weight_grad(const float *staged, void *gw, int dtype, int groups, int cdg, int csg, int K,
                                      cudaStream_t stream);
cudaError_t launch_split_f32(const float *src, void *hi, void *lo, int64_t n, cudaStream_t stream);
// the same split of a [B, C, S] tensor plus sum_out[c] = sum over batch and space, in one pass; only where
// can_split_f32_with_channel_sum says so (S a multiple of 4, pointers aligned for 16- / 8-byte accesses)
bool can_split_f32_with_channel_sum(const float *src, const void *hi, const void *lo, int S);
cudaError_t launch_split_f32_channel_sum(const float *src, void *hi, void *lo, int B, int C, int S, float *sum_out,
                                         cudaStream_t stream);
cudaError_t launch_to_channels_last(const void *src, void *dst, int B, int C, int S, int elem_bytes,
                                    cudaStream_t stream);
cudaError_t launch_pack_weight_ks(const void *w, int dtype, int mode, int groups, int cdg, int csg, int K, void *hi,
                                  void *lo, cudaStream_t stream);

int tuning_int(const char *name, int fallback);

// Address of the per-device status word the tensor-core kernels report failed bounded waits in.
int *device_status_word();

}  // namespace tvdcn_b200
