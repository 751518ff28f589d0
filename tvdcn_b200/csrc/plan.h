// Engine choice and workspace layout of one forward / backward call (internal).
#pragma once

#include <cuda_runtime.h>
#include <stddef.h>

#include "../../include/tvdcn_b200.h"
#include "kernels.h"

namespace tvdcn_b200 {

constexpr size_t NO_BUF = (size_t)-1;

struct Plan {
    bool tensor = false;           // tensor-core (tcgen05) kernels chosen
    const char *why_not = "";      // reason the tensor-core kernels were not chosen
    size_t total = 0;              // workspace bytes
    // SIMT path: accumulation buffers for 16-bit outputs (byte offsets into the workspace)
    size_t img_acc = NO_BUF;       // sampled-image-shaped accumulator (grad_input / transposed output)
    size_t gw_acc = NO_BUF;
    size_t goff_acc = NO_BUF;
    size_t gmask_acc = NO_BUF;
    // tensor path: staged copies (see sm100 kernels)
    size_t img_cl = NO_BUF;        // sampled image, channels-last, 16-bit (hi part in split mode)
    size_t img_cl_lo = NO_BUF;     // low part of the split
    size_t w_pack = NO_BUF;        // weights packed per (group, tap) K-major
    size_t w_pack_lo = NO_BUF;
    size_t dense_cl = NO_BUF;
    size_t dense_cl_lo = NO_BUF;
    size_t status = NO_BUF;        // device status word written by kernels with bounded waits
};

inline size_t align_up(size_t v, size_t a = 256) { return (v + a - 1) / a * a; }

Plan plan_forward(const tvdcn_problem *p);
Plan plan_backward(const tvdcn_problem *p, bool want_input, bool want_weight, bool want_offset, bool want_mask);

GeoHost make_geo_host(const tvdcn_problem *p);
int fail(int code, const char *fmt, ...);
int cuda_fail(cudaError_t e, const char *what);

// tensor-core path (sm100 kernels); only called when the plan says so
int tensor_forward(const tvdcn_problem *p, const GeoHost &g, const Plan &pl, const void *input, const void *weight,
                   const void *offset, const void *mask, const void *bias, void *output, char *ws,
                   cudaStream_t stream);
int tensor_backward(const tvdcn_problem *p, const GeoHost &g, const Plan &pl, const void *grad_output,
                    const void *input, const void *weight, const void *offset, const void *mask, void *grad_input,
                    void *grad_weight, void *grad_offset, void *grad_mask, void *grad_bias, char *ws,
                    cudaStream_t stream);

}  // namespace tvdcn_b200
