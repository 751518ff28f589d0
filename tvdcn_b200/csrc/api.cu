// C ABI (include/tvdcn_b200.h): validation, engine choice, workspace layout, kernel sequencing.
#include <cstdlib>
#include <atomic>
#include <cstdarg>
#include <cstdio>
#include <cstring>
#include <map>
#include <mutex>
#include <string>
#include <vector>

#include "../../include/tvdcn_b200.h"
#include "kernels.h"
#include "plan.h"
#include "sm100_ptx.cuh"

namespace tvdcn_b200 {

static std::atomic<uint64_t> g_launches{0};
void count_launch(int n) { g_launches.fetch_add((uint64_t)n, std::memory_order_relaxed); }

// ---- optional per-kernel timing (CUDA events on the launching stream) -----------------------------
struct TimedLaunch {
    const char *name;
    cudaEvent_t start, stop;
};
static std::atomic<int> g_timing{0};
static std::mutex g_timing_mu;
static std::vector<TimedLaunch> g_timed;

LaunchScope::LaunchScope(const char *name, cudaStream_t stream) : name_(name), stream_(stream) {
    count_launch();
    if (g_timing.load(std::memory_order_relaxed)) {
        if (cudaEventCreate(&start_) == cudaSuccess) cudaEventRecord(start_, stream_);
        else start_ = nullptr;
    }
}

LaunchScope::~LaunchScope() {
    if (start_ == nullptr) return;
    cudaEvent_t stop;
    if (cudaEventCreate(&stop) != cudaSuccess) { cudaEventDestroy(start_); return; }
    cudaEventRecord(stop, stream_);
    std::lock_guard<std::mutex> lk(g_timing_mu);
    g_timed.push_back({name_, start_, stop});
}

static thread_local char g_err[512] = "";

int fail(int code, const char *fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof(g_err), fmt, ap);
    va_end(ap);
    return code;
}

int cuda_fail(cudaError_t e, const char *what) {
    return fail(TVDCN_ERR_CUDA, "%s: %s", what, cudaGetErrorString(e));
}

static int64_t prod(const int64_t *v, int n) {
    int64_t r = 1;
    for (int i = 0; i < n; ++i) r *= v[i];
    return r;
}

int check_problem(const tvdcn_problem *p) {
    if (p == nullptr) return fail(TVDCN_ERR_INVALID, "problem is NULL");
    if (p->dim < 1 || p->dim > 3) return fail(TVDCN_ERR_INVALID, "dim must be 1, 2 or 3 (got %d)", p->dim);
    if (p->dtype < TVDCN_F32 || p->dtype > TVDCN_BF16) return fail(TVDCN_ERR_INVALID, "unknown dtype %d", p->dtype);
    if ((p->flags & ~TVDCN_FLAG_REUSE_STAGED_INPUT) != 0) return fail(TVDCN_ERR_INVALID, "unknown flags 0x%x", p->flags);
    const bool aux_ok = p->aux_dtype == p->dtype ||
                        (p->aux_dtype == TVDCN_F32 && (p->dtype == TVDCN_F16 || p->dtype == TVDCN_BF16));
    if (!aux_ok)
        return fail(TVDCN_ERR_INVALID, "aux_dtype must equal dtype, or be f32 beside a 16-bit dtype (got %d / %d)",
                    p->dtype, p->aux_dtype);
    if (p->batch < 0 || p->in_channels <= 0 || p->out_channels <= 0)
        return fail(TVDCN_ERR_INVALID, "batch / channel counts must be positive");
    if (p->groups <= 0 || p->in_channels % p->groups != 0 || p->out_channels % p->groups != 0)
        return fail(TVDCN_ERR_INVALID, "in_channels (%lld) and out_channels (%lld) must be divisible by groups (%d)",
                    (long long)p->in_channels, (long long)p->out_channels, p->groups);
    const int64_t cs = p->transposed ? p->out_channels : p->in_channels;
    if (p->offset_groups < 0 || (p->offset_groups > 0 && cs % p->offset_groups != 0))
        return fail(TVDCN_ERR_INVALID, "sampled channels (%lld) must be divisible by offset_groups (%d)",
                    (long long)cs, p->offset_groups);
    if (p->mask_groups < 0 || (p->mask_groups > 0 && cs % p->mask_groups != 0))
        return fail(TVDCN_ERR_INVALID, "sampled channels (%lld) must be divisible by mask_groups (%d)",
                    (long long)cs, p->mask_groups);
    for (int a = 0; a < p->dim; ++a) {
        if (p->kernel[a] <= 0 || p->stride[a] <= 0 || p->dilation[a] <= 0 || p->padding[a] < 0 ||
            p->in_size[a] <= 0)
            return fail(TVDCN_ERR_INVALID, "axis %d: kernel %d stride %d padding %d dilation %d in_size %lld", a,
                        p->kernel[a], p->stride[a], p->padding[a], p->dilation[a], (long long)p->in_size[a]);
        if (p->transposed && p->output_padding[a] < 0)
            return fail(TVDCN_ERR_INVALID, "axis %d: negative output_padding", a);
    }
    return TVDCN_OK;
}

static int check_sizes(const tvdcn_problem *p) {
    for (int a = 0; a < p->dim; ++a)
        if (p->out_size[a] <= 0)
            return fail(TVDCN_ERR_INVALID, "calculated output size too small (axis %d: %lld)", a,
                        (long long)p->out_size[a]);
    const int64_t lim = INT32_MAX;
    if (prod(p->in_size, p->dim) > lim || prod(p->out_size, p->dim) > lim ||
        p->batch * prod(p->in_size, p->dim) > (int64_t)1 << 40)
        return fail(TVDCN_ERR_UNSUPPORTED, "spatial extent exceeds 32-bit per-image indexing");
    if (p->batch > lim || p->in_channels > 1 << 20 || p->out_channels > 1 << 20)
        return fail(TVDCN_ERR_UNSUPPORTED, "batch / channel count too large");
    return TVDCN_OK;
}

GeoHost make_geo_host(const tvdcn_problem *p) {
    GeoHost g;
    memset(&g, 0, sizeof(g));
    g.dim = p->dim;
    g.B = (int)p->batch;
    g.Cs = (int)(p->transposed ? p->out_channels : p->in_channels);
    g.Cd = (int)(p->transposed ? p->in_channels : p->out_channels);
    g.groups = p->groups;
    g.og = p->offset_groups;
    g.mg = p->mask_groups;
    g.K = 1;
    g.S = 1;
    g.P = 1;
    for (int a = 0; a < p->dim; ++a) {
        g.img[a] = (int)(p->transposed ? p->out_size[a] : p->in_size[a]);
        g.grid[a] = (int)(p->transposed ? p->in_size[a] : p->out_size[a]);
        g.ker[a] = p->kernel[a];
        g.stride[a] = p->stride[a];
        g.pad[a] = p->padding[a];
        g.dil[a] = p->dilation[a];
        g.K *= g.ker[a];
        g.S *= g.img[a];
        g.P *= g.grid[a];
    }
    return g;
}

// One status word per device, living in the library's own device memory.
__device__ int g_tc_status;

int *device_status_word() {
    static int *cached[64] = {nullptr};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
    if (cached[dev] == nullptr) {
        void *addr = nullptr;
        if (cudaGetSymbolAddress(&addr, g_tc_status) != cudaSuccess) return nullptr;
        cached[dev] = (int *)addr;
    }
    return cached[dev];
}

// The channels-last copy of the sampled image is shared by every tensor-core kernel of one call; the entry
// points reset this marker, the first user stages the image.
static thread_local const void *t_staged_image = nullptr;

static cudaError_t stage_image(const tvdcn_problem *p, const GeoHost &g, const Plan &pl, const void *img, char *ws,
                               cudaStream_t stream) {
    if (t_staged_image == img) return cudaSuccess;
    const int es = p->dtype == TVDCN_F32 ? 4 : 2;
    cudaError_t e = launch_to_channels_last(img, ws + pl.img_cl, g.B, g.Cs, g.S, es, stream);
    // Row B*S of the staged image is all zeros: corners that fall outside the image (and the positions past the
    // end of the last tile) read it, so that an Inf or NaN elsewhere in the image cannot leak into results that
    // the reference computes without touching that pixel (0 x Inf = NaN).
    if (e == cudaSuccess)
        e = cudaMemsetAsync(ws + pl.img_cl + (size_t)g.B * g.S * g.Cs * es, 0, (size_t)g.Cs * es, stream);
    if (e == cudaSuccess) t_staged_image = img;
    return e;
}

// sample -> GEMM on the tensor cores: stage the image channels-last, pack the weights per tap, run.
static cudaError_t run_sample_gemm_tc(const tvdcn_problem *p, const GeoHost &g, const Plan &pl, const void *img,
                                      const void *weight, const void *offset, const void *mask, const void *bias,
                                      void *out, char *ws, cudaStream_t stream) {
    const int mode = tc_mode_of(p->dtype);
    int *status = device_status_word();
    if (status == nullptr) return cudaErrorInvalidDevice;
    void *w_hi = ws + pl.w_pack;
    void *w_lo = pl.w_pack_lo != NO_BUF ? (void *)(ws + pl.w_pack_lo) : nullptr;
    cudaError_t e = stage_image(p, g, pl, img, ws, stream);
    if (e != cudaSuccess) return e;
    e = launch_pack_weight_ks(weight, p->dtype, mode, g.groups, g.Cd / g.groups, g.Cs / g.groups, g.K, w_hi, w_lo,
                              stream);
    if (e != cudaSuccess) return e;
    return launch_sample_gemm_tc(g, mode, ws + pl.img_cl, w_hi, w_lo, (const float *)offset, (const float *)mask,
                                 (const float *)bias, out, status, stream);
}

// GEMM -> scatter / coordinate gradients on the tensor cores.  `img` (the sampled image) is needed only for
// goff / gmask; `scatter_out` (data type of the problem, [B, Cs, *img]) receives the scattered image plus
// `bias`; goff / gmask are f32 outputs that the caller has zeroed.
static cudaError_t run_gemm_scatter_tc(const tvdcn_problem *p, const GeoHost &g, const Plan &pl, const void *dense,
                                       const void *weight, const void *offset, const void *mask, const void *img,
                                       void *scatter_out, const void *bias, void *goff, void *gmask, char *ws,
                                       cudaStream_t stream) {
    const int mode = tc_mode_of(p->dtype);
    int *status = device_status_word();
    if (status == nullptr) return cudaErrorInvalidDevice;
    void *w_hi = ws + pl.w_pack_kd;
    void *w_lo = pl.w_pack_kd_lo != NO_BUF ? (void *)(ws + pl.w_pack_kd_lo) : nullptr;
    cudaError_t e = launch_pack_weight_kd(weight, p->dtype, mode, g.groups, g.Cd / g.groups, g.Cs / g.groups, g.K, w_hi, w_lo,
                              stream);
    if (e != cudaSuccess) return e;
    const bool want_coord = goff != nullptr || gmask != nullptr;
    if (want_coord) {
        e = stage_image(p, g, pl, img, ws, stream);
        if (e != cudaSuccess) return e;
    }
    float *acc = nullptr;
    if (scatter_out != nullptr) {
        acc = (float *)(ws + pl.img_grad_cl);
        e = cudaMemsetAsync(acc, 0, (size_t)g.B * g.S * g.Cs * sizeof(float), stream);
        if (e != cudaSuccess) return e;
    }
    e = launch_gemm_scatter_tc(g, mode, dense, w_hi, w_lo, want_coord ? ws + pl.img_cl : nullptr,
                               (const float *)offset, (const float *)mask, acc, (float *)goff, (float *)gmask, status,
                               stream);
    if (e != cudaSuccess) return e;
    if (scatter_out != nullptr)
        e = launch_from_channels_last_bias(acc, (const float *)bias, scatter_out, p->dtype, g.B, g.Cs, g.S, stream);
    return e;
}

// sampled weight gradient on the tensor cores; `gw_acc` is zero-initialised f32.  `dense_channel_sum` (f32, Cd
// values, may be NULL): wanted sum of the dense tensor over batch and space -- where the dense tensor is split into
// bf16 parts anyway (f32 data) the same pass takes it and `*summed` says so, else the caller runs channel_sum.
static cudaError_t run_sample_wgrad_tc(const tvdcn_problem *p, const GeoHost &g, const Plan &pl, const void *dense,
                                       const void *img, const void *offset, const void *mask, void *gw_acc, char *ws,
                                       cudaStream_t stream, float *dense_channel_sum = nullptr,
                                       bool *summed = nullptr) {
    const int mode = tc_mode_of(p->dtype);
    int *status = device_status_word();
    if (status == nullptr) return cudaErrorInvalidDevice;
    cudaError_t e = stage_image(p, g, pl, img, ws, stream);
    if (e != cudaSuccess) return e;
    const void *d_hi = dense, *d_lo = nullptr;
    if (summed) *summed = false;
    if (p->dtype == TVDCN_F32) {
        if (dense_channel_sum != nullptr &&
            can_split_f32_with_channel_sum((const float *)dense, ws + pl.dense_hi, ws + pl.dense_lo, g.P)) {
            e = launch_split_f32_channel_sum((const float *)dense, ws + pl.dense_hi, ws + pl.dense_lo, g.B, g.Cd, g.P,
                                             dense_channel_sum, stream);
            if (summed) *summed = true;
        } else {
            e = launch_split_f32((const float *)dense, ws + pl.dense_hi, ws + pl.dense_lo,
                                 (int64_t)g.B * g.Cd * g.P, stream);
        }
        if (e != cudaSuccess) return e;
        d_hi = ws + pl.dense_hi;
        d_lo = ws + pl.dense_lo;
    }
    return launch_sample_wgrad_tc(g, mode, d_hi, d_lo, ws + pl.img_cl, (const float *)offset, (const float *)mask,
                                  (float *)gw_acc, status, stream);
}

// Waits on a barrier that nothing arrives on, with a small poll limit, and reports the time-out the way the
// tensor-core kernels do.
__global__ void bounded_wait_selftest_kernel(int *status, uint32_t max_polls) {
    __shared__ uint64_t bar;
    if (threadIdx.x == 0) {
        ptx::mbar_init(&bar, 1);
        ptx::fence_mbar_init();
    }
    __syncthreads();
    bool done = false;
    for (uint32_t i = 0; i < max_polls && !done; ++i) done = ptx::mbar_try_wait(&bar, 0);
    if (!done && threadIdx.x == 0) atomicExch(status, 900);
}

// Copies a non-zero status word to host memory the device can write (mapped pinned memory): a store from a
// kernel, so the copy engines, which may be busy with a caller's own large transfers, are not involved.
__global__ void publish_status_kernel(const int *status, int *host_word) {
    const int v = *status;
    if (v != 0) *host_word = v;
}

}  // namespace tvdcn_b200

using namespace tvdcn_b200;

#define CUDA_TRY(expr)                                   \
    do {                                                 \
        cudaError_t e__ = (expr);                        \
        if (e__ != cudaSuccess) return cuda_fail(e__, #expr); \
    } while (0)

extern "C" {

int tvdcn_b200_problem_finalize(tvdcn_problem *p) {
    int rc = check_problem(p);
    if (rc) return rc;
    for (int a = 0; a < 3; ++a) p->out_size[a] = 1;
    for (int a = 0; a < p->dim; ++a) {
        const int64_t in = p->in_size[a], k = p->kernel[a], s = p->stride[a], pd = p->padding[a],
                      d = p->dilation[a];
        if (!p->transposed) {
            const int64_t num = in + 2 * pd - (d * (k - 1) + 1);
            p->out_size[a] = num < 0 ? 0 : num / s + 1;
        } else {
            p->out_size[a] = (in - 1) * s - 2 * pd + d * (k - 1) + 1 + p->output_padding[a];
        }
    }
    for (int a = p->dim; a < 3; ++a) p->in_size[a] = 1;
    return check_sizes(p);
}

size_t tvdcn_b200_forward_workspace_bytes(const tvdcn_problem *p) {
    if (check_problem(p) || check_sizes(p)) return 0;
    return plan_forward(p).total;
}

size_t tvdcn_b200_backward_workspace_bytes(const tvdcn_problem *p) {
    if (check_problem(p) || check_sizes(p)) return 0;
    return plan_backward(p, true, true, true, true).total;
}

const char *tvdcn_b200_engine_name(const tvdcn_problem *p, int backward) {
    if (check_problem(p) || check_sizes(p)) return "invalid";
    const Plan pl = backward ? plan_backward(p, true, true, true, true) : plan_forward(p);
    return pl.tensor ? "tcgen05" : "simt";
}

static int check_ws(const Plan &pl, void *ws, size_t bytes) {
    if (pl.total == 0) return TVDCN_OK;
    if (ws == nullptr || bytes < pl.total)
        return fail(TVDCN_ERR_WORKSPACE, "workspace of %zu bytes required, %zu given", pl.total, bytes);
    if (reinterpret_cast<uintptr_t>(ws) % 256 != 0)
        return fail(TVDCN_ERR_WORKSPACE, "workspace must be 256-byte aligned");
    return TVDCN_OK;
}

int tvdcn_b200_deform_conv_forward(const tvdcn_problem *p, const void *input, const void *weight,
                                   const void *offset, const void *mask, const void *bias, void *output,
                                   void *workspace, size_t workspace_bytes, void *cuda_stream) {
    int rc = check_problem(p);
    if (rc) return rc;
    rc = check_sizes(p);
    if (rc) return rc;
    if (p->batch == 0) return TVDCN_OK;  // nothing to compute; empty tensors may have NULL storage
    if (input == nullptr || weight == nullptr || output == nullptr)
        return fail(TVDCN_ERR_INVALID, "input, weight and output must not be NULL");
    if ((p->offset_groups > 0) != (offset != nullptr))
        return fail(TVDCN_ERR_INVALID, "offset pointer and offset_groups disagree");
    if ((p->mask_groups > 0) != (mask != nullptr))
        return fail(TVDCN_ERR_INVALID, "mask pointer and mask_groups disagree");
    cudaStream_t stream = (cudaStream_t)cuda_stream;
    const Plan pl = plan_forward(p);
    if (p->engine == TVDCN_ENGINE_TENSOR && !pl.tensor)
        return fail(TVDCN_ERR_UNSUPPORTED, "shape not covered by the tensor-core kernels: %s", pl.why_not);
    rc = check_ws(pl, workspace, workspace_bytes);
    if (rc) return rc;
    char *ws = (char *)workspace;
    t_staged_image = nullptr;
    const GeoHost g = make_geo_host(p);
    const int dt = p->dtype, aux = p->aux_dtype;

    if (pl.tc_sg) {
        CUDA_TRY(run_sample_gemm_tc(p, g, pl, input, weight, offset, mask, bias, output, ws, stream));
        return TVDCN_OK;
    }

    if (!p->transposed) {
        CUDA_TRY(launch_sample_gemm(g, dt, aux, input, weight, offset, mask, bias, output, stream));
        return TVDCN_OK;
    }
    if (pl.tc_gs) {
        CUDA_TRY(run_gemm_scatter_tc(p, g, pl, input, weight, offset, mask, nullptr, output, bias, nullptr, nullptr, ws,
                                     stream));
        return TVDCN_OK;
    }
    // transposed: output (= sampled image) starts as the bias and receives the scatter
    const int64_t n_out = (int64_t)g.B * g.Cs * g.S;
    void *acc = pl.img_acc != NO_BUF ? (void *)(ws + pl.img_acc) : output;
    CUDA_TRY(launch_fill_bias(dt, aux, bias, g.B, g.Cs, g.S, acc, stream));
    CUDA_TRY(launch_gemm_scatter(g, dt, aux, input, weight, offset, mask, nullptr, acc, nullptr, nullptr, stream));
    if (pl.img_acc != NO_BUF) CUDA_TRY(launch_cast_from_acc(dt, acc, output, n_out, stream));
    return TVDCN_OK;
}

// Side stream of the backward pass: the weight-gradient kernel and the bias sum do not depend on the scatter
// kernel, so they run beside it and fill the SMs that the scatter kernel's last, partial wave of CTAs leaves
// idle.  One stream and two events per host thread and device, created on first use and kept; fork and join are
// event waits, so the caller's stream still orders the whole call (and a capture of it picks both streams up).
// TVDCN_B200_OVERLAP=0 keeps everything on the caller's stream, and so does tvdcn_b200_timing_enable(1).
struct SideStream {
    cudaStream_t stream = nullptr;
    cudaEvent_t fork = nullptr, join = nullptr;
    bool tried = false;
};
static SideStream *side_stream() {
    static thread_local SideStream per_device[64];
    static const bool enabled = [] {
        const char *v = getenv("TVDCN_B200_OVERLAP");
        return v == nullptr || v[0] != '0';
    }();
    // per-kernel timing wants every kernel alone on the GPU
    if (!enabled || g_timing.load(std::memory_order_relaxed)) return nullptr;
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
    SideStream &s = per_device[dev];
    if (!s.tried) {
        s.tried = true;
        // highest priority: the weight-gradient CTAs take the SMs the scatter kernel frees first, so the weight
        // gradient is complete early in the call and its all-reduce can run under the rest of the scatter
        int least = 0, greatest = 0;
        (void)cudaDeviceGetStreamPriorityRange(&least, &greatest);
        if (cudaStreamCreateWithPriority(&s.stream, cudaStreamNonBlocking, greatest) != cudaSuccess ||
            cudaEventCreateWithFlags(&s.fork, cudaEventDisableTiming) != cudaSuccess ||
            cudaEventCreateWithFlags(&s.join, cudaEventDisableTiming) != cudaSuccess) {
            s.stream = nullptr;
            (void)cudaGetLastError();
        }
    }
    return s.stream != nullptr ? &s : nullptr;
}

int tvdcn_b200_deform_conv_backward(const tvdcn_problem *p, const void *grad_output, const void *input,
                                    const void *weight, const void *offset, const void *mask, void *grad_input,
                                    void *grad_weight, void *grad_offset, void *grad_mask, void *grad_bias,
                                    void *workspace, size_t workspace_bytes, void *cuda_stream) {
    return tvdcn_b200_deform_conv_backward_ex(p, grad_output, input, weight, offset, mask, grad_input, grad_weight,
                                              grad_offset, grad_mask, grad_bias, workspace, workspace_bytes,
                                              cuda_stream, nullptr);
}

int tvdcn_b200_deform_conv_backward_ex(const tvdcn_problem *p, const void *grad_output, const void *input,
                                       const void *weight, const void *offset, const void *mask, void *grad_input,
                                       void *grad_weight, void *grad_offset, void *grad_mask, void *grad_bias,
                                       void *workspace, size_t workspace_bytes, void *cuda_stream,
                                       void *weight_grad_ready) {
    int rc = check_problem(p);
    if (rc) return rc;
    rc = check_sizes(p);
    if (rc) return rc;
    cudaStream_t stream = (cudaStream_t)cuda_stream;
    const GeoHost g = make_geo_host(p);
    const int dt = p->dtype, aux = p->aux_dtype;
    const size_t es = dtype_size(dt), as = dtype_size(aux);
    const int64_t n_w = (int64_t)g.Cd * (g.Cs / g.groups) * g.K;
    const int64_t n_off = (int64_t)g.B * g.og * g.K * g.dim * g.P;
    const int64_t n_mask = (int64_t)g.B * g.mg * g.K * g.P;
    const int64_t n_img = (int64_t)g.B * g.Cs * g.S;
    const int64_t n_dense = (int64_t)g.B * g.Cd * g.P;
    if (p->batch == 0) {
        if (grad_weight) CUDA_TRY(cudaMemsetAsync(grad_weight, 0, n_w * es, stream));
        if (grad_bias) CUDA_TRY(cudaMemsetAsync(grad_bias, 0, (size_t)p->out_channels * as, stream));
        if (weight_grad_ready) CUDA_TRY(cudaEventRecord((cudaEvent_t)weight_grad_ready, stream));
        return TVDCN_OK;  // empty batch: the sums over the batch are zero, empty tensors may be NULL
    }
    if (grad_output == nullptr || input == nullptr || weight == nullptr)
        return fail(TVDCN_ERR_INVALID, "grad_output, input and weight must not be NULL");
    if ((p->offset_groups > 0) != (offset != nullptr))
        return fail(TVDCN_ERR_INVALID, "offset pointer and offset_groups disagree");
    if ((p->mask_groups > 0) != (mask != nullptr))
        return fail(TVDCN_ERR_INVALID, "mask pointer and mask_groups disagree");
    if (grad_offset != nullptr && offset == nullptr)
        return fail(TVDCN_ERR_INVALID, "grad_offset requested without offset");
    if (grad_mask != nullptr && mask == nullptr) return fail(TVDCN_ERR_INVALID, "grad_mask requested without mask");
    const Plan pl = plan_backward(p, grad_input != nullptr, grad_weight != nullptr, grad_offset != nullptr,
                                  grad_mask != nullptr);
    if (p->engine == TVDCN_ENGINE_TENSOR && !pl.tensor)
        return fail(TVDCN_ERR_UNSUPPORTED, "shape not covered by the tensor-core kernels: %s", pl.why_not);
    rc = check_ws(pl, workspace, workspace_bytes);
    if (rc) return rc;
    char *ws = (char *)workspace;
    // the caller may vouch that the forward call's staging of `input` is still at the start of this workspace
    // (only where the forward call for this problem stages the image at all, and at the same offset)
    t_staged_image = nullptr;
    if ((p->flags & TVDCN_FLAG_REUSE_STAGED_INPUT) && !p->transposed && pl.tensor) {
        const Plan fwd = plan_forward(p);
        if (fwd.img_cl != NO_BUF && fwd.img_cl == pl.img_cl) t_staged_image = input;
    }

    const size_t acs = dtype_size(acc_dtype(dt));
    // accumulation targets: the outputs themselves when they already have the accumulation type
    void *gw_acc = grad_weight ? (pl.gw_acc != NO_BUF ? (void *)(ws + pl.gw_acc) : grad_weight) : nullptr;
    void *goff_acc = grad_offset ? (pl.goff_acc != NO_BUF ? (void *)(ws + pl.goff_acc) : grad_offset) : nullptr;
    void *gmask_acc = grad_mask ? (pl.gmask_acc != NO_BUF ? (void *)(ws + pl.gmask_acc) : grad_mask) : nullptr;
    if (gw_acc) CUDA_TRY(cudaMemsetAsync(gw_acc, 0, n_w * acs, stream));
    if (goff_acc) CUDA_TRY(cudaMemsetAsync(goff_acc, 0, n_off * acs, stream));
    if (gmask_acc) CUDA_TRY(cudaMemsetAsync(gmask_acc, 0, n_mask * acs, stream));

    // The weight-gradient kernel reads 16-bit dense tensors by TMA straight from the caller's pointer, which must
    // then sit on a 16-byte boundary (a tensor view with a storage offset may not): the SIMT kernel takes over.
    const void *dense_for_w = p->transposed ? input : grad_output;
    const bool tc_sw = pl.tc_sw && (p->dtype == TVDCN_F32 || (reinterpret_cast<uintptr_t>(dense_for_w) & 15) == 0);

    // the tensor-core weight-gradient kernel accumulates in a staged layout: convert right behind it
    // (for conv with f32 data and f32 bias the split of grad_output also takes grad_bias)
    bool bias_summed = false;
    auto wgrad_tc = [&](const void *dense, const void *img, cudaStream_t st) -> cudaError_t {
        float *sum_out = (!p->transposed && grad_bias != nullptr && aux == TVDCN_F32) ? (float *)grad_bias : nullptr;
        cudaError_t e = run_sample_wgrad_tc(p, g, pl, dense, img, offset, mask, gw_acc, ws, st, sum_out, &bias_summed);
        if (e != cudaSuccess) return e;
        return launch_unpack_weight_grad((const float *)gw_acc, grad_weight, dt, g.groups, g.Cd / g.groups,
                                         g.Cs / g.groups, g.K, st);
    };

    // fork: weight gradient + bias sum on the side stream when both sides run on the tensor cores
    SideStream *side = (tc_sw && gw_acc && (pl.tc_gs || pl.tc_sg)) ? side_stream() : nullptr;
    cudaStream_t wstream = stream;
    if (side != nullptr) {
        CUDA_TRY(stage_image(p, g, pl, p->transposed ? grad_output : input, ws, stream));
        CUDA_TRY(cudaEventRecord(side->fork, stream));
        CUDA_TRY(cudaStreamWaitEvent(side->stream, side->fork, 0));
        wstream = side->stream;
    }

    if (!p->transposed) {
        // sampled image = input, dense = grad_output
        void *gi_acc = grad_input ? (pl.img_acc != NO_BUF ? (void *)(ws + pl.img_acc) : grad_input) : nullptr;
        if (side != nullptr) {
            CUDA_TRY(wgrad_tc(grad_output, input, wstream));
            if (grad_bias && !bias_summed)
                CUDA_TRY(launch_channel_sum(dt, aux, grad_output, g.B, g.Cd, g.P, grad_bias, wstream));
        }
        if (pl.tc_gs) {
            CUDA_TRY(run_gemm_scatter_tc(p, g, pl, grad_output, weight, offset, mask, input, grad_input, nullptr,
                                         goff_acc, gmask_acc, ws, stream));
            gi_acc = nullptr;
        } else {
            if (gi_acc) CUDA_TRY(cudaMemsetAsync(gi_acc, 0, n_img * acs, stream));
            if (gi_acc || goff_acc || gmask_acc)
                CUDA_TRY(launch_gemm_scatter(g, dt, aux, grad_output, weight, offset, mask, input, gi_acc, goff_acc,
                                             gmask_acc, stream));
        }
        if (side != nullptr) {
            // already queued beside the scatter kernel
        } else if (gw_acc && tc_sw)
            CUDA_TRY(wgrad_tc(grad_output, input, stream));
        else if (gw_acc)
            CUDA_TRY(launch_sample_wgrad(g, dt, aux, grad_output, input, offset, mask, gw_acc, stream));
        if (grad_bias && side == nullptr && !bias_summed)
            CUDA_TRY(launch_channel_sum(dt, aux, grad_output, g.B, g.Cd, g.P, grad_bias, stream));
        if (gi_acc && pl.img_acc != NO_BUF) CUDA_TRY(launch_cast_from_acc(dt, gi_acc, grad_input, n_img, stream));
    } else {
        // sampled image = grad_output, dense = input
        if (side != nullptr) {
            CUDA_TRY(wgrad_tc(input, grad_output, wstream));
            if (grad_bias) CUDA_TRY(launch_channel_sum(dt, aux, grad_output, g.B, g.Cs, g.S, grad_bias, wstream));
        }
        if ((goff_acc || gmask_acc) && pl.tc_gs)
            CUDA_TRY(run_gemm_scatter_tc(p, g, pl, input, weight, offset, mask, grad_output, nullptr, nullptr, goff_acc,
                                         gmask_acc, ws, stream));
        else if (goff_acc || gmask_acc)
            CUDA_TRY(launch_gemm_scatter(g, dt, aux, input, weight, offset, mask, grad_output, nullptr, goff_acc,
                                         gmask_acc, stream));
        if (grad_input && pl.tc_sg)
            CUDA_TRY(run_sample_gemm_tc(p, g, pl, grad_output, weight, offset, mask, nullptr, grad_input, ws, stream));
        else if (grad_input)
            CUDA_TRY(launch_sample_gemm(g, dt, aux, grad_output, weight, offset, mask, nullptr, grad_input, stream));
        if (side != nullptr) {
            // already queued beside the other kernels
        } else if (gw_acc && tc_sw)
            CUDA_TRY(wgrad_tc(input, grad_output, stream));
        else if (gw_acc)
            CUDA_TRY(launch_sample_wgrad(g, dt, aux, input, grad_output, offset, mask, gw_acc, stream));
        if (grad_bias && side == nullptr)
            CUDA_TRY(launch_channel_sum(dt, aux, grad_output, g.B, g.Cs, g.S, grad_bias, stream));
        (void)n_dense;
    }
    // grad_weight / grad_bias are final on the side stream: the tensor-core kernel's staged sum is converted there
    const bool gw_in_place = true;
    if (side != nullptr) {  // join
        if (weight_grad_ready && gw_in_place)
            CUDA_TRY(cudaEventRecord((cudaEvent_t)weight_grad_ready, side->stream));
        CUDA_TRY(cudaEventRecord(side->join, side->stream));
        CUDA_TRY(cudaStreamWaitEvent(stream, side->join, 0));
    }
    if (gw_acc && pl.gw_acc != NO_BUF && !tc_sw) CUDA_TRY(launch_cast_from_acc(dt, gw_acc, grad_weight, n_w, stream));
    if (weight_grad_ready && !(side != nullptr && gw_in_place))
        CUDA_TRY(cudaEventRecord((cudaEvent_t)weight_grad_ready, stream));
    if (goff_acc && pl.goff_acc != NO_BUF) CUDA_TRY(launch_cast_from_acc(aux, goff_acc, grad_offset, n_off, stream));
    if (gmask_acc && pl.gmask_acc != NO_BUF)
        CUDA_TRY(launch_cast_from_acc(aux, gmask_acc, grad_mask, n_mask, stream));
    return TVDCN_OK;
}

int tvdcn_b200_mask_softmax_forward(int32_t dtype, int64_t batch, int64_t mask_groups, int64_t taps,
                                    int64_t spatial, const void *in, void *out, void *cuda_stream) {
    if (dtype < TVDCN_F32 || dtype > TVDCN_BF16) return fail(TVDCN_ERR_INVALID, "unknown dtype %d", dtype);
    if (batch < 0 || mask_groups <= 0 || taps <= 0 || spatial < 0 || taps > INT32_MAX)
        return fail(TVDCN_ERR_INVALID, "mask_softmax: bad extents");
    if (batch * spatial == 0) return TVDCN_OK;
    if (in == nullptr || out == nullptr) return fail(TVDCN_ERR_INVALID, "mask_softmax: NULL pointer");
    CUDA_TRY(launch_mask_softmax_fwd(dtype, batch * mask_groups, (int)taps, spatial, in, out,
                                     (cudaStream_t)cuda_stream));
    return TVDCN_OK;
}

int tvdcn_b200_mask_softmax_backward(int32_t dtype, int64_t batch, int64_t mask_groups, int64_t taps,
                                     int64_t spatial, const void *grad_out, const void *out, void *grad_in,
                                     void *cuda_stream) {
    if (dtype < TVDCN_F32 || dtype > TVDCN_BF16) return fail(TVDCN_ERR_INVALID, "unknown dtype %d", dtype);
    if (batch < 0 || mask_groups <= 0 || taps <= 0 || spatial < 0 || taps > INT32_MAX)
        return fail(TVDCN_ERR_INVALID, "mask_softmax: bad extents");
    if (batch * spatial == 0) return TVDCN_OK;
    if (grad_out == nullptr || out == nullptr || grad_in == nullptr)
        return fail(TVDCN_ERR_INVALID, "mask_softmax: NULL pointer");
    CUDA_TRY(launch_mask_softmax_bwd(dtype, batch * mask_groups, (int)taps, spatial, grad_out, out, grad_in,
                                     (cudaStream_t)cuda_stream));
    return TVDCN_OK;
}

int tvdcn_b200_selftest_bounded_wait(int max_polls, void *cuda_stream) {
    if (max_polls < 1 || max_polls > 4096) return fail(TVDCN_ERR_INVALID, "max_polls must be in [1, 4096]");
    int *status = device_status_word();
    if (status == nullptr) return fail(TVDCN_ERR_CUDA, "status word not found");
    count_launch();
    bounded_wait_selftest_kernel<<<1, 32, 0, (cudaStream_t)cuda_stream>>>(status, (uint32_t)max_polls);
    CUDA_TRY(cudaGetLastError());
    return TVDCN_OK;
}

int tvdcn_b200_cuda_version(void) { return CUDART_VERSION; }

const char *tvdcn_b200_cuda_arch_flags(void) { return "sm_100a"; }

const char *tvdcn_b200_last_error(void) { return g_err; }

void tvdcn_b200_timing_enable(int on) { g_timing.store(on ? 1 : 0, std::memory_order_relaxed); }

size_t tvdcn_b200_timing_report(char *buf, size_t cap) {
    std::vector<TimedLaunch> taken;
    {
        std::lock_guard<std::mutex> lk(g_timing_mu);
        taken.swap(g_timed);
    }
    struct Agg { uint64_t n = 0; double ms = 0; };
    std::map<std::string, Agg> agg;
    for (auto &t : taken) {
        float ms = 0.f;
        if (cudaEventSynchronize(t.stop) == cudaSuccess && cudaEventElapsedTime(&ms, t.start, t.stop) == cudaSuccess) {
            Agg &a = agg[t.name];
            a.n += 1;
            a.ms += ms;
        }
        cudaEventDestroy(t.start);
        cudaEventDestroy(t.stop);
    }
    std::string out;
    for (auto &kv : agg) {
        char line[160];
        snprintf(line, sizeof(line), "%s %llu %.6f\n", kv.first.c_str(), (unsigned long long)kv.second.n, kv.second.ms);
        out += line;
    }
    if (buf != nullptr && cap > 0) {
        const size_t n = out.size() < cap - 1 ? out.size() : cap - 1;
        memcpy(buf, out.data(), n);
        buf[n] = 0;
    }
    return out.size();
}

int tvdcn_b200_device_status(void) {
    int *word = device_status_word();
    if (word == nullptr) return -1;
    if (cudaDeviceSynchronize() != cudaSuccess) return -1;
    int value = 0;
    if (cudaMemcpy(&value, word, sizeof(int), cudaMemcpyDeviceToHost) != cudaSuccess) return -1;
    if (value != 0) cudaMemset(word, 0, sizeof(int));
    return value;
}

const int *tvdcn_b200_device_status_address(void) { return device_status_word(); }

int tvdcn_b200_publish_status(int *host_word_device_ptr, void *cuda_stream) {
    if (host_word_device_ptr == nullptr) return fail(TVDCN_ERR_INVALID, "host_word_device_ptr is NULL");
    const int *status = device_status_word();
    if (status == nullptr) return fail(TVDCN_ERR_CUDA, "status word not found");
    publish_status_kernel<<<1, 1, 0, (cudaStream_t)cuda_stream>>>(status, host_word_device_ptr);
    CUDA_TRY(cudaGetLastError());
    return TVDCN_OK;
}

uint64_t tvdcn_b200_launch_count(void) { return g_launches.load(std::memory_order_relaxed); }

}  // extern "C"

// ---- forward without a caller-provided workspace ---------------------------------------------------------
// Scratch for tvdcn_b200_deform_conv_forward_static.  The array lives in this library's device image: every
// GPU that loads the library keeps these bytes until the process exits.  In host code the name below is only
// a handle for cudaGetSymbolAddress -- it is not a device address and must never be handed to a kernel.
#define TVDCN_STATIC_SCRATCH_BYTES (16u << 20)
static __device__ __align__(256) unsigned char g_static_scratch[TVDCN_STATIC_SCRATCH_BYTES];

// Device address of the scratch array on the current device; looked up once per device.
static cudaError_t static_scratch_address(void **out) {
    static void *cached[64] = {nullptr};
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return e;
    if (dev < 0 || dev >= 64) return cudaErrorInvalidDevice;
    if (cached[dev] == nullptr) {
        void *addr = nullptr;
        e = cudaGetSymbolAddress(&addr, g_static_scratch);
        if (e != cudaSuccess) return e;
        cached[dev] = addr;
    }
    *out = cached[dev];
    return cudaSuccess;
}

extern "C" {

size_t tvdcn_b200_static_scratch_bytes(void) { return TVDCN_STATIC_SCRATCH_BYTES; }

int tvdcn_b200_deform_conv_forward_static(const tvdcn_problem *p, const void *input, const void *weight,
                                          const void *offset, const void *mask, const void *bias, void *output,
                                          void *cuda_stream) {
    int rc = check_problem(p);
    if (rc) return rc;
    rc = check_sizes(p);
    if (rc) return rc;
    const size_t need = plan_forward(p).total;
    if (need > TVDCN_STATIC_SCRATCH_BYTES)
        return fail(TVDCN_ERR_WORKSPACE,
                    "this problem needs %zu bytes of scratch, more than the %u bytes built into the library; use "
                    "tvdcn_b200_deform_conv_forward with a workspace of your own",
                    need, (unsigned)TVDCN_STATIC_SCRATCH_BYTES);
    void *scratch = nullptr;
    if (need > 0) {
        const cudaError_t e = static_scratch_address(&scratch);
        if (e != cudaSuccess) return cuda_fail(e, "cudaGetSymbolAddress(static scratch)");
    }
    // The forward kernels overwrite every scratch byte they later read (staged image, packed weights) and
    // zero the scatter accumulator themselves, so nothing left by an earlier call can leak into this one.
    return tvdcn_b200_deform_conv_forward(p, input, weight, offset, mask, bias, output, scratch, need, cuda_stream);
}

}  // extern "C"
