/*
 * tvdcn_b200 -- C ABI of the B200 (sm_100a) deformable-convolution path.
 *
 * Plain C: device pointers, sizes and a CUDA stream handle; no framework types.  Every tensor
 * is dense and laid out exactly as the reference operator receives it after its own
 * .contiguous() calls ([batch, channels, *spatial], spatial outermost-first, i.e. D,H,W).
 * All pointers are device pointers on the current CUDA device; all work is enqueued on the
 * given stream and nothing synchronises the host.
 *
 * The reference exposes this path as twelve dispatcher operators (tvdcn::deform_conv{1,2,3}d,
 * tvdcn::deform_conv_transpose{1,2,3}d and their _backward twins).  The dimension and the
 * "transposed" flag are fields of tvdcn_problem here, so one forward and one backward entry
 * point cover all twelve; the comments on each declaration name the reference functions it
 * replaces (paths inside the tvdcn project).
 *
 * Every function returns a tvdcn_status (0 = ok).  tvdcn_b200_last_error() returns a
 * human-readable message for the last failing call on the calling thread.
 */
#ifndef TVDCN_B200_H
#define TVDCN_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef enum tvdcn_dtype {
    TVDCN_F32 = 0,
    TVDCN_F64 = 1,
    TVDCN_F16 = 2,
    TVDCN_BF16 = 3
} tvdcn_dtype;

typedef enum tvdcn_status {
    TVDCN_OK = 0,
    TVDCN_ERR_INVALID = 1,      /* inconsistent problem description or null pointer      */
    TVDCN_ERR_UNSUPPORTED = 2,  /* legal for the reference but not implemented here      */
    TVDCN_ERR_WORKSPACE = 3,    /* workspace missing, misaligned or too small            */
    TVDCN_ERR_CUDA = 4,         /* a CUDA runtime call failed (message has the detail)   */
    TVDCN_ERR_DEVICE = 5        /* a kernel reported a failed bounded wait / self-check  */
} tvdcn_status;

/* Which implementation may be chosen for the GEMM-shaped parts. */
typedef enum tvdcn_engine {
    TVDCN_ENGINE_AUTO = 0,     /* tensor-core (tcgen05) kernels where the shape allows, else SIMT */
    TVDCN_ENGINE_SIMT = 1,     /* force the generic SIMT kernels (any shape, any dtype)            */
    TVDCN_ENGINE_TENSOR = 2    /* require the tensor-core kernels; TVDCN_ERR_UNSUPPORTED otherwise */
} tvdcn_engine;

/*
 * One deformable convolution (or transposed convolution) problem.
 * Fill everything except out_size, then call tvdcn_b200_problem_finalize().
 *
 * Channel-group conventions follow the reference: weight is
 *   conv:        [out_channels, in_channels / groups, *kernel]
 *   transposed:  [in_channels,  out_channels / groups, *kernel]
 * offset is [batch, offset_groups * taps * dim, *grid], channel order ((g * taps + tap) * dim + axis)
 * with axis 0 the outermost spatial axis; mask is [batch, mask_groups * taps, *grid].
 * "grid" is the output extent for the conv and the INPUT extent for the transposed op, and
 * offset/mask groups divide the channels of the sampled image (in_channels for the conv,
 * out_channels for the transposed op)
 * (tvdcn/csrc/ops/cuda/deform_conv2d_kernel.cpp:270-298,
 *  tvdcn/csrc/ops/cuda/deform_conv_transpose2d_kernel.cpp:223-266, :339-362).
 */
typedef struct tvdcn_problem {
    int32_t dim;               /* 1, 2 or 3 */
    int32_t transposed;        /* 0: deform_conv, 1: deform_conv_transpose */
    int32_t dtype;             /* tvdcn_dtype of input, weight, output and their gradients */
    int32_t aux_dtype;         /* tvdcn_dtype of offset, mask, bias and their gradients:
                                  equal to dtype, or TVDCN_F32 beside a 16-bit dtype */
    int64_t batch;
    int64_t in_channels;
    int64_t out_channels;
    int64_t in_size[3];        /* spatial extent of input, first `dim` entries used */
    int64_t out_size[3];       /* spatial extent of output (written by finalize)    */
    int32_t kernel[3];
    int32_t stride[3];
    int32_t padding[3];
    int32_t dilation[3];
    int32_t output_padding[3]; /* transposed only */
    int32_t groups;
    int32_t offset_groups;     /* 0: no offset tensor (integer-grid sampling) */
    int32_t mask_groups;       /* 0: no mask tensor (factor 1)                */
    int32_t engine;            /* tvdcn_engine */
    int32_t flags;             /* TVDCN_FLAG_* bits, 0 by default */
} tvdcn_problem;

/*
 * Backward only, deform_conv (not transposed): the workspace passed to this backward call is the one the forward
 * call for the same problem and the same `input` tensor ran with last, and nothing has written to it or to `input`
 * since.  The backward call then reuses the forward call's channels-last staging of `input` (it sits at the start of
 * both workspaces) instead of staging it again.  (No counterpart in the reference, which re-reads its inputs.)
 * The caller vouches for all of that; with the flag clear the backward call stages the input itself.
 * Ignored where no staging exists (SIMT kernels, transposed operator).
 */
#define TVDCN_FLAG_REUSE_STAGED_INPUT 1

/* Validates the description and computes out_size:
 *   conv        (in + 2p - (d(k-1)+1)) / s + 1     tvdcn/csrc/ops/cuda/deform_conv2d_kernel.cpp:167-168
 *   transposed  (in-1)s - 2p + d(k-1) + 1 + op     tvdcn/csrc/ops/cuda/deform_conv_transpose2d_kernel.cpp:172-173
 */
int tvdcn_b200_problem_finalize(tvdcn_problem *p);

/* Scratch bytes the forward / backward call needs for this problem (0 is possible).
 * The workspace must be 256-byte aligned.  Its contents need not be initialised. */
size_t tvdcn_b200_forward_workspace_bytes(const tvdcn_problem *p);
size_t tvdcn_b200_backward_workspace_bytes(const tvdcn_problem *p);

/*
 * Forward.  Replaces deform_conv{1,2,3}d_forward_kernel
 *   (tvdcn/csrc/ops/cuda/deform_conv1d_kernel.cpp:85-341, deform_conv2d_kernel.cpp:85-385,
 *    deform_conv3d_kernel.cpp:85-429) when p->transposed == 0 and
 * deform_conv_transpose{1,2,3}d_forward_kernel
 *   (tvdcn/csrc/ops/cuda/deform_conv_transpose1d_kernel.cpp, deform_conv_transpose2d_kernel.cpp:85-372,
 *    deform_conv_transpose3d_kernel.cpp) when p->transposed == 1.
 * offset / mask / bias may be NULL exactly when offset_groups / mask_groups are 0 / no bias.
 * output is fully overwritten.
 */
int tvdcn_b200_deform_conv_forward(const tvdcn_problem *p,
                                   const void *input, const void *weight,
                                   const void *offset, const void *mask, const void *bias,
                                   void *output,
                                   void *workspace, size_t workspace_bytes,
                                   void *cuda_stream);

/*
 * Forward for hosts that cannot give the library a workspace.  (No counterpart in the reference: its
 * operators allocate their column buffer through PyTorch on every call.)
 *
 * Some embedders own device memory but no allocator they may call at this point: an engine plugin that is
 * only handed input and output pointers, a runtime that carves one arena at start-up and forbids cudaMalloc
 * afterwards because it synchronises the device and fragments the arena, a host that must not allocate
 * between frames.  For them this entry point takes the same arguments as tvdcn_b200_deform_conv_forward
 * minus the workspace and uses a scratch array compiled into the library instead:
 * tvdcn_b200_static_scratch_bytes() bytes (16 MiB) of device memory that every GPU which loads the library
 * holds until the process exits.  It calls no cudaMalloc / cudaFree and no allocating library routine.
 *
 *  - A problem whose forward workspace (tvdcn_b200_forward_workspace_bytes) exceeds that size is refused with
 *    TVDCN_ERR_WORKSPACE and a message that names both sizes; nothing is launched.
 *  - The first call on each device looks up the array's device address (cudaGetSymbolAddress, with that
 *    device current).  Make that first call outside any stream capture.
 *  - All calls share the one array, and it keeps whatever the previous call left there.  The kernels
 *    rewrite everything they read from it, so consecutive calls on one stream are independent; two calls that
 *    overlap on the GPU (different streams, different threads) race on it and corrupt each other.
 *  - Results are those of tvdcn_b200_deform_conv_forward for the same problem.
 */
int tvdcn_b200_deform_conv_forward_static(const tvdcn_problem *p,
                                          const void *input, const void *weight,
                                          const void *offset, const void *mask, const void *bias,
                                          void *output, void *cuda_stream);
size_t tvdcn_b200_static_scratch_bytes(void);

/*
 * Backward.  Replaces deform_conv{1,2,3}d_backward_kernel
 *   (tvdcn/csrc/ops/cuda/deform_conv1d_kernel.cpp:343-559, deform_conv2d_kernel.cpp:387-642,
 *    deform_conv3d_kernel.cpp:431-725) and deform_conv_transpose{1,2,3}d_backward_kernel
 *   (tvdcn/csrc/ops/cuda/deform_conv_transpose2d_kernel.cpp:374-636 and its 1d/3d twins).
 * Every non-NULL gradient pointer is fully overwritten (no pre-zeroing needed); a NULL
 * gradient pointer skips that gradient.  grad_bias has out_channels elements.
 *
 * Streams: everything is ordered by cuda_stream.  When the tensor-core kernels run, the weight gradient and the
 * bias sum are queued on a second, library-owned stream that forks from cuda_stream and joins it again before
 * the call returns (event waits only, nothing blocks the host); work queued on cuda_stream after the call sees
 * all results.  The library creates that stream and its two events once per host thread and device, on the
 * first such call (make it outside any stream capture).  TVDCN_B200_OVERLAP=0 in the environment keeps all
 * kernels on cuda_stream.
 */
int tvdcn_b200_deform_conv_backward(const tvdcn_problem *p,
                                    const void *grad_output,
                                    const void *input, const void *weight,
                                    const void *offset, const void *mask,
                                    void *grad_input, void *grad_weight,
                                    void *grad_offset, void *grad_mask, void *grad_bias,
                                    void *workspace, size_t workspace_bytes,
                                    void *cuda_stream);

/* The same call with one more argument for data-parallel training: `weight_grad_ready`, a cudaEvent_t the caller
 * owns (or NULL), is recorded as soon as grad_weight and grad_bias hold their final values -- on the library's
 * second stream when it is in use, well before the input / offset / mask gradients are done -- so that the
 * all-reduce of the weight gradients can start under the rest of the backward pass.  No counterpart in the
 * reference (its backward, tvdcn/csrc/ops/cuda/deform_conv2d_kernel.cpp:387-642, has no streams and no
 * multi-GPU path). */
int tvdcn_b200_deform_conv_backward_ex(const tvdcn_problem *p,
                                       const void *grad_output,
                                       const void *input, const void *weight,
                                       const void *offset, const void *mask,
                                       void *grad_input, void *grad_weight,
                                       void *grad_offset, void *grad_mask, void *grad_bias,
                                       void *workspace, size_t workspace_bytes,
                                       void *cuda_stream, void *weight_grad_ready);

/*
 * Softmax over the `taps` kernel points of each mask group:
 *   mask viewed as [batch, mask_groups, taps, spatial], normalised along taps.
 * Replaces the torch.softmax call of mask_softmax{1,2,3}d
 *   (tvdcn/ops/activations/mask_softmax.py:19-49, 52-88, 91-126).
 */
int tvdcn_b200_mask_softmax_forward(int32_t dtype, int64_t batch, int64_t mask_groups,
                                    int64_t taps, int64_t spatial,
                                    const void *in, void *out, void *cuda_stream);

/* grad_in = out * (grad_out - sum_taps(grad_out * out)); autograd of the softmax above. */
int tvdcn_b200_mask_softmax_backward(int32_t dtype, int64_t batch, int64_t mask_groups,
                                     int64_t taps, int64_t spatial,
                                     const void *grad_out, const void *out, void *grad_in,
                                     void *cuda_stream);

/* CUDA runtime version the library was built with, and the architectures it carries.
 * Replace tvdcn::_cuda_version / tvdcn::_cuda_arch_flags (tvdcn/csrc/tvdcn.cpp:24-53). */
int tvdcn_b200_cuda_version(void);
const char *tvdcn_b200_cuda_arch_flags(void);

/* Message of the last failing call on this thread ("" if none). */
const char *tvdcn_b200_last_error(void);

/* Kernels with bounded waits (the tensor-core kernels wait on barriers) record a non-zero code in a
 * per-device status word when a wait runs out instead of hanging.  This call synchronises the current
 * device, returns the word (0 = no kernel reported a problem, -1 = the query itself failed) and clears it. */
int tvdcn_b200_device_status(void);

/* Device address of that status word on the current device (NULL if it cannot be found). */
const int *tvdcn_b200_device_status_address(void);

/* For a caller that must not synchronise: enqueues on `cuda_stream` a one-thread kernel that, if the status word is
 * non-zero, stores it to `host_word_device_ptr` -- the device-side address (cudaHostGetDevicePointer) of an int in
 * mapped pinned host memory that the caller zeroed.  The caller looks at the host int later.  A kernel store, not a
 * copy: it does not queue behind the caller's own transfers on the copy engines.  The PyTorch front end does this
 * after every operator call and raises at the next one.  No counterpart in the reference. */
int tvdcn_b200_publish_status(int *host_word_device_ptr, void *cuda_stream);

/* Self test of the bounded waits: launches, on `cuda_stream`, one small kernel that waits (at most `max_polls`
 * polls of about 20 microseconds, 1 <= max_polls <= 4096) on a barrier nothing ever arrives on, gives up and
 * records code 900 in the status word -- the path a real kernel takes when a wait runs out.  No counterpart in
 * the reference, whose kernels never wait. */
int tvdcn_b200_selftest_bounded_wait(int max_polls, void *cuda_stream);

/* Number of kernels this library has launched in this process so far (monotonic). */
uint64_t tvdcn_b200_launch_count(void);

/* Per-kernel timing for benchmarks.  While enabled, every kernel launch of this library is bracketed by
 * CUDA events on its stream.  tvdcn_b200_timing_report() waits for the recorded launches, writes one line
 * per kernel name, "name launches total_ms\n", into buf (NUL-terminated, truncated to cap), clears the
 * record and returns the untruncated length.  Do not enable it inside a stream capture. */
void tvdcn_b200_timing_enable(int on);
size_t tvdcn_b200_timing_report(char *buf, size_t cap);

/* Name of the engine that the forward / backward call would use for this problem
 * ("simt" or "tcgen05"); for tests and benchmarks. */
const char *tvdcn_b200_engine_name(const tvdcn_problem *p, int backward);

#ifdef __cplusplus
}
#endif
#endif /* TVDCN_B200_H */
