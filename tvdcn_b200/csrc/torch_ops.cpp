// PyTorch dispatcher front end: registers the tvdcn::* operators and forwards them to the C ABI.
//
// Schemas are the reference's, verbatim (tvdcn/csrc/ops/deform_conv2d.cpp:117-126,
// tvdcn/csrc/ops/deform_conv_transpose2d.cpp:125-136 and the 1d / 3d twins; tvdcn/csrc/tvdcn.cpp:50-53),
// so Python code and TorchScript graphs written against the reference bind to these kernels
// unchanged.  Keys: CUDA (forward and backward), Autograd (both) and Autocast (forward).  There
// is no CPU key: a CPU tensor raises the dispatcher's "no kernel" error.
//
// Differences from the reference front end, all deliberate:
//  * work is enqueued on the current CUDA stream (the reference launches on the legacy stream);
//  * absent offset / mask / bias are handled in autograd (the reference's Function crashes on
//    undefined tensors with recent torch);
//  * input and weight may be f16 / bf16 while offset, mask and bias stay f32;
//  * under autocast the input and weight are cast to the autocast dtype and offset, mask and bias
//    to f32 (the reference casts everything to f32: tvdcn/csrc/ops/autocast/deform_conv2d_kernel.cpp:19-30);
//  * the transposed forward checks weight.size(0) == input channels explicitly;
//  * tvdcn::mask_softmax{1,2,3}d are operators here (plain torch.softmax in the reference).
#include <ATen/ATen.h>
#include <ATen/autocast_mode.h>
#include <ATen/core/dispatch/Dispatcher.h>
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/autograd.h>
#include <torch/library.h>

#include <cuda_runtime.h>

#include <array>
#include <cstdlib>
#include <string>
#include <vector>

#include "../../include/tvdcn_b200.h"

namespace tvdcn_b200 {
namespace {

using at::Tensor;
using OptTensor = std::optional<at::Tensor>;
using torch::autograd::AutogradContext;
using torch::autograd::variable_list;

template <int D>
std::array<int64_t, D> ntuple(at::IntArrayRef x) {
    // a one-element list is broadcast, as tvdcn/csrc/ops/utils/ntuple.h:6-22 does
    std::array<int64_t, D> r{};
    if ((int)x.size() == D) {
        for (int i = 0; i < D; ++i) r[i] = x[i];
    } else if (x.size() == 1) {
        for (int i = 0; i < D; ++i) r[i] = x[0];
    } else {
        TORCH_CHECK(false, "Expected a sequence of ", D, " elements. Got ", x.size());
    }
    return r;
}

int to_dtype(at::ScalarType t, const char *op) {
    switch (t) {
        case at::kFloat: return TVDCN_F32;
        case at::kDouble: return TVDCN_F64;
        case at::kHalf: return TVDCN_F16;
        case at::kBFloat16: return TVDCN_BF16;
        default: TORCH_CHECK(false, "\"", op, "\" not implemented for '", c10::toString(t), "'");
    }
    return -1;
}

bool has(const OptTensor &t) { return t.has_value() && t->defined(); }

template <int D, bool TR>
std::string op_name() {
    return std::string("deform_conv") + (TR ? "_transpose" : "") + std::to_string(D) + "d";
}

template <int D>
std::string dims_str(const std::array<int64_t, D> &v) {
    std::string s;
    for (int i = 0; i < D; ++i) s += (i ? ", " : "") + std::to_string(v[i]);
    return s;
}

// Everything one call needs after validation.
struct Call {
    tvdcn_problem prob;
    Tensor input, weight, offset, mask, bias;  // contiguous, batched; undefined when absent
    bool unbatched = false;
};

// Argument checks of deform_conv{N}d_forward_kernel / deform_conv_transpose{N}d_forward_kernel
// (tvdcn/csrc/ops/cuda/deform_conv2d_kernel.cpp:95-268, deform_conv_transpose2d_kernel.cpp:95-266), messages kept.
template <int D, bool TR>
Call prepare(const Tensor &input, const Tensor &weight, const OptTensor &offset, const OptTensor &mask,
             const OptTensor &bias, at::IntArrayRef stride, at::IntArrayRef padding, at::IntArrayRef output_padding,
             at::IntArrayRef dilation, int64_t groups) {
    const std::string name = op_name<D, TR>();
    Call c;
    const bool deformable = has(offset), modulated = has(mask), with_bias = has(bias);
    c.unbatched = input.dim() == D + 1;

    TORCH_CHECK(input.is_cuda(), name, ": expected a CUDA tensor for input (this build has no CPU backend)");
    auto same_device = [&](const Tensor &t, const char *what) {
        TORCH_CHECK(t.is_cuda() && t.device() == input.device(), "Expected tensor for argument ", what,
                    " to be on the same device as input (", input.device(), "), but it is on ", t.device());
    };
    same_device(weight, "weight");
    if (deformable) same_device(*offset, "offset");
    if (modulated) same_device(*mask, "mask");
    if (with_bias) same_device(*bias, "bias");

    const auto dt = input.scalar_type();
    TORCH_CHECK(weight.scalar_type() == dt, "Expected tensor for argument weight to have the same type as tensor "
                "for argument input; but type ", weight.scalar_type(), " does not equal ", dt);
    const bool low = dt == at::kHalf || dt == at::kBFloat16;
    at::ScalarType aux = dt;
    bool aux_set = false;
    auto check_aux = [&](const Tensor &t, const char *what) {
        const auto tt = t.scalar_type();
        TORCH_CHECK(tt == dt || (low && tt == at::kFloat), "Expected tensor for argument ", what,
                    " to have the same type as input (", dt, ")", low ? " or Float" : "", "; got ", tt);
        TORCH_CHECK(!aux_set || tt == aux, "offset, mask and bias must share one dtype; got ", aux, " and ", tt);
        aux = tt;
        aux_set = true;
    };
    if (deformable) check_aux(*offset, "offset");
    if (modulated) check_aux(*mask, "mask");
    if (with_bias) check_aux(*bias, "bias");
    if (!aux_set && low) aux = at::kFloat;  // nothing constrains it; f32 keeps the tensor-core kernels eligible

    c.input = input.contiguous();
    c.weight = weight.contiguous();
    if (deformable) c.offset = offset->contiguous();
    if (modulated) c.mask = mask->contiguous();
    if (with_bias) c.bias = bias->contiguous();

    TORCH_CHECK(c.unbatched || c.input.dim() == D + 2, "Expected ", D + 1, "D (unbatched) or ", D + 2,
                "D (batched) input to ", name, ", but got input of size: ", c.input.sizes());
    TORCH_CHECK(c.weight.dim() == D + 2, "Expected ", D + 2, "D weight");
    TORCH_CHECK(!deformable || c.offset.dim() == (c.unbatched ? D + 1 : D + 2), "Expected ", D + 1,
                "D (unbatched) or ", D + 2, "D (batched) offset, but got offset of size: ",
                deformable ? c.offset.sizes() : at::IntArrayRef{});
    TORCH_CHECK(!modulated || c.mask.dim() == (c.unbatched ? D + 1 : D + 2), "Expected ", D + 1,
                "D (unbatched) or ", D + 2, "D (batched) mask, but got mask of size: ",
                modulated ? c.mask.sizes() : at::IntArrayRef{});
    if (c.unbatched) {
        c.input = c.input.unsqueeze(0);
        if (deformable) c.offset = c.offset.unsqueeze(0);
        if (modulated) c.mask = c.mask.unsqueeze(0);
    }

    const auto st = ntuple<D>(stride), pd = ntuple<D>(padding), dl = ntuple<D>(dilation);
    std::array<int64_t, D> op{};
    if (TR) op = ntuple<D>(output_padding);

    tvdcn_problem &p = c.prob;
    memset(&p, 0, sizeof(p));
    p.dim = D;
    p.transposed = TR ? 1 : 0;
    p.dtype = to_dtype(dt, name.c_str());
    p.aux_dtype = to_dtype(aux, name.c_str());
    p.batch = c.input.size(0);
    p.in_channels = c.input.size(1);
    p.out_channels = TR ? c.weight.size(1) * groups : c.weight.size(0);
    p.groups = (int32_t)groups;
    std::array<int64_t, D> ker{};
    int64_t taps = 1;
    for (int a = 0; a < D; ++a) {
        ker[a] = c.weight.size(2 + a);
        taps *= ker[a];
        p.in_size[a] = c.input.size(2 + a);
        p.kernel[a] = (int32_t)ker[a];
        p.stride[a] = (int32_t)st[a];
        p.padding[a] = (int32_t)pd[a];
        p.dilation[a] = (int32_t)dl[a];
        p.output_padding[a] = (int32_t)op[a];
    }
    for (int a = 0; a < D; ++a) TORCH_CHECK(ker[a] > 0, "weight kernel extents: (", dims_str<D>(ker), ")");
    for (int a = 0; a < D; ++a) TORCH_CHECK(st[a] > 0, "stride: (", dims_str<D>(st), ")");
    for (int a = 0; a < D; ++a) TORCH_CHECK(pd[a] >= 0, "padding: (", dims_str<D>(pd), ")");
    for (int a = 0; a < D; ++a) TORCH_CHECK(dl[a] > 0, "dilation: (", dims_str<D>(dl), ")");
    TORCH_CHECK(groups > 0, "groups must be positive");
    if (!TR) {
        TORCH_CHECK(c.weight.size(1) * groups == p.in_channels, "weight.size(1) * groups (", c.weight.size(1) * groups,
                    ") must equal the number of input channels (", p.in_channels, ")");
        TORCH_CHECK(c.weight.size(0) % groups == 0, "weight.size(0) must be divisible by groups");
    } else {
        TORCH_CHECK(c.weight.size(0) == p.in_channels, "weight.size(0) (", c.weight.size(0),
                    ") must equal the number of input channels (", p.in_channels, ")");
        TORCH_CHECK(c.weight.size(0) % groups == 0, "weight.size(0) must be divisible by groups");
    }

    const int64_t off_unit = D * taps;
    const int64_t offset_groups = deformable ? c.offset.size(1) / off_unit : 0;
    const int64_t mask_groups = modulated ? c.mask.size(1) / taps : 0;
    p.offset_groups = (int32_t)offset_groups;
    p.mask_groups = (int32_t)mask_groups;

    // output extent first (needed by the grid checks of the conv)
    std::array<int64_t, D> out{};
    for (int a = 0; a < D; ++a)
        out[a] = TR ? (p.in_size[a] - 1) * st[a] - 2 * pd[a] + dl[a] * (ker[a] - 1) + 1 + op[a]
                    : (p.in_size[a] + 2 * pd[a] - (dl[a] * (ker[a] - 1) + 1)) / st[a] + 1;
    std::array<int64_t, D> grid{};
    for (int a = 0; a < D; ++a) grid[a] = TR ? p.in_size[a] : out[a];
    const char *grid_what = TR ? "input dims" : "computed output dims";
    const char *own_what = TR ? "input dims" : "output dims";

    if (deformable) {
        TORCH_CHECK(c.offset.size(0) == c.input.size(0), "invalid batch size of offset");
        TORCH_CHECK(offset_groups > 0,
                    "The shape of the offset tensor at dimension 1 is not valid. It should be a multiple of ", D,
                    " * prod(weight.shape[2:]).\nGot offset.size(1)=", c.offset.size(1), ", while ", D,
                    " * prod(weight.shape[2:])=", off_unit);
        TORCH_CHECK(c.input.size(1) % offset_groups == 0, "input channels (", c.input.size(1),
                    ") must be divisible by offset_groups (", offset_groups, ")");
        TORCH_CHECK(c.offset.size(1) == offset_groups * off_unit, "offset.shape[1] is not valid. got: ",
                    c.offset.size(1), " expected: ", offset_groups * off_unit);
        std::array<int64_t, D> og{};
        bool ok = true;
        for (int a = 0; a < D; ++a) { og[a] = c.offset.size(2 + a); ok = ok && og[a] == grid[a]; }
        TORCH_CHECK(ok, "offset ", own_what, ": (", dims_str<D>(og), ") - ", grid_what, ": (", dims_str<D>(grid), ")");
    }
    if (modulated) {
        TORCH_CHECK(c.mask.size(0) == c.input.size(0), "invalid batch size of mask");
        TORCH_CHECK(mask_groups > 0,
                    "The shape of the mask tensor at dimension 1 is not valid. It should be a multiple of "
                    "prod(weight.shape[2:]).\nGot mask.size(1)=", c.mask.size(1), ", while prod(weight.shape[2:])=",
                    taps);
        TORCH_CHECK(c.input.size(1) % mask_groups == 0, "input channels (", c.input.size(1),
                    ") must be divisible by mask_groups (", mask_groups, ")");
        TORCH_CHECK(c.mask.size(1) == mask_groups * taps, "mask.shape[1] is not valid. got: ", c.mask.size(1),
                    " expected: ", mask_groups * taps);
        std::array<int64_t, D> mgd{};
        bool ok = true;
        for (int a = 0; a < D; ++a) { mgd[a] = c.mask.size(2 + a); ok = ok && mgd[a] == grid[a]; }
        TORCH_CHECK(ok, "mask ", own_what, ": (", dims_str<D>(mgd), ") - ", grid_what, ": (", dims_str<D>(grid), ")");
    }
    if (with_bias)
        TORCH_CHECK(c.bias.dim() == 1 && c.bias.size(0) == p.out_channels, "bias must have ", p.out_channels,
                    " elements, got size ", c.bias.sizes());
    for (int a = 0; a < D; ++a)
        TORCH_CHECK(out[a] > 0, "Calculated output size too small - (", dims_str<D>(out), ")");

    const int rc = tvdcn_b200_problem_finalize(&p);
    TORCH_CHECK(rc == TVDCN_OK, name, ": ", tvdcn_b200_last_error());
    return c;
}

// ---- status of the bounded waits, without a synchronisation per call --------------------------------------
// The tensor-core kernels give up on a barrier wait that runs out and leave a code in a per-device word; their
// outputs are then incomplete.  After every operator call a one-thread kernel, behind the call's kernels on the same
// stream, stores a non-zero word into one mapped pinned host integer per device (a store, not a copy: a copy would
// queue behind the caller's own transfers on the copy engines); the next operator call on that device looks at the
// integer first and raises.  With TVDCN_B200_CHECK_STATUS=1 every call synchronises and raises itself.
struct StatusWatch {
    int *pinned = nullptr;       // host view of the mapped pinned word
    int *pinned_dev = nullptr;   // the same word as the device addresses it
    bool tried = false;
};
StatusWatch &status_watch(int device) {
    static StatusWatch per_device[64];
    StatusWatch &w = per_device[device & 63];
    if (!w.tried) {
        w.tried = true;
        void *dev_view = nullptr;
        if (cudaHostAlloc(reinterpret_cast<void **>(&w.pinned), sizeof(int), cudaHostAllocMapped) == cudaSuccess &&
            cudaHostGetDevicePointer(&dev_view, w.pinned, 0) == cudaSuccess) {
            *w.pinned = 0;
            w.pinned_dev = static_cast<int *>(dev_view);
        } else {
            w.pinned = nullptr;
        }
    }
    return w;
}
bool check_every_call() {
    static const bool on = [] {
        const char *v = getenv("TVDCN_B200_CHECK_STATUS");
        return v != nullptr && v[0] == '1';
    }();
    return on;
}
[[noreturn]] void raise_status(int code) {
    TORCH_CHECK(false, "tvdcn: a tensor-core kernel of an earlier call gave up on a bounded wait (code ", code,
                "); the tensors that call returned are incomplete");
    abort();
}
// before an operator's own work
void check_earlier_calls(int device) {
    StatusWatch &w = status_watch(device);
    if (w.pinned == nullptr) return;
    const int seen = *reinterpret_cast<volatile int *>(w.pinned);
    if (seen != 0) {
        *w.pinned = 0;
        (void)tvdcn_b200_device_status();   // synchronises and clears the device word
        raise_status(seen);
    }
}
// after an operator's kernels have been enqueued on `stream`
void watch_this_call(int device, cudaStream_t stream) {
    if (check_every_call()) {
        const int code = tvdcn_b200_device_status();
        if (code != 0) raise_status(code);
        return;
    }
    StatusWatch &w = status_watch(device);
    if (w.pinned != nullptr) (void)tvdcn_b200_publish_status(w.pinned_dev, stream);
}

Tensor make_workspace(size_t bytes, const Tensor &like) {
    return at::empty({(int64_t)bytes}, like.options().dtype(at::kByte));
}

const void *ptr(const Tensor &t) { return t.defined() ? t.data_ptr() : nullptr; }

template <int D, bool TR>
Tensor forward_cuda_impl(const Tensor &input, const Tensor &weight, const OptTensor &offset, const OptTensor &mask,
                         const OptTensor &bias, at::IntArrayRef stride, at::IntArrayRef padding,
                         at::IntArrayRef output_padding, at::IntArrayRef dilation, int64_t groups) {
    c10::cuda::CUDAGuard guard(input.device());
    check_earlier_calls(input.device().index());
    Call c = prepare<D, TR>(input, weight, offset, mask, bias, stride, padding, output_padding, dilation, groups);
    std::vector<int64_t> shape{c.prob.batch, c.prob.out_channels};
    for (int a = 0; a < D; ++a) shape.push_back(c.prob.out_size[a]);
    Tensor out = at::empty(shape, c.input.options());
    const size_t wsb = tvdcn_b200_forward_workspace_bytes(&c.prob);
    Tensor ws = make_workspace(wsb, c.input);
    auto stream = at::cuda::getCurrentCUDAStream();
    const int rc = tvdcn_b200_deform_conv_forward(&c.prob, ptr(c.input), ptr(c.weight), ptr(c.offset), ptr(c.mask),
                                                  ptr(c.bias), out.data_ptr(), wsb ? ws.data_ptr() : nullptr, wsb,
                                                  stream.stream());
    TORCH_CHECK(rc == TVDCN_OK, op_name<D, TR>(), ": ", tvdcn_b200_last_error());
    watch_this_call(input.device().index(), stream.stream());
    if (c.unbatched) out = out.squeeze(0);
    return out;
}

template <int D, bool TR>
std::tuple<Tensor, Tensor, Tensor, Tensor, Tensor> backward_cuda_impl(
    const Tensor &grad, const Tensor &input, const Tensor &weight, const OptTensor &offset, const OptTensor &mask,
    const OptTensor &bias, at::IntArrayRef stride, at::IntArrayRef padding, at::IntArrayRef output_padding,
    at::IntArrayRef dilation, int64_t groups) {
    c10::cuda::CUDAGuard guard(input.device());
    check_earlier_calls(input.device().index());
    Call c = prepare<D, TR>(input, weight, offset, mask, bias, stride, padding, output_padding, dilation, groups);
    Tensor g = grad.contiguous();
    if (c.unbatched) g = g.unsqueeze(0);
    TORCH_CHECK(g.scalar_type() == c.input.scalar_type() && g.device() == c.input.device(),
                "grad must have the dtype and device of input");
    TORCH_CHECK(g.dim() == D + 2 && g.size(0) == c.prob.batch && g.size(1) == c.prob.out_channels,
                "grad has the wrong shape: ", g.sizes());
    for (int a = 0; a < D; ++a)
        TORCH_CHECK(g.size(2 + a) == c.prob.out_size[a], "grad has the wrong shape: ", g.sizes());

    Tensor g_input = at::empty_like(c.input);
    Tensor g_weight = at::empty_like(c.weight);
    Tensor g_offset = c.offset.defined() ? at::empty_like(c.offset) : Tensor();
    Tensor g_mask = c.mask.defined() ? at::empty_like(c.mask) : Tensor();
    Tensor g_bias = c.bias.defined() ? at::empty_like(c.bias) : Tensor();
    const size_t wsb = tvdcn_b200_backward_workspace_bytes(&c.prob);
    Tensor ws = make_workspace(wsb, c.input);
    auto stream = at::cuda::getCurrentCUDAStream();
    const int rc = tvdcn_b200_deform_conv_backward(
        &c.prob, g.data_ptr(), ptr(c.input), ptr(c.weight), ptr(c.offset), ptr(c.mask), g_input.data_ptr(),
        g_weight.data_ptr(), g_offset.defined() ? g_offset.data_ptr() : nullptr,
        g_mask.defined() ? g_mask.data_ptr() : nullptr, g_bias.defined() ? g_bias.data_ptr() : nullptr,
        wsb ? ws.data_ptr() : nullptr, wsb, stream.stream());
    TORCH_CHECK(rc == TVDCN_OK, "_", op_name<D, TR>(), "_backward: ", tvdcn_b200_last_error());
    watch_this_call(input.device().index(), stream.stream());
    if (c.unbatched) {
        g_input = g_input.squeeze(0);
        if (g_offset.defined()) g_offset = g_offset.squeeze(0);
        if (g_mask.defined()) g_mask = g_mask.squeeze(0);
    }
    g_input = g_input.view_as(input);
    g_weight = g_weight.view_as(weight);
    return std::make_tuple(g_input, g_weight, g_offset, g_mask, g_bias);
}

// ---- dispatcher re-entry ------------------------------------------------------------------
template <int D, bool TR>
struct Ops {
    using FwdConv = Tensor(const Tensor &, const Tensor &, const OptTensor &, const OptTensor &, const OptTensor &,
                           at::IntArrayRef, at::IntArrayRef, at::IntArrayRef, int64_t);
    using FwdTr = Tensor(const Tensor &, const Tensor &, const OptTensor &, const OptTensor &, const OptTensor &,
                         at::IntArrayRef, at::IntArrayRef, at::IntArrayRef, at::IntArrayRef, int64_t);
    using Grads = std::tuple<Tensor, Tensor, Tensor, Tensor, Tensor>;
    using BwdConv = Grads(const Tensor &, const Tensor &, const Tensor &, const OptTensor &, const OptTensor &,
                          const OptTensor &, at::IntArrayRef, at::IntArrayRef, at::IntArrayRef, int64_t);
    using BwdTr = Grads(const Tensor &, const Tensor &, const Tensor &, const OptTensor &, const OptTensor &,
                        const OptTensor &, at::IntArrayRef, at::IntArrayRef, at::IntArrayRef, at::IntArrayRef,
                        int64_t);

    static Tensor call_forward(const Tensor &input, const Tensor &weight, const OptTensor &offset,
                               const OptTensor &mask, const OptTensor &bias, at::IntArrayRef stride,
                               at::IntArrayRef padding, at::IntArrayRef output_padding, at::IntArrayRef dilation,
                               int64_t groups) {
        const std::string n = "tvdcn::" + op_name<D, TR>();
        if constexpr (TR) {
            static auto op = c10::Dispatcher::singleton().findSchemaOrThrow(n.c_str(), "").template typed<FwdTr>();
            return op.call(input, weight, offset, mask, bias, stride, padding, output_padding, dilation, groups);
        } else {
            static auto op = c10::Dispatcher::singleton().findSchemaOrThrow(n.c_str(), "").template typed<FwdConv>();
            return op.call(input, weight, offset, mask, bias, stride, padding, dilation, groups);
        }
    }

    static Grads call_backward(const Tensor &grad, const Tensor &input, const Tensor &weight, const OptTensor &offset,
                               const OptTensor &mask, const OptTensor &bias, at::IntArrayRef stride,
                               at::IntArrayRef padding, at::IntArrayRef output_padding, at::IntArrayRef dilation,
                               int64_t groups) {
        const std::string n = "tvdcn::_" + op_name<D, TR>() + "_backward";
        if constexpr (TR) {
            static auto op = c10::Dispatcher::singleton().findSchemaOrThrow(n.c_str(), "").template typed<BwdTr>();
            return op.call(grad, input, weight, offset, mask, bias, stride, padding, output_padding, dilation,
                           groups);
        } else {
            static auto op = c10::Dispatcher::singleton().findSchemaOrThrow(n.c_str(), "").template typed<BwdConv>();
            return op.call(grad, input, weight, offset, mask, bias, stride, padding, dilation, groups);
        }
    }
};

OptTensor opt(const Tensor &t) { return t.defined() ? OptTensor(t) : OptTensor(); }

// ---- autograd -----------------------------------------------------------------------------
// Saves the five tensors like the reference (tvdcn/csrc/ops/autograd/deform_conv2d_kernel.cpp:23-45) and
// returns all five gradients from one backward call (:48-92).
template <int D, bool TR>
class ConvFunction : public torch::autograd::Function<ConvFunction<D, TR>> {
   public:
    static variable_list forward(AutogradContext *ctx, const Tensor &input, const Tensor &weight,
                                 const OptTensor &offset, const OptTensor &mask, const OptTensor &bias,
                                 std::vector<int64_t> stride, std::vector<int64_t> padding,
                                 std::vector<int64_t> output_padding, std::vector<int64_t> dilation, int64_t groups) {
        at::AutoDispatchBelowADInplaceOrView guard;
        Tensor out = Ops<D, TR>::call_forward(input, weight, offset, mask, bias, stride, padding, output_padding,
                                              dilation, groups);
        ctx->save_for_backward({input, weight, has(offset) ? *offset : Tensor(), has(mask) ? *mask : Tensor(),
                                has(bias) ? *bias : Tensor()});
        ctx->saved_data["stride"] = stride;
        ctx->saved_data["padding"] = padding;
        ctx->saved_data["output_padding"] = output_padding;
        ctx->saved_data["dilation"] = dilation;
        ctx->saved_data["groups"] = groups;
        return {out};
    }

    static variable_list backward(AutogradContext *ctx, const variable_list &grad_output) {
        auto saved = ctx->get_saved_variables();
        auto stride = ctx->saved_data["stride"].toIntVector();
        auto padding = ctx->saved_data["padding"].toIntVector();
        auto output_padding = ctx->saved_data["output_padding"].toIntVector();
        auto dilation = ctx->saved_data["dilation"].toIntVector();
        auto groups = ctx->saved_data["groups"].toInt();
        auto grads = Ops<D, TR>::call_backward(grad_output[0], saved[0], saved[1], opt(saved[2]), opt(saved[3]),
                                               opt(saved[4]), stride, padding, output_padding, dilation, groups);
        return {std::get<0>(grads), std::get<1>(grads), std::get<2>(grads), std::get<3>(grads), std::get<4>(grads),
                Tensor(), Tensor(), Tensor(), Tensor(), Tensor()};
    }
};

// The backward operator is itself not differentiable, as in the reference (:96-144).
template <int D, bool TR>
class ConvBackwardFunction : public torch::autograd::Function<ConvBackwardFunction<D, TR>> {
   public:
    static variable_list forward(AutogradContext *ctx, const Tensor &grad, const Tensor &input, const Tensor &weight,
                                 const OptTensor &offset, const OptTensor &mask, const OptTensor &bias,
                                 std::vector<int64_t> stride, std::vector<int64_t> padding,
                                 std::vector<int64_t> output_padding, std::vector<int64_t> dilation, int64_t groups) {
        at::AutoDispatchBelowADInplaceOrView guard;
        auto grads = Ops<D, TR>::call_backward(grad, input, weight, offset, mask, bias, stride, padding,
                                               output_padding, dilation, groups);
        // autograd cannot wrap undefined outputs: absent gradients travel as empty tensors and are
        // turned back into undefined ones by the caller
        auto placeholder = [&](const Tensor &t) { return t.defined() ? t : at::empty({0}, input.options()); };
        return {std::get<0>(grads), std::get<1>(grads), placeholder(std::get<2>(grads)),
                placeholder(std::get<3>(grads)), placeholder(std::get<4>(grads))};
    }
    static variable_list backward(AutogradContext *, const variable_list &) {
        TORCH_CHECK(false, "double backwards on ", op_name<D, TR>(), " not supported");
    }
};

template <int D>
Tensor conv_autograd(const Tensor &input, const Tensor &weight, const OptTensor &offset, const OptTensor &mask,
                     const OptTensor &bias, at::IntArrayRef stride, at::IntArrayRef padding, at::IntArrayRef dilation,
                     int64_t groups) {
    return ConvFunction<D, false>::apply(input, weight, offset, mask, bias, stride.vec(), padding.vec(),
                                         std::vector<int64_t>{0}, dilation.vec(), groups)[0];
}
template <int D>
Tensor convtr_autograd(const Tensor &input, const Tensor &weight, const OptTensor &offset, const OptTensor &mask,
                       const OptTensor &bias, at::IntArrayRef stride, at::IntArrayRef padding,
                       at::IntArrayRef output_padding, at::IntArrayRef dilation, int64_t groups) {
    return ConvFunction<D, true>::apply(input, weight, offset, mask, bias, stride.vec(), padding.vec(),
                                        output_padding.vec(), dilation.vec(), groups)[0];
}
template <int D>
std::tuple<Tensor, Tensor, Tensor, Tensor, Tensor> conv_backward_autograd(
    const Tensor &grad, const Tensor &input, const Tensor &weight, const OptTensor &offset, const OptTensor &mask,
    const OptTensor &bias, at::IntArrayRef stride, at::IntArrayRef padding, at::IntArrayRef dilation, int64_t groups) {
    auto r = ConvBackwardFunction<D, false>::apply(grad, input, weight, offset, mask, bias, stride.vec(),
                                                   padding.vec(), std::vector<int64_t>{0}, dilation.vec(), groups);
    return std::make_tuple(r[0], r[1], has(offset) ? r[2] : Tensor(), has(mask) ? r[3] : Tensor(),
                           has(bias) ? r[4] : Tensor());
}
template <int D>
std::tuple<Tensor, Tensor, Tensor, Tensor, Tensor> convtr_backward_autograd(
    const Tensor &grad, const Tensor &input, const Tensor &weight, const OptTensor &offset, const OptTensor &mask,
    const OptTensor &bias, at::IntArrayRef stride, at::IntArrayRef padding, at::IntArrayRef output_padding,
    at::IntArrayRef dilation, int64_t groups) {
    auto r = ConvBackwardFunction<D, true>::apply(grad, input, weight, offset, mask, bias, stride.vec(),
                                                  padding.vec(), output_padding.vec(), dilation.vec(), groups);
    return std::make_tuple(r[0], r[1], has(offset) ? r[2] : Tensor(), has(mask) ? r[3] : Tensor(),
                           has(bias) ? r[4] : Tensor());
}

// ---- CUDA key -----------------------------------------------------------------------------
template <int D>
Tensor conv_cuda(const Tensor &input, const Tensor &weight, const OptTensor &offset, const OptTensor &mask,
                 const OptTensor &bias, at::IntArrayRef stride, at::IntArrayRef padding, at::IntArrayRef dilation,
                 int64_t groups) {
    return forward_cuda_impl<D, false>(input, weight, offset, mask, bias, stride, padding, {0}, dilation, groups);
}
template <int D>
Tensor convtr_cuda(const Tensor &input, const Tensor &weight, const OptTensor &offset, const OptTensor &mask,
                   const OptTensor &bias, at::IntArrayRef stride, at::IntArrayRef padding,
                   at::IntArrayRef output_padding, at::IntArrayRef dilation, int64_t groups) {
    return forward_cuda_impl<D, true>(input, weight, offset, mask, bias, stride, padding, output_padding, dilation,
                                      groups);
}
template <int D>
std::tuple<Tensor, Tensor, Tensor, Tensor, Tensor> conv_backward_cuda(
    const Tensor &grad, const Tensor &input, const Tensor &weight, const OptTensor &offset, const OptTensor &mask,
    const OptTensor &bias, at::IntArrayRef stride, at::IntArrayRef padding, at::IntArrayRef dilation, int64_t groups) {
    return backward_cuda_impl<D, false>(grad, input, weight, offset, mask, bias, stride, padding, {0}, dilation,
                                        groups);
}
template <int D>
std::tuple<Tensor, Tensor, Tensor, Tensor, Tensor> convtr_backward_cuda(
    const Tensor &grad, const Tensor &input, const Tensor &weight, const OptTensor &offset, const OptTensor &mask,
    const OptTensor &bias, at::IntArrayRef stride, at::IntArrayRef padding, at::IntArrayRef output_padding,
    at::IntArrayRef dilation, int64_t groups) {
    return backward_cuda_impl<D, true>(grad, input, weight, offset, mask, bias, stride, padding, output_padding,
                                       dilation, groups);
}

// ---- autocast -----------------------------------------------------------------------------
OptTensor cast_opt(const OptTensor &t, at::ScalarType to) {
    if (!has(t)) return OptTensor();
    return OptTensor(at::autocast::cached_cast(to, *t, c10::DeviceType::CUDA));
}
template <int D>
Tensor conv_autocast(const Tensor &input, const Tensor &weight, const OptTensor &offset, const OptTensor &mask,
                     const OptTensor &bias, at::IntArrayRef stride, at::IntArrayRef padding, at::IntArrayRef dilation,
                     int64_t groups) {
    c10::impl::ExcludeDispatchKeyGuard no_autocast(c10::DispatchKey::Autocast);
    const auto low = at::autocast::get_autocast_dtype(c10::DeviceType::CUDA);
    return Ops<D, false>::call_forward(at::autocast::cached_cast(low, input, c10::DeviceType::CUDA),
                                       at::autocast::cached_cast(low, weight, c10::DeviceType::CUDA),
                                       cast_opt(offset, at::kFloat), cast_opt(mask, at::kFloat),
                                       cast_opt(bias, at::kFloat), stride, padding, {0}, dilation, groups);
}
template <int D>
Tensor convtr_autocast(const Tensor &input, const Tensor &weight, const OptTensor &offset, const OptTensor &mask,
                       const OptTensor &bias, at::IntArrayRef stride, at::IntArrayRef padding,
                       at::IntArrayRef output_padding, at::IntArrayRef dilation, int64_t groups) {
    c10::impl::ExcludeDispatchKeyGuard no_autocast(c10::DispatchKey::Autocast);
    const auto low = at::autocast::get_autocast_dtype(c10::DeviceType::CUDA);
    return Ops<D, true>::call_forward(at::autocast::cached_cast(low, input, c10::DeviceType::CUDA),
                                      at::autocast::cached_cast(low, weight, c10::DeviceType::CUDA),
                                      cast_opt(offset, at::kFloat), cast_opt(mask, at::kFloat),
                                      cast_opt(bias, at::kFloat), stride, padding, output_padding, dilation, groups);
}

// ---- mask softmax ---------------------------------------------------------------------------
template <int D>
int64_t softmax_taps(const Tensor &mask, at::IntArrayRef kernel_size) {
    const auto ks = ntuple<D>(kernel_size);
    int64_t taps = 1;
    for (int a = 0; a < D; ++a) taps *= ks[a];
    TORCH_CHECK(mask.dim() == D + 2, "mask_softmax", D, "d expects a ", D + 2, "D mask, got size ", mask.sizes());
    TORCH_CHECK(taps > 0 && mask.size(1) / taps > 0,
                "The shape of the mask tensor at dimension 1 is not valid. It should be a multiple of "
                "prod(kernel_size).\nGot mask.size(1)=", mask.size(1), ", while prod(kernel_size)=", taps);
    TORCH_CHECK(mask.size(1) % taps == 0, "mask.size(1) (", mask.size(1), ") is not a multiple of prod(kernel_size) (",
                taps, ")");
    return taps;
}

Tensor softmax_fwd_raw(const Tensor &mask, int64_t taps) {
    c10::cuda::CUDAGuard guard(mask.device());
    Tensor in = mask.contiguous();
    Tensor out = at::empty_like(in);
    int64_t spatial = 1;
    for (int64_t a = 2; a < in.dim(); ++a) spatial *= in.size(a);
    const int rc = tvdcn_b200_mask_softmax_forward(to_dtype(in.scalar_type(), "mask_softmax"), in.size(0),
                                                   in.size(1) / taps, taps, spatial, in.data_ptr(), out.data_ptr(),
                                                   at::cuda::getCurrentCUDAStream().stream());
    TORCH_CHECK(rc == TVDCN_OK, "mask_softmax: ", tvdcn_b200_last_error());
    return out;
}

Tensor softmax_bwd_cuda(const Tensor &grad, const Tensor &out, int64_t taps) {
    c10::cuda::CUDAGuard guard(out.device());
    Tensor g = grad.contiguous(), y = out.contiguous();
    TORCH_CHECK(g.sizes() == y.sizes() && g.scalar_type() == y.scalar_type(), "grad and out must match");
    Tensor gi = at::empty_like(y);
    int64_t spatial = 1;
    for (int64_t a = 2; a < y.dim(); ++a) spatial *= y.size(a);
    const int rc = tvdcn_b200_mask_softmax_backward(to_dtype(y.scalar_type(), "mask_softmax"), y.size(0),
                                                    y.size(1) / taps, taps, spatial, g.data_ptr(), y.data_ptr(),
                                                    gi.data_ptr(), at::cuda::getCurrentCUDAStream().stream());
    TORCH_CHECK(rc == TVDCN_OK, "mask_softmax backward: ", tvdcn_b200_last_error());
    return gi;
}

template <int D>
Tensor softmax_cuda(const Tensor &mask, at::IntArrayRef kernel_size) {
    return softmax_fwd_raw(mask, softmax_taps<D>(mask, kernel_size));
}

Tensor call_softmax_bwd(const Tensor &grad, const Tensor &out, int64_t taps) {
    static auto op = c10::Dispatcher::singleton()
                         .findSchemaOrThrow("tvdcn::_mask_softmax_backward", "")
                         .typed<Tensor(const Tensor &, const Tensor &, int64_t)>();
    return op.call(grad, out, taps);
}

template <int D>
class SoftmaxFunction : public torch::autograd::Function<SoftmaxFunction<D>> {
   public:
    static variable_list forward(AutogradContext *ctx, const Tensor &mask, std::vector<int64_t> kernel_size) {
        at::AutoDispatchBelowADInplaceOrView guard;
        const std::string n = "tvdcn::mask_softmax" + std::to_string(D) + "d";
        static auto op = c10::Dispatcher::singleton()
                             .findSchemaOrThrow(n.c_str(), "")
                             .template typed<Tensor(const Tensor &, at::IntArrayRef)>();
        Tensor out = op.call(mask, kernel_size);
        int64_t taps = 1;
        for (auto k : ntuple<D>(kernel_size)) taps *= k;
        ctx->save_for_backward({out});
        ctx->saved_data["taps"] = taps;
        return {out};
    }
    static variable_list backward(AutogradContext *ctx, const variable_list &grad_output) {
        auto saved = ctx->get_saved_variables();
        at::AutoDispatchBelowADInplaceOrView guard;
        return {call_softmax_bwd(grad_output[0], saved[0], ctx->saved_data["taps"].toInt()), Tensor()};
    }
};
template <int D>
Tensor softmax_autograd(const Tensor &mask, at::IntArrayRef kernel_size) {
    return SoftmaxFunction<D>::apply(mask, kernel_size.vec())[0];
}

int64_t cuda_version() { return tvdcn_b200_cuda_version(); }
std::string cuda_arch_flags() { return tvdcn_b200_cuda_arch_flags(); }
int64_t launch_count() { return (int64_t)tvdcn_b200_launch_count(); }

}  // namespace

TORCH_LIBRARY(tvdcn, m) {
#define TVDCN_DEF_CONV(D)                                                                                         \
    m.def("tvdcn::deform_conv" #D "d(Tensor input, Tensor weight, Tensor? offset=None, Tensor? mask=None, "        \
          "Tensor? bias=None, SymInt[" #D "] stride=1, SymInt[" #D "] padding=0, SymInt[" #D "] dilation=1, "      \
          "SymInt groups=1) -> Tensor");                                                                          \
    m.def("tvdcn::_deform_conv" #D "d_backward(Tensor grad, Tensor input, Tensor weight, Tensor? offset=None, "    \
          "Tensor? mask=None, Tensor? bias=None, SymInt[" #D "] stride=1, SymInt[" #D "] padding=0, SymInt[" #D    \
          "] dilation=1, SymInt groups=1) -> (Tensor, Tensor, Tensor, Tensor, Tensor)");                          \
    m.def("tvdcn::deform_conv_transpose" #D "d(Tensor input, Tensor weight, Tensor? offset=None, "                 \
          "Tensor? mask=None, Tensor? bias=None, SymInt[" #D "] stride=1, SymInt[" #D "] padding=0, SymInt[" #D    \
          "] output_padding=0, SymInt[" #D "] dilation=1, SymInt groups=1) -> Tensor");                           \
    m.def("tvdcn::_deform_conv_transpose" #D "d_backward(Tensor grad, Tensor input, Tensor weight, "               \
          "Tensor? offset=None, Tensor? mask=None, Tensor? bias=None, SymInt[" #D "] stride=1, SymInt[" #D         \
          "] padding=0, SymInt[" #D "] output_padding=0, SymInt[" #D "] dilation=1, SymInt groups=1) -> "          \
          "(Tensor, Tensor, Tensor, Tensor, Tensor)");                                                            \
    m.def("tvdcn::mask_softmax" #D "d(Tensor mask, int[" #D "] kernel_size) -> Tensor");
    TVDCN_DEF_CONV(1)
    TVDCN_DEF_CONV(2)
    TVDCN_DEF_CONV(3)
#undef TVDCN_DEF_CONV
    m.def("tvdcn::_mask_softmax_backward(Tensor grad, Tensor out, int taps) -> Tensor");
    m.def("tvdcn::_cuda_version() -> int", &cuda_version);
    m.def("tvdcn::_cuda_arch_flags() -> str", &cuda_arch_flags);
    m.def("tvdcn::_launch_count() -> int", &launch_count);
}

#define TVDCN_IMPL_ALL(D, conv, convb, convtr, convtrb)                          \
    m.impl("deform_conv" #D "d", TORCH_FN(conv<D>));                             \
    m.impl("_deform_conv" #D "d_backward", TORCH_FN(convb<D>));                  \
    m.impl("deform_conv_transpose" #D "d", TORCH_FN(convtr<D>));                 \
    m.impl("_deform_conv_transpose" #D "d_backward", TORCH_FN(convtrb<D>));

TORCH_LIBRARY_IMPL(tvdcn, CUDA, m) {
    TVDCN_IMPL_ALL(1, conv_cuda, conv_backward_cuda, convtr_cuda, convtr_backward_cuda)
    TVDCN_IMPL_ALL(2, conv_cuda, conv_backward_cuda, convtr_cuda, convtr_backward_cuda)
    TVDCN_IMPL_ALL(3, conv_cuda, conv_backward_cuda, convtr_cuda, convtr_backward_cuda)
    m.impl("mask_softmax1d", TORCH_FN(softmax_cuda<1>));
    m.impl("mask_softmax2d", TORCH_FN(softmax_cuda<2>));
    m.impl("mask_softmax3d", TORCH_FN(softmax_cuda<3>));
    m.impl("_mask_softmax_backward", TORCH_FN(softmax_bwd_cuda));
}

TORCH_LIBRARY_IMPL(tvdcn, Autograd, m) {
    TVDCN_IMPL_ALL(1, conv_autograd, conv_backward_autograd, convtr_autograd, convtr_backward_autograd)
    TVDCN_IMPL_ALL(2, conv_autograd, conv_backward_autograd, convtr_autograd, convtr_backward_autograd)
    TVDCN_IMPL_ALL(3, conv_autograd, conv_backward_autograd, convtr_autograd, convtr_backward_autograd)
    m.impl("mask_softmax1d", TORCH_FN(softmax_autograd<1>));
    m.impl("mask_softmax2d", TORCH_FN(softmax_autograd<2>));
    m.impl("mask_softmax3d", TORCH_FN(softmax_autograd<3>));
}

TORCH_LIBRARY_IMPL(tvdcn, Autocast, m) {
    m.impl("deform_conv1d", TORCH_FN(conv_autocast<1>));
    m.impl("deform_conv2d", TORCH_FN(conv_autocast<2>));
    m.impl("deform_conv3d", TORCH_FN(conv_autocast<3>));
    m.impl("deform_conv_transpose1d", TORCH_FN(convtr_autocast<1>));
    m.impl("deform_conv_transpose2d", TORCH_FN(convtr_autocast<2>));
    m.impl("deform_conv_transpose3d", TORCH_FN(convtr_autocast<3>));
}

}  // namespace tvdcn_b200
