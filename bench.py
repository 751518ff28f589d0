#!/usr/bin/env python
"""Benchmark of the deformable-convolution step (forward + backward) on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--config 1..5] [--mode fp32|bf16] [--impl ours|reference]

One "step" is one forward + backward pass of the configured operator over one batch of seeded synthetic
tensors (for config 2 the mask is produced by mask_softmax2d inside the step, forward and backward).
Rank 0 prints ONE JSON line.  Keys beyond the usual ones:

  value        images/s with every input already resident in HBM, all ranks together.  --gpus N shards the
               configuration's batch over the ranks (strong scaling, config 2: 128 / 64 / 32 / 16 images per
               rank); the only exchange is the all-reduce of [grad_weight|grad_bias].  "weak" carries the figure
               with the configuration's whole batch on every GPU.
  modes        the configuration's other data mode (bf16 input / weight for configurations 2 and 5), measured in
               the same process after the headline mode: value, kernels, roofline, e2e, clocks
  operator_step_ms  the same device-resident step through the public PyTorch operators (fresh outputs and
               workspace per call), beside the C-ABI step that `value` times
  grad_check   N > 1: the all-reduced gradient against the sum of the ranks' buckets and against one GPU computing
               the whole batch (outside the timed regions)
  e2e          the same metric through the public operators (tvdcn_b200.ops.*, autograd) with HOST buffers:
               pinned host -> device copies of every step's inputs and device -> host copies of its results
               are inside the timed region, on copy streams beside the compute stream (prefetching loader)
  roofline     dominant kernel: algorithmic FLOPs (or bytes) per launch / CUDA-event time per launch, against
               the measured peak in MEASURED_PEAKS.json (fallback figures if the file is absent)
  cpu_baseline the reference's own CPU implementation (oracle/_ref) timed on this box's host cores on a
               bounded sample of the same workload (rank 0, 1 GPU only)
  reference_cuda  the reference's own CUDA backend (built from its sources for sm_100 into oracle/_ref) timed on
               the same GPU on the same device-resident step, fp32 (rank 0, 1 GPU only; a reported baseline)

With --impl reference the whole run is the reference's CPU implementation on a bounded sample per step.
"""
from __future__ import annotations

import argparse
import ctypes
import json
import math
import os
import sys
import threading
import time
from dataclasses import dataclass
from typing import Optional, Tuple

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import torch  # noqa: E402


@dataclass(frozen=True)
class Config:
    name: str
    dim: int
    transposed: bool
    batch: int
    cin: int
    cout: int
    in_size: Tuple[int, ...]
    kernel: Tuple[int, ...]
    stride: Tuple[int, ...]
    padding: Tuple[int, ...]
    dilation: Tuple[int, ...]
    groups: int
    offset_groups: int
    mask_groups: int
    offset_std: float
    softmax_mask: bool
    bound: str  # which roofline bounds the step

    @property
    def taps(self):
        return math.prod(self.kernel)

    @property
    def out_size(self):
        if not self.transposed:
            return tuple((i + 2 * p - (d * (k - 1) + 1)) // s + 1 for i, k, s, p, d in
                         zip(self.in_size, self.kernel, self.stride, self.padding, self.dilation))
        return tuple((i - 1) * s - 2 * p + d * (k - 1) + 1 for i, k, s, p, d in
                     zip(self.in_size, self.kernel, self.stride, self.padding, self.dilation))

    @property
    def grid(self):
        return self.in_size if self.transposed else self.out_size

    def flops_per_pass(self, batch):
        """One GEMM pass: 2 * C_out * (C_in / groups) * taps * batch * grid positions."""
        return 2.0 * self.cout * (self.cin / self.groups) * self.taps * batch * math.prod(self.grid)

    def algorithmic_bytes(self, batch, esize=4):
        """Every tensor of the operator's signature read or written once, forward + backward."""
        x = batch * self.cin * math.prod(self.in_size)
        y = batch * self.cout * math.prod(self.out_size)
        off = batch * self.offset_groups * self.taps * self.dim * math.prod(self.grid)
        m = batch * self.mask_groups * self.taps * math.prod(self.grid)
        w = self.cout * self.cin // self.groups * self.taps
        fwd = x + off + m + w + self.cout + y
        bwd = y + x + off + m + w + x + w + off + m + self.cout
        return (fwd + bwd) * esize


CONFIGS = {
    1: Config('deform_conv2d N4 C64->64 56x56 k3 s1 p1 og1 mask', 2, False, 4, 64, 64, (56, 56), (3, 3), (1, 1),
              (1, 1), (1, 1), 1, 1, 1, 1.5, False, 'hbm'),
    2: Config('deform_conv2d N128 C256->256 28x28 k3 s1 p1 og4 mg1 softmax-mask (DCNv2 block)', 2, False, 128, 256,
              256, (28, 28), (3, 3), (1, 1), (1, 1), (1, 1), 1, 4, 1, 2.0, True, 'tensor'),
    3: Config('deform_conv1d N64 C512->512 L4096 k5 d2 p4 g8 og8 mask', 1, False, 64, 512, 512, (4096,), (5,), (1,),
              (4,), (2,), 8, 8, 1, 3.0, False, 'hbm'),
    4: Config('deform_conv3d N8 C64->64 16x56x56 k3 s1 p1 og1 mask', 3, False, 8, 64, 64, (16, 56, 56), (3, 3, 3),
              (1, 1, 1), (1, 1, 1), (1, 1, 1), 1, 1, 1, 1.0, False, 'tensor'),
    5: Config('deform_conv_transpose2d N64 C256->128 32x32->64x64 k4 s2 p1 og2 mask', 2, True, 64, 256, 128,
              (32, 32), (4, 4), (2, 2), (1, 1), (1, 1), 1, 2, 1, 1.5, False, 'tensor'),
}


def make_inputs(cfg: Config, batch: int, seed: int, pin: bool = False):
    """Seeded float32 host tensors with the distributions the configuration names."""
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(batch, cfg.cin, *cfg.in_size, generator=g)
    if not cfg.transposed:
        wshape = (cfg.cout, cfg.cin // cfg.groups, *cfg.kernel)
        fan_in = cfg.cin // cfg.groups * cfg.taps
    else:
        wshape = (cfg.cin, cfg.cout // cfg.groups, *cfg.kernel)
        fan_in = cfg.cout // cfg.groups * cfg.taps
    bound = 1.0 / math.sqrt(fan_in)  # kaiming_uniform_(a=sqrt(5)) of _ConvNd.reset_parameters
    w = (torch.rand(*wshape, generator=g) * 2 - 1) * bound
    bias = torch.randn(cfg.cout, generator=g) * 0.01
    off = torch.randn(batch, cfg.offset_groups * cfg.taps * cfg.dim, *cfg.grid, generator=g) * cfg.offset_std
    if cfg.softmax_mask:
        m = torch.randn(batch, cfg.mask_groups * cfg.taps, *cfg.grid, generator=g)  # logits
    else:
        m = torch.rand(batch, cfg.mask_groups * cfg.taps, *cfg.grid, generator=g)
    go = torch.randn(batch, cfg.cout, *cfg.out_size, generator=g)
    ts = dict(x=x, w=w, bias=bias, off=off, m=m, go=go)
    if pin:
        ts = {k: v.pin_memory() for k, v in ts.items()}
    return ts


# ------------------------------------------------------------------------------------------------------
# clocks
# ------------------------------------------------------------------------------------------------------
class ClockSampler:
    """Samples SM clock and throttle reasons of one GPU through NVML while the timed region runs."""

    REASONS = {
        0x8: 'hw_slowdown', 0x40: 'hw_thermal_slowdown', 0x20: 'sw_thermal_slowdown', 0x4: 'sw_power_cap',
        0x80: 'hw_power_brake', 0x2: 'applications_clocks', 0x100: 'display_clock', 0x10: 'sync_boost',
    }

    def __init__(self, index: int):
        self.samples, self.reasons, self.max_mhz = [], set(), None
        self._stop = threading.Event()
        self._thread = None
        try:
            import pynvml
            pynvml.nvmlInit()
            self._nv = pynvml
            self._h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self._h, pynvml.NVML_CLOCK_SM)
        except Exception:  # NVML missing: report nulls
            self._nv = None

    def _run(self):
        while not self._stop.is_set():
            try:
                self.samples.append(self._nv.nvmlDeviceGetClockInfo(self._h, self._nv.NVML_CLOCK_SM))
                bits = self._nv.nvmlDeviceGetCurrentClocksEventReasons(self._h)
                for b, n in self.REASONS.items():
                    if bits & b:
                        self.reasons.add(n)
            except Exception:
                pass
            self._stop.wait(0.01)

    def __enter__(self):
        if self._nv is not None:
            self._thread = threading.Thread(target=self._run, daemon=True)
            self._thread.start()
        return self

    def __exit__(self, *a):
        self._stop.set()
        if self._thread is not None:
            self._thread.join()

    def summary(self):
        s = sorted(self.samples)
        return {'sm_mhz': s[len(s) // 2] if s else None, 'sm_max_mhz': self.max_mhz,
                'reasons': sorted(self.reasons), 'samples': len(s)}


# ------------------------------------------------------------------------------------------------------
# reference (CPU) arm
# ------------------------------------------------------------------------------------------------------
def reference_step(cfg: Config, ts):
    """Forward + backward with the reference's own CPU kernels (oracle/_ref), float32."""
    name = f"deform_conv{'_transpose' if cfg.transposed else ''}{cfg.dim}d"
    op = getattr(torch.ops.tvdcn_ref, name)
    bop = getattr(torch.ops.tvdcn_ref, '_' + name + '_backward')
    if cfg.transposed:
        args = (cfg.stride, cfg.padding, (0,) * cfg.dim, cfg.dilation, cfg.groups)
    else:
        args = (cfg.stride, cfg.padding, cfg.dilation, cfg.groups)
    mask = ts['m']
    if cfg.softmax_mask:  # the reference's mask_softmax is a torch.softmax over the taps
        b = mask.shape[0]
        logits = mask
        mask = torch.softmax(logits.view(b, cfg.mask_groups, cfg.taps, -1), 2).view_as(logits)
    out = op(ts['x'], ts['w'], ts['off'], mask, ts['bias'], *args)
    grads = bop(ts['go'], ts['x'], ts['w'], ts['off'], mask, ts['bias'], *args)
    if cfg.softmax_mask:
        y = mask.view(b, cfg.mask_groups, cfg.taps, -1)
        gm = grads[3].view_as(y)
        _ = y * (gm - (gm * y).sum(2, keepdim=True))
    return out, grads


def load_reference():
    from oracle import build_ref
    if build_ref.load():
        return True
    if build_ref.reference_present():
        build_ref.build()
        return build_ref.load()
    return False


def time_reference(cfg: Config, sample_batch: int, steps: int, warmup: int, seed: int):
    torch.set_num_threads(os.cpu_count() or 1)
    ts = make_inputs(cfg, sample_batch, seed)
    for _ in range(warmup):
        reference_step(cfg, ts)
    t0 = time.perf_counter()
    for _ in range(steps):
        reference_step(cfg, ts)
    dt = (time.perf_counter() - t0) / max(steps, 1)
    return sample_batch / dt, dt


def reference_sample_size(cfg: Config, wanted: float) -> int:
    """Images per timed pass of the reference: the reference works through the batch in blocks of
    n_parallel_imgs = the largest divisor of the batch that is <= 32 (32 at the configurations' full sizes), so
    the sample is a multiple of 32 wherever the configuration has that many images -- its blocking, column
    buffer and GEMM shapes are then the ones of the full workload."""
    nb = int(max(1, min(cfg.batch, wanted)))
    if cfg.batch >= 32:
        nb = max(32, nb // 32 * 32)
    return nb


def cpu_baseline(cfg: Config, seed: int, budget_s: float = 15.0):
    """Bounded sample of the workload on the host cores: about `budget_s` seconds of CPU work."""
    if not load_reference():
        return None
    probe = min(2, cfg.batch)
    ips, dt = time_reference(cfg, probe, 1, 1, seed)
    per_image = dt / probe
    nb = reference_sample_size(cfg, budget_s / 2 / max(per_image, 1e-9))
    ips, dt = time_reference(cfg, nb, 2, 0, seed)
    return {'value': ips, 'unit': 'images/s', 'cores': os.cpu_count(), 'kind': 'reference',
            'sample': f'{nb} of {cfg.batch} images of the same workload, fp32, 2 timed fwd+bwd passes, '
                      f'{dt:.2f} s each; torch threads {torch.get_num_threads()}, '
                      f'OpenMP loops on all {os.cpu_count()} cores, scatter loop serial as in the reference'}


def reference_cuda_baseline(cfg: Config, ts, device, steps: int = 5, warmup: int = 2):
    """The reference's CUDA backend (im2col + cuBLAS + atomic col2im, fp32) on the same device-resident step."""
    from oracle import build_ref
    if not build_ref.load_cuda():
        return {'unavailable': 'oracle/_ref/libtvdcn_ref_cuda.so is not built (python oracle/build_ref.py --cuda)'}
    dts = {k: v.to(device) for k, v in ts.items()}
    secs = timed(lambda: reference_step(cfg, dts), steps, warmup, lambda: None)
    batch = dts['x'].shape[0]
    return {'value': batch * steps / secs, 'unit': 'images/s', 'ms_per_step': secs / steps * 1e3, 'dtype': 'f32',
            'steps': steps, 'kind': "reference CUDA kernels built from the reference sources for sm_100, "
                                    "torch's cuBLAS GEMMs, TF32 off"}


def run_reference_arm(args, cfg):
    rank = int(os.environ.get('RANK', '0'))
    if rank != 0:
        return
    if not load_reference():
        emit(json.dumps({'impl': 'reference', 'unavailable': 'oracle/_ref is not built and the reference '
                          'checkout is not present on this machine'}))
        return
    seed = 1000 + args.config
    probe = min(2, cfg.batch)
    _, dt = time_reference(cfg, probe, 1, 1, seed)
    total = max(args.steps + args.warmup, 1)
    nb = reference_sample_size(cfg, 120.0 / total / max(dt / probe, 1e-9))
    ips, dt = time_reference(cfg, nb, args.steps, args.warmup, seed)
    flops = 3 * cfg.flops_per_pass(nb)
    line = {
        'impl': 'reference', 'metric': METRIC, 'value': ips, 'unit': 'images/s', 'n_gpus': args.gpus,
        'steps': args.steps, 'warmup': args.warmup, 'ms_per_step': dt * 1e3, 'higher_is_better': True,
        'scaling': args.scaling, 'vs_baseline': None, 'dtype': 'f32', 'data': 'synthetic (seeded, CPU generator)',
        'config': {'workload': cfg.name, 'sample_images_per_step': nb},
        'effective_tflops': flops / dt / 1e12,
        'cpu_baseline': {'value': ips, 'unit': 'images/s', 'cores': os.cpu_count(), 'kind': 'reference',
                         'sample': f'{nb} of {cfg.batch} images per step, fp32, reference CPU kernels built from '
                                   f'the reference sources (oracle/build_ref.py)'},
        'e2e': {'value': ips, 'unit': 'images/s', 'h2d_bytes_per_step': 0, 'd2h_bytes_per_step': 0},
        'gpu_launches': 0,
    }
    emit(json.dumps(line))


# ------------------------------------------------------------------------------------------------------
# our arm
# ------------------------------------------------------------------------------------------------------
METRIC = 'deform_conv fwd+bwd images/s'


def peaks():
    path = os.path.join(ROOT, 'MEASURED_PEAKS.json')
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return {'hbm_gbs': p['hbm_gbs'], 'tflops_burst': p['bf16_tflops'],
                'tflops_sustained': p.get('bf16_tflops_sustained', p['bf16_tflops']), 'source': 'measured'}
    return {'hbm_gbs': 6650.0, 'tflops_burst': 1590.0, 'tflops_sustained': 1400.0, 'source': 'fallback'}


def known_traffic(kernel: str, config: int, mode: str):
    """DRAM bytes per launch (dram__bytes_read.sum + dram__bytes_write.sum) from the ncu captures summarised
    under profiles/; None where no capture exists.  The figures are for the configuration's full batch on one GPU."""
    table = {
        # config 2: full-size launches (profiles/config2_tensor_kernels.md)
        'dcn_fwd_tc/cfg2/bf16': 85.16e6 + 20.91e6,
        'dcn_dgrad_tc/cfg2/bf16': 330.5e6 + 102.6e6,
        'dcn_wgrad_tc/cfg2/bf16': 137.7e6 + 3.81e6,
        'dcn_fwd_tc/cfg2/fp32': 137.8e6 + 64.83e6,
        'dcn_dgrad_tc/cfg2/fp32': 487.1e6 + 116.9e6,
        'dcn_wgrad_tc/cfg2/fp32': 243.0e6 + 7.46e6,
        # configs 3-5: captured on a cut batch (profiles/config3_config4_config5_tensor_kernels.md) and scaled to
        # the full batch by the images processed -- tiles are independent, traffic grows in proportion
        'dcn_fwd_tc/cfg3/fp32': (73.8e6 + 29.55e6) * 8,
        'dcn_dgrad_tc/cfg3/fp32': (214.6e6 + 44.33e6) * 8,
        'dcn_wgrad_tc/cfg3/fp32': (141.5e6 + 4.76e6) * 8,
        'dcn_fwd_tc/cfg4/fp32': (70.56e6 + 7.59e6) * 4,
        'dcn_dgrad_tc/cfg4/fp32': (229.9e6 + 61.28e6) * 4,
        'dcn_wgrad_tc/cfg4/fp32': (95.28e6 + 3.93e6) * 4,
        'dcn_fwd_tc/cfg5/fp32': (40.98e6 + 0.15e6) * 4,
        'dcn_dgrad_tc/cfg5/fp32': (58.56e6 + 0.50e6 + 63.9e6 + 1.27e6) / 2 * 4,   # two launches per step, mean
        'dcn_wgrad_tc/cfg5/fp32': (57.76e6 + 0.70e6) * 4,
    }
    return table.get(f'{kernel}/cfg{config}/{mode}')


class DeviceStep:
    """The step on device-resident tensors, straight through the C ABI with preallocated outputs."""

    def __init__(self, cfg: Config, ts, mode: str, device, bucket):
        from tvdcn_b200 import cabi
        self.cfg, self.cabi, self.L = cfg, cabi, cabi.lib()
        dt = torch.bfloat16 if mode == 'bf16' else torch.float32
        self.x = ts['x'].to(device, dt)
        self.w = ts['w'].to(device, dt)
        self.go = ts['go'].to(device, dt)
        self.off = ts['off'].to(device)
        self.m_in = ts['m'].to(device)
        self.bias = ts['bias'].to(device)
        self.mask = torch.empty_like(self.m_in) if cfg.softmax_mask else self.m_in
        self.out = torch.empty_like(self.go)
        self.gx = torch.empty_like(self.x)
        self.goff = torch.empty_like(self.off)
        self.gmask = torch.empty_like(self.mask)
        self.glogits = torch.empty_like(self.mask) if cfg.softmax_mask else None
        if dt == torch.float32:
            self.gw, self.gb = bucket.weight_view, bucket.bias_view
            self.gw16 = None
        else:  # 16-bit weight gradient is written in bf16, then widened into the f32 bucket
            self.gw16 = torch.empty_like(self.w)
            self.gw, self.gb = self.gw16, bucket.bias_view
        self.bucket = bucket
        code = {torch.float32: cabi.F32, torch.bfloat16: cabi.BF16}[dt]
        self.p = cabi.make_problem(cfg.dim, cfg.transposed, code, self.x.shape[0], cfg.cin, cfg.cout, cfg.in_size,
                                   cfg.kernel, cfg.stride, cfg.padding, cfg.dilation, cfg.groups,
                                   cfg.offset_groups, cfg.mask_groups, None, cabi.F32)
        # the backward call follows the forward call on the same workspace: it may reuse the staged input
        self.p_bwd = cabi.Problem.from_buffer_copy(self.p)
        self.p_bwd.flags = cabi.FLAG_REUSE_STAGED_INPUT
        pp = ctypes.byref(self.p)
        n = max(self.L.tvdcn_b200_forward_workspace_bytes(pp), self.L.tvdcn_b200_backward_workspace_bytes(pp), 256)
        self.ws = torch.empty(n, dtype=torch.uint8, device=device)
        self.engine = (self.L.tvdcn_b200_engine_name(pp, 0).decode(), self.L.tvdcn_b200_engine_name(pp, 1).decode())
        self.gw_ready = torch.cuda.Event()
        self.gw_ready.record()      # creates the underlying cudaEvent_t
        import torch.distributed as dist
        # only a step with an exchange asks for the "weight gradient ready" event (the call then puts the weight
        # gradient first); a single GPU has nobody waiting for it
        self.exchange = dist.is_available() and dist.is_initialized() and dist.get_world_size() > 1
        self.copy_stream = torch.cuda.Stream(device, priority=-1)
        self.gw_copied = torch.cuda.Event()

    def __call__(self):
        cfg, L, cabi = self.cfg, self.L, self.cabi
        vp = lambda t: ctypes.c_void_p(t.data_ptr())
        st = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
        pp = ctypes.byref(self.p)
        b = self.x.shape[0]
        sp = math.prod(cfg.grid)
        if cfg.softmax_mask:
            cabi.check(L.tvdcn_b200_mask_softmax_forward(cabi.F32, b, cfg.mask_groups, cfg.taps, sp, vp(self.m_in),
                                                         vp(self.mask), st))
        cabi.check(L.tvdcn_b200_deform_conv_forward(pp, vp(self.x), vp(self.w), vp(self.off), vp(self.mask),
                                                    vp(self.bias), vp(self.out), vp(self.ws), self.ws.numel(), st))
        # the event is recorded when grad_weight / grad_bias are final (on the library's second stream, while the
        # scatter kernel still runs): the all-reduce starts there, not at the end of the backward pass
        cabi.check(L.tvdcn_b200_deform_conv_backward_ex(ctypes.byref(self.p_bwd), vp(self.go), vp(self.x),
                                                        vp(self.w), vp(self.off), vp(self.mask), vp(self.gx),
                                                        vp(self.gw), vp(self.goff), vp(self.gmask), vp(self.gb),
                                                        vp(self.ws), self.ws.numel(), st,
                                                        ctypes.c_void_p(self.gw_ready.cuda_event)
                                                        if self.exchange else None))
        if self.gw16 is not None and self.exchange:
            # 16-bit grad_weight goes into the f32 bucket on a stream of its own, behind the same event
            self.copy_stream.wait_event(self.gw_ready)
            with torch.cuda.stream(self.copy_stream):
                self.bucket.weight_view.copy_(self.gw16)
                self.gw_copied.record(self.copy_stream)
            self.bucket.all_reduce_async(after=self.gw_copied)
        elif self.gw16 is not None:
            self.bucket.weight_view.copy_(self.gw16)
            self.bucket.all_reduce_async()
        else:
            self.bucket.all_reduce_async(after=self.gw_ready if self.exchange else None)
        if cfg.softmax_mask:
            cabi.check(L.tvdcn_b200_mask_softmax_backward(cabi.F32, b, cfg.mask_groups, cfg.taps, sp, vp(self.gmask),
                                                          vp(self.mask), vp(self.glogits), st))
        self.bucket.wait()


class HostStep:
    """The step a user of the public API runs when the data lives in host memory.

    Three streams, as a training loop with a prefetching loader runs it: a copy-in stream brings step i+1's
    inputs from pinned host memory into the second of two device buffer sets while the compute stream runs
    step i through the public operators, and a copy-out stream writes step i-1's results (output, all
    gradients) to pinned host memory.  Every step's inputs and results cross PCIe inside the timed region;
    `finish()` makes the compute stream wait for the last copy-out so that the closing event covers it.
    """
    NAMES = ('x', 'off', 'm', 'go')

    def __init__(self, cfg: Config, ts_pinned, mode: str, device, bucket):
        import tvdcn_b200
        self.ops = tvdcn_b200.ops
        self.cfg, self.mode, self.device, self.bucket = cfg, mode, device, bucket
        self.dt = torch.bfloat16 if mode == 'bf16' else torch.float32
        # host tensors in the data type the operator consumes (bf16 images for the bf16 mode)
        self.host_in = {}
        for k in self.NAMES:
            t = ts_pinned[k]
            if k in ('x', 'go') and self.dt != t.dtype:
                t = t.to(self.dt).pin_memory()
            self.host_in[k] = t
        self.dev_in = [{k: torch.empty(v.shape, dtype=v.dtype, device=device) for k, v in self.host_in.items()}
                       for _ in range(2)]
        self.w = ts_pinned['w'].to(device, self.dt).requires_grad_(True)
        self.bias = ts_pinned['bias'].to(device).requires_grad_(True)
        self.s_in, self.s_out = torch.cuda.Stream(device), torch.cuda.Stream(device)
        self.in_done = [None, None]      # event: inputs of the step that uses buffer set b have landed
        self.comp_done = [None, None]    # event: the step that used buffer set b has finished
        self.out_done = [None, None]     # event: results of that step are in host memory
        self.keep = [None, None]         # device results, alive until their copy-out has been waited for
        self.host_out = [None, None]
        self.step = 0
        self.h2d = sum(v.numel() * v.element_size() for v in self.host_in.values())
        self.d2h = 0

    def _copy_in(self, b):
        """Queue the host -> device copies into buffer set b (after the step that last read it)."""
        if self.comp_done[b] is not None:
            self.s_in.wait_event(self.comp_done[b])
        with torch.cuda.stream(self.s_in):
            for k in self.NAMES:
                self.dev_in[b][k].copy_(self.host_in[k], non_blocking=True)
            ev = torch.cuda.Event()
            ev.record(self.s_in)
        self.in_done[b] = ev

    def __call__(self):
        cfg, ops = self.cfg, self.ops
        cur = torch.cuda.current_stream(self.device)
        b = self.step & 1
        if self.in_done[b] is None:
            self._copy_in(b)                       # first step: nothing was prefetched
        cur.wait_event(self.in_done[b])
        self.in_done[b] = None
        if self.out_done[b] is not None:           # results of step - 2 may be freed only after their copy-out
            cur.wait_event(self.out_done[b])
        self.keep[b] = None
        d = self.dev_in[b]
        x = d['x'].detach().requires_grad_(True)
        off = d['off'].detach().requires_grad_(True)
        m = d['m'].detach().requires_grad_(True)
        go = d['go']
        mask = getattr(ops, f'mask_softmax{cfg.dim}d')(m, cfg.kernel) if cfg.softmax_mask else m
        self.w.grad = None
        self.bias.grad = None
        if cfg.transposed:
            out = getattr(ops, f'deform_conv_transpose{cfg.dim}d')(x, self.w, off, mask, self.bias, cfg.stride,
                                                                   cfg.padding, 0, cfg.dilation, cfg.groups)
        else:
            out = getattr(ops, f'deform_conv{cfg.dim}d')(x, self.w, off, mask, self.bias, cfg.stride, cfg.padding,
                                                         cfg.dilation, cfg.groups)
        out.backward(go)
        self.bucket.weight_view.copy_(self.w.grad)
        self.bucket.bias_view.copy_(self.bias.grad)
        self.bucket.all_reduce_async()
        self.bucket.wait()
        results = [out.detach(), x.grad, off.grad, m.grad, self.bucket.flat.clone()]
        ev = torch.cuda.Event()
        ev.record(cur)
        self.comp_done[b] = ev
        # next step's inputs into the other buffer set, this step's results out
        self._copy_in(b ^ 1)
        if self.host_out[b] is None:
            self.host_out[b] = [torch.empty(r.shape, dtype=r.dtype, pin_memory=True) for r in results]
            self.d2h = sum(h.numel() * h.element_size() for h in self.host_out[b])
        self.s_out.wait_event(ev)
        with torch.cuda.stream(self.s_out):
            for h, r in zip(self.host_out[b], results):
                h.copy_(r, non_blocking=True)
            eo = torch.cuda.Event()
            eo.record(self.s_out)
        self.out_done[b] = eo
        self.keep[b] = results
        self.step += 1

    def finish(self):
        """Order the compute stream after every queued copy-out (call before the closing event)."""
        cur = torch.cuda.current_stream(self.device)
        for ev in self.out_done:
            if ev is not None:
                cur.wait_event(ev)


class OperatorStep:
    """The device-resident step through the public operators (torch.ops.tvdcn.* via tvdcn_b200.ops, autograd):
    every call allocates its outputs and workspace and stages its own inputs, unlike the C-ABI step of `value`."""

    def __init__(self, cfg: Config, ts, mode: str, device):
        import tvdcn_b200
        self.ops, self.cfg = tvdcn_b200.ops, cfg
        dt = torch.bfloat16 if mode == 'bf16' else torch.float32
        self.x = ts['x'].to(device, dt).requires_grad_(True)
        self.w = ts['w'].to(device, dt).requires_grad_(True)
        self.go = ts['go'].to(device, dt)
        self.off = ts['off'].to(device).requires_grad_(True)
        self.m = ts['m'].to(device).requires_grad_(True)
        self.bias = ts['bias'].to(device).requires_grad_(True)

    def __call__(self):
        cfg, ops = self.cfg, self.ops
        for t in (self.x, self.w, self.off, self.m, self.bias):
            t.grad = None
        mask = getattr(ops, f'mask_softmax{cfg.dim}d')(self.m, cfg.kernel) if cfg.softmax_mask else self.m
        if cfg.transposed:
            out = getattr(ops, f'deform_conv_transpose{cfg.dim}d')(self.x, self.w, self.off, mask, self.bias,
                                                                   cfg.stride, cfg.padding, 0, cfg.dilation, cfg.groups)
        else:
            out = getattr(ops, f'deform_conv{cfg.dim}d')(self.x, self.w, self.off, mask, self.bias, cfg.stride,
                                                         cfg.padding, cfg.dilation, cfg.groups)
        out.backward(self.go)


def timed(fn, steps, warmup, barrier):
    for _ in range(warmup):
        fn()
    barrier()
    torch.cuda.synchronize()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for _ in range(steps):
        fn()
    if hasattr(fn, 'finish'):
        fn.finish()
    stop.record()
    torch.cuda.synchronize()
    barrier()
    return start.elapsed_time(stop) / 1e3  # seconds for all steps


_RESULT_FD = None


def claim_stdout():
    """Keep stdout for the one JSON line: whatever libraries print to file descriptor 1 (NCCL's version banner,
    for one) goes to stderr from here on."""
    global _RESULT_FD
    if _RESULT_FD is None:
        sys.stdout.flush()
        _RESULT_FD = os.dup(1)
        os.dup2(2, 1)


def emit(line: str):
    sys.stdout.flush()
    if _RESULT_FD is None:
        print(line, flush=True)
    else:
        os.write(_RESULT_FD, (line + '\n').encode())


def dominant_roofline(cfg: Config, kernels: dict, batch: int, config_index: int, mode: str, pk: dict):
    """Roofline entry of the kernel with the largest share of the step."""
    gemm_like = {'sample_gemm', 'gemm_scatter', 'sample_wgrad', 'dcn_fwd_tc', 'dcn_wgrad_tc', 'dcn_dgrad_tc'}
    if not kernels:
        return None
    dom = max(kernels, key=lambda k: kernels[k]['ms_per_step'])
    ms = kernels[dom]['ms_per_launch']
    traffic = known_traffic(dom, config_index, mode)
    if traffic is not None:
        traffic *= batch / cfg.batch      # the captures are for the whole batch; traffic grows with the images
    if cfg.bound == 'tensor' and dom in gemm_like:
        ach = cfg.flops_per_pass(batch) / (ms / 1e3) / 1e12
        # a kernel of about a millisecond timed by events between other kernels: the burst figure is the denominator
        peak = pk['tflops_burst']
        return {'kernel': dom, 'bound': 'tensor', 'achieved': ach, 'peak': peak, 'unit': 'TFLOP/s',
                'frac': ach / peak, 'frac_of_sustained': ach / pk['tflops_sustained'],
                'traffic': traffic,
                'peak_source': pk['source'] + ' bf16 dense, burst (of measured)',
                'note': 'algorithmic FLOPs of one GEMM pass (2*Cout*Cin/g*taps*N*P) / CUDA-event time'}
    # share of the step's algorithmic bytes: a GEMM-shaped kernel touches about a third of them
    share = cfg.algorithmic_bytes(batch) / 3 if dom in gemm_like else cfg.algorithmic_bytes(batch)
    ach = share / (ms / 1e3) / 1e9
    return {'kernel': dom, 'bound': 'hbm', 'achieved': ach, 'peak': pk['hbm_gbs'], 'unit': 'GB/s',
            'frac': ach / pk['hbm_gbs'], 'traffic': traffic,
            'peak_source': pk['source'] + ' copy bandwidth (of measured)'}


def measure_mode(cfg: Config, config_index: int, mode: str, ts, batch: int, device, bucket, world: int, barrier,
                 args, L, local: int, want_e2e: bool):
    """One data mode of the step on this rank's batch shard: device-resident throughput, per-kernel times, the
    roofline of the dominant kernel, the end-to-end figure and the clocks seen during the timed region."""
    import torch.distributed as dist
    step = DeviceStep(cfg, ts, mode, device, bucket)
    with ClockSampler(local) as clocks:
        for _ in range(args.warmup):
            step()
        launches1 = L.tvdcn_b200_launch_count()
        secs = timed(step, args.steps, 0, barrier)
        launches2 = L.tvdcn_b200_launch_count()
    t = torch.tensor([secs], device=device, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    secs = t.item()
    global_batch = batch_total(batch, device, world)
    value = global_batch * args.steps / secs

    # per-kernel durations for the roofline: same step, kernels bracketed by CUDA events
    L.tvdcn_b200_timing_enable(1)
    ksteps = max(3, min(args.steps, 10))
    for _ in range(ksteps):
        step()
    torch.cuda.synchronize()
    L.tvdcn_b200_timing_enable(0)
    buf = ctypes.create_string_buffer(1 << 14)
    L.tvdcn_b200_timing_report(buf, len(buf))
    kernels = {}
    for line in buf.value.decode().splitlines():
        name, n, ms = line.split()
        kernels[name] = {'launches_per_step': int(n) / ksteps, 'ms_per_launch': float(ms) / int(n),
                         'ms_per_step': float(ms) / ksteps}
    pk = peaks()
    roofline = dominant_roofline(cfg, kernels, batch, config_index, mode, pk)

    # the same step through the public operators (fresh workspace and outputs per call, no staging reuse), still on
    # device-resident tensors: what a PyTorch user of the operators sees beside the C-ABI figure above
    e2e = None
    ops_step_ms = None
    if want_e2e:
        host = HostStep(cfg, ts, mode, device, bucket)
        esteps = max(3, min(args.steps, 10))
        esecs = timed(host, esteps, 2, barrier)
        t = torch.tensor([esecs], device=device, dtype=torch.float64)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e = {'value': global_batch * esteps / t.item(), 'unit': 'images/s', 'h2d_bytes_per_step': host.h2d,
               'd2h_bytes_per_step': host.d2h, 'steps': esteps}
        ops = OperatorStep(cfg, ts, mode, device)
        ops_step_ms = timed(ops, esteps, 2, barrier) / esteps * 1e3
    step_s = secs / args.steps
    flops = 3 * cfg.flops_per_pass(global_batch)
    nbytes = cfg.algorithmic_bytes(global_batch, 4 if mode == 'fp32' else 2)
    return {
        'value': value, 'unit': 'images/s', 'ms_per_step': step_s * 1e3,
        'dtype': 'f32' if mode == 'fp32' else 'bf16 input/weight, f32 accumulate, f32 offset/mask',
        'effective_tflops': flops / step_s / 1e12,
        'tensor_frac_of_peak': flops / step_s / 1e12 / pk['tflops_sustained'] / world,
        'algorithmic_gbs': nbytes / step_s / 1e9,
        'hbm_frac_of_peak': nbytes / step_s / 1e9 / pk['hbm_gbs'] / world,
        'kernels': kernels, 'roofline': roofline, 'e2e': e2e, 'operator_step_ms': ops_step_ms,
        'gpu_launches': int(launches2 - launches1), 'clocks': clocks.summary(), 'engine_fwd_bwd': step.engine,
    }, step


def batch_total(batch: int, device, world: int) -> int:
    """Images all ranks process per step (the shards may differ by one image)."""
    if world == 1:
        return batch
    import torch.distributed as dist
    t = torch.tensor([batch], device=device, dtype=torch.int64)
    dist.all_reduce(t)
    return int(t.item())


def allreduce_overlap(step, device):
    """One diagnostic step (outside the timed regions): where the all-reduce of the weight gradients runs relative
    to the backward pass, from CUDA events.  Times in ms since the start of the step."""
    bucket = step.bucket
    torch.cuda.synchronize()
    t0, t_end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    bucket.timing = []
    t0.record()
    step()
    t_end.record()
    torch.cuda.synchronize()
    ev = bucket.timing
    bucket.timing = None
    if not ev:
        return None
    return {'allreduce_start_ms': t0.elapsed_time(ev[0]), 'allreduce_end_ms': t0.elapsed_time(ev[1]),
            'step_end_ms': t0.elapsed_time(t_end),
            'note': 'the exchange starts when the weight-gradient kernel finishes on the second stream and ends '
                    'before the step does: it runs under the scatter kernel'}


def check_reduced_gradient(cfg: Config, step, ts_global, device, world: int, rank: int):
    """Outside every timed region: the all-reduced [grad_weight | grad_bias] must equal (a) the sum of the ranks'
    own buckets and (b), on rank 0, the gradient one GPU computes for the whole global batch.  Returns the two
    normalised max errors (rank 0), which must be <= 1e-5 for f32 data."""
    import torch.distributed as dist
    from tvdcn_b200.data_parallel import GradBucket
    bucket = step.bucket
    step()                                   # fills and all-reduces the bucket
    torch.cuda.synchronize()
    reduced = bucket.flat.clone()
    # (a) local buckets: the same step with the exchange switched off
    saved = bucket.all_reduce_async
    bucket.all_reduce_async = lambda *a, **k: None
    step()
    torch.cuda.synchronize()
    bucket.all_reduce_async = saved
    local = bucket.flat.clone()
    parts = [torch.empty_like(local) for _ in range(world)]
    dist.all_gather(parts, local)
    total = torch.stack(parts).double().sum(0)
    denom = total.abs().max().clamp_min(1e-30)
    err_sum = ((reduced.double() - total).abs().max() / denom).item()
    err_one = None
    if rank == 0 and ts_global is not None:
        solo = GradBucket(ts_global['w'].shape, cfg.cout, dtype=torch.float32, device=device)
        solo.all_reduce_async = lambda *a, **k: None     # rank 0 alone: no collective
        one = DeviceStep(cfg, ts_global, 'fp32', device, solo)
        one()
        torch.cuda.synchronize()
        err_one = ((reduced.double() - solo.flat.double()).abs().max() / denom).item()
        del one, solo
    return {'vs_sum_of_rank_buckets': err_sum, 'vs_one_gpu_whole_batch': err_one, 'tolerance': 1e-5}


def main():
    claim_stdout()
    ap = argparse.ArgumentParser()
    ap.add_argument('--gpus', type=int, default=1)
    ap.add_argument('--steps', type=int, default=50)
    ap.add_argument('--warmup', type=int, default=5)
    ap.add_argument('--config', type=int, default=2, choices=sorted(CONFIGS))
    ap.add_argument('--mode', default='fp32', choices=['fp32', 'bf16'],
                    help='data mode of the headline figures; the other mode of configurations 2 and 5 is measured in '
                         'the same run and reported under "modes"')
    ap.add_argument('--impl', default='ours', choices=['ours', 'reference'])
    ap.add_argument('--scaling', default='strong', choices=['strong', 'weak'],
                    help='strong (default): the configuration\'s batch is sharded over the GPUs; weak: every GPU '
                         'gets the configuration\'s whole batch')
    ap.add_argument('--batch', type=int, default=0, help='global batch (default: the configuration\'s)')
    ap.add_argument('--no-cpu-baseline', action='store_true')
    ap.add_argument('--no-e2e', action='store_true')
    ap.add_argument('--no-other-mode', action='store_true', help='measure only --mode')
    ap.add_argument('--no-ref-cuda', action='store_true',
                    help="skip timing the reference's own CUDA backend (oracle/_ref/libtvdcn_ref_cuda.so, fp32) on "
                         'this GPU, reported as "reference_cuda" (1 GPU only)')
    args = ap.parse_args()
    cfg = CONFIGS[args.config]
    if args.warmup < 3 and args.impl == 'ours':
        args.warmup = 3

    if args.impl == 'reference':
        run_reference_arm(args, cfg)
        return

    import torch.distributed as dist
    from tvdcn_b200 import cabi
    from tvdcn_b200.data_parallel import GradBucket, shard_bounds

    world = int(os.environ.get('WORLD_SIZE', '1'))
    rank = int(os.environ.get('RANK', '0'))
    local = int(os.environ.get('LOCAL_RANK', '0'))
    assert torch.cuda.is_available(), 'bench.py needs a CUDA device; there is no CPU fallback'
    torch.cuda.set_device(local)
    device = torch.device('cuda', local)
    if world > 1:
        # the exchange's kernel needs only a few SMs, but needs them while the scatter kernel holds them all: on a
        # high-priority stream its CTAs go first whenever an SM frees up
        dist.init_process_group('nccl', device_id=device,
                                pg_options=dist.ProcessGroupNCCL.Options(is_high_priority_stream=True))
    barrier = (lambda: dist.barrier()) if world > 1 else (lambda: None)

    # Strong scaling: every rank generates the same global batch (CPU generator, seed 1000 + config) and keeps its
    # contiguous slice; weights and bias are replicas.  Weak scaling: every rank has a whole batch of its own.
    global_batch = args.batch or cfg.batch
    pin = not args.no_e2e
    ts_global = None
    if args.scaling == 'strong':
        ts_global = make_inputs(cfg, global_batch, 1000 + args.config)
        b0, b1 = shard_bounds(global_batch, rank, world)
        ts = {k: (v if k in ('w', 'bias') else v[b0:b1].contiguous()) for k, v in ts_global.items()}
        if pin:
            ts = {k: v.pin_memory() for k, v in ts.items()}
        batch = b1 - b0
        if world == 1 or rank != 0:
            ts_global = None
    else:
        batch = global_batch
        ts = make_inputs(cfg, batch, 1000 + args.config + 7919 * rank, pin=pin)
    assert batch > 0, 'more GPUs than images'
    bucket = GradBucket(ts['w'].shape, cfg.cout, dtype=torch.float32, device=device)
    L = cabi.lib()
    L.tvdcn_b200_timing_enable.argtypes = [ctypes.c_int]
    L.tvdcn_b200_timing_report.argtypes = [ctypes.c_char_p, ctypes.c_size_t]
    L.tvdcn_b200_timing_report.restype = ctypes.c_size_t

    head, step = measure_mode(cfg, args.config, args.mode, ts, batch, device, bucket, world, barrier, args, L, local,
                              not args.no_e2e)
    grad_check, overlap = None, None
    if world > 1 and args.mode == 'fp32':
        grad_check = check_reduced_gradient(cfg, step, ts_global, device, world, rank)
        overlap = allreduce_overlap(step, device)
    del step
    modes = {}
    other = 'bf16' if args.mode == 'fp32' else 'fp32'
    if not args.no_other_mode and args.config in (2, 5):
        modes[other], _ = measure_mode(cfg, args.config, other, ts, batch, device, bucket, world, barrier, args, L,
                                       local, not args.no_e2e)
        del _
    # the other way of scaling, device-resident figure only
    weak = None
    if world > 1 and args.scaling == 'strong':
        tw = make_inputs(cfg, cfg.batch, 1000 + args.config + 7919 * rank)
        wstep = DeviceStep(cfg, tw, args.mode, device, bucket)
        wsecs = timed(wstep, args.steps, args.warmup, barrier)
        t = torch.tensor([wsecs], device=device, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        weak = {'value': cfg.batch * world * args.steps / t.item(), 'unit': 'images/s',
                'ms_per_step': t.item() / args.steps * 1e3, 'per_gpu_batch': cfg.batch}
        del wstep, tw

    base = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        base = cpu_baseline(cfg, 1000 + args.config)

    ref_cuda = None
    if rank == 0 and world == 1 and not args.no_ref_cuda:
        try:
            ref_cuda = reference_cuda_baseline(cfg, ts, device)
        except Exception as e:  # a baseline must never cost the measurement
            ref_cuda = {'unavailable': f'{type(e).__name__}: {e}'[:200]}

    if rank == 0:
        total = head['value'] * head['ms_per_step'] / 1e3     # images per step, all ranks
        nbytes = cfg.algorithmic_bytes(batch, 4)
        line = {
            'metric': METRIC, 'value': head['value'], 'unit': 'images/s', 'n_gpus': world, 'steps': args.steps,
            'warmup': args.warmup, 'ms_per_step': head['ms_per_step'], 'higher_is_better': True,
            'scaling': args.scaling, 'vs_baseline': None, 'dtype': head['dtype'],
            'data': 'synthetic (seeded, CPU generator)',
            'config': {'workload': cfg.name, 'config_index': args.config, 'per_gpu_batch': batch,
                       'global_batch': int(round(total)), 'parallelism': f'dp{world}',
                       'engine_fwd_bwd': head['engine_fwd_bwd'],
                       'l2': 'inputs larger than L2 (no flush needed)' if nbytes > 126e6 * 2
                             else 'working set of one rank near L2 size; not flushed'},
            'effective_tflops': head['effective_tflops'], 'tensor_frac_of_peak': head['tensor_frac_of_peak'],
            'algorithmic_gbs': head['algorithmic_gbs'], 'hbm_frac_of_peak': head['hbm_frac_of_peak'],
            'kernels': head['kernels'], 'roofline': head['roofline'], 'cpu_baseline': base,
            'reference_cuda': ref_cuda, 'e2e': head['e2e'], 'operator_step_ms': head['operator_step_ms'],
            'gpu_launches': head['gpu_launches'], 'clocks': head['clocks'],
            'modes': modes, 'weak': weak, 'grad_check': grad_check, 'allreduce_overlap': overlap,
        }
        emit(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


if __name__ == '__main__':
    main()
