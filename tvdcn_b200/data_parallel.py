"""Batch-dimension data parallelism for the deformable-convolution step.

Every image is independent in the forward pass and in grad_input / grad_offset / grad_mask; only
grad_weight and grad_bias are sums over the batch.  So each rank (one process per GPU) owns a contiguous
slice of the batch and a full replica of weight and bias, and the only exchange per step is one SUM
all-reduce over a flat buffer ``[grad_weight | grad_bias]`` (about 2.4 MB for a 256 x 256 x 3 x 3 layer).
The all-reduce runs on a side stream so that it overlaps whatever the compute stream does next.

Works with any ``torch.distributed`` backend (NCCL on GPUs, gloo in the CPU tests).
"""
from __future__ import annotations

from typing import Optional, Sequence, Tuple

import torch
import torch.distributed as dist


def shard_bounds(n_total: int, rank: int, world: int) -> Tuple[int, int]:
    """Contiguous, near-equal split of ``n_total`` items: rank r gets [begin, end)."""
    if world <= 0 or not 0 <= rank < world:
        raise ValueError(f'bad rank {rank} / world {world}')
    base, extra = divmod(n_total, world)
    begin = rank * base + min(rank, extra)
    return begin, begin + base + (1 if rank < extra else 0)


def shard_batch(tensors: Sequence[Optional[torch.Tensor]], rank: int, world: int):
    """Slice every tensor that has a batch axis (all but weight / bias are passed here) along dim 0."""
    out = []
    for t in tensors:
        if t is None:
            out.append(None)
            continue
        b, e = shard_bounds(t.shape[0], rank, world)
        out.append(t[b:e])
    return tuple(out)


class GradBucket:
    """Flat buffer that holds grad_weight and grad_bias back to back, all-reduced in one call.

    ``weight_view`` / ``bias_view`` alias the buffer, so kernels can write their gradients straight into
    it (they are passed as the grad_weight / grad_bias pointers of the backward entry point).

    For the exchange to run under the rest of the backward pass, create the NCCL process group with
    ``pg_options=ProcessGroupNCCL.Options(is_high_priority_stream=True)``: the scatter kernel occupies every SM,
    and a collective kernel of normal priority only gets SMs in that kernel's last wave.
    """

    def __init__(self, weight_shape, bias_elems: int, dtype=torch.float32, device='cpu', group=None):
        wn = 1
        for s in weight_shape:
            wn *= s
        self.flat = torch.zeros(wn + bias_elems, dtype=dtype, device=device)
        self.weight_view = self.flat[:wn].view(*weight_shape)
        self.bias_view = self.flat[wn:] if bias_elems else None
        self.group = group
        self._work = None
        self._event = None
        self._side = torch.cuda.Stream(device=device) if self.flat.is_cuda else None
        self.timing = None      # set to [] to have the next all_reduce_async bracket the exchange with timing events

    def all_reduce_async(self, after: Optional["torch.cuda.Event"] = None) -> None:
        """Start the SUM all-reduce.  On CUDA it is ordered after the current stream's work so far, or, when
        ``after`` is given, only after that event (the "weight gradient ready" event of the backward call), so
        that it runs under the rest of the backward pass."""
        if not dist.is_initialized() or dist.get_world_size(self.group) == 1:
            return
        if self._side is not None:
            if after is not None:
                self._side.wait_event(after)
            else:
                self._side.wait_stream(torch.cuda.current_stream(self.flat.device))
            with torch.cuda.stream(self._side):
                if self.timing is not None:      # [start, end] events of this exchange, for overlap diagnostics
                    self.timing = [torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)]
                    self.timing[0].record(self._side)
                dist.all_reduce(self.flat, op=dist.ReduceOp.SUM, group=self.group)
                if self.timing is not None:
                    self.timing[1].record(self._side)
                self._event = torch.cuda.Event()
                self._event.record(self._side)
        else:
            self._work = dist.all_reduce(self.flat, op=dist.ReduceOp.SUM, group=self.group, async_op=True)

    def wait(self) -> None:
        """Make the current stream (or the host, on CPU) wait for the all-reduce."""
        if self._event is not None:
            torch.cuda.current_stream(self.flat.device).wait_event(self._event)
            self._event = None
        if self._work is not None:
            self._work.wait()
            self._work = None
