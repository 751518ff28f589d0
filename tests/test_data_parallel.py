"""World-size-2 gloo run of the batch-sharded step on CPU: shards + one bucket all-reduce reproduce the
single-process gradients.  The compute is the CPU oracle; only the sharding / exchange logic is under test."""
import os
import sys

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import cases
from tvdcn_b200.data_parallel import GradBucket, shard_batch, shard_bounds


def test_shard_bounds_cover_the_batch():
    for n in (0, 1, 7, 128):
        for w in (1, 2, 3, 8):
            spans = [shard_bounds(n, r, w) for r in range(w)]
            assert spans[0][0] == 0 and spans[-1][1] == n
            assert all(a[1] == b[0] for a, b in zip(spans, spans[1:]))
            sizes = [e - b for b, e in spans]
            assert max(sizes) - min(sizes) <= 1
    with pytest.raises(ValueError):
        shard_bounds(4, 2, 2)


def _worker(rank, world, port, transposed, ret):
    os.environ['MASTER_ADDR'] = '127.0.0.1'
    os.environ['MASTER_PORT'] = str(port)
    dist.init_process_group('gloo', rank=rank, world_size=world)
    try:
        case = cases.reference_fixture(2, transposed, True, True, groups=2, offset_groups=4, mask_groups=2, batch=5)
        x, w, off, mask, bias, go = cases.make_inputs(case, seed=31)
        xs, offs, masks, gos = shard_batch((x, off, mask, go), rank, world)
        res = cases.run_oracle(cases.Case(**{**case.__dict__, 'batch': xs.shape[0]}), xs, w, offs, masks, bias, gos)
        bucket = GradBucket(w.shape, bias.numel(), dtype=torch.float64)
        bucket.weight_view.copy_(res[2])
        bucket.bias_view.copy_(res[5])
        bucket.all_reduce_async()
        bucket.wait()
        full = cases.run_oracle(case, x, w, off, mask, bias, go)
        b, e = shard_bounds(case.batch, rank, world)
        ok = (cases.nerr(bucket.weight_view, full[2]) < 1e-12 and cases.nerr(bucket.bias_view, full[5]) < 1e-12
              and cases.nerr(res[0], full[0][b:e]) < 1e-12 and cases.nerr(res[1], full[1][b:e]) < 1e-12
              and cases.nerr(res[3], full[3][b:e]) < 1e-12 and cases.nerr(res[4], full[4][b:e]) < 1e-12)
        ret[rank] = bool(ok)
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize('transposed', [False, True])
def test_two_rank_step_matches_single_process(transposed):
    import socket
    with socket.socket() as s:
        s.bind(('127.0.0.1', 0))
        port = s.getsockname()[1]
    ctx = mp.get_context('spawn')
    with ctx.Manager() as mgr:
        ret = mgr.dict()
        procs = [ctx.Process(target=_worker, args=(r, 2, port, transposed, ret)) for r in range(2)]
        for p in procs:
            p.start()
        for p in procs:
            p.join(120)
            assert p.exitcode == 0
        assert ret.get(0) is True and ret.get(1) is True
