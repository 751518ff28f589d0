"""Seeded random sweep over shapes: ragged extents, strides, dilations, groups, offset / mask groups, with and
without offset / mask / bias, conv and transposed, 1d-3d.  Half of the draws have 64-channel multiples per group
(tensor-core kernels, f32 split and bf16), the other half arbitrary channel counts (SIMT kernels, f32 and f64).

Checker: the restated oracle in f64 on the CPU (itself pinned to the reference).  Tolerances as everywhere:
1e-4 for f32 / f64 data, 2e-2 for bf16 data (normalised max error, f32 offset / mask / bias).
grad_offset is compared away from its discontinuities only: offsets are drawn so that no sampling position
lies within 1e-3 of an integer (where f32 and f64 may floor to different cells).
"""
import math
import random

import pytest
import torch

import cases
from cases import Case, nerr, run_cabi, run_oracle

pytestmark = pytest.mark.gpu


def draw_case(rng: random.Random, idx: int, tensor: bool) -> Case:
    dim = rng.choice([1, 2, 2, 3])
    transposed = rng.random() < 0.35
    groups = rng.choice([1, 1, 2])
    if tensor:
        cin = 64 * groups * rng.choice([1, 2])
        cout = 64 * groups * rng.choice([1, 2])
        sampled = cout if transposed else cin
        og = rng.choice([g for g in (1, 2, 4) if (sampled // g) % 64 == 0 and sampled % g == 0])
        mg = rng.choice([g for g in (1, 2) if (sampled // g) % 64 == 0 and sampled % g == 0])
    else:
        cin = groups * rng.choice([1, 3, 4, 6])
        cout = groups * rng.choice([1, 2, 5])
        sampled = cout if transposed else cin
        og = rng.choice([g for g in (1, 2, 3) if sampled % g == 0])
        mg = rng.choice([g for g in (1, 2, 3) if sampled % g == 0])
    if rng.random() < 0.15:
        og = 0
    if rng.random() < 0.25:
        mg = 0
    lim = {1: 40, 2: 13, 3: 7}[dim]
    kernel = tuple(rng.randint(1, 3) for _ in range(dim))
    dilation = tuple(rng.randint(1, 2) for _ in range(dim))
    stride = tuple(rng.randint(1, 2) for _ in range(dim))
    padding = tuple(rng.randint(0, 2) for _ in range(dim))
    in_size = tuple(rng.randint(max(3, d * (k - 1) + 1), lim) for k, d in zip(kernel, dilation))
    opad = ()
    if transposed:
        padding = tuple(min(p, d * (k - 1)) for p, k, d in zip(padding, kernel, dilation))
        opad = tuple(rng.randint(0, max(s, d) - 1) for s, d in zip(stride, dilation))
    batch = rng.randint(1, 3)
    # (positions per image are left ragged on purpose: the tensor-core weight gradient needs a multiple of 8 and
    # hands the other shapes to the SIMT kernel, so both engines meet inside one backward call)
    return Case(f'rand{idx}', dim, transposed, batch, cin, cout, in_size, kernel, stride, padding, dilation, opad,
                groups, og, mg, rng.random() < 0.7, rng.choice([0.5, 1.5, 3.0]))


def make_inputs_off_integers(case: Case, seed: int):
    """Like cases.make_inputs, with every sampling position kept >= 1e-3 away from an integer."""
    x, w, off, mask, bias, go = cases.make_inputs(case, seed=seed, dtype=torch.float64)
    if off is not None:
        frac = off - torch.floor(off)
        near = (frac < 1e-3) | (frac > 1 - 1e-3)
        off = torch.where(near, torch.floor(off) + 0.37, off)
        off = off.float().double()          # the values the GPU sees
        frac = off - torch.floor(off)
        assert not ((frac < 5e-4) | (frac > 1 - 5e-4)).any()
    return x, w, off, mask, bias, go


def _draws(tensor: bool, n: int):
    rng = random.Random(20240611 + int(tensor))
    out = []
    while len(out) < n:
        c = draw_case(rng, len(out), tensor)
        if min(c.out_size) < 1:
            continue
        out.append(c)
    return out


TENSOR_DRAWS = _draws(True, 24)
SIMT_DRAWS = _draws(False, 24)


def _check(case, dtype, tol, seed):
    x, w, off, mask, bias, go = make_inputs_off_integers(case, seed)
    q = lambda t, d: None if t is None else t.to(d)
    aux = torch.float32 if dtype != torch.float64 else torch.float64
    host = (q(x, dtype), q(w, dtype), q(off, aux), q(mask, aux), q(bias, aux), q(go, dtype))
    ref = run_oracle(case, *(None if t is None else t.double() for t in host))
    got = run_cabi(case, *(None if t is None else t.cuda() for t in host))
    for name, a, r in zip(cases.NAMES, got, ref):
        if r is None:
            assert a is None, f'{case} {name}'
            continue
        assert a is not None, f'{case} {name}'
        if float(r.abs().max()) == 0.0:
            assert float(a.double().abs().max()) <= tol, f'{case} {name}'
            continue
        e = nerr(a, r)
        assert e <= tol, f'{case}\n{name}: normalised max error {e:.3e}'


@pytest.mark.parametrize('case', TENSOR_DRAWS, ids=[c.name for c in TENSOR_DRAWS])
@pytest.mark.parametrize('dtype,tol', [(torch.float32, 1e-4), (torch.bfloat16, 2e-2)], ids=['f32', 'bf16'])
def test_random_tensor_shapes(case, dtype, tol):
    _check(case, dtype, tol, seed=101)


@pytest.mark.parametrize('case', SIMT_DRAWS, ids=[c.name for c in SIMT_DRAWS])
@pytest.mark.parametrize('dtype,tol', [(torch.float32, 1e-4), (torch.float64, 1e-10)], ids=['f32', 'f64'])
def test_random_simt_shapes(case, dtype, tol):
    _check(case, dtype, tol, seed=202)
