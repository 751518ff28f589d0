#!/usr/bin/env python
"""Writes the golden vectors of tests/golden/*.pt from the reference's own CPU implementation.

Run in a container that has the reference checkout:  python oracle/build_ref.py && python tests/golden/make_golden.py
Each file holds the seeded float64 inputs of one case and the six results (output + five gradients) that
``torch.ops.tvdcn_ref.*`` (the reference's CPU kernels, built by oracle/build_ref.py) returned for them.
The cases are the reference's own anisotropic test fixture for every operator and dimension, with the
offset / mask switched on and off and with non-trivial channel groups.
"""
import os
import sys
from dataclasses import asdict

import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, 'tests'))

from oracle import build_ref  # noqa: E402
import cases  # noqa: E402


def golden_cases():
    out = []
    for dim in (1, 2, 3):
        for tr in (False, True):
            b = 1 if dim == 3 else 2  # keeps the committed files small
            out.append(cases.reference_fixture(dim, tr, True, True, batch=b))
            out.append(cases.reference_fixture(dim, tr, True, False, batch=b))
            out.append(cases.reference_fixture(dim, tr, False, True, batch=b))
            out.append(cases.reference_fixture(dim, tr, False, False, batch=b))
            out.append(cases.reference_fixture(dim, tr, True, True, groups=2, offset_groups=4, mask_groups=2,
                                               batch=b))
    return out


def main():
    if not build_ref.load():
        raise SystemExit('oracle/_ref is not built; run python oracle/build_ref.py first')
    for i, c in enumerate(golden_cases()):
        inputs = cases.make_inputs(c, seed=100 + i)
        results = cases.run_reference(c, *inputs)
        torch.save({'case': asdict(c), 'seed': 100 + i, 'inputs': inputs, 'results': results},
                   os.path.join(HERE, c.name + '.pt'))
        print(c.name, [None if r is None else tuple(r.shape) for r in results])


if __name__ == '__main__':
    main()
