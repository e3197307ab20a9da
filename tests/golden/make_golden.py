"""Generates tests/golden/*.npz from the CPU oracle (oracle/evoformer_oracle.py) on seeded inputs.

The reference project ships no golden vectors for this path and its JAX implementation cannot be imported where
this runs, so these fixtures pin the ORACLE (against accidental edits), not the reference.  Run from the repo root:
    python tests/golden/make_golden.py
"""
import os
import sys

import numpy as np
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, 'oracle'))

import evoformer_oracle as O  # noqa: E402
from bindcraft2_b200 import synthetic  # noqa: E402

CASES = {
    # name: (weight seed, input seed, N, S, depth, masked residues)
    'evoformer_block_n32_s2': (11, 12, 32, 2, 1, 0),
    'evoformer_block_n32_s1_masked': (13, 14, 32, 1, 1, 5),
    'evoformer_stack2_n32_s1': (15, 16, 32, 1, 2, 0),
}


def run_case(wseed, iseed, n, s, depth, masked):
    torch.set_num_threads(1)  # fixed reduction order
    p = synthetic.make_evoformer_params(wseed, depth)
    inp = synthetic.make_block_inputs(iseed, n, s, masked=masked)
    r = O.stack_fwd_bwd(p, inp, depth, dtype=torch.float64)
    # a strided sample keeps the files small; sums pin everything else
    out = {}
    for k, v in r.items():
        v = v.double()
        out[k + '_sample'] = v.flatten()[::97].numpy().astype(np.float64)
        out[k + '_sum'] = np.array(float(v.sum()))
        out[k + '_abs_sum'] = np.array(float(v.abs().sum()))
    return out


if __name__ == '__main__':
    here = os.path.dirname(os.path.abspath(__file__))
    for name, args in CASES.items():
        np.savez_compressed(os.path.join(here, name + '.npz'), **run_case(*args))
        print('wrote', name)
