"""Generates tests/golden/*.npz from the CPU oracles (oracle/*.py) on seeded inputs.

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

import embedder_oracle as EO  # noqa: E402
import evoformer_oracle as O  # noqa: E402
import structure_oracle as SO  # noqa: E402
from bindcraft2_b200 import synthetic  # noqa: E402

CASES = {
    # name: (weight seed, input seed, N, S, depth, masked residues)
    'evoformer_block_n32_s2': (11, 12, 32, 2, 1, 0),
    'evoformer_block_n32_s1_masked': (13, 14, 32, 1, 1, 5),
    'evoformer_stack2_n32_s1': (15, 16, 32, 1, 2, 0),
}


# the other oracles: name -> callable returning the dict of outputs
def _extra_msa():
    p = synthetic.make_evoformer_params(21, 1, cm=64, is_extra_msa=True)
    inp = synthetic.make_block_inputs(22, 32, 4, cm=64, masked=3)
    return O.stack_fwd_bwd(p, inp, 1, is_extra_msa=True, dtype=torch.float64)


def _post_trunk():
    p = synthetic.add_structure_head_params(synthetic.make_structure_params(31), 32)
    tables = synthetic.make_structure_tables(33)
    inp = synthetic.add_structure_head_inputs(synthetic.make_structure_inputs(34, 12, masked=2), 35)
    return SO.structure_heads_fwd_bwd(p, tables, inp, depth=3, dtype=torch.float64)


def _embedder():
    return EO.embedder_fwd_bwd(synthetic.make_embedder_params(41), synthetic.make_embedder_inputs(42, 8, 40, s=2),
                               dtype=torch.float64)


OTHER = {'extra_msa_block_n32_s4_masked': _extra_msa, 'post_trunk_n12_depth3': _post_trunk, 'embedder_n48_s2': _embedder}


def _summarise(r):
    out = {}
    for k, v in r.items():
        v = v.double()
        out[k + '_sample'] = v.flatten()[::97].numpy().astype(np.float64)
        out[k + '_sum'] = np.array(float(v.sum()))
        out[k + '_abs_sum'] = np.array(float(v.abs().sum()))
    return out


def run_other(name):
    torch.set_num_threads(1)
    return _summarise(OTHER[name]())


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
    for name in OTHER:
        np.savez_compressed(os.path.join(here, name + '.npz'), **run_other(name))
        print('wrote', name)
