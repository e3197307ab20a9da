"""CPU tests of the oracle: golden fixtures, precision agreement, gradient check, mask inertness."""
import os

import numpy as np
import pytest
import torch

import evoformer_oracle as O
from bindcraft2_b200 import synthetic

GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), 'golden')


def _golden_cases():
    import importlib.util
    spec = importlib.util.spec_from_file_location('make_golden', os.path.join(GOLD, 'make_golden.py'))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


@pytest.mark.parametrize('name', ['evoformer_block_n32_s2', 'evoformer_block_n32_s1_masked', 'evoformer_stack2_n32_s1'])
def test_oracle_matches_golden(name):
    mg = _golden_cases()
    got = mg.run_case(*mg.CASES[name])
    want = np.load(os.path.join(GOLD, name + '.npz'))
    for k in want.files:
        np.testing.assert_allclose(got[k], want[k], rtol=1e-9, atol=1e-9, err_msg=f'{name}:{k}')


@pytest.mark.parametrize('name', ['extra_msa_block_n32_s4_masked', 'post_trunk_n12_depth3', 'embedder_n48_s2'])
def test_other_oracles_match_golden(name):
    """The extra-MSA block (global column attention), the post-trunk call and the embedder against their fixtures."""
    mg = _golden_cases()
    got = mg.run_other(name)
    want = np.load(os.path.join(GOLD, name + '.npz'))
    for k in want.files:
        np.testing.assert_allclose(got[k], want[k], rtol=1e-9, atol=1e-9, err_msg=f'{name}:{k}')


def test_fp32_agrees_with_fp64():
    p = synthetic.make_evoformer_params(1, 1)
    inp = synthetic.make_block_inputs(2, 32, 2)
    a = O.stack_fwd_bwd(p, inp, 1, dtype=torch.float32)
    b = O.stack_fwd_bwd(p, inp, 1, dtype=torch.float64)
    # forward agrees to fp32 rounding; the gradients carry a few ReLU units whose sign differs between the two
    # precisions, each of which moves its rows of the gradient by O(1)
    for k in ('msa', 'pair'):
        assert O.rel_l2(a[k], b[k]) < 1e-5, k
    for k in ('d_msa', 'd_pair'):
        assert O.rel_l2(a[k], b[k]) < 5e-3, k


def test_block_is_not_identity():
    """The reference zero-initialises the last layer of every residual branch, which would make a random-init block
    the identity; the synthetic weights must not."""
    p = synthetic.make_evoformer_params(3, 1)
    inp = synthetic.make_block_inputs(4, 32, 1)
    r = O.stack_fwd_bwd(p, inp, 1)
    assert O.rel_l2(r['pair'], inp['pair']) > 0.3
    assert O.rel_l2(r['msa'], inp['msa']) > 0.3


def test_input_gradient_matches_finite_difference():
    p = {k: v.double() for k, v in synthetic.make_evoformer_params(5, 1).items()}
    inp = synthetic.make_block_inputs(6, 32, 1)
    r = O.stack_fwd_bwd(p, inp, 1, dtype=torch.float64)
    g = torch.Generator().manual_seed(0)
    direction = torch.randn(inp['pair'].shape, generator=g, dtype=torch.float64)

    def loss(pair):
        m, q = O.evoformer_stack(p, inp['msa'].double(), pair, inp['msa_mask'].double(), inp['pair_mask'].double(), 1)
        return float((m * inp['ct_msa'].double()).sum() + (q * inp['ct_pair'].double()).sum())

    eps = 1e-6  # small enough that no ReLU unit changes sign inside the stencil
    fd = (loss(inp['pair'].double() + eps * direction) - loss(inp['pair'].double() - eps * direction)) / (2 * eps)
    an = float((r['d_pair'] * direction).sum())
    assert abs(fd - an) / abs(an) < 1e-5


def test_masked_pad_is_inert():
    """Zero-padding with a masked pad leaves the real corner unchanged (the contract behind the reference's
    pad-to-32 rule, bindcraft/af/native.py:927-972)."""
    p = synthetic.make_evoformer_params(7, 1)
    small = synthetic.make_block_inputs(8, 24, 1)
    n, pad = 24, 8
    big = {
        'msa': torch.nn.functional.pad(small['msa'], (0, 0, 0, pad)),
        'pair': torch.nn.functional.pad(small['pair'], (0, 0, 0, pad, 0, pad)),
        'msa_mask': torch.nn.functional.pad(small['msa_mask'], (0, pad)),
        'pair_mask': torch.nn.functional.pad(small['pair_mask'], (0, pad, 0, pad)),
        'ct_msa': torch.nn.functional.pad(small['ct_msa'], (0, 0, 0, pad)),
        'ct_pair': torch.nn.functional.pad(small['ct_pair'], (0, 0, 0, pad, 0, pad)),
    }
    a = O.stack_fwd_bwd(p, small, 1, dtype=torch.float64)
    b = O.stack_fwd_bwd(p, big, 1, dtype=torch.float64)
    assert O.rel_l2(b['pair'][:n, :n], a['pair']) < 1e-9
    assert O.rel_l2(b['msa'][:, :n], a['msa']) < 1e-9
    assert O.rel_l2(b['d_pair'][:n, :n], a['d_pair']) < 1e-9


def test_opm_matches_reference_einsum_order():
    """The oracle's single einsum equals the reference's two-step form (modules.py:1195-1198)."""
    g = torch.Generator().manual_seed(0)
    left = torch.randn(3, 8, 32, generator=g, dtype=torch.float64)
    right = torch.randn(3, 8, 32, generator=g, dtype=torch.float64)
    w = torch.randn(32, 32, 16, generator=g, dtype=torch.float64)
    lt = left.permute(0, 2, 1)
    act = torch.einsum('acb,ade->dceb', lt, right)
    ref = torch.einsum('dceb,cef->dbf', act, w).permute(1, 0, 2)
    mine = torch.einsum('bdce,cef->bdf', torch.einsum('abc,ade->bdce', left, right), w)
    assert O.rel_l2(mine, ref) < 1e-12


def test_dropout_hash_restatement_is_self_consistent():
    """The numpy statement of the reference's mask hash (native/common.cuh:944-981) against a scalar Python statement
    of the same recurrence, plus the keep rates it has to produce (0.75 for the pair sites, 0.85 for the MSA rows)."""
    import numpy as np

    def scalar(a, b, c, d):
        m = 0xffffffff
        h = (a * 0x9e3779b9) & m
        for v, k in ((b, 0x85ebca6b), (c, 0xc2b2ae35), (d, 0x27d4eb2f)):
            h ^= (v + k + ((h << 6) & m) + (h >> 2)) & m
        h ^= h >> 15
        h = (h * 0x2c1b3c6d) & m
        h ^= h >> 12
        h = (h * 0x297a2d39) & m
        h ^= h >> 15
        return h

    idx = np.arange(0, 5000, 7)
    got = O.dropout_hash(987654321, 47, 5, idx)
    assert got.dtype == np.uint32
    assert (got == np.array([scalar(987654321, 47, 5, int(i)) for i in idx], dtype=np.uint32)).all()
    for mod, rate in ((2, 0.25), (1, 0.15)):
        t = O.dropout_scale_table(11, 3, mod, 224, 128, rate)
        vals = sorted(set(t.flatten().tolist()))
        assert len(vals) == 2 and vals[0] == 0.0 and abs(vals[1] - 1.0 / (1.0 - rate)) < 1e-6
        assert abs(float((t > 0).float().mean()) - (1.0 - rate)) < 0.01
    m = O.block_dropout_masks(5, 0, 32, 128, 256)
    assert m['triangle_attention_ending_node'].shape == (32, 1, 128)
    assert m['triangle_multiplication_outgoing'].shape == (1, 32, 128)
    assert m['msa_row_attention_with_pair_bias'].shape == (1, 32, 256)
