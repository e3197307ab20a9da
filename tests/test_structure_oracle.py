"""CPU checks that anchor the structure-module oracle (the reference ships no vectors for it): invariance of the
invariant point attention under a global rigid motion, a finite-difference gradient check, fp32 vs fp64 agreement."""
import math

import torch

import structure_oracle as SO
from bindcraft2_b200 import synthetic


def _rand_rot(g):
    q = torch.randn(4, generator=g, dtype=torch.float64)
    q = q / q.norm()
    w, x, y, z = q
    return torch.tensor([[1 - 2 * (y * y + z * z), 2 * (x * y - w * z), 2 * (x * z + w * y)],
                         [2 * (x * y + w * z), 1 - 2 * (x * x + z * z), 2 * (y * z - w * x)],
                         [2 * (x * z - w * y), 2 * (y * z + w * x), 1 - 2 * (x * x + y * y)]], dtype=torch.float64)


def test_ipa_is_invariant_under_global_rigid_motion():
    g = torch.Generator().manual_seed(3)
    p = {k: v.double() for k, v in synthetic.make_structure_params(1).items()}
    n = 12
    act = torch.randn(n, 384, generator=g, dtype=torch.float64)
    pair = torch.randn(n, n, 128, generator=g, dtype=torch.float64)
    mask = torch.ones(n, dtype=torch.float64)
    rot = torch.stack([_rand_rot(g) for _ in range(n)])
    trans = torch.randn(n, 3, generator=g, dtype=torch.float64)
    base = SO.invariant_point_attention(p, act, pair, mask, rot, trans)
    G, t = _rand_rot(g), torch.randn(3, generator=g, dtype=torch.float64)
    moved = SO.invariant_point_attention(p, act, pair, mask, G @ rot, trans @ G.T + t)
    assert SO.rel_l2(moved, base) < 1e-10


def test_quaternion_rotation_is_orthonormal():
    g = torch.Generator().manual_seed(4)
    x, y, z = torch.randn(3, 7, generator=g, dtype=torch.float64)
    r = SO.quat_to_rot(x, y, z)
    eye = torch.eye(3, dtype=torch.float64).expand(7, 3, 3)
    assert torch.allclose(r @ r.transpose(-1, -2), eye, atol=1e-12)
    assert torch.allclose(torch.linalg.det(r), torch.ones(7, dtype=torch.float64), atol=1e-12)


def test_gradient_matches_finite_differences_fp64():
    p = synthetic.make_structure_params(5)
    inp = synthetic.make_structure_inputs(6, 10, masked=2)
    out = SO.structure_core_fwd_bwd(p, inp, depth=3, dtype=torch.float64)
    pp = {k: v.double() for k, v in p.items()}

    def loss(single, pair):
        a, r, t = SO.structure_core(pp, single, pair, inp['seq_mask'].double(), 3)
        return float((a * inp['ct_act'].double()).sum() + (r * inp['ct_rot'].double()).sum() + (t * inp['ct_trans'].double()).sum())

    g = torch.Generator().manual_seed(7)
    s0, p0 = inp['single'].double(), inp['pair'].double()
    for _ in range(3):
        ds = torch.randn(s0.shape, generator=g, dtype=torch.float64)
        dp = torch.randn(p0.shape, generator=g, dtype=torch.float64)
        eps = 1e-6
        fd = (loss(s0 + eps * ds, p0 + eps * dp) - loss(s0 - eps * ds, p0 - eps * dp)) / (2 * eps)
        an = float((out['d_single'] * ds).sum() + (out['d_pair'] * dp).sum())
        assert abs(fd - an) <= 1e-5 * max(1.0, abs(an)), (fd, an)


def test_fp32_agrees_with_fp64():
    p = synthetic.make_structure_params(8)
    inp = synthetic.make_structure_inputs(9, 16)
    a = SO.structure_core_fwd_bwd(p, inp, depth=8, dtype=torch.float32)
    b = SO.structure_core_fwd_bwd(p, inp, depth=8, dtype=torch.float64)
    for k in a:
        assert SO.rel_l2(a[k], b[k]) < 2e-4, (k, SO.rel_l2(a[k], b[k]))
    # eight iterations with these weights move the frames, so the rigid path is exercised
    assert float(b['trans'].abs().max()) > 1.0
    assert float((b['rot'] - torch.eye(3, dtype=torch.float64)).abs().max()) > 0.1


def test_heads_and_sidechains_gradient_fp64():
    p = synthetic.add_structure_head_params(synthetic.make_structure_params(11), 12)
    tables = synthetic.make_structure_tables(13)
    inp = synthetic.add_structure_head_inputs(synthetic.make_structure_inputs(14, 9, masked=1), 15)
    out = SO.structure_heads_fwd_bwd(p, tables, inp, depth=2, dtype=torch.float64)
    assert out['atom14'].shape == (9, 14, 3) and out['dgram'].shape == (9, 9, 64)
    assert torch.allclose(out['dgram'], out['dgram'].transpose(0, 1))  # the distogram is symmetrised
    pp = {k: v.double() for k, v in p.items()}

    def loss(single, pair):
        outs = SO.structure_heads(pp, tables, single, pair, inp['seq_mask'].double(), inp['aatype'], 2)
        return float(sum((o * inp['ct_' + k].double()).sum() for k, o in zip(SO.HEAD_OUTS, outs)))

    g = torch.Generator().manual_seed(16)
    s0, p0 = inp['single'].double(), inp['pair'].double()
    ds = torch.randn(s0.shape, generator=g, dtype=torch.float64)
    dp = torch.randn(p0.shape, generator=g, dtype=torch.float64)
    eps = 1e-6
    fd = (loss(s0 + eps * ds, p0 + eps * dp) - loss(s0 - eps * ds, p0 - eps * dp)) / (2 * eps)
    an = float((out['d_single'] * ds).sum() + (out['d_pair'] * dp).sum())
    assert abs(fd - an) <= 1e-5 * max(1.0, abs(an)), (fd, an)


def test_sidechain_atoms_follow_the_backbone_frame():
    """Moving the backbone frame by a rigid motion moves every present atom by the same motion."""
    p = {k: v.double() for k, v in synthetic.add_structure_head_params(synthetic.make_structure_params(21), 22).items()}
    tables = synthetic.make_structure_tables(23)
    g = torch.Generator().manual_seed(24)
    n = 6
    act = torch.randn(n, 384, generator=g, dtype=torch.float64)
    ini = torch.randn(n, 384, generator=g, dtype=torch.float64)
    aatype = torch.randint(0, 21, (n,), generator=g)
    rot = torch.stack([_rand_rot(g) for _ in range(n)])
    trans = torch.randn(n, 3, generator=g, dtype=torch.float64)
    base = SO.sidechain_atoms(p, tables, act, ini, rot, trans, aatype)
    G, t = _rand_rot(g), torch.randn(3, generator=g, dtype=torch.float64)
    moved = SO.sidechain_atoms(p, tables, act, ini, G @ rot, trans @ G.T + t, aatype)
    mask = tables['atom14_mask'].double()[aatype][..., None]
    assert torch.allclose(moved, (base @ G.T + t) * mask, atol=1e-9)
