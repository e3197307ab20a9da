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


def test_monomer_ipa_layout_conversion_roundtrip():
    """``native.monomer_structure_params_to_multimer`` (reference: bindcraft/af/native.py:365-411): fuse the per-role
    projections of a synthetic multimer-layout parameter set into the monomer checkpoint layout with an independently
    written inverse, convert, and get the originals back."""
    import numpy as np
    from bindcraft2_b200 import native, synthetic
    heads = 12
    src = {'param/' + k: v.numpy() for k, v in synthetic.make_structure_params(77).items()}
    ipa = 'param/fold_iteration/invariant_point_attention/'
    rng = np.random.default_rng(5)
    for role, width in (('q', 16), ('k', 16), ('v', 16)):  # the monomer checkpoint has biases on the scalar projections
        src[f'{ipa}{role}_scalar_projection/bias'] = rng.standard_normal((heads, width)).astype(np.float32)
    fused = {k: v for k, v in src.items() if 'scalar_projection' not in k and 'point_projection' not in k and 'quat_rigid' not in k}
    n_in = src[ipa + 'q_scalar_projection/weights'].shape[0]

    def scal(names):
        w = np.concatenate([src[ipa + n + '/weights'].reshape(n_in, heads, -1) for n in names], -1)
        b = np.concatenate([src[ipa + n + '/bias'].reshape(heads, -1) for n in names], -1)
        return w.reshape(n_in, -1), b.reshape(-1)

    def pts(names):
        ws, bs = [], []
        for n in names:
            w = src[ipa + n + '/point_projection/weights']           # [in, heads, 3*p]: per head x.., y.., z..
            b = src[ipa + n + '/point_projection/bias']
            ws.append(w.reshape(n_in, heads, 3, -1))
            bs.append(b.reshape(heads, 3, -1))
        w = np.concatenate(ws, -1).transpose(0, 2, 1, 3)             # [in, 3, heads, points of all roles]
        b = np.concatenate(bs, -1).transpose(1, 0, 2)
        return w.reshape(n_in, -1), b.reshape(-1)

    fused[ipa + 'q_scalar/weights'], fused[ipa + 'q_scalar/bias'] = scal(['q_scalar_projection'])
    fused[ipa + 'kv_scalar/weights'], fused[ipa + 'kv_scalar/bias'] = scal(['k_scalar_projection', 'v_scalar_projection'])
    fused[ipa + 'q_point_local/weights'], fused[ipa + 'q_point_local/bias'] = pts(['q_point_projection'])
    fused[ipa + 'kv_point_local/weights'], fused[ipa + 'kv_point_local/bias'] = pts(['k_point_projection', 'v_point_projection'])
    for nm in ('weights', 'bias'):
        fused['param/fold_iteration/affine_update/' + nm] = src['param/fold_iteration/quat_rigid/rigid/' + nm]
    back = native.monomer_structure_params_to_multimer(fused, heads)
    assert sorted(back) == sorted(src)
    for k in src:
        np.testing.assert_array_equal(back[k].reshape(src[k].shape), src[k], err_msg=k)
    # a set already in the multimer layout passes through untouched
    same = native.monomer_structure_params_to_multimer(src, heads)
    assert all(same[k] is src[k] for k in src)
