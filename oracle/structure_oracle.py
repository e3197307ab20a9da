"""CPU oracle for the structure-module core (TEST INFRASTRUCTURE ONLY, PARITY UNPINNED).

A plain PyTorch restatement of the reference's fold iteration without its side-chain and head branches: single/pair
layer norms, initial projection, eight shared-weight iterations of invariant point attention + transition + backbone
update, as the reference JAX code defines them.  Gradients come from autograd.  Only ``tests/``,
``__graft_entry__.smoke()`` and ``bench.py``'s CPU legs may import this file; the product never does.

Parity is unpinned: the reference holds no golden vectors for this path and JAX is not installable here, so the
restatement is anchored by its own checks (rigid-motion invariance, finite differences, fp32 vs fp64) in
``tests/test_structure_oracle.py``.

Reference (paths inside the reference project):
  bindcraft/af/alphafold/model/folding_multimer.py:65-137   QuatRigid
  bindcraft/af/alphafold/model/folding_multimer.py:140-185  PointProjection
  bindcraft/af/alphafold/model/folding_multimer.py:188-371  InvariantPointAttention
  bindcraft/af/alphafold/model/folding_multimer.py:374-474  FoldIteration (the rotation gradient is NOT stopped, :467)
  bindcraft/af/alphafold/model/folding_multimer.py:477-556  generate_monomer_rigids (identity start, shared weights)
  bindcraft/af/alphafold/model/geometry/rotation_matrix.py:117-140, rigid_matrix_vector.py:37-55, vector.py:87-93
  bindcraft/af/alphafold/model/config.py:574-605            multimer structure-module hyper-parameters
"""
from __future__ import annotations

import math
from typing import Dict

import torch

Params = Dict[str, torch.Tensor]

C_S, C_Z, HEADS, SCALAR_QK, SCALAR_V, POINT_QK, POINT_V = 384, 128, 12, 16, 16, 4, 8
NUM_LAYER, POSITION_SCALE, DIST_EPS = 8, 20.0, 1e-8
IPA = 'fold_iteration/invariant_point_attention'


def layer_norm(x, scale, offset, eps=1e-5):
    """common_modules.py:127-184."""
    mu = x.mean(-1, keepdim=True)
    var = ((x - mu) ** 2).mean(-1, keepdim=True)
    return (x - mu) * torch.rsqrt(var + eps) * scale + offset


def quat_to_rot(x, y, z):
    """Rot3Array.from_quaternion with w = 1 and normalisation (rotation_matrix.py:117-140). Returns [..., 3, 3]."""
    w = torch.ones_like(x)
    inv = torch.rsqrt(torch.clamp(w * w + x * x + y * y + z * z, min=1e-6))
    w, x, y, z = w * inv, x * inv, y * inv, z * inv
    rows = [1 - 2 * (y * y + z * z), 2 * (x * y - w * z), 2 * (x * z + w * y),
            2 * (x * y + w * z), 1 - 2 * (x * x + z * z), 2 * (y * z - w * x),
            2 * (x * z - w * y), 2 * (y * z + w * x), 1 - 2 * (x * x + y * y)]
    return torch.stack(rows, -1).reshape(*x.shape, 3, 3)


def point_projection(p: Params, name, act, rot, trans, npts):
    """PointProjection (folding_multimer.py:140-185): Linear -> split x|y|z on the last axis -> global frame.
    Returns global and local points, each [N, H, P, 3]."""
    w = p[f'{IPA}/{name}/point_projection/weights'].reshape(C_S, HEADS * 3 * npts)
    b = p[f'{IPA}/{name}/point_projection/bias'].reshape(HEADS * 3 * npts)
    loc = (act @ w + b).reshape(-1, HEADS, 3, npts).permute(0, 1, 3, 2)  # [N, H, P, xyz]
    glob = torch.einsum('nab,nhpb->nhpa', rot, loc) + trans[:, None, None, :]
    return glob, loc


def invariant_point_attention(p: Params, act, pair_ln, mask, rot, trans):
    """InvariantPointAttention.__call__ (folding_multimer.py:219-371). act [N,384], pair_ln [N,N,128], mask [N]."""
    n = act.shape[0]
    point_w = math.sqrt(1.0 / (max(POINT_QK, 1) * 9.0 / 2)) * torch.nn.functional.softplus(p[f'{IPA}/trainable_point_weights'])
    q_pt, _ = point_projection(p, 'q_point_projection', act, rot, trans, POINT_QK)
    k_pt, _ = point_projection(p, 'k_point_projection', act, rot, trans, POINT_QK)
    d2 = ((q_pt[:, None] - k_pt[None, :]) ** 2).sum(-1)                      # [q, k, H, P]
    logits = -0.5 * (point_w[:, None] * d2).sum(-1)                          # [q, k, H]
    def scalar(name, width):
        # no bias in the multimer model (folding_multimer.py:236-247); the monomer checkpoint carries one (optional entry)
        y = (act @ p[f'{IPA}/{name}/weights'].reshape(C_S, -1)).reshape(n, HEADS, width)
        b = p.get(f'{IPA}/{name}/bias')
        return y if b is None else y + b.reshape(HEADS, width)
    q_s = scalar('q_scalar_projection', SCALAR_QK)
    k_s = scalar('k_scalar_projection', SCALAR_QK)
    q_s = q_s * math.sqrt(1.0 / SCALAR_QK)
    logits = logits + torch.einsum('qhc,khc->qkh', q_s, k_s)
    logits = logits + pair_ln @ p[f'{IPA}/attention_2d/weights'] + p[f'{IPA}/attention_2d/bias']
    m2 = mask[:, None] * mask[None, :]
    logits = logits - 1e5 * (1.0 - m2[..., None])
    logits = logits * math.sqrt(1.0 / 3)
    attn = torch.softmax(logits, dim=1)                                      # over keys
    v_s = scalar('v_scalar_projection', SCALAR_V)
    res_scalar = torch.einsum('qkh,khc->qhc', attn, v_s).reshape(n, -1)
    v_pt, _ = point_projection(p, 'v_point_projection', act, rot, trans, POINT_V)
    res_pt_glob = torch.einsum('qkh,khpa->qhpa', attn, v_pt)                 # [N, H, P, 3]
    res_pt_loc = torch.einsum('nba,nhpb->nhpa', rot, res_pt_glob - trans[:, None, None, :])  # R^T (x - t)
    norms = torch.sqrt(torch.clamp((res_pt_loc ** 2).sum(-1), min=DIST_EPS ** 2)).reshape(n, -1)
    res_2d = torch.einsum('ijh,ijc->ihc', attn, pair_ln).reshape(n, -1)
    flat = res_pt_loc.reshape(n, HEADS * POINT_V, 3)
    final = torch.cat([res_scalar, flat[..., 0], flat[..., 1], flat[..., 2], norms, res_2d], -1)  # [N, 2112]
    return final @ p[f'{IPA}/output_projection/weights'] + p[f'{IPA}/output_projection/bias']


def fold_dropout_masks(seed, iteration, n, channels=384):
    """The two elementwise masks of one fold iteration as the reference's native path draws them (native/foldit.cuh:152-166:
    module ids 21 and 22, rate 0.1, depth index = iteration, mask index = flat [N, C] index)."""
    from evoformer_oracle import dropout_scale_table
    return tuple(dropout_scale_table(seed, iteration, mod, n, channels, 0.1) for mod in (21, 22))


def fold_iteration(p: Params, act, rot, trans, pair_ln, mask, drop=None):
    """FoldIteration.__call__ without the side-chain branch (folding_multimer.py:397-474).  ``drop``: the two dropout
    scale masks [N,384]; the reference drops the WHOLE activation after each residual add (folding_multimer.py:408-412,
    428, 449: safe_dropout with broadcast_dim None), not a module delta as the Evoformer does."""
    f = 'fold_iteration'
    act = act + invariant_point_attention(p, act, pair_ln, mask, rot, trans)
    if drop is not None:
        act = act * drop[0].to(act.dtype)
    act = layer_norm(act, p[f'{f}/attention_layer_norm/scale'], p[f'{f}/attention_layer_norm/offset'])
    x = act
    for i, nm in enumerate(('transition', 'transition_1', 'transition_2')):
        x = x @ p[f'{f}/{nm}/weights'] + p[f'{f}/{nm}/bias']
        if i < 2:
            x = torch.relu(x)
    act = act + x
    if drop is not None:
        act = act * drop[1].to(act.dtype)
    act = layer_norm(act, p[f'{f}/transition_layer_norm/scale'], p[f'{f}/transition_layer_norm/offset'])
    upd = act @ p[f'{f}/quat_rigid/rigid/weights'] + p[f'{f}/quat_rigid/rigid/bias']   # [N, 6]: qx qy qz tx ty tz
    u_rot = quat_to_rot(upd[:, 0], upd[:, 1], upd[:, 2])
    new_trans = torch.einsum('nab,nb->na', rot, upd[:, 3:6]) + trans                   # rigid @ update
    new_rot = rot @ u_rot
    return act, new_rot, new_trans


def structure_core(p: Params, single, pair, seq_mask, depth=NUM_LAYER, dropout_seed=None):
    """generate_monomer_rigids (folding_multimer.py:477-556) with identity initial frames.
    Returns the final activations [N,384], rotations [N,3,3] and translations [N,3] (scaled by position_scale, as the
    reference's 'final_rigids')."""
    n = single.shape[0]
    act = layer_norm(single, p['single_layer_norm/scale'], p['single_layer_norm/offset'])
    act = act @ p['initial_projection/weights'] + p['initial_projection/bias']
    pair_ln = layer_norm(pair, p['pair_layer_norm/scale'], p['pair_layer_norm/offset'])
    rot = torch.eye(3, dtype=single.dtype).expand(n, 3, 3).contiguous()
    trans = torch.zeros(n, 3, dtype=single.dtype)
    for it in range(depth):
        drop = None if dropout_seed is None else fold_dropout_masks(dropout_seed, it, n, act.shape[-1])
        act, rot, trans = fold_iteration(p, act, rot, trans, pair_ln, seq_mask, drop)
    # 20 in the multimer model, 10 in the monomer model (config.py:595 / :357); an optional entry of the parameter dict
    scale = float(p['position_scale']) if 'position_scale' in p else POSITION_SCALE
    return act, rot, trans * scale


def structure_core_fwd_bwd(p: Params, inp, depth=NUM_LAYER, dtype=torch.float32):
    """Forward and gradients wrt single and pair (weights frozen) for cotangents ct_act, ct_rot, ct_trans."""
    pp = {k: v.to(dtype) for k, v in p.items()}
    single = inp['single'].to(dtype).clone().requires_grad_(True)
    pair = inp['pair'].to(dtype).clone().requires_grad_(True)
    act, rot, trans = structure_core(pp, single, pair, inp['seq_mask'].to(dtype), depth)
    loss = (act * inp['ct_act'].to(dtype)).sum() + (rot * inp['ct_rot'].to(dtype)).sum() + (trans * inp['ct_trans'].to(dtype)).sum()
    d_single, d_pair = torch.autograd.grad(loss, [single, pair])
    return dict(act=act.detach(), rot=rot.detach(), trans=trans.detach(), d_single=d_single, d_pair=d_pair)


# ----------------------------------------------------------------------------- side chains and heads
SC = 'fold_iteration/rigid_sidechain'


def _compose(r1, t1, r2, t2):
    """Rigid3Array.__matmul__ (rigid_matrix_vector.py:37-40): (r1,t1) o (r2,t2)."""
    return r1 @ r2, torch.einsum('...ab,...b->...a', r1, t2) + t1


def sidechain_atoms(p: Params, tables, act, initial_act, rot, trans, aatype):
    """MultiRigidSidechain (folding_multimer.py:950-1033) + torsion_angles_to_frames and
    frames_and_literature_positions_to_atom14_pos (all_atom_multimer.py:370-469).
    rot/trans: backbone frames with the translation in Angstrom.  tables: dict with default_frame [21,8,4,4],
    atom14_to_group [21,14] (int), atom14_lit_pos [21,14,3], atom14_mask [21,14].  Returns atom14 positions [N,14,3]."""
    lin = lambda name, x: x @ p[f'{SC}/{name}/weights'] + p[f'{SC}/{name}/bias']
    x = lin('input_projection', torch.relu(act)) + lin('input_projection_1', torch.relu(initial_act))
    for suffix in ('', '_1'):
        old = x
        x = lin('resblock1' + suffix, torch.relu(x))
        x = lin('resblock2' + suffix, torch.relu(x))
        x = x + old
    n = act.shape[0]
    ua = lin('unnormalized_angles', torch.relu(x)).reshape(n, 7, 2)
    ang = ua / torch.sqrt(torch.clamp((ua ** 2).sum(-1, keepdim=True), min=1e-12))
    m = tables['default_frame'].to(act.dtype)[aatype]                      # [N,8,4,4]
    r_d, t_d = m[..., :3, :3], m[..., :3, 3]
    sin = torch.cat([torch.zeros(n, 1, dtype=act.dtype), ang[..., 0]], -1)  # [N,8]
    cos = torch.cat([torch.ones(n, 1, dtype=act.dtype), ang[..., 1]], -1)
    zero, one = torch.zeros_like(sin), torch.ones_like(sin)
    rotx = torch.stack([one, zero, zero, zero, cos, -sin, zero, sin, cos], -1).reshape(n, 8, 3, 3)
    r_a, t_a = r_d @ rotx, t_d                                             # default o rotation about x
    frames_r, frames_t = [r_a[:, k] for k in range(5)], [t_a[:, k] for k in range(5)]
    r, t = r_a[:, 4], t_a[:, 4]
    for k in (5, 6, 7):
        r, t = _compose(r, t, r_a[:, k], t_a[:, k])
        frames_r.append(r)
        frames_t.append(t)
    fr, ft = torch.stack(frames_r, 1), torch.stack(frames_t, 1)            # to backbone, [N,8,...]
    gr, gt = _compose(rot[:, None], trans[:, None], fr, ft)                # to global
    grp = tables['atom14_to_group'][aatype].long()                          # [N,14]
    idx = torch.arange(n)[:, None]
    ar, at = gr[idx, grp], gt[idx, grp]                                     # [N,14,3,3], [N,14,3]
    lit = tables['atom14_lit_pos'].to(act.dtype)[aatype]
    pos = torch.einsum('nkab,nkb->nka', ar, lit) + at
    return pos * tables['atom14_mask'].to(act.dtype)[aatype][..., None]


def heads(p: Params, single, pair, act):
    """Distogram (modules.py:1091-1125), predicted aligned error (:823-861), pLDDT (:777-820) and experimentally
    resolved (:864-906) logits."""
    half = pair @ p['distogram_head/half_logits/weights'] + p['distogram_head/half_logits/bias']
    dgram = half + half.transpose(0, 1)
    pae = pair @ p['predicted_aligned_error_head/logits/weights'] + p['predicted_aligned_error_head/logits/bias']
    h = layer_norm(act, p['predicted_lddt_head/input_layer_norm/scale'], p['predicted_lddt_head/input_layer_norm/offset'])
    h = torch.relu(h @ p['predicted_lddt_head/act_0/weights'] + p['predicted_lddt_head/act_0/bias'])
    h = torch.relu(h @ p['predicted_lddt_head/act_1/weights'] + p['predicted_lddt_head/act_1/bias'])
    plddt = h @ p['predicted_lddt_head/logits/weights'] + p['predicted_lddt_head/logits/bias']
    expres = single @ p['experimentally_resolved_head/logits/weights'] + p['experimentally_resolved_head/logits/bias']
    return dgram, pae, plddt, expres


def structure_heads(p: Params, tables, single, pair, seq_mask, aatype, depth=NUM_LAYER, dropout_seed=None):
    """What the reference's post-trunk call returns (native/ffi.cu:1009-1025): atom14 [N,14,3], distogram logits
    [N,N,64], aligned-error logits [N,N,64], pLDDT logits [N,50], experimentally-resolved logits [N,37]."""
    act, rot, trans = structure_core(p, single, pair, seq_mask, depth, dropout_seed=dropout_seed)
    initial_act = layer_norm(single, p['single_layer_norm/scale'], p['single_layer_norm/offset'])
    atom14 = sidechain_atoms(p, tables, act, initial_act, rot, trans, aatype)
    return (atom14,) + heads(p, single, pair, act)


HEAD_OUTS = ('atom14', 'dgram', 'pae', 'plddt', 'expres')


def structure_heads_fwd_bwd(p: Params, tables, inp, depth=NUM_LAYER, dtype=torch.float32, dropout_seed=None):
    pp = {k: v.to(dtype) for k, v in p.items()}
    single = inp['single'].to(dtype).clone().requires_grad_(True)
    pair = inp['pair'].to(dtype).clone().requires_grad_(True)
    outs = structure_heads(pp, tables, single, pair, inp['seq_mask'].to(dtype), inp['aatype'], depth,
                           dropout_seed=dropout_seed)
    loss = sum((o * inp['ct_' + k].to(dtype)).sum() for k, o in zip(HEAD_OUTS, outs))
    d_single, d_pair = torch.autograd.grad(loss, [single, pair])
    res = {k: o.detach() for k, o in zip(HEAD_OUTS, outs)}
    res.update(d_single=d_single, d_pair=d_pair)
    return res


def rel_l2(a, b):
    return float((a.double() - b.double()).norm() / max(float(b.double().norm()), 1e-30))
