"""CPU oracle for the multimer input embedder (TEST INFRASTRUCTURE ONLY, PARITY UNPINNED: the reference holds no
vectors for it and JAX is not installable here; anchored by the checks in tests/test_embedder_oracle.py).

Restates, in plain PyTorch with autograd for the gradients:
  bindcraft/af/alphafold/model/modules_multimer.py:447-510  preprocess_1d / preprocess_msa / left_single / right_single
  bindcraft/af/alphafold/model/modules_multimer.py:358-433  _relative_encoding (use_chain_relative, max_relative_idx 32,
                                                            max_relative_chain 2) followed by position_activations
Only tests/, __graft_entry__.smoke() and bench.py's CPU legs may import this file."""
from __future__ import annotations

import torch

MAX_REL, MAX_CHAIN = 32, 2


def relative_features(residue_index, asym_id, entity_id, sym_id, dtype):
    """The [N,N,73] concatenation of one-hots of _relative_encoding (modules_multimer.py:377-428)."""
    ri, asym, ent, sym = (t.long() for t in (residue_index, asym_id, entity_id, sym_id))
    same_asym = asym[:, None] == asym[None, :]
    clipped = torch.clamp(ri[:, None] - ri[None, :] + MAX_REL, 0, 2 * MAX_REL)
    final = torch.where(same_asym, clipped, torch.full_like(clipped, 2 * MAX_REL + 1))
    rel_pos = torch.nn.functional.one_hot(final, 2 * MAX_REL + 2).to(dtype)
    same_ent = ent[:, None] == ent[None, :]
    rel_chain = torch.clamp(sym[:, None] - sym[None, :] + MAX_CHAIN, 0, 2 * MAX_CHAIN)
    final_chain = torch.where(same_ent, rel_chain, torch.full_like(rel_chain, 2 * MAX_CHAIN + 1))
    chain = torch.nn.functional.one_hot(final_chain, 2 * MAX_CHAIN + 2).to(dtype)
    return torch.cat([rel_pos, same_ent.to(dtype)[..., None], chain], -1)


def embedder(p, target_feat, msa_feat, residue_index, asym_id, entity_id, sym_id):
    """msa [S,N,256], pair [N,N,128].

    Multimer weights (``position_activations``): as modules_multimer.py:447-510 + :358-433, plus the one thing the
    reference's NATIVE embedder adds to that: rows whose target_feat is all zero (padding) get preprocess_1d = 0 after
    the Linear, bias included (native/embed.cuh:189-197,313).
    Monomer weights (``pair_activiations``, the monomer model's own spelling): target_feat is 22 wide, the relative
    encoding is one 65-bin one-hot of the clipped residue offset (modules.py:1471-1485), no chain terms, no feature mask
    (native/embed.cuh:43-62)."""
    lin = lambda name, x: x @ p[f'{name}/weights'] + p[f'{name}/bias']
    monomer = 'pair_activiations/weights' in p
    pre1d = lin('preprocess_1d', target_feat)
    if not monomer:
        pre1d = pre1d * (target_feat.sum(-1, keepdim=True) != 0).to(pre1d.dtype)
    msa = pre1d[None] + lin('preprocess_msa', msa_feat)
    pair = lin('left_single', target_feat)[:, None] + lin('right_single', target_feat)[None]
    if monomer:
        ri = residue_index.long()
        rel = torch.nn.functional.one_hot(torch.clamp(ri[:, None] - ri[None, :] + MAX_REL, 0, 2 * MAX_REL),
                                          2 * MAX_REL + 1).to(target_feat.dtype)
        return msa, pair + lin('pair_activiations', rel)
    rel = relative_features(residue_index, asym_id, entity_id, sym_id, target_feat.dtype)
    return msa, pair + lin('position_activations', rel)


def embedder_fwd_bwd(p, inp, dtype=torch.float32):
    pp = {k: v.to(dtype) for k, v in p.items()}
    tf = inp['target_feat'].to(dtype).clone().requires_grad_(True)
    mf = inp['msa_feat'].to(dtype).clone().requires_grad_(True)
    msa, pair = embedder(pp, tf, mf, inp['residue_index'], inp['asym_id'], inp['entity_id'], inp['sym_id'])
    loss = (msa * inp['ct_msa'].to(dtype)).sum() + (pair * inp['ct_pair'].to(dtype)).sum()
    d_tf, d_mf = torch.autograd.grad(loss, [tf, mf])
    return dict(msa=msa.detach(), pair=pair.detach(), d_target_feat=d_tf, d_msa_feat=d_mf)
