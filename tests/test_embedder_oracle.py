"""CPU checks of the embedder oracle: the relative encoding selects exactly three rows of the position weight, and the
gradient matches finite differences."""
import torch

import embedder_oracle as EO
from bindcraft2_b200 import synthetic


def test_relative_features_are_three_one_hots():
    inp = synthetic.make_embedder_inputs(1, 10, 90)
    rel = EO.relative_features(inp['residue_index'], inp['asym_id'], inp['entity_id'], inp['sym_id'], torch.float64)
    assert rel.shape == (100, 100, 73)
    assert torch.all(rel[..., :66].sum(-1) == 1) and torch.all(rel[..., 67:].sum(-1) == 1)
    assert torch.all(rel[:10, 10:, 65] == 1)       # other chain -> the extra bin
    assert rel[10, 99, 0] == 1 and rel[99, 10, 64] == 1   # offsets beyond +-32 inside one chain are clipped
    assert torch.all(rel[:10, :10, 66] == 1) and torch.all(rel[:10, 10:, 66] == 0)


def test_gradient_matches_finite_differences():
    p = synthetic.make_embedder_params(2)
    inp = synthetic.make_embedder_inputs(3, 6, 14, s=2)
    out = EO.embedder_fwd_bwd(p, inp, dtype=torch.float64)
    pp = {k: v.double() for k, v in p.items()}
    g = torch.Generator().manual_seed(4)
    dt = torch.randn(inp['target_feat'].shape, generator=g, dtype=torch.float64)
    dm = torch.randn(inp['msa_feat'].shape, generator=g, dtype=torch.float64)

    def loss(tf, mf):
        msa, pair = EO.embedder(pp, tf, mf, inp['residue_index'], inp['asym_id'], inp['entity_id'], inp['sym_id'])
        return float((msa * inp['ct_msa'].double()).sum() + (pair * inp['ct_pair'].double()).sum())

    tf0, mf0, eps = inp['target_feat'].double(), inp['msa_feat'].double(), 1e-6
    fd = (loss(tf0 + eps * dt, mf0 + eps * dm) - loss(tf0 - eps * dt, mf0 - eps * dm)) / (2 * eps)
    an = float((out['d_target_feat'] * dt).sum() + (out['d_msa_feat'] * dm).sum())
    assert abs(fd - an) <= 1e-6 * max(1.0, abs(an))


def test_feature_mask_and_monomer_variant():
    """Padding rows (all-zero target features) get preprocess_1d = 0 in the multimer embedder (the reference's native
    embedder, native/embed.cuh:189-197) but not in the monomer one, whose pair term is a single 65-bin one-hot of the
    clipped residue offset."""
    import torch
    from bindcraft2_b200 import synthetic
    p = synthetic.make_embedder_params(31)
    inp = synthetic.make_embedder_inputs(32, 6, 10, 1, n_pad=3)
    msa, pair = EO.embedder(p, inp['target_feat'], inp['msa_feat'], inp['residue_index'], inp['asym_id'], inp['entity_id'],
                            inp['sym_id'])
    only_msa = inp['msa_feat'] @ p['preprocess_msa/weights'] + p['preprocess_msa/bias']
    assert torch.allclose(msa[:, -3:], only_msa[:, -3:])            # padding rows: no preprocess_1d term, not even its bias
    assert not torch.allclose(msa[:, :3], only_msa[:, :3])
    pm = synthetic.make_embedder_params(33, monomer=True)
    im = synthetic.make_embedder_inputs(34, 6, 10, 1, monomer=True, n_pad=3)
    assert im['target_feat'].shape[1] == 22 and float(im['target_feat'][:, 0].abs().sum()) == 0
    msa_m, pair_m = EO.embedder(pm, im['target_feat'], im['msa_feat'], im['residue_index'], im['asym_id'], im['entity_id'],
                                im['sym_id'])
    only = im['msa_feat'] @ pm['preprocess_msa/weights'] + pm['preprocess_msa/bias']
    assert torch.allclose(msa_m[:, -3:] - only[:, -3:], pm['preprocess_1d/bias'].expand(1, 3, -1), atol=1e-6)  # bias kept
    i, j = 2, 5
    off = int(im['residue_index'][i] - im['residue_index'][j])
    want = (im['target_feat'][i] @ pm['left_single/weights'] + pm['left_single/bias'] + im['target_feat'][j] @ pm['right_single/weights']
            + pm['right_single/bias'] + pm['pair_activiations/weights'][min(max(off + 32, 0), 64)] + pm['pair_activiations/bias'])
    assert torch.allclose(pair_m[i, j], want, atol=1e-5)
