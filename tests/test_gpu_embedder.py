"""GPU parity of the input embedder (fp32 on both sides: relative L2 <= 1e-5) through the C ABI."""
import pytest
import torch

import embedder_oracle as EO
from bindcraft2_b200 import synthetic

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize('nb,nt,s,monomer,n_pad', [(8, 24, 1, False, 0), (80, 144, 2, False, 0), (20, 44, 1, False, 9),
                                                  (16, 48, 1, True, 0), (40, 88, 2, True, 5)])
def test_embedder_matches_oracle(lib, tmp_path, nb, nt, s, monomer, n_pad):
    """Multimer embedder, the same with trailing padding rows (all-zero target features: the reference's native embedder
    zeroes preprocess_1d there, forward and backward), and the monomer model's embedder (22-wide target features, 65-bin
    ``pair_activiations``, no chain terms, no feature mask), selected by the manifest."""
    from bindcraft2_b200 import native
    p = synthetic.make_embedder_params(501 + nb, monomer=monomer)
    inp = synthetic.make_embedder_inputs(502 + nb, nb, nt, s, monomer=monomer, n_pad=n_pad)
    wdir = native.weights_from_flat(p, str(tmp_path / 'w'))
    t = {k: v.cuda().contiguous() for k, v in inp.items()}
    msa, pair = native.embedder_fwd(t['target_feat'], t['msa_feat'], t['residue_index'], t['asym_id'], t['entity_id'],
                                    t['sym_id'], weights_dir=wdir)
    d_tf, d_mf = native.embedder_bwd(t['ct_msa'], t['ct_pair'], t['target_feat'], weights_dir=wdir)
    torch.cuda.synchronize()
    want = EO.embedder_fwd_bwd(p, inp, dtype=torch.float64)
    got = dict(msa=msa, pair=pair, d_target_feat=d_tf, d_msa_feat=d_mf)
    for k, w in want.items():
        err = float((got[k].cpu().double() - w).norm() / w.norm())
        print(k, f'{err:.2e}')
        assert err <= 1e-5, (k, err)
