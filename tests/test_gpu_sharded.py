"""GPU tests of the axially sharded Evoformer stack (one complex over P ranks, pair representation split by rows).

The partitioned path is run on ONE GPU with its P ranks as host threads of the library (``bc2_test_sharded_local``: the
exchange steps become device copies behind host barriers; the kernels, plans and index maps are those a multi-process
run over NCCL uses) and compared with the unsharded stack on the same inputs, and with the CPU oracle.  Tolerances: the
path's stated ones (relative L2 <= 2e-2, cosine >= 0.999).  Forward results are expected to agree far more closely,
since every element goes through the same kernels in the same order; gradients differ by the order of the fp32 atomic
sums of the attention bias gradient."""
import pytest
import torch

import evoformer_oracle as O
from bindcraft2_b200 import native, synthetic

pytestmark = pytest.mark.gpu

REL_L2 = 2e-2
COSINE = 0.999


def _both(lib, tmp_path, world, n, s, depth, masked=0, wseed=501, iseed=502):
    params = synthetic.make_evoformer_params(wseed, depth)
    inp = synthetic.make_block_inputs(iseed, n, s, masked=masked)
    wdir = native.weights_from_flat(params, str(tmp_path / 'w'))
    dev = 'cuda:0'
    t = {k: v.to(dev).contiguous() for k, v in inp.items()}
    seed = torch.zeros(2, dtype=torch.int32, device=dev)
    p, m, psave, msave = native.evoformer_fwd(t['pair'], t['msa'], t['pair_mask'], t['msa_mask'], seed, depth=depth, save=1,
                                              weights_dir=wdir, own_save=0)
    dp, dm = native.evoformer_bwd(t['ct_pair'], t['ct_msa'], t['pair_mask'], t['msa_mask'], psave, msave, seed, depth=depth,
                                  weights_dir=wdir, own_save=0)
    torch.cuda.synchronize()
    one = dict(pair=p.cpu(), msa=m.cpu(), d_pair=dp.cpu(), d_msa=dm.cpu())
    sp, sm, sdp, sdm = native.sharded_local_step(world, t['pair'], t['msa'], t['pair_mask'], t['msa_mask'], t['ct_pair'],
                                                 t['ct_msa'], depth=depth, weights_dir=wdir)
    torch.cuda.synchronize()
    assert lib.bc2_device_status() == 0
    many = dict(pair=sp.cpu(), msa=sm.cpu(), d_pair=sdp.cpu(), d_msa=sdm.cpu())
    return one, many, params, inp


def _report(tag, a, b):
    rep = {k: (O.rel_l2(a[k], b[k]), O.cosine(a[k], b[k])) for k in b}
    print(tag, {k: (float('%.3g' % x), round(c, 6)) for k, (x, c) in rep.items()})
    return rep


@pytest.mark.parametrize('world', [2, 4])
def test_sharded_matches_unsharded_n128(lib, tmp_path, world):
    """Two blocks, N_res = 128, two alignment rows, the last 7 residues masked out: bands of 64 / 32 rows."""
    one, many, _, _ = _both(lib, tmp_path, world, 128, 2, 2, masked=7)
    rep = _report(f'P={world} sharded vs one GPU', many, one)
    for k in ('pair', 'msa'):
        assert rep[k][0] <= 1e-3, rep
    for k in ('d_pair', 'd_msa'):
        assert rep[k][0] <= REL_L2 and rep[k][1] >= COSINE, rep


def test_sharded_one_rank_is_the_unsharded_stack(lib, tmp_path):
    """world = 1: every exchange is a copy onto itself."""
    one, many, _, _ = _both(lib, tmp_path, 1, 64, 1, 1)
    rep = _report('P=1 sharded vs one GPU', many, one)
    for k in ('pair', 'msa'):
        assert rep[k][0] <= 1e-3, rep
    for k in ('d_pair', 'd_msa'):
        assert rep[k][0] <= REL_L2 and rep[k][1] >= COSINE, rep


def test_sharded_matches_oracle_single_block(lib, tmp_path):
    """One block at N_res = 128, S = 1 over two ranks against the CPU oracle, with the bf16-operand floor of the case."""
    one, many, params, inp = _both(lib, tmp_path, 2, 128, 1, 1, wseed=101, iseed=102)
    want = O.stack_fwd_bwd(params, inp, 1)
    with O.bf16_operands():
        floor = O.stack_fwd_bwd(params, inp, 1)
    rep = _report('P=2 sharded vs oracle', many, want)
    flo = _report('bf16 floor vs oracle ', floor, want)
    for k in ('pair', 'msa'):
        assert rep[k][0] <= REL_L2, rep
    for k in ('d_pair', 'd_msa'):
        assert rep[k][0] <= max(REL_L2, 1.3 * flo[k][0]), (rep, flo)
        assert rep[k][1] >= min(COSINE, 1 - 1.7 * (1 - flo[k][1])), (rep, flo)


def test_sharded_general_attention_kernels_n288(lib, tmp_path):
    """N_res = 288 (> 256 keys: streamed K/V forward, keys split over CTAs backward), two ranks with bands of 144 rows
    (not a multiple of the 128-row GEMM tile)."""
    one, many, _, _ = _both(lib, tmp_path, 2, 288, 1, 1)
    rep = _report('P=2 N=288 sharded vs one GPU', many, one)
    for k in ('pair', 'msa'):
        assert rep[k][0] <= 1e-3, rep
    for k in ('d_pair', 'd_msa'):
        assert rep[k][0] <= REL_L2 and rep[k][1] >= COSINE, rep


def test_sharded_dropout_uses_the_same_masks(lib, tmp_path):
    """Dropout on (the native counter-hash masks): the sharded stack over two ranks and the unsharded stack get the same
    {seed, enabled} words and must drop the same elements, including the ending-node mask, which the sharded stack
    applies on the transposed band."""
    n, s, depth = 128, 1, 2
    params = synthetic.make_evoformer_params(611, depth)
    inp = synthetic.make_block_inputs(612, n, s)
    wdir = native.weights_from_flat(params, str(tmp_path / 'w'))
    dev = 'cuda:0'
    t = {k: v.to(dev).contiguous() for k, v in inp.items()}
    seed = torch.tensor([1234, 1], dtype=torch.int32, device=dev)
    kw = dict(depth=depth, weights_dir=wdir, dropout=1)
    p, m, psave, msave = native.evoformer_fwd(t['pair'], t['msa'], t['pair_mask'], t['msa_mask'], seed, save=1, own_save=0, **kw)
    dp, dm = native.evoformer_bwd(t['ct_pair'], t['ct_msa'], t['pair_mask'], t['msa_mask'], psave, msave, seed, own_save=0, **kw)
    p0, _, _, _ = native.evoformer_fwd(t['pair'], t['msa'], t['pair_mask'], t['msa_mask'], seed, save=0, depth=depth,
                                       weights_dir=wdir, dropout=0)
    torch.cuda.synchronize()
    one = dict(pair=p.cpu(), msa=m.cpu(), d_pair=dp.cpu(), d_msa=dm.cpu())
    sp, sm, sdp, sdm = native.sharded_local_step(2, t['pair'], t['msa'], t['pair_mask'], t['msa_mask'], t['ct_pair'],
                                                 t['ct_msa'], seed=seed, **kw)
    torch.cuda.synchronize()
    assert lib.bc2_device_status() == 0
    many = dict(pair=sp.cpu(), msa=sm.cpu(), d_pair=sdp.cpu(), d_msa=sdm.cpu())
    rep = _report('P=2 sharded vs one GPU, dropout on', many, one)
    assert O.rel_l2(p.cpu(), p0.cpu()) > 1e-2  # the masks did something
    for k in ('pair', 'msa'):
        assert rep[k][0] <= 1e-3, rep
    for k in ('d_pair', 'd_msa'):
        assert rep[k][0] <= REL_L2 and rep[k][1] >= COSINE, rep


def test_sharded_eight_ranks_n256(lib, tmp_path):
    """The full box's partition on one GPU: eight ranks, bands of 32 rows, 16 tri-mul channels per rank."""
    one, many, _, _ = _both(lib, tmp_path, 8, 256, 1, 1, wseed=701, iseed=702)
    rep = _report('P=8 N=256 sharded vs one GPU', many, one)
    for k in ('pair', 'msa'):
        assert rep[k][0] <= 1e-3, rep
    for k in ('d_pair', 'd_msa'):
        assert rep[k][0] <= REL_L2 and rep[k][1] >= COSINE, rep
