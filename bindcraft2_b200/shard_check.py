"""Checks the multi-process sharded Evoformer stack against the unsharded one on the same seeded inputs.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node P --master-addr 127.0.0.1 --master-port 29541 \
        -m bindcraft2_b200.shard_check --n-res 256 --msa-rows 2 --depth 2

One process per GPU.  Every rank runs its band through ``native.sharded_evoformer_fwd/bwd`` (exchange steps over NCCL
inside the library); rank 0 also runs the whole complex through ``native.evoformer_fwd/bwd`` on its own GPU, gathers the
bands and prints one JSON line with the relative L2 differences.  Exit status 1 if a difference exceeds the path's
tolerance (forward 1e-3, gradients 2e-2 relative L2 / cosine 0.999).
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import tempfile

import torch
import torch.distributed as dist


def _rel(a: torch.Tensor, b: torch.Tensor) -> float:
    return float((a.double() - b.double()).norm() / b.double().norm().clamp_min(1e-30))


def _cos(a: torch.Tensor, b: torch.Tensor) -> float:
    a, b = a.double().flatten(), b.double().flatten()
    return float((a @ b) / (a.norm() * b.norm()).clamp_min(1e-30))


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument('--n-res', type=int, default=256)
    ap.add_argument('--msa-rows', type=int, default=2)
    ap.add_argument('--depth', type=int, default=2)
    ap.add_argument('--masked', type=int, default=5)
    args = ap.parse_args()
    from bindcraft2_b200 import native, synthetic
    world, rank = int(os.environ.get('WORLD_SIZE', '1')), int(os.environ.get('RANK', '0'))
    local = int(os.environ.get('LOCAL_RANK', '0'))
    torch.cuda.set_device(local)
    dev = torch.device('cuda', local)
    saved = os.dup(1)
    os.dup2(2, 1)  # stdout carries the one JSON line only
    try:
        dist.init_process_group('nccl', device_id=dev)
        dist.barrier()
        native.shard_init()
    finally:
        os.dup2(saved, 1)
        os.close(saved)
    n, s, depth = args.n_res, args.msa_rows, args.depth
    wdir = os.path.join(tempfile.gettempdir(), f'bc2_shard_check_d{depth}')
    if rank == 0 and not os.path.exists(os.path.join(wdir, '.complete')):
        native.weights_from_flat(synthetic.make_evoformer_params(901, depth), wdir)
        open(os.path.join(wdir, '.complete'), 'w').write('ok')
    dist.barrier()
    inp = synthetic.make_block_inputs(902, n, s, masked=args.masked)  # identical on every rank (seeded)
    lo, hi = native.band_of(n, world, rank)
    t = {k: (v[lo:hi] if k in ('pair', 'ct_pair') else v).contiguous().to(dev) for k, v in inp.items()}
    kw = dict(depth=depth, weights_dir=wdir)
    p, m, psave, msave = native.sharded_evoformer_fwd(t['pair'], t['msa'], t['pair_mask'], t['msa_mask'], save=1, **kw)
    dp, dm = native.sharded_evoformer_bwd(t['ct_pair'], t['ct_msa'], t['pair_mask'], t['msa_mask'], psave, msave, **kw)
    torch.cuda.synchronize()
    bands_p = [torch.empty_like(p) for _ in range(world)]
    bands_d = [torch.empty_like(dp) for _ in range(world)]
    msas = [torch.empty_like(dm) for _ in range(world)]
    dist.all_gather(bands_p, p)
    dist.all_gather(bands_d, dp)
    dist.all_gather(msas, dm)
    rc = 0
    if rank == 0:
        full = {k: v.to(dev).contiguous() for k, v in inp.items()}
        seed = torch.zeros(2, dtype=torch.int32, device=dev)
        rp, rm, ps, ms = native.evoformer_fwd(full['pair'], full['msa'], full['pair_mask'], full['msa_mask'], seed, save=1,
                                              own_save=0, **kw)
        rdp, rdm = native.evoformer_bwd(full['ct_pair'], full['ct_msa'], full['pair_mask'], full['msa_mask'], ps, ms, seed,
                                        own_save=0, **kw)
        torch.cuda.synchronize()
        sp, sd = torch.cat(bands_p), torch.cat(bands_d)
        out = {'world': world, 'n_res': n, 'msa_rows': s, 'depth': depth,
               'pair_rel_l2': _rel(sp, rp), 'msa_rel_l2': _rel(m, rm),
               'd_pair_rel_l2': _rel(sd, rdp), 'd_pair_cos': _cos(sd, rdp),
               'd_msa_rel_l2': _rel(dm, rdm), 'd_msa_cos': _cos(dm, rdm),
               'd_msa_spread_over_ranks': max(_rel(x, msas[0]) for x in msas)}
        ok = (out['pair_rel_l2'] <= 1e-3 and out['msa_rel_l2'] <= 1e-3 and out['d_pair_rel_l2'] <= 2e-2 and
              out['d_msa_rel_l2'] <= 2e-2 and out['d_pair_cos'] >= 0.999 and out['d_msa_cos'] >= 0.999)
        out['ok'] = bool(ok)
        print(json.dumps(out))
        rc = 0 if ok else 1
    flag = torch.tensor([rc], device=dev)
    dist.broadcast(flag, src=0)
    native.shard_finalize()
    dist.destroy_process_group()
    return int(flag.item())


if __name__ == '__main__':
    sys.exit(main())
