"""World-size-2 CPU (gloo) test of the exchange layouts of the sharded Evoformer stack.

The library's exchange steps are pack -> equal-chunk exchange -> strided unpack.  Here two gloo ranks hold bands of small
tensors and perform the same three layout changes with the same chunk orders and strides the C++ uses
(``ShardedEvoStack::transpose_bands``, ``TriMul::planes_to_channels`` / ``channels_to_planes``, ``gather_bias`` in
bindcraft2_b200/csrc), and the results are compared with the whole-tensor answer.  Also checks ``native.band_of``."""
import os
import sys

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _all_to_all(chunks):
    """Equal-chunk all-to-all on a backend without one: rank r receives chunk r of every rank, in rank order."""
    world = dist.get_world_size()
    mine = torch.stack(chunks)
    everyone = [torch.empty_like(mine) for _ in range(world)]
    dist.all_gather(everyone, mine)
    return [everyone[src][dist.get_rank()] for src in range(world)]


def _transpose_bands(band, n, world):
    """band [R][n][C] of x  ->  band [R][n][C] of x^T (rows of x^T = columns of x)."""
    R, C = band.shape[0], band.shape[2]
    # stage[q][jj][ii][:] = x[ii][q*R + jj][:]
    stage = [band[:, q * R:(q + 1) * R].permute(1, 0, 2).contiguous() for q in range(world)]
    recv = _all_to_all(stage)
    out = torch.empty(R, n, C)
    for r in range(world):  # 2-D copy: R rows of R*C values into columns [r*R, (r+1)*R)
        out[:, r * R:(r + 1) * R] = recv[r]
    return out


def _planes_to_channels(planes, n, world):
    """band planes [npl][R*n]  ->  whole planes [npl/world][n*n] of this rank's channel group."""
    npl, M = planes.shape
    per = npl // world
    recv = _all_to_all([planes[q * per:(q + 1) * per].contiguous() for q in range(world)])
    out = torch.empty(per, n * n)
    for r in range(world):
        out[:, r * M:(r + 1) * M] = recv[r]
    return out


def _channels_to_planes(whole, n, world):
    per, M = whole.shape[0], whole.shape[1] // world
    recv = _all_to_all([whole[:, q * M:(q + 1) * M].contiguous() for q in range(world)])
    return torch.cat(recv)  # planes of rank 0's channels, then rank 1's, ...


def _gather_bias(compact, n, world):
    """compact [H][n keys][R local queries]  ->  whole [H][n keys][n queries]."""
    H, _, R = compact.shape
    everyone = [torch.empty_like(compact) for _ in range(world)]
    dist.all_gather(everyone, compact)
    out = torch.empty(H, n, n)
    for r in range(world):
        out[:, :, r * R:(r + 1) * R] = everyone[r]
    return out


def _worker(rank, world, port, out):
    sys.path.insert(0, ROOT)
    from bindcraft2_b200 import native
    os.environ.update(MASTER_ADDR='127.0.0.1', MASTER_PORT=str(port))
    dist.init_process_group('gloo', rank=rank, world_size=world)
    n, C, Hc, H = 16, 4, 8, 2
    g = torch.Generator().manual_seed(7)
    x = torch.randn(n, n, C, generator=g)          # pair stream
    planes = torch.randn(Hc, n, n, generator=g)     # tri-mul operand, channel-major whole planes
    bias = torch.randn(H, n, n, generator=g)        # [head][key][query]
    lo, hi = native.band_of(n * 8, world, rank)     # the library's rule (multiples of 32 and of 8*world)
    assert (lo, hi) == (rank * n * 8 // world, (rank + 1) * n * 8 // world)
    R = n // world
    lo, hi = rank * R, (rank + 1) * R
    ok = {}
    xt = _transpose_bands(x[lo:hi].contiguous(), n, world)
    ok['transpose'] = torch.equal(xt, x.transpose(0, 1)[lo:hi])
    ok['transpose_back'] = torch.equal(_transpose_bands(xt, n, world), x[lo:hi])
    band_planes = planes[:, lo:hi].reshape(Hc, R * n).contiguous()
    per = Hc // world
    whole = _planes_to_channels(band_planes, n, world)
    ok['planes_to_channels'] = torch.equal(whole, planes[rank * per:(rank + 1) * per].reshape(per, n * n))
    ok['channels_to_planes'] = torch.equal(_channels_to_planes(whole, n, world), band_planes)
    ok['bias'] = torch.equal(_gather_bias(bias[:, :, lo:hi].contiguous(), n, world), bias)
    out[rank] = ok
    dist.destroy_process_group()


def test_exchange_layouts_two_ranks():
    world = 2
    with mp.Manager() as m:
        out = m.dict()
        mp.spawn(_worker, args=(world, 29737, out), nprocs=world, join=True)
        res = dict(out)
    for rank in range(world):
        assert all(res[rank].values()), res


def test_band_of_rejects_uneven_splits():
    sys.path.insert(0, ROOT)
    from bindcraft2_b200 import native
    assert native.band_of(768, 8, 3) == (288, 384)
    with pytest.raises(ValueError):
        native.band_of(224, 8, 0)   # 28 rows per band: not a multiple of 8
    with pytest.raises(ValueError):
        native.band_of(100, 2, 0)   # not a multiple of 32


def test_unique_id_and_uninitialised_call(lib):
    """Host-side paths that need no GPU: rank 0 can create the exchange-group id (NCCL is bound at run time), and a
    sharded call before bc2_shard_init comes back as a status code with a message, not a crash."""
    import ctypes
    buf = (ctypes.c_uint8 * 128)()
    assert lib.bc2_shard_unique_id(ctypes.addressof(buf)) == 0
    assert any(buf)
    rc = lib.bc2_evoformer_sharded_fwd(None, 1, 1, 1, 1, None, 64, 1, 1, 0, 0, b'/nonexistent', 1, 1, None, None)
    assert rc != 0
    assert lib.bc2_last_error()
