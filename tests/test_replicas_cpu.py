"""World-size-2 test of the benchmark's multi-GPU plumbing on CPU (gloo): replicas get distinct seeded trajectories,
no collective touches the data path, and every reported time is the maximum over ranks."""
import os
import sys

import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _worker(rank, world, port, out):
    sys.path.insert(0, ROOT)
    import bench
    os.environ.update(MASTER_ADDR='127.0.0.1', MASTER_PORT=str(port))
    dist.init_process_group('gloo', rank=rank, world_size=world)
    inp = bench.make_inputs(bench.trajectory_seed(rank), 20, 44, 1)
    ms = bench.max_over_ranks([10.0 + rank, 5.0 - rank], torch.device('cpu'))
    sums = [torch.zeros(1, dtype=torch.float64) for _ in range(world)]
    dist.all_gather(sums, inp['pair'].double().sum().reshape(1))
    out[rank] = (ms, [float(x) for x in sums], tuple(inp['pair'].shape))
    dist.destroy_process_group()


def test_two_replicas_distinct_inputs_and_max_timing():
    world = 2
    with mp.Manager() as m:
        out = m.dict()
        mp.spawn(_worker, args=(world, 29731, out), nprocs=world, join=True)
        res = dict(out)
    for rank in range(world):
        ms, sums, shape = res[rank]
        assert ms == [11.0, 5.0]          # max over ranks of (10, 11) and (5, 4)
        assert shape == (64, 64, 128)
        assert abs(sums[0] - sums[1]) > 1e-3  # the two replicas work on different sequences


def test_reference_arm_runs_on_rank0_only(monkeypatch, capsys):
    sys.path.insert(0, ROOT)
    import bench
    monkeypatch.setenv('RANK', '1')
    args = type('A', (), dict(n_res=32, msa_rows=1, depth=1, steps=1, warmup=0, gpus=2))()
    bench.run_reference(args)
    assert capsys.readouterr().out == ''
