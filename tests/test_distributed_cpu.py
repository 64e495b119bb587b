"""Shard bookkeeping and the totals exchange with two gloo ranks on the CPU."""
import os
import socket
import sys

import numpy as np
import pytest
import torch
import torch.multiprocessing as mp

from habitat_b200 import distributed as hd

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_shard_bounds_cover_everything():
    for n in (0, 1, 5, 64, 1000, 1 << 20, (1 << 20) + 3):
        for world in (1, 2, 3, 4, 8):
            for fn in (hd.shard_bounds, lambda a, b, c: hd.shard_bounds_aligned(a, b, c, 4),
                       lambda a, b, c: hd.shard_bounds_aligned(a, b, c, 256)):   # the benchmark's kernel shards
                edges = [fn(n, r, world) for r in range(world)]
                assert edges[0][0] == 0 and edges[-1][1] == n
                assert all(a[1] == b[0] for a, b in zip(edges, edges[1:]))
                assert all(lo <= hi for lo, hi in edges)
            sizes = [hi - lo for lo, hi in (hd.shard_bounds(n, r, world) for r in range(world))]
            assert max(sizes) - min(sizes) <= 1
            for r in range(world - 1):
                for align in (4, 256):
                    assert hd.shard_bounds_aligned(n, r, world, align)[1] % align == 0 or \
                        hd.shard_bounds_aligned(n, r, world, align)[1] == n


def _worker(rank, world, port, n, out_dir):
    sys.path.insert(0, ROOT)
    os.environ.update(RANK=str(rank), WORLD_SIZE=str(world), MASTER_ADDR="127.0.0.1",
                      MASTER_PORT=str(port))
    from habitat_b200 import device_table, workloads
    from habitat_b200 import distributed as hdist
    from oracle import wave as owave
    hdist.init("gloo")
    devs = device_table.load_device_file()
    specs = [devs[name].spec_tuple() for name in workloads.BENCH_DEVICES]
    kernels = workloads.make_kernels(n, seed=77)

    def totals(lo, hi):
        # the CPU oracle stands in for the device kernels, which need a GPU
        part = {k: v[lo:hi] for k, v in kernels.items()}
        res = owave.wave_scale_batch(specs, 0, list(range(6)), part, want_limits=False)
        return torch.from_numpy(np.nansum(res["scaled_ns"], axis=1))

    total = hdist.sharded_totals(n, totals)
    rows = torch.full((rank + 2, 3), float(rank), dtype=torch.float64)
    gathered = hdist.allgather_rows(rows)
    if rank == 0:
        np.save(os.path.join(out_dir, "total.npy"), total.numpy())
        np.save(os.path.join(out_dir, "gathered.npy"), gathered.numpy())
    torch.distributed.barrier()
    torch.distributed.destroy_process_group()


def test_two_rank_totals_match_one_rank(tmp_path):
    from habitat_b200 import device_table, workloads
    from oracle import wave as owave
    n = 10007
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    mp.spawn(_worker, args=(2, port, n, str(tmp_path)), nprocs=2, join=True)
    devs = device_table.load_device_file()
    specs = [devs[name].spec_tuple() for name in workloads.BENCH_DEVICES]
    ref = owave.wave_scale_batch(specs, 0, list(range(6)), workloads.make_kernels(n, seed=77),
                                 want_limits=False)
    want = np.nansum(ref["scaled_ns"], axis=1)
    got = np.load(tmp_path / "total.npy")
    assert np.allclose(got, want, rtol=1e-12)
    gathered = np.load(tmp_path / "gathered.npy")
    assert gathered.shape == (5, 3) and (gathered[:2] == 0).all() and (gathered[2:] == 1).all()


def _peer_worker(rank, world, port, out_dir):
    sys.path.insert(0, ROOT)
    os.environ.update(RANK=str(rank), WORLD_SIZE=str(world), MASTER_ADDR="127.0.0.1",
                      MASTER_PORT=str(port))
    from habitat_b200 import distributed as hdist
    hdist.init("gloo")
    # no GPU here: creating the mailbox fails on every rank.  Every rank must still walk through
    # the same collectives and come out with the same verdict instead of waiting for the others.
    try:
        hdist.PeerTotals()
        verdict = "created"
    except RuntimeError as exc:
        verdict = "refused: %s" % exc
    hdist.host_barrier()
    with open(os.path.join(out_dir, "peer%d.txt" % rank), "w") as f:
        f.write(verdict)
    torch.distributed.destroy_process_group()


def test_peer_setup_fails_on_every_rank_together(tmp_path):
    if torch.cuda.is_available():
        pytest.skip("exercises the no-GPU failure path")
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    mp.spawn(_peer_worker, args=(2, port, str(tmp_path)), nprocs=2, join=True)
    texts = [open(tmp_path / ("peer%d.txt" % r)).read() for r in range(2)]
    assert all(t.startswith("refused: peer exchange could not be set up on rank(s) [0, 1]") for t in texts), texts
