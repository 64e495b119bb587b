"""Totals exchanged between GPUs inside the reduction kernels (csrc/peer_exchange.cu).

On one GPU the ranks of a group are walked through one after the other (publish for every
rank, then gather for every rank: no kernel ever waits for a later one); with two or more GPUs
a real two-process run goes through CUDA IPC and the fused publish-and-gather kernel."""
import os
import socket
import sys

import numpy as np
import pytest
import torch

from habitat_b200 import _native, batched, device_table, workloads
from habitat_b200 import distributed as hd

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_one_rank_equals_the_local_sums():
    g = workloads.rng(61)
    planes = g.uniform(0, 1e6, size=(6, 70001)).astype(np.float32)
    planes[:, ::9] = np.nan
    keys = g.integers(0, 8, size=planes.shape[1]).astype(np.uint8)
    d_p, d_k = torch.from_numpy(planes).cuda(), torch.from_numpy(keys).cuda()
    peer = hd.PeerTotals(0, 1)
    for _ in range(3):                                   # both parities of the mailbox
        assert torch.equal(peer.plane_sum(d_p), batched.plane_sum(d_p))
        assert torch.equal(peer.group_sum(d_p[2], d_k, 6), batched.group_sum(d_p[2], d_k, 6))
    devs = [device_table.load_device_file()[n] for n in workloads.BENCH_DEVICES]
    for n_kernels in (40000, 2200000):                   # the longer list takes a cluster of blocks per value
        kb = batched.KernelBatch.from_numpy(workloads.make_kernels(n_kernels, seed=4))
        part = batched.WavePartials(n_kernels, 6)
        for _ in range(2):
            batched.wave_scale(kb, devs[0], devs, partials=part)
            assert torch.equal(peer.partials_sum(part), part.totals())
    v = torch.arange(1, 65, dtype=torch.float64, device="cuda")
    assert torch.equal(peer.allreduce_(v.clone()), v)
    with pytest.raises(_native.HabitatNativeError) as err:
        peer.allreduce_(torch.zeros(65, dtype=torch.float64, device="cuda"))
    assert err.value.status == _native.HB_ERR_TOO_LARGE
    peer.check_status()
    peer.close()


@pytest.mark.parametrize("world", [2, 8])
def test_ranks_walked_through_on_one_gpu(world):
    peers = [hd.PeerTotals(r, world, connect=False) for r in range(world)]
    for p in peers:
        p.connect_local(peers)
    g = workloads.rng(62)
    for call in range(4):                                # slot reuse across calls, both parities
        vals = [torch.from_numpy(g.uniform(-1e9, 1e9, size=30)).cuda() for _ in range(world)]
        want = torch.zeros(30, dtype=torch.float64, device="cuda")
        for v in vals:                                   # the kernel adds in rank order
            want = want + v
        work = [v.clone() for v in vals]
        for r in range(world):
            peers[r].allreduce_(work[r], phase=1)        # publish: stores into every mailbox
        for r in range(world):
            peers[r].allreduce_(work[r], phase=2)        # gather: every flag is already there
        for r in range(world):
            peers[r].check_status()
            assert torch.equal(work[r], want), (call, r)
    for p in peers:
        p.close()


def test_a_peer_that_never_shows_up_times_out():
    """Bounded wait: rank 0 gathers although rank 1 never published; after the limit the kernel
    records whom it waited for, leaves NaN and returns, and the context stays usable."""
    peers = [hd.PeerTotals(r, 2, connect=False) for r in range(2)]
    for p in peers:
        p.connect_local(peers)
    peers[0].set_wait(0.02)
    v = torch.ones(3, dtype=torch.float64, device="cuda")
    peers[0].allreduce_(v, phase=3)                      # publishes, then waits for rank 1 in vain
    with pytest.raises(_native.HabitatNativeError) as err:
        peers[0].check_status()
    assert err.value.status == _native.HB_ERR_DEVICE_TIMEOUT and "rank 1" in str(err.value)
    assert torch.isnan(v).all()
    peers[0].check_status()                              # reported once
    assert float(batched.plane_sum(torch.ones((1, 100), dtype=torch.float32, device="cuda"))[0]) == 100.0
    for p in peers:
        p.close()


def _worker(rank, world, port, out_dir):
    sys.path.insert(0, ROOT)
    os.environ.update(RANK=str(rank), WORLD_SIZE=str(world), MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    import torch.distributed as dist
    torch.cuda.set_device(rank)
    dist.init_process_group("gloo")
    from habitat_b200 import batched as b
    from habitat_b200 import distributed as hdist
    from habitat_b200 import workloads as w
    peer = hdist.PeerTotals()
    g = w.rng(70)
    planes = g.uniform(0, 1e6, size=(6, 50000)).astype(np.float32)
    keys = g.integers(0, 6, size=50000).astype(np.uint8)
    lo, hi = hdist.shard_bounds(50000, rank, world)
    d_p = torch.from_numpy(np.ascontiguousarray(planes[:, lo:hi])).cuda()
    d_k = torch.from_numpy(keys[lo:hi]).cuda()
    hdist.host_barrier()
    outs = []
    for _ in range(5):
        outs.append((peer.plane_sum(d_p).cpu().numpy(), peer.group_sum(d_p[1], d_k, 6).cpu().numpy()))
    peer.check_status()
    local = b.plane_sum(d_p).cpu().numpy()
    np.save(os.path.join(out_dir, "rank%d.npy" % rank), np.concatenate([outs[-1][0], outs[-1][1], local]))
    # totals that the wave-scaling kernel itself starts (this rank's 256-aligned shard of 60,000 kernels)
    from habitat_b200 import device_table as dt
    devs = [dt.load_device_file()[n] for n in w.BENCH_DEVICES]
    kernels = w.make_kernels(60000, seed=12)
    klo, khi = hdist.shard_bounds_aligned(60000, rank, world, 256)
    kb = b.KernelBatch.from_numpy({k: v[klo:khi] for k, v in kernels.items()})
    part = b.WavePartials(khi - klo, 6)
    b.wave_scale(kb, devs[0], devs, partials=part)
    fused = peer.partials_sum(part).cpu().numpy()
    peer.check_status()
    np.save(os.path.join(out_dir, "fused%d.npy" % rank), fused)
    assert all(np.array_equal(o[0], outs[0][0]) and np.array_equal(o[1], outs[0][1]) for o in outs)
    hdist.host_barrier()
    peer.close()
    dist.destroy_process_group()


def test_two_gpus_exchange_through_ipc(tmp_path):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    mp.spawn(_worker, args=(2, port, str(tmp_path)), nprocs=2, join=True)
    a, b = np.load(tmp_path / "rank0.npy"), np.load(tmp_path / "rank1.npy")
    assert np.array_equal(a[:12], b[:12])                         # same bits on both ranks
    assert np.array_equal(a[:6], a[12:] + b[12:])                 # rank-order sum of the local sums
    g = workloads.rng(70)
    planes = g.uniform(0, 1e6, size=(6, 50000)).astype(np.float32)
    keys = g.integers(0, 6, size=50000).astype(np.uint8)
    assert np.allclose(a[:6], planes.astype(np.float64).sum(axis=1), rtol=1e-12)
    assert np.allclose(a[6:12], [planes[1][keys == k].astype(np.float64).sum() for k in range(6)], rtol=1e-12)
    f0, f1 = np.load(tmp_path / "fused0.npy"), np.load(tmp_path / "fused1.npy")
    assert np.array_equal(f0, f1)
    devs = [device_table.load_device_file()[n] for n in workloads.BENCH_DEVICES]
    kb = batched.KernelBatch.from_numpy(workloads.make_kernels(60000, seed=12))
    part = batched.WavePartials(60000, 6)
    batched.wave_scale(kb, devs[0], devs, partials=part)
    np.testing.assert_allclose(f0, part.totals().cpu().numpy(), rtol=1e-14)
