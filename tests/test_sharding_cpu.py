"""The multi-rank path on CPU: two gloo ranks shard a batch, each computes its
block (with the CPU oracle standing in for the GPU kernels) and the gathered
result must equal the unsharded scan."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from neuronspark_b200.sharding import batch_shard


def test_batch_shard_covers_everything_once():
    for total in (0, 1, 7, 32, 256, 1023):
        for world in (1, 2, 3, 8):
            seen = []
            for r in range(world):
                s, n = batch_shard(total, world, r)
                seen += list(range(s, s + n))
            assert seen == list(range(total))
            counts = [batch_shard(total, world, r)[1] for r in range(world)]
            assert max(counts) - min(counts) <= 1
    with pytest.raises(ValueError):
        batch_shard(4, 2, 2)


def _pack(spike):  # [T, cols] {0,1} -> int32 [T, ceil(cols/32)], bit i of word w = column 32w+i
    T, cols = spike.shape
    pad = (-cols) % 32
    s = np.pad(spike.astype(np.uint32), ((0, 0), (0, pad))).reshape(T, -1, 32)
    return (s << np.arange(32, dtype=np.uint32)).sum(-1).astype(np.uint32).view(np.int32)


def _worker(rank, world, port, total_b, out):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from neuronspark_b200 import sharding
        from oracle import oracle as orc
        T, D = 40, 24
        g = torch.Generator().manual_seed(7)
        beta = torch.sigmoid(2 + 0.5 * torch.randn(T, total_b, D, generator=g))
        u = torch.randn(T, total_b, D, generator=g)
        vth = 0.1 + torch.nn.functional.softplus(torch.randn(T, total_b, D, generator=g))
        v0 = torch.zeros(total_b, D)
        mine = [sharding.shard_time_major(t, world, rank) for t in (beta, u, vth)]
        s0, n0 = sharding.batch_shard(total_b, world, rank)
        spike, _, vlast = orc.plif_selective_fwd(*(m.numpy() for m in mine), v0[s0:s0 + n0].numpy())
        packed = torch.from_numpy(_pack(spike.reshape(T, -1)))
        dense = sharding.gather_packed_spikes(packed, (n0, D), total_b)
        vl = sharding.gather_batch(torch.from_numpy(vlast), total_b, 0)
        ref_s, _, ref_v = orc.plif_selective_fwd(beta.numpy(), u.numpy(), vth.numpy(), v0.numpy())
        ok = bool(np.array_equal(dense.numpy(), ref_s.astype(np.uint8))
                  and np.array_equal(vl.numpy(), ref_v))
        out[rank] = ok
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("total_b", [4, 5])
def test_two_rank_sharded_scan_matches_unsharded(total_b):
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    out = mp.Manager().dict()
    mp.spawn(_worker, args=(2, port, total_b, out), nprocs=2, join=True)
    assert out[0] and out[1]
