"""Multi-rank host logic on CPU ranks (gloo, world_size 2 and 4): head / sequence partition and the gather
order reproduce the single-rank layout; a rank that fails before the gather surfaces as an error on the
others instead of a hang."""

import datetime
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from kvm_paper_b200 import sharding


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _init(rank, world, port, timeout_s=60):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=timeout_s))


def _fake_mixer_out(q, k):
    """Stand-in for the per-head kernels: depends only on the head's own q/k (as the real mixer does)."""
    B, H, T, D = q.shape
    g = H // k.size(1)
    kk = k.repeat_interleave(g, dim=1)
    return (q * 2 + kk.flip(-1)).transpose(1, 2).reshape(B, T, H * D)


def _worker_heads(rank, world, port, ret):
    _init(rank, world, port)
    torch.manual_seed(0)
    B, H, Hkv, T, D = 2, 8, 4, 5, 4
    q, k = torch.randn(B, H, T, D), torch.randn(B, Hkv, T, D)
    v, gate = torch.randn(B, Hkv, T, D), torch.randn(B, Hkv, T, 1)
    ql, kl, vl, gl = sharding.shard_heads(q, k, v, gate, rank, world)
    assert ql.size(1) == H // world and kl.size(1) == Hkv // world and gl.size(1) == Hkv // world
    full = sharding.gather_heads(_fake_mixer_out(ql, kl), world)
    ok = torch.equal(full, _fake_mixer_out(q, k))
    # decode: sequences
    n_seq = 8
    outs = torch.arange(n_seq * 3, dtype=torch.float32).view(n_seq, 3)
    sl = sharding.sequence_shard(n_seq, rank, world)
    ok = ok and torch.equal(sharding.gather_sequences(outs[sl], world), outs)
    steps = torch.randn(6, n_seq, 3)
    ok = ok and torch.equal(sharding.gather_sequences(steps[:, sl], world, seq_dim=1), steps)
    ret[rank] = bool(ok)
    dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 4])
def test_gather_reproduces_single_rank_layout(world):
    port = _free_port()
    ret = mp.Manager().dict()
    mp.spawn(_worker_heads, args=(world, port, ret), nprocs=world, join=True)
    assert all(ret.get(r) for r in range(world)), dict(ret)


def _worker_failure(rank, world, port, ret):
    _init(rank, world, port, timeout_s=5)
    x = torch.ones(1, 2, 4)
    try:
        if rank == 1:
            raise RuntimeError("rank 1 fails before the gather (injected on the host)")
        sharding.gather_heads(x, world)
        ret[rank] = "no error"
    except RuntimeError as e:
        ret[rank] = "injected" if "injected" in str(e) else "collective error"
    # no destroy: the group is broken on purpose


def test_failed_rank_surfaces_as_error_not_hang():
    port = _free_port()
    ret = mp.Manager().dict()
    mp.spawn(_worker_failure, args=(2, port, ret), nprocs=2, join=True)
    assert ret.get(1) == "injected"
    assert ret.get(0) == "collective error", dict(ret)


def test_partition_arithmetic_and_errors():
    assert sharding.head_shard(16, 16, 3, 8) == (slice(6, 8), slice(6, 8))
    assert sharding.head_shard(32, 8, 1, 4) == (slice(8, 16), slice(2, 4))  # GQA groups stay whole
    covered = []
    for r in range(4):
        qs, _ = sharding.head_shard(32, 8, r, 4)
        covered += list(range(qs.start, qs.stop))
    assert covered == list(range(32))
    with pytest.raises(ValueError):
        sharding.head_shard(16, 6, 0, 4)
    with pytest.raises(ValueError):
        sharding.head_shard(16, 16, 8, 8)
    with pytest.raises(ValueError):
        sharding.sequence_shard(10, 0, 4)
    assert sharding.sequence_shard(64, 7, 8) == slice(56, 64)
