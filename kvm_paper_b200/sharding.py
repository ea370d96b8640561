"""Sharding of the KVM mixer over the GPUs of one node: heads for prefill, sequences for decode.

Every (batch, kv-head) pair owns an independent memory and window, so no term of the mixer crosses heads
or sequences: each rank runs the kernels on its slice and the only collective is one all-gather of the
mixer outputs (NCCL over NVLink on GPUs, gloo on CPU ranks in the tests), or no collective at all where the block
attention kernel stores its tiles into every rank's output itself (``GatheredPrefillOutput``).  The reference has no
counterpart (it is data-parallel only).
"""

from __future__ import annotations

import torch
import torch.distributed as dist


def head_shard(n_q_heads: int, n_kv_heads: int, rank: int, world: int) -> tuple[slice, slice]:
    """Contiguous slice of query heads and of kv heads owned by ``rank`` (GQA groups stay whole)."""
    if n_q_heads % n_kv_heads:
        raise ValueError("n_q_heads must be a multiple of n_kv_heads")
    if n_kv_heads % world:
        raise ValueError(f"{n_kv_heads} kv heads cannot be split over {world} ranks")
    if not 0 <= rank < world:
        raise ValueError(f"rank {rank} outside [0, {world})")
    kv = n_kv_heads // world
    g = n_q_heads // n_kv_heads
    return slice(rank * kv * g, (rank + 1) * kv * g), slice(rank * kv, (rank + 1) * kv)


def shard_heads(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, gate: torch.Tensor, rank: int, world: int):
    """Views of the post-QKV tensors ([B,H,T,D] layout) for this rank's heads."""
    qs, kvs = head_shard(q.size(1), k.size(1), rank, world)
    return q[:, qs], k[:, kvs], v[:, kvs], gate[:, kvs]


def gather_heads(out_local: torch.Tensor, world: int, group=None) -> torch.Tensor:
    """[B,T,h_loc*D] per rank -> [B,T,H*D] on every rank, heads in rank order (the single-rank layout)."""
    if world == 1:
        return out_local
    out_local = out_local.contiguous()
    B, T, hd = out_local.shape
    buf = torch.empty((world * B, T, hd), device=out_local.device, dtype=out_local.dtype)  # rank-major concatenation
    dist.all_gather_into_tensor(buf, out_local, group=group)
    if out_local.is_cuda and (hd * out_local.element_size()) % 16 == 0:
        # the library's copy kernel puts the heads in rank order (a strided tensor copy of this shape runs at a third of
        # its speed)
        from . import _lib
        full = torch.empty((B, T, world * hd), device=out_local.device, dtype=out_local.dtype)
        rc = _lib.load().kvm_interleave_shards(full.data_ptr(), buf.data_ptr(), world, B * T, hd * out_local.element_size(),
                                               torch.cuda.current_stream(out_local.device).cuda_stream)
        _lib.check(rc)
        return full
    return buf.view(world, B, T, hd).permute(1, 2, 0, 3).reshape(B, T, world * hd)


class GatheredPrefillOutput:
    """Output buffers of a head-sharded prefill that every rank's attention kernel writes into directly (peer stores
    over NVLink), so that no collective follows the kernels: each rank holds ``n_buffers`` tensors [B, T, H*D] in
    symmetric memory and knows its peers' addresses of them.  ``run`` enqueues this rank's prefill and returns the
    buffer that holds all heads once every rank has finished, which a small all-reduce behind the kernels establishes
    (stream-ordered on every rank).  The buffers alternate, so that a rank that is already in its next call does not
    write into a buffer a slower rank's consumer is still reading."""

    def __init__(self, batch: int, seq_len: int, n_q_heads_total: int, head_dim: int, device, group=None, n_buffers: int = 2):
        import torch.distributed._symmetric_memory as symm_mem
        self.group = group if group is not None else dist.group.WORLD
        self.rank, self.world = dist.get_rank(self.group), dist.get_world_size(self.group)
        self.buffers, self.ptrs = [], []
        for _ in range(n_buffers):
            t = symm_mem.empty((batch, seq_len, n_q_heads_total * head_dim), dtype=torch.bfloat16, device=device)
            hdl = symm_mem.rendezvous(t, self.group)
            self.buffers.append(t)
            self.ptrs.append([int(p) for p in hdl.buffer_ptrs])
        self._flag = torch.zeros(1, device=device, dtype=torch.int32)
        self._turn = 0

    def run(self, runner, q, k, v, gate, **kwargs) -> torch.Tensor:
        i = self._turn
        self._turn = (i + 1) % len(self.buffers)
        runner.run_gathered(q, k, v, gate, self.rank, self.ptrs[i], **kwargs)
        dist.all_reduce(self._flag, group=self.group)  # behind every rank's kernels: all tiles have been stored everywhere
        return self.buffers[i]


def sequence_shard(n_seq: int, rank: int, world: int) -> slice:
    """Contiguous slice of sequences owned by ``rank`` (decode)."""
    if n_seq % world:
        raise ValueError(f"{n_seq} sequences cannot be split evenly over {world} ranks")
    if not 0 <= rank < world:
        raise ValueError(f"rank {rank} outside [0, {world})")
    per = n_seq // world
    return slice(rank * per, (rank + 1) * per)


def gather_sequences(out_local: torch.Tensor, world: int, seq_dim: int = 0, group=None) -> torch.Tensor:
    """Per-rank decode outputs with the local sequences on ``seq_dim`` -> all sequences in rank order."""
    if world == 1:
        return out_local
    x = out_local.movedim(seq_dim, 0).contiguous()
    full = torch.empty((world * x.size(0),) + tuple(x.shape[1:]), device=x.device, dtype=x.dtype)
    dist.all_gather_into_tensor(full, x, group=group)
    return full.movedim(0, seq_dim)
