"""Run under torchrun on N GPUs: head-sharded prefill and sequence-sharded decode, gathered over NCCL, must
equal the single-GPU result bit for bit (sharding changes no arithmetic); so must the prefill whose attention kernel
gathers by itself (peer stores).  Prints MULTI_GPU_OK on rank 0."""

import os
import sys

import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

from kvm_paper_b200 import ops, sharding  # noqa: E402
from oracle import kvm_oracle as ko  # noqa: E402
from tests import gpu_helpers as gh  # noqa: E402


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(int(os.environ["LOCAL_RANK"]))
    dist.init_process_group("nccl")
    g = torch.Generator().manual_seed(4)
    B, Hq, Hkv, T, D, C = 2, 8, 4, 128 * 5 + 17, 128, 128
    q = torch.nn.functional.layer_norm(torch.randn(B, T, Hq, D, generator=g), (D,)).bfloat16().transpose(1, 2)
    k = torch.nn.functional.layer_norm(torch.randn(B, T, Hkv, D, generator=g), (D,)).bfloat16().transpose(1, 2)
    v = torch.randn(B, T, Hkv, D, generator=g).bfloat16().transpose(1, 2)
    gate = (1 + torch.nn.functional.elu(torch.randn(B, T, Hkv, 1, generator=g))).bfloat16().transpose(1, 2)
    temps = dict(front_head_temp=torch.linspace(0.9, 1.2, Hq), state_head_temp=torch.linspace(1.1, 0.8, Hq))
    full = gh.bf16_spec(ko.KvmSpec(Hq, Hkv, D, D, 64, C, 2, 4, 1, "plus_one", state_min_len=C, **temps))
    qs, kvs = sharding.head_shard(Hq, Hkv, rank, world)
    import dataclasses
    local = dataclasses.replace(full, num_attention_heads=qs.stop - qs.start, num_key_value_heads=kvs.stop - kvs.start,
                                front_head_temp=full.front_head_temp[qs], state_head_temp=full.state_head_temp[qs])
    ql, kl, vl, gl = sharding.shard_heads(q, k, v, gate, rank, world)
    _, _, res = gh.device_prefill(local, ql, kl, vl, gl, want_route=False)
    y = sharding.gather_heads(res.out, world)
    ok = True
    # the same prefill with the attention kernel storing its tiles into every rank's output itself (no collective):
    # every rank's buffer must equal the NCCL-gathered output, on both of the alternating buffers
    gathered = sharding.GatheredPrefillOutput(B, T, Hq, D, torch.device("cuda"))
    dev_in = [t.to("cuda", torch.bfloat16) for t in (ql, kl, vl, gl)]
    for turn in range(3):
        y2 = gathered.run(res.runner, *dev_in)
        torch.cuda.synchronize()
        if not torch.equal(y2, y):
            d = (y2.float() - y.float()).abs()
            print(f"rank {rank}: gathered prefill (call {turn}) differs from the all-gathered one: max abs", float(d.max()), flush=True)
            ok = False
        dist.barrier()  # nobody writes into a buffer that a peer is still comparing
    if rank == 0:
        _, _, ref = gh.device_prefill(full, q, k, v, gate, want_route=False)
        ok = torch.equal(y, ref.out)
        if not ok:
            d = (y.float() - ref.out.float()).abs()
            print("prefill mismatch: max abs", float(d.max()), "first bad index", d.nonzero()[0].tolist(), flush=True)
    # decode: sequences sharded, every rank holds its own cache
    n_seq, n_steps = 4, 20
    spec = gh.bf16_spec(ko.KvmSpec(2, 2, 64, 64, 32, 32, 2, 8, 1, "power_law", state_growth_factor=4.0, state_min_len=32))
    sl = sharding.sequence_shard(n_seq, rank, world)
    Tq = 32 * 3 + 30
    dq = torch.randn(n_seq, 2, Tq + n_steps, 64, generator=g).bfloat16()
    dk = torch.nn.functional.layer_norm(torch.randn(n_seq, 2, Tq + n_steps, 64, generator=g), (64,)).bfloat16()
    dv = torch.randn(n_seq, 2, Tq + n_steps, 64, generator=g).bfloat16()
    dg = (1 + torch.nn.functional.elu(torch.randn(n_seq, 2, Tq + n_steps, 1, generator=g))).bfloat16()

    def decode(seqs):
        p, plan, r = gh.device_prefill(spec, dq[seqs, :, :Tq], dk[seqs, :, :Tq], dv[seqs, :, :Tq], dg[seqs, :, :Tq], want_route=False)
        cache = ops.decode_cache_from_prefill(p, r, dk[seqs, :, :Tq].cuda(), dv[seqs, :, :Tq].cuda(), dg[seqs, :, :Tq].cuda(), gh.desired_fn(spec))
        steps = lambda t: t[seqs, :, Tq:].permute(2, 0, 1, 3).unsqueeze(3).contiguous().cuda()  # noqa: E731
        return cache.run(steps(dq), steps(dk), steps(dv), steps(dg))

    out = sharding.gather_sequences(decode(sl), world, seq_dim=1)
    if rank == 0:
        ref_dec = decode(slice(0, n_seq))
        if not torch.equal(out, ref_dec):
            d = (out.float() - ref_dec.float()).abs()
            print("decode mismatch: max abs", float(d.max()), "first bad index", d.nonzero()[0].tolist(), flush=True)
            ok = False
    flag = torch.tensor([1 if ok else 0], device="cuda")
    dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    if rank == 0:
        print("MULTI_GPU_OK" if int(flag.item()) == 1 else "MULTI_GPU_MISMATCH")
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
