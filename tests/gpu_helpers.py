"""Helpers of the GPU parity tests: run the CUDA path for an oracle spec, turn its routing trace into
the oracle's decision format, and compare the two sides."""

from __future__ import annotations

import torch

from kvm_paper_b200 import ops
from oracle import kvm_oracle as ko
from tests.helpers import assert_close_bf16


def layer_params(spec: ko.KvmSpec, device="cuda") -> ops.LayerParams:
    D = spec.d_qk_head
    cfg = ops.LayerConfig(
        n_q_heads=spec.num_attention_heads, n_kv_heads=spec.num_key_value_heads, head_dim=D,
        chunk_len=spec.chunk_len, n_bswa_chunks=spec.n_bswa_chunks, rope_dim=spec.rope_partial_dim,
        sink_len=spec.sink_len, gate_keys=bool(spec.kvm_use_merge_gate_keys),
        gate_values=bool(spec.kvm_use_merge_gate_values), gate_appends=bool(spec.kvm_apply_merge_gate_to_appends),
        gate_initial=bool(spec.kvm_apply_merge_gate_to_initial_state), ln_eps=spec.ln_eps)
    w = spec.ln_weight if spec.ln_weight is not None else torch.ones(D)
    b = spec.ln_bias if spec.ln_bias is not None else torch.zeros(D)
    ft = spec.front_head_temp if spec.kvm_use_head_temps else None
    st = spec.state_head_temp if spec.kvm_use_head_temps else None
    return ops.LayerParams(cfg, w, b, ft, st, device)


def desired_fn(spec: ko.KvmSpec):
    return lambda ctx, avail, cur: ko.desired_state_len(spec, ctx, avail, cur)


def bf16_spec(spec: ko.KvmSpec) -> ko.KvmSpec:
    """The same spec with its parameter vectors rounded to bf16 (what a bf16 module holds)."""
    import dataclasses
    conv = lambda t: None if t is None else t.detach().cpu().to(torch.bfloat16)  # noqa: E731
    return dataclasses.replace(spec, ln_weight=conv(spec.ln_weight), ln_bias=conv(spec.ln_bias),
                               front_head_temp=conv(spec.front_head_temp), state_head_temp=conv(spec.state_head_temp))


def device_prefill(spec: ko.KvmSpec, q, k, v, gate, want_route=True, memory_capacity=None, phases=3):
    params = layer_params(spec)
    T = q.size(2)
    plan = ops.build_prefill_plan(T, spec.chunk_len, spec.n_bswa_chunks, desired_fn(spec))
    dev = [t.to("cuda", torch.bfloat16) for t in (q, k, v, gate)]
    res = ops.prefill_forward(params, *dev, plan, want_route=want_route, memory_capacity=memory_capacity,
                              phases=phases, check=True)
    torch.cuda.synchronize()
    return params, plan, res


def decisions_from_route(route_u: torch.Tensor, B: int, Hkv: int):
    """route_u [B*Hkv, C] int32 of one update -> {"append_idx": [B,Hkv,n_app] | None, "best_idx": [B,Hkv,n_merge] | None}."""
    r = route_u.cpu().long().view(B, Hkv, -1)
    app_mask = r < 0
    n_app = int(app_mask[0, 0].sum())
    assert bool((app_mask.sum(-1) == n_app).all()), "append count differs between kv rows"
    C = r.size(-1)
    idx = torch.arange(C).view(1, 1, C).expand_as(r)
    append_idx = idx[app_mask].view(B, Hkv, n_app) if n_app else None
    best = r[~app_mask].view(B, Hkv, C - n_app) if n_app < C else None
    if n_app:
        # appended rows must be consecutive in token order
        rows = (-(r[app_mask]) - 1).view(B, Hkv, n_app)
        assert bool((rows[..., 1:] - rows[..., :-1] == 1).all()) if n_app > 1 else True
    return {"append_idx": append_idx, "best_idx": best}


def summarize(trace):
    out = dict(updates=len(trace), merge_tokens=0, merge_differ=0, merge_differ_fp32=0, merge_illegal=0,
               append_rows_differ=0, append_rows_illegal=0)
    for r in trace:
        if r.best_idx is not None:
            out["merge_tokens"] += r.best_idx.numel()
        for key in ("merge_differ", "merge_differ_fp32", "merge_illegal", "append_rows_differ", "append_rows_illegal"):
            out[key] += getattr(r, key)
    return out


def assert_routing_ok(summary, max_ambiguous_frac=5e-3):
    """Bit-exact on every decision outside the stated tie tolerance; ties are counted and bounded."""
    assert summary["merge_illegal"] == 0, summary
    assert summary["append_rows_illegal"] == 0, summary
    if summary["merge_tokens"]:
        assert summary["merge_differ"] <= max(2, max_ambiguous_frac * summary["merge_tokens"]), summary


def compare_memory(mem: ops.MemoryBuffers, state, S: int, what=""):
    B, Hkv, _, D = state["kvm_s_k"].shape
    k_sum = mem.k_sum[:, :S].view(B, Hkv, S, D).cpu()
    v_sum = mem.v_sum[:, :S].view(B, Hkv, S, D).cpu()
    vlen = mem.vlen[:, :S].view(B, Hkv, S, 1).cpu()
    assert state["kvm_s_k"].size(2) == S, (state["kvm_s_k"].shape, S)
    # carried sums grow with the number of merged tokens: tolerance relative to their scale
    scale_k = max(1.0, float(state["kvm_s_k"].float().abs().max()))
    scale_v = max(1.0, float(state["kvm_s_v"].float().abs().max()))
    assert_close_bf16(k_sum, state["kvm_s_k"], what + " kvm_s_k", max_abs_tol=2e-2 * scale_k)
    assert_close_bf16(v_sum, state["kvm_s_v"], what + " kvm_s_v", max_abs_tol=2e-2 * scale_v)
    assert torch.allclose(vlen, state["kvm_s_vlen"].float(), rtol=1e-5, atol=1e-6), what + " kvm_s_vlen"


def fp32_spec(spec: ko.KvmSpec) -> ko.KvmSpec:
    import dataclasses
    conv = lambda t: None if t is None else t.detach().cpu().float()  # noqa: E731
    return dataclasses.replace(spec, ln_weight=conv(spec.ln_weight), ln_bias=conv(spec.ln_bias),
                               front_head_temp=conv(spec.front_head_temp), state_head_temp=conv(spec.state_head_temp))
