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


def assert_routing_ok(summary, max_beyond_fp32_noise=2):
    """The oracle followed the device's decisions (teacher forcing) and classified each one: identical to its own,
    different inside fp32 summation noise, different inside the tie tolerance (the oracle's memory is a
    separately rounded copy of the device's, so near-ties can flip), or wrong.  Nothing may be wrong, and the
    number of flipped near-ties that fp32 noise alone does not explain is bounded by an explicit count."""
    assert summary["merge_illegal"] == 0, summary
    assert summary["append_rows_illegal"] == 0, summary
    assert summary["merge_differ"] - summary["merge_differ_fp32"] <= max_beyond_fp32_noise, summary


def exact_routing_check(spec: ko.KvmSpec, res: ops.PrefillResult, gate: torch.Tensor):
    """Routing exactness on IDENTICAL operands: for every update and kv row the novelty scores and the merge
    logits are recomputed in float64 from the device's own prepared keys and the device's own memory version
    (read from the prefill workspace), and the device's decisions are classified against them.

    With identical operands the only legitimate difference is the summation order of the fp32 accumulation
    (bf16 x bf16 products are exact), so: a merge target may differ from the float64 first-argmax only if its
    float64 logit is within fp32 noise of the maximum, and an append set must lie between the tokens strictly
    below and at most one bf16 rounding step above the cut.  Returns counters."""
    runner, plan, route = res.runner, res.plan, res.route
    views = {k: v.cpu() for k, v in runner.workspace_views().items()}
    C, sink = spec.chunk_len, spec.sink_len
    rows = route.size(0)
    Hkv = spec.num_key_value_heads
    route = route.cpu().long()
    pk_all = views["prepared_keys"]
    g_all = gate.cpu().reshape(rows, -1).float()           # [B*Hkv, T]
    out = dict(updates=0, merge_tokens=0, merge_differ=0, merge_beyond_fp32_noise=0, append_rows=0,
               append_rows_differ=0, append_rows_illegal=0, appended_rows_recomputed=0, max_gap=0.0)
    ln_w = (spec.ln_weight if spec.ln_weight is not None else torch.ones(spec.d_qk_head)).float()
    ln_b = (spec.ln_bias if spec.ln_bias is not None else torch.zeros(spec.d_qk_head)).float()
    for u in range(1, plan.n_updates + 1):
        S0, n_app = plan.state_before[u], plan.n_append[u]
        S1 = S0 + n_app
        r = route[:, u]                                                        # [rows, C]
        pk = pk_all[:, u * C:(u + 1) * C]                                       # [rows, C, D] bf16
        g = g_all[:, u * C:(u + 1) * C]
        gk = (pk.float() * g.unsqueeze(-1)).bfloat16() if spec.kvm_use_merge_gate_keys else pk
        idx_old = views["versions"][:, plan.version_row[u - 1]:plan.version_row[u - 1] + S0].long()
        mem_old = torch.gather(views["pool_k"], 1, idx_old.unsqueeze(-1).expand(-1, -1, pk.size(-1)))   # [rows, S0, D]
        appended = r < 0
        out["updates"] += 1
        if 0 < n_app < C:
            nov = torch.bmm(pk.double(), mem_old.double().transpose(1, 2)).float().bfloat16().float().amax(-1)   # [rows, C]
            own = torch.argsort(nov, dim=-1, stable=True)[:, :n_app].sort(-1).values
            got = torch.arange(C).expand(rows, C)[appended].view(rows, n_app)
            d, bad = ko._check_forced_append(nov.view(1, rows, C), n_app, own.view(1, rows, n_app), got.view(1, rows, n_app))
            out["append_rows"] += rows
            out["append_rows_differ"] += d
            out["append_rows_illegal"] += bad
        if n_app == C:
            continue
        mem = mem_old
        if n_app:
            idx_new = views["versions"][:, plan.version_row[u] + S0:plan.version_row[u] + S1].long()
            new_rows = torch.gather(views["pool_k"], 1, idx_new.unsqueeze(-1).expand(-1, -1, pk.size(-1))).clone()
            for row in range(rows):
                tok = torch.nonzero(appended[row]).flatten()
                touched = set(r[row][~appended[row]].tolist())
                for j in range(n_app):
                    if S0 + j in touched:   # the version holds the row after this update's merges: rebuild its pre-merge view
                        src = (gk if spec.kvm_apply_merge_gate_to_appends else pk)[row, tok[j]].float()
                        new_rows[row, j] = torch.nn.functional.layer_norm(src, (src.numel(),), ln_w, ln_b, spec.ln_eps).bfloat16()
                        out["appended_rows_recomputed"] += 1
            mem = torch.cat([mem_old, new_rows], 1)
        logits = torch.bmm(gk.double(), mem.double().transpose(1, 2))           # [rows, C, S1]
        logits[:, :, :min(sink, S1)] = float("-inf")
        top, arg = logits.max(-1)
        merged = ~appended
        choice = r.clamp_min(0)
        gap = top - logits.gather(-1, choice.unsqueeze(-1)).squeeze(-1)
        differ = merged & (choice != arg)
        noise = 1e-5 * top.abs().clamp_min(1.0)
        out["merge_tokens"] += int(merged.sum())
        out["merge_differ"] += int(differ.sum())
        out["merge_beyond_fp32_noise"] += int((merged & (gap > noise)).sum())
        if bool(merged.any()):
            out["max_gap"] = max(out["max_gap"], float(gap[merged].max()))
    return out


def record_counts(name: str, counts: dict):
    """Print the decision counts of a parity test (and append them to the file named by KVM_PARITY_LOG)."""
    import json
    import os
    line = json.dumps({"test": name, **counts})
    print(line)
    path = os.environ.get("KVM_PARITY_LOG")
    if path:
        with open(path, "a") as f:
            f.write(line + "\n")


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
