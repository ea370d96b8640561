"""CPU oracle for the Key-Value-Means (KVM) sequence mixer at the post-QKV boundary.

TEST INFRASTRUCTURE ONLY.  This file is the checker that the CUDA path is compared with; it is
never the thing that is shipped or measured as the product.  Only the test-suite, the repository's
smoke check and the benchmark's CPU-baseline / reference arm may import it.

It is a plain-PyTorch restatement of the reference's eager mixer, written as free functions over a
small spec object, using the same tensor operations in the same order as the reference so that on
the CPU it reproduces the reference bit for bit (pinned by the golden fixtures under
``tests/golden`` which were produced by running the reference itself; see ``tests/golden/make_golden.py``).

Reference files followed (paths inside the reference project):
  model/kvm_mixer.py                      eager mixer ("historical golden")
  model/kvm_fp32_routing_reference.py     same, merge-routing logits in fp32 (the routing oracle)
  model/tokenshift.py, model/value_residual_mixin.py, model/rwkv7_backbone.py   the prologue behind the projections

Tensor layouts: q [B,Hq,T,D], k [B,Hkv,T,D], v [B,Hkv,T,Dv], merge_gate [B,Hkv,T,1];
outputs are the pre-``c_proj`` activations [B,T,Hq*Dv].
"""

from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import Any

import torch
import torch.nn.functional as F


@dataclass
class KvmSpec:
    """Every quantity the eager mixer reads from its config and parameters
    (model/kvm_mixer.py:79-118)."""

    num_attention_heads: int
    num_key_value_heads: int
    d_qk_head: int
    d_v_head: int
    rope_partial_dim: int
    chunk_len: int
    n_bswa_chunks: int = 2
    n_max_d_chunks: int = 1
    sink_len: int = 1
    state_budget_mode: str = "fixed"
    state_growth_factor: float = 1.0
    state_growth_exponent: float = 0.5
    state_round_down: int = 1
    state_min_len: int = -1
    state_saturation_n: int | None = None
    kvm_use_merge_gate_keys: int = 1
    kvm_use_merge_gate_values: int = 1
    kvm_apply_merge_gate_to_initial_state: int = 0
    kvm_apply_merge_gate_to_appends: int = 0
    kvm_use_head_temps: int = 1
    kvm_use_vlens: int = 1
    ln_eps: float = 1e-5
    # "plus_one" is not a reference mode: it is the "one new mean per block" schedule of the
    # benchmark configuration, realised in the reference by overriding _desired_state_len.
    ln_weight: torch.Tensor | None = None
    ln_bias: torch.Tensor | None = None
    front_head_temp: torch.Tensor | None = None
    state_head_temp: torch.Tensor | None = None
    # "fp32" follows model/kvm_fp32_routing_reference.py:24-49, "key_dtype" follows
    # model/kvm_mixer.py:321-340.
    routing: str = "fp32"

    @property
    def max_state_len(self) -> int:
        return self.chunk_len * self.n_max_d_chunks

    @property
    def kv_group_size(self) -> int:
        return self.num_attention_heads // self.num_key_value_heads


@dataclass
class UpdateRecord:
    """What one memory update decided; filled when a trace list is passed."""

    ctx_len: int
    available_context: int
    state_before: int
    state_after: int
    n_append: int
    append_idx: torch.Tensor | None  # [B,Hkv,n_append] token indices inside the block
    merge_idx: torch.Tensor | None  # [B,Hkv,n_merge]
    best_idx: torch.Tensor | None  # [B,Hkv,n_merge] slot chosen for each merged token
    margin: torch.Tensor | None  # [B,Hkv,n_merge] fp32 top-1 minus top-2 logit
    append_scores: torch.Tensor | None = None  # [B,Hkv,C] fp32 novelty scores
    # filled when decisions are forced from outside (see ``forced`` below)
    append_rows_differ: int = 0    # kv rows whose forced append set differs from the oracle's own
    append_rows_illegal: int = 0   # ... and is not explained by a tie / one-ulp score difference at the cut
    merge_differ: int = 0          # merged tokens whose forced row differs from the oracle's own argmax
    merge_differ_fp32: int = 0     # ... with an oracle-side logit gap within fp32 summation noise
    merge_illegal: int = 0         # ... with a gap larger than the stated tie tolerance


# ----------------------------------------------------------------------------- small helpers


def _round_down_to_multiple(x: int, multiple: int) -> int:
    # model/kvm_mixer.py:25-28
    x_i = max(int(x), 0)
    multiple_i = max(int(multiple), 1)
    return (x_i // multiple_i) * multiple_i


def lower_right_causal_mask(q_len: int, kv_len: int, device) -> torch.Tensor:
    # model/kvm_mixer.py:16-22
    off = kv_len - q_len
    q_idx = torch.arange(q_len, device=device).unsqueeze(1)
    kv_idx = torch.arange(kv_len, device=device).unsqueeze(0)
    return kv_idx <= (q_idx + off)


def _gather_by_idx(x: torch.Tensor, idx: torch.Tensor) -> torch.Tensor:
    # model/kvm_mixer.py:31-33
    return x.gather(2, idx.unsqueeze(-1).expand(-1, -1, -1, int(x.size(-1))))


def _ln(spec: KvmSpec, x: torch.Tensor) -> torch.Tensor:
    # nn.LayerNorm(d_qk_head) named ln_s_k, model/kvm_mixer.py:93
    w = spec.ln_weight
    b = spec.ln_bias
    if w is None:
        w = torch.ones(spec.d_qk_head, dtype=x.dtype, device=x.device)
    if b is None:
        b = torch.zeros(spec.d_qk_head, dtype=x.dtype, device=x.device)
    return F.layer_norm(x, (spec.d_qk_head,), w.to(x.dtype), b.to(x.dtype), spec.ln_eps)


def _repeat_kv(spec: KvmSpec, x: torch.Tensor) -> torch.Tensor:
    # model/value_residual_mixin.py:278-281
    if spec.kv_group_size == 1:
        return x
    return x.repeat_interleave(spec.kv_group_size, dim=1)


def prepare_state_update_k(spec: KvmSpec, k_block: torch.Tensor) -> torch.Tensor:
    # model/kvm_mixer.py:120-129: rotary dims zeroed, then the shared LayerNorm.
    r = spec.rope_partial_dim
    return _ln(spec, torch.cat([torch.zeros_like(k_block[..., :r]), k_block[..., r:]], dim=-1))


def desired_state_len(spec: KvmSpec, ctx_len: int, available_context: int, current: int) -> int:
    # model/kvm_mixer.py:131-165
    ctx = max(int(ctx_len), 0)
    avail = max(int(available_context), 0)
    cur = max(int(current), 0)
    mode = spec.state_budget_mode
    if mode == "fixed":
        target = spec.state_min_len
    elif mode == "power_law":
        target = int(math.floor(spec.state_growth_factor * (float(ctx) ** spec.state_growth_exponent)))
        target = _round_down_to_multiple(target, spec.state_round_down)
        target = max(target, spec.state_min_len)
    elif mode == "kvm_saturation":
        t = float(ctx)
        target = int(math.floor((float(spec.state_saturation_n) * t) / (float(spec.state_saturation_n) + t)))
        target = _round_down_to_multiple(target, spec.state_round_down)
        target = max(target, spec.state_min_len)
    elif mode == "plus_one":
        # benchmark schedule: one new mean per block (an override of the method above)
        return max(min(cur + 1, avail, spec.max_state_len), cur)
    else:
        raise ValueError(f"Unsupported state_budget_mode={mode!r}")
    target = min(target, avail, spec.max_state_len)
    return max(target, cur)


def bswa_begin_for_total_len(spec: KvmSpec, total_len: int) -> int:
    # model/kvm_mixer.py:167-172
    end = _round_down_to_multiple(total_len + spec.chunk_len - 1, spec.chunk_len)
    return max(0, end - spec.n_bswa_chunks * spec.chunk_len)


# ----------------------------------------------------------------------------- attention


def _temps(spec: KvmSpec, like: torch.Tensor):
    # model/kvm_mixer.py:212-217 and :419-422; a tensor of ones (the reference's initial value)
    # when the spec carries no temperatures, so that the same broadcast multiply is executed
    if spec.kvm_use_head_temps:
        H = spec.num_attention_heads
        st, fr = spec.state_head_temp, spec.front_head_temp
        if st is None:
            st = torch.ones(H, dtype=like.dtype, device=like.device)
        if fr is None:
            fr = torch.ones(H, dtype=like.dtype, device=like.device)
        return st.view(1, H, 1, 1), fr.view(1, H, 1, 1)
    return 1.0, 1.0


def front_attention(spec: KvmSpec, q, k, v) -> torch.Tensor:
    # model/kvm_mixer.py:174-192 with is_causal=True (call site :423-432)
    _, front = _temps(spec, k)
    return F.scaled_dot_product_attention(
        q, _repeat_kv(spec, k) * front, _repeat_kv(spec, v), is_causal=True
    )


def attend_with_state_and_bswa(spec: KvmSpec, q, bswa_k, bswa_v, s_k, s_v, s_vlen) -> torch.Tensor:
    # model/kvm_mixer.py:194-229
    s_k_norm = _repeat_kv(spec, _ln(spec, s_k))
    bswa_k = _repeat_kv(spec, bswa_k)
    if spec.kvm_use_vlens:
        s_v_norm = (F.normalize(s_v.float(), dim=-1) * s_vlen).bfloat16()
    else:
        s_v_norm = s_v / s_vlen
    s_v_norm = _repeat_kv(spec, s_v_norm)
    bswa_v = _repeat_kv(spec, bswa_v)
    st, fr = _temps(spec, q)
    k_star = torch.cat([s_k_norm * st, bswa_k * fr], dim=2)
    v_star = torch.cat([s_v_norm, bswa_v], dim=2)
    if v_star.dtype != q.dtype:
        # the reference hard-codes .bfloat16() on the memory values; torch.cat promotes back to the
        # window dtype, so fp32 runs see bf16-rounded memory values in fp32 storage
        v_star = v_star.to(q.dtype)
    mask = lower_right_causal_mask(int(q.size(2)), int(k_star.size(2)), q.device)
    return F.scaled_dot_product_attention(q, k_star, v_star, attn_mask=mask, is_causal=False)


# ----------------------------------------------------------------------------- memory update


def split_append_merge_idx_by_maxsim(k_block, n_append: int, k_ref, want_scores: bool = False):
    # model/kvm_mixer.py:44-75
    B, H, C = int(k_block.size(0)), int(k_block.size(1)), int(k_block.size(2))
    n_append = min(max(int(n_append), 0), C)
    n_merge = C - n_append
    all_idx = torch.arange(C, device=k_block.device, dtype=torch.long).view(1, 1, C).expand(B, H, C)
    empty = all_idx[:, :, :0]
    if C == 0:
        return empty, empty, None
    if n_append == 0:
        return empty, all_idx, None
    if n_merge == 0:
        return all_idx, empty, None
    if int(k_ref.size(2)) == 0:
        return all_idx[:, :, n_merge:], all_idx[:, :, :n_merge], None
    scores = torch.matmul(k_block, k_ref.transpose(-1, -2)).float().max(dim=-1).values
    sorted_idx = torch.argsort(scores, dim=-1, descending=False)
    append_idx, _ = torch.sort(sorted_idx[..., :n_append], dim=-1)
    merge_idx, _ = torch.sort(sorted_idx[..., n_append:], dim=-1)
    return append_idx, merge_idx, (scores if want_scores else None)


def append_to_state(spec: KvmSpec, s_k, s_v, s_vlen, k_new, v_new):
    # model/kvm_mixer.py:231-248
    if int(k_new.size(2)) == 0:
        return s_k, s_v, s_vlen
    if spec.kvm_use_vlens:
        vlen_new = torch.norm(v_new.float(), dim=-1, keepdim=True)
    else:
        vlen_new = torch.ones_like(v_new[..., :1])
    return (
        torch.cat([s_k, k_new], dim=2),
        torch.cat([s_v, v_new], dim=2),
        torch.cat([s_vlen, vlen_new], dim=2),
    )


# Tie tolerances of the decision comparison (used only when decisions are forced from outside):
# a forced merge row is accepted if its oracle-side logit is within MERGE_TIE_TOL of the maximum
# (one bf16 rounding step of one key element moves a logit by about this much); gaps below
# MERGE_FP32_TOL * max(1,|logit|) are plain fp32 summation-order noise.
MERGE_TIE_TOL = 2e-2
MERGE_FP32_TOL = 1e-5


def merge_into_state(spec: KvmSpec, k_merge, v_merge, s_k, s_v, s_vlen, protected_slots: int, rec=None,
                     forced_best: torch.Tensor | None = None):
    # fp32 routing: model/kvm_fp32_routing_reference.py:24-49; key dtype: model/kvm_mixer.py:321-340
    s_k_norm = _ln(spec, s_k)
    if spec.routing == "fp32":
        logits = torch.matmul(k_merge.float(), s_k_norm.float().transpose(-1, -2))
    else:
        logits = torch.matmul(k_merge, s_k_norm.transpose(-1, -2))
    logits[..., :protected_slots] = float("-inf")
    best = logits.max(dim=-1, keepdim=True).indices
    own_best = best
    if forced_best is not None:
        fb = forced_best.long().unsqueeze(-1)
        top = logits.float().max(dim=-1, keepdim=True).values
        gap = top - logits.float().gather(-1, fb)
        differ = fb != best
        if rec is not None:
            rec.merge_differ = int(differ.sum())
            rec.merge_differ_fp32 = int((differ & (gap <= MERGE_FP32_TOL * top.abs().clamp_min(1.0))).sum())
            rec.merge_illegal = int((differ & ~(gap <= MERGE_TIE_TOL)).sum())
        best = fb
    scores = torch.scatter(
        torch.zeros_like(logits, dtype=k_merge.dtype), -1, best, torch.ones_like(logits, dtype=k_merge.dtype)
    )
    if rec is not None:
        rec.best_idx = own_best.squeeze(-1).clone()
        if int(logits.size(-1)) >= 2:
            top2 = logits.float().topk(2, dim=-1).values
            rec.margin = top2[..., 0] - top2[..., 1]
    s_k = s_k + (scores.mT @ k_merge)
    s_v = s_v + (scores.mT @ v_merge)
    if not spec.kvm_use_vlens:
        s_vlen = s_vlen + scores.sum(-1, keepdim=True)
    return s_k, s_v, s_vlen


def update_state_from_overflow_tokens(
    spec: KvmSpec, s_k, s_v, s_vlen, overflow_k, overflow_v, merge_gate, ctx_len: int, available_context: int,
    trace: list | None = None, forced: dict | None = None,
):
    """``forced`` (test use): {"append_idx": [B,Hkv,n_append] sorted token indices or None,
    "best_idx": [B,Hkv,n_merge] memory rows or None}.  The oracle then follows these decisions instead
    of its own, after recording whether each one is identical to its own, a legal tie, or wrong."""
    # model/kvm_mixer.py:250-319
    if int(overflow_k.size(2)) == 0:
        return s_k, s_v, s_vlen
    k_un = prepare_state_update_k(spec, overflow_k)
    v_un = overflow_v
    k_g = k_un * merge_gate if spec.kvm_use_merge_gate_keys else k_un
    v_g = v_un * merge_gate if spec.kvm_use_merge_gate_values else v_un
    if spec.kvm_apply_merge_gate_to_appends:
        k_ap, v_ap = k_g, v_g
    else:
        k_ap, v_ap = k_un, v_un
    cur = int(s_k.size(2))
    desired = desired_state_len(spec, ctx_len, available_context, cur)
    overflow_len = int(k_un.size(2))
    n_append = min(max(desired - cur, 0), overflow_len)
    rec = None
    if trace is not None:
        rec = UpdateRecord(int(ctx_len), int(available_context), cur, cur + n_append, n_append, None, None, None, None)
        trace.append(rec)
    if n_append > 0:
        want_sc = rec is not None or forced is not None
        append_idx, merge_idx, sc = split_append_merge_idx_by_maxsim(k_un, n_append, _ln(spec, s_k), want_sc)
        if rec is not None:
            rec.append_idx, rec.merge_idx, rec.append_scores = append_idx.clone(), merge_idx.clone(), sc
        if forced is not None and forced.get("append_idx") is not None and sc is not None:
            f_app = forced["append_idx"].long()
            differ_rows, illegal_rows = _check_forced_append(sc, n_append, append_idx, f_app)
            if rec is not None:
                rec.append_rows_differ, rec.append_rows_illegal = differ_rows, illegal_rows
            member = torch.zeros(sc.shape, dtype=torch.bool)
            member.scatter_(-1, f_app, True)
            all_idx = torch.arange(overflow_len).view(1, 1, -1).expand_as(member)
            append_idx = f_app
            merge_idx = all_idx[~member].view(sc.size(0), sc.size(1), overflow_len - n_append)
        k_append = _gather_by_idx(k_ap, append_idx)
        v_append = _gather_by_idx(v_ap, append_idx)
        k_merge = _gather_by_idx(k_g, merge_idx)
        v_merge = _gather_by_idx(v_g, merge_idx)
        s_k, s_v, s_vlen = append_to_state(spec, s_k, s_v, s_vlen, k_append, v_append)
    else:
        k_merge, v_merge = k_g, v_g
    if int(k_merge.size(2)) == 0:
        return s_k, s_v, s_vlen
    cur = int(s_k.size(2))
    protected = min(spec.sink_len, cur)
    if cur <= protected:
        raise AssertionError("KVM state update requires at least one non-sink slot before merging.")
    return merge_into_state(spec, k_merge, v_merge, s_k, s_v, s_vlen, protected, rec,
                            forced_best=None if forced is None else forced.get("best_idx"))


def _check_forced_append(scores, n_append: int, own_idx, forced_idx):
    """Rows whose forced append set differs from the oracle's, and how many of those are not explained
    by equal (or one-bf16-step apart) scores at the cut between appended and merged tokens."""
    differ = illegal = 0
    B, H, C = scores.shape
    for b in range(B):
        for h in range(H):
            own = set(own_idx[b, h].tolist())
            got = set(forced_idx[b, h].tolist())
            if own == got:
                continue
            differ += 1
            sc = scores[b, h]
            thr = float(sc.sort().values[n_append - 1])
            tol = abs(thr) * 2.0 ** -7 + 1e-6
            must = {i for i in range(C) if float(sc[i]) < thr - tol}
            may = {i for i in range(C) if float(sc[i]) <= thr + tol}
            if not (must <= got <= may) or len(got) != n_append:
                illegal += 1
    return differ, illegal


# ----------------------------------------------------------------------------- prefill / decode


def prefill(spec: KvmSpec, q, k, v, merge_gate, *, training: bool = False, trace: list | None = None,
            snapshots: list | None = None, forced: list | None = None):
    """model/kvm_mixer.py:403-516 up to (not including) ``c_proj``.

    Returns (y [B,T,Hq*Dv], state) where ``state`` holds exactly the entries the reference writes
    into its cache (model/kvm_mixer.py:501-514) plus ``total_len``.
    ``snapshots`` (optional list) receives (s_k, s_v, s_vlen) as seen by each recurrent query block.
    """
    B, _, T, _ = q.size()
    C = spec.chunk_len
    bswa_len = spec.n_bswa_chunks * C
    front = min(T, bswa_len)
    outs = [front_attention(spec, q[:, :, :front], k[:, :, :front], v[:, :, :front])]

    init_len = min(T, C)
    s_k = prepare_state_update_k(spec, k[..., :init_len, :])
    s_v = v[..., :init_len, :]
    if spec.kvm_apply_merge_gate_to_initial_state:
        s_k = s_k * merge_gate[..., :init_len, :]
        s_v = s_v * merge_gate[..., :init_len, :]
    if spec.kvm_use_vlens:
        s_vlen = torch.norm(v[..., :init_len, :].float(), dim=-1, keepdim=True)
    else:
        s_vlen = torch.ones_like(v[..., :init_len, :1])
    coverage = init_len
    n_upd = 0

    for qb in range(front, T, C):
        qe = min(T, qb + C)
        bb = bswa_begin_for_total_len(spec, qe)
        if bb != coverage:
            raise AssertionError("KVM prefill state coverage drifted from the active BSWA window.")
        if snapshots is not None:
            snapshots.append((s_k.clone(), s_v.clone(), s_vlen.clone()))
        outs.append(
            attend_with_state_and_bswa(spec, q[:, :, qb:qe], k[:, :, bb:qe], v[:, :, bb:qe], s_k, s_v, s_vlen)
        )
        if training and qe >= T:
            break
        nb = bswa_begin_for_total_len(spec, min(T, qe + C))
        if nb > bb:
            s_k, s_v, s_vlen = update_state_from_overflow_tokens(
                spec, s_k, s_v, s_vlen, k[:, :, bb:nb], v[:, :, bb:nb], merge_gate[:, :, bb:nb],
                ctx_len=qe, available_context=nb, trace=trace,
                forced=None if forced is None else forced[n_upd],
            )
            n_upd += 1
            coverage = nb

    y = torch.cat(outs, dim=-2).transpose(1, 2).contiguous().view(B, T, -1)
    bb = bswa_begin_for_total_len(spec, T)
    if coverage != max(init_len, bb):
        raise AssertionError("KVM prefill state progression drifted from the decode-state bookkeeping.")
    state = {
        "kvm_s_k": s_k,
        "kvm_s_v": s_v,
        "kvm_s_vlen": s_vlen,
        "kvm_state_coverage_len": coverage,
        "kvm_bswa_begin": bb,
        "kvm_bswa_k": k[:, :, bb:, :],
        "kvm_bswa_v": v[:, :, bb:, :],
        "kvm_bswa_merge_gate": merge_gate[:, :, bb:, :],
        "total_len": T,
    }
    return y, state


def decode_step(spec: KvmSpec, q, k, v, merge_gate, state: dict[str, Any], trace: list | None = None,
                forced: dict | None = None):
    """model/kvm_mixer.py:572-713 up to ``c_proj``; returns (y [B,1,Hq*Dv], new state)."""
    B, _, n, _ = q.size()
    if n != 1:
        raise AssertionError("KVM cached decode expects single-token inputs.")
    C = spec.chunk_len
    s_k, s_v, s_vlen = state["kvm_s_k"], state["kvm_s_v"], state["kvm_s_vlen"]
    old_begin = int(state["kvm_bswa_begin"])
    coverage = int(state["kvm_state_coverage_len"])
    past = int(state["total_len"])
    full_k = torch.cat([state["kvm_bswa_k"], k], dim=2)
    full_v = torch.cat([state["kvm_bswa_v"], v], dim=2)
    full_g = torch.cat([state["kvm_bswa_merge_gate"], merge_gate], dim=2)
    total = past + 1
    direct_target = min(total, C)
    new_begin = bswa_begin_for_total_len(spec, total)
    new_cov = max(direct_target, new_begin)

    if coverage < direct_target:
        lo = max(coverage - old_begin, 0)
        hi = max(direct_target - old_begin, 0)
        s_k, s_v, s_vlen = append_to_state(
            spec, s_k, s_v, s_vlen, prepare_state_update_k(spec, full_k[:, :, lo:hi]), full_v[:, :, lo:hi]
        )
        coverage = direct_target
    if coverage > new_cov:
        raise AssertionError("KVM cache state coverage cannot shrink during decoding.")
    if coverage < new_cov:
        lo = max(coverage - old_begin, 0)
        hi = max(new_cov - old_begin, 0)
        if hi - lo != C:
            raise AssertionError("KVM decode can only materialize one overflow BSWA chunk per step.")
        s_k, s_v, s_vlen = update_state_from_overflow_tokens(
            spec, s_k, s_v, s_vlen, full_k[:, :, lo:hi], full_v[:, :, lo:hi], full_g[:, :, lo:hi],
            ctx_len=spec.n_bswa_chunks * C + coverage, available_context=coverage + C, trace=trace,
            forced=forced,
        )
        coverage = new_cov
    lo = max(new_begin - old_begin, 0)
    hi = max(total - old_begin, 0)
    nk, nv, ng = full_k[:, :, lo:hi], full_v[:, :, lo:hi], full_g[:, :, lo:hi]
    active = int(s_k.size(2)) if new_begin > 0 else 0
    out = attend_with_state_and_bswa(spec, q, nk, nv, s_k[:, :, :active], s_v[:, :, :active], s_vlen[:, :, :active])
    y = out.transpose(1, 2).contiguous().view(B, 1, -1)
    new_state = {
        "kvm_s_k": s_k,
        "kvm_s_v": s_v,
        "kvm_s_vlen": s_vlen,
        "kvm_state_coverage_len": coverage,
        "kvm_bswa_begin": new_begin,
        "kvm_bswa_k": nk,
        "kvm_bswa_v": nv,
        "kvm_bswa_merge_gate": ng,
        "total_len": total,
    }
    return y, new_state


def slot_histogram(best_idx: torch.Tensor, n_slots: int) -> torch.Tensor:
    """Per-slot count of routed tokens for one update: [B,Hkv,n_slots] int64."""
    B, H, _ = best_idx.shape
    out = torch.zeros(B, H, n_slots, dtype=torch.long)
    out.scatter_add_(2, best_idx.long().cpu(), torch.ones_like(best_idx, dtype=torch.long).cpu())
    return out


# ------------------------------------------------------------------------------------------------ prologue
def prologue(q_lin, k_lin, v_lin, gate_lin, *, n_q_heads: int, n_kv_heads: int, shift=None, prev=None, ln_q=None, ln_k=None,
             ln_eps: float = 1e-5, position_embeddings=None):
    """What the reference does between its projections and the mixer's post-QKV tensors, on the projections' outputs
    ([B,T,H*D]; v after a pre-shift value residual): token shift ``x + scale * (previous token - x)`` with the cached
    last token of the previous call or the first token itself (model/tokenshift.py:11-37,
    model/value_residual_mixin.py:219-224), per-head LayerNorm of q and k (model/value_residual_mixin.py:230-235),
    rotary embedding on interleaved pairs with the sign folded into the sine table (model/rwkv7_backbone.py:76-88),
    merge gate ``1 + elu(.)`` and the head-major views (model/kvm_mixer.py:381-399).  The same tensor operations in the
    same order as the reference, so every intermediate is rounded where the reference rounds it.

    shift = (x_q, x_k, x_v) or None; prev = (q, k, v) rows [B,1,H*D] or None; ln_q / ln_k = (weight, bias) or None.
    Returns q [B,Hq,T,D], k, v [B,Hkv,T,D], merge_gate [B,Hkv,T,1]."""
    B, T, _ = q_lin.shape

    def shifted(x, scale, prev_token):
        if prev_token is None:
            prev_token = x[:, :1]
        elif prev_token.dtype != x.dtype:
            prev_token = prev_token.to(x.dtype)
        return x + scale * (torch.cat([prev_token, x[:, :-1]], dim=1) - x)

    q, k, v = q_lin, k_lin, v_lin
    if shift is not None:
        pv = prev if prev is not None else (None, None, None)
        q, k, v = shifted(q, shift[0], pv[0]), shifted(k, shift[1], pv[1]), shifted(v, shift[2], pv[2])
    q = q.reshape(B, T, n_q_heads, -1)
    k = k.reshape(B, T, n_kv_heads, -1)
    v = v.reshape(B, T, n_kv_heads, -1)
    if ln_q is not None:
        q = F.layer_norm(q, (q.size(-1),), ln_q[0], ln_q[1], ln_eps)
        k = F.layer_norm(k, (k.size(-1),), ln_k[0], ln_k[1], ln_eps)
    if position_embeddings is not None:
        cos, sin = position_embeddings

        def rotary(x):
            flipped = x.view(*x.shape[:-1], x.shape[-1] // 2, 2).flip(-1).view(x.shape)
            return cos * x + sin * flipped

        q, k = rotary(q), rotary(k)
    if gate_lin is not None:
        gate = 1.0 + F.elu(gate_lin.view(B, T, n_kv_heads, 1)).transpose(1, 2)
    else:
        gate = torch.ones((B, n_kv_heads, T, 1), dtype=torch.float)
    return q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2), gate
