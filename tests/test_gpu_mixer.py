"""The drop-in class on the GPU: ``SequenceMixer.forward_inference`` with a carried-state cache, prefill then
single-token steps, as ``Block.forward_attn`` of the reference drives it (model/rwkv7_backbone.py:219-227,
model/kvm_mixer.py:527-570), with the weights and hidden inputs of the golden fixtures.

The prologue (projections, token shift, LayerNorm, RoPE, gate) runs in PyTorch on the GPU here and ran on the
CPU when the reference produced the fixtures; bf16 GEMMs of the two differ in the last bit of some elements, so
the chain of evidence is: (1) the post-QKV tensors the class produces on the GPU equal the reference's up to
bf16 rounding; (2) what the class returns equals the oracle evaluated on exactly those tensors (the oracle
follows the device's routing decisions after classifying each one); (3) where every decision also equals the
one the reference itself recorded, the result is compared with the reference's own activations."""

import pytest
import torch

from kvm_paper_b200 import ops
from kvm_paper_b200.mixer import SequenceMixer, StatesCache
from oracle import kvm_oracle as ko
from tests import gpu_helpers as gh
from tests.helpers import (assert_close_bf16, load_fixture, max_abs, mean_rel, mixer_from_fixture, rotary_tables,
                           spec_from_fixture)

pytestmark = pytest.mark.gpu

BF16_FIXTURES = ["powerlaw_bf16", "plusone_bf16", "saturation_bf16"]


def _drive(m, cfg, fix, cache, n_decode, captured=None):
    """Prefill then ``n_decode`` single-token calls through forward_inference; ``captured`` (a list) receives
    (post-QKV tensors, routing decisions) of every call."""
    T, B = fix["case"]["T"], fix["case"]["B"]
    x, vf = fix["x"].cuda(), None if fix["v_first"] is None else fix["v_first"].cuda()
    cut = lambda t, a, b: None if t is None else t[:, a:b]  # noqa: E731
    if captured is not None:
        m.capture_routes = True
        for name in ("forward_prefill", "forward_single"):
            inner = getattr(m, name)

            def wrapped(q, k, v, g, *a, _inner=inner, **kw):
                y = _inner(q, k, v, g, *a, **kw)
                route = None if m.last_route is None else m.last_route.clone()
                captured.append(((q.clone(), k.clone(), v.clone(), g.clone()), route))
                return y

            setattr(m, name, wrapped)
    pos = torch.arange(T).view(1, T).expand(B, T)
    rot = tuple(t.cuda() for t in rotary_tables(cfg, m.d_qk_head, pos))
    ys = []
    with torch.no_grad():
        y_prefill = m.forward_inference(x[:, :T], cut(vf, 0, T), rot, None, cache)
        for i in range(n_decode):
            pos = torch.full((B, 1), T + i, dtype=torch.long)
            rot = tuple(t.cuda() for t in rotary_tables(cfg, m.d_qk_head, pos))
            ys.append(m.forward_inference(x[:, T + i:T + i + 1], cut(vf, T + i, T + i + 1), rot, None, cache).clone())
    return y_prefill, (torch.cat(ys, 1) if ys else None)


@pytest.mark.parametrize("name", BF16_FIXTURES)
def test_forward_inference_prefill_then_decode_matches_reference(name):
    fix = load_fixture(name)
    cfg, m = mixer_from_fixture(fix)
    m.c_proj = torch.nn.Identity()          # the fixtures hold the pre-projection activations
    m.check_device_status = True            # every call also reads the kernels' status word
    m = m.cuda()
    n_decode = fix["case"]["n_decode"]
    B, Hkv = fix["case"]["B"], m.num_key_value_heads
    cache = StatesCache()
    captured = []
    y_prefill, y_decode = _drive(m, cfg, fix, cache, n_decode, captured)
    assert y_prefill.shape == fix["y_prefill"].shape and len(captured) == 1 + n_decode

    # (1) the prologue on the GPU against the reference's post-QKV tensors: equal up to bf16 rounding
    (q, k, v, g), route = captured[0]
    for got, key in ((q, "q"), (k, "k"), (v, "v"), (g, "merge_gate")):
        want = fix["post_qkv"][key]
        assert got.shape == want.shape
        assert mean_rel(got.cpu(), want) <= 2e-3 and max_abs(got.cpu(), want) <= 2.0 ** -5 * max(1.0, float(want.abs().max())), key

    # (2) the kernels behind the class against the oracle on the class's own post-QKV tensors
    spec = gh.bf16_spec(spec_from_fixture(fix))
    plan = m.make_prefill_plan(fix["case"]["T"])
    forced = [gh.decisions_from_route(route[:, u], B, Hkv) for u in range(1, plan.n_updates + 1)]
    trace = []
    with torch.no_grad():
        y_ref, state = ko.prefill(spec, q.cpu(), k.cpu(), v.cpu(), g.cpu(), trace=trace, forced=forced)
        refs = []
        for (dq, dk, dv, dg), r in captured[1:]:
            f = None if r is None else gh.decisions_from_route(r, B, Hkv)
            y, state = ko.decode_step(spec, dq.cpu(), dk.cpu(), dv.cpu(), dg.cpu(), state, trace=trace, forced=f)
            refs.append(y)
    y_dec_ref = torch.cat(refs, 1)
    summary = gh.summarize(trace)
    gh.assert_routing_ok(summary)
    assert_close_bf16(y_prefill.cpu(), y_ref, f"{name} forward_inference prefill vs oracle")
    assert_close_bf16(y_decode.cpu(), y_dec_ref, f"{name} forward_inference decode vs oracle")

    # the carried state in the reference's eager layout, against the oracle's
    T = fix["case"]["T"]
    assert cache.get_seq_length(m.layer_idx) == T + n_decode
    dc = cache.get_states(m.layer_idx)[SequenceMixer._CACHE_DECODE]
    assert isinstance(dc, ops.KvmDecodeCache) and dc.owner is m
    sd, want = dc.logical_state_dict(), fix["state_final"]
    assert sd["kvm_state_coverage_len"] == want["kvm_state_coverage_len"] and sd["kvm_bswa_begin"] == want["kvm_bswa_begin"]
    assert sd["kvm_s_k"].shape == want["kvm_s_k"].shape
    gh.compare_memory(dc.memory, state, state["kvm_s_k"].size(2), name + " carried memory")
    for key in ("kvm_bswa_k", "kvm_bswa_v", "kvm_bswa_merge_gate"):
        assert torch.equal(sd[key].cpu(), state[key]), key
    for key in ("att_q_final_token", "att_k_final_token", "att_v_final_token", "att_x_final_token"):
        assert key in cache.get_states(m.layer_idx)   # token-shift / value-residual carry-overs of the prologue

    # (3) against the reference's own activations, where the device took exactly the reference's decisions
    same = len(trace) == len(fix["updates"])
    for rec, want_u in zip(trace, fix["updates"]):
        for mine, theirs in ((rec.best_idx, want_u.get("best_idx")), (rec.append_idx, want_u.get("append_idx"))):
            same = same and ((mine is None) == (theirs is None)) and (mine is None or torch.equal(mine, theirs))
    same = same and summary["merge_differ"] == 0 and summary["append_rows_differ"] == 0
    print(f"{name}: decisions identical to the reference's: {same}; vs reference prefill mean-rel "
          f"{mean_rel(y_prefill.cpu(), fix['y_prefill']):.3e}, decode mean-rel {mean_rel(y_decode.cpu(), fix['y_decode']):.3e}")
    if same:
        # inputs differ by bf16 rounding of the prologue, so the bound is wider than the kernel tolerance
        assert_close_bf16(y_prefill.cpu(), fix["y_prefill"], f"{name} vs reference prefill", max_abs_tol=0.25, mean_rel_tol=2e-2)
        assert_close_bf16(y_decode.cpu(), fix["y_decode"], f"{name} vs reference decode", max_abs_tol=0.25, mean_rel_tol=2e-2)


def test_forward_single_rejects_a_cache_of_another_mixer_and_drifted_lengths():
    fix = load_fixture("powerlaw_bf16")
    cfg, m = mixer_from_fixture(fix)
    m.c_proj = torch.nn.Identity()
    m = m.cuda()
    cache = StatesCache()
    _drive(m, cfg, fix, cache, 1)
    _, other = mixer_from_fixture(fix)
    other.c_proj = torch.nn.Identity()
    other = other.cuda()
    T = fix["case"]["T"]
    x = fix["x"].cuda()[:, T + 1:T + 2]
    vf = fix["v_first"].cuda()[:, T + 1:T + 2]
    rot = tuple(t.cuda() for t in rotary_tables(cfg, m.d_qk_head, torch.full((1, 1), T + 1, dtype=torch.long)))
    with torch.no_grad():
        with pytest.raises(RuntimeError):      # the decode state belongs to `m`
            other.forward_inference(x, vf, rot, None, cache)
        cache._seen[m.layer_idx] += 3           # the layer cache and the device cache disagree on the length
        with pytest.raises(AssertionError):
            m.forward_inference(x, vf, rot, None, cache)
