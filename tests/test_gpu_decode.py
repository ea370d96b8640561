"""GPU parity of the decode path (ring write, boundary memory update, split-K attention)."""

import pytest
import torch

from kvm_paper_b200 import ops
from oracle import kvm_oracle as ko
from tests.helpers import SMALL_FIXTURES, load_fixture, spec_from_fixture, assert_close_bf16
from tests import gpu_helpers as gh

pytestmark = pytest.mark.gpu


def _decode_against_oracle(spec, cache, state, dq, dk, dv, dg, seqs=None):
    """Step the device cache and the oracle in lockstep; the oracle follows the device's routing
    decisions after checking them (see oracle ``forced``)."""
    B = dq.size(0)
    Hkv = spec.num_key_value_heads
    trace = []
    ys_dev, ys_ref = [], []
    for i in range(dq.size(2)):
        qi, ki, vi, gi = (t[:, :, i:i + 1] for t in (dq, dk, dv, dg))
        out = cache.step(qi.cuda(), ki.cuda(), vi.cuda(), gi.cuda(), want_route=True).clone()
        forced = None
        if cache._last_any_update:
            forced = gh.decisions_from_route(cache.route, B, Hkv)
        with torch.no_grad():
            y, state = ko.decode_step(spec, qi, ki, vi, gi, state, trace=trace, forced=forced)
        ys_dev.append(out.cpu())
        ys_ref.append(y)
    return torch.cat(ys_dev, 1), torch.cat(ys_ref, 1), state, trace


@pytest.mark.parametrize("name", SMALL_FIXTURES)
def test_decode_after_prefill_matches_oracle(name):
    fix = load_fixture(name)
    if fix["decode_qkv"] is None:
        pytest.skip("fixture has no decode steps")
    spec = gh.bf16_spec(spec_from_fixture(fix))
    pq = fix["post_qkv"]
    q, k, v, g = (pq[n].to(torch.bfloat16) for n in ("q", "k", "v", "merge_gate"))
    B = q.size(0)
    params, plan, res = gh.device_prefill(spec, q, k, v, g)
    forced = [gh.decisions_from_route(res.route[:, u], B, spec.num_key_value_heads) for u in range(1, plan.n_updates + 1)]
    ptrace = []
    with torch.no_grad():
        _, state = ko.prefill(spec, q, k, v, g, forced=forced, trace=ptrace)
    cache = ops.decode_cache_from_prefill(params, res, k.cuda(), v.cuda(), g.cuda(), gh.desired_fn(spec))
    dq, dk, dv, dg = (t.to(torch.bfloat16) for t in fix["decode_qkv"])
    y_dev, y_ref, state, trace = _decode_against_oracle(spec, cache, state, dq, dk, dv, dg)
    gh.assert_routing_ok(gh.summarize(trace))
    assert_close_bf16(y_dev, y_ref, f"{name} decode activations")
    total = gh.summarize(ptrace + trace)
    if pq["q"].dtype == torch.bfloat16 and total["merge_differ"] == 0 and total["append_rows_differ"] == 0:
        assert_close_bf16(y_dev, fix["y_decode"], f"{name} decode activations vs reference fixture")
    # carried state in the reference's eager layout
    sd = cache.logical_state_dict()
    S = state["kvm_s_k"].size(2)
    assert sd["kvm_s_k"].size(2) == S
    assert sd["kvm_state_coverage_len"] == state["kvm_state_coverage_len"]
    assert sd["kvm_bswa_begin"] == state["kvm_bswa_begin"]
    gh.compare_memory(cache.memory, state, S, name + " decode")
    assert torch.equal(sd["kvm_bswa_k"].cpu(), state["kvm_bswa_k"])
    assert torch.equal(sd["kvm_bswa_v"].cpu(), state["kvm_bswa_v"])
    assert torch.equal(sd["kvm_bswa_merge_gate"].cpu(), state["kvm_bswa_merge_gate"])
    assert cache.total_len.cpu().tolist() == [state["total_len"]] * B
    assert cache.state_len.cpu().tolist() == [S] * B


RAGGED_CASES = {
    # query heads, kv heads, head dim, rope dim, block, contexts, decode steps
    "gqa2_d64": (4, 2, 64, 32, 32, [70, 150, 97, 255, 31, 128], 70),
    # 16 query heads on one kv head (two 8-wide head tiles per MMA), rows longer than one 128-row chunk
    "gqa16_d128": (16, 1, 128, 64, 128, [380, 640, 127, 500], 40),
    # one query head per kv head, head dim 32 (unswizzled TMA boxes)
    "mha_d32": (2, 2, 32, 16, 64, [200, 66, 450], 70),
    # block of 512 tokens: the boundary update reads the block from global memory instead of staging it
    "gqa2_c512": (2, 1, 128, 64, 512, [1530, 2040, 1000], 30),
}


@pytest.mark.parametrize("case", sorted(RAGGED_CASES))
def test_decode_ragged_batch_matches_per_sequence_oracle(case):
    """Sequences with different context lengths in one batch (the reference cannot batch these): every
    sequence is checked against its own B=1 oracle run; different sequences cross block boundaries at
    different steps."""
    torch.manual_seed(21)
    Hq, Hkv, D, rope, C, lens, n_steps = RAGGED_CASES[case]
    spec = ko.KvmSpec(Hq, Hkv, D, D, rope, C, 2, 8, 1, "power_law", state_growth_factor=4.0, state_min_len=C)
    _ragged_batch_against_oracle(spec, lens, n_steps)


def test_decode_benchmark_range_contexts_match_per_sequence_oracle():
    """Contexts from the range of the decode benchmark (4096 .. 65536 tokens, 16 heads x 128, block 256, one new
    mean per block: memories of 270 .. 507 rows, rows spanning several 128-row chunks and several CTAs), 260
    steps so that every sequence crosses a block boundary, each sequence against its own B=1 oracle run."""
    torch.manual_seed(22)
    spec = gh.bf16_spec(ko.KvmSpec(16, 16, 128, 128, 64, 256, 2, 4, 1, "plus_one", state_min_len=256))
    traces = _ragged_batch_against_oracle(spec, [65000, 4100, 33023, 20479, 48000], 260)
    total = gh.summarize([r for t in traces for r in t])
    gh.record_counts("decode_benchmark_range", total)
    assert total["updates"] >= 5 and total["merge_tokens"] >= 5 * 16 * 255


def _ragged_batch_against_oracle(spec, lens, n_steps):
    Hq, Hkv, D, C = spec.num_attention_heads, spec.num_key_value_heads, spec.d_qk_head, spec.chunk_len
    B = len(lens)
    params = gh.layer_params(spec)
    states, inputs = [], []
    cache = ops.KvmDecodeCache(params, B, 2 * C, gh.desired_fn(spec))
    for b, T in enumerate(lens):
        q = torch.randn(1, Hq, T + n_steps, D).bfloat16()
        k = torch.nn.functional.layer_norm(torch.randn(1, Hkv, T + n_steps, D), (D,)).bfloat16()
        v = torch.randn(1, Hkv, T + n_steps, D).bfloat16()
        g = (1 + torch.nn.functional.elu(torch.randn(1, Hkv, T + n_steps, 1))).bfloat16()
        inputs.append((q, k, v, g))
        _, plan, res = gh.device_prefill(spec, q[:, :, :T], k[:, :, :T], v[:, :, :T], g[:, :, :T])
        forced = [gh.decisions_from_route(res.route[:, u], 1, Hkv) for u in range(1, plan.n_updates + 1)]
        with torch.no_grad():
            _, st = ko.prefill(spec, q[:, :, :T], k[:, :, :T], v[:, :, :T], g[:, :, :T], forced=forced)
        states.append(st)
        S = plan.final_state_len
        bb = plan.bswa_begin
        cache.load_sequence(b, k_sum=res.memory.k_sum[:, :S], v_sum=res.memory.v_sum[:, :S], vlen=res.memory.vlen[:, :S],
                            k_attn=res.memory.k_attn[:, :S], v_attn=res.memory.v_attn[:, :S],
                            window_k=k[0, :, bb:T].cuda(), window_v=v[0, :, bb:T].cuda(), window_gate=g[0, :, bb:T].cuda(),
                            total_len=T)
    cache.commit_lengths()
    traces = [[] for _ in lens]
    for i in range(n_steps):
        step_in = [torch.cat([inp[j][:, :, lens[b] + i: lens[b] + i + 1] for b, inp in enumerate(inputs)], 0) for j in range(4)]
        out = cache.step(*(t.cuda() for t in step_in), want_route=True).clone().cpu()
        for b in range(B):
            forced = None
            if cache._last_n_append is not None and cache._last_n_append[b] >= 0:
                forced = gh.decisions_from_route(cache.route[b * Hkv:(b + 1) * Hkv], 1, Hkv)
            with torch.no_grad():
                y, states[b] = ko.decode_step(spec, *(t[b:b + 1] for t in step_in), states[b], trace=traces[b], forced=forced)
            assert_close_bf16(out[b:b + 1], y, f"seq {b} step {i}", mean_rel_tol=5e-3)
    for b in range(B):
        gh.assert_routing_ok(gh.summarize(traces[b]))
        sd = cache.logical_state_dict(b)
        assert sd["kvm_s_k"].size(2) == states[b]["kvm_s_k"].size(2)
        assert torch.equal(sd["kvm_bswa_k"].cpu(), states[b]["kvm_bswa_k"])
        scale = max(1.0, float(states[b]["kvm_s_k"].float().abs().max()))
        assert_close_bf16(sd["kvm_s_k"].cpu(), states[b]["kvm_s_k"], f"seq {b} kvm_s_k", max_abs_tol=2e-2 * scale)
    assert cache.total_len.cpu().tolist() == [t + n_steps for t in lens]
    assert sum(len(t) for t in traces) >= 2  # boundary updates happened
    cache.check_status()                     # no kernel reported an expired wait
    return traces


def test_decode_adopts_reference_eager_cache():
    """A cache written in the reference's eager layout (from the fixture) is adopted: the attention
    view of the memory is rebuilt on the device and decoding continues from it."""
    fix = load_fixture("powerlaw_bf16")
    spec = gh.bf16_spec(spec_from_fixture(fix))
    params = gh.layer_params(spec)
    st = fix["state_prefill"]
    B, Hkv, S, D = st["kvm_s_k"].shape
    cache = ops.KvmDecodeCache(params, B, S + spec.chunk_len, gh.desired_fn(spec))
    for b in range(B):
        cache.load_sequence(b, k_sum=st["kvm_s_k"][b].cuda(), v_sum=st["kvm_s_v"][b].cuda(), vlen=st["kvm_s_vlen"][b].cuda(),
                            window_k=st["kvm_bswa_k"][b].cuda(), window_v=st["kvm_bswa_v"][b].cuda(),
                            window_gate=st["kvm_bswa_merge_gate"][b].cuda(), total_len=st["total_len"])
    cache.commit_lengths(refresh_attention_view=True)
    dq, dk, dv, dg = fix["decode_qkv"]
    state = {k: v for k, v in st.items()}
    y_dev, y_ref, state, trace = _decode_against_oracle(spec, cache, state, dq, dk, dv, dg)
    summary = gh.summarize(trace)
    gh.assert_routing_ok(summary)
    assert_close_bf16(y_dev, y_ref, "decode from adopted eager cache vs oracle")
    if summary["merge_differ"] == 0 and summary["append_rows_differ"] == 0:
        assert_close_bf16(y_dev, fix["y_decode"], "decode from adopted eager cache vs reference fixture")


def test_decode_run_equals_step_by_step():
    """kvm_decode_run (n tokens in one C call) gives the same bits as n calls of kvm_decode_step."""
    torch.manual_seed(9)
    spec = ko.KvmSpec(4, 2, 64, 64, 32, 32, 2, 8, 1, "power_law", state_growth_factor=4.0, state_min_len=32)
    B, T, n = 3, 32 * 4 + 20, 50
    q = torch.randn(B, 4, T, 64).bfloat16()
    k = torch.nn.functional.layer_norm(torch.randn(B, 2, T, 64), (64,)).bfloat16()
    v = torch.randn(B, 2, T, 64).bfloat16()
    g = (1 + torch.nn.functional.elu(torch.randn(B, 2, T, 1))).bfloat16()
    params, plan, res = gh.device_prefill(spec, q, k, v, g)
    mk = lambda: ops.decode_cache_from_prefill(params, res, k.cuda(), v.cuda(), g.cuda(), gh.desired_fn(spec))  # noqa: E731
    c1, c2 = mk(), mk()
    dq = torch.randn(n, B, 4, 1, 64).bfloat16().cuda()
    dk = torch.nn.functional.layer_norm(torch.randn(n, B, 2, 1, 64), (64,)).bfloat16().cuda()
    dv = torch.randn(n, B, 2, 1, 64).bfloat16().cuda()
    dg = (1 + torch.nn.functional.elu(torch.randn(n, B, 2, 1, 1))).bfloat16().cuda()
    want = torch.stack([c1.step(dq[i], dk[i], dv[i], dg[i]).clone().view(B, -1) for i in range(n)])
    got = c2.run(dq, dk, dv, dg)
    torch.cuda.synchronize()
    assert torch.equal(got, want)
    assert torch.equal(c1.memory.k_sum, c2.memory.k_sum) and torch.equal(c1.total_len, c2.total_len)
    assert c1.update_count == c2.update_count and c1.update_count >= 3


def test_decode_counters_and_lengths_stay_consistent_when_most_ctas_have_no_work():
    """One short sequence: the chunk list has one or two entries, so all but one or two CTAs of the persistent
    grid have no work.  The lengths may only advance once every CTA has read them: after every step the
    lengths are exact and the workspace counters are back at zero (a CTA that saw advanced lengths would take
    work of the next token and leave counters behind)."""
    torch.manual_seed(3)
    spec = ko.KvmSpec(2, 1, 64, 64, 32, 32, 2, 4, 1, "power_law", state_growth_factor=4.0, state_min_len=32)
    T, n = 40, 150
    q = torch.randn(1, 2, T + n, 64).bfloat16().cuda()
    k = torch.nn.functional.layer_norm(torch.randn(1, 1, T + n, 64), (64,)).bfloat16().cuda()
    v = torch.randn(1, 1, T + n, 64).bfloat16().cuda()
    g = (1 + torch.nn.functional.elu(torch.randn(1, 1, T + n, 1))).bfloat16().cuda()
    params, plan, res = gh.device_prefill(spec, q[:, :, :T], k[:, :, :T], v[:, :, :T], g[:, :, :T])
    cache = ops.decode_cache_from_prefill(params, res, k[:, :, :T], v[:, :, :T], g[:, :, :T], gh.desired_fn(spec))
    n_counters = cache.kv_rows + cache.batch + 1
    for i in range(T, T + n):
        cache.step(*(t[:, :, i:i + 1] for t in (q, k, v, g)))
        head = cache._ws[: 4 * n_counters].view(torch.int32)
        assert cache.total_len.cpu().tolist() == [i + 1], f"step {i - T}"
        assert cache.state_len.cpu().tolist() == [int(cache.state_len_h[0])]
        assert int(head.abs().sum()) == 0, f"step {i - T}: counters {head.cpu().tolist()}"
    cache.check_status()
