"""GPU parity of the prefill path (memory chain + block attention) through the C ABI."""

import pytest
import torch

from oracle import kvm_oracle as ko
from tests.helpers import (SMALL_FIXTURES, load_fixture, spec_from_fixture, assert_close_bf16, max_abs,
                           assert_not_worse_than_reference)
from tests import gpu_helpers as gh

pytestmark = pytest.mark.gpu


def _oracle_following_device(spec, q, k, v, g, res, plan, B):
    Hkv = spec.num_key_value_heads
    forced = [gh.decisions_from_route(res.route[:, u], B, Hkv) for u in range(1, plan.n_updates + 1)]
    trace = []
    with torch.no_grad():
        y, st = ko.prefill(spec, q, k, v, g, trace=trace, forced=forced)
    return y, st, trace


@pytest.mark.parametrize("name", SMALL_FIXTURES)
def test_prefill_matches_oracle_and_reference_fixture(name):
    fix = load_fixture(name)
    spec = gh.bf16_spec(spec_from_fixture(fix))
    pq = fix["post_qkv"]
    q, k, v, g = (pq[n].to(torch.bfloat16) for n in ("q", "k", "v", "merge_gate"))
    B = q.size(0)
    params, plan, res = gh.device_prefill(spec, q, k, v, g)
    # schedule equals what the reference walked through
    recs = fix["updates"][: fix["n_prefill_updates"]]
    assert plan.n_updates == len(recs)
    assert plan.state_before[1:] == [r["state_before"] for r in recs]
    assert [a + b for a, b in zip(plan.state_before, plan.n_append)][1:] == [r["state_after"] for r in recs]

    y, st, trace = _oracle_following_device(spec, q, k, v, g, res, plan, B)
    summary = gh.summarize(trace)
    gh.assert_routing_ok(summary)
    assert_close_bf16(res.out.cpu(), y, f"{name} activations vs oracle")
    gh.compare_memory(res.memory, st, plan.final_state_len, name)
    # fp32 evaluation of the same bf16 inputs along the same memory trajectory
    forced = [gh.decisions_from_route(res.route[:, u], B, spec.num_key_value_heads) for u in range(1, plan.n_updates + 1)]
    with torch.no_grad():
        y32, _ = ko.prefill(gh.fp32_spec(spec), q.float(), k.float(), v.float(), g.float(), forced=forced)
    assert_not_worse_than_reference(res.out.cpu(), y, y32, name)

    if pq["q"].dtype == torch.bfloat16 and summary["merge_differ"] == 0 and summary["append_rows_differ"] == 0:
        # every decision equals the reference's own: compare directly with what the reference produced
        # (after a legal tie-break difference the two memory trajectories are no longer comparable)
        assert_close_bf16(res.out.cpu(), fix["y_prefill"], f"{name} activations vs reference fixture")
        if True:
            for u, r in enumerate(recs, start=1):
                d = gh.decisions_from_route(res.route[:, u], B, spec.num_key_value_heads)
                if "append_idx" in r and 0 < r["append_idx"].size(-1) < spec.chunk_len:
                    assert torch.equal(d["append_idx"], r["append_idx"])
                if "best_idx" in r:
                    assert torch.equal(d["best_idx"], r["best_idx"])
            gh.compare_memory(res.memory, fix["state_prefill"], plan.final_state_len, name + " (fixture)")


def test_prefill_config1_shape_routing_exact():
    """Benchmark configuration 1 (B1 T4096 8x64 C128, 256 fixed means) in bf16 storage: every one of the
    28 x 8 x 128 merge decisions equals the oracle's own (no tie tolerance needed), activations and
    memory within the bf16 tolerance."""
    from tests.golden.make_golden import config1_inputs

    q, k, v, g = (t.to(torch.bfloat16) for t in config1_inputs())
    spec = ko.KvmSpec(8, 8, 64, 64, 32, 128, 2, 2, 1, "fixed", state_min_len=256)
    params, plan, res = gh.device_prefill(spec, q, k, v, g)
    y, st, trace = _oracle_following_device(spec, q, k, v, g, res, plan, 1)
    summary = gh.summarize(trace)
    gh.assert_routing_ok(summary)
    assert summary["merge_tokens"] == 28 * 8 * 128
    assert summary["merge_differ"] - summary["merge_differ_fp32"] <= 2, summary
    assert_close_bf16(res.out.cpu(), y, "config1 activations")
    gh.compare_memory(res.memory, st, 256, "config1")
    # per-slot counts of every update equal the oracle's histogram
    for u, rec in enumerate(trace, start=1):
        if rec.best_idx is None:
            continue
        if rec.merge_differ == 0:
            d = gh.decisions_from_route(res.route[:, u], 1, 8)
            assert torch.equal(ko.slot_histogram(d["best_idx"], rec.state_after),
                               ko.slot_histogram(rec.best_idx, rec.state_after))


@pytest.mark.parametrize("T", [1, 15, 16, 17, 33, 48, 49, 100])
def test_prefill_ragged_lengths(T):
    """Prompts shorter than a block, shorter than the window, and ragged ends."""
    torch.manual_seed(T)
    spec = ko.KvmSpec(4, 2, 32, 32, 16, 16, 2, 2, 1, "power_law", state_growth_factor=2.0, state_min_len=16)
    B = 2
    q = torch.randn(B, 4, T, 32).bfloat16()
    k = torch.randn(B, 2, T, 32).bfloat16()
    v = torch.randn(B, 2, T, 32).bfloat16()
    g = (1 + torch.nn.functional.elu(torch.randn(B, 2, T, 1))).bfloat16()
    params, plan, res = gh.device_prefill(spec, q, k, v, g)
    y, st, trace = _oracle_following_device(spec, q, k, v, g, res, plan, B)
    gh.assert_routing_ok(gh.summarize(trace))
    assert_close_bf16(res.out.cpu(), y, f"T={T}")
    gh.compare_memory(res.memory, st, plan.final_state_len, f"T={T}")


def test_prefill_strided_inputs_and_determinism():
    """Transposed [B,T,H,D] views are consumed without copies; two runs give identical bits."""
    torch.manual_seed(3)
    spec = ko.KvmSpec(4, 4, 128, 128, 64, 64, 2, 4, 1, "plus_one", state_min_len=64)
    B, T = 2, 64 * 9 + 20
    q = torch.randn(B, T, 4, 128).bfloat16().transpose(1, 2)
    k = torch.nn.functional.layer_norm(torch.randn(B, T, 4, 128), (128,)).bfloat16().transpose(1, 2)
    v = torch.randn(B, T, 4, 128).bfloat16().transpose(1, 2)
    g = (1 + torch.nn.functional.elu(torch.randn(B, T, 4, 1))).bfloat16().transpose(1, 2)
    _, plan, r1 = gh.device_prefill(spec, q, k, v, g)
    _, _, r2 = gh.device_prefill(spec, q, k, v, g)
    assert torch.equal(r1.out, r2.out) and torch.equal(r1.route, r2.route)
    assert torch.equal(r1.memory.k_sum, r2.memory.k_sum) and torch.equal(r1.memory.v_attn, r2.memory.v_attn)
    y, st, trace = _oracle_following_device(spec, q, k, v, g, r1, plan, B)
    gh.assert_routing_ok(gh.summarize(trace))
    assert_close_bf16(r1.out.cpu(), y, "strided")
    gh.compare_memory(r1.memory, st, plan.final_state_len, "strided")


def test_prefill_rejects_bad_arguments():
    spec = ko.KvmSpec(2, 2, 32, 32, 16, 16, 2, 2, 1, "fixed", state_min_len=16)
    q = torch.randn(1, 2, 40, 32).bfloat16()
    g = torch.ones(1, 2, 40, 1).bfloat16()
    with pytest.raises(Exception) as ei:
        gh.device_prefill(spec, q, q, q, g, memory_capacity=8)  # smaller than the memory the plan builds
    assert "capacity" in str(ei.value)
