"""Size-independent properties of the device path at the benchmark's full sequence length (T = 32768,
16 heads x 128, block 256, one new mean per block): the oracle needs minutes for these sizes, so the
checks are properties the algorithm guarantees at any size — determinism, causality (a prefix of the
prompt gives the prefix of the output, bit for bit), conservation of the routed tokens, convexity of the
attention output, and agreement of the decode path with the prefill path one token later."""

import pytest
import torch

from kvm_paper_b200 import ops
from oracle import kvm_oracle as ko
from tests.helpers import assert_close_bf16
from tests import gpu_helpers as gh

pytestmark = pytest.mark.gpu

H, D, C, T_FULL = 16, 128, 256, 32768


def _spec():
    return gh.bf16_spec(ko.KvmSpec(H, H, D, D, 64, C, 2, 4, 1, "plus_one", state_min_len=C))


def _inputs(B, T, seed):
    g = torch.Generator(device="cuda").manual_seed(seed)
    ln = torch.nn.functional.layer_norm
    q = ln(torch.randn(B, T, H, D, generator=g, device="cuda"), (D,)).bfloat16().transpose(1, 2)
    k = ln(torch.randn(B, T, H, D, generator=g, device="cuda"), (D,)).bfloat16().transpose(1, 2)
    v = torch.randn(B, T, H, D, generator=g, device="cuda").bfloat16().transpose(1, 2)
    gate = (1 + torch.nn.functional.elu(0.5 * torch.randn(B, T, H, 1, generator=g, device="cuda"))).bfloat16().transpose(1, 2)
    return q, k, v, gate


def _prefill(spec, q, k, v, gate, T=None, want_route=False):
    T = q.size(2) if T is None else T
    params = gh.layer_params(spec)
    plan = ops.build_prefill_plan(T, spec.chunk_len, spec.n_bswa_chunks, gh.desired_fn(spec))
    res = ops.prefill_forward(params, q[:, :, :T], k[:, :, :T], v[:, :, :T], gate[:, :, :T], plan, want_route=want_route,
                              check=True)
    torch.cuda.synchronize()
    return params, plan, res


def test_full_length_prefill_is_deterministic_and_causal():
    spec = _spec()
    q, k, v, gate = _inputs(1, T_FULL, seed=11)
    _, plan, a = _prefill(spec, q, k, v, gate)
    out_a, ks_a, vs_a = a.out.clone(), a.memory.k_sum.clone(), a.memory.v_sum.clone()
    _, _, b = _prefill(spec, q, k, v, gate)
    assert torch.equal(out_a, b.out) and torch.equal(ks_a, b.memory.k_sum) and torch.equal(vs_a, b.memory.v_sum)
    assert bool(torch.isfinite(out_a.float()).all())
    # a prefix of the prompt (whole blocks) gives exactly the prefix of the output: later tokens never reach back
    half = T_FULL // 2
    _, plan_h, c = _prefill(spec, q, k, v, gate, T=half)
    assert torch.equal(c.out, out_a[:, :half])
    # the schedule: one new mean per block once the window has filled
    assert plan.final_state_len == C + (T_FULL // C - spec.n_bswa_chunks - 1)
    assert plan_h.final_state_len == C + (half // C - spec.n_bswa_chunks - 1)


def test_full_length_routing_conserves_tokens_and_mass():
    """Every token of a consumed block is appended or merged exactly once, targets lie inside the memory
    and outside the sink rows, and the carried value sums hold the mass of all routed (gated) values."""
    spec = _spec()
    q, k, v, gate = _inputs(1, T_FULL, seed=12)
    _, plan, res = _prefill(spec, q, k, v, gate, want_route=True)
    route = res.route.cpu().long()  # [kv rows, n_updates + 1, C]
    n_upd = plan.n_updates
    S = C
    for u in range(1, n_upd + 1):
        r = route[:, u]
        appended = r < 0
        assert bool((appended.sum(-1) == 1).all()), f"update {u}: one append per block"
        rows = -(r[appended]) - 1
        assert bool((rows == S).all()), f"update {u}: the appended row is the next free row"
        S += 1
        merged = r[~appended]
        assert int(merged.min()) >= spec.sink_len and int(merged.max()) < S, f"update {u}: merge target outside [sink, S)"
    assert S == plan.final_state_len
    # mass: sum of the carried value sums == sum of the gated values of all consumed tokens (bf16 rounding per
    # scatter bounds the relative error of the per-row-dimension totals)
    n_tok = (n_upd + 1) * C
    vf, gf = v[0, :, :n_tok].float(), gate[0, :, :n_tok].float()
    gv = vf.clone()
    gv[:, C:] = (vf[:, C:] * gf[:, C:]).bfloat16().float()  # the initial block is stored ungated, appends ungated
    first_app = torch.zeros(H, n_tok, dtype=torch.bool)
    for u in range(1, n_upd + 1):
        first_app[:, u * C:(u + 1) * C] = route[:, u] < 0
    gv[first_app.cuda()] = vf[first_app.cuda()]
    want = gv.sum(1)  # [H, D]
    got = res.memory.v_sum[:, :S].float().sum(1)
    scale = gv.abs().sum(1)
    assert float(((got - want).abs() / scale).max()) < 2e-3


def test_full_length_attention_output_is_a_convex_combination():
    """Every output row is a convex combination of window values and memory values; a memory value row is
    a unit vector times the norm of the value it was appended with (merges never change that norm), so no
    output element can exceed the largest value norm of its head."""
    spec = _spec()
    q, k, v, gate = _inputs(1, T_FULL, seed=13)
    _, plan, res = _prefill(spec, q, k, v, gate)
    bound = v[0].float().norm(dim=-1).amax(1)                      # [H] largest value norm per head
    out = res.out[0].float().view(T_FULL, H, D)
    assert bool(torch.isfinite(out).all())
    assert bool((out.abs().amax(-1) <= bound.view(1, H) * (1 + 2.0 ** -6)).all())
    # and the output is not degenerate: rows differ along the sequence
    assert float(out.std()) > 1e-2


def test_decode_after_full_length_prefill_matches_prefill_of_one_more_token():
    """The decode path (ring + memory, persistent TMA kernel) and the prefill path (tcgen05 kernel) must
    agree on token T when the first T tokens are the same."""
    spec = _spec()
    T = T_FULL - C + 7   # inside a block, memory and window both long
    q, k, v, gate = _inputs(1, T + 1, seed=14)
    params, plan, res = _prefill(spec, q, k, v, gate, T=T)
    cache = ops.decode_cache_from_prefill(params, res, k[:, :, :T], v[:, :, :T], gate[:, :, :T], gh.desired_fn(spec))
    y_dec = cache.step(q[:, :, T:T + 1], k[:, :, T:T + 1], v[:, :, T:T + 1], gate[:, :, T:T + 1]).clone()
    _, _, full = _prefill(spec, q, k, v, gate, T=T + 1)
    assert_close_bf16(y_dec.cpu(), full.out[:, T:T + 1].cpu(), "decode vs prefill at token T")
