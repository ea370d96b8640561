"""The CPU oracle reproduces what the reference itself computed (fixtures made by
tests/golden/make_golden.py): integer decisions and carried memory exactly, attention outputs to
within the CPU attention kernel's thread-partition noise."""

import pytest
import torch

from oracle import kvm_oracle as ko
from tests.helpers import SMALL_FIXTURES, load_fixture, spec_from_fixture, max_abs


def _check_updates(trace, records):
    assert len(trace) == len(records)
    for got, want in zip(trace, records):
        assert got.ctx_len == want["ctx_len"] and got.available_context == want["available_context"]
        assert got.state_before == want["state_before"] and got.state_after == want["state_after"]
        if "append_idx" in want:
            assert torch.equal(got.append_idx, want["append_idx"])
            assert torch.equal(got.merge_idx, want["merge_idx"])
        if "best_idx" in want:
            assert torch.equal(got.best_idx, want["best_idx"])


def _check_state(got, want, exact=True):
    for key, val in want.items():
        if isinstance(val, torch.Tensor):
            assert got[key].shape == val.shape, key
            assert torch.equal(got[key], val), f"{key}: max-abs {max_abs(got[key], val)}"
        else:
            assert got[key] == val, key


@pytest.mark.parametrize("name", SMALL_FIXTURES)
def test_oracle_matches_reference_fixture(name):
    fix = load_fixture(name)
    spec = spec_from_fixture(fix)
    pq = fix["post_qkv"]
    tol = 2e-6 if pq["q"].dtype == torch.float32 else 1.6e-2  # bf16: at most one rounding step of O(1) values
    trace = []
    with torch.no_grad():
        y, state = ko.prefill(spec, pq["q"], pq["k"], pq["v"], pq["merge_gate"], trace=trace)
        assert y.shape == fix["y_prefill"].shape
        assert max_abs(y, fix["y_prefill"]) <= tol
        assert (y == fix["y_prefill"]).float().mean() > 0.99
        _check_updates(trace, fix["updates"][: fix["n_prefill_updates"]])
        _check_state(state, fix["state_prefill"])
        if fix["decode_qkv"] is not None:
            dq, dk, dv, dg = fix["decode_qkv"]
            ys = []
            dtrace = []
            for i in range(dq.size(2)):
                yi, state = ko.decode_step(spec, dq[:, :, i:i + 1], dk[:, :, i:i + 1], dv[:, :, i:i + 1],
                                           dg[:, :, i:i + 1], state, trace=dtrace)
                ys.append(yi)
            yd = torch.cat(ys, dim=1)
            assert max_abs(yd, fix["y_decode"]) <= tol
            _check_updates(dtrace, fix["updates"][fix["n_prefill_updates"]:])
            _check_state(state, fix["state_final"])


def test_oracle_matches_reference_config1():
    """Configuration 1 of the benchmark (fp32, B1 T4096, 8x64, C=128, 256 means): routing of all
    28 merge blocks exact, activations and memory equal on the stored samples."""
    from tests.golden.make_golden import config1_inputs

    fix = load_fixture("config1_fp32")
    q, k, v, g = config1_inputs()
    spec = ko.KvmSpec(8, 8, 64, 64, 32, 128, 2, 2, 1, "fixed", state_min_len=256)
    trace = []
    with torch.no_grad():
        y, st = ko.prefill(spec, q, k, v, g, trace=trace)
    assert len(trace) == fix["n_updates"]
    assert [r.state_before for r in trace] == fix["state_before"]
    assert [r.state_after for r in trace] == fix["state_after"]
    best = torch.stack([r.best_idx for r in trace if r.best_idx is not None], 0)
    assert torch.equal(best.to(torch.int16), fix["best_idx"])
    assert max_abs(y[:, ::7, ::5], fix["y_sample"]) <= 2e-6
    assert torch.equal(st["kvm_s_k"][:, :, ::3, ::2], fix["s_k_sample"])
    assert torch.equal(st["kvm_s_v"][:, :, ::3, ::2], fix["s_v_sample"])
    assert torch.equal(st["kvm_s_vlen"], fix["s_vlen"])
    assert st["kvm_state_coverage_len"] == fix["coverage"] and st["kvm_bswa_begin"] == fix["bswa_begin"]


def test_oracle_prefill_then_decode_equals_longer_prefill():
    """prefill(T) followed by n decode steps walks the same memory trajectory as prefill(T+n)."""
    torch.manual_seed(5)
    spec = ko.KvmSpec(2, 2, 32, 32, 16, 16, 2, 4, 1, "power_law", state_growth_factor=3.0, state_min_len=16)
    B, T, n = 1, 70, 45
    q = torch.randn(B, 2, T + n, 32)
    k = torch.randn(B, 2, T + n, 32)
    v = torch.randn(B, 2, T + n, 32)
    g = 1 + torch.nn.functional.elu(torch.randn(B, 2, T + n, 1))
    with torch.no_grad():
        y_full, st_full = ko.prefill(spec, q, k, v, g)
        y, st = ko.prefill(spec, q[:, :, :T], k[:, :, :T], v[:, :, :T], g[:, :, :T])
        for i in range(T, T + n):
            yi, st = ko.decode_step(spec, q[:, :, i:i + 1], k[:, :, i:i + 1], v[:, :, i:i + 1], g[:, :, i:i + 1], st)
            assert max_abs(yi, y_full[:, i:i + 1]) < 1e-5
    assert max_abs(st["kvm_s_k"], st_full["kvm_s_k"]) < 1e-4
    assert st["kvm_s_k"].shape == st_full["kvm_s_k"].shape


def _projections(m, x, vf):
    """The reference's projections and pre-shift value residual (plain GEMMs and elementwise ops on the CPU)."""
    q, k, v = m.c_q(x), m.c_k(x), m.c_v(x)
    if m.value_residual_mode == "linear":
        v = (1 - m.lamb) * v + m.lamb * vf.view_as(v)
    elif m.value_residual_mode == "rwkv":
        v = v + (vf.to(v.dtype) - v) * m._value_gate(x).to(v.dtype)
    gated = m.config.kvm_use_merge_gate_keys or m.config.kvm_use_merge_gate_values
    return q, k, v, (m.key_weighting(x) if gated else None)


@pytest.mark.parametrize("name", SMALL_FIXTURES)
def test_oracle_prologue_matches_reference_fixture(name):
    """``oracle.prologue`` on the projections of the fixture's hidden inputs gives the post-QKV tensors the reference
    recorded, bit for bit, for the prompt and for cached single-token calls."""
    from tests.helpers import mixer_from_fixture, rotary_tables
    fix = load_fixture(name)
    cfg, m = mixer_from_fixture(fix)
    if m.value_residual_mode == "rwkv_post_tokenshift":
        pytest.skip("post-shift value residual: not part of the fused prologue")
    T, B = fix["case"]["T"], fix["case"]["B"]
    x, vf = fix["x"], fix["v_first"]
    shift = (m.x_q, m.x_k, m.x_v) if m.tokenshift_mode == "rwkv" else None
    has_ln = isinstance(m.ln_q, torch.nn.LayerNorm)
    kw = dict(n_q_heads=m.num_attention_heads, n_kv_heads=m.num_key_value_heads, shift=shift,
              ln_q=(m.ln_q.weight, m.ln_q.bias) if has_ln else None, ln_k=(m.ln_k.weight, m.ln_k.bias) if has_ln else None,
              ln_eps=m.ln_q.eps if has_ln else 1e-5)
    with torch.no_grad():
        lin = _projections(m, x[:, :T], None if vf is None else vf[:, :T])
        pos = torch.arange(T).view(1, T).expand(B, T)
        got = ko.prologue(*lin, position_embeddings=rotary_tables(cfg, m.d_qk_head, pos), **kw)
        pq = fix["post_qkv"]
        for g, w in zip(got, (pq["q"], pq["k"], pq["v"], pq["merge_gate"])):
            assert g.shape == w.shape and torch.equal(g, w)
        if fix["decode_qkv"] is not None:
            dq, dk, dv, dg = fix["decode_qkv"]
            prev = tuple(t[:, -1:] for t in lin[:3])
            for i in range(min(5, dq.size(2))):
                lin = _projections(m, x[:, T + i:T + i + 1], None if vf is None else vf[:, T + i:T + i + 1])
                pos = torch.full((B, 1), T + i, dtype=torch.long)
                got = ko.prologue(*lin, position_embeddings=rotary_tables(cfg, m.d_qk_head, pos), prev=prev, **kw)
                for g, w in zip(got, (dq, dk, dv, dg)):
                    assert torch.equal(g, w[:, :, i:i + 1])
                prev = tuple(lin[:3])
