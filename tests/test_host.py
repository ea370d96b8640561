"""Host-side logic on the CPU: schedule tables, the PyTorch prologue of the drop-in mixer against
what the reference computed, the C-ABI library's exports and the error conventions."""

import ctypes
import os
import re
import types

import pytest
import torch

from kvm_paper_b200 import _lib, ops
from kvm_paper_b200.mixer import SequenceMixer, StatesCache
from oracle import kvm_oracle as ko
from tests.helpers import SMALL_FIXTURES, load_fixture, spec_from_fixture
from tests.helpers import config_from_fixture as _config_from_fixture, mixer_from_fixture as _mixer_from_fixture, rotary_tables as _rotary

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.mark.parametrize("name", SMALL_FIXTURES)
def test_prologue_matches_reference(name):
    """forward_prefix (projections, token shift, value residual, LayerNorm, RoPE, gate) reproduces the
    post-QKV tensors the reference produced, for the prefill and for cached single-token steps."""
    fix = load_fixture(name)
    cfg, m = _mixer_from_fixture(fix)
    T = fix["case"]["T"]
    B = fix["case"]["B"]
    x, vf = fix["x"], fix["v_first"]
    cache = StatesCache()
    with torch.no_grad():
        pos = torch.arange(T).view(1, T).expand(B, T)
        q, k, v, g = m.forward_prefix(x[:, :T], None if vf is None else vf[:, :T], _rotary(cfg, m.d_qk_head, pos), None, cache)
        pq = fix["post_qkv"]
        for got, want in ((q, pq["q"]), (k, pq["k"]), (v, pq["v"]), (g, pq["merge_gate"])):
            assert got.shape == want.shape and torch.equal(got, want)
        cache.update(1, offset=T)
        if fix["decode_qkv"] is not None:
            dq, dk, dv, dg = fix["decode_qkv"]
            for i in range(min(5, dq.size(2))):
                pos = torch.full((B, 1), T + i, dtype=torch.long)
                q, k, v, g = m.forward_prefix(x[:, T + i:T + i + 1], None if vf is None else vf[:, T + i:T + i + 1],
                                              _rotary(cfg, m.d_qk_head, pos), None, cache)
                cache.update(1, offset=1)
                assert torch.equal(q, dq[:, :, i:i + 1]) and torch.equal(k, dk[:, :, i:i + 1])
                assert torch.equal(v, dv[:, :, i:i + 1]) and torch.equal(g, dg[:, :, i:i + 1])


@pytest.mark.parametrize("name", SMALL_FIXTURES)
def test_prefill_plan_matches_reference_trace(name):
    fix = load_fixture(name)
    cfg, m = _mixer_from_fixture(fix)
    plan = m.make_prefill_plan(fix["case"]["T"])
    recs = fix["updates"][: fix["n_prefill_updates"]]
    assert plan.n_updates == len(recs)
    for u, r in enumerate(recs, start=1):
        assert plan.state_before[u] == r["state_before"]
        assert plan.state_before[u] + plan.n_append[u] == r["state_after"]
        assert (u + cfg.n_bswa_chunks) * cfg.chunk_len == r["ctx_len"] and (u + 1) * cfg.chunk_len == r["available_context"]
    st = fix["state_prefill"]
    assert plan.final_state_len == st["kvm_s_k"].size(2)
    assert plan.final_coverage == st["kvm_state_coverage_len"] and plan.bswa_begin == st["kvm_bswa_begin"]


@pytest.mark.parametrize("mode", ["fixed", "power_law", "kvm_saturation"])
def test_schedule_methods_equal_oracle(mode):
    cfg = types.SimpleNamespace(**vars(_config_from_fixture(load_fixture("powerlaw_bf16"))))
    cfg.state_budget_mode = mode
    cfg.state_saturation_n = 777
    cfg.state_growth_factor, cfg.state_round_down, cfg.state_min_len, cfg.n_max_d_chunks = 16.0, 8, 32, 40
    m = SequenceMixer(cfg, 0)
    spec = ko.KvmSpec(2, 2, 64, 64, 32, cfg.chunk_len, cfg.n_bswa_chunks, cfg.n_max_d_chunks, 1, mode,
                      state_growth_factor=16.0, state_round_down=8, state_min_len=32, state_saturation_n=777)
    for ctx in list(range(0, 3000, 37)) + [65536, 262144]:
        for cur in (0, 32, 500):
            assert m._desired_state_len(ctx, ctx - 64, cur) == ko.desired_state_len(spec, ctx, ctx - 64, cur)
    for total in range(0, 400):
        assert m._bswa_begin_for_total_len(total) == ko.bswa_begin_for_total_len(spec, total)


def test_decode_host_bookkeeping_follows_oracle_lengths():
    """The host mirror of the ragged decode cache (who updates when, how many rows) agrees with the
    oracle's per-sequence walk; no device needed."""
    spec = ko.KvmSpec(2, 2, 32, 32, 16, 16, 2, 6, 1, "power_law", state_growth_factor=3.0, state_min_len=16)
    fake = ops.KvmDecodeCache.__new__(ops.KvmDecodeCache)
    import numpy as np
    lens = [3, 16, 31, 32, 48, 100]
    fake.cfg = ops.LayerConfig(2, 2, 32, 16, 2, 16, 1)
    fake.batch = len(lens)
    fake.desired_state_len = lambda c, a, s: ko.desired_state_len(spec, c, a, s)
    fake.update_count = 0
    fake.total_len_h = np.array(lens, dtype=np.int64)
    states = []
    for T in lens:
        plan = ops.build_prefill_plan(T, 16, 2, fake.desired_state_len)
        states.append(dict(S=plan.final_state_len, total=T))
    fake.state_len_h = np.array([s["S"] for s in states], dtype=np.int64)
    for step in range(80):
        n_app, max_rows = fake._plan_step()
        for b, st in enumerate(states):
            past = st["total"]
            total = past + 1
            nb = ko.bswa_begin_for_total_len(spec, total)
            cov_old = max(min(past, 16), ko.bswa_begin_for_total_len(spec, past))
            cov_new = max(min(total, 16), nb)
            expect = -1
            if cov_old < min(total, 16):
                st["S"] += 1
            elif cov_new > cov_old:
                des = ko.desired_state_len(spec, 32 + cov_old, cov_old + 16, st["S"])
                expect = min(max(des - st["S"], 0), 16)
                st["S"] += expect
            st["total"] = total
            got = -1 if n_app is None else int(n_app[b])
            assert got == expect, (step, b, got, expect)
            assert fake.state_len_h[b] == st["S"] and fake.total_len_h[b] == total
        rows = [(st["S"] if ko.bswa_begin_for_total_len(spec, st["total"]) > 0 else 0) + st["total"] - ko.bswa_begin_for_total_len(spec, st["total"]) for st in states]
        assert max_rows == max(rows)


def test_library_exports_every_declared_symbol():
    header = open(os.path.join(ROOT, "include", "kvm_b200.h")).read()
    declared = set(re.findall(r"^(?:int|size_t|const char\*)\s+(kvm_[a-z_0-9]+)\s*\(", header, flags=re.M))
    assert declared, "no entry points parsed from the header"
    lib = _lib.load()
    for name in sorted(declared):
        assert hasattr(lib, name), f"{name} is declared in include/kvm_b200.h but not exported"
    assert set(_lib.EXPORTS) <= declared
    assert lib.kvm_abi_version() >= 100


def test_abi_argument_errors_are_reported_without_a_device():
    lib = _lib.load()
    layer = _lib.KvmLayer(4, 3, 64, 32, 2, 32, 1, 1, 1, 0, 0, 1e-5, 8, 8, 8, 8)
    mem = _lib.KvmMemory(8, 8, 8, 8, 8, 16)
    t4 = _lib.KvmTensor4(16, 8, 8, 8)
    rc = lib.kvm_prefill_forward(ctypes.byref(layer), 1, 64, t4, t4, t4, t4, 8, (_lib.KvmUpdatePlan * 1)(), 0, 0, mem,
                                 16, None, 256, 0, 3, None)
    assert rc == 1 and b"n_q_heads" in lib.kvm_last_error_string()
    layer.n_kv_heads = 2
    layer.head_dim = 48
    rc = lib.kvm_decode_step(ctypes.byref(layer), 1, _lib.KvmDecodeCache(mem, 8, 8, 8, 8, 8), t4, t4, t4, t4, None, 0, 16,
                             16, None, 256, 1024, None)
    assert rc == 5 and b"head_dim" in lib.kvm_last_error_string()
    with pytest.raises(ValueError):
        _lib.check(rc)
    layer.head_dim = 64
    plan = (_lib.KvmUpdatePlan * 1)(_lib.KvmUpdatePlan(0, 32, -1, 0))
    mem.capacity = 8  # the initial memory alone needs 32 rows
    rc = lib.kvm_prefill_forward(ctypes.byref(layer), 1, 40, t4, t4, t4, t4, 8, plan, 0, 0, mem, 16, None, 256, 1 << 20, 3, None)
    assert rc == 2 and b"capacity" in lib.kvm_last_error_string()
    with pytest.raises(_lib.KvmError):
        _lib.check(rc)
    # the self-gathering prefill: rank count, rank, buffer addresses and kernel shape are checked before anything else
    bases = (ctypes.c_void_p * 2)(4096, 8192)
    args = (ctypes.byref(layer), 1, 40, t4, t4, t4, t4, 8, plan, 0, 0, mem)
    tail = (None, 256, 1 << 20, 3, None)
    assert lib.kvm_prefill_forward_gathered(*args, 1, 0, bases, *tail) == 1 and b"n_ranks" in lib.kvm_last_error_string()
    assert lib.kvm_prefill_forward_gathered(*args, 2, 2, bases, *tail) == 1
    bad = (ctypes.c_void_p * 2)(4096, 8200)
    assert lib.kvm_prefill_forward_gathered(*args, 2, 0, bad, *tail) == 1 and b"aligned" in lib.kvm_last_error_string()
    assert lib.kvm_prefill_forward_gathered(*args, 2, 0, bases, *tail) == 5 and b"head_dim 128" in lib.kvm_last_error_string()
    # the prologue: token-shift scales for all of q, k, v or for none
    pro = _lib.KvmPrologue()
    pro.q_lin = pro.k_lin = pro.v_lin = 4096
    pro.shift_q = 4096
    rc = lib.kvm_prologue_forward(ctypes.byref(layer), 1, 40, ctypes.byref(pro), 4096, 4096, 4096, 4096, 0, None, 0, None)
    assert rc == 1 and b"token-shift" in lib.kvm_last_error_string()


def test_mixer_error_conventions():
    fix = load_fixture("powerlaw_bf16")
    cfg, m = _mixer_from_fixture(fix)
    pq = fix["post_qkv"]
    with pytest.raises(ValueError):
        m.forward_prefill(pq["q"], pq["k"], pq["v"], pq["merge_gate"], None, None, torch.ones(1), None)
    with pytest.raises(RuntimeError):  # no CPU path
        m.forward_prefill(pq["q"], pq["k"], pq["v"], pq["merge_gate"], None, None, None, None)
    with pytest.raises(AssertionError):
        m.forward_single(pq["q"][:, :, :2], pq["k"][:, :, :2], pq["v"][:, :, :2], pq["merge_gate"][:, :, :2], None, None, None, StatesCache())
    with pytest.raises(ValueError):
        m.forward_single(pq["q"][:, :, :1], pq["k"][:, :, :1], pq["v"][:, :, :1], pq["merge_gate"][:, :, :1], None, None, None, None)
    bad = types.SimpleNamespace(**vars(cfg))
    bad.kvm_use_vlens = 0
    with pytest.raises(ValueError):
        SequenceMixer(bad, 0)
    bad = types.SimpleNamespace(**vars(cfg))
    bad.state_budget_mode = "nope"
    with pytest.raises(ValueError):
        SequenceMixer(bad, 0)._desired_state_len(100, 100, 0)
    # every parameter carries the optimizer label the reference's trainer asserts on
    assert all(getattr(p, "label", None) for p in m.parameters())
