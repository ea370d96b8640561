"""The drop-in class on the GPU: ``SequenceMixer.forward_inference`` with a carried-state cache, prefill then
single-token steps, as ``Block.forward_attn`` of the reference drives it (model/rwkv7_backbone.py:219-227,
model/kvm_mixer.py:527-570), compared with what the reference itself produced for the same weights and
inputs (the golden fixtures: pre-``c_proj`` activations of the prefill and of every decode step, final
carried state)."""

import pytest
import torch

from kvm_paper_b200 import ops
from kvm_paper_b200.mixer import SequenceMixer, StatesCache
from tests.helpers import assert_close_bf16, load_fixture, max_abs, mean_rel, mixer_from_fixture, rotary_tables

pytestmark = pytest.mark.gpu

BF16_FIXTURES = ["powerlaw_bf16", "plusone_bf16", "saturation_bf16"]


def _drive(m, cfg, fix, cache, n_decode):
    T, B = fix["case"]["T"], fix["case"]["B"]
    x, vf = fix["x"].cuda(), None if fix["v_first"] is None else fix["v_first"].cuda()
    cut = lambda t, a, b: None if t is None else t[:, a:b]  # noqa: E731
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
    cache = StatesCache()
    y_prefill, y_decode = _drive(m, cfg, fix, cache, n_decode)
    assert y_prefill.shape == fix["y_prefill"].shape
    print(f"{name}: prefill max-abs {max_abs(y_prefill.cpu(), fix['y_prefill']):.3e} mean-rel {mean_rel(y_prefill.cpu(), fix['y_prefill']):.3e}; "
          f"decode max-abs {max_abs(y_decode.cpu(), fix['y_decode']):.3e} mean-rel {mean_rel(y_decode.cpu(), fix['y_decode']):.3e}")
    assert_close_bf16(y_prefill.cpu(), fix["y_prefill"], f"{name} forward_inference prefill")
    assert_close_bf16(y_decode.cpu(), fix["y_decode"], f"{name} forward_inference decode")
    # the carried state in the reference's eager layout
    T = fix["case"]["T"]
    assert cache.get_seq_length(m.layer_idx) == T + n_decode
    dc = cache.get_states(m.layer_idx)[SequenceMixer._CACHE_DECODE]
    assert isinstance(dc, ops.KvmDecodeCache) and dc.owner is m
    sd, want = dc.logical_state_dict(), fix["state_final"]
    assert sd["kvm_state_coverage_len"] == want["kvm_state_coverage_len"] and sd["kvm_bswa_begin"] == want["kvm_bswa_begin"]
    assert sd["kvm_s_k"].shape == want["kvm_s_k"].shape
    scale_k = max(1.0, float(want["kvm_s_k"].float().abs().max()))
    scale_v = max(1.0, float(want["kvm_s_v"].float().abs().max()))
    assert_close_bf16(sd["kvm_s_k"].cpu(), want["kvm_s_k"], f"{name} kvm_s_k", max_abs_tol=2e-2 * scale_k)
    assert_close_bf16(sd["kvm_s_v"].cpu(), want["kvm_s_v"], f"{name} kvm_s_v", max_abs_tol=2e-2 * scale_v)
    assert torch.allclose(sd["kvm_s_vlen"].cpu(), want["kvm_s_vlen"].float(), rtol=1e-5, atol=1e-6)
    for key in ("kvm_bswa_k", "kvm_bswa_v", "kvm_bswa_merge_gate"):
        assert torch.equal(sd[key].cpu(), want[key]), key
    # the token-shift / value-residual carry-overs of the prologue live in the same cache entry
    for key in ("att_q_final_token", "att_k_final_token", "att_v_final_token", "att_x_final_token"):
        assert key in cache.get_states(m.layer_idx)


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
