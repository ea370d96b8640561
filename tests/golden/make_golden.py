"""Generate the golden fixtures in this directory by running the reference itself on the CPU.

Usage (only where the reference checkout is available; it is not needed to run the tests):

    python tests/golden/make_golden.py --reference /path/to/KVM-paper

For every case the script builds the reference's eager mixer
(``model.kvm_fp32_routing_reference.SequenceMixer`` unless the case says ``golden``), runs
``forward_inference`` (prefill, then single-token decode steps) with a ``StatesDictCache`` and stores:

  * the mixer's parameters and the hidden input ``x`` (small cases), or the seeds that regenerate
    them (large case),
  * the post-QKV tensors q, k, v, merge_gate that the prologue produced,
  * the pre-``c_proj`` activations of the prefill and of every decode step,
  * the carried state after prefill and after the last decode step,
  * per memory update: append indices, merge indices, the routed slot of every merged token and the
    fp32 top-2 logit margin.

The fixtures pin (a) the CPU oracle in ``oracle/kvm_oracle.py`` and (b) the host-side prologue of
the drop-in mixer; the CUDA kernels are then compared with the oracle and with these fixtures.
"""

from __future__ import annotations

import argparse
import os
import sys

import torch

HERE = os.path.dirname(os.path.abspath(__file__))


def _cases():
    base = dict(
        vocab_size=64,
        num_hidden_layers=2,
        use_tokenshift_att=1,
        use_value_residual=1,
        sink_len=1,
        n_bswa_chunks=2,
        state_round_down=1,
        param_dtype=None,
    )
    return {
        # fp32, GQA, fixed memory, ragged T, decode across two block boundaries
        "fixed_gqa_fp32": dict(
            cfg=dict(base, hidden_size=64, num_attention_heads=4, num_key_value_heads=2, d_head=32,
                     rope_partial_dim=16, chunk_len=16, n_max_d_chunks=2, state_budget_mode="fixed",
                     state_min_len=32),
            dtype="float32", B=2, T=110, n_decode=40, seed=11),
        # bf16, power-law growth, appends ranked by novelty
        "powerlaw_bf16": dict(
            cfg=dict(base, hidden_size=128, num_attention_heads=2, d_head=64, rope_partial_dim=32,
                     chunk_len=32, n_max_d_chunks=8, state_budget_mode="power_law",
                     state_growth_factor=4.0, state_growth_exponent=0.5, state_min_len=32),
            dtype="bfloat16", B=1, T=400, n_decode=70, seed=12),
        # bf16, one new mean per block (benchmark schedule), gates applied to appends, 2 sinks
        "plusone_bf16": dict(
            cfg=dict(base, hidden_size=128, num_attention_heads=2, d_head=64, rope_partial_dim=32,
                     chunk_len=32, n_max_d_chunks=4, state_budget_mode="fixed", state_min_len=32,
                     sink_len=2, kvm_apply_merge_gate_to_appends=1),
            plus_one=True, dtype="bfloat16", B=1, T=230, n_decode=40, seed=13),
        # prompt shorter than one block, decode grows the direct memory and crosses W*C
        "short_prompt_fp32": dict(
            cfg=dict(base, hidden_size=64, num_attention_heads=2, d_head=32, rope_partial_dim=32,
                     chunk_len=16, n_max_d_chunks=1, state_budget_mode="fixed", state_min_len=16,
                     kvm_apply_merge_gate_to_initial_state=0, sink_len=0),
            dtype="float32", B=1, T=5, n_decode=60, seed=14),
        # saturation schedule, head_dim 128 with partial rope, no value residual / token shift
        "saturation_bf16": dict(
            cfg=dict(base, hidden_size=256, num_attention_heads=2, d_head=128, rope_partial_dim=64,
                     chunk_len=32, n_max_d_chunks=4, state_budget_mode="kvm_saturation",
                     state_saturation_n=96, state_min_len=32, use_tokenshift_att=0, use_value_residual=0),
            dtype="bfloat16", B=1, T=200, n_decode=10, seed=15),
    }


def _build(ref_root, case):
    from model.rwkv7_backbone import MixerConfig, RotaryEmbedding
    from model.kvm_fp32_routing_reference import SequenceMixer as Fp32Mixer

    dtype = getattr(torch, case["dtype"])
    cfg = MixerConfig(**case["cfg"])
    torch.manual_seed(case["seed"])
    old = torch.get_default_dtype()
    torch.set_default_dtype(dtype)
    try:
        mixer = Fp32Mixer(cfg, 1)
    finally:
        torch.set_default_dtype(old)
    g = torch.Generator().manual_seed(case["seed"] + 1000)
    with torch.no_grad():
        # the repository initialises these to neutral values; perturb them so every term is exercised
        mixer.ln_s_k.weight.copy_((1.0 + 0.1 * torch.randn(mixer.ln_s_k.weight.shape, generator=g)).to(dtype))
        mixer.ln_s_k.bias.copy_((0.05 * torch.randn(mixer.ln_s_k.bias.shape, generator=g)).to(dtype))
        mixer.front_head_temp.copy_((1.0 + 0.2 * torch.rand(mixer.front_head_temp.shape, generator=g)).to(dtype))
        mixer.state_head_temp.copy_((1.0 + 0.2 * torch.rand(mixer.state_head_temp.shape, generator=g)).to(dtype))
        mixer.key_weighting.weight.copy_((0.2 * torch.randn(mixer.key_weighting.weight.shape, generator=g)).to(dtype))
        if hasattr(mixer, "v_gate1"):
            mixer.v_gate1.weight.copy_((0.05 * torch.randn(mixer.v_gate1.weight.shape, generator=g)).to(dtype))
    mixer.c_proj = torch.nn.Identity()  # compare the pre-projection activations
    mixer.eval()
    if case.get("plus_one"):
        def _plus_one(ctx_len, available_context, current_state_len, _m=mixer):
            cur = max(int(current_state_len), 0)
            return max(min(cur + 1, max(int(available_context), 0), _m.max_state_len), cur)
        mixer._desired_state_len = _plus_one
    rotary = RotaryEmbedding(mixer.d_qk_head, cfg.rope_partial_dim, cfg.rope_theta)
    return cfg, mixer, rotary, g


def _trace_hooks(mixer, records):
    """Record routing decisions by wrapping the two decision functions of the reference."""
    import model.kvm_mixer as km

    orig_split = km._split_append_merge_idx_by_maxsim
    orig_merge = mixer._merge_into_state
    orig_update = mixer._update_state_from_overflow_tokens
    cur = {}

    def split(k_block, n_append, k_ref):
        a, m = orig_split(k_block, n_append, k_ref)
        cur["append_idx"], cur["merge_idx"] = a.clone(), m.clone()
        return a, m

    def merge(k_merge, v_merge, s_k, s_v, s_vlen, protected_slots):
        s_k_norm = mixer.ln_s_k(s_k)
        logits = torch.matmul(k_merge.float(), s_k_norm.float().transpose(-1, -2))
        logits[..., :protected_slots] = float("-inf")
        cur["best_idx"] = logits.max(dim=-1).indices.clone()
        if logits.size(-1) >= 2:
            t2 = logits.topk(2, dim=-1).values
            cur["margin"] = (t2[..., 0] - t2[..., 1]).clone()
        return orig_merge(k_merge, v_merge, s_k, s_v, s_vlen, protected_slots)

    def update(s_k, s_v, s_vlen, overflow_k, overflow_v, merge_gate, ctx_len, available_context):
        cur.clear()
        before = int(s_k.size(2))
        out = orig_update(s_k, s_v, s_vlen, overflow_k=overflow_k, overflow_v=overflow_v,
                          merge_gate=merge_gate, ctx_len=ctx_len, available_context=available_context)
        rec = dict(ctx_len=int(ctx_len), available_context=int(available_context), state_before=before,
                   state_after=int(out[0].size(2)))
        rec.update({k: v for k, v in cur.items()})
        records.append(rec)
        return out

    km._split_append_merge_idx_by_maxsim = split
    mixer._merge_into_state = merge
    mixer._update_state_from_overflow_tokens = update

    def undo():
        km._split_append_merge_idx_by_maxsim = orig_split

    return undo


def _state_of(cache, layer_idx):
    st = cache.get_states(layer_idx)
    out = {}
    for key, val in st.items():
        if key.startswith("kvm_"):
            out[key] = val.clone() if isinstance(val, torch.Tensor) else val
    out["total_len"] = cache.get_seq_length(layer_idx)
    return out


def run_case(ref_root, name, case):
    from model.statesdictcache import StatesDictCache

    cfg, mixer, rotary, g = _build(ref_root, case)
    dtype = getattr(torch, case["dtype"])
    B, T, n_dec = case["B"], case["T"], case["n_decode"]
    x_all = torch.randn(B, T + n_dec, cfg.hidden_size, generator=g).to(dtype)
    v_first_all = torch.randn(B, T + n_dec, mixer.value_projection_size, generator=g).to(dtype)
    use_vf = mixer.value_residual_mode != "none"

    records: list = []
    undo = _trace_hooks(mixer, records)
    cache = StatesDictCache()
    post_qkv = {}
    orig_prefill = mixer.forward_prefill

    def cap_prefill(q, k, v, merge_gate, *a, **kw):
        post_qkv.update(q=q.clone(), k=k.clone(), v=v.clone(), merge_gate=merge_gate.clone())
        return orig_prefill(q, k, v, merge_gate, *a, **kw)

    mixer.forward_prefill = cap_prefill
    dec_qkv = []
    orig_single = mixer.forward_single

    def cap_single(q, k, v, merge_gate, *a, **kw):
        dec_qkv.append((q.clone(), k.clone(), v.clone(), merge_gate.clone()))
        return orig_single(q, k, v, merge_gate, *a, **kw)

    mixer.forward_single = cap_single
    with torch.no_grad():
        pos = torch.arange(T).view(1, T).expand(B, T)
        y_prefill = mixer.forward_inference(
            x_all[:, :T], v_first_all[:, :T] if use_vf else None, rotary(pos), None, cache)
        n_prefill_updates = len(records)
        state_prefill = _state_of(cache, mixer.layer_idx)
        y_dec = []
        for i in range(n_dec):
            pos = torch.full((B, 1), T + i, dtype=torch.long)
            y_dec.append(mixer.forward_inference(
                x_all[:, T + i:T + i + 1], v_first_all[:, T + i:T + i + 1] if use_vf else None,
                rotary(pos), None, cache))
        state_final = _state_of(cache, mixer.layer_idx)
    undo()

    sd = {k: v.clone() for k, v in mixer.state_dict().items()}
    fix = dict(
        name=name, case={k: v for k, v in case.items()}, state_dict=sd, x=x_all, v_first=v_first_all if use_vf else None,
        post_qkv=post_qkv,
        decode_qkv=tuple(torch.cat([d[i] for d in dec_qkv], dim=2) for i in range(4)) if dec_qkv else None,
        y_prefill=y_prefill, y_decode=torch.cat(y_dec, dim=1) if y_dec else None,
        state_prefill=state_prefill, state_final=state_final,
        updates=records, n_prefill_updates=n_prefill_updates,
        torch_version=str(torch.__version__),
    )
    path = os.path.join(HERE, f"{name}.pt")
    torch.save(fix, path)
    n_app = sum(1 for r in records if "append_idx" in r)
    print(f"{name}: T={T} updates={len(records)} (prefill {n_prefill_updates}, with ranked appends {n_app}) "
          f"final S={state_final['kvm_s_k'].size(2)} -> {os.path.getsize(path) / 1024:.0f} KiB")


def run_config1(ref_root):
    """BASELINE configuration 1: one layer, fp32, B1 T4096 d512 8x64, C=128, fixed 256 means, seed 0.

    ``rope_partial_dim`` is 32: with the repository default of 64 every dimension of a 64-wide head is
    rotary, the prepared keys are all equal to the LayerNorm bias and routing is degenerate.
    Tensors are too large to commit; the fixture stores the routing decisions (exact integers), the
    minimum top-2 margin and strided samples of the activations and of the carried state.  The
    post-QKV inputs are regenerated on the test side from the same seeds with plain torch calls."""
    from model.rwkv7_backbone import MixerConfig
    from model.kvm_fp32_routing_reference import SequenceMixer as Fp32Mixer

    cfg = MixerConfig(vocab_size=64, num_hidden_layers=1, hidden_size=512, num_attention_heads=8, d_head=64,
                      rope_partial_dim=32, chunk_len=128, n_bswa_chunks=2, n_max_d_chunks=2,
                      state_budget_mode="fixed", state_min_len=256, sink_len=1, param_dtype=None)
    torch.manual_seed(0)
    mixer = Fp32Mixer(cfg, 0)
    mixer.c_proj = torch.nn.Identity()
    mixer.eval()
    q, k, v, gate = config1_inputs()
    records: list = []
    undo = _trace_hooks(mixer, records)
    from model.statesdictcache import StatesDictCache
    cache = StatesDictCache()
    with torch.no_grad():
        y = mixer.forward_prefill(q, k, v, gate, None, None, None, cache)
    undo()
    st = _state_of(cache, 0)
    best = torch.stack([r["best_idx"] for r in records if "best_idx" in r], 0).to(torch.int16)
    margin = torch.stack([r["margin"] for r in records if "margin" in r], 0)
    fix = dict(
        n_updates=len(records),
        state_before=[r["state_before"] for r in records], state_after=[r["state_after"] for r in records],
        best_idx=best, min_margin=float(margin.min()),
        y_sample=y[:, ::7, ::5].clone(), y_abs_mean=float(y.abs().mean()),
        s_k_sample=st["kvm_s_k"][:, :, ::3, ::2].clone(), s_v_sample=st["kvm_s_v"][:, :, ::3, ::2].clone(),
        s_vlen=st["kvm_s_vlen"].clone(), coverage=st["kvm_state_coverage_len"], bswa_begin=st["kvm_bswa_begin"],
        torch_version=str(torch.__version__),
    )
    path = os.path.join(HERE, "config1_fp32.pt")
    torch.save(fix, path)
    print(f"config1: updates={len(records)} min margin={fix['min_margin']:.3e} -> {os.path.getsize(path) / 1024:.0f} KiB")


def config1_inputs():
    """Seeded post-QKV inputs with the value distributions of configuration 1 (per-head LayerNorm'd
    q/k of unit variance, v ~ N(0,1), gate = 1 + elu(N(0,1)*0.5)); plain torch, no reference code."""
    g = torch.Generator().manual_seed(0)
    B, H, T, D = 1, 8, 4096, 64
    q = torch.nn.functional.layer_norm(torch.randn(B, T, H, D, generator=g), (D,)).transpose(1, 2)
    k = torch.nn.functional.layer_norm(torch.randn(B, T, H, D, generator=g), (D,)).transpose(1, 2)
    v = torch.randn(B, T, H, D, generator=g).transpose(1, 2)
    gate = (1.0 + torch.nn.functional.elu(0.5 * torch.randn(B, T, H, 1, generator=g))).transpose(1, 2)
    return q, k, v, gate


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True, help="path of the reference checkout")
    ap.add_argument("--only", default=None)
    args = ap.parse_args()
    sys.path.insert(0, args.reference)
    for name, case in _cases().items():
        if args.only in (None, name):
            run_case(args.reference, name, case)
    if args.only in (None, "config1"):
        run_config1(args.reference)


if __name__ == "__main__":
    main()
