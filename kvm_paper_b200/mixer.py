"""Drop-in Key-Value-Means sequence mixer backed by the sm_100a kernels of libkvm_b200.

Select it in the reference project by layering one config line
(``token_mixer_class_path: kvm_paper_b200.mixer.SequenceMixer``, see ``configs/kvm_b200.yaml``); it
has the constructor, config fields, parameter names, ``forward`` / ``forward_inference`` /
``forward_prefill`` / ``forward_single`` signatures and carried-state layout of
``model.kvm_mixer.SequenceMixer`` and ``model.kvm_triton_mixer.SequenceMixer`` of the reference.

Host code (this file) = the projections, token shift, value residual, q/k LayerNorm, RoPE and merge
gate in PyTorch (reference: model/value_residual_mixin.py:173-237, model/kvm_mixer.py:367-401);
everything between the post-QKV tensors and the input of ``c_proj`` runs in the CUDA library.
There is no CPU or eager fallback: without a CUDA device or without the built library the
attention entry points raise.
"""

from __future__ import annotations

import math
from typing import Any

import torch
import torch.nn.functional as F
from torch import nn

from . import ops


def set_label(label: str, module, mup_d_in_ratio=None):
    """Tag parameters for the reference's optimizer grouping (it asserts every parameter has one)."""
    if isinstance(module, torch.Tensor):
        module.label = label
        module.mup_d_in_ratio = mup_d_in_ratio
    else:
        for p in module.parameters():
            set_label(label, p, mup_d_in_ratio)
    return module


def _orthogonal_scaled(rows: int, cols: int, scale: float) -> torch.Tensor:
    w = torch.empty(rows, cols, dtype=torch.float)
    gain = (rows / cols) ** 0.5 if rows > cols else 1
    return torch.nn.init.orthogonal_(w, gain * scale)


def token_shift(x: torch.Tensor, scale: torch.Tensor, prev_token: torch.Tensor | None) -> torch.Tensor:
    """x + scale * (previous token - x); the first token uses itself when no cached token exists
    (reference: model/tokenshift.py:11-37)."""
    if prev_token is None:
        prev_token = x[:, :1]
    elif prev_token.dtype != x.dtype or prev_token.device != x.device:
        prev_token = prev_token.to(device=x.device, dtype=x.dtype)
    return x + scale * (torch.cat([prev_token, x[:, :-1]], dim=1) - x)


def apply_rotary(x_bthd: torch.Tensor, position_embeddings) -> torch.Tensor:
    """Interleaved-pair rotary embedding with precomputed (cos, signed sin) tables
    (reference: model/rwkv7_backbone.py:76-88)."""
    cos, sin = position_embeddings
    assert cos.size(1) == x_bthd.size(1), f"{cos.size()} {x_bthd.size()}"
    flipped = x_bthd.view(*x_bthd.shape[:-1], x_bthd.shape[-1] // 2, 2).flip(-1).view(x_bthd.shape)
    return cos * x_bthd + sin * flipped


class StatesCache:
    """Minimal per-layer dict cache with the interface of the reference's ``StatesDictCache``
    (model/statesdictcache.py:150-187) for use outside the reference project."""

    def __init__(self):
        self._layers: dict[int, dict[str, Any]] = {}
        self._seen: dict[int, int] = {}

    def get_seq_length(self, layer_idx: int = 0) -> int:
        return self._seen.get(layer_idx, 0)

    def get_states(self, layer_idx: int) -> dict[str, Any]:
        return self._layers.setdefault(layer_idx, {})

    def update(self, layer_idx: int, offset: int = 1, states_dict: dict[str, Any] | None = None, **_):
        d = self._layers.setdefault(layer_idx, {})
        if states_dict:
            d.update(states_dict)
        self._seen[layer_idx] = self._seen.get(layer_idx, 0) + offset
        return d


class SequenceMixer(nn.Module):
    """KVM mixer; parameter names equal the reference's so its checkpoints load unchanged."""

    # When set, every prefill / decode call synchronises and raises if a kernel reported a device-side timeout
    # (a bounded wait that ran out).  Off by default: the reference's mixers never synchronise either.
    check_device_status = False
    # Validation hook (the reference's Triton mixer has ``capture_state_snapshots`` for the same purpose): when
    # set, every prefill / decode call also records the routing decision of every consumed token in
    # ``last_route`` ([B*Hkv, n_updates+1, C] after a prefill, [B*Hkv, C] or None after a decode step;
    # >= 0: memory row merged into, -(1+row): appended as that row).
    capture_routes = False
    # prompts of bf16 modules go through the one-kernel prologue (kvm_prologue_forward); False keeps the PyTorch prefix
    use_fused_prologue = True
    last_route = None

    _CACHE_DECODE = "kvm_b200_decode_cache"
    _CACHE_S_K = "kvm_s_k"
    _CACHE_S_V = "kvm_s_v"
    _CACHE_S_VLEN = "kvm_s_vlen"
    _CACHE_STATE_COVERAGE_LEN = "kvm_state_coverage_len"
    _CACHE_BSWA_BEGIN = "kvm_bswa_begin"
    _CACHE_BSWA_K = "kvm_bswa_k"
    _CACHE_BSWA_V = "kvm_bswa_v"
    _CACHE_BSWA_MERGE_GATE = "kvm_bswa_merge_gate"
    _CACHE_Q_FINAL = "att_q_final_token"
    _CACHE_K_FINAL = "att_k_final_token"
    _CACHE_V_FINAL = "att_v_final_token"
    _CACHE_X_FINAL = "att_x_final_token"

    def __init__(self, config, layer_idx: int):
        super().__init__()
        self.layer_idx = layer_idx
        self.config = config
        if not config.kvm_use_vlens:
            raise ValueError("kvm_b200 mixer requires kvm_use_vlens=1")
        H = self.num_attention_heads = config.num_attention_heads
        Hkv = self.num_key_value_heads = (
            config.num_key_value_heads if getattr(config, "num_key_value_heads", None) is not None else H)
        if Hkv <= 0:
            raise ValueError("num_key_value_heads must be positive")
        if H % Hkv:
            raise ValueError("num_attention_heads must be divisible by num_key_value_heads")
        self.kv_group_size = H // Hkv
        hidden = self.hidden_size = config.hidden_size
        d_head = getattr(config, "d_head", None)
        self.d_qk_head = getattr(config, "d_qk_head", None) or d_head or hidden // H
        self.d_v_head = getattr(config, "d_v_head", None) or d_head or hidden // H
        if self.d_qk_head != self.d_v_head or self.d_qk_head not in (32, 64, 128):
            raise ValueError(f"kvm_b200 mixer supports d_qk_head == d_v_head in (32, 64, 128), got "
                             f"{self.d_qk_head}/{self.d_v_head}")
        d_q, d_k, d_v, d_out = H * self.d_qk_head, Hkv * self.d_qk_head, Hkv * self.d_v_head, H * self.d_v_head
        self.q_projection_size, self.k_projection_size = d_q, d_k
        self.value_projection_size, self.attention_output_size = d_v, d_out

        # --- shared prologue parameters (reference: model/value_residual_mixin.py:15-166); creation order
        # and initialisers match so that the same seed yields the same weights
        self.tokenshift_mode = config.kvm_token_shift_mode if config.use_tokenshift_att else "none"
        if self.tokenshift_mode == "rwkv":
            ratio = 1.0 - (layer_idx / config.num_hidden_layers)
            with torch.no_grad():
                self.x_q = set_label("scalars", nn.Parameter(1.0 - torch.pow(_ramp(d_q), 0.2 * ratio)))
                self.x_k = set_label("scalars", nn.Parameter(1.0 - torch.pow(_ramp(d_k), 0.7 * ratio)))
                self.x_v = set_label("scalars", nn.Parameter(1.0 - torch.pow(_ramp(d_v), 0.7 * ratio)))
        self.c_q = set_label("matrix_params", nn.Linear(hidden, d_q, bias=False))
        self.c_k = set_label("matrix_params", nn.Linear(hidden, d_k, bias=False))
        self.c_v = set_label("matrix_params", nn.Linear(hidden, d_v, bias=False))
        self.ln_q = set_label("scalars", nn.LayerNorm(self.d_qk_head))
        self.ln_k = set_label("scalars", nn.LayerNorm(self.d_qk_head))
        self.c_proj = set_label("matrix_params", nn.Linear(d_out, hidden, bias=False))
        with torch.no_grad():
            self.c_proj.weight.zero_()

        self.lamb = None
        self.value_residual_mode = "none"
        if config.use_value_residual:
            mode = config.kvm_value_residual_mode
            assert mode in ["linear", "rwkv", "rwkv_post_tokenshift"], f"Unsupported value residual mode: {mode!r}"
            self.value_residual_mode = mode
            if mode == "linear":
                self.lamb = set_label("scalars", nn.Parameter(torch.tensor(0.5)))
            else:
                if not hasattr(self, "x_v"):
                    self.x_v = set_label("scalars", nn.Parameter(torch.zeros(d_v)))
                lora = lambda c: max(32, int(round((1.3 * (c ** 0.5)) / 32) * 32))  # noqa: E731
                d_lora, d_lora_base = lora(hidden), lora(config.mup_base_dim)
                self.v_gate1 = set_label("matrix_params", nn.Linear(hidden, d_lora, bias=False))
                self.v_gate2 = set_label("matrix_params", nn.Linear(d_lora, d_v, bias=False),
                                         mup_d_in_ratio=d_lora / d_lora_base)
                with torch.no_grad():
                    self.v_gate1.weight.zero_()
                    self.v_gate2.weight.copy_(_orthogonal_scaled(d_lora, d_v, 0.1).T)
                    lin = torch.zeros(d_v)
                    for i in range(d_v):
                        lin[i] = i / max(d_v - 1, 1) - 0.5
                self.v_gate0 = set_label(
                    "scalars", nn.Parameter(torch.zeros(1, 1, d_v) + 0.73 - lin.view(1, 1, d_v) * 0.4))
                if mode == "rwkv_post_tokenshift" and d_v != hidden:
                    self.x_v_hidden = set_label("scalars", nn.Parameter(torch.zeros(hidden)))

        # --- KVM parameters and schedule fields (reference: model/kvm_mixer.py:88-118)
        self.rope_partial_dim = config.rope_partial_dim if config.rope_partial_dim > 0 else self.d_qk_head
        self.ln_s_k = set_label("scalars", nn.LayerNorm(self.d_qk_head))
        self.sink_len = config.sink_len
        self.chunk_len = config.chunk_len
        self.n_max_d_chunks = config.n_max_d_chunks
        self.n_bswa_chunks = config.n_bswa_chunks
        self.max_state_len = self.chunk_len * self.n_max_d_chunks
        self.state_budget_mode = config.state_budget_mode
        self.state_growth_factor = config.state_growth_factor
        self.state_growth_exponent = config.state_growth_exponent
        self.state_round_down = config.state_round_down
        self.state_min_len = config.state_min_len
        self.state_saturation_n = config.state_saturation_n
        if config.kvm_use_merge_gate_keys or config.kvm_use_merge_gate_values:
            self.key_weighting = set_label("matrix_params", nn.Linear(hidden, Hkv, bias=False))
        if config.kvm_use_head_temps:
            self.front_head_temp = set_label("scalars", nn.Parameter(torch.ones(H)))
            self.state_head_temp = set_label("scalars", nn.Parameter(torch.ones(H)))
        if self.chunk_len % 16 or not (16 <= self.chunk_len <= 512):
            raise ValueError(f"kvm_b200 mixer needs chunk_len to be a multiple of 16 in [16, 512], got {self.chunk_len}")
        self._params_cache: tuple | None = None

    # ------------------------------------------------------------------ schedule (host integers)
    def _desired_state_len(self, ctx_len: int, available_context: int, current_state_len: int) -> int:
        """Target number of memory rows (reference: model/kvm_mixer.py:131-165)."""
        ctx = max(int(ctx_len), 0)
        avail = max(int(available_context), 0)
        cur = max(int(current_state_len), 0)
        rd = max(int(self.state_round_down), 1)
        if self.state_budget_mode == "fixed":
            target = self.state_min_len
        elif self.state_budget_mode == "power_law":
            target = int(math.floor(self.state_growth_factor * (float(ctx) ** self.state_growth_exponent)))
            target = max((max(target, 0) // rd) * rd, self.state_min_len)
        elif self.state_budget_mode == "kvm_saturation":
            t = float(ctx)
            n = float(self.state_saturation_n)
            target = int(math.floor((n * t) / (n + t)))
            target = max((max(target, 0) // rd) * rd, self.state_min_len)
        else:
            raise ValueError(f"Unsupported state_budget_mode={self.state_budget_mode!r}")
        return max(min(target, avail, self.max_state_len), cur)

    def _bswa_begin_for_total_len(self, total_len: int) -> int:
        return ops.bswa_begin_for_total_len(total_len, self.chunk_len, self.n_bswa_chunks)

    def make_prefill_plan(self, seq_len: int) -> ops.PrefillPlan:
        return ops.build_prefill_plan(seq_len, self.chunk_len, self.n_bswa_chunks, self._desired_state_len)

    # ------------------------------------------------------------------ device parameters
    def layer_params(self, device) -> ops.LayerParams:
        """fp32 device copies of ln_s_k and the head temperatures, rebuilt when a parameter changes."""
        temps = (self.front_head_temp, self.state_head_temp) if self.config.kvm_use_head_temps else (None, None)
        key = (str(device), self.ln_s_k.weight._version, self.ln_s_k.bias._version,
               self.ln_s_k.weight.data_ptr(), *(0 if t is None else t._version for t in temps))
        if self._params_cache is None or self._params_cache[0] != key:
            cfg = ops.LayerConfig(
                n_q_heads=self.num_attention_heads, n_kv_heads=self.num_key_value_heads, head_dim=self.d_qk_head,
                chunk_len=self.chunk_len, n_bswa_chunks=self.n_bswa_chunks, rope_dim=self.rope_partial_dim,
                sink_len=self.sink_len, gate_keys=bool(self.config.kvm_use_merge_gate_keys),
                gate_values=bool(self.config.kvm_use_merge_gate_values),
                gate_appends=bool(self.config.kvm_apply_merge_gate_to_appends),
                gate_initial=bool(self.config.kvm_apply_merge_gate_to_initial_state), ln_eps=float(self.ln_s_k.eps))
            params = ops.LayerParams(cfg, self.ln_s_k.weight, self.ln_s_k.bias, temps[0], temps[1], device)
            self._params_cache = (key, params)
        return self._params_cache[1]

    # ------------------------------------------------------------------ prologue (host PyTorch)
    def get_first_layer_kwargs(self, x0, x, x_prior_token=None, **kwargs):
        del x0, x_prior_token, kwargs
        if self.value_residual_mode == "none":
            return {"v_first": None}
        return {"v_first": self.c_v(x)}

    def _value_gate(self, x):
        return torch.sigmoid(self.v_gate0 + self.v_gate2(self.v_gate1(x)))

    def calc_qkv(self, x, v_first, past_key_values):
        """Projections, value residual, token shift and per-head q/k LayerNorm
        (reference: model/value_residual_mixin.py:173-237)."""
        B, T, _ = x.size()
        states = past_key_values.get_states(self.layer_idx) if past_key_values is not None else {}
        past_len = past_key_values.get_seq_length(self.layer_idx) if past_key_values is not None else 0
        if past_len > 0 and T != 1:
            raise AssertionError("cached decode expects single-token inputs.")
        q, k, v = self.c_q(x), self.c_k(x), self.c_v(x)
        if self.value_residual_mode == "linear":
            v = (1 - self.lamb) * v + self.lamb * v_first.view_as(v)
        elif self.value_residual_mode == "rwkv":
            v = v + (v_first.to(v.dtype) - v) * self._value_gate(x).to(v.dtype)
        q_prev = k_prev = v_prev = x_prev = None
        if past_key_values is not None:
            q_prev, k_prev = states.get(self._CACHE_Q_FINAL), states.get(self._CACHE_K_FINAL)
            v_prev, x_prev = states.get(self._CACHE_V_FINAL), states.get(self._CACHE_X_FINAL)
            past_key_values.update(self.layer_idx, offset=0, states_dict={
                self._CACHE_Q_FINAL: q[:, -1:].detach(), self._CACHE_K_FINAL: k[:, -1:].detach(),
                self._CACHE_V_FINAL: v[:, -1:].detach(), self._CACHE_X_FINAL: x[:, -1:].detach()})
        if self.tokenshift_mode == "rwkv":
            q = token_shift(q, self.x_q, q_prev)
            k = token_shift(k, self.x_k, k_prev)
            v = token_shift(v, self.x_v, v_prev)
        if self.value_residual_mode == "rwkv_post_tokenshift":
            shift = self.x_v if self.value_projection_size == self.hidden_size else self.x_v_hidden
            xv = token_shift(x, shift.view(1, 1, self.hidden_size), x_prev)
            v = v + (v_first.to(v.dtype) - v) * self._value_gate(xv).to(v.dtype)
        q = self.ln_q(q.reshape(B, T, self.num_attention_heads, -1))
        k = self.ln_k(k.reshape(B, T, self.num_key_value_heads, -1))
        v = v.reshape(B, T, self.num_key_value_heads, -1)
        return q, k, v

    def forward_prefix(self, x, v_first, position_embeddings, attention_mask, past_key_values=None, **kwargs):
        """Everything upstream of the C ABI: returns q [B,Hq,T,D], k, v [B,Hkv,T,D], gate [B,Hkv,T,1]
        (reference: model/kvm_mixer.py:367-401)."""
        B, T, _ = x.size()
        q, k, v = self.calc_qkv(x, v_first, past_key_values)
        q = apply_rotary(q, position_embeddings)
        k = apply_rotary(k, position_embeddings)
        if self.config.kvm_use_merge_gate_keys or self.config.kvm_use_merge_gate_values:
            gate = 1.0 + F.elu(self.key_weighting(x).view(B, T, self.num_key_value_heads, 1)).transpose(1, 2)
        else:
            gate = torch.ones((B, self.num_key_value_heads, T, 1), device=x.device, dtype=torch.float)
        return q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2), gate

    def prologue_params(self, device) -> ops.PrologueParams:
        ln = isinstance(self.ln_q, nn.LayerNorm)
        shift = self.tokenshift_mode == "rwkv"
        return ops.PrologueParams(device, shift_q=self.x_q if shift else None, shift_k=self.x_k if shift else None,
                                  shift_v=self.x_v if shift else None, ln_q=self.ln_q if ln else None,
                                  ln_k=self.ln_k if ln else None, ln_eps=self.ln_q.eps if ln else 1e-5)

    def fused_prologue_applies(self, x: torch.Tensor) -> bool:
        """The one-kernel prologue covers bf16 modules on CUDA with head dims the kernel is built for and a value
        path without the post-shift residual (that variant mixes values after the token shift)."""
        return (x.is_cuda and x.dtype == torch.bfloat16 and self.c_q.weight.dtype == torch.bfloat16
                and self.d_qk_head in (32, 64, 128) and self.value_projection_size == self.num_key_value_heads * self.d_qk_head
                and self.value_residual_mode != "rwkv_post_tokenshift")

    def forward_prefix_fused(self, x, v_first, position_embeddings, past_key_values=None, runner=None):
        """``forward_prefix`` with everything behind the projections in one kernel (``kvm_prologue_forward``): the
        projections and the value residual are torch GEMMs / elementwise ops as in ``calc_qkv``; token shift, q/k
        LayerNorm, rotary embedding and merge gate run fused, and with ``runner`` the prepared keys of the prompt are
        written into its workspace (reference: model/value_residual_mixin.py:173-237, model/kvm_mixer.py:367-401)."""
        B, T, _ = x.size()
        states = past_key_values.get_states(self.layer_idx) if past_key_values is not None else {}
        past_len = past_key_values.get_seq_length(self.layer_idx) if past_key_values is not None else 0
        if past_len > 0 and T != 1:
            raise AssertionError("cached decode expects single-token inputs.")
        q, k, v = self.c_q(x), self.c_k(x), self.c_v(x)
        if self.value_residual_mode == "linear":
            v = (1 - self.lamb) * v + self.lamb * v_first.view_as(v)
        elif self.value_residual_mode == "rwkv":
            v = v + (v_first.to(v.dtype) - v) * self._value_gate(x).to(v.dtype)
        prev = None
        if past_key_values is not None:
            prev = (states.get(self._CACHE_Q_FINAL), states.get(self._CACHE_K_FINAL), states.get(self._CACHE_V_FINAL))
            past_key_values.update(self.layer_idx, offset=0, states_dict={
                self._CACHE_Q_FINAL: q[:, -1:].detach(), self._CACHE_K_FINAL: k[:, -1:].detach(),
                self._CACHE_V_FINAL: v[:, -1:].detach(), self._CACHE_X_FINAL: x[:, -1:].detach()})
        gated = self.config.kvm_use_merge_gate_keys or self.config.kvm_use_merge_gate_values
        gate_lin = self.key_weighting(x) if gated else None
        dev = x.device
        return ops.prologue_forward(self.layer_params(dev), self.prologue_params(dev), q.contiguous(), k.contiguous(),
                                    v.contiguous(), gate_lin, position_embeddings, prev=prev, runner=runner)

    # ------------------------------------------------------------------ module entry points
    def _prompt_fused(self, x, v_first, position_embeddings, attention_mask, past_key_values, **kwargs):
        """A prompt through the one-kernel prologue, which also leaves the prepared keys in the prefill's workspace."""
        params = self.layer_params(x.device)
        runner = ops.PrefillRunner(params, x.size(0), self.make_prefill_plan(int(x.size(1))), want_route=self.capture_routes)
        q, k, v, gate = self.forward_prefix_fused(x, v_first, position_embeddings, past_key_values, runner=runner)
        return self.forward_prefill(q, k, v, gate, v_first, position_embeddings, attention_mask, past_key_values,
                                    _prefill_runner=runner, **kwargs)

    def forward(self, x, v_first, position_embeddings, attention_mask, past_key_values=None, **kwargs):
        if self.use_fused_prologue and attention_mask is None and self.fused_prologue_applies(x):
            return self._prompt_fused(x, v_first, position_embeddings, attention_mask, past_key_values, **kwargs)
        q, k, v, gate = self.forward_prefix(x, v_first, position_embeddings, attention_mask, past_key_values, **kwargs)
        return self.forward_prefill(q, k, v, gate, v_first, position_embeddings, attention_mask, past_key_values, **kwargs)

    def forward_inference(self, x, v_first, position_embeddings, attention_mask, past_key_values=None, **kwargs):
        past_len = past_key_values.get_seq_length(self.layer_idx) if past_key_values is not None else 0
        if past_len == 0 and self.use_fused_prologue and attention_mask is None and self.fused_prologue_applies(x):
            return self._prompt_fused(x, v_first, position_embeddings, attention_mask, past_key_values, **kwargs)
        if past_len > 0 and self.use_fused_prologue and attention_mask is None and self.fused_prologue_applies(x):
            # cached single-token step: the same kernel, shifting against the previous call's last token
            q, k, v, gate = self.forward_prefix_fused(x, v_first, position_embeddings, past_key_values)
        else:
            q, k, v, gate = self.forward_prefix(x, v_first, position_embeddings, attention_mask, past_key_values, **kwargs)
        fn = self.forward_single if past_len > 0 else self.forward_prefill
        return fn(q, k, v, gate, v_first, position_embeddings, attention_mask, past_key_values, **kwargs)

    def _require_cuda(self, t: torch.Tensor):
        if not t.is_cuda:
            raise RuntimeError("kvm_b200 mixer runs on CUDA tensors only (there is no CPU path)")
        if torch.is_grad_enabled() and t.requires_grad:
            raise ValueError("kvm_b200 mixer implements inference (prefill/decode) only; call it under torch.no_grad()")

    def prefill_raw(self, q, k, v, merge_gate, *, want_route: bool = False, memory_capacity: int | None = None, runner=None):
        """Operator-boundary prefill: returns ops.PrefillResult (pre-``c_proj`` activations, final memory).
        ``runner``: the runner whose workspace the fused prologue filled with this prompt's prepared keys."""
        self._require_cuda(q)
        plan = self.make_prefill_plan(int(q.size(2))) if runner is None else runner.plan
        params = self.layer_params(q.device)
        return ops.prefill_forward(params, q, k, v, merge_gate, plan, want_route=want_route,
                                   memory_capacity=memory_capacity, check=self.check_device_status,
                                   runner=runner, keys_prepared=runner is not None)

    def forward_prefill(self, q, k, v, merge_gate, v_first, position_embeddings, attention_mask,
                        past_key_values=None, **kwargs):
        """Reference: model/kvm_mixer.py:403-516, model/kvm_triton_mixer.py:560-664."""
        del v_first, position_embeddings
        if attention_mask is not None:
            raise ValueError("kvm_b200 mixer does not support attention_mask")
        T = int(q.size(2))
        res = self.prefill_raw(q, k, v, merge_gate, want_route=self.capture_routes, runner=kwargs.pop("_prefill_runner", None))
        if self.capture_routes:
            self.last_route = res.route
        y = self.c_proj(res.out.to(q.dtype))
        if past_key_values is not None:
            plan = res.plan
            init_len = min(T, self.chunk_len)
            if plan.final_coverage != max(init_len, self._bswa_begin_for_total_len(T)):
                raise AssertionError("KVM prefill state progression drifted from the decode-state bookkeeping.")
            cache = ops.decode_cache_from_prefill(self.layer_params(q.device), res, k, v, merge_gate,
                                                  self._desired_state_len, owner=self)
            past_key_values.update(self.layer_idx, offset=T, states_dict={self._CACHE_DECODE: cache})
        return y

    def _cache_from_eager_states(self, states: dict, total_len: int, device) -> ops.KvmDecodeCache:
        """Adopt a cache written by the reference's eager mixer (model/kvm_mixer.py:501-514)."""
        s_k = states[self._CACHE_S_K]
        B, Hkv, S, D = s_k.shape
        cache = ops.KvmDecodeCache(self.layer_params(device), B, S + self.chunk_len, self._desired_state_len, owner=self)
        for b in range(B):
            cache.load_sequence(
                b, k_sum=states[self._CACHE_S_K][b], v_sum=states[self._CACHE_S_V][b], vlen=states[self._CACHE_S_VLEN][b],
                window_k=states[self._CACHE_BSWA_K][b], window_v=states[self._CACHE_BSWA_V][b],
                window_gate=states[self._CACHE_BSWA_MERGE_GATE][b], total_len=total_len)
        cache.commit_lengths(refresh_attention_view=True)
        return cache

    def forward_single(self, q, k, v, merge_gate, v_first, position_embeddings, attention_mask,
                       past_key_values=None, **kwargs):
        """One cached decode token (reference: model/kvm_mixer.py:572-713, model/kvm_triton_mixer.py:668-715)."""
        del v_first, position_embeddings, kwargs
        if attention_mask is not None:
            raise ValueError("kvm_b200 mixer does not support attention_mask")
        if past_key_values is None:
            raise ValueError("KVM cached decode requires past_key_values")
        if int(q.size(2)) != 1:
            raise AssertionError(
                "KVM cached decode expects single-token inputs. Multi-token decode with past_key_values is not supported.")
        self._require_cuda(q)
        states = past_key_values.get_states(self.layer_idx)
        past_len = past_key_values.get_seq_length(self.layer_idx)
        cache = states.get(self._CACHE_DECODE)
        if cache is None and self._CACHE_S_K in states:
            cache = self._cache_from_eager_states(states, past_len, q.device)
        if not isinstance(cache, ops.KvmDecodeCache):
            raise RuntimeError("KVM cache is missing its decode state; run a prefill with this cache before decoding")
        if cache.owner is not self:
            raise RuntimeError("KVM decode cache belongs to another mixer")
        if int(cache.total_len_h[0]) != past_len or len(set(cache.total_len_h.tolist())) != 1:
            raise AssertionError(f"KVM decode cache length disagrees with the layer cache: {cache.total_len_h.tolist()} != {past_len}")
        out = cache.step(q, k, v, merge_gate, want_route=self.capture_routes)
        if self.capture_routes:
            self.last_route = cache.route if cache._last_any_update else None
        if self.check_device_status:
            cache.check_status()
        past_key_values.update(self.layer_idx, offset=1, states_dict={self._CACHE_DECODE: cache})
        return self.c_proj(out.to(q.dtype))


def _ramp(n: int) -> torch.Tensor:
    out = torch.ones(n)
    for i in range(n):
        out[i] = i / n
    return out
