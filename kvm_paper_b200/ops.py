"""Host side of the KVM operators: schedule tables, device buffers and the calls into libkvm_b200.

PyTorch is used for device memory and streams only; every kernel runs inside the C-ABI library.
Names follow the reference: "memory" = the compressed key/value means (``kvm_s_k`` / ``kvm_s_v`` /
``kvm_s_vlen``), "window" = the block sliding window (BSWA), "block" = ``chunk_len`` tokens.
"""

from __future__ import annotations

import ctypes as C
import math
from dataclasses import dataclass
from typing import Any, Callable

import numpy as np
import torch

from . import _lib
from ._lib import KvmDecodeCache as _CCache
from ._lib import KvmLayer, KvmMemory, KvmTensor4, KvmUpdatePlan



def _ptr(t: torch.Tensor | None) -> int | None:
    return None if t is None else t.data_ptr()


def _stream_ptr(device) -> int:
    return torch.cuda.current_stream(device).cuda_stream


def _tensor4(t: torch.Tensor, name: str) -> KvmTensor4:
    """[B,H,T,D] view with a contiguous last dimension -> C descriptor (strides in elements)."""
    if t.dim() != 4:
        raise ValueError(f"{name} must be 4-dimensional, got {tuple(t.shape)}")
    if t.dtype != torch.bfloat16:
        raise ValueError(f"{name} must be bfloat16, got {t.dtype}")
    if not t.is_cuda:
        raise RuntimeError(f"{name} must live on a CUDA device")
    if t.size(-1) > 1 and t.stride(-1) != 1:
        t = t.contiguous()
    return KvmTensor4(t.data_ptr(), t.stride(0), t.stride(1), t.stride(2))


def _as_bf16_view(t: torch.Tensor) -> torch.Tensor:
    """Keep strided views as they are; only fix dtype / inner stride."""
    if t.dtype != torch.bfloat16:
        t = t.to(torch.bfloat16)
    if t.size(-1) > 1 and t.stride(-1) != 1:
        t = t.contiguous()
    return t


@dataclass
class LayerConfig:
    """Static description of one mixer layer (mirror of ``kvm_layer``)."""

    n_q_heads: int
    n_kv_heads: int
    head_dim: int
    chunk_len: int
    n_bswa_chunks: int
    rope_dim: int
    sink_len: int
    gate_keys: bool = True
    gate_values: bool = True
    gate_appends: bool = False
    gate_initial: bool = False
    ln_eps: float = 1e-5


class LayerParams:
    """Device copies (fp32) of the small parameter vectors the kernels read, plus the C struct."""

    def __init__(self, cfg: LayerConfig, ln_weight: torch.Tensor, ln_bias: torch.Tensor,
                 front_temp: torch.Tensor | None, state_temp: torch.Tensor | None, device):
        self.cfg = cfg
        dev = torch.device(device)
        self.device = dev
        self.ln_w = ln_weight.detach().to(dev, torch.float32).contiguous()
        self.ln_b = ln_bias.detach().to(dev, torch.float32).contiguous()
        ones = torch.ones(cfg.n_q_heads, device=dev, dtype=torch.float32)
        self.front = ones if front_temp is None else front_temp.detach().to(dev, torch.float32).contiguous()
        self.state = ones if state_temp is None else state_temp.detach().to(dev, torch.float32).contiguous()
        self.c = KvmLayer(
            cfg.n_q_heads, cfg.n_kv_heads, cfg.head_dim, cfg.chunk_len, cfg.n_bswa_chunks, cfg.rope_dim,
            cfg.sink_len, int(cfg.gate_keys), int(cfg.gate_values), int(cfg.gate_appends), int(cfg.gate_initial),
            float(cfg.ln_eps), self.ln_w.data_ptr(), self.ln_b.data_ptr(), self.front.data_ptr(), self.state.data_ptr())


# --------------------------------------------------------------------------------------- schedule

def bswa_begin_for_total_len(total_len: int, chunk_len: int, n_bswa_chunks: int) -> int:
    """Start of the block sliding window for a sequence of ``total_len`` tokens
    (reference: model/kvm_mixer.py:167-172)."""
    end = ((max(int(total_len), 0) + chunk_len - 1) // chunk_len) * chunk_len
    return max(0, end - n_bswa_chunks * chunk_len)


@dataclass
class PrefillPlan:
    """Per-update schedule of one prefill (uniform over the batch)."""

    seq_len: int
    state_before: list[int]
    n_append: list[int]
    version_row: list[int]
    total_version_rows: int
    final_state_len: int
    final_coverage: int
    bswa_begin: int

    @property
    def n_updates(self) -> int:
        return len(self.n_append) - 1

    def to_ctypes(self):
        arr = (KvmUpdatePlan * len(self.n_append))()
        for i, (sb, na, vr) in enumerate(zip(self.state_before, self.n_append, self.version_row)):
            arr[i] = KvmUpdatePlan(sb, na, vr, 0)
        return arr

    def to_tensor(self, device) -> torch.Tensor:
        t = torch.tensor([[sb, na, vr, 0] for sb, na, vr in zip(self.state_before, self.n_append, self.version_row)],
                         dtype=torch.int32)
        return t.to(device, non_blocking=True)


def build_prefill_plan(seq_len: int, chunk_len: int, n_bswa_chunks: int,
                       desired_state_len: Callable[[int, int, int], int], keep_versions: bool = True) -> PrefillPlan:
    """Walk the block loop of the reference prefill (model/kvm_mixer.py:450-488) on integers only.

    ``desired_state_len(ctx_len, available_context, current)`` is the mixer's own schedule method, so an
    overridden schedule flows through unchanged."""
    T, Cn, W = int(seq_len), int(chunk_len), int(n_bswa_chunks)
    n_blocks = (T + Cn - 1) // Cn
    init = min(T, Cn)
    state_before, n_append, version_row = [0], [init], [0]
    S = init
    rows = 0
    n_plan = n_blocks - W if n_blocks > W else 1
    keeps_versions = n_blocks > W
    if keeps_versions:
        rows = _round8(S)
    for u in range(1, n_plan):
        ctx_len = (u + W) * Cn
        available = (u + 1) * Cn
        desired = int(desired_state_len(ctx_len, available, S))
        na = min(max(desired - S, 0), Cn)
        state_before.append(S)
        n_append.append(na)
        S += na
        version_row.append(rows)
        rows += _round8(S)
    if not keeps_versions or not keep_versions:
        # no query block reads a memory version (short prompt), or only the final memory is wanted
        version_row = [-1] * len(n_append)
        rows = 0
    bb = bswa_begin_for_total_len(T, Cn, W)
    return PrefillPlan(T, state_before, n_append, version_row, rows, S, max(init, bb), bb)


def _round8(x: int) -> int:
    return (x + 7) // 8 * 8


# ----------------------------------------------------------------------------------------- memory

class MemoryBuffers:
    """The compressed memory of ``n_rows`` kv rows with ``capacity`` rows each."""

    def __init__(self, n_rows: int, capacity: int, head_dim: int, device):
        self.n_rows, self.capacity, self.head_dim = n_rows, int(capacity), head_dim
        kw = dict(device=device, dtype=torch.bfloat16)
        self.k_sum = torch.zeros(n_rows, capacity, head_dim, **kw)
        self.v_sum = torch.zeros(n_rows, capacity, head_dim, **kw)
        self.vlen = torch.zeros(n_rows, capacity, device=device, dtype=torch.float32)
        self.k_attn = torch.zeros(n_rows, capacity, head_dim, **kw)
        self.v_attn = torch.zeros(n_rows, capacity, head_dim, **kw)

    def c(self) -> KvmMemory:
        return KvmMemory(self.k_sum.data_ptr(), self.v_sum.data_ptr(), self.vlen.data_ptr(),
                         self.k_attn.data_ptr(), self.v_attn.data_ptr(), self.capacity)

    def grown(self, new_capacity: int) -> "MemoryBuffers":
        out = MemoryBuffers(self.n_rows, new_capacity, self.head_dim, self.k_sum.device)
        n = self.capacity
        for name in ("k_sum", "v_sum", "vlen", "k_attn", "v_attn"):
            getattr(out, name)[:, :n].copy_(getattr(self, name))
        return out


@dataclass
class PrefillResult:
    out: torch.Tensor                 # [B, T, Hq*D] bf16, the input of c_proj
    memory: MemoryBuffers
    plan: PrefillPlan
    route: torch.Tensor | None        # [B*Hkv, n_updates+1, C] int32 if requested
    runner: Any = None                # the PrefillRunner that produced it (workspace inspection)


class PrologueParams:
    """Device copies of what the fused prologue reads besides the projections: token-shift scales (bf16),
    per-head LayerNorm of q and k (fp32), all optional as in the reference module
    (model/value_residual_mixin.py:60-98)."""

    def __init__(self, device, *, shift_q=None, shift_k=None, shift_v=None, ln_q=None, ln_k=None, ln_eps: float = 1e-5):
        dev = torch.device(device)
        shifts = [None if t is None else t.detach().to(dev, torch.bfloat16).reshape(-1).contiguous() for t in (shift_q, shift_k, shift_v)]
        if any(t is None for t in shifts) and not all(t is None for t in shifts):
            raise ValueError("token-shift scales must be given for q, k and v or for none")
        self.shift_q, self.shift_k, self.shift_v = shifts
        if (ln_q is None) != (ln_k is None):
            raise ValueError("LayerNorm must be given for q and k or for neither")
        self.ln = None
        if ln_q is not None:
            self.ln = tuple(t.detach().to(dev, torch.float32).contiguous() for t in (ln_q.weight, ln_q.bias, ln_k.weight, ln_k.bias))
        self.ln_eps = float(ln_eps)


def prologue_forward(params: LayerParams, pro: PrologueParams, q_lin: torch.Tensor, k_lin: torch.Tensor, v_lin: torch.Tensor,
                     gate_lin: torch.Tensor | None, position_embeddings, *, prev=None, runner: "PrefillRunner | None" = None,
                     out: tuple | None = None):
    """Token shift, q/k LayerNorm, rotary embedding and merge gate in one kernel over the projection outputs
    ([B,T,H*D] bf16).  Returns q [B,Hq,T,D], k, v [B,Hkv,T,D], gate [B,Hkv,T,1] as views of [B,T,H,D] / [B,Hkv,T]
    buffers, the layouts the reference hands its mixer (model/kvm_mixer.py:397-399).  With ``runner`` the prepared
    keys of the tokens that memory updates consume are written into that runner's workspace, and its ``run`` may
    be called with ``keys_prepared=True``.  ``prev`` = (q, k, v) rows [B,1,H*D] of the previous call's last token.
    ``out`` = preallocated (q [B,T,Hq,D], k, v [B,T,Hkv,D], gate [B,Hkv,T]) bf16 buffers to write into."""
    cfg = params.cfg
    B, T, _ = q_lin.shape
    D, Hq, Hkv = cfg.head_dim, cfg.n_q_heads, cfg.n_kv_heads
    for name, t, h in (("q", q_lin, Hq), ("k", k_lin, Hkv), ("v", v_lin, Hkv)):
        if t.dtype != torch.bfloat16 or not t.is_cuda or not t.is_contiguous() or t.shape != (B, T, h * D):
            raise ValueError(f"{name} projection must be a contiguous bf16 CUDA tensor [B,T,{h * D}], got {tuple(t.shape)} {t.dtype}")
    keep = []
    arg = _lib.KvmPrologue()
    arg.q_lin, arg.k_lin, arg.v_lin = q_lin.data_ptr(), k_lin.data_ptr(), v_lin.data_ptr()
    if gate_lin is not None:
        gate_lin = gate_lin.to(torch.bfloat16).reshape(B, T, Hkv).contiguous()
        keep.append(gate_lin)
        arg.gate_lin = gate_lin.data_ptr()
    if pro.shift_q is not None:
        arg.shift_q, arg.shift_k, arg.shift_v = pro.shift_q.data_ptr(), pro.shift_k.data_ptr(), pro.shift_v.data_ptr()
        if prev is not None and all(t is not None for t in prev):
            pv = [t.to(q_lin.device, torch.bfloat16).reshape(B, -1).contiguous() for t in prev]
            keep += pv
            arg.prev_q, arg.prev_k, arg.prev_v = (t.data_ptr() for t in pv)
    if pro.ln is not None:
        arg.ln_q_w, arg.ln_q_b, arg.ln_k_w, arg.ln_k_b = (t.data_ptr() for t in pro.ln)
        arg.ln_qk_eps = pro.ln_eps
    if position_embeddings is not None:
        cos, sin = position_embeddings
        cs = [t.to(q_lin.device, torch.bfloat16).reshape(-1, T, D).contiguous() for t in (cos, sin)]
        if cs[0].size(0) not in (1, B):
            raise ValueError(f"rotary tables must have batch 1 or {B}, got {cs[0].size(0)}")
        keep += cs
        arg.cos, arg.sin = cs[0].data_ptr(), cs[1].data_ptr()
        arg.rope_stride_b = 0 if cs[0].size(0) == 1 else T * D
    dev = q_lin.device
    if out is not None:
        q, k, v, gate = out
        for t, shape in ((q, (B, T, Hq, D)), (k, (B, T, Hkv, D)), (v, (B, T, Hkv, D)), (gate, (B, Hkv, T))):
            if tuple(t.shape) != shape or t.dtype != torch.bfloat16 or not t.is_contiguous() or t.device != dev:
                raise ValueError(f"out buffer must be a contiguous bf16 tensor {shape} on {dev}, got {tuple(t.shape)} {t.dtype}")
    else:
        q = torch.empty(B, T, Hq, D, device=dev, dtype=torch.bfloat16)
        k = torch.empty(B, T, Hkv, D, device=dev, dtype=torch.bfloat16)
        v = torch.empty(B, T, Hkv, D, device=dev, dtype=torch.bfloat16)
        gate = torch.empty(B, Hkv, T, device=dev, dtype=torch.bfloat16)
    ws_ptr, ws_bytes, ver_rows = None, 0, 0
    if runner is not None:
        if runner.batch != B or runner.plan.seq_len != T:
            raise ValueError("runner was built for another batch or sequence length")
        ws_ptr, ws_bytes, ver_rows = runner.ws.data_ptr(), runner.ws_bytes, runner.plan.total_version_rows
    rc = _lib.load().kvm_prologue_forward(C.byref(params.c), B, T, C.byref(arg), q.data_ptr(), k.data_ptr(), v.data_ptr(),
                                          gate.data_ptr(), ver_rows, ws_ptr, ws_bytes, _stream_ptr(dev))
    _lib.check(rc)
    del keep  # (the kernel is enqueued on the current stream: torch's allocator keeps the blocks until it has run)
    return q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2), gate.unsqueeze(-1)


class PrefillRunner:
    """Preallocated buffers for repeated prefills of one shape (memory, workspace with the row pool and version tables, output).

    ``run`` only enqueues kernels on the current stream; nothing is allocated per call."""

    def __init__(self, params: LayerParams, batch: int, plan: PrefillPlan, *, memory_capacity: int | None = None,
                 want_route: bool = False):
        lib = _lib.load()
        cfg = params.cfg
        self.params, self.plan, self.batch = params, plan, int(batch)
        dev = params.device
        cap = max(plan.final_state_len, 1) if memory_capacity is None else int(memory_capacity)
        self.memory = MemoryBuffers(batch * cfg.n_kv_heads, cap, cfg.head_dim, dev)
        self.ws_bytes = lib.kvm_prefill_workspace_bytes(C.byref(params.c), batch, plan.seq_len, plan.total_version_rows)
        self.ws = torch.empty(self.ws_bytes, device=dev, dtype=torch.uint8)
        self.out = torch.empty(batch, plan.seq_len, cfg.n_q_heads * cfg.head_dim, device=dev, dtype=torch.bfloat16)
        self.route = None
        if want_route:
            self.route = torch.zeros(batch * cfg.n_kv_heads, plan.n_updates + 1, cfg.chunk_len, device=dev, dtype=torch.int32)
        self.plan_dev = plan.to_tensor(dev)
        self.plan_host = plan.to_ctypes()

    def run(self, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, gate: torch.Tensor,
            phases: int = _lib.PREFILL_CHAIN | _lib.PREFILL_ATTENTION, *, keys_prepared: bool = False) -> torch.Tensor:
        """``keys_prepared``: ``prologue_forward(..., runner=self)`` has written the prepared keys of this prompt into
        the workspace; the chain phase skips its own pass over the keys."""
        cfg, plan = self.params.cfg, self.plan
        if keys_prepared:
            phases |= _lib.PREFILL_KEYS_PREPARED
        B, Hq, T, D = q.shape
        if (B, Hq, D) != (self.batch, cfg.n_q_heads, cfg.head_dim) or k.shape != (B, cfg.n_kv_heads, T, D) or v.shape != k.shape:
            raise ValueError(f"shape mismatch: q {tuple(q.shape)}, k {tuple(k.shape)}, v {tuple(v.shape)} for {cfg}")
        if gate.shape != (B, cfg.n_kv_heads, T, 1):
            raise ValueError(f"merge gate must be [B,Hkv,T,1], got {tuple(gate.shape)}")
        if T != plan.seq_len:
            raise ValueError("plan was built for another sequence length")
        q, k, v, gate = (_as_bf16_view(t) for t in (q, k, v, gate))
        rc = _lib.load().kvm_prefill_forward(
            C.byref(self.params.c), B, T, _tensor4(q, "q"), _tensor4(k, "k"), _tensor4(v, "v"), _tensor4(gate, "gate"),
            self.plan_dev.data_ptr(), self.plan_host, plan.n_updates, plan.total_version_rows, self.memory.c(),
            self.out.data_ptr(), _ptr(self.route), self.ws.data_ptr(), self.ws_bytes, phases,
            _stream_ptr(self.params.device))
        _lib.check(rc)
        return self.out

    def run_gathered(self, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, gate: torch.Tensor, rank: int, out_ptrs: list[int],
                     phases: int = _lib.PREFILL_CHAIN | _lib.PREFILL_ATTENTION, *, keys_prepared: bool = False) -> None:
        """One rank of a head-sharded prefill whose attention kernel writes this rank's heads into every rank's
        [B,T,world*Hq*D] output (``out_ptrs``: addresses of all ranks' buffers as this process sees them, see
        ``sharding.GatheredPrefillOutput``).  Nothing is returned: a buffer is complete once every rank's call has
        finished (the caller synchronises the ranks)."""
        cfg, plan = self.params.cfg, self.plan
        B, Hq, T, D = q.shape
        if (B, Hq, D) != (self.batch, cfg.n_q_heads, cfg.head_dim) or k.shape != (B, cfg.n_kv_heads, T, D) or v.shape != k.shape:
            raise ValueError(f"shape mismatch: q {tuple(q.shape)}, k {tuple(k.shape)}, v {tuple(v.shape)} for {cfg}")
        if gate.shape != (B, cfg.n_kv_heads, T, 1) or T != plan.seq_len:
            raise ValueError("merge gate must be [B,Hkv,T,1] and the plan built for this sequence length")
        if keys_prepared:
            phases |= _lib.PREFILL_KEYS_PREPARED
        q, k, v, gate = (_as_bf16_view(t) for t in (q, k, v, gate))
        bases = (C.c_void_p * len(out_ptrs))(*out_ptrs)
        rc = _lib.load().kvm_prefill_forward_gathered(
            C.byref(self.params.c), B, T, _tensor4(q, "q"), _tensor4(k, "k"), _tensor4(v, "v"), _tensor4(gate, "gate"),
            self.plan_dev.data_ptr(), self.plan_host, plan.n_updates, plan.total_version_rows, self.memory.c(),
            len(out_ptrs), int(rank), bases, _ptr(self.route), self.ws.data_ptr(), self.ws_bytes, phases,
            _stream_ptr(self.params.device))
        _lib.check(rc)

    def check_status(self) -> None:
        """Synchronise and raise if a kernel of the last run reported a device-side timeout."""
        rc = _lib.load().kvm_prefill_status(self.ws.data_ptr(), _stream_ptr(self.params.device))
        _lib.check(rc)

    def workspace_views(self) -> dict[str, torch.Tensor]:
        """Views (no copies) of what the last run left in the workspace, for inspection: the row pool of the
        memory's attention view ``pool_k`` / ``pool_v`` [kv rows, pool_rows, D], the version tables
        ``versions`` [kv rows, total_version_rows] (entry ``plan.version_row[u] + r`` = pool row of memory
        row ``r`` after update ``u``) and the prepared keys ``prepared_keys`` [kv rows, (n_updates+1)*C, D]."""
        cfg, plan = self.params.cfg, self.plan
        lay = _lib.KvmPrefillLayout()
        _lib.check(_lib.load().kvm_prefill_workspace_layout(C.byref(self.params.c), self.batch, plan.seq_len,
                                                            plan.total_version_rows, C.byref(lay)))
        rows, D = self.batch * cfg.n_kv_heads, cfg.head_dim

        def view(offset, shape, dtype):
            n = math.prod(shape) * torch.empty((), dtype=dtype).element_size()
            return self.ws[offset:offset + n].view(dtype).view(shape)

        out = {"pool_k": view(lay.pool_k_offset, (rows, lay.pool_rows, D), torch.bfloat16),
               "pool_v": view(lay.pool_v_offset, (rows, lay.pool_rows, D), torch.bfloat16),
               "versions": view(lay.version_table_offset, (rows, plan.total_version_rows), torch.int32)}
        if plan.n_updates > 0:
            out["prepared_keys"] = view(lay.prepared_keys_offset, (rows, (plan.n_updates + 1) * cfg.chunk_len, D),
                                        torch.bfloat16)
        return out


class HostPrefill:
    """Prefill whose inputs and output live in pinned host memory (a serving front end that receives the
    post-QKV tensors of a request batch on the host): the batch is cut into slices of sequences and slice
    i+1 is copied in while slice i is computed and slice i-1 is copied out, on three streams (copy-in,
    the caller's current stream, copy-out) with two sets of device buffers.

    Host tensors are laid out as the projections produce them: q [B,T,Hq,D], k/v [B,T,Hkv,D],
    gate [B,T,Hkv,1], out [B,T,Hq*D], all bf16 and pinned."""

    def __init__(self, params: LayerParams, batch: int, plan: PrefillPlan, slice_batch: int = 1):
        cfg = params.cfg
        if batch % slice_batch:
            raise ValueError(f"batch {batch} is not a multiple of the slice size {slice_batch}")
        dev = params.device
        self.params, self.plan, self.batch, self.bs = params, plan, int(batch), int(slice_batch)
        T, D = plan.seq_len, cfg.head_dim
        kw = dict(device=dev, dtype=torch.bfloat16)
        self.runners = [PrefillRunner(params, self.bs, plan) for _ in range(2)]
        self.dev_in = [(torch.empty(self.bs, T, cfg.n_q_heads, D, **kw), torch.empty(self.bs, T, cfg.n_kv_heads, D, **kw),
                        torch.empty(self.bs, T, cfg.n_kv_heads, D, **kw), torch.empty(self.bs, T, cfg.n_kv_heads, 1, **kw))
                       for _ in range(2)]
        self.s_in, self.s_out = torch.cuda.Stream(device=dev), torch.cuda.Stream(device=dev)
        self.ev_kv = [torch.cuda.Event() for _ in range(2)]      # keys, values and gates of the slot have arrived
        self.ev_in = [torch.cuda.Event() for _ in range(2)]      # ... and the queries
        self.ev_comp = [torch.cuda.Event() for _ in range(2)]    # the slot's kernels are done (inputs free, output ready)
        self.ev_out = [torch.cuda.Event() for _ in range(2)]     # the slot's output has left the device

    def run(self, hq: torch.Tensor, hk: torch.Tensor, hv: torch.Tensor, hg: torch.Tensor, h_out: torch.Tensor) -> torch.Tensor:
        for name, t in (("q", hq), ("k", hk), ("v", hv), ("gate", hg), ("out", h_out)):
            if t.is_cuda or not t.is_pinned() or t.dtype != torch.bfloat16 or t.size(0) != self.batch:
                raise ValueError(f"{name} must be a pinned bf16 host tensor with batch {self.batch}")
        cur = torch.cuda.current_stream(self.params.device)
        self.s_in.wait_stream(cur)  # whatever produced the host buffers' contents is ordered before the copies
        n = self.batch // self.bs
        for i in range(n):
            slot, lo = i % 2, i * self.bs
            with torch.cuda.stream(self.s_in):
                if i >= 2:
                    self.s_in.wait_event(self.ev_comp[slot])  # slice i-2 no longer reads these device buffers
                # keys, values and gates first: the memory trajectory does not need the queries
                for d, h in zip(self.dev_in[slot][1:], (hk, hv, hg)):
                    d.copy_(h[lo:lo + self.bs], non_blocking=True)
                self.ev_kv[slot].record(self.s_in)
                self.dev_in[slot][0].copy_(hq[lo:lo + self.bs], non_blocking=True)
                self.ev_in[slot].record(self.s_in)
            dq, dk, dv, dg = (t.transpose(1, 2) for t in self.dev_in[slot])
            cur.wait_event(self.ev_kv[slot])
            self.runners[slot].run(dq, dk, dv, dg, phases=_lib.PREFILL_CHAIN)
            cur.wait_event(self.ev_in[slot])
            if i >= 2:
                cur.wait_event(self.ev_out[slot])  # the slot's output buffer has been copied out
            out = self.runners[slot].run(dq, dk, dv, dg, phases=_lib.PREFILL_ATTENTION)
            self.ev_comp[slot].record(cur)
            with torch.cuda.stream(self.s_out):
                self.s_out.wait_event(self.ev_comp[slot])
                h_out[lo:lo + self.bs].copy_(out, non_blocking=True)
                self.ev_out[slot].record(self.s_out)
        for slot in range(min(2, n)):
            cur.wait_event(self.ev_out[slot])  # the call is complete, in stream order, when the output is on the host
        return h_out


def prefill_forward(params: LayerParams, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, gate: torch.Tensor,
                    plan: PrefillPlan, *, memory_capacity: int | None = None, want_route: bool = False,
                    phases: int = _lib.PREFILL_CHAIN | _lib.PREFILL_ATTENTION, check: bool = False,
                    runner: "PrefillRunner | None" = None, keys_prepared: bool = False) -> PrefillResult:
    """Whole-prompt prefill through ``kvm_prefill_forward``.

    q [B,Hq,T,D], k/v [B,Hkv,T,D], gate [B,Hkv,T,1]; strided views are passed as they are."""
    if q.dim() != 4:
        raise ValueError(f"q must be [B,Hq,T,D], got {tuple(q.shape)}")
    if not q.is_cuda:
        raise RuntimeError("kvm_b200 runs on CUDA tensors only (there is no CPU path)")
    if runner is None:  # (a caller that ran the fused prologue brings the runner whose workspace holds the prepared keys)
        runner = PrefillRunner(params, q.size(0), plan, memory_capacity=memory_capacity, want_route=want_route)
    out = runner.run(q, k, v, gate, phases=phases, keys_prepared=keys_prepared)
    if check:
        runner.check_status()
    # buffers are released by the caching allocator in stream order
    return PrefillResult(out, runner.memory, plan, runner.route, runner)


# ------------------------------------------------------------------------------------ decode cache

class KvmDecodeCache:
    """Device-resident decode state of one layer for ``batch`` sequences with ragged lengths.

    Replaces the reference's ``TritonKVMDecodeCache`` (model/kvm_triton_decode.py:34-400): preallocated
    memory rows, a ring of the last ``W*C`` tokens (token t at slot ``t mod W*C``) and per-sequence
    lengths on the device; ``logical_state_dict`` returns the reference's eager cache layout."""

    cache_representation = "preallocated memory rows + W*C-token ring, per-sequence lengths on device"

    def __init__(self, params: LayerParams, batch: int, state_capacity: int,
                 desired_state_len: Callable[[int, int, int], int], owner: Any = None):
        cfg = params.cfg
        self.params, self.cfg, self.batch, self.owner = params, cfg, int(batch), owner
        self.desired_state_len = desired_state_len
        dev = params.device
        self.device = dev
        self.kv_rows = batch * cfg.n_kv_heads
        self.ring_capacity = cfg.n_bswa_chunks * cfg.chunk_len
        self.memory = MemoryBuffers(self.kv_rows, max(int(state_capacity), 1), cfg.head_dim, dev)
        kw = dict(device=dev, dtype=torch.bfloat16)
        self.ring_k = torch.zeros(self.kv_rows, self.ring_capacity, cfg.head_dim, **kw)
        self.ring_v = torch.zeros(self.kv_rows, self.ring_capacity, cfg.head_dim, **kw)
        self.ring_gate = torch.zeros(self.kv_rows, self.ring_capacity, **kw)
        self.total_len = torch.zeros(batch, device=dev, dtype=torch.int32)
        self.state_len = torch.zeros(batch, device=dev, dtype=torch.int32)
        self.total_len_h = np.zeros(batch, dtype=np.int64)
        self.state_len_h = np.zeros(batch, dtype=np.int64)
        self.update_count = 0
        self.out = torch.empty(batch, 1, cfg.n_q_heads * cfg.head_dim, **kw)
        self.route = None
        self._last_any_update, self._last_n_append = False, None
        self._n_append = torch.full((batch,), -1, device=dev, dtype=torch.int32)
        # host staging of the per-step append counts: a small ring of pinned buffers, each guarded by an event
        # recorded behind its copy, so that a later step never overwrites a buffer the copy engine still reads
        self._n_append_pinned = [torch.full((batch,), -1, dtype=torch.int32).pin_memory() for _ in range(4)]
        self._n_append_events = [None] * 4
        self._n_append_slot = 0
        self._alloc_workspace()

    def _alloc_workspace(self):
        lib = _lib.load()
        self._max_rows_bound = self.memory.capacity + self.ring_capacity
        self._ws_bytes = lib.kvm_decode_workspace_bytes(C.byref(self.params.c), self.batch, self._max_rows_bound)
        # the counter region at the head of the workspace must start at zero; the kernels leave it zero
        self._ws = torch.zeros(self._ws_bytes, device=self.device, dtype=torch.uint8)

    # -- construction ---------------------------------------------------------------------------
    def load_sequence(self, b: int, *, k_sum, v_sum, vlen, window_k, window_v, window_gate, total_len: int,
                      k_attn=None, v_attn=None):
        """Install the state of sequence ``b``: memory rows [Hkv,S,D] (+vlen [Hkv,S]) and the window
        tokens [Hkv,R,D] which are the last R tokens of a sequence of ``total_len`` tokens."""
        cfg = self.cfg
        Hkv, S = k_sum.shape[0], k_sum.shape[1]
        R = window_k.shape[1]
        if S > self.memory.capacity:
            self._reserve(S)
        rows = slice(b * Hkv, (b + 1) * Hkv)
        self.memory.k_sum[rows, :S].copy_(k_sum)
        self.memory.v_sum[rows, :S].copy_(v_sum)
        self.memory.vlen[rows, :S].copy_(vlen.reshape(Hkv, S).float())
        if k_attn is not None:
            self.memory.k_attn[rows, :S].copy_(k_attn)
            self.memory.v_attn[rows, :S].copy_(v_attn)
        begin = total_len - R
        if begin != bswa_begin_for_total_len(total_len, cfg.chunk_len, cfg.n_bswa_chunks):
            raise AssertionError("window tensors do not match the block sliding window of this length")
        slots = (torch.arange(begin, total_len, device=self.device) % self.ring_capacity)
        self.ring_k[rows].index_copy_(1, slots, window_k.to(self.device, torch.bfloat16))
        self.ring_v[rows].index_copy_(1, slots, window_v.to(self.device, torch.bfloat16))
        self.ring_gate[rows].index_copy_(1, slots, window_gate.reshape(Hkv, R).to(self.device, torch.bfloat16))
        self.total_len_h[b] = total_len
        self.state_len_h[b] = S

    def commit_lengths(self, refresh_attention_view: bool = False):
        """Upload the host-side lengths after ``load_sequence`` calls; optionally rebuild
        ``k_attn`` / ``v_attn`` from the carried sums (when those were not supplied)."""
        self.total_len.copy_(torch.from_numpy(self.total_len_h.astype(np.int32)))
        self.state_len.copy_(torch.from_numpy(self.state_len_h.astype(np.int32)))
        if refresh_attention_view:
            rc = _lib.load().kvm_memory_refresh(C.byref(self.params.c), self.batch, self.memory.c(),
                                                self.state_len.data_ptr(), _stream_ptr(self.device))
            _lib.check(rc)

    def _reserve(self, required: int):
        if required <= self.memory.capacity:
            return
        new_cap = max(required, int(self.memory.capacity * 1.5) + self.cfg.chunk_len)
        self.memory = self.memory.grown(new_cap)
        self._alloc_workspace()

    # -- schedule -------------------------------------------------------------------------------
    def _plan_step(self):
        """Host bookkeeping of one token: which sequences run a memory update and how many rows it
        appends (reference: model/kvm_mixer.py:617-669).  Returns (n_append array or None, max_rows)."""
        cfg = self.cfg
        Cn, W = cfg.chunk_len, cfg.n_bswa_chunks
        tl, sl = self.total_len_h, self.state_len_h
        cross = (tl % Cn == 0) & (tl // Cn > W)
        n_app = None
        if cross.any():
            n_app = np.full(self.batch, -1, dtype=np.int32)
            for b in np.nonzero(cross)[0]:
                cov = int(tl[b]) - W * Cn          # coverage before this step
                cur = int(sl[b])
                desired = int(self.desired_state_len(W * Cn + cov, cov + Cn, cur))
                na = min(max(desired - cur, 0), Cn)
                if cur + na <= min(cfg.sink_len, cur + na) and na < Cn:
                    raise AssertionError("KVM state update requires at least one non-sink slot before merging.")
                n_app[b] = na
                sl[b] = cur + na
            self.update_count += int(cross.sum())
        direct = (tl < Cn) & (sl == tl)
        sl[direct] += 1
        tl += 1
        begin = np.maximum(0, ((tl + Cn - 1) // Cn) * Cn - W * Cn)
        rows = np.where(begin > 0, sl, 0) + (tl - begin)
        return n_app, int(rows.max())

    # -- one token ------------------------------------------------------------------------------
    def step(self, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, gate: torch.Tensor, *,
             want_route: bool = False) -> torch.Tensor:
        """One decode token for every sequence: q [B,Hq,1,D], k/v [B,Hkv,1,D], gate [B,Hkv,1,1].
        Returns [B,1,Hq*D] (a buffer owned by the cache, overwritten by the next step)."""
        lib = _lib.load()
        cfg = self.cfg
        B = self.batch
        if q.shape != (B, cfg.n_q_heads, 1, cfg.head_dim) or k.shape != (B, cfg.n_kv_heads, 1, cfg.head_dim):
            raise ValueError(f"decode expects one token per sequence, got q {tuple(q.shape)} k {tuple(k.shape)}")
        q, k, v, gate = (_as_bf16_view(t) for t in (q, k, v, gate))
        n_app, max_rows = self._plan_step()
        if int(self.state_len_h.max()) > self.memory.capacity:
            need = int(self.state_len_h.max())
            self._reserve(need)
        any_update = n_app is not None
        self._last_any_update, self._last_n_append = any_update, n_app
        if any_update:
            slot = self._n_append_slot
            self._n_append_slot = (slot + 1) % len(self._n_append_pinned)
            if self._n_append_events[slot] is not None:
                self._n_append_events[slot].synchronize()
            self._n_append_pinned[slot].copy_(torch.from_numpy(n_app))
            self._n_append.copy_(self._n_append_pinned[slot], non_blocking=True)
            ev = self._n_append_events[slot] or torch.cuda.Event()
            ev.record(torch.cuda.current_stream(self.device))
            self._n_append_events[slot] = ev
            if want_route:
                self.route = torch.zeros(self.kv_rows, cfg.chunk_len, device=self.device, dtype=torch.int32)
        ccache = _CCache(self.memory.c(), self.ring_k.data_ptr(), self.ring_v.data_ptr(), self.ring_gate.data_ptr(),
                         self.total_len.data_ptr(), self.state_len.data_ptr())
        rc = lib.kvm_decode_step(
            C.byref(self.params.c), B, ccache, _tensor4(q, "q"), _tensor4(k, "k"), _tensor4(v, "v"),
            _tensor4(gate, "gate"), self._n_append.data_ptr() if any_update else None,
            int((n_app >= 0).sum()) if any_update else 0,
            min(max_rows, self._max_rows_bound), self.out.data_ptr(),
            _ptr(self.route) if (any_update and want_route) else None,
            self._ws.data_ptr(), self._ws_bytes, _stream_ptr(self.device))
        _lib.check(rc)
        return self.out

    def run(self, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, gate: torch.Tensor) -> torch.Tensor:
        """``n`` consecutive decode tokens with inputs already on the device (teacher-forced / synthetic
        decoding): q [n,B,Hq,1,D], k/v [n,B,Hkv,1,D], gate [n,B,Hkv,1,1], contiguous.  Returns [n,B,Hq*D].
        The host walks the per-sequence schedule a piece of 32 tokens at a time and issues one C call per piece, so
        that the device works on one piece while the next is planned."""
        lib = _lib.load()
        cfg, B = self.cfg, self.batch
        n = q.size(0)
        if q.shape != (n, B, cfg.n_q_heads, 1, cfg.head_dim) or k.shape != (n, B, cfg.n_kv_heads, 1, cfg.head_dim):
            raise ValueError(f"run expects [n,B,H,1,D] inputs, got q {tuple(q.shape)} k {tuple(k.shape)}")
        q, k, v, gate = (t.to(torch.bfloat16).contiguous() for t in (q, k, v, gate))
        out = torch.empty(n, B, cfg.n_q_heads * cfg.head_dim, device=self.device, dtype=torch.bfloat16)
        keep = [q, k, v, gate]
        # The schedule is walked and issued in pieces: while the device works on one piece the host plans the next
        # (a walk of all n tokens up front would leave the device idle for its whole duration).
        piece = 32
        for lo in range(0, n, piece):
            m = min(piece, n - lo)
            n_app = np.full((m, B), -1, dtype=np.int32)
            any_upd = (C.c_int32 * m)()
            max_rows = (C.c_int32 * m)()
            for i in range(m):
                na, mr = self._plan_step()
                if na is not None:
                    n_app[i] = na
                    any_upd[i] = int((na >= 0).sum())
                max_rows[i] = min(mr, self.memory.capacity + self.ring_capacity)
            if int(self.state_len_h.max()) > self.memory.capacity:
                self._reserve(int(self.state_len_h.max()))
                bound = self.memory.capacity + self.ring_capacity
                for i in range(m):
                    max_rows[i] = min(max_rows[i], bound)
            n_app_dev = torch.from_numpy(n_app).to(self.device, non_blocking=True) if any(any_upd) else None
            ccache = _CCache(self.memory.c(), self.ring_k.data_ptr(), self.ring_v.data_ptr(), self.ring_gate.data_ptr(),
                             self.total_len.data_ptr(), self.state_len.data_ptr())
            rc = lib.kvm_decode_run(
                C.byref(self.params.c), B, ccache, m, _tensor4(q[lo], "q"), _tensor4(k[lo], "k"), _tensor4(v[lo], "v"),
                _tensor4(gate[lo], "gate"), q.stride(0), k.stride(0), gate.stride(0),
                n_app_dev.data_ptr() if n_app_dev is not None else None, any_upd, max_rows,
                out[lo].data_ptr(), self._ws.data_ptr(), self._ws_bytes, _stream_ptr(self.device))
            _lib.check(rc)
            keep.append(n_app_dev)
        self._keepalive = tuple(keep)
        return out

    def check_status(self) -> None:
        """Synchronise and raise if a decode kernel reported a device-side timeout since the last check."""
        rc = _lib.load().kvm_decode_status(C.byref(self.params.c), self.batch, self._ws.data_ptr(), _stream_ptr(self.device))
        _lib.check(rc)

    # -- inspection -----------------------------------------------------------------------------
    def logical_state_dict(self, b: int | None = None) -> dict[str, Any]:
        """The reference's eager cache entries (model/kvm_mixer.py:501-525).  For a batch with uniform
        lengths ``b`` may be omitted; otherwise the entries of sequence ``b`` are returned with a
        leading batch dimension of 1."""
        cfg = self.cfg
        if b is None:
            if len(set(self.total_len_h.tolist())) != 1 or len(set(self.state_len_h.tolist())) != 1:
                raise ValueError("ragged cache: pass the sequence index")
            seqs = list(range(self.batch))
            b0 = 0
        else:
            seqs = [b]
            b0 = b
        Hkv, D = cfg.n_kv_heads, cfg.head_dim
        total = int(self.total_len_h[b0])
        S = int(self.state_len_h[b0])
        begin = bswa_begin_for_total_len(total, cfg.chunk_len, cfg.n_bswa_chunks)
        coverage = max(min(total, cfg.chunk_len), begin)
        rows = torch.cat([torch.arange(s * Hkv, (s + 1) * Hkv) for s in seqs]).to(self.device)
        slots = torch.arange(begin, total, device=self.device) % self.ring_capacity
        nb = len(seqs)
        return {
            "kvm_s_k": self.memory.k_sum[rows, :S].reshape(nb, Hkv, S, D),
            "kvm_s_v": self.memory.v_sum[rows, :S].reshape(nb, Hkv, S, D),
            "kvm_s_vlen": self.memory.vlen[rows, :S].reshape(nb, Hkv, S, 1),
            "kvm_state_coverage_len": coverage,
            "kvm_bswa_begin": begin,
            "kvm_bswa_k": self.ring_k[rows][:, slots].reshape(nb, Hkv, total - begin, D),
            "kvm_bswa_v": self.ring_v[rows][:, slots].reshape(nb, Hkv, total - begin, D),
            "kvm_bswa_merge_gate": self.ring_gate[rows][:, slots].reshape(nb, Hkv, total - begin, 1),
        }

    def persistent_metadata(self) -> dict[str, Any]:
        return {
            "total_len": self.total_len_h.tolist(),
            "active_state_len": self.state_len_h.tolist(),
            "state_capacity": self.memory.capacity,
            "recent_capacity": self.ring_capacity,
            "update_count": self.update_count,
            "cache_representation": self.cache_representation,
        }


def decode_cache_from_prefill(params: LayerParams, res: PrefillResult, k: torch.Tensor, v: torch.Tensor,
                              gate: torch.Tensor, desired_state_len, owner=None, extra_capacity: int | None = None) -> KvmDecodeCache:
    """Build the decode cache of a batch right after its prefill (uniform lengths)."""
    cfg = params.cfg
    B, Hkv, T, D = k.shape
    plan = res.plan
    S = plan.final_state_len
    extra = cfg.chunk_len if extra_capacity is None else extra_capacity
    cache = KvmDecodeCache(params, B, S + extra, desired_state_len, owner)
    mem = res.memory
    n = min(mem.capacity, cache.memory.capacity)
    for name in ("k_sum", "v_sum", "vlen", "k_attn", "v_attn"):
        getattr(cache.memory, name)[:, :n].copy_(getattr(mem, name)[:, :n])
    bb = plan.bswa_begin
    slots = torch.arange(bb, T, device=k.device) % cache.ring_capacity
    cache.ring_k.index_copy_(1, slots, k[:, :, bb:].reshape(B * Hkv, T - bb, D).to(torch.bfloat16))
    cache.ring_v.index_copy_(1, slots, v[:, :, bb:].reshape(B * Hkv, T - bb, D).to(torch.bfloat16))
    cache.ring_gate.index_copy_(1, slots, gate[:, :, bb:].reshape(B * Hkv, T - bb).to(torch.bfloat16))
    cache.total_len_h[:] = T
    cache.state_len_h[:] = S
    cache.commit_lengths()
    return cache
