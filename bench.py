"""Benchmark of the KVM sequence-mixer hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl b200|reference] [--no-decode]

Workload (N=1): one KVM layer, bf16 prefill, batch 4 x 32768 tokens, 16 heads x 128, block 256,
memory growing by one mean per block (cap 1024) -- the configuration the headline metric
"KVM prefill tok/s @32k" is quoted on.  Synthetic seeded inputs: hidden ~ LayerNorm(N(0,1)), random-init
projection weights (seed 1); the post-QKV tensors are produced once by the mixer's own PyTorch prologue,
the timed step is the operator between the post-QKV tensors and the input of ``c_proj`` (the boundary the
reference's own kernel benchmark times).  For N>1 (torchrun) heads are sharded over the ranks and the
step includes the NCCL all-gather of the mixer outputs.

One JSON line is printed by rank 0:  value = prefill tokens/s (inputs resident in HBM), e2e = the same
through the public operator call with pinned HOST buffers (H2D of q,k,v,gate and D2H of the output inside
the timed region), roofline = block-attention kernel against the measured bf16 tensor peak,
cpu_baseline = the CPU oracle (a port of the reference's eager mixer) on a bounded sample,
decode = decode tokens/s of 64 ragged sequences (the second half of the metric), power_law = the same prefill
with the reference's native 16*sqrt(T) schedule (cap 1024), check = the kernels' status words after the timed
loops and one head of the timed output against the oracle.
"""

from __future__ import annotations

import argparse
import json
import math
import os
import subprocess
import sys
import threading
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

CFG2 = dict(B=4, T=32768, H=16, D=128, C=256, W=2, cap_chunks=4, rope=64, sink=1, hidden=2048)
CFG3 = dict(n_seq=64, ctx_lo=4096, ctx_hi=65536, steps=512, H=16, D=128, C=256, W=2, cap_chunks=4, rope=64, sink=1)
METRIC = "kvm_prefill_tokens_per_s_T32768"
UNIT = "tokens/s"


def _peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return dict(bf16_tflops=float(p["bf16_tflops"]), hbm_gbs=float(p["hbm_gbs"]), source="measured")
    return dict(bf16_tflops=1590.0, hbm_gbs=6650.0, source="fallback")


def plus_one_schedule(max_state_len):
    def desired(ctx_len, available_context, current):
        cur = max(int(current), 0)
        return max(min(cur + 1, max(int(available_context), 0), max_state_len), cur)
    return desired


def attention_pairs(T, C, W, plan):
    """Exact (query, key) pair count of one (batch, head) row: causal front + window + memory."""
    F = min(T, W * C)
    pairs = F * (F + 1) // 2
    for j in range(W, (T + C - 1) // C):
        qb, qe = j * C, min(T, (j + 1) * C)
        n = qe - qb
        bb = max(0, (j + 1 - W) * C)
        S = plan.state_before[j - W] + plan.n_append[j - W]
        pairs += n * (qb - bb) + n * (n + 1) // 2 + n * S
    return pairs


class ClockSampler:
    """Samples SM clock and throttle reasons while the timed region runs: NVML every 5 ms when the
    bindings are importable (read-only queries), else nvidia-smi every 200 ms."""

    Q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")
    MASKS = (("hw_slowdown", 0x8), ("hw_thermal_slowdown", 0x40), ("sw_thermal_slowdown", 0x20), ("sw_power_cap", 0x4))

    def __init__(self, index):
        self.index, self.rows, self._stop = index, [], threading.Event()
        self._nvml = None
        try:
            import pynvml
            pynvml.nvmlInit()
            # torch's device index follows CUDA_VISIBLE_DEVICES: translate to the physical index for NVML
            vis = os.environ.get("CUDA_VISIBLE_DEVICES")
            phys = int(vis.split(",")[index]) if vis and all(x.strip().isdigit() for x in vis.split(",")) else index
            self._handle = pynvml.nvmlDeviceGetHandleByIndex(phys)
            self._nvml = pynvml
        except Exception:
            self._nvml = None
        self._t = threading.Thread(target=self._run, daemon=True)

    def _sample_nvml(self):
        n = self._nvml
        sm = n.nvmlDeviceGetClockInfo(self._handle, n.NVML_CLOCK_SM)
        mx = n.nvmlDeviceGetMaxClockInfo(self._handle, n.NVML_CLOCK_SM)
        try:
            bits = n.nvmlDeviceGetCurrentClocksEventReasons(self._handle)
        except Exception:
            bits = n.nvmlDeviceGetCurrentClocksThrottleReasons(self._handle)
        self.rows.append([str(sm), str(mx)] + ["Active" if bits & m else "Not Active" for _, m in self.MASKS])

    def _run(self):
        while not self._stop.is_set():
            try:
                if self._nvml is not None:
                    self._sample_nvml()
                else:
                    out = subprocess.run(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-i", str(self.index)],
                                         capture_output=True, text=True, timeout=5).stdout.strip()
                    if out:
                        self.rows.append([c.strip() for c in out.split(",")])
            except Exception:
                pass
            self._stop.wait(0.005 if self._nvml is not None else 0.2)

    def __enter__(self):
        self._t.start()
        return self

    def __exit__(self, *a):
        self._stop.set()
        self._t.join(timeout=6)

    def summary(self):
        sm = sorted(int(r[0]) for r in self.rows if r and r[0].isdigit())
        mx = [int(r[1]) for r in self.rows if len(r) > 1 and r[1].isdigit()]
        names = [n for n, _ in self.MASKS]
        reasons = sorted({n for r in self.rows for n, c in zip(names, r[2:6]) if c.lower().startswith("active")})
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": max(mx) if mx else None, "reasons": reasons,
                "samples": len(self.rows), "source": "nvml" if self._nvml is not None else "nvidia-smi"}


# ------------------------------------------------------------------------------------ workload

def make_mixer(cfg, heads, device):
    """The drop-in mixer with random-init weights (seed 1) for `heads` of the layer's heads."""
    import types

    from kvm_paper_b200.mixer import SequenceMixer

    c = types.SimpleNamespace(
        num_attention_heads=heads, num_key_value_heads=None, d_qk_head=None, d_v_head=None, d_head=cfg["D"],
        hidden_size=cfg["hidden"], num_hidden_layers=1, mup_base_dim=768, rope_partial_dim=cfg["rope"],
        use_value_residual=0, kvm_value_residual_mode="rwkv", kvm_token_shift_mode="rwkv", use_tokenshift_att=0,
        kvm_apply_merge_gate_to_initial_state=0, kvm_apply_merge_gate_to_appends=0, kvm_use_merge_gate_keys=1,
        kvm_use_merge_gate_values=1, kvm_use_head_temps=1, kvm_use_vlens=1, sink_len=cfg["sink"], chunk_len=cfg["C"],
        n_max_d_chunks=cfg["cap_chunks"], n_bswa_chunks=cfg["W"], state_budget_mode="fixed", state_growth_factor=1.0,
        state_growth_exponent=0.5, state_round_down=1, state_min_len=cfg["C"], state_saturation_n=None)
    torch.manual_seed(1)
    old = torch.get_default_dtype()
    torch.set_default_dtype(torch.bfloat16)
    try:
        m = SequenceMixer(c, 0)
    finally:
        torch.set_default_dtype(old)
    m._desired_state_len = plus_one_schedule(m.max_state_len)
    return m.to(device).eval()


def rotary_tables(T, D, rope, device):
    freq = (1 / 10000.0) ** torch.linspace(0.0, 1.0, steps=rope // 2, dtype=torch.float32, device=device)
    freq = torch.cat([freq.repeat_interleave(2), freq.new_zeros(D - rope)])
    theta = torch.arange(T, device=device, dtype=torch.float32).view(1, T, 1, 1) * freq.view(1, 1, 1, -1)
    cos, sin = theta.cos().bfloat16(), theta.sin().bfloat16()
    sin[..., 1::2] *= -1
    return cos, sin


def post_qkv_inputs(cfg, heads, head0, device, batch=None, T=None):
    """Seeded synthetic post-QKV tensors for heads [head0, head0+heads) of the layer: the full layer's
    projection weights are drawn with seed 1 and sliced, so every sharding sees the same numbers."""
    B = cfg["B"] if batch is None else batch
    T = cfg["T"] if T is None else T
    full = make_mixer(cfg, cfg["H"], device)
    D = cfg["D"]
    sl = slice(head0 * D, (head0 + heads) * D)
    g = torch.Generator(device=device).manual_seed(1)
    cos, sin = rotary_tables(T, D, cfg["rope"], device)
    qs, ks, vs, gs = [], [], [], []
    with torch.no_grad():
        for b in range(B):  # one batch row at a time keeps the transient projections small
            x = torch.randn(1, T, cfg["hidden"], generator=g, device=device, dtype=torch.float32)
            x = torch.nn.functional.layer_norm(x, (cfg["hidden"],)).bfloat16()
            q = torch.nn.functional.linear(x, full.c_q.weight[sl]).view(1, T, heads, D)
            k = torch.nn.functional.linear(x, full.c_k.weight[sl]).view(1, T, heads, D)
            v = torch.nn.functional.linear(x, full.c_v.weight[sl]).view(1, T, heads, D)
            q, k = full.ln_q(q), full.ln_k(k)
            from kvm_paper_b200.mixer import apply_rotary
            q, k = apply_rotary(q, (cos, sin)), apply_rotary(k, (cos, sin))
            gate = 1.0 + torch.nn.functional.elu(torch.nn.functional.linear(x, full.key_weighting.weight[head0:head0 + heads]))
            qs.append(q); ks.append(k); vs.append(v); gs.append(gate.view(1, T, heads, 1))
    # [B,T,h,D] storage, handed to the operator as the transposed [B,h,T,D] views the mixer produces
    q, k, v, gate = (torch.cat(t, 0) for t in (qs, ks, vs, gs))
    return q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2), gate.transpose(1, 2)


# ------------------------------------------------------------------------------------- b200 arm

def run_b200(args):
    import torch.distributed as dist

    from kvm_paper_b200 import _lib, ops

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        if world == 1 and args.gpus > 1:
            raise SystemExit("launch with torchrun --nproc-per-node N for --gpus N")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        # the output gather runs alone (nothing to overlap it with): let NCCL use more of the GPU than its default
        os.environ.setdefault("NCCL_MIN_NCHANNELS", "64")
        os.environ.setdefault("NCCL_NTHREADS", "512")
        dist.init_process_group("nccl", device_id=dev)
    _lib.load()
    cfg = CFG2
    H, D, B, T, C, W = cfg["H"], cfg["D"], cfg["B"], cfg["T"], cfg["C"], cfg["W"]
    if H % world:
        raise SystemExit(f"{H} heads cannot be sharded over {world} ranks")
    h_loc = H // world
    head0 = rank * h_loc

    if args.decode_only:
        d = run_decode(args, dev, rank, world, _peaks())
        if rank == 0:
            print(json.dumps({"metric": d["metric"], "value": d["value"], "unit": UNIT, "n_gpus": world, "decode": d}))
        return
    mixer = make_mixer(cfg, h_loc, dev)
    q, k, v, gate = post_qkv_inputs(cfg, h_loc, head0, dev)
    plan = mixer.make_prefill_plan(T)
    params = mixer.layer_params(dev)
    runner = ops.PrefillRunner(params, B, plan)
    from kvm_paper_b200 import sharding

    # N > 1: the attention kernel stores every tile of this rank's heads into all ranks' [B,T,H*D] buffers itself (peer
    # stores over NVLink while other tiles are computed); `--nccl-gather` takes the all-gather + head-order copy instead
    gathered = None
    if world > 1 and not args.nccl_gather:
        try:
            gathered = sharding.GatheredPrefillOutput(B, T, cfg["H"], D, dev)
        except Exception as exc:  # no peer access between these GPUs: the collective instead (the line says which ran)
            print(f"[bench] symmetric memory unavailable ({exc}); gathering with NCCL", file=sys.stderr)
        ok_all = torch.tensor([1 if gathered is not None else 0], device=dev)
        dist.all_reduce(ok_all, op=dist.ReduceOp.MIN)  # every rank takes the same route
        if int(ok_all.item()) == 0:
            gathered = None

    def step():
        if gathered is not None:
            return gathered.run(runner, q, k, v, gate)  # [B,T,H*D] on every rank, complete behind a one-word all-reduce
        out = runner.run(q, k, v, gate)
        return sharding.gather_heads(out, world)  # [B,T,H*D] on every rank (NCCL all-gather + the library's head-order copy)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    n_warm = args.warmup if args.prefill_only else max(args.warmup, 3)
    for _ in range(n_warm):
        step()
    barrier()
    ev = [torch.cuda.Event(enable_timing=True) for _ in range(args.steps + 1)]
    with ClockSampler(local) as clocks:
        barrier()
        ev[0].record()
        for i in range(args.steps):
            step()
            ev[i + 1].record()
        barrier()
    total_ms = ev[0].elapsed_time(ev[-1])
    t = torch.tensor([total_ms], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    total_ms = float(t.item())
    ms_per_step = total_ms / args.steps
    value = B * T / (ms_per_step * 1e-3)

    # ---- per-phase kernel times (CUDA events on the launching stream), attention roofline
    def time_phase(phases, reps):
        runner.run(q, k, v, gate, phases=phases)
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(reps):
            runner.run(q, k, v, gate, phases=phases)
        b.record()
        torch.cuda.synchronize()
        return a.elapsed_time(b) / reps

    n_rep = 1 if args.prefill_only else max(3, args.steps // 2)
    chain_ms = time_phase(_lib.PREFILL_CHAIN, n_rep)
    attn_ms = time_phase(_lib.PREFILL_ATTENTION, n_rep)
    runner.run(q, k, v, gate)  # leave a whole prefill in the buffers (the status word belongs to a whole prefill)
    gathered_ok = None
    if gathered is not None:  # the self-gathered output holds this rank's heads exactly as the plain call computes them
        full = step()
        torch.cuda.synchronize()
        gathered_ok = bool(torch.equal(full[:, :, rank * h_loc * D:(rank + 1) * h_loc * D], runner.out))
        if world > 1:
            dist.barrier()
    peaks = _peaks()
    pairs = attention_pairs(T, C, W, plan)
    attn_flops = 4.0 * D * pairs * B * h_loc          # QK^T and PV of this rank's heads
    achieved = attn_flops / (attn_ms * 1e-3) / 1e12
    roofline = {"bound": "tensor", "kernel": "kvm_attn_prefill_tc_kernel", "achieved": round(achieved, 2),
                "peak": peaks["bf16_tflops"], "unit": "TFLOP/s", "frac": round(achieved / peaks["bf16_tflops"], 4),
                "peak_source": peaks["source"], "traffic": _traffic("kvm_attn_prefill_tc_kernel", B * h_loc * T),
                "ms": round(attn_ms, 4), "chain_ms": round(chain_ms, 4),
                "algorithmic_flops": attn_flops}

    # ---- the timed kernels reported nothing, and what they computed is what the oracle computes (one head)
    check = {"prefill_status": "ok"}
    if gathered_ok is not None:
        check["self_gathered_output_equals_local"] = gathered_ok
    try:
        runner.check_status()
    except Exception as exc:  # a bounded device-side wait ran out: the number above is not a measurement
        check["prefill_status"] = str(exc)
    if rank == 0 and not args.no_cpu:
        check["oracle_head0"] = oracle_check(mixer, params, plan, q, k, v, gate, runner.out)

    # ---- the reference's native schedule on the same inputs: 16 * sqrt(context), at most 1024 means
    power_law = None
    if not args.prefill_only:
        power_law = run_power_law(mixer, params, q, k, v, gate, B, T, C, W, D, h_loc, peaks, max(3, args.steps // 2))

    # ---- the fused prologue in front of the operator (token shift, q/k LayerNorm, rotary, gate, prepared keys)
    prologue = None
    if not args.prefill_only:
        prologue = run_prologue(runner, params, q, k, v, gate, B, T, C, D, h_loc, peaks, dev, max(3, args.steps // 2))

    # ---- end to end through the operator call with host buffers
    e2e = None
    if not args.prefill_only:
        hq, hk, hv, hg = (torch.empty(t_.shape, dtype=t_.dtype).pin_memory() for t_ in
                          (q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2), gate.transpose(1, 2)))
        for h_, d_ in ((hq, q), (hk, k), (hv, v), (hg, gate)):
            h_.copy_(d_.transpose(1, 2))
        h_out = torch.empty(B, T, h_loc * D, dtype=torch.bfloat16).pin_memory()
        # the package's host-buffer entry point: copy-in, kernels and copy-out of consecutive sequences overlap
        # sequences per slice: as many as keep every kv row's cluster of 8 CTAs resident (16 kv rows), so that ranks
        # with few heads do not run one chain per sequence
        slice_batch = max(d for d in range(1, B + 1) if B % d == 0 and (d == 1 or d * h_loc <= 16))
        host_prefill = ops.HostPrefill(runner.params, B, plan, slice_batch=slice_batch)

        def e2e_step():
            host_prefill.run(hq, hk, hv, hg, h_out)

        n_e2e = max(2, min(args.steps, 5))
        e2e_step()
        barrier()
        a, b_ = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(n_e2e):
            e2e_step()
        b_.record()
        barrier()
        t2 = torch.tensor([a.elapsed_time(b_) / n_e2e], device=dev, dtype=torch.float64)
        if world > 1:
            dist.all_reduce(t2, op=dist.ReduceOp.MAX)
        h2d = sum(t_.numel() * t_.element_size() for t_ in (hq, hk, hv, hg))
        e2e = {"value": round(B * T / (float(t2.item()) * 1e-3), 1), "unit": UNIT, "ms_per_step": round(float(t2.item()), 3),
               "h2d_bytes_per_step": h2d * world, "d2h_bytes_per_step": h_out.numel() * 2 * world,
               "sequences_per_slice": slice_batch}
        del hq, hk, hv, hg, h_out, host_prefill

    del runner, q, k, v, gate
    torch.cuda.empty_cache()
    decode = None if args.no_decode else run_decode(args, dev, rank, world, peaks)

    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu:
        cpu = cpu_baseline(cfg, seconds_hint=20, eager_gpu_too=True)

    if rank == 0:
        line = {
            "metric": METRIC, "value": round(value, 1), "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": n_warm, "ms_per_step": round(ms_per_step, 4), "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": ("BASELINE configs[1]: single KVM layer bf16 prefill, B4 x T32768, 16 heads x 128, "
                                    "block 256, +1 mean per block (cap 1024), post-QKV operator boundary")
                       if (B, T) == (4, 32768) else f"REDUCED profiling case of configs[1]: B{B} x T{T}",
                       "global_batch": B, "seq_len": T, "heads_per_gpu": h_loc,
                       "parallelism": f"heads/{world}" + ("" if world == 1 else (" + all-gather of outputs" if gathered is None else
                                                                                 " + outputs stored into every rank's buffer by the attention kernel (peer stores)")),
                       "l2": "inputs (1.6 GB) larger than L2, no flush needed"},
            # per step: prepared + gated keys, chain (routing and keys), value deltas, value rows, block attention
            "e2e": e2e, "gpu_launches": 5 * args.steps,
            "roofline": roofline, "cpu_baseline": cpu,
            "clocks": clocks.summary(), "decode": decode, "power_law": power_law, "prologue": prologue, "check": check,
        }
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


def oracle_check(mixer, params, plan, q, k, v, gate, out):
    """Batch row 0, head 0 of the timed configuration against the CPU oracle: the device prefill is repeated once
    with its routing decisions recorded (it must give the timed output bit for bit), the oracle follows those
    decisions after classifying them, activations are compared."""
    from kvm_paper_b200 import ops
    from oracle import kvm_oracle as ko
    from tests import gpu_helpers as gh

    cfg = params.cfg
    D = cfg.head_dim
    one = ops.LayerConfig(1, 1, D, cfg.chunk_len, cfg.n_bswa_chunks, cfg.rope_dim, cfg.sink_len, cfg.gate_keys,
                          cfg.gate_values, cfg.gate_appends, cfg.gate_initial, cfg.ln_eps)
    p1 = ops.LayerParams(one, params.ln_w, params.ln_b, params.front[:1], params.state[:1], params.device)
    sl = [t[:1, :1] for t in (q, k, v, gate)]
    res = ops.prefill_forward(p1, *sl, plan, want_route=True, check=True)
    same_bits = bool(torch.equal(res.out[0, :, :D], out[0, :, :D]))
    spec = ko.KvmSpec(1, 1, D, D, cfg.rope_dim, cfg.chunk_len, cfg.n_bswa_chunks, mixer.n_max_d_chunks, cfg.sink_len, "plus_one",
                      state_min_len=cfg.chunk_len, ln_weight=params.ln_w.cpu().bfloat16(), ln_bias=params.ln_b.cpu().bfloat16(),
                      front_head_temp=params.front[:1].cpu().bfloat16(), state_head_temp=params.state[:1].cpu().bfloat16())
    forced = [gh.decisions_from_route(res.route[:, u], 1, 1) for u in range(1, plan.n_updates + 1)]
    trace = []
    with torch.no_grad():
        y, _ = ko.prefill(spec, *(t.cpu() for t in sl), trace=trace, forced=forced)
    summ = gh.summarize(trace)
    d = (res.out.float().cpu() - y.float()).abs()
    return {"same_bits_as_timed_output": same_bits, "max_abs": round(float(d.max()), 5),
            "mean_rel": round(float(d.mean() / y.float().abs().mean()), 5), "merge_decisions": summ["merge_tokens"],
            "merge_differ": summ["merge_differ"], "merge_illegal": summ["merge_illegal"],
            "append_rows_illegal": summ["append_rows_illegal"],
            "ok": bool(same_bits and float(d.max()) <= 2e-2 and summ["merge_illegal"] == 0 and summ["append_rows_illegal"] == 0)}


def run_prologue(runner, params, q, k, v, gate, B, T, C, D, h_loc, peaks, dev, reps):
    """The one-kernel prologue on synthetic projection outputs of the bench shape, alone and in front of the prefill
    that then skips its own pass over the keys (HBM-bound: every tensor is read once and written once)."""
    from kvm_paper_b200 import _lib, ops
    g = torch.Generator(device=dev).manual_seed(5)
    mk = lambda *shape: torch.randn(*shape, device=dev, generator=g).to(torch.bfloat16)  # noqa: E731
    q_lin, k_lin, v_lin, g_lin = mk(B, T, h_loc * D), mk(B, T, h_loc * D), mk(B, T, h_loc * D), mk(B, T, h_loc)

    class _LN:
        weight, bias = torch.ones(D) + 0.1 * torch.randn(D), 0.05 * torch.randn(D)

    pro = ops.PrologueParams(dev, shift_q=0.3 * torch.rand(h_loc * D), shift_k=0.3 * torch.rand(h_loc * D),
                             shift_v=0.3 * torch.rand(h_loc * D), ln_q=_LN, ln_k=_LN)
    rot = rotary_tables(T, D, params.cfg.rope_dim, dev)
    rot = tuple(t.reshape(1, T, D).to(torch.bfloat16) for t in rot)

    def timed(fn):
        fn()
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(reps):
            fn()
        b.record()
        torch.cuda.synchronize()
        return a.elapsed_time(b) / reps

    res = {}
    bufs = (torch.empty(B, T, h_loc, D, device=dev, dtype=torch.bfloat16), torch.empty(B, T, h_loc, D, device=dev, dtype=torch.bfloat16),
            torch.empty(B, T, h_loc, D, device=dev, dtype=torch.bfloat16), torch.empty(B, h_loc, T, device=dev, dtype=torch.bfloat16))

    def pro_only():
        res["t"] = ops.prologue_forward(params, pro, q_lin, k_lin, v_lin, g_lin, rot, runner=runner, out=bufs)

    ms = timed(pro_only)
    pq, pk_, pv, pg = res["t"]
    fused_ms = timed(lambda: (pro_only(), runner.run(pq, pk_, pv, pg, keys_prepared=True)))
    chain_prepared_ms = timed(lambda: runner.run(pq, pk_, pv, pg, phases=_lib.PREFILL_CHAIN, keys_prepared=True))
    chain_plain_ms = timed(lambda: runner.run(pq, pk_, pv, pg, phases=_lib.PREFILL_CHAIN))
    n_tok = (runner.plan.n_updates + 1) * C if runner.plan.n_updates > 0 else 0
    rows = B * h_loc
    nbytes = 2 * (3 * B * T * h_loc * D * 2) + 2 * rows * n_tok * D * 2 + 2 * B * T * h_loc * 2
    runner.run(q, k, v, gate)  # the bench inputs' prefill back in the buffers
    return {"kernel": "kvm_prologue_kernel", "ms": round(ms, 4), "algorithmic_bytes": nbytes,
            "achieved": round(nbytes / (ms * 1e-3) / 1e9, 1), "unit": "GB/s", "peak": peaks["hbm_gbs"],
            "frac": round(nbytes / (ms * 1e-3) / 1e9 / peaks["hbm_gbs"], 4),
            "chain_ms_keys_prepared": round(chain_prepared_ms, 4), "chain_ms_own_pass": round(chain_plain_ms, 4),
            "prologue_plus_prefill_ms": round(fused_ms, 4),
            "inputs": "synthetic projection outputs (randn bf16), token shift + LayerNorm + rotary + gate all on"}


def run_power_law(mixer, params, q, k, v, gate, B, T, C, W, D, h_loc, peaks, reps):
    """Prefill tokens/s with the reference's native schedule (power_law, factor 16, exponent 0.5, cap 1024 means)."""
    import math as _m

    from kvm_paper_b200 import _lib, ops

    cap = mixer.max_state_len

    def desired(ctx_len, available_context, current):
        target = max(int(_m.floor(16.0 * (float(max(int(ctx_len), 0)) ** 0.5))), C)
        return max(min(target, max(int(available_context), 0), cap), max(int(current), 0))

    plan = ops.build_prefill_plan(T, C, W, desired)
    runner = ops.PrefillRunner(params, B, plan)

    def timed(phases):
        runner.run(q, k, v, gate, phases=phases)
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(reps):
            runner.run(q, k, v, gate, phases=phases)
        b.record()
        torch.cuda.synchronize()
        return a.elapsed_time(b) / reps

    total = timed(_lib.PREFILL_CHAIN | _lib.PREFILL_ATTENTION)
    chain = timed(_lib.PREFILL_CHAIN)
    attn = timed(_lib.PREFILL_ATTENTION)
    status = "ok"
    try:
        runner.run(q, k, v, gate)
        runner.check_status()
    except Exception as exc:
        status = str(exc)
    flops = 4.0 * D * attention_pairs(T, C, W, plan) * B * h_loc
    tf = flops / (attn * 1e-3) / 1e12
    return {"schedule": "power_law 16*sqrt(context), cap 1024 means", "final_means": plan.final_state_len,
            "max_appends_per_block": max(plan.n_append[1:]), "value": round(B * T / (total * 1e-3), 1), "unit": UNIT,
            "ms_per_step": round(total, 4), "chain_ms": round(chain, 4), "attention_ms": round(attn, 4),
            "attention_tflops": round(tf, 1), "attention_frac": round(tf / peaks["bf16_tflops"], 4),
            "algorithmic_flops": flops, "status": status}


def run_long_context(args):
    """`--long-context`: BASELINE configs[4] (not the default line): batch 1, T = 262144, 32 heads x 128, blocks of 512
    tokens, power-law memory 16*sqrt(context) capped at 4096 means, keys from a seeded mixture of 64 Gaussian clusters;
    heads sharded over the ranks, outputs gathered.  Blocks of 512 tokens take the general chain kernel."""
    import math as _m

    import torch.distributed as dist

    from kvm_paper_b200 import _lib, ops, sharding
    rank, world, local = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1)), int(os.environ.get("LOCAL_RANK", 0))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        os.environ.setdefault("NCCL_MIN_NCHANNELS", "64")
        os.environ.setdefault("NCCL_NTHREADS", "512")
        dist.init_process_group("nccl", device_id=dev)
    H, D, C, W, T, cap = 32, 128, 512, 2, 262144 if args.seq_len is None else args.seq_len, 4096
    h_loc = H // world
    cfg = ops.LayerConfig(n_q_heads=h_loc, n_kv_heads=h_loc, head_dim=D, chunk_len=C, n_bswa_chunks=W, rope_dim=64, sink_len=1)
    g0 = torch.Generator().manual_seed(4)
    params = ops.LayerParams(cfg, 1.0 + 0.1 * torch.randn(D, generator=g0), 0.05 * torch.randn(D, generator=g0), None, None, dev)

    def desired(ctx_len, available_context, current):
        target = max(int(_m.floor(16.0 * (float(max(int(ctx_len), 0)) ** 0.5))), C)
        return max(min(target, max(int(available_context), 0), cap), max(int(current), 0))

    plan = ops.build_prefill_plan(T, C, W, desired)
    g = torch.Generator(device=dev).manual_seed(40)          # the same cluster centres on every rank,
    centers = torch.randn(64, D, generator=g, device=dev)
    g = torch.Generator(device=dev).manual_seed(41 + rank)   # this rank's heads
    ln = torch.nn.functional.layer_norm
    which = torch.randint(0, 64, (1, T, h_loc), generator=g, device=dev)
    k = ln(centers[which] + 0.5 * torch.randn(1, T, h_loc, D, generator=g, device=dev), (D,)).bfloat16().transpose(1, 2)
    del which
    q = ln(torch.randn(1, T, h_loc, D, generator=g, device=dev), (D,)).bfloat16().transpose(1, 2)
    v = torch.randn(1, T, h_loc, D, generator=g, device=dev).bfloat16().transpose(1, 2)
    gate = (1 + torch.nn.functional.elu(0.5 * torch.randn(1, T, h_loc, 1, generator=g, device=dev))).bfloat16().transpose(1, 2)
    runner = ops.PrefillRunner(params, 1, plan)
    gathered = sharding.GatheredPrefillOutput(1, T, H, D, dev) if world > 1 and not args.nccl_gather else None

    def step():
        if gathered is not None:
            return gathered.run(runner, q, k, v, gate)
        return sharding.gather_heads(runner.run(q, k, v, gate), world)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(max(args.warmup, 3)):
        step()
    barrier()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with ClockSampler(local) as clocks:
        barrier()
        a.record()
        for _ in range(args.steps):
            step()
        b.record()
        barrier()
    t = torch.tensor([a.elapsed_time(b) / args.steps], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms = float(t.item())

    def timed(phases):
        runner.run(q, k, v, gate, phases=phases)
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        runner.run(q, k, v, gate, phases=phases)
        b.record()
        torch.cuda.synchronize()
        return a.elapsed_time(b)

    chain_ms, attn_ms = timed(_lib.PREFILL_CHAIN), timed(_lib.PREFILL_ATTENTION)
    runner.run(q, k, v, gate)
    status = "ok"
    try:
        runner.check_status()
    except Exception as exc:
        status = str(exc)
    peaks = _peaks()
    flops = 4.0 * D * attention_pairs(T, C, W, plan) * h_loc
    tf = flops / (attn_ms * 1e-3) / 1e12
    if rank == 0:
        print(json.dumps({
            "metric": f"kvm_prefill_tokens_per_s_T{T}", "value": round(T / (ms * 1e-3), 1), "unit": UNIT, "n_gpus": world,
            "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": round(ms, 3), "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": "BASELINE configs[4]: long-context KVM layer, B1 x T262144, 32 heads x 128, block 512, power-law "
                                   "memory capped at 4096 means, keys from 64 Gaussian clusters, post-QKV operator boundary",
                       "seq_len": T, "heads_per_gpu": h_loc, "parallelism": f"heads/{world}" + ("" if world == 1 else (" + all-gather of outputs" if gathered is None else
                                                                                 " + outputs stored into every rank's buffer by the attention kernel (peer stores)")),
                       "final_means": plan.final_state_len, "updates": plan.n_updates,
                       "chain_kernel": "general chain kernel (blocks of 512 tokens)"},
            "chain_ms": round(chain_ms, 3), "attention_ms": round(attn_ms, 3), "attention_tflops": round(tf, 1),
            "attention_frac": round(tf / peaks["bf16_tflops"], 4), "status": status, "clocks": clocks.summary()}))
    if world > 1:
        dist.destroy_process_group()


# DRAM traffic of the dominant kernels from ncu captures (dram__bytes_read.sum + dram__bytes_write.sum of one
# launch), scaled to this run's launch by the units it processes; the captures and their commands are the
# summaries under profiles/ named after these kernels.
NCU_TRAFFIC = {
    # B1 x T16384 x 16 heads: 289.0 MB + 50.9 MB per launch -> bytes per (head, token)
    "kvm_attn_prefill_tc_kernel": (289.0e6 + 50.9e6) / (16 * 16384),
    # decode workload of this bench: 399.0 MB + 3.6 MB per launch for 397 MB of algorithmic K/V rows
    "kvm_decode_attn_kernel": (399.0e6 + 3.6e6) / 397.0e6,
}


def _traffic(kernel, units):
    """DRAM bytes per launch: ncu bytes per unit (see NCU_TRAFFIC) x the units of one launch."""
    return round(NCU_TRAFFIC[kernel] * units) if kernel in NCU_TRAFFIC else None


def run_decode(args, dev, rank, world, peaks):
    """Decode tokens/s of 64 sequences with ragged prefilled contexts, sequences sharded over ranks."""
    import numpy as np
    import torch.distributed as dist

    from kvm_paper_b200 import ops

    c = CFG3
    n_loc = c["n_seq"] // world
    rng = np.random.RandomState(3)
    ctx = rng.randint(c["ctx_lo"], c["ctx_hi"] + 1, size=c["n_seq"])
    mine = ctx[rank * n_loc:(rank + 1) * n_loc]
    cfgm = dict(CFG2, H=c["H"])
    mixer = make_mixer(cfgm, c["H"], dev)
    params = mixer.layer_params(dev)
    H, D, C, W = c["H"], c["D"], c["C"], c["W"]
    steps = c["steps"] if args.decode_steps is None else args.decode_steps
    cache = ops.KvmDecodeCache(params, n_loc, 1024 + C, mixer._desired_state_len)
    gen = torch.Generator(device=dev).manual_seed(3 + rank)
    for b, T in enumerate(mine.tolist()):
        # state built by a seeded chain-only prefill of this sequence's context
        k = torch.nn.functional.layer_norm(torch.randn(1, T, H, D, generator=gen, device=dev), (D,)).bfloat16().transpose(1, 2)
        v = torch.randn(1, T, H, D, generator=gen, device=dev).bfloat16().transpose(1, 2)
        g = (1 + torch.nn.functional.elu(torch.randn(1, T, H, 1, generator=gen, device=dev))).bfloat16().transpose(1, 2)
        plan = ops.build_prefill_plan(T, C, W, mixer._desired_state_len, keep_versions=False)
        r = ops.PrefillRunner(params, 1, plan)
        r.run(k, k, v, g, phases=1)
        S, bb = plan.final_state_len, plan.bswa_begin
        m = r.memory
        cache.load_sequence(b, k_sum=m.k_sum[:, :S], v_sum=m.v_sum[:, :S], vlen=m.vlen[:, :S], k_attn=m.k_attn[:, :S],
                            v_attn=m.v_attn[:, :S], window_k=k[0, :, bb:], window_v=v[0, :, bb:], window_gate=g[0, :, bb:],
                            total_len=T)
        del r, k, v, g
    cache.commit_lengths()
    q = torch.randn(steps, n_loc, H, 1, D, generator=gen, device=dev).bfloat16()
    k = torch.nn.functional.layer_norm(torch.randn(steps, n_loc, H, 1, D, generator=gen, device=dev), (D,)).bfloat16()
    v = torch.randn(steps, n_loc, H, 1, D, generator=gen, device=dev).bfloat16()
    g = (1 + torch.nn.functional.elu(torch.randn(steps, n_loc, H, 1, 1, generator=gen, device=dev))).bfloat16()
    from kvm_paper_b200 import sharding
    # algorithmic bytes of the timed steps: memory + window rows of every sequence, K and V, bf16
    tl, sl = cache.total_len_h.copy(), cache.state_len_h.copy()
    snap = (cache.memory.k_sum.clone(), cache.memory.v_sum.clone(), cache.memory.vlen.clone(), cache.memory.k_attn.clone(),
            cache.memory.v_attn.clone(), cache.ring_k.clone(), cache.ring_v.clone(), cache.ring_gate.clone())

    def restore():
        for dst, src in zip((cache.memory.k_sum, cache.memory.v_sum, cache.memory.vlen, cache.memory.k_attn,
                             cache.memory.v_attn, cache.ring_k, cache.ring_v, cache.ring_gate), snap):
            dst.copy_(src)
        cache.total_len_h[:] = tl
        cache.state_len_h[:] = sl
        cache.commit_lengths()

    def host_walk():
        """Algorithmic K/V bytes of the timed steps (memory + window rows of every sequence, bf16), from a
        host-only walk of the per-sequence schedule."""
        import copy
        fake = copy.copy(cache)
        fake.total_len_h, fake.state_len_h = cache.total_len_h.copy(), cache.state_len_h.copy()
        fake.update_count = 0
        nbytes = 0
        for _ in range(steps):
            fake._plan_step()
            begin = np.maximum(0, ((fake.total_len_h + C - 1) // C) * C - W * C)
            rows = np.where(begin > 0, fake.state_len_h, 0) + (fake.total_len_h - begin)
            nbytes += int(rows.sum()) * H * 2 * D * 2
        return nbytes

    nbytes = host_walk()

    def run_all():
        out = cache.run(q, k, v, g)       # one C call per 32 tokens: two kernel launches per token
        return sharding.gather_sequences(out, world, seq_dim=1)  # [steps, all sequences, H*D]

    run_all()  # warm-up pass over the whole trajectory
    restore()
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    a, b_ = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0 = time.perf_counter()
    a.record()
    run_all()
    b_.record()
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    wall = time.perf_counter() - t0
    t = torch.tensor([a.elapsed_time(b_)], device=dev, dtype=torch.float64)
    nb = torch.tensor([float(nbytes)], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        dist.all_reduce(nb, op=dist.ReduceOp.SUM)
    ms = float(t.item())
    gbs = float(nb.item()) / world / (ms * 1e-3) / 1e9  # per GPU
    status = "ok"
    try:
        cache.check_status()
    except Exception as exc:
        status = str(exc)
    n_memory_updates = int(cache.update_count)
    # the drop-in route: one call of KvmDecodeCache.step per token (what forward_single does), host bookkeeping,
    # pinned copy and ctypes call included
    restore()
    n_api = min(steps, 256)
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    for i in range(n_api):
        cache.step(q[i], k[i], v[i], g[i])
    torch.cuda.synchronize()
    api_ms = (time.perf_counter() - t0) * 1e3 / n_api
    return {"metric": "kvm_decode_tokens_per_s", "value": round(c["n_seq"] * steps / (ms * 1e-3), 1), "unit": UNIT,
            "sequences": c["n_seq"], "steps": steps, "ms_per_step": round(ms / steps, 4),
            "host_wall_ms_per_step": round(wall * 1e3 / steps, 4), "memory_updates": n_memory_updates,
            "status": status, "step_api_ms_per_token": round(api_ms, 4),
            "step_api_tokens_per_s": round(n_loc * world / (api_ms * 1e-3), 1),
            "workload": "BASELINE configs[2]: 64 ragged sequences, contexts U[4096,65536] (seed 3), 16 heads x 128, "
                        "block 256, +1 mean per block; sequences sharded over ranks",
            "roofline": {"bound": "hbm", "kernel": "kvm_decode_attn_kernel", "achieved": round(gbs, 1),
                         "peak": peaks["hbm_gbs"], "unit": "GB/s", "frac": round(gbs / peaks["hbm_gbs"], 4),
                         "peak_source": peaks["source"],
                         "traffic": _traffic("kvm_decode_attn_kernel", float(nb.item()) / world / steps),
                         "note": "algorithmic K/V bytes of all steps / whole-step device time (ring write, boundary updates "
                                 "and combine included); achieved, traffic per token"}}


# ------------------------------------------------------------------------------------ CPU oracle

def cpu_baseline(cfg, seconds_hint=20, heads=4, T=None, eager_gpu_too=False):
    """The CPU oracle (port of the reference's eager mixer) on a bounded sample of the prefill workload:
    batch 1, `heads` of the 16 heads, full length; throughput scaled by heads/16 (work is linear in heads)."""
    from oracle import kvm_oracle as ko

    T = cfg["T"] if T is None else T
    D = cfg["D"]
    threads = os.cpu_count() or 1
    torch.set_num_threads(threads)
    spec = ko.KvmSpec(heads, heads, D, D, cfg["rope"], cfg["C"], cfg["W"], cfg["cap_chunks"], cfg["sink"], "plus_one",
                      state_min_len=cfg["C"])
    g = torch.Generator().manual_seed(1)
    q = torch.nn.functional.layer_norm(torch.randn(1, T, heads, D, generator=g), (D,)).bfloat16().transpose(1, 2)
    k = torch.nn.functional.layer_norm(torch.randn(1, T, heads, D, generator=g), (D,)).bfloat16().transpose(1, 2)
    v = torch.randn(1, T, heads, D, generator=g).bfloat16().transpose(1, 2)
    gate = (1 + torch.nn.functional.elu(torch.randn(1, T, heads, 1, generator=g))).bfloat16().transpose(1, 2)
    times = []
    with torch.no_grad():
        t0 = time.perf_counter()
        ko.prefill(spec, q, k, v, gate)
        first = time.perf_counter() - t0
        reps = max(1, min(5, int(seconds_hint / max(first, 1e-3)) - 1))
        for _ in range(reps):
            t0 = time.perf_counter()
            ko.prefill(spec, q, k, v, gate)
            times.append(time.perf_counter() - t0)
    best = sorted(times)[len(times) // 2] if times else first
    value = T * (heads / cfg["H"]) / cfg["B"] * cfg["B"] / best  # layer-equivalent tokens/s for one batch row stream
    eager_gpu = None
    if eager_gpu_too and torch.cuda.is_available():
        # the same port with its tensors on the GPU: what the reference's eager (non-Triton) mixer costs on this B200
        # (one PyTorch launch per operation of every block), on the whole workload
        dev = torch.device("cuda", torch.cuda.current_device())
        spec_f = ko.KvmSpec(cfg["H"], cfg["H"], D, D, cfg["rope"], cfg["C"], cfg["W"], cfg["cap_chunks"], cfg["sink"], "plus_one",
                            state_min_len=cfg["C"])
        gg = torch.Generator(device=dev).manual_seed(1)
        mk = lambda *shape: torch.randn(*shape, generator=gg, device=dev)  # noqa: E731
        Bf, Hf = cfg["B"], cfg["H"]
        qg = torch.nn.functional.layer_norm(mk(Bf, T, Hf, D), (D,)).bfloat16().transpose(1, 2)
        kg = torch.nn.functional.layer_norm(mk(Bf, T, Hf, D), (D,)).bfloat16().transpose(1, 2)
        vg = mk(Bf, T, Hf, D).bfloat16().transpose(1, 2)
        gateg = (1 + torch.nn.functional.elu(mk(Bf, T, Hf, 1))).bfloat16().transpose(1, 2)
        tg = []
        with torch.no_grad():
            ko.prefill(spec_f, qg, kg, vg, gateg)
            for _ in range(3):
                torch.cuda.synchronize()
                t0 = time.perf_counter()
                ko.prefill(spec_f, qg, kg, vg, gateg)
                torch.cuda.synchronize()
                tg.append(time.perf_counter() - t0)
        tgm = sorted(tg)[1]
        eager_gpu = {"value": round(Bf * T / tgm, 1), "unit": UNIT, "ms_per_step": round(tgm * 1e3, 2),
                     "sample": f"oracle/kvm_oracle.py prefill with CUDA tensors, the whole workload (B{Bf} x {Hf} heads x T={T}), median of 3"}
        del qg, kg, vg, gateg
        torch.cuda.empty_cache()
    return {"value": round(value, 1), "unit": UNIT, "cores": threads, "kind": "port", "eager_port_on_this_gpu": eager_gpu,
            "sample": f"oracle/kvm_oracle.py prefill, bf16, batch 1 x {heads} of {cfg['H']} heads x T={T}, median of {len(times) or 1} runs "
                      f"({best:.2f} s each); value = T * ({heads}/{cfg['H']}) / time (work is linear in heads and batch)",
            "torch": torch.__version__}


def run_reference(args):
    """Reference arm: the reference's own CPU implementation of the path.  The reference is Python and is
    not present on the benchmark box, so its line-by-line CPU port (oracle/) is what is timed."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    cfg = CFG2
    steps = max(1, min(args.steps, 3))
    cpu = cpu_baseline(cfg, seconds_hint=10 * steps)
    line = {"impl": "reference", "metric": METRIC, "value": cpu["value"], "unit": UNIT, "n_gpus": args.gpus,
            "steps": steps, "warmup": 1, "ms_per_step": None, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": "BASELINE configs[1] (bounded sample, see cpu_baseline.sample)", "global_batch": cfg["B"],
                       "seq_len": cfg["T"], "parallelism": "host CPU threads"},
            "cpu_baseline": cpu,
            "e2e": {"value": cpu["value"], "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--no-decode", action="store_true")
    ap.add_argument("--no-cpu", action="store_true")
    ap.add_argument("--decode-steps", type=int, default=None)
    # smaller cases of the same kernels for profiler captures (the JSON line then names the reduced shape)
    ap.add_argument("--batch", type=int, default=None)
    ap.add_argument("--seq-len", type=int, default=None)
    ap.add_argument("--prefill-only", action="store_true", help="skip e2e, decode and the CPU baseline")
    ap.add_argument("--decode-only", action="store_true", help="run only the decode workload")
    ap.add_argument("--nccl-gather", action="store_true", help="N > 1: gather the outputs with an NCCL all-gather instead of the attention kernel's peer stores")
    ap.add_argument("--long-context", action="store_true", help="BASELINE configs[4] (T=262144, 32 heads, block 512, 4096 means) instead of the default line")
    ap.add_argument("--decode-seqs", type=int, default=None)
    args = ap.parse_args()
    if args.batch is not None:
        CFG2["B"] = args.batch
    if args.seq_len is not None:
        CFG2["T"] = args.seq_len
    if args.decode_seqs is not None:
        CFG3["n_seq"] = args.decode_seqs
    if args.prefill_only:
        args.no_decode = args.no_cpu = True
    if args.impl == "reference":
        run_reference(args)
    elif args.long_context:
        run_long_context(args)
    else:
        run_b200(args)


if __name__ == "__main__":
    main()
