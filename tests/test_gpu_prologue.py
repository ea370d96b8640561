"""The fused prologue kernel (``kvm_prologue_forward``): token shift, q/k LayerNorm, rotary embedding, merge gate and
the prepared keys in one pass over the projection outputs.

Evidence chain: (1) fed with the projection outputs computed on the CPU from the fixtures' weights and hidden inputs
(the same GEMMs the reference ran), the kernel reproduces the post-QKV tensors the reference recorded, bit for bit
except where an fp32 LayerNorm sum lands within rounding distance of a bf16 tie (under one element per thousand, one
or two bf16 steps); the same for cached single-token calls, which shift against the previous call's last token; (2) the
prepared keys it leaves in a prefill workspace are the ones the prefill's own pass writes, bit for bit, and a prefill
that skips that pass returns the same output and memory; (3) the class's fused prefix equals its PyTorch prefix on
the same GPU GEMM outputs up to the same rounding allowance."""

import pytest
import torch

from kvm_paper_b200 import ops
from kvm_paper_b200.mixer import StatesCache
from tests import gpu_helpers as gh
from tests.helpers import load_fixture, mixer_from_fixture, rotary_tables

pytestmark = pytest.mark.gpu

BF16_FIXTURES = ["powerlaw_bf16", "plusone_bf16", "saturation_bf16"]
# elements that may differ from the reference by one bf16 step (fp32 LayerNorm sums are ordered differently)
MAX_OFF_FRACTION = 2e-3


def _assert_bf16_equal_up_to_ties(got: torch.Tensor, want: torch.Tensor, what: str):
    """Equal bits, except for at most MAX_OFF_FRACTION of the elements, and those within two bf16 steps of an O(1)
    value (a LayerNorm output one step off passes through two rounded rotary products)."""
    assert got.shape == want.shape, (what, got.shape, want.shape)
    g, w = got.float().cpu(), want.float().cpu()
    diff = (g - w).abs()
    bound = 2.0 * 2.0 ** -7 * torch.clamp(torch.maximum(g.abs(), w.abs()), min=1.0)
    assert bool((diff <= bound).all()), f"{what}: an element is more than two bf16 steps off (max diff {diff.max().item()})"
    frac = float((diff > 0).float().mean())
    assert frac <= MAX_OFF_FRACTION, f"{what}: {frac:.2e} of the elements differ from the reference"


def _cpu_projections(m, x, vf):
    """c_q, c_k, c_v (+ the pre-shift value residual) and key_weighting on the CPU, as the reference evaluated them."""
    with torch.no_grad():
        q, k, v = m.c_q(x), m.c_k(x), m.c_v(x)
        if m.value_residual_mode == "linear":
            v = (1 - m.lamb) * v + m.lamb * vf.view_as(v)
        elif m.value_residual_mode == "rwkv":
            v = v + (vf.to(v.dtype) - v) * m._value_gate(x).to(v.dtype)
        gated = m.config.kvm_use_merge_gate_keys or m.config.kvm_use_merge_gate_values
        g = m.key_weighting(x) if gated else None
    return q, k, v, g


@pytest.mark.parametrize("name", BF16_FIXTURES)
def test_prologue_kernel_reproduces_the_reference_post_qkv(name):
    fix = load_fixture(name)
    cfg, m = mixer_from_fixture(fix)
    if m.value_residual_mode == "rwkv_post_tokenshift":
        pytest.skip("post-shift value residual is applied by the caller")
    T, B = fix["case"]["T"], fix["case"]["B"]
    x, vf = fix["x"], fix["v_first"]
    dev = torch.device("cuda")
    params, pro = m.layer_params(dev), m.prologue_params(dev)
    q_lin, k_lin, v_lin, g_lin = _cpu_projections(m, x[:, :T], None if vf is None else vf[:, :T])
    pos = torch.arange(T).view(1, T).expand(B, T)
    rot = rotary_tables(cfg, m.d_qk_head, pos)
    q, k, v, g = ops.prologue_forward(params, pro, q_lin.to(dev), k_lin.to(dev), v_lin.to(dev),
                                      None if g_lin is None else g_lin.to(dev), tuple(t.to(dev) for t in rot))
    pq = fix["post_qkv"]
    _assert_bf16_equal_up_to_ties(q, pq["q"], f"{name} q")
    _assert_bf16_equal_up_to_ties(k, pq["k"], f"{name} k")
    assert torch.equal(v.cpu(), pq["v"].to(torch.bfloat16)), f"{name}: values (token shift only) must match bit for bit"
    _assert_bf16_equal_up_to_ties(g, pq["merge_gate"], f"{name} gate")
    # cached single-token calls: the token shift takes the previous call's last projection outputs
    if fix["decode_qkv"] is not None:
        dq, dk, dv, dg = fix["decode_qkv"]
        prev = (q_lin[:, -1:], k_lin[:, -1:], v_lin[:, -1:])
        for i in range(min(4, dq.size(2))):
            xi = x[:, T + i:T + i + 1]
            ql, kl, vl, gl = _cpu_projections(m, xi, None if vf is None else vf[:, T + i:T + i + 1])
            rot = rotary_tables(cfg, m.d_qk_head, torch.full((B, 1), T + i, dtype=torch.long))
            q1, k1, v1, g1 = ops.prologue_forward(params, pro, ql.to(dev), kl.to(dev), vl.to(dev), None if gl is None else gl.to(dev),
                                                  tuple(t.to(dev) for t in rot), prev=tuple(t.to(dev) for t in prev))
            _assert_bf16_equal_up_to_ties(q1, dq[:, :, i:i + 1], f"{name} decode q {i}")
            _assert_bf16_equal_up_to_ties(k1, dk[:, :, i:i + 1], f"{name} decode k {i}")
            assert torch.equal(v1.cpu(), dv[:, :, i:i + 1].to(torch.bfloat16))
            _assert_bf16_equal_up_to_ties(g1, dg[:, :, i:i + 1], f"{name} decode gate {i}")
            prev = (ql, kl, vl)


@pytest.mark.parametrize("D,C,Hq,Hkv,T", [(128, 128, 4, 2, 1000), (128, 256, 2, 2, 1536), (64, 32, 4, 2, 300)])
def test_prefill_with_prepared_keys_equals_the_plain_prefill(D, C, Hq, Hkv, T):
    """The prologue writes the prepared / gated keys into the runner's workspace; the prefill that skips its own pass
    over the keys returns the same bits (tensor-core chain at D = 128, general chain at D = 64)."""
    from oracle import kvm_oracle as ko
    dev = torch.device("cuda")
    B = 2
    spec = ko.KvmSpec(num_attention_heads=Hq, num_key_value_heads=Hkv, d_qk_head=D, d_v_head=D, rope_partial_dim=D // 2,
                      chunk_len=C, n_bswa_chunks=2, n_max_d_chunks=4, sink_len=1, state_budget_mode="power_law",
                      state_growth_factor=6.0, state_min_len=C,
                      ln_weight=1.0 + 0.1 * torch.randn(D, generator=torch.Generator().manual_seed(1)),
                      ln_bias=0.05 * torch.randn(D, generator=torch.Generator().manual_seed(2)))
    params = gh.layer_params(spec, dev)
    g = torch.Generator(device="cpu").manual_seed(7)
    mk = lambda *s: torch.randn(*s, generator=g).to(torch.bfloat16).to(dev)  # noqa: E731
    q_lin, k_lin, v_lin, g_lin = mk(B, T, Hq * D), mk(B, T, Hkv * D), mk(B, T, Hkv * D), mk(B, T, Hkv)

    class _LN:  # the two fields PrologueParams reads
        def __init__(self, seed):
            gg = torch.Generator().manual_seed(seed)
            self.weight = 1.0 + 0.1 * torch.randn(D, generator=gg)
            self.bias = 0.05 * torch.randn(D, generator=gg)

    pro = ops.PrologueParams(dev, shift_q=0.3 * torch.rand(Hq * D, generator=g), shift_k=0.3 * torch.rand(Hkv * D, generator=g),
                             shift_v=0.3 * torch.rand(Hkv * D, generator=g), ln_q=_LN(3), ln_k=_LN(4))
    pos = torch.arange(T).view(1, T)
    cfg = type("Cfg", (), {"rope_partial_dim": D // 2})
    rot = tuple(t.to(dev) for t in rotary_tables(cfg, D, pos))
    plan = ops.build_prefill_plan(T, C, 2, gh.desired_fn(spec))
    fused = ops.PrefillRunner(params, B, plan)
    q, k, v, gate = ops.prologue_forward(params, pro, q_lin, k_lin, v_lin, g_lin, rot, runner=fused)
    out_fused = fused.run(q, k, v, gate, keys_prepared=True).clone()
    fused.check_status()
    plain = ops.PrefillRunner(params, B, plan)
    out_plain = plain.run(q, k, v, gate).clone()
    plain.check_status()
    assert plan.n_updates > 0
    assert torch.equal(fused.workspace_views()["prepared_keys"], plain.workspace_views()["prepared_keys"])
    assert torch.equal(out_fused, out_plain)
    for a, b in ((fused.memory.k_sum, plain.memory.k_sum), (fused.memory.v_sum, plain.memory.v_sum),
                 (fused.memory.k_attn, plain.memory.k_attn), (fused.memory.v_attn, plain.memory.v_attn)):
        assert torch.equal(a, b)


@pytest.mark.parametrize("name", BF16_FIXTURES)
def test_class_fused_prefix_equals_its_pytorch_prefix(name):
    fix = load_fixture(name)
    cfg, m = mixer_from_fixture(fix)
    m = m.cuda()
    T, B = fix["case"]["T"], fix["case"]["B"]
    x = fix["x"][:, :T].cuda()
    vf = None if fix["v_first"] is None else fix["v_first"][:, :T].cuda()
    if not m.fused_prologue_applies(x):
        pytest.skip("fused prologue does not cover this module")
    pos = torch.arange(T).view(1, T).expand(B, T)
    rot = tuple(t.cuda() for t in rotary_tables(cfg, m.d_qk_head, pos))
    with torch.no_grad():
        want = m.forward_prefix(x, vf, rot, None, StatesCache())
        got = m.forward_prefix_fused(x, vf, rot, StatesCache())
    for a, b, what in zip(got, want, ("q", "k", "v", "gate")):
        _assert_bf16_equal_up_to_ties(a, b.to(torch.bfloat16), f"{name} {what}")


@pytest.mark.parametrize("D,Hq,Hkv,T,with_prev,with_shift", [(128, 4, 2, 777, False, True), (128, 2, 2, 1, True, True), (64, 4, 2, 333, True, True),
                                                               (32, 2, 1, 100, False, False)])
def test_prologue_kernel_matches_the_oracle_on_random_inputs(D, Hq, Hkv, T, with_prev, with_shift):
    """Kernel against ``oracle.prologue`` (the reference's own tensor operations on the CPU) on seeded inputs: ragged
    lengths (the last lane groups of the grid run past the end), a cached previous token, per-batch rotary tables."""
    from oracle import kvm_oracle as ko
    dev = torch.device("cuda")
    B = 3
    g = torch.Generator().manual_seed(100 + T)
    rnd = lambda *s: torch.randn(*s, generator=g).to(torch.bfloat16)  # noqa: E731
    q_lin, k_lin, v_lin, g_lin = rnd(B, T, Hq * D), rnd(B, T, Hkv * D), rnd(B, T, Hkv * D), rnd(B, T, Hkv)
    shift = tuple((0.5 * torch.rand(n, generator=g)).to(torch.bfloat16) for n in (Hq * D, Hkv * D, Hkv * D)) if with_shift else None
    prev = (rnd(B, 1, Hq * D), rnd(B, 1, Hkv * D), rnd(B, 1, Hkv * D)) if with_prev else None
    ln = [(1.0 + 0.1 * torch.randn(D, generator=g)).to(torch.bfloat16) if i % 2 == 0 else (0.05 * torch.randn(D, generator=g)).to(torch.bfloat16)
          for i in range(4)]
    pos = torch.stack([torch.arange(T) + 17 * b for b in range(B)])  # a different offset per sequence
    cfg = type("Cfg", (), {"rope_partial_dim": D // 2})
    rot = rotary_tables(cfg, D, pos)
    with torch.no_grad():
        want = ko.prologue(q_lin, k_lin, v_lin, g_lin, n_q_heads=Hq, n_kv_heads=Hkv, shift=shift, prev=prev,
                           ln_q=(ln[0], ln[1]), ln_k=(ln[2], ln[3]), position_embeddings=rot)
    spec = ko.KvmSpec(num_attention_heads=Hq, num_key_value_heads=Hkv, d_qk_head=D, d_v_head=D, rope_partial_dim=D // 2, chunk_len=32)
    params = gh.layer_params(spec, dev)

    class _LN:
        def __init__(self, w, b):
            self.weight, self.bias = w, b

    pro = ops.PrologueParams(dev, shift_q=None if shift is None else shift[0], shift_k=None if shift is None else shift[1],
                             shift_v=None if shift is None else shift[2], ln_q=_LN(ln[0], ln[1]), ln_k=_LN(ln[2], ln[3]))
    got = ops.prologue_forward(params, pro, q_lin.to(dev), k_lin.to(dev), v_lin.to(dev), g_lin.to(dev), tuple(t.to(dev) for t in rot),
                               prev=None if prev is None else tuple(t.to(dev) for t in prev))
    for a, b, what in zip(got, want, ("q", "k", "v", "gate")):
        _assert_bf16_equal_up_to_ties(a, b, f"D{D} T{T} {what}")
    assert torch.equal(got[2].cpu(), want[2])  # token shift alone: the same bits
