"""The decode step for callers that cannot allocate device memory (`kvm_decode_step_static`).

Who needs it: code that is handed tensors and a stream by a runtime which owns all device memory and does not
let its plug-ins call cudaMalloc (an inference server with a sealed memory pool, a callback that runs while the
framework forbids allocation).  Such a caller cannot provide the workspace `kvm_decode_step` wants, so this entry
point keeps that scratch in a fixed 32 MiB array inside the library.

The test drives two identical decode caches for two consecutive tokens, one through the ordinary entry point and
one through the static-scratch entry point (called directly through the C ABI), and requires identical output
bits, identical memory and identical lengths.  The first token crosses a block boundary (a memory update runs),
the second does not, so both kernel paths use the scratch; the second call also sees the scratch as the first
left it.  A shape beyond the built-in scratch must be refused with a capacity error.  This file is collected last
so that a failure here cannot hide the result of any other test.
"""

import ctypes as C

import pytest
import torch

from kvm_paper_b200 import _lib, ops
from kvm_paper_b200.ops import _tensor4
from oracle import kvm_oracle as ko
from tests import gpu_helpers as gh

pytestmark = pytest.mark.gpu


def _static_step(cache: ops.KvmDecodeCache, q, k, v, g):
    """One token through kvm_decode_step_static; host bookkeeping as in KvmDecodeCache.step."""
    lib = _lib.load()
    n_app, max_rows = cache._plan_step()
    any_update = n_app is not None
    if any_update:
        cache._n_append.copy_(torch.from_numpy(n_app).to(cache.device))
    ccache = _lib.KvmDecodeCache(cache.memory.c(), cache.ring_k.data_ptr(), cache.ring_v.data_ptr(),
                                 cache.ring_gate.data_ptr(), cache.total_len.data_ptr(), cache.state_len.data_ptr())
    rc = lib.kvm_decode_step_static(
        C.byref(cache.params.c), cache.batch, ccache, _tensor4(q, "q"), _tensor4(k, "k"), _tensor4(v, "v"),
        _tensor4(g, "gate"), cache._n_append.data_ptr() if any_update else None, int(any_update), max_rows,
        cache.out.data_ptr(), None, torch.cuda.current_stream().cuda_stream)
    _lib.check(rc)
    return cache.out


def test_static_scratch_decode_equals_workspace_decode():
    torch.manual_seed(7)
    spec = ko.KvmSpec(4, 2, 64, 64, 32, 32, 2, 4, 1, "power_law", state_growth_factor=4.0, state_min_len=32)
    B, T = 3, 32 * 5  # the next token starts a new block: the first decode step runs a memory update
    q = torch.randn(B, 4, T + 2, 64).bfloat16().cuda()
    k = torch.nn.functional.layer_norm(torch.randn(B, 2, T + 2, 64), (64,)).bfloat16().cuda()
    v = torch.randn(B, 2, T + 2, 64).bfloat16().cuda()
    g = (1 + torch.nn.functional.elu(torch.randn(B, 2, T + 2, 1))).bfloat16().cuda()
    params, plan, res = gh.device_prefill(spec, q[:, :, :T], k[:, :, :T], v[:, :, :T], g[:, :, :T])
    mk = lambda: ops.decode_cache_from_prefill(params, res, k[:, :, :T], v[:, :, :T], g[:, :, :T], gh.desired_fn(spec))  # noqa: E731
    ref_cache, static_cache = mk(), mk()
    updates = 0
    for i in range(T, T + 2):
        step = [t[:, :, i:i + 1] for t in (q, k, v, g)]
        want = ref_cache.step(*step).clone()
        updates += int(ref_cache._last_any_update)
        got = _static_step(static_cache, *step).clone()
        torch.cuda.synchronize()
        assert torch.equal(got, want), f"token {i - T}: outputs differ (max {float((got.float() - want.float()).abs().max())})"
        assert torch.equal(static_cache.total_len, ref_cache.total_len)
        assert torch.equal(static_cache.state_len, ref_cache.state_len)
        for name in ("k_sum", "v_sum", "vlen", "k_attn", "v_attn"):
            assert torch.equal(getattr(static_cache.memory, name), getattr(ref_cache.memory, name)), name
        assert torch.equal(static_cache.ring_k, ref_cache.ring_k) and torch.equal(static_cache.ring_gate, ref_cache.ring_gate)
    assert updates == 1, "the first of the two tokens was meant to run a memory update"


def test_static_scratch_rejects_oversized_shapes():
    """Beyond the built-in scratch the call must fail with a capacity error before anything is launched."""
    lib = _lib.load()
    cfg = ops.LayerConfig(64, 64, 128, 512, 2, 64, 1)
    params = ops.LayerParams(cfg, torch.ones(128), torch.zeros(128), None, None, "cuda")
    batch = 64  # 4096 kv rows x 512 x 128 x 2 x 2 bytes of routing scratch alone: far more than 32 MiB
    assert lib.kvm_decode_workspace_bytes(C.byref(params.c), batch, 4096) > _lib.STATIC_SCRATCH_BYTES
    mem = _lib.KvmMemory(256, 256, 256, 256, 256, 4096)
    t4 = _lib.KvmTensor4(256, 128, 128, 128)
    rc = lib.kvm_decode_step_static(C.byref(params.c), batch, _lib.KvmDecodeCache(mem, 256, 256, 256, 256, 256),
                                    t4, t4, t4, t4, None, 0, 4096, 256, None, None)
    assert rc == 2
    msg = lib.kvm_last_error_string().decode()
    assert "scratch" in msg and str(_lib.STATIC_SCRATCH_BYTES) in msg
    with pytest.raises(_lib.KvmError):
        _lib.check(rc)
