"""The device status word: how a bounded device-side wait that ran out reaches the caller.

The kernels never wait without a limit; a wait that expires stores KVM_ERR_DEVICE_TIMEOUT in a status word of
the call's workspace and the kernel leaves through its normal exit.  These tests cover the host half of that
path by writing the word from the host (no kernel is made to time out here), and the rule that an
attention-only call does not erase what the chain call of the same prefill reported."""

import pytest
import torch

from kvm_paper_b200 import _lib, ops
from oracle import kvm_oracle as ko
from tests import gpu_helpers as gh

pytestmark = pytest.mark.gpu


def _small_prefill():
    torch.manual_seed(1)
    spec = ko.KvmSpec(2, 2, 64, 64, 32, 32, 2, 4, 1, "power_law", state_growth_factor=4.0, state_min_len=32)
    T = 32 * 5 + 3
    q = torch.randn(1, 2, T, 64).bfloat16().cuda()
    k = torch.nn.functional.layer_norm(torch.randn(1, 2, T, 64), (64,)).bfloat16().cuda()
    v = torch.randn(1, 2, T, 64).bfloat16().cuda()
    g = (1 + torch.nn.functional.elu(torch.randn(1, 2, T, 1))).bfloat16().cuda()
    params = gh.layer_params(spec)
    plan = ops.build_prefill_plan(T, spec.chunk_len, spec.n_bswa_chunks, gh.desired_fn(spec))
    return spec, params, plan, (q, k, v, g)


def test_prefill_status_word_is_reported_once_and_survives_an_attention_only_call():
    spec, params, plan, inputs = _small_prefill()
    runner = ops.PrefillRunner(params, 1, plan)
    runner.run(*inputs)
    runner.check_status()                                   # clean run: nothing to report
    word = runner.ws[:4].view(torch.int32)
    runner.run(*inputs, phases=_lib.PREFILL_CHAIN)
    word.fill_(3)                                           # as if a wait of the chain kernel had run out
    runner.run(*inputs, phases=_lib.PREFILL_ATTENTION)      # must not erase it
    with pytest.raises(_lib.KvmError) as err:
        runner.check_status()
    assert err.value.code == 3 and "timeout" in str(err.value)
    runner.check_status()                                   # reported once, then cleared
    word.fill_(3)
    runner.run(*inputs)                                     # a call that includes the chain phase opens a new word
    runner.check_status()


def test_decode_status_word_is_reported_once():
    spec, params, plan, (q, k, v, g) = _small_prefill()
    res = ops.prefill_forward(params, q, k, v, g, plan)
    cache = ops.decode_cache_from_prefill(params, res, k, v, g, gh.desired_fn(spec))
    step = [t[:, :, -1:] for t in (q, k, v, g)]
    cache.step(*step)
    cache.check_status()
    word = cache._ws[4 * (cache.kv_rows + cache.batch): 4 * (cache.kv_rows + cache.batch + 1)].view(torch.int32)
    word.fill_(3)
    with pytest.raises(_lib.KvmError) as err:
        cache.check_status()
    assert err.value.code == 3
    cache.check_status()
    cache.step(*step)
    cache.check_status()
