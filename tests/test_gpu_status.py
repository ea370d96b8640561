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


def test_a_withheld_arrival_runs_a_bounded_wait_out_and_the_kernel_returns():
    """The device half of the path.  With the test hook of the ABI the chain kernel's issuing thread withholds one
    barrier arrival of the first update and the wait limit is a fraction of a millisecond: the warps that wait for
    that arrival give up, every role of every CTA of the cluster leaves through the common exit (tensor memory
    freed, nothing in flight), the kernels behind it see the status and do nothing, and the host reads
    KVM_ERR_DEVICE_TIMEOUT.  Nothing faults and nothing hangs: the next ordinary run on the same buffers is clean
    and gives the bits of an undisturbed run."""
    torch.manual_seed(2)
    C, H, T = 128, 2, 128 * 5 + 9
    spec = gh.bf16_spec(ko.KvmSpec(H, H, 128, 128, 64, C, 2, 4, 1, "plus_one", state_min_len=C))
    q = torch.nn.functional.layer_norm(torch.randn(1, T, H, 128), (128,)).bfloat16().transpose(1, 2).cuda()
    k = torch.nn.functional.layer_norm(torch.randn(1, T, H, 128), (128,)).bfloat16().transpose(1, 2).cuda()
    v = torch.randn(1, T, H, 128).bfloat16().transpose(1, 2).cuda()
    g = (1 + torch.nn.functional.elu(0.5 * torch.randn(1, T, H, 1))).bfloat16().transpose(1, 2).cuda()
    params = gh.layer_params(spec)
    plan = ops.build_prefill_plan(T, C, 2, gh.desired_fn(spec))
    want = ops.prefill_forward(params, q, k, v, g, plan, check=True)
    want_out, want_k = want.out.clone(), want.memory.k_sum.clone()
    runner = ops.PrefillRunner(params, 1, plan)
    runner.ws.zero_()
    runner.run(q, k, v, g, phases=_lib.PREFILL_CHAIN | _lib.PREFILL_ATTENTION | _lib.PREFILL_TEST_WITHHOLD_ARRIVAL)
    with pytest.raises(_lib.KvmError) as err:
        runner.check_status()
    assert err.value.code == 3
    runner.check_status()               # reported once
    out = runner.run(q, k, v, g)        # the device and the buffers are fine
    runner.check_status()
    assert torch.equal(out, want_out) and torch.equal(runner.memory.k_sum, want_k)
