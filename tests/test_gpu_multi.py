"""Two-GPU parity (skipped on a single-GPU box): sharded + gathered results equal the single-GPU results."""

import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    import socket
    with socket.socket(socket.AF_INET, socket.SOCK_STREAM) as sock:
        sock.bind(("127.0.0.1", 0))
        return sock.getsockname()[1]


@pytest.mark.skipif(not torch.cuda.is_available() or torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_two_gpu_results_equal_single_gpu():
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    res = None
    for _ in range(2):
        cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr", "127.0.0.1",
               "--master-port", str(_free_port()), os.path.join(ROOT, "tests", "multi_gpu_check.py")]
        res = subprocess.run(cmd, capture_output=True, text=True, timeout=600, env=env, cwd=ROOT)
        if res.returncode == 0:
            break
        # Only a rendezvous that failed to start (port taken between probing and binding) is tried again, on a new
        # port.  Anything that ran kernels -- a mismatch, a CUDA error, a crash of a rank -- fails at once: the
        # same job is never run twice on the GPUs.
        text = res.stdout + res.stderr
        rendezvous = any(m in text for m in ("Address already in use", "EADDRINUSE", "RendezvousConnectionError",
                                             "RendezvousTimeoutError", "failed to connect to", "TCPStore"))
        ran = any(m in text for m in ("MULTI_GPU_", "CUDA error", "cudaError", "mismatch", "Xid", "illegal"))
        if not rendezvous or ran:
            break
    assert res.returncode == 0, res.stdout[-2000:] + res.stderr[-2000:]
    assert "MULTI_GPU_OK" in res.stdout, res.stdout[-2000:] + res.stderr[-2000:]


def test_interleave_shards_equals_the_strided_copy():
    """The copy kernel behind ``gather_heads`` (one GPU is enough): [shards, tokens, shard] -> [tokens, shards * shard]."""
    from kvm_paper_b200 import _lib

    torch.manual_seed(0)
    for world, tokens, hd in ((2, 1000, 1024), (8, 333, 256), (4, 7, 8)):
        buf = torch.randn(world, tokens, hd, device="cuda").bfloat16()
        full = torch.empty(tokens, world * hd, device="cuda", dtype=torch.bfloat16)
        rc = _lib.load().kvm_interleave_shards(full.data_ptr(), buf.data_ptr(), world, tokens, hd * 2,
                                               torch.cuda.current_stream().cuda_stream)
        _lib.check(rc)
        assert torch.equal(full, buf.permute(1, 0, 2).reshape(tokens, world * hd))
    with pytest.raises(ValueError):  # argument errors are ValueErrors, as in the reference
        _lib.check(_lib.load().kvm_interleave_shards(full.data_ptr(), buf.data_ptr(), 2, 4, 10, None))  # not a multiple of 16
