"""accb_peer_*: exchanges between processes (one per GPU) by the library's own kernels over NVLink peer mappings.
With one GPU only the single-rank forms run; with two or more, tests/peer_ranks.py runs under torchrun with one
rank per GPU (never several ranks on one GPU: their kernels wait for one another) and is checked against NCCL."""
import os
import subprocess
import sys

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_peer_single_rank_forms(accb, ctx, torch_cuda, rng):
    t = torch_cuda
    peer = accb.Peer(ctx, 0, 1, 1 << 16, lambda b: [b])
    x = rng.integers(-50, 50, 1000).astype(np.int32)
    view = t.as_tensor(peer.array(256, (1000,), np.int32), device="cuda")  # the buffer seen as a tensor, no copy
    view.copy_(t.from_numpy(x).cuda())
    got = t.zeros(1000, dtype=t.int32, device="cuda")
    peer.allreduce(256, 1000, np.int32, "add", got)
    peer.gather(256, 64, got[:16])
    peer.barrier()
    peer.status()
    assert np.array_equal(got.cpu().numpy(), x)
    with pytest.raises(accb.AccbError):
        peer.gather(1 << 20, 64, got)  # outside the buffer
    with pytest.raises(accb.AccbError):
        peer.allreduce(256, 10, np.float32, "xor", got)  # bitwise combination of floats
    peer.destroy()


def test_a_rank_that_never_arrives_runs_the_wait_into_its_limit(accb, ctx, torch_cuda, monkeypatch):
    """The failure is made on the host: this process claims to be rank 0 of 2 and nobody plays rank 1, so rank 1's
    flag is never set.  The barrier kernel gives up after its limit (one second here), finishes normally, and the
    status call reports ETIMEOUT; the context stays usable."""
    t = torch_cuda
    monkeypatch.setenv("ACCB_PEER_TIMEOUT_MS", "1000")
    peer = accb.Peer(ctx, 0, 2, 4096, None)
    peer.barrier()
    with pytest.raises(accb.AccbError) as e:
        peer.status()
    assert e.value.status == accb.ETIMEOUT
    peer.status()  # the error word was cleared
    x = t.arange(10, device="cuda")
    assert int(x.sum()) == 45  # the device still answers
    peer.destroy()


def test_peer_exchanges_match_nccl_on_two_or_more_gpus(torch_cuda):
    n = torch_cuda.cuda.device_count()
    if n < 2:
        pytest.skip("needs two GPUs: ranks that wait for one another never share a GPU")
    world = 4 if n >= 4 else 2
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    out = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}",
                          "--master-addr", "127.0.0.1", "--master-port", "29577",
                          os.path.join(ROOT, "tests", "peer_ranks.py")], capture_output=True, text=True, env=env, timeout=600)
    assert out.returncode == 0, out.stdout[-2000:] + out.stderr[-4000:]
    assert out.stdout.count("PEER-OK") == world, out.stdout[-2000:] + out.stderr[-2000:]
