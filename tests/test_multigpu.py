"""Multi-GPU tests: fused tensor-parallel kernels, fused data-parallel optimizer, 3-D Llama.
Each launches tests/mgpu_worker.py under torchrun on the GPUs of this box."""
import json
import os
import re
import socket
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu
HERE = os.path.dirname(os.path.abspath(__file__))


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _run(n, *args, timeout=600, extra_env=None):
    if torch.cuda.device_count() < n:
        pytest.skip(f"needs {n} GPUs")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={n}", "--master-addr", "127.0.0.1",
           "--master-port", str(_free_port()), os.path.join(HERE, "mgpu_worker.py"), *map(str, args)]
    # guard regions around every symmetric buffer: a peer store outside its range fails the test
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", COGITO_SYMM_CANARY="1", **(extra_env or {}))
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=timeout, env=env)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    found = re.findall(r"RESULT (\{[^{}]*\})", r.stdout)      # ranks may interleave their lines
    assert len(found) == n, r.stdout[-2000:]
    res = [json.loads(s) for s in found]
    assert all(o["canaries_ok"] for o in res), res
    return res


def _close(res, tol):
    for out in res:
        assert out["status"][0] == 0, out
        assert out["ref"][-1] < out["ref"][0]
        for a, b in zip(out["ref"], out["got"]):
            assert abs(a - b) < tol, out


@pytest.mark.parametrize("n", [2, 4, 8])
def test_tensor_parallel_gpt2(n):
    _close(_run(n, "tp"), 0.05)


@pytest.mark.parametrize("n,overlap", [(2, "1"), (4, "0"), (8, "0")])
def test_tensor_parallel_gpt2_other_schedule(n, overlap):
    """The same comparison with the two-halves-on-two-streams schedule forced on where it is off by
    default (2 ranks) and off where it is on by default (4 and 8 ranks)."""
    _close(_run(n, "tp", extra_env={"COGITO_TP_OVERLAP": overlap}), 0.05)


def test_tensor_parallel_gpt2_peer_load_transport():
    """Without the NVSwitch multicast path: shards pulled with peer loads, partials summed by the owner."""
    _close(_run(2, "tp", extra_env={"COGITO_TP_NVLS": "0"}), 0.05)


@pytest.mark.parametrize("n", [2, 4, 8])
def test_data_parallel_fused_adam(n):
    _close(_run(n, "dp"), 0.05)


@pytest.mark.parametrize("dp,tp,pp", [(1, 1, 2), (1, 2, 1), (2, 1, 1), (1, 2, 2), (2, 2, 2)])
def test_3d_llama(dp, tp, pp):
    res = _run(dp * tp * pp, "3d", dp, tp, pp)
    _close(res, 0.05)
    if pp > 1:
        assert any(r["p2p_bytes"] > 0 for r in res)


@pytest.mark.parametrize("n", [2, 4, 8])
def test_tensor_parallel_int4_serving(n):
    for out in _run(n, "serve"):
        assert out["status"][0] == 0, out
        assert out["fused"] and out["tokens_agree"], out
        assert max(out["got"]) < 0.06, out              # logits of the split engine vs the unsplit one, relative to their range (bf16 sums in another order)


def test_3d_llama_interleaved_schedule():
    """Two pipeline ranks with two model chunks each (virtual stages 0..3), tick-synchronous executor over NCCL."""
    res = _run(2, "3d", 1, 1, 2, 2)
    _close(res, 0.05)
    assert max(r["p2p_bytes"] for r in res) > 0


def test_3d_llama_with_loss_scaling_and_clipping():
    """tp 2: the overflow flag and the clipping norm are those of the whole replica (all-reduced over its ranks)."""
    _close(_run(2, "3d", 1, 2, 1, 1, "scaled"), 0.05)


@pytest.mark.parametrize("dp,tp,pp,recompute", [(1, 2, 1, "block"), (1, 1, 2, "stage"), (1, 2, 2, "block")])
def test_3d_llama_activation_recompute(dp, tp, pp, recompute):
    """Same losses with the activations of every block (or stage) dropped and recomputed in backward."""
    _close(_run(dp * tp * pp, "3d", dp, tp, pp, 1, "plain", recompute), 0.05)


def test_3d_llama_scaled_keeps_the_fused_data_parallel_optimizer():
    """dp 2 x tp 2 with loss scaling and clipping: the bucketed all-reduce + Adam kernels run with statistics of
    the whole job."""
    res = _run(4, "3d", 2, 2, 1, 1, "scaled")
    _close(res, 0.05)
    assert all(r["fused_dp"] == "DPFusedAdam" for r in res)
