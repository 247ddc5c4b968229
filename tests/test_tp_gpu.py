"""Tensor parallelism on 2+ GPUs: fused all-reduce + RMSNorm kernel and a TP engine run.

Each test spawns one process per GPU with torchrun (rendezvous on 127.0.0.1) and is skipped when
fewer than two GPUs are visible.
"""
import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _run(script, nproc, extra_env=None, timeout=300):
    env = dict(os.environ)
    env.update(extra_env or {})
    env["PYTHONPATH"] = ROOT + os.pathsep + env.get("PYTHONPATH", "")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={nproc}",
           "--master-addr", "127.0.0.1", "--master-port", "29571", os.path.join(ROOT, "tests", script)]
    r = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=timeout)
    assert r.returncode == 0, r.stdout[-6000:] + r.stderr[-2000:]
    return r.stdout


def _ngpu():
    return torch.cuda.device_count() if torch.cuda.is_available() else 0


@pytest.mark.skipif(_ngpu() < 2, reason="needs 2 GPUs")
@pytest.mark.parametrize("multimem", ["1", "0"])
def test_fused_allreduce_norm(multimem):
    out = _run("mp_tp_allreduce_norm.py", min(_ngpu(), 8) if _ngpu() in (2, 4, 8) else 2, {"XLLM_TP_MULTIMEM": multimem})
    assert "ALLREDUCE_NORM_OK" in out


@pytest.mark.skipif(_ngpu() < 2, reason="needs 2 GPUs")
@pytest.mark.parametrize("multimem", ["1", "0"])
def test_oneshot_allreduce_norm_argmax_gather(multimem):
    """One-shot fused all-reduce (+residual +RMSNorm), sharded arg-max and logits gather; eager and graph."""
    env = {"XLLM_TP_MULTIMEM": multimem, "XLLM_TP_ONESHOT_TOKENS": "4096"}   # the one-shot form at every size tested
    if multimem == "0":
        env["XLLM_TP_ONESHOT_TOKENS_P2P"] = "2048"     # exercise the peer-load form at every size
    out = _run("mp_tp_oneshot.py", min(_ngpu(), 8) if _ngpu() in (2, 4, 8) else 2, env)
    assert "ONESHOT_OK" in out
    print(out[out.index("ONESHOT_OK"):].splitlines()[0])


@pytest.mark.skipif(_ngpu() < 2, reason="needs 2 GPUs")
@pytest.mark.parametrize("multimem", ["1", "0"])
def test_fused_gemm_reduce_scatter_norm(multimem):
    """tcgen05 GEMM whose epilogue pushes tiles to the owner ranks + owner-side reduce/norm/all-gather."""
    out = _run("mp_tp_gemm_rs.py", min(_ngpu(), 8) if _ngpu() in (2, 4, 8) else 2, {"XLLM_TP_MULTIMEM": multimem})
    assert "GEMM_RS_OK" in out
    print(out[out.index("GEMM_RS_OK"):].splitlines()[0])


@pytest.mark.skipif(_ngpu() < 2, reason="needs 2 GPUs")
def test_expert_parallel_all_to_all():
    """Dispatch / combine over peer memory around the grouped GEMMs against a one-rank reference."""
    out = _run("mp_ep_a2a.py", min(_ngpu(), 8) if _ngpu() in (2, 4, 8) else 2)
    assert "EP_A2A_OK" in out
    print(out[out.index("EP_A2A_OK"):].splitlines()[0])


@pytest.mark.skipif(_ngpu() < 2, reason="needs 2 GPUs")
@pytest.mark.parametrize("push_min", ["512", "8"])
def test_tp_engine_matches_single_gpu(push_min):
    """push_min=8 sends every prefill through the GEMM -> reduce-scatter push path."""
    out = _run("mp_tp_engine.py", 2, {"XLLM_TP_PUSH_MIN_TOKENS": push_min})
    assert "TP_ENGINE_OK" in out


@pytest.mark.skipif(_ngpu() < 2, reason="needs 2 GPUs")
def test_eagle3_head_under_tensor_parallelism():
    """TP2 target reducing through NCCL, the EAGLE-3 head replicated: speculation leaves the greedy output
    where the single-GPU engine puts it (same tolerance as the plain TP run)."""
    out = _run("mp_tp_engine.py", 2, {"SPEC": "eagle3"})
    assert "TP_ENGINE_OK eagle3-replicated-head" in out


@pytest.mark.skipif(_ngpu() < 2, reason="needs 2 GPUs")
def test_moe_engine_with_expert_parallel_all_to_all():
    """Qwen3-MoE-shaped model, TP=EP=2: prefill through the all-to-all path, decode graphs through the
    replicate path; tokens must match the single-GPU engine."""
    out = _run("mp_tp_engine.py", 2, {"MODEL": "moe"})
    assert "TP_ENGINE_OK moe-ep-a2a" in out


@pytest.mark.skipif(_ngpu() < 2, reason="needs 2 GPUs")
def test_pd_disaggregation_two_processes_peer_push():
    """Prefill instance on GPU 0, decode instance on GPU 1, separate processes: KV pushed per layer
    from inside the prefill forward, control messages over a socket, tokens equal one engine's."""
    out = _run("mp_pd.py", 2, timeout=600)
    assert "PD_OK" in out
    print(out[out.index("PD_OK"):].splitlines()[0])


@pytest.mark.skipif(_ngpu() < 2, reason="needs 2 GPUs")
def test_ulysses_all_to_all_over_peer_memory():
    out = _run("mp_ulysses_a2a.py", min(_ngpu(), 8) if _ngpu() in (2, 4, 8) else 2)
    assert "ULYSSES_A2A_OK" in out
    print(out[out.index("ULYSSES_A2A_OK"):].splitlines()[0])


@pytest.mark.skipif(_ngpu() < 2, reason="needs 2 GPUs")
def test_expert_replacement_moves_weights_between_gpus():
    out = _run("mp_eplb.py", min(_ngpu(), 8) if _ngpu() in (2, 4, 8) else 2)
    assert "EPLB_OK" in out
    print(out[out.index("EPLB_OK"):].splitlines()[0])
