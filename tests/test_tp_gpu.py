"""Fused tensor-parallel kernels on 2+ GPUs (spawned with torch.distributed.run); skipped on one GPU."""
import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _run(script, nproc, port, timeout=240, extra_env=None):
    env = dict(os.environ)
    env.update(extra_env or {})
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={nproc}", "--master-addr", "127.0.0.1",
           "--master-port", str(port), os.path.join(ROOT, "tests", script)]
    return subprocess.run(cmd, capture_output=True, text=True, timeout=timeout, env=env, cwd=ROOT)


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_fused_tp_kernels_two_gpus():
    p = _run("mp_tp_fused.py", 2, 29611)
    assert "TP_FUSED_OK 2" in p.stdout, p.stdout[-3000:] + p.stderr[-3000:]


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_fused_tp_kernels_in_switch_reduction_two_gpus():
    """The fused GEMM -> reduce-scatter / all-reduce kernel with its reduction in the NVLink switch (partials stay local,
    the owner reads them with multimem.ld_reduce). Every rank runs to the end: no wait is made to run out here."""
    p = _run("mp_tp_fused.py", 2, 29620, extra_env={"B2_TEST_NVLS": "1"})
    assert "TP_FUSED_OK 2" in p.stdout, p.stdout[-3000:] + p.stderr[-3000:]


@pytest.mark.skipif(torch.cuda.device_count() < 4, reason="needs 4 GPUs")
def test_fused_tp_kernels_all_gpus():
    n = 8 if torch.cuda.device_count() >= 8 else 4
    p = _run("mp_tp_fused.py", n, 29612)
    assert f"TP_FUSED_OK {n}" in p.stdout, p.stdout[-3000:] + p.stderr[-3000:]
    p = _run("mp_tp_fused.py", n, 29621, extra_env={"B2_TEST_NVLS": "1"})
    assert f"TP_FUSED_OK {n}" in p.stdout, p.stdout[-3000:] + p.stderr[-3000:]


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_expert_parallel_moe_two_gpus():
    p = _run("mp_ep.py", 2, 29613)
    assert "EP_OK 2" in p.stdout, p.stdout[-3000:] + p.stderr[-3000:]


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_symmetric_collectives_two_gpus():
    p = _run("mp_coll.py", 2, 29614)
    assert "COLL_OK 2" in p.stdout, p.stdout[-3000:] + p.stderr[-3000:]


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_symmetric_collectives_in_switch_reduction_two_gpus():
    """The same collectives with the multicast mapping on: all-reduce and all-reduce + residual + RMSNorm reduce inside
    the NVLink switch (multimem.ld_reduce / multimem.st). Not a failure test: every rank runs to the end."""
    p = _run("mp_coll.py", 2, 29618, extra_env={"B2_TEST_NVLS": "1"})
    assert "COLL_OK 2" in p.stdout, p.stdout[-3000:] + p.stderr[-3000:]


@pytest.mark.skipif(torch.cuda.device_count() < 4, reason="needs 4 GPUs")
def test_symmetric_collectives_and_moe_all_gpus():
    n = 8 if torch.cuda.device_count() >= 8 else 4
    p = _run("mp_coll.py", n, 29615)
    assert f"COLL_OK {n}" in p.stdout, p.stdout[-3000:] + p.stderr[-3000:]
    p = _run("mp_coll.py", n, 29619, extra_env={"B2_TEST_NVLS": "1"})
    assert f"COLL_OK {n}" in p.stdout, p.stdout[-3000:] + p.stderr[-3000:]
    p = _run("mp_ep.py", n, 29616)
    assert f"EP_OK {n}" in p.stdout, p.stdout[-3000:] + p.stderr[-3000:]


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_tensor_parallel_llama_matches_single_process_model():
    n = 2
    p = _run("mp_tp_engine.py", n, 29617)
    assert f"TP_ENGINE_OK {n}" in p.stdout, p.stdout[-3000:] + p.stderr[-3000:]


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_expert_parallel_engine_eager_and_graph_decode_agree():
    p = _run("mp_ep_engine.py", 2, 29618, extra_env={"NCCL_NVLS_ENABLE": "0"})
    assert "EP_ENGINE_OK 2" in p.stdout, p.stdout[-3000:] + p.stderr[-3000:]
