"""Multi-GPU tests (one process per GPU, NCCL): library collectives and the fused NVLink
kernels must agree with each other and with the fp32 oracle."""
import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)


def _ngpu():
    return torch.cuda.device_count() if torch.cuda.is_available() else 0


def _run(nproc, *args, timeout=600, **extra_env):
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", PYTHONPATH=ROOT, **extra_env)
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={nproc}",
           "--master-addr", "127.0.0.1", "--master-port", "29631", os.path.join(HERE, "gpu_dist_worker.py"), *args]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=timeout, env=env, cwd=ROOT)
    assert r.returncode == 0, f"worker failed:\n{r.stdout[-4000:]}\n{r.stderr[-4000:]}"
    return r.stdout


@pytest.mark.skipif(_ngpu() < 2, reason="needs 2 GPUs")
@pytest.mark.parametrize("case", ["dp2_library", "dp2_fused", "pp2", "fused_kernels", "pp2_1f1b", "dp2_uneven_library",
                                  "pp2_gloo", "dp2_1f1b_fused", "pp2_1f1b_tail",
                                  "dp2_1f1b_tail_fused"])
def test_two_gpus(case):
    out = _run(2, case)
    assert "WORKER_OK" in out


CANDIDATES = os.environ.get("ZORSE_TEST_CANDIDATES") == "1"   # paths that have not yet run on hardware


@pytest.mark.skipif(_ngpu() < 2 or not CANDIDATES, reason="needs 2 GPUs and ZORSE_TEST_CANDIDATES=1")
@pytest.mark.parametrize("case", ["fused_kernels_v2", "fused_kernels_v3"])
def test_two_gpus_candidates(case):
    out = _run(2, case, timeout=300)
    assert "WORKER_OK" in out


@pytest.mark.skipif(_ngpu() < 2 or not CANDIDATES, reason="needs 2 GPUs and ZORSE_TEST_CANDIDATES=1")
@pytest.mark.parametrize("variant", ["2", "3"])
def test_two_gpus_nvls_training(variant):
    """Fused collectives with the in-switch reduction (2) and with the parameter push that replaces
    the all-gather (3) must land on the parameters of the library-collectives run."""
    out = _run(2, "dp2_fused", timeout=300, ZORSE_RS_ADAM_VARIANT=variant)
    assert "WORKER_OK" in out


@pytest.mark.skipif(_ngpu() < 2 or not CANDIDATES, reason="needs 2 GPUs and ZORSE_TEST_CANDIDATES=1")
def test_tensor_parallel_two_gpus():
    """One lane of two tensor-parallel processes trains like two data-parallel ranks on the same batch."""
    out = _run(2, "tp2_library", timeout=300)
    assert "WORKER_OK" in out


@pytest.mark.skipif(_ngpu() < 2 or not CANDIDATES, reason="needs 2 GPUs and ZORSE_TEST_CANDIDATES=1")
def test_tensor_parallel_lane_kernels_two_gpus():
    """The lane kernels alone (no trainer): scatter GEMM + sum, sum + norm + push, plain push, against NCCL."""
    out = _run(2, "tp_kernels", timeout=300)
    assert "WORKER_OK" in out


@pytest.mark.skipif(_ngpu() < 2 or not CANDIDATES, reason="needs 2 GPUs and ZORSE_TEST_CANDIDATES=1")
def test_tensor_parallel_scatter_gemm_two_gpus():
    """Same job with the reduce-scatter sent from inside the row-split GEMMs (scatter epilogue + rs_finish)."""
    out = _run(2, "tp2_library", timeout=300, ZORSE_TP_FUSED="1")
    assert "WORKER_OK" in out


@pytest.mark.skipif(_ngpu() < 4 or not CANDIDATES, reason="needs 4 GPUs and ZORSE_TEST_CANDIDATES=1")
def test_tensor_parallel_four_gpus():
    out = _run(4, "tp2_library", timeout=300)
    assert "WORKER_OK" in out


@pytest.mark.skipif(_ngpu() < 4, reason="needs 4 GPUs")
@pytest.mark.parametrize("case", ["pp2dp2_library", "pp2dp2_fused", "pp2dp2_1f1b_library", "pp2dp2_1f1b_fused"])
def test_four_gpus(case):
    out = _run(4, case)
    assert "WORKER_OK" in out


@pytest.mark.skipif(_ngpu() < 4 or not CANDIDATES, reason="needs 4 GPUs and ZORSE_TEST_CANDIDATES=1")
def test_four_gpus_tail_deferral_with_fused_collectives():
    """Two stages x 2-way fused ZeRO with the last stage's weight gradients held back: its two halves ran on hardware
    (`pp2_1f1b_tail`, `dp2_1f1b_tail_fused`), this combination has not."""
    out = _run(4, "pp2dp2_1f1b_tail_fused")
    assert "WORKER_OK" in out
