"""Needs 2+ GPUs: fused all-gather->GEMM / GEMM->reduce-scatter kernels against their NCCL twins."""
import os

import pytest
import torch

from jaxpp_b200.launch import launch

pytestmark = [pytest.mark.gpu, pytest.mark.multigpu]
WORKER = os.path.join(os.path.dirname(os.path.abspath(__file__)), "mgpu_worker.py")


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs at least 2 GPUs")
def test_fused_tensor_parallel_kernels_two_gpus():
    rc = launch([WORKER, "fused_tp"], 2, env={"NCCL_NVLS_ENABLE": "0"}, timeout_s=300)
    assert rc == 0
