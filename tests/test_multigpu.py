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


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs at least 2 GPUs")
def test_mixtral_step_with_expert_parallelism_two_gpus():
    rc = launch([WORKER, "moe_train"], 2, env={"NCCL_NVLS_ENABLE": "0"}, timeout_s=240)
    assert rc == 0


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs at least 2 GPUs")
def test_sharded_optimizer_state_two_gpus():
    rc = launch([WORKER, "zero"], 2, env={"NCCL_NVLS_ENABLE": "0"}, timeout_s=240)
    assert rc == 0


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs at least 2 GPUs")
def test_ring_attention_two_gpus():
    rc = launch([WORKER, "ring_attention"], 2, env={"NCCL_NVLS_ENABLE": "0"}, timeout_s=240)
    assert rc == 0


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs at least 2 GPUs")
@pytest.mark.parametrize("scenario", ["dp_overlap", "vocab_parallel", "ring_attention_zigzag"])
def test_overlapped_gradient_reduction_vocab_parallel_head_and_zigzag_ring_two_gpus(scenario):
    rc = launch([WORKER, scenario], 2, env={"NCCL_NVLS_ENABLE": "0"}, timeout_s=300)
    assert rc == 0


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs at least 2 GPUs")
def test_fused_moe_dispatch_combine_two_gpus():
    rc = launch([WORKER, "fused_moe"], 2, env={"NCCL_NVLS_ENABLE": "0"}, timeout_s=300)
    assert rc == 0


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs at least 2 GPUs")
@pytest.mark.parametrize("scenario", ["pp_std", "pp_interleaved", "pp_zb", "pp_tied"])
def test_pipeline_over_nccl_p2p_two_gpus(scenario):
    rc = launch([WORKER, scenario], 2, env={"NCCL_NVLS_ENABLE": "0"}, timeout_s=300)
    assert rc == 0


@pytest.mark.skipif(torch.cuda.device_count() < 4, reason="needs at least 4 GPUs")
@pytest.mark.parametrize("scenario", ["pp2_tp2_std", "pp2_tp2_interleaved"])
def test_pipeline_times_tensor_parallel_four_gpus(scenario):
    rc = launch([WORKER, scenario], 4, env={"NCCL_NVLS_ENABLE": "0"}, timeout_s=180)
    assert rc == 0


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs at least 2 GPUs")
@pytest.mark.parametrize("scenario", ["p2p_native", "pp_std", "pp_interleaved"])
def test_native_nccl_p2p_backend_two_gpus(scenario):
    rc = launch([WORKER, scenario], 2, env={"NCCL_NVLS_ENABLE": "0", "JAXPP_B200_P2P": "native"}, timeout_s=90)
    assert rc == 0
