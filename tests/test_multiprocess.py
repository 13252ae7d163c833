"""Multi-process runs on one node over gloo (CPU ranks): the per-rank programs, the point-to-point backend,
tensor-parallel ops and resharding, each against a locally computed oracle."""
import os
import sys

import pytest

from jaxpp_b200.launch import launch

WORKER = os.path.join(os.path.dirname(os.path.abspath(__file__)), "mp_worker.py")


def run(scenario, nproc, **extra_env):
    rc = launch([WORKER, scenario], nproc, env={"CUDA_VISIBLE_DEVICES": "", "OMP_NUM_THREADS": "1", **extra_env}, timeout_s=300)
    assert rc == 0, f"scenario {scenario} failed with exit code {rc}"


@pytest.mark.parametrize("scenario,nproc", [
    ("pp_std1f1b", 2), ("pp_interleaved", 2), ("pp_zb", 3), ("pp_dualpipev", 2),
])
def test_pipeline_ranks_as_processes(scenario, nproc):
    run(scenario, nproc)


def test_tensor_parallel_two_ranks():
    run("tp2", 2)


def test_pipeline_times_tensor_parallel():
    run("pp2_tp2", 4)


def test_reshard_round_trip():
    run("reshard", 4)


def test_cross_stage_stack_is_one_all_gather_with_uneven_owners():
    run("stack", 2)


def test_pipeline_times_data_parallel():
    run("pp2_dp2_gpt2", 4)


@pytest.mark.parametrize("scenario", ["pp2_dp2_gpt2", "pp2_dp2_gpt2_zero", "pp2_ep2_mixtral"])
def test_gradient_reduction_issued_from_the_last_backward_matches_the_after_loop_form(scenario):
    """Data-parallel gradient all-reduce (or reduce-scatter with sharded optimizer state) hooked into the task that adds
    the last microbatch's weight gradient, against the same collectives run after the loop: identical bits."""
    run(scenario, 4, TEST_OVERLAP="1")


def test_pipeline_times_expert_parallel_moe():
    run("pp2_ep2_mixtral", 4)


@pytest.mark.parametrize("scenario", ["pp2_dp2_gpt2_zero", "pp2_ep2_mixtral_zero"])
def test_optimizer_state_sharded_over_data_parallel_ranks(scenario):
    run(scenario, 4)


@pytest.mark.parametrize("scenario", ["pp2_tp2", "pp2_dp2_gpt2_zero", "pp2_ep2_mixtral"])
def test_gradient_clipping_by_global_norm_across_stages_and_shards(scenario):
    """The clip coefficient needs the norm over every pipeline stage and every tensor- / expert-parallel shard or
    optimizer-state slice; the oracle is the un-sharded, un-pipelined step with the same (active) threshold."""
    run(scenario, 4, TEST_CLIP="0.05")


@pytest.mark.parametrize("nproc", [2, 4])
def test_ring_attention_over_a_sequence_split_across_ranks(nproc):
    run("ring_attention", nproc)


def test_pipeline_times_context_parallel():
    """2 pipeline ranks x 2 context-parallel ranks (every sequence split in two chunks, ring attention, RoPE offsets,
    gradients summed over the axis) against the un-sharded step; with gradient clipping on."""
    run("pp2_cp2_llama", 4)
    run("pp2_cp2_llama", 4, TEST_CLIP="0.05")
    run("pp2_cp2_llama_zigzag", 4)      # pieces r and 2n-1-r per rank: balanced causal work


def test_expert_parallel_blocks_under_activation_recompute():
    """The dispatch / combine exchanges of a mixture-of-experts block run again inside the backward task when the
    block is recomputed: every expert-parallel rank repeats them in the same order."""
    run("pp2_ep2_mixtral", 4, TEST_RECOMPUTE="1")


@pytest.mark.parametrize("scenario,nproc", [("tp2", 2), ("pp2_tp2", 4)])
def test_vocabulary_parallel_output_projection_and_cross_entropy(scenario, nproc):
    """The output projection split by vocabulary rows over the tensor-parallel ranks: sharded logits, log-sum-exps
    combined across ranks, the label's logit from its owner; against the un-sharded step (gradient clipping on, so
    the sharded head also enters the global norm)."""
    run(scenario, nproc, TEST_VOCAB_PARALLEL="1", TEST_CLIP="0.05")
