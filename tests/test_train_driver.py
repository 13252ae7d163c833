"""The training driver end to end on CPU ranks: run, checkpoint, resume, metrics file."""
import json
import os
import sys

from jaxpp_b200.launch import launch


def test_train_driver_checkpoint_and_resume(tmp_path):
    ck, mt = str(tmp_path / "ckpt"), str(tmp_path / "m.jsonl")
    base = ["-m", "jaxpp_b200.train", "--config", "llama7b_pp2tp2", "--tiny", "--device", "cpu", "--ckpt-dir", ck,
            "--ckpt-every", "2", "--metrics", mt, "--lr", "0.01"]
    env = {"CUDA_VISIBLE_DEVICES": "", "OMP_NUM_THREADS": "1",
           "PYTHONPATH": os.path.dirname(os.path.dirname(os.path.abspath(__file__)))}
    assert launch(base + ["--steps", "2"], 4, env=env, timeout_s=300) == 0
    assert os.path.exists(os.path.join(ck, "step_00000002", "manifest.json"))
    manifest = json.load(open(os.path.join(ck, "step_00000002", "manifest.json")))["entries"]
    wq = manifest["params/layers/000/wqkv"]
    assert wq["spec"] == ["model", None] and len(wq["shards"]) == 2          # one file per tensor-parallel shard
    assert len(manifest["params/layers/000/attn_norm"]["shards"]) == 1      # replicated: written once
    assert launch(base + ["--steps", "2", "--resume"], 4, env=env, timeout_s=300) == 0
    recs = [json.loads(l) for l in open(mt)]
    assert [r["step"] for r in recs] == [0, 1, 2, 3] and all(r["tokens_per_s"] > 0 for r in recs)
    assert os.path.exists(os.path.join(ck, "step_00000004", "manifest.json"))


def test_train_driver_with_sharded_optimizer_state(tmp_path):
    """Pipeline x data parallel with master weights and moments sharded over the data-parallel ranks: the flat
    slices are checkpointed as one global 1-d array split over the data axis, and the run resumes from them."""
    ck = str(tmp_path / "ckpt")
    base = ["-m", "jaxpp_b200.train", "--config", "gpt2xl_pp2dp4", "--tiny", "--device", "cpu", "--ckpt-dir", ck,
            "--ckpt-every", "1", "--lr", "0.01", "--shard-optimizer", "--clip-grad-norm", "1.0"]
    env = {"CUDA_VISIBLE_DEVICES": "", "OMP_NUM_THREADS": "1",
           "PYTHONPATH": os.path.dirname(os.path.dirname(os.path.abspath(__file__)))}
    assert launch(base + ["--steps", "1"], 8, env=env, timeout_s=300) == 0
    manifest = json.load(open(os.path.join(ck, "step_00000001", "manifest.json")))["entries"]
    m = manifest["m/layers/000/wqkv"]
    assert m["spec"] == ["data"] and len(m["shards"]) == 4 and len(m["shape"]) == 1
    assert len(manifest["params/layers/000/wqkv"]["shards"]) == 1           # parameters stay replicated
    assert launch(base + ["--steps", "1", "--resume"], 8, env=env, timeout_s=300) == 0
    assert os.path.exists(os.path.join(ck, "step_00000002", "manifest.json"))


def test_train_driver_with_unequal_half_block_stages(tmp_path):
    """``--stage-layers`` with a stage boundary between the two halves of a block: the run checkpoints, and a run with
    equal stages resumes from that checkpoint (parameters are stored by name, whichever rank owns them)."""
    ck = str(tmp_path / "ckpt")
    base = ["-m", "jaxpp_b200.train", "--config", "llama7b_pp2tp2", "--tiny", "--device", "cpu", "--ckpt-dir", ck,
            "--ckpt-every", "1", "--lr", "0.01"]
    env = {"CUDA_VISIBLE_DEVICES": "", "OMP_NUM_THREADS": "1",
           "PYTHONPATH": os.path.dirname(os.path.dirname(os.path.abspath(__file__)))}
    assert launch(base + ["--steps", "1", "--stage-layers", "1,1,1.5,0.5"], 4, env=env, timeout_s=300) == 0
    assert os.path.exists(os.path.join(ck, "step_00000001", "manifest.json"))
    assert launch(base + ["--steps", "1", "--resume"], 4, env=env, timeout_s=300) == 0
    assert os.path.exists(os.path.join(ck, "step_00000002", "manifest.json"))
