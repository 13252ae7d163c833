"""The example programs run end to end on CPU at their default (small) sizes, and the tutorial's snippets execute
in order (the reference ships examples/basic.py, examples/mpmd_reshard.py and examples/tutorial.ipynb)."""
import importlib.util
import os
import re

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def load(name):
    spec = importlib.util.spec_from_file_location(f"example_{name}", os.path.join(ROOT, "examples", f"{name}.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


@pytest.mark.parametrize("schedule,pp", [("std", 2), ("interleaved", 2), ("zb", 3), ("dualpipev", 2)])
def test_basic_example_single_controller(schedule, pp, capsys):
    load("basic").main(["--pp", str(pp), "--schedule", schedule, "--train-steps", "2", "--num-ubatches", "6", "--device", "cpu"])
    out = capsys.readouterr().out
    assert "SUCCESS" in out and out.count("PASS") == 4


def test_basic_example_one_process_per_rank():
    with pytest.raises(SystemExit) as e:
        load("basic").main(["--pp", "2", "--train-steps", "1", "--device", "cpu", "--multi-process"])
    assert e.value.code == 0


def test_reshard_example(capsys):
    with pytest.warns(DeprecationWarning, match="pipeline_enter_stage"):
        load("mpmd_reshard").main(["--device", "cpu"])
    out = capsys.readouterr().out
    assert "gradients match plain autograd" in out and "W1.is_deleted()=True" in out
    with pytest.raises(SystemExit) as e:
        load("mpmd_reshard").main(["--device", "cpu", "--multi-process"])
    assert e.value.code == 0


def test_inference_example(capsys):
    load("inference").main(["--pp", "2", "--stages", "4", "--device", "cpu"])
    assert "matches the un-pipelined forward" in capsys.readouterr().out


def test_tutorial_snippets_execute_in_order(capsys):
    text = open(os.path.join(ROOT, "examples", "tutorial.md")).read()
    upto = text.index("## 7.")
    blocks = re.findall(r"```python\n(.*?)```", text[:upto], flags=re.S)
    assert len(blocks) >= 7
    g = torch.Generator().manual_seed(0)
    params = [{"w1": torch.randn(32, 16, generator=g) * 0.2, "b1": torch.zeros(32), "w2": torch.randn(16, 32, generator=g) * 0.2,
               "g": torch.ones(16), "b": torch.zeros(16)} for _ in range(4)]
    env = {"params": params, "batch": torch.randn(4, 8, 16, generator=g)}
    for i, code in enumerate(blocks):
        exec(compile(code, f"tutorial block {i}", "exec"), env)
        if i == 0:   # the hand-written accumulation loop of section 1 runs as it stands
            losses, new_params = env["step"](params, env["batch"])
            assert losses.shape == (4,) and len(new_params) == 4
    assert env["losses"].mpmd_idxs == (1,) and env["new_params"][0]["w1"].mpmd_idxs == (0,)
    assert "n_tasks" in capsys.readouterr().out
