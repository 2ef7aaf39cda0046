"""On a machine without a CUDA device every entry point fails at once and says why: nothing falls back to the CPU."""

import json
import subprocess
import sys
from pathlib import Path

import pytest
import torch

import helpers
from prefixserve_b200.weights import write_random_model

ROOT = Path(__file__).resolve().parents[1]
pytestmark = pytest.mark.skipif(torch.cuda.is_available(), reason="a machine without a GPU is what this is about")


@pytest.fixture(scope="module")
def folder(tmp_path_factory):
    path = tmp_path_factory.mktemp("tiny")
    write_random_model(path, helpers.TINY_A["cfg"], 1, std=0.1, gain_noise=0.1, dtype=torch.bfloat16)
    return path


def test_trace_replay_refuses_to_run(folder, tmp_path):
    step = {"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [0, 2]}], "end": []}
    done = subprocess.run([str(ROOT / "bin" / "trace_run"), "--model", str(folder), "--dtype", "float32", "--out", str(tmp_path / "out"),
                           "--max-tokens", "64"], input=json.dumps(step) + "\n", capture_output=True, text=True)
    assert done.returncode != 0 and "done 0" not in done.stdout
    assert "no CUDA device" in done.stderr and "no CPU path" in done.stderr
    assert not list((tmp_path / "out").glob("*.f32"))


def test_the_command_line_refuses_to_generate(folder):
    done = subprocess.run([sys.executable, "-m", "prefixserve_b200", "--model", str(folder), "--prompt-ids", "5,17,3", "--max-tokens", "4"],
                          capture_output=True, text=True, cwd=ROOT)
    assert done.returncode != 0
    assert "CUDA" in done.stderr


def test_an_op_on_cpu_tensors_is_refused():
    from prefixserve_b200 import ops
    from prefixserve_b200.ops import KernelError
    with pytest.raises(KernelError):
        ops.linear(torch.zeros(2, 8), torch.zeros(4, 8))
