"""The single-process example scripts run on CPU with their toy shapes."""

import os
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.mark.parametrize("script", ["pretrain_vlm.py", "pretrain_vlm_processor.py", "pretrain_vlm_lora.py", "pretrain_valm.py",
                                    "pretrain_vlm_from_checkpoints.py"])
def test_example_runs(script):
    env = dict(os.environ, CUDA_VISIBLE_DEVICES="")
    res = subprocess.run([sys.executable, os.path.join(ROOT, "examples", script), "--steps", "1"], capture_output=True, text=True,
                         timeout=300, env=env, cwd=ROOT)
    assert res.returncode == 0, res.stderr[-2000:]
    assert res.stdout.strip(), "the example printed nothing"
