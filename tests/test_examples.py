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


@pytest.mark.parametrize("script,procs,flags,lines", [
    ("distributed/run_vlm_hybrid.py", 4, ["--backend", "gloo", "--steps", "2", "--microbatches", "2", "--shape", "moe_tiny",
                                          "--ep", "2", "--ep-capacity", "1.5"], 4),
    ("distributed/run_vlm_ddp.py", 2, ["--backend", "gloo", "--steps", "2", "--shape", "tiny"], 2),
])
def test_distributed_examples_on_gloo_ranks(script, procs, flags, lines):
    """The distributed scripts as gloo ranks: the plugin-API script (encoder stage + LLM stage; with ``--ep 2`` two such
    replicas whose MoE experts are sharded over the replicas) and the data-parallel script."""
    from tests.dist_utils import free_port

    env = dict(os.environ, CUDA_VISIBLE_DEVICES="")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={procs}", "--master-addr", "127.0.0.1",
           "--master-port", str(free_port()), os.path.join(ROOT, "examples", script), *flags]
    res = subprocess.run(cmd, capture_output=True, text=True, timeout=420, env=env, cwd=ROOT)
    assert res.returncode == 0, res.stderr[-2000:]
    losses = [float(line.split()[-1]) for line in res.stdout.splitlines() if line.startswith("step ")]
    assert len(losses) == lines and all(l == l and l < 20 for l in losses), res.stdout
