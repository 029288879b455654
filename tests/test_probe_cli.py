"""The micro-benchmark command lines that the kernel documentation names exist (their bodies need GPUs)."""

import os
import re
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _choices(module: str) -> set[str]:
    res = subprocess.run([sys.executable, "-m", module, "--help"], capture_output=True, text=True, timeout=300, cwd=ROOT,
                         env=dict(os.environ, CUDA_VISIBLE_DEVICES=""))
    assert res.returncode == 0, res.stderr[-1500:]
    sets = [set(m.split(",")) for m in re.findall(r"\{([^}]*)\}", res.stdout.replace("\n", "").replace(" ", ""))]
    assert sets, res.stdout
    return max(sets, key=len)  # the positional argument: what to measure


@pytest.mark.parametrize("module,named", [
    ("cornstarch_b200.utils.kernel_probe", ["gemm", "gemm_grouped", "gemm_sustained", "attn_fwd", "attn_bwd", "elementwise", "adamw", "mma_issue",
                                            "gemm_ar_local", "grad_reduce_local", "moe_push_local", "attn_fwd_pulled"]),
    ("cornstarch_b200.utils.comm_probe", ["gemm_allreduce", "sp_linear", "cp_attention", "grad_reduce", "moe_exchange", "moe_layer"]),
])
def test_probe_command_lines(module, named):
    have = _choices(module)
    assert set(named) <= have, set(named) - have
    doc = open(os.path.join(ROOT, "docs", "using_cornstarch", "kernels.md")).read()
    for name in named:
        assert f"`{name}" in doc or f"{name}`" in doc, f"{name} is not documented in kernels.md"
