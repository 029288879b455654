"""The kernels at the shapes the benchmark runs them at, each against an fp32 PyTorch statement of the same operation:
attention at S = 8192 with 32 query / 8 key heads of width 128 under a one-image bitfield mask (forward and backward),
the SigLIP encoder's attention (729 tokens, 16 heads of width 72) backward, and the 8192 x 28672 x 4096 gate|up GEMM.
The oracle is evaluated on one key head's group of query heads at a time to bound its memory."""

import pytest
import torch

from cornstarch_b200.ops import attention as A
from cornstarch_b200.ops.gemm import gemm

pytestmark = pytest.mark.gpu


def _rel(a, b):
    a, b = a.float(), b.float()
    return (a - b).abs().max().item() / max(1.0, b.abs().max().item())


def _one_image_bits(S, image_tokens=729, start=16):
    text = (1 << 62) | 1 | 2
    bits = torch.full((1, S), text, dtype=torch.int64)
    bits[0, start : start + image_tokens] = 2
    return bits.cuda()


def test_attention_llama8b_shape_bitfield_forward_backward():
    S, Hq, Hk, D = 8192, 32, 8, 128
    g = torch.Generator().manual_seed(0)
    q = torch.randn(1, S, Hq, D, generator=g).cuda().bfloat16()
    k = torch.randn(1, S, Hk, D, generator=g).cuda().bfloat16()
    v = torch.randn(1, S, Hk, D, generator=g).cuda().bfloat16()
    do = torch.randn(1, S, Hq, D, generator=g).cuda().bfloat16()
    mask = A.AttnMask.bitfield(_one_image_bits(S))
    out, lse = A.attention_forward(q, k, v, mask)
    dq, dk, dv = A.attention_backward(do, q, k, v, out, lse, mask)
    group = Hq // Hk
    for hk in (0, Hk - 1):  # two key heads: the oracle of one group holds 4 x 8192 x 8192 fp32 scores
        hs = slice(hk * group, (hk + 1) * group)
        qf = q[:, :, hs].float().requires_grad_(True)
        kf = k[:, :, hk : hk + 1].float().requires_grad_(True)
        vf = v[:, :, hk : hk + 1].float().requires_grad_(True)
        ro, _ = A.attention_reference(qf, kf, vf, mask)
        ro.backward(do[:, :, hs].float())
        # 5e-3 relative to the largest reference value, the bound the reference's own kernel tests use
        # (tests/test_kernel/test_bitfield_attention.py:196-204)
        assert _rel(out[:, :, hs], ro) <= 5e-3
        assert _rel(dq[:, :, hs], qf.grad) <= 5e-3
        assert _rel(dk[:, :, hk : hk + 1], kf.grad) <= 5e-3
        assert _rel(dv[:, :, hk : hk + 1], vf.grad) <= 5e-3
        del qf, kf, vf, ro
        torch.cuda.empty_cache()


def test_attention_siglip_shape_backward():
    B, S, H, D = 4, 729, 16, 72
    g = torch.Generator().manual_seed(1)
    q, k, v, do = (torch.randn(B, S, H, D, generator=g).cuda().bfloat16() for _ in range(4))
    mask = A.AttnMask.full()
    out, lse = A.attention_forward(q, k, v, mask)
    dq, dk, dv = A.attention_backward(do, q, k, v, out, lse, mask)
    qf, kf, vf = (t.float().requires_grad_(True) for t in (q, k, v))
    ro, _ = A.attention_reference(qf, kf, vf, mask)
    ro.backward(do.float())
    assert _rel(out, ro) <= 5e-3
    assert _rel(dq, qf.grad) <= 5e-3
    assert _rel(dk, kf.grad) <= 5e-3
    assert _rel(dv, vf.grad) <= 5e-3


def test_gemm_gate_up_shape():
    M, N, K = 8192, 28672, 4096
    g = torch.Generator().manual_seed(2)
    a = torch.randn(M, K, generator=g).cuda().bfloat16()
    b = (torch.randn(N, K, generator=g) * 0.02).cuda().bfloat16()
    y = gemm(a, b)
    # fp32 reference on a band of rows and all columns, and on a band of columns and all rows (the whole product in fp32
    # would need 0.9 GB for the result alone; the bands cross every tile row and tile column)
    rows = torch.arange(0, M, 37, device="cuda")
    ref_r = a[rows].float() @ b.float().t()
    assert _rel(y[rows], ref_r) <= 5e-3
    cols = torch.arange(0, N, 53, device="cuda")
    ref_c = a.float() @ b[cols].float().t()
    assert _rel(y[:, cols], ref_c) <= 5e-3
