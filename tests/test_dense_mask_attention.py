"""Flash attention with a dense boolean mask and / or an additive bias on the attention kernels
(``flash_attn_func(q, k, v, bias, mask)``), over the grid of the reference's own test
(tests/test_kernel/test_attention.py:10-108: head dims 32 / 64 / 128, query x key lengths from 57 to 1024, its
"multimodal" mask) plus a random mask, a bias, GQA and batches; forward and gradients against an fp32 PyTorch oracle
within the reference's tolerance (5e-3)."""

import pytest
import torch

from cornstarch_b200.kernel.attention import flash_attn_func
from cornstarch_b200.ops import attention as A

pytestmark = pytest.mark.gpu

SEQLENS = [(128, 128), (128, 1024), (1024, 128), (1024, 1024), (57, 57), (144, 144), (283, 283)]


def _oracle(q, k, v, mask, bias, g):
    qf, kf, vf = (t.detach().float().requires_grad_() for t in (q, k, v))
    m = A.AttnMask.from_dense(mask, bias)
    o, _ = A.attention_reference(qf, kf, vf, m)
    dq, dk, dv = torch.autograd.grad(o, (qf, kf, vf), g.float())
    return o, dq, dk, dv


def _multimodal_mask(B, Sq, Sk, dev):
    mask = torch.tril(torch.ones(B, Sq, Sk, device=dev, dtype=torch.bool), diagonal=0)
    mask[:, 12:24, :] = False
    mask[:, 12:24, 12:24] = True
    mask[:, 36:56, :] = False
    mask[:, 36:56, 36:56] = True
    return mask


def _check(got, want):
    """Outputs: the reference's tolerance (rtol = atol = 5e-3).  Gradients: the same relative tolerance with the absolute
    part scaled by the largest gradient entry: they are sums over up to 1024 products of bf16-rounded probabilities, so
    their rounding error grows with the magnitude of the sum, and the oracle here is fp32 (the reference's own test
    compares two bf16 implementations with each other)."""
    for a, b, name in zip(got, want, ("o", "dq", "dk", "dv")):
        atol = 5e-3 if name == "o" else 5e-3 * max(1.0, float(b.float().abs().max()))
        torch.testing.assert_close(a.float(), b.float(), rtol=5e-3, atol=atol, msg=lambda m, n=name: f"{n}: {m}")


@pytest.mark.parametrize("head_dim", [32, 64, 128])
@pytest.mark.parametrize("seqlen", SEQLENS, ids=[f"{a}x{b}" for a, b in SEQLENS])
def test_dense_mask_grid_of_the_reference(head_dim, seqlen):
    dev = torch.device("cuda")
    Sq, Sk = seqlen
    torch.manual_seed(0)
    q = (torch.randn(1, Sq, 12, head_dim, device=dev) * 0.5).bfloat16().requires_grad_()
    k = (torch.randn(1, Sk, 12, head_dim, device=dev) * 0.5).bfloat16().requires_grad_()
    v = (torch.randn(1, Sk, 12, head_dim, device=dev) * 0.5).bfloat16().requires_grad_()
    mask = _multimodal_mask(1, Sq, Sk, dev)
    out = flash_attn_func(q, k, v, mask=mask)
    g = torch.randn_like(out)
    dq, dk, dv = torch.autograd.grad(out, (q, k, v), g)
    _check((out, dq, dk, dv), _oracle(q, k, v, mask, None, g))


@pytest.mark.parametrize("case", ["random_mask", "bias_only", "mask_and_bias", "vector_bias", "gqa_batch"])
def test_dense_mask_and_bias_variants(case):
    dev = torch.device("cuda")
    torch.manual_seed(1)
    B, Sq, Sk, Hq, Hk, D = (2, 300, 411, 8, 2, 64) if case == "gqa_batch" else (1, 283, 283, 6, 6, 64)
    q = (torch.randn(B, Sq, Hq, D, device=dev) * 0.5).bfloat16().requires_grad_()
    k = (torch.randn(B, Sk, Hk, D, device=dev) * 0.5).bfloat16().requires_grad_()
    v = (torch.randn(B, Sk, Hk, D, device=dev) * 0.5).bfloat16().requires_grad_()
    mask = bias = None
    if case in ("random_mask", "mask_and_bias", "gqa_batch"):
        mask = torch.rand(B, Sq, Sk, device=dev) < 0.6
        mask[:, :, 0] = True  # no fully masked row (an fp32 softmax over an empty row is undefined in the oracle too)
        mask[:, 130:260, 128:256] = False  # a whole tile without an allowed pair
        mask[:, 0:128, 128:256] = True     # a whole tile with every pair allowed
    if case in ("bias_only", "mask_and_bias", "gqa_batch"):
        bias = torch.randn(B, Hq, Sq, Sk, device=dev)
    if case == "vector_bias":
        bias = torch.randn(1, Hq, 1, Sk, device=dev)  # ALiBi-style: one value per head and key
    out = flash_attn_func(q, k, v, bias=bias, mask=mask)
    g = torch.randn_like(out)
    dq, dk, dv = torch.autograd.grad(out, (q, k, v), g)
    _check((out, dq, dk, dv), _oracle(q, k, v, mask, bias, g))


def test_cornstarch_attention_forward_stays_on_the_kernel(monkeypatch):
    """The HF attention-interface adapter with a dense mask calls the native forward (never the PyTorch statement)."""
    from cornstarch_b200.kernel.interface import cornstarch_attention_forward

    calls = []
    real = A.attention_forward
    monkeypatch.setattr(A, "attention_forward", lambda *a, **k: (calls.append(1), real(*a, **k))[1])
    monkeypatch.setattr(A, "attention_reference", lambda *a, **k: (_ for _ in ()).throw(AssertionError("PyTorch path used")))
    dev = torch.device("cuda")
    q = torch.randn(1, 4, 200, 64, device=dev).bfloat16()
    mask = _multimodal_mask(1, 200, 200, dev)
    out, _ = cornstarch_attention_forward(None, q, q, q, mask)
    assert calls and out.shape == (1, 200, 4, 64)
