"""Packed variable-length attention (the calling convention of flash-attn's varlen functions, which the reference uses
for InternViT, cornstarch/models/intern_vit/flash_attention.py) against per-sequence softmax attention in fp32."""

import math

import pytest
import torch

import cornstarch_b200.kernel.attention as KA


def _per_sequence(q, k, v, cu, causal):
    outs = []
    for a, b in zip(cu[:-1], cu[1:]):
        qq, kk, vv = (t[a:b].transpose(0, 1).float() for t in (q, k, v))
        s = qq @ kk.transpose(-1, -2) / math.sqrt(q.shape[-1])
        if causal:
            s = s.masked_fill(~torch.ones(b - a, b - a, dtype=torch.bool, device=q.device).tril(), float("-inf"))
        outs.append((s.softmax(-1) @ vv).transpose(0, 1))
    return torch.cat(outs)


def _case(device, dtype, limit, causal, tol):
    torch.manual_seed(0)
    lens = [37, 130, 5, 200, 128]
    cu = torch.tensor([0] + torch.tensor(lens).cumsum(0).tolist(), dtype=torch.int32, device=device)
    q, k, v = (torch.randn(sum(lens), 4, 64, device=device, dtype=dtype).requires_grad_(True) for _ in range(3))
    old, KA._MAX_PACKED_SEQUENCES = KA._MAX_PACKED_SEQUENCES, limit
    try:
        out = KA.flash_attn_varlen_func(q, k, v, cu, max(lens), causal=causal)
    finally:
        KA._MAX_PACKED_SEQUENCES = old
    qr, kr, vr = (t.detach().float().requires_grad_(True) for t in (q, k, v))
    want = _per_sequence(qr, kr, vr, cu.tolist(), causal)
    assert (out.float() - want).abs().max().item() < tol
    w = torch.randn_like(want)
    (out.float() * w).sum().backward()
    (want * w).sum().backward()
    for got, ref in ((q.grad, qr.grad), (k.grad, kr.grad), (v.grad, vr.grad)):
        assert (got.float() - ref).abs().max().item() < tol * max(1.0, ref.abs().max().item())


@pytest.mark.parametrize("causal", [False, True])
@pytest.mark.parametrize("limit", [60, 2], ids=["one_masked_sequence", "padded_batch"])
def test_varlen_matches_per_sequence_attention(limit, causal):
    # fp32 on the CPU: the packed and the per-sequence products sum in different orders (1e-5 failed once on a many-core host)
    _case("cpu", torch.float32, limit, causal, 1e-4)


@pytest.mark.gpu
@pytest.mark.parametrize("causal", [False, True])
@pytest.mark.parametrize("limit", [60, 2], ids=["one_masked_sequence", "padded_batch"])
def test_varlen_on_the_kernel(limit, causal):
    _case("cuda", torch.bfloat16, limit, causal, 4e-2)


def test_flash_attention_module_with_padding_mask():
    torch.manual_seed(1)
    B, S, H, D = 2, 50, 2, 16
    qkv = torch.randn(B, S, 3, H, D)
    keep = torch.ones(B, S, dtype=torch.bool)
    keep[1, 30:] = False
    out, _ = KA.FlashAttention()(qkv, key_padding_mask=keep)
    assert out.shape == (B, S, H, D) and out[1, 30:].abs().max() == 0
    cu = [0, 50]
    full = _per_sequence(qkv[0, :, 0], qkv[0, :, 1], qkv[0, :, 2], cu, False)
    assert torch.allclose(out[0], full, atol=1e-5)
    part = _per_sequence(qkv[1, :30, 0], qkv[1, :30, 1], qkv[1, :30, 2], [0, 30], False)
    assert torch.allclose(out[1, :30], part, atol=1e-5)
    # the packed form of the same call
    packed = torch.cat([qkv[0], qkv[1, :30]])
    out2, _ = KA.FlashAttention()(packed, cu_seqlens=torch.tensor([0, 50, 80], dtype=torch.int32), max_s=50)
    assert torch.allclose(out2, torch.cat([out[0], out[1, :30]]), atol=1e-5)
