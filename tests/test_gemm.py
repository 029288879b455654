"""tcgen05 GEMM vs an fp32 PyTorch reference: every operand orientation, tile width, ragged edges,
bias / activation / accumulate epilogues."""

import pytest
import torch

from cornstarch_b200.ops.gemm import gemm, gemm_reference

pytestmark = pytest.mark.gpu


def _mk(M, N, K, a_mn, b_mn, dev="cuda"):
    g = torch.Generator(device="cpu").manual_seed(M * 7 + N * 3 + K)
    a = torch.randn((K, M) if a_mn else (M, K), generator=g).to(dev, torch.bfloat16)
    b = torch.randn((K, N) if b_mn else (N, K), generator=g).to(dev, torch.bfloat16)
    return a, b


def _check(out, ref, K):
    tol = 2e-2 * (K ** 0.5) / 8 + 1e-2
    err = (out.float() - ref.float()).abs().max().item()
    scale = ref.float().abs().max().item() + 1e-6
    assert err <= 8e-3 * scale + tol * 0.05, f"max err {err} (scale {scale})"


@pytest.mark.parametrize("a_mn", [False, True])
@pytest.mark.parametrize("b_mn", [False, True])
@pytest.mark.parametrize("tile_n", [128, 256])
@pytest.mark.parametrize("shape", [(128, 256, 64), (256, 512, 256), (384, 1024, 1024), (1000, 776, 520), (729, 1152, 4304)])
def test_gemm_orientations(a_mn, b_mn, tile_n, shape):
    M, N, K = shape
    a, b = _mk(M, N, K, a_mn, b_mn)
    out = gemm(a, b, a_mn, b_mn, tile_n=tile_n)
    ref = gemm_reference(a, b, a_mn, b_mn, out_dtype=torch.float32)
    torch.cuda.synchronize()
    _check(out, ref, K)


@pytest.mark.parametrize("act", [None, "gelu_tanh", "gelu", "silu"])
def test_gemm_bias_act(act):
    M, N, K = 512, 768, 384
    a, b = _mk(M, N, K, False, False)
    bias = torch.randn(N, device="cuda").to(torch.bfloat16)
    out = gemm(a, b, bias=bias, act=act)
    ref = gemm_reference(a, b, bias=bias, act=act, out_dtype=torch.float32)
    _check(out, ref, K)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_gemm_accumulate(dtype):
    M, N, K = 640, 512, 2048
    a, b = _mk(M, N, K, True, True)
    c0 = torch.randn(M, N, device="cuda").to(dtype)
    out = c0.clone()
    gemm(a, b, True, True, out=out, accumulate=True)
    ref = gemm_reference(a, b, True, True, out_dtype=torch.float32) + c0.float()
    _check(out, ref, K)


def test_gemm_strided_views_and_persistence():
    # operands that are column slices of wider buffers (fused qkv style) and more tiles than SMs
    M, N, K = 4096, 4096, 512
    big = torch.randn(M, K + 256, device="cuda").to(torch.bfloat16)
    a = big[:, 128 : 128 + K]
    b = torch.randn(N, K, device="cuda").to(torch.bfloat16)
    outbuf = torch.zeros(M, N + 64, device="cuda", dtype=torch.bfloat16)
    out = outbuf[:, :N]
    gemm(a, b, out=out)
    ref = a.float() @ b.float().t()
    _check(out, ref, K)
    assert outbuf[:, N:].abs().max().item() == 0


def test_gemm_status_clean():
    from cornstarch_b200.ops import _native as nat

    assert nat.check_status() == 0
