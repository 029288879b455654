"""Grouped (per-expert) linears: one GEMM launch over all groups against one ``F.linear`` per group in fp32, forward, input
gradients and weight gradients; the capacity-mode MoE pass built on it against the experts run one after the other."""

import pytest
import torch
import torch.nn.functional as F

from cornstarch_b200.ops.gemm import grouped_gemm, grouped_gemm_supported
from cornstarch_b200.ops.linear import _GroupedLinearFn, grouped_multi_linear


def _reference(x, groups, R):
    outs = []
    for g, ws in enumerate(groups):
        seg = x[g * R : (g + 1) * R]
        outs.append(torch.cat([F.linear(seg, w) for w in ws], dim=-1))
    return torch.cat(outs, dim=0)


def _make(G, R, K, widths, dtype, device):
    gen = torch.Generator().manual_seed(0)
    x = (torch.randn(G * R, K, generator=gen) * 0.5).to(dtype).to(device)
    groups = [[(torch.randn(n, K, generator=gen) * 0.1).to(dtype).to(device) for n in widths] for _ in range(G)]
    return x, groups


def _leaves(groups, widths, adjacent):
    """Trainable copies of the weights: separate tensors, or (adjacent) one stacked leaf per group with the weights as views
    that sit back to back in its storage, as the optimizer's parameter arena lays them out."""
    if not adjacent:
        leaves = [w.clone().requires_grad_() for ws in groups for w in ws]
        n = len(widths)
        return leaves, [leaves[n * g : n * (g + 1)] for g in range(len(groups))]
    leaves = [torch.cat(ws, dim=0).contiguous().requires_grad_() for ws in groups]
    views = []
    for leaf in leaves:
        o, ws = 0, []
        for n in widths:
            ws.append(leaf[o : o + n])
            o += n
        views.append(ws)
    return leaves, views


@pytest.mark.parametrize("adjacent", [False, True])
def test_grouped_linear_autograd_on_cpu(adjacent):
    G, R, K, widths = 3, 8, 16, [12, 20]
    x, groups = _make(G, R, K, widths, torch.float32, "cpu")
    xa, xb = x.clone().requires_grad_(), x.clone().requires_grad_()
    la, ga = _leaves(groups, widths, adjacent)
    lb, gb = _leaves(groups, widths, adjacent)
    ya = _reference(xa, ga, R)
    yb = _GroupedLinearFn.apply(xb, R, len(widths), *[w for ws in gb for w in ws])
    assert torch.allclose(ya, yb, atol=1e-5)
    gy = torch.randn_like(ya)
    ya.backward(gy)
    yb.backward(gy)
    assert torch.allclose(xa.grad, xb.grad, atol=1e-5)
    for wa, wb in zip(la, lb):
        assert torch.allclose(wa.grad, wb.grad, atol=1e-5)


def test_grouped_multi_linear_without_the_native_path():
    """On the CPU ``grouped_multi_linear`` is one ``F.linear`` per group: every weight sees only its group's rows."""
    G, R, K, widths = 2, 8, 16, [12]
    x, groups = _make(G, R, K, widths, torch.float32, "cpu")
    ws = [g[0].requires_grad_() for g in groups]
    y = grouped_multi_linear(x, [[w] for w in ws], R)
    y.sum().backward()
    for g, w in enumerate(ws):
        assert torch.allclose(w.grad, x[g * R : (g + 1) * R].sum(0).expand_as(w), atol=1e-5)


def test_grouped_pass_over_experts_equals_the_loop_on_cpu():
    from cornstarch_b200.models.moe import _SwiGLUExpert, experts_forward_grouped

    torch.manual_seed(0)
    experts = torch.nn.ModuleList([_SwiGLUExpert(16, 24) for _ in range(3)])
    x3 = torch.randn(3, 8, 16)
    want = torch.stack([experts[e](x3[e], "silu") for e in range(3)])
    got = experts_forward_grouped(experts, x3, "silu")
    assert torch.allclose(want, got, atol=1e-6)


@pytest.mark.gpu
@pytest.mark.parametrize("b_mn_major", [False, True])
@pytest.mark.parametrize("G,R,N,K", [(3, 256, 384, 320), (8, 512, 1024, 512), (2, 256, 96, 64)])
def test_grouped_gemm_one_launch(G, R, N, K, b_mn_major):
    gen = torch.Generator().manual_seed(1)
    a = (torch.randn(G * R, K, generator=gen) * 0.5).bfloat16().cuda()
    shape = (K, N) if b_mn_major else (N, K)
    bs = [(torch.randn(*shape, generator=gen) * 0.1).bfloat16().cuda() for _ in range(G)]
    assert grouped_gemm_supported(a, bs, R)
    out = grouped_gemm(a, bs, R, b_mn_major=b_mn_major)
    for g in range(G):
        B = bs[g].float().t() if b_mn_major else bs[g].float()
        want = a[g * R : (g + 1) * R].float() @ B.t()
        err = (out[g * R : (g + 1) * R].float() - want).abs().max().item()
        assert err <= 5e-3 * max(1.0, want.abs().max().item()), (g, err)
    # accumulate into an fp32 output
    acc = torch.ones(G * R, N, device="cuda")
    grouped_gemm(a, bs, R, b_mn_major=b_mn_major, out=acc, accumulate=True)
    assert torch.allclose(acc - 1.0, out.float(), atol=2e-2, rtol=2e-2)
    from cornstarch_b200.ops import _native as nat

    nat.check_status()


@pytest.mark.gpu
@pytest.mark.parametrize("adjacent", [False, True])
def test_grouped_multi_linear_on_the_device(adjacent):
    G, R, K, widths = 4, 256, 256, [384, 384]
    x, groups = _make(G, R, K, widths, torch.bfloat16, "cuda")
    leaves, gb = _leaves(groups, widths, adjacent)
    xa = x.float().requires_grad_()
    ga = [[w.float().requires_grad_() for w in ws] for ws in groups]
    xb = x.clone().requires_grad_()
    ya = _reference(xa, ga, R)
    yb = grouped_multi_linear(xb, gb, R)
    gy = torch.randn_like(ya)
    ya.backward(gy)
    yb.backward(gy.bfloat16())

    def close(got, want, what):
        err = (got.float() - want).abs().max().item()
        assert err <= 2e-2 * max(1.0, want.abs().max().item()), (what, err)

    close(yb, ya, "y")
    close(xb.grad, xa.grad, "dx")
    want = [torch.cat([w.grad for w in ws], dim=0) for ws in ga] if adjacent else [w.grad for ws in ga for w in ws]
    for i, (leaf, w) in enumerate(zip(leaves, want)):
        close(leaf.grad, w, f"dW[{i}]")
