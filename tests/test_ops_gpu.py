"""Fused elementwise / norm / loss / optimizer kernels vs plain PyTorch fp32 statements of the same ops."""

import pytest
import torch
import torch.nn.functional as F

from cornstarch_b200.ops import elementwise as E
from cornstarch_b200.ops.cross_entropy import linear_cross_entropy
from cornstarch_b200.ops.linear import linear, multi_linear
from cornstarch_b200.optim.fused_adamw import FusedAdamW

pytestmark = pytest.mark.gpu
TOL = 2e-2


def close(a, b, tol=TOL):
    a, b = a.float(), b.float()
    err = (a - b).abs().max().item()
    assert err <= tol * max(1.0, b.abs().max().item()), f"max err {err} vs scale {b.abs().max().item()}"


@pytest.mark.parametrize("H", [64, 1152, 4096, 8192])
@pytest.mark.parametrize("ln", [False, True])
@pytest.mark.parametrize("res", [False, True])
def test_norm_fwd_bwd(H, ln, res):
    T = 300
    x = torch.randn(T, H, device="cuda").bfloat16().requires_grad_(True)
    r = torch.randn(T, H, device="cuda").bfloat16().requires_grad_(True) if res else None
    w = (1 + 0.1 * torch.randn(H, device="cuda")).bfloat16().requires_grad_(True)
    b = (0.1 * torch.randn(H, device="cuda")).bfloat16().requires_grad_(True) if ln else None
    out = E.layer_norm(x, w, b, 1e-5, r) if ln else E.rms_norm(x, w, 1e-6, r)
    y, h = out if res else (out, None)
    xf, wf = x.detach().float().requires_grad_(True), w.detach().float().requires_grad_(True)
    rf = r.detach().float().requires_grad_(True) if res else None
    bf = b.detach().float().requires_grad_(True) if ln else None
    hf = xf + rf if res else xf
    hq = hf.detach().bfloat16().float() + (hf - hf.detach()) if res else hf  # forward normalises the bf16-rounded stream
    yf = E._norm_ref(hq, wf, bf, 1e-5 if ln else 1e-6, ln, 0.0)
    close(y, yf)
    gy = torch.randn_like(y)
    gh = torch.randn_like(y) if res else None
    if res:
        torch.autograd.backward([y, h], [gy, gh])
        torch.autograd.backward([yf, hf], [gy.float(), gh.float()])
        close(h, hf)
        close(r.grad, rf.grad)
    else:
        y.backward(gy)
        yf.backward(gy.float())
    close(x.grad, xf.grad)
    close(w.grad, wf.grad, 5e-2)
    if ln:
        close(b.grad, bf.grad, 5e-2)


def test_rope_inplace_fwd_bwd():
    B, S, Hq, Hk, D = 2, 96, 8, 2, 128
    W = (Hq + 2 * Hk) * D
    cos, sin = E.rope_tables(256, D, 500000.0, "cuda")
    pos = torch.randint(0, 256, (B, S), device="cuda").int()
    base = torch.randn(B, S, W, device="cuda").bfloat16()
    x = base.clone().requires_grad_(True)
    y = E.rope_(x * 1.0, cos, sin, pos, Hq + Hk, D)
    ref_in = base.float().requires_grad_(True)
    qk = E._rope_ref(ref_in[..., : (Hq + Hk) * D].reshape(B, S, Hq + Hk, D), cos, sin, pos, D)
    ref = torch.cat([qk.reshape(B, S, -1), ref_in[..., (Hq + Hk) * D :]], dim=-1)
    close(y, ref)
    g = torch.randn_like(y)
    y.backward(g.clone())
    ref.backward(g.float())
    close(x.grad, ref_in.grad)


@pytest.mark.parametrize("act", ["silu", "gelu_pytorch_tanh"])
def test_glu(act):
    x = torch.randn(333, 2 * 1408, device="cuda").bfloat16().requires_grad_(True)
    y = E.glu(x, act)
    xf = x.detach().float().requires_grad_(True)
    yf = E._act_ref(xf[..., :1408], act) * xf[..., 1408:]
    close(y, yf)
    g = torch.randn_like(y)
    y.backward(g)
    yf.backward(g.float())
    close(x.grad, xf.grad)


@pytest.mark.parametrize("name", ["gelu", "gelu_pytorch_tanh", "quick_gelu", "silu"])
def test_activation(name):
    x = (3 * torch.randn(257, 512, device="cuda")).bfloat16().requires_grad_(True)
    y = E.activation(x, name)
    xf = x.detach().float().requires_grad_(True)
    yf = E._act_ref(xf, name)
    close(y, yf)
    g = torch.randn_like(y)
    y.backward(g)
    yf.backward(g.float())
    close(x.grad, xf.grad)


def test_embed_merge_fwd_bwd():
    V, H, T, NF = 500, 256, 300, 40
    w = torch.randn(V, H, device="cuda").bfloat16().requires_grad_(True)
    feats = torch.randn(NF, H, device="cuda").bfloat16().requires_grad_(True)
    src = torch.randint(0, V, (T,), device="cuda").int()
    where = torch.randperm(T, device="cuda")[:NF]
    src[where] = -(torch.arange(NF, device="cuda").int()) - 1
    out = E.embed_merge(w, src, feats)
    ref = torch.where((src < 0)[:, None], feats.float()[(-src.long() - 1).clamp(min=0)], w.float()[src.long().clamp(min=0)])
    close(out, ref, 1e-6)
    g = torch.randn_like(out)
    out.backward(g)
    wf, ff = w.detach().float().requires_grad_(True), feats.detach().float().requires_grad_(True)
    ref2 = torch.where((src < 0)[:, None], ff[(-src.long() - 1).clamp(min=0)], wf[src.long().clamp(min=0)])
    ref2.backward(g.float())
    close(w.grad, wf.grad)
    close(feats.grad, ff.grad)


def test_merge_features_into_given_embeddings():
    """The merge kernel with already embedded tokens as its table (what a vocabulary-parallel model does after its
    embedding all-reduce): row t keeps ``flat[t]`` or takes a feature row; both inputs get their gradients."""
    from cornstarch_b200.ops.elementwise import embed_merge

    T, H, NF = 1000, 256, 37
    flat = torch.randn(T, H, device="cuda").bfloat16().requires_grad_(True)
    feats = torch.randn(NF, H, device="cuda").bfloat16().requires_grad_(True)
    src = torch.arange(T, device="cuda", dtype=torch.int32)
    where = torch.randperm(T, device="cuda")[:NF].sort().values
    src[where] = -(torch.arange(NF, device="cuda", dtype=torch.int32)) - 1
    out = embed_merge(flat, src, feats)
    ff, fe = flat.detach().float().requires_grad_(True), feats.detach().float().requires_grad_(True)
    ref = ff.clone()
    ref[where] = fe
    close(out, ref)
    g = torch.randn_like(out)
    out.backward(g)
    ref.backward(g.float())
    close(flat.grad, ff.grad)
    close(feats.grad, fe.grad)


@pytest.mark.parametrize("keep", [False, True])
@pytest.mark.parametrize("V", [1000, 128256])
def test_linear_cross_entropy(V, keep):
    """``keep``: the logits stay resident for the backward pass (what small problems do by default) or are recomputed."""
    T, H = 700, 256
    h = torch.randn(T, H, device="cuda").bfloat16().requires_grad_(True)
    w = (0.05 * torch.randn(V, H, device="cuda")).bfloat16().requires_grad_(True)
    labels = torch.randint(0, V, (T,), device="cuda")
    labels[::7] = -100
    loss = linear_cross_entropy(h, w, labels, chunk=256, keep_logits=keep)
    hf, wf = h.detach().float().requires_grad_(True), w.detach().float().requires_grad_(True)
    ref = F.cross_entropy(F.linear(hf, wf), labels, ignore_index=-100)
    assert abs(loss.item() - ref.item()) < 2e-2 * max(1.0, abs(ref.item()))
    (loss * 3.0).backward()
    (ref * 3.0).backward()
    close(h.grad, hf.grad, 3e-2)
    close(w.grad, wf.grad, 3e-2)


def test_multi_linear_fused_and_main_grad():
    T, K = 512, 256
    flat = (0.05 * torch.randn(3 * 128 * K, device="cuda")).bfloat16()
    ws = [torch.nn.Parameter(flat[i * 128 * K : (i + 1) * 128 * K].view(128, K)) for i in range(3)]
    gflat = torch.zeros(3 * 128 * K, device="cuda", dtype=torch.bfloat16)
    for i, w in enumerate(ws):
        w.main_grad = gflat[i * 128 * K : (i + 1) * 128 * K].view(128, K)
    x = torch.randn(T, K, device="cuda").bfloat16().requires_grad_(True)
    y = multi_linear(x, ws)
    ref = torch.cat([F.linear(x.float(), w.float()) for w in ws], dim=-1)
    close(y, ref)
    g = torch.randn_like(y)
    y.backward(g)
    close(x.grad, g.float() @ torch.cat([w.float() for w in ws], dim=0))
    close(gflat.view(384, K), g.float().t() @ x.float(), 3e-2)
    assert all(w.grad is None for w in ws)


def test_linear_bias_grad():
    x = torch.randn(300, 128, device="cuda").bfloat16().requires_grad_(True)
    w = torch.nn.Parameter((0.1 * torch.randn(64, 128, device="cuda")).bfloat16())
    b = torch.nn.Parameter(torch.randn(64, device="cuda").bfloat16())
    y = linear(x, w, b)
    g = torch.randn_like(y)
    y.backward(g)
    close(y, F.linear(x.float(), w.float(), b.float()))
    close(b.grad, g.float().sum(0), 3e-2)
    close(w.grad, g.float().t() @ x.float(), 3e-2)


def test_fused_adamw_matches_reference_math():
    torch.manual_seed(0)
    p_gpu = [torch.nn.Parameter(torch.randn(257, 64, device="cuda").bfloat16()), torch.nn.Parameter(torch.randn(64, device="cuda").bfloat16())]
    p_cpu = [torch.nn.Parameter(p.detach().float().cpu().clone()) for p in p_gpu]
    opt_g = FusedAdamW([{"params": [p_gpu[0]], "weight_decay": 0.1}, {"params": [p_gpu[1]], "weight_decay": 0.0}], lr=1e-2, max_norm=1.0)
    opt_c = FusedAdamW([{"params": [p_cpu[0]], "weight_decay": 0.1}, {"params": [p_cpu[1]], "weight_decay": 0.0}], lr=1e-2, max_norm=1.0)
    assert opt_g.use_arena and not opt_c.use_arena
    for step in range(3):
        gs = [torch.randn_like(p, dtype=torch.float32) for p in p_cpu]
        for p, g in zip(p_gpu, gs):
            p.main_grad.copy_(g.cuda().to(p.main_grad.dtype))
        for p, g in zip(p_cpu, gs):
            p.grad = g.bfloat16().float()
        opt_g.step()
        opt_c.step()
        opt_g.zero_grad()
    for pg, pc in zip(p_gpu, p_cpu):
        close(pg.detach().cpu(), pc.detach(), 1e-2)
    assert float(p_gpu[0].main_grad.abs().max()) == 0.0


def test_smoke_entry():
    import __graft_entry__ as g

    g.smoke()


def test_fused_adamw_split_master_equals_fp32_master():
    """Master weights kept as bf16 parameter + 16-bit remainder follow exactly the trajectory of whole fp32 master
    weights; the bf16 parameters agree except where the master sits exactly between two bf16 values."""
    torch.manual_seed(1)
    init = torch.randn(1 << 18, device="cuda").bfloat16()
    runs = {}
    for split in (False, True):
        p = torch.nn.Parameter(init.clone())
        # no clipping: the gradient norm is summed with atomics, so two runs may differ in its last bit
        opt = FusedAdamW([{"params": [p], "weight_decay": 0.05}], lr=3e-3, max_norm=0.0, split_master=split)
        assert opt.use_arena and opt._regions[0][1].split_master == split
        g = torch.Generator(device="cuda").manual_seed(7)
        for _ in range(5):
            p.main_grad.copy_(torch.randn(init.shape, device="cuda", generator=g).bfloat16())
            opt.step()
        runs[split] = (opt._regions[0][1].master_weights().clone(), p.detach().clone(), opt.state_dict())
    assert torch.equal(runs[True][0], runs[False][0])
    diff = runs[True][1].float() - runs[False][1].float()
    assert int((diff != 0).sum()) <= 64 and float(diff.abs().max()) <= float(init.float().abs().max()) * 2.0 ** -7
    # a state dict written by one representation loads into the other
    p2 = torch.nn.Parameter(init.clone())
    opt2 = FusedAdamW([{"params": [p2], "weight_decay": 0.05}], lr=3e-3, max_norm=0.0, split_master=True)
    opt2.load_state_dict(runs[False][2])
    assert torch.equal(opt2._regions[0][1].master_weights(), runs[False][0])
