"""Flash attention kernels (tcgen05) vs the fp32 dense-mask reference: causal / full / bitfield masks,
GQA, ragged sequence lengths, head dims 32..128, strided q/k/v views, explicit positions."""

import math

import pytest
import torch

from cornstarch_b200.ops import attention as A

pytestmark = pytest.mark.gpu
# Bound on max|kernel - oracle| / max(1, max|oracle|).  The outputs are bf16: one unit in the last place at the largest
# magnitude is 2^-8 = 3.9e-3 of it, and P is rounded to bf16 before P V (and dS before dK / dQ), so a few such roundings
# add up on the small, short cases here (10 of 120 cases exceed 5e-3).  At the benchmark shapes, where sums run
# over thousands of keys, the kernels stay inside the reference's 5e-3 (tests/test_benchmark_shapes.py).
TOL = 5e-3 * 4


def make_bitfield(B, S, n_modal=2, seed=0, pad_tail=0):
    """text = bit0 | bit62 | all modality bits; modality i = 1 << (i+1); zeros = padding."""
    g = torch.Generator().manual_seed(seed)
    text = (1 << 62) | 1
    for i in range(n_modal):
        text |= 1 << (i + 1)
    bits = torch.full((B, S), text, dtype=torch.int64)
    for b in range(B):
        pos = 0
        for i in range(n_modal):
            L = int(torch.randint(max(S // 16, 1), max(S // 4, 2), (1,), generator=g))
            start = int(torch.randint(pos, max(pos + 1, S - (n_modal - i) * L - 1), (1,), generator=g))
            bits[b, start : start + L] = 1 << (i + 1)
            pos = start + L
        if pad_tail:
            bits[b, S - pad_tail :] = 0
    return bits


def _qkv(B, Sq, Sk, Hq, Hk, D, seed=0):
    g = torch.Generator().manual_seed(seed)
    q = torch.randn(B, Sq, Hq, D, generator=g).cuda().bfloat16()
    k = torch.randn(B, Sk, Hk, D, generator=g).cuda().bfloat16()
    v = torch.randn(B, Sk, Hk, D, generator=g).cuda().bfloat16()
    return q, k, v


def _close(a, b, tol=TOL):
    a, b = a.float(), b.float()
    err = (a - b).abs().max().item()
    assert err <= tol * max(1.0, b.abs().max().item()), f"max err {err}"


@pytest.mark.parametrize("D", [32, 64, 72, 128])
@pytest.mark.parametrize("S", [57, 128, 283, 1024])
@pytest.mark.parametrize("mode", ["causal", "full"])
def test_fwd_dense_modes(D, S, mode):
    q, k, v = _qkv(2, S, S, 4, 4, D, seed=S + D)
    mask = A.AttnMask.causal() if mode == "causal" else A.AttnMask.full()
    o, lse = A.attention_forward(q, k, v, mask)
    ro, rlse = A.attention_reference(q, k, v, mask)
    _close(o, ro)
    _close(lse, rlse, 2e-2)


@pytest.mark.parametrize("hk", [1, 2, 3, 6])
@pytest.mark.parametrize("S", [144, 512, 1200])
@pytest.mark.parametrize("prefix", [False, True])
def test_fwd_bitfield_gqa(hk, S, prefix):
    B, Hq, D = 2, 6, 64
    q, k, v = _qkv(B, S, S, Hq, hk, D, seed=S + hk)
    bits = make_bitfield(B, S, seed=S, pad_tail=5).cuda()
    mask = A.AttnMask.bitfield(bits, prefix_causal=prefix)
    o, lse = A.attention_forward(q, k, v, mask)
    ro, rlse = A.attention_reference(q, k, v, mask)
    _close(o, ro)
    finite = torch.isfinite(rlse)
    assert torch.equal(torch.isfinite(lse), finite)
    _close(lse[finite], rlse[finite], 2e-2)


def test_mask_classes_match_dense():
    B, S = 2, 777
    bits = make_bitfield(B, S, n_modal=3, seed=3, pad_tail=9).cuda()
    for mode in (A.MASK_BITFIELD, A.MASK_BITFIELD_PREFIX_CAUSAL, A.MASK_CAUSAL, A.MASK_FULL):
        m = A.AttnMask(mode=mode, q_bits=bits, k_bits=bits)
        got = A.classify_mask(m, B, S, S, "cuda")
        ref = A.classify_mask(A.AttnMask(mode=mode, q_bits=bits.cpu(), k_bits=bits.cpu()), B, S, S, "cpu")
        assert torch.equal(got.cpu(), ref)


def test_fwd_strided_qkv_and_cross_lengths():
    # q/k/v as slices of one fused projection buffer; Sq != Sk with explicit positions (context-parallel style)
    B, Sq, Sk, Hq, Hk, D = 1, 256, 640, 8, 2, 128
    g = torch.Generator().manual_seed(5)
    fused = torch.randn(B, Sk, (Hq + 2 * Hk) * D, generator=g).cuda().bfloat16()
    qfull = fused[..., : Hq * D].view(B, Sk, Hq, D)
    k = fused[..., Hq * D : (Hq + Hk) * D].view(B, Sk, Hk, D)
    v = fused[..., (Hq + Hk) * D :].view(B, Sk, Hk, D)
    rows = torch.arange(128, 128 + Sq)
    q = qfull[:, 128 : 128 + Sq]
    q_pos = rows[None].int().cuda()
    k_pos = torch.arange(Sk)[None].int().cuda()
    mask = A.AttnMask(mode=A.MASK_CAUSAL, q_pos=q_pos, k_pos=k_pos)
    o, lse = A.attention_forward(q, k, v, mask)
    ro, rlse = A.attention_reference(q, k, v, mask)
    _close(o, ro)
    _close(lse, rlse, 2e-2)


def _ref_grads(q, k, v, mask, do):
    qf, kf, vf = (t.detach().float().requires_grad_(True) for t in (q, k, v))
    o, _ = A.attention_reference(qf, kf, vf, mask)
    o.backward(do.float())
    return qf.grad, kf.grad, vf.grad


@pytest.mark.parametrize("D", [32, 64, 72, 128])
@pytest.mark.parametrize("S", [57, 128, 283, 512])
@pytest.mark.parametrize("mode", ["causal", "full"])
def test_bwd_dense_modes(D, S, mode):
    q, k, v = _qkv(2, S, S, 4, 2, D, seed=S * 3 + D)
    mask = A.AttnMask.causal() if mode == "causal" else A.AttnMask.full()
    do = torch.randn_like(q)
    o, lse = A.attention_forward(q, k, v, mask)
    dq, dk, dv = A.attention_backward(do, q, k, v, o, lse, mask)
    rq, rk, rv = _ref_grads(q, k, v, mask, do)
    _close(dq, rq)
    _close(dk, rk)
    _close(dv, rv)


@pytest.mark.parametrize("hk", [1, 2, 3, 6])
@pytest.mark.parametrize("S", [144, 1024])
@pytest.mark.parametrize("prefix", [False, True])
def test_bwd_bitfield_gqa(hk, S, prefix):
    B, Hq, D = 2, 6, 64
    q, k, v = _qkv(B, S, S, Hq, hk, D, seed=S + hk + 11)
    bits = make_bitfield(B, S, seed=S + 1, pad_tail=7).cuda()
    mask = A.AttnMask.bitfield(bits, prefix_causal=prefix)
    do = torch.randn_like(q)
    o, lse = A.attention_forward(q, k, v, mask)
    dq, dk, dv = A.attention_backward(do, q, k, v, o, lse, mask)
    rq, rk, rv = _ref_grads(q, k, v, mask, do)
    _close(dq, rq)
    _close(dk, rk)
    _close(dv, rv)


def test_bwd_deterministic_dkdv():
    q, k, v = _qkv(1, 640, 640, 8, 2, 128, seed=9)
    mask = A.AttnMask.causal()
    do = torch.randn_like(q)
    o, lse = A.attention_forward(q, k, v, mask)
    a = A.attention_backward(do, q, k, v, o, lse, mask)
    b = A.attention_backward(do, q, k, v, o, lse, mask)
    assert torch.equal(a[1], b[1]) and torch.equal(a[2], b[2])


def test_autograd_function_strided():
    B, S, Hq, Hk, D = 1, 384, 8, 2, 128
    fused = torch.randn(B, S, (Hq + 2 * Hk) * D, device="cuda").bfloat16().requires_grad_(True)
    q = fused[..., : Hq * D].view(B, S, Hq, D)
    k = fused[..., Hq * D : (Hq + Hk) * D].view(B, S, Hk, D)
    v = fused[..., (Hq + Hk) * D :].view(B, S, Hk, D)
    o = A.attention(q, k, v, A.AttnMask.causal())
    w = torch.randn_like(o)
    (o.float() * w.float()).sum().backward()
    ff = fused.detach().float().requires_grad_(True)
    qf = ff[..., : Hq * D].view(B, S, Hq, D)
    kf = ff[..., Hq * D : (Hq + Hk) * D].view(B, S, Hk, D)
    vf = ff[..., (Hq + Hk) * D :].view(B, S, Hk, D)
    ro, _ = A.attention_reference(qf, kf, vf, A.AttnMask.causal())
    (ro * w.float()).sum().backward()
    _close(fused.grad, ff.grad)


def test_status_clean_after_attention():
    from cornstarch_b200.ops import _native as nat

    assert nat.check_status() == 0


@pytest.mark.parametrize("sizes,my_seg", [([512, 512], 1), ([300, 180, 420], 0), ([128, 640], 1)])
@pytest.mark.parametrize("mode", ["causal", "bitfield"])
def test_kv_segments_local(sizes, my_seg, mode):
    """K/V given as several tensors (the layout of context parallelism, here all on one GPU): forward and backward
    equal the single-tensor kernels on the concatenation; the mask lives in the padded gathered index space."""
    from cornstarch_b200.parallel.cp_fused import attention_segments_local, padded_layout

    B, Hq, Hk, D = 2, 4, 2, 128
    S = sum(sizes)
    q, k, v = _qkv(B, S, S, Hq, Hk, D, seed=S)
    do = torch.randn(B, S, Hq, D, generator=torch.Generator().manual_seed(1)).cuda().bfloat16()
    pos = torch.arange(S, dtype=torch.int32).cuda()[None].expand(B, -1).contiguous()
    bits = make_bitfield(B, S, seed=S, pad_tail=3).cuda() if mode == "bitfield" else None
    ref_mask = A.AttnMask(mode=A.MASK_BITFIELD if bits is not None else A.MASK_CAUSAL, q_bits=bits, k_bits=bits, q_pos=pos, k_pos=pos)
    ro, rlse = A.attention_forward(q, k, v, ref_mask)
    rdq, rdk, rdv = A.attention_backward(do, q, k, v, ro, rlse, ref_mask)
    starts, total = padded_layout(sizes)
    kp = torch.full((B, total), -1, dtype=torch.int32, device="cuda")
    kb = torch.zeros((B, total), dtype=torch.int64, device="cuda") if bits is not None else None
    ks, vs, off = [], [], 0
    for s0, n in zip(starts, sizes):
        kp[:, s0 : s0 + n] = pos[:, off : off + n]
        if kb is not None:
            kb[:, s0 : s0 + n] = bits[:, off : off + n]
        ks.append(k[:, off : off + n].contiguous())
        vs.append(v[:, off : off + n].contiguous())
        off += n
    mask = A.AttnMask(mode=ref_mask.mode, q_bits=bits, k_bits=kb, q_pos=pos, k_pos=kp)
    o, lse, dq, dks, dvs = attention_segments_local(q, ks, vs, mask, my_seg=my_seg, do=do)
    _close(o, ro)
    fin = torch.isfinite(rlse)
    _close(lse[fin], rlse[fin], 2e-2)
    _close(dq, rdq)
    _close(torch.cat(dks, dim=1), rdk)
    _close(torch.cat(dvs, dim=1), rdv)


@pytest.mark.gpu
@pytest.mark.parametrize("sizes,my_seg,pull", [((256, 384), 1, 3), ((200, 128, 333), 0, 8), ((1024, 1024), 1, 24)])
def test_kv_segments_pulled(sizes, my_seg, pull):
    """The forward with pulling thread blocks (the first blocks copy every other segment once, the query tiles read the
    copies) equals the forward that reads the segments where they are."""
    from cornstarch_b200.parallel.cp_fused import attention_segments_local, padded_layout

    B, Hq, Hk, D = 2, 4, 2, 128
    S = sum(sizes)
    q, k, v = _qkv(B, S, S, Hq, Hk, D, seed=S + 1)
    pos = torch.arange(S, dtype=torch.int32).cuda()[None].expand(B, -1).contiguous()
    starts, total = padded_layout(sizes)
    kp = torch.full((B, total), -1, dtype=torch.int32, device="cuda")
    ks, vs, off = [], [], 0
    for s0, n in zip(starts, sizes):
        kp[:, s0 : s0 + n] = pos[:, off : off + n]
        ks.append(k[:, off : off + n].contiguous())
        vs.append(v[:, off : off + n].contiguous())
        off += n
    mask = A.AttnMask(mode=A.MASK_CAUSAL, q_pos=pos, k_pos=kp)
    ro, rlse = attention_segments_local(q, ks, vs, mask, my_seg=my_seg)
    o, lse = attention_segments_local(q, ks, vs, mask, my_seg=my_seg, pull_ctas=pull)
    torch.cuda.synchronize()
    assert torch.equal(o, ro)
    assert torch.equal(lse, rlse)


@pytest.mark.parametrize("instance", [False, True])
def test_bitfield_mask_builder_kernel_matches_pytorch_statement(instance):
    """The int64 bitfield mask built by one kernel launch equals the PyTorch statement of the same builder (CPU path):
    several modalities, runs that straddle the 1024-token scan chunks, adjacent runs of different ids, padding."""
    from cornstarch_b200.kernel import interface as I

    g = torch.Generator().manual_seed(5)
    B, S = 3, 5000
    ids = torch.randint(0, 900, (B, S), generator=g)
    tok = {"vision": 998, "audio": 999}
    for b in range(B):
        pos = 3
        for run in range(70 if instance else 9):  # more than 61 runs: the instance bits wrap around
            n = int(torch.randint(1, 90, (1,), generator=g))
            if pos + n >= S:
                break
            ids[b, pos : pos + n] = 998 if (run + b) % 3 else 999
            pos += n + int(torch.randint(0, 40, (1,), generator=g))  # gap 0: two runs of different ids touch
    pad = torch.ones(B, S, dtype=torch.long)
    pad[1, 4700:] = 0
    build = I.create_instance_bitfield_attention_mask if instance else I.create_bitfield_attention_mask
    want = build(ids, tok, pad)
    got = build(ids.cuda(), tok, pad.cuda())
    assert got.dtype == torch.int64 and torch.equal(got.cpu(), want)
    assert torch.equal(build(ids.cuda(), tok).cpu(), build(ids, tok))
