"""NVTX range placement (CPU) and race checks of the kernels without a sanitizer (GPU): every output element is
written (outputs are poisoned with NaN first) and repeated launches give bitwise identical results where the
algorithm is deterministic."""

import pytest
import torch

from cornstarch_b200.utils import trace


def test_nvtx_ranges_wrap_optimizer_step():
    from cornstarch_b200.optim.fused_adamw import FusedAdamW

    p = torch.nn.Parameter(torch.randn(16, 8))
    opt = FusedAdamW([{"params": [p], "weight_decay": 0.0}], lr=1e-2)
    p.grad = torch.ones_like(p)
    trace.recorded = []
    try:
        opt.step()
    finally:
        names, trace.recorded = trace.recorded, None
    assert names == ["optimizer/fused_adamw_step"]


def test_timeline_is_inert_without_a_gpu():
    """``timeline(True)`` records CUDA events around the ranges; without CUDA it stays off and the ranges do nothing."""
    if torch.cuda.is_available():
        pytest.skip("covers the CPU behaviour")
    trace.timeline(True)
    with trace.nvtx_range("pipeline/forward_microbatch"):
        pass
    assert trace.timeline_totals() == {}
    trace.timeline(False)


@pytest.mark.gpu
def test_timeline_sums_device_time_per_range():
    trace.timeline(True)
    x = torch.randn(4096, 4096, device="cuda")
    for _ in range(3):
        with trace.nvtx_range("work"):
            x = x @ x.t() * 1e-4
    totals = trace.timeline_totals()
    trace.timeline(False)
    assert totals["work"][0] == 3 and totals["work"][1] > 0
    assert trace.timeline_totals() == {}


def _poisoned_allocations():
    """Fill the caching allocator's free blocks with NaN bit patterns so that ``torch.empty`` outputs start poisoned."""
    junk = [torch.full((n,), float("nan"), device="cuda", dtype=torch.float32) for n in (1 << 24, 1 << 22, 1 << 20, 1 << 18)]
    del junk


@pytest.mark.gpu
def test_gemm_writes_every_element_and_is_deterministic():
    from cornstarch_b200.ops.gemm import gemm

    torch.manual_seed(0)
    a = torch.randn(1000, 520, device="cuda").bfloat16()
    b = torch.randn(776, 520, device="cuda").bfloat16()
    _poisoned_allocations()
    outs = [gemm(a, b) for _ in range(3)]
    torch.cuda.synchronize()
    assert torch.isfinite(outs[0].float()).all()
    assert all(torch.equal(outs[0], o) for o in outs[1:])


@pytest.mark.gpu
@pytest.mark.parametrize("S", [1000, 2048])
def test_attention_writes_every_element_and_dkdv_are_deterministic(S):
    from cornstarch_b200.ops import attention as A

    torch.manual_seed(1)
    q = torch.randn(1, S, 8, 128, device="cuda").bfloat16()
    k = torch.randn(1, S, 2, 128, device="cuda").bfloat16()
    v = torch.randn(1, S, 2, 128, device="cuda").bfloat16()
    do = torch.randn(1, S, 8, 128, device="cuda").bfloat16()
    mask = A.AttnMask.causal()
    _poisoned_allocations()
    o1, l1 = A.attention_forward(q, k, v, mask)
    o2, l2 = A.attention_forward(q, k, v, mask)
    assert torch.isfinite(o1.float()).all() and torch.isfinite(l1).all()
    assert torch.equal(o1, o2) and torch.equal(l1, l2)
    _poisoned_allocations()
    g1 = A.attention_backward(do, q, k, v, o1, l1, mask)
    g2 = A.attention_backward(do, q, k, v, o1, l1, mask)
    for t in g1:
        assert torch.isfinite(t.float()).all()
    # dK / dV are accumulated in tensor memory by one thread block each: same bits every run.  dQ is summed by
    # reduce-adds whose order is not fixed: equal up to fp32 rounding.
    assert torch.equal(g1[1], g2[1]) and torch.equal(g1[2], g2[2])
    assert torch.allclose(g1[0].float(), g2[0].float(), atol=2e-2, rtol=2e-2)


@pytest.mark.gpu
def test_norm_and_glu_are_deterministic():
    from cornstarch_b200.ops import elementwise as E

    torch.manual_seed(2)
    x = torch.randn(4096, 1024, device="cuda").bfloat16().requires_grad_()
    w = torch.randn(1024, device="cuda").bfloat16().requires_grad_()
    gu = torch.randn(4096, 2048, device="cuda").bfloat16().requires_grad_()
    res = []
    for _ in range(2):
        _poisoned_allocations()
        y = E.rms_norm(x, w, 1e-6)
        z = E.glu(gu, "silu")
        gx, gw, ggu = torch.autograd.grad([y, z], [x, w, gu], [torch.ones_like(y), torch.ones_like(z)])
        res.append((y.detach(), z.detach(), gx, gw, ggu))
    for a, b in zip(*res):
        assert torch.isfinite(a.float()).all()
        assert torch.equal(a, b)


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_gradient_norm_is_bitwise_repeatable(dtype):
    """The sum of squares behind gradient clipping is the same bit pattern on every launch (block sums are added in block
    order): data-parallel replicas that hold equal gradients must scale them by equal factors, else they drift apart."""
    from cornstarch_b200.ops import _native as nat

    lib = nat.lib()
    torch.manual_seed(0)
    g = (torch.randn(50_000_003, device="cuda") * 1e-2).to(dtype)
    scratch = torch.zeros(4096, device="cuda")
    st = torch.cuda.current_stream().cuda_stream
    outs = []
    for _ in range(8):
        out = torch.zeros(1, device="cuda")
        nat.check(lib.csb_sumsq(g.data_ptr(), int(dtype == torch.float32), g.numel(), out.data_ptr(), scratch.data_ptr(),
                                scratch.numel(), st), "csb_sumsq")
        outs.append(out)
    torch.cuda.synchronize()
    assert all(torch.equal(o, outs[0]) for o in outs[1:])
    ref = g.double().pow(2).sum().item()
    assert abs(outs[0].item() - ref) <= 1e-5 * ref
    # two launches into the same accumulator add up; the ticket counter is back at zero for the next launch
    out = torch.zeros(1, device="cuda")
    for _ in range(2):
        nat.check(lib.csb_sumsq(g.data_ptr(), int(dtype == torch.float32), g.numel(), out.data_ptr(), scratch.data_ptr(),
                                scratch.numel(), st), "csb_sumsq")
    assert abs(out.item() - 2 * ref) <= 1e-5 * 2 * ref
    assert scratch.view(torch.int32)[0].item() == 0


def test_split_master_weights_are_exact():
    """fp32 master weights kept as bf16 parameter + int16 remainder: any fp32 value survives the split exactly, and the
    parameter is the master rounded to bf16 (half away from zero)."""
    from cornstarch_b200.optim.fused_adamw import _Region

    torch.manual_seed(0)
    p = torch.nn.Parameter(torch.randn(4096).bfloat16())
    region = _Region([p], torch.bfloat16, None, None, split_master=True)
    assert region.master is None and region.resid.dtype == torch.int16
    assert torch.equal(region.master_weights(), p.data.float())  # starts as the parameter itself
    vals = torch.cat([torch.randn(4000) * 3, torch.tensor([0.0, -0.0, 1.0, -1.0, 1e-30, -1e-30, 3.0e38, -3.0e38]),
                      torch.randn(88) * 1e-6])
    # exact ties of the rounding (lower half == 0x8000), both signs
    ties = ((torch.randn(64).bfloat16().view(torch.int16).to(torch.int32) << 16) + 0x8000).view(torch.float32)
    vals[:64] = ties
    region.set_master_weights(slice(0, 4096), vals)
    assert torch.equal(region.master_weights().view(torch.int32), vals.view(torch.int32))
    err = (p.data.float() - vals).abs()
    assert bool((err <= vals.abs() * 2.0 ** -8).all())  # half a unit in the last place of bf16 (8 significant bits)
    not_tie = torch.ones(4096, dtype=torch.bool)
    not_tie[:64] = False
    assert torch.equal(p.data[not_tie], vals.bfloat16()[not_tie])  # same as round-to-nearest-even away from ties
    region.reset_master_weights()
    assert torch.equal(region.master_weights(), p.data.float())


def test_overlapped_reduce_covers_every_element_once():
    """What the layer hooks reduced plus what ``finish`` adds is a partition of the flat buffer."""
    from cornstarch_b200.parallel.dp_fused import OverlappedGradReduce as O

    assert O.gaps([], 640) == [(0, 640)]
    assert O.gaps([(128, 256), (0, 64)], 640) == [(64, 128), (256, 640)]
    assert O.gaps([(0, 640)], 640) == []
    done = [(320, 448), (448, 576), (64, 320)]
    pieces = sorted(done + O.gaps(done, 640))
    assert pieces[0][0] == 0 and pieces[-1][1] == 640 and all(a[1] == b[0] for a, b in zip(pieces, pieces[1:]))
