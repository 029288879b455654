"""Micro-benchmarks of single kernels at the shapes of the headline model, with roofline fractions.

    python -m cornstarch_b200.utils.kernel_probe gemm --m 8192 --n 28672 --k 4096
    python -m cornstarch_b200.utils.kernel_probe attn_fwd --seq 8192
    python -m cornstarch_b200.utils.kernel_probe attn_bwd --seq 4096 --iters 1 --warmup 0     # small case for a profiler
    python -m cornstarch_b200.utils.kernel_probe all

Timing: CUDA events on the launching stream, warm-up first, synchronise on both sides; between timed
launches a 256 MB buffer is rewritten so that inputs do not sit in the 126 MB L2 (``--no-flush`` turns
that off).  Peaks come from ``MEASURED_PEAKS.json`` at the repository root when present (fractions are
then "of measured"), else from the stated fallback (6.65 TB/s, 1.59 PFLOP/s: "of fallback").
"""

from __future__ import annotations

import argparse
import json
import os

import torch

from ..ops import attention as A
from ..ops import elementwise as E
from ..ops.gemm import gemm

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.isfile(p):
        d = json.load(open(p))
        return d["hbm_gbs"] * 1e9, d["bf16_tflops"] * 1e12, "measured"
    return 6.65e12, 1.59e15, "fallback"


class Flusher:
    def __init__(self, enabled=True):
        self.buf = torch.empty(256 * 1024 * 1024, dtype=torch.uint8, device="cuda") if enabled else None

    def __call__(self):
        if self.buf is not None:
            self.buf.fill_(1)


def timeit(fn, iters, warmup, flush: Flusher):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    total = 0.0
    for _ in range(iters):
        flush()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize()
        total += e0.elapsed_time(e1)
    return total / max(iters, 1)


def report(name, ms, flops=0.0, bytes_=0.0, **extra):
    bw, fl, src = peaks()
    out = {"kernel": name, "ms": round(ms, 4)}
    if flops:
        out["tflops"] = round(flops / ms / 1e9, 1)
        out[f"frac_of_{src}_bf16_peak"] = round(flops / (ms / 1e3) / fl, 3)
    if bytes_:
        out["gbs"] = round(bytes_ / ms / 1e6, 1)
        out[f"frac_of_{src}_hbm_peak"] = round(bytes_ / (ms / 1e3) / bw, 3)
    out.update(extra)
    print(json.dumps(out), flush=True)


def probe_gemm(a, flush):
    M, N, K = a.m, a.n, a.k
    for amn, bmn, tag in ((0, 0, "fwd y=xW^T"), (0, 1, "dx=dyW"), (1, 1, "dW=dy^Tx")):
        A_ = torch.randn((K, M) if amn else (M, K), device="cuda").bfloat16()
        B_ = torch.randn((K, N) if bmn else (N, K), device="cuda").bfloat16()
        out = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
        ms = timeit(lambda: gemm(A_, B_, bool(amn), bool(bmn), out=out), a.iters, a.warmup, flush)
        report(f"gemm[{tag}]", ms, flops=2.0 * M * N * K, M=M, N=N, K=K)


def _qkv(a):
    B, S, Hq, Hk, D = a.batch, a.seq, a.heads, a.kv_heads, a.head_dim
    q = torch.randn(B, S, Hq, D, device="cuda").bfloat16()
    k = torch.randn(B, S, Hk, D, device="cuda").bfloat16()
    v = torch.randn(B, S, Hk, D, device="cuda").bfloat16()
    mask = A.AttnMask.causal() if a.mask == "causal" else A.AttnMask.full()
    return q, k, v, mask


def _attn_flops(a, bwd=False):
    f = 4.0 * a.batch * a.heads * a.seq * a.seq * a.head_dim * (0.5 if a.mask == "causal" else 1.0)
    return f * 2.5 if bwd else f


def probe_attn_fwd(a, flush):
    q, k, v, mask = _qkv(a)
    mask.classes(a.batch, a.seq, a.seq, q.device)
    ms = timeit(lambda: A.attention_forward(q, k, v, mask), a.iters, a.warmup, flush)
    report("attn_fwd", ms, flops=_attn_flops(a), S=a.seq, mask=a.mask, D=a.head_dim)


def probe_attn_bwd(a, flush):
    q, k, v, mask = _qkv(a)
    o, lse = A.attention_forward(q, k, v, mask)
    do = torch.randn_like(o)
    ms = timeit(lambda: A.attention_backward(do, q, k, v, o, lse, mask), a.iters, a.warmup, flush)
    report("attn_bwd", ms, flops=_attn_flops(a, True), S=a.seq, mask=a.mask, D=a.head_dim)


def probe_elementwise(a, flush):
    T, H, I = a.m, 4096, 14336
    x = torch.randn(T, H, device="cuda").bfloat16()
    r = torch.randn_like(x)
    w = torch.ones(H, device="cuda").bfloat16()
    ms = timeit(lambda: E.rms_norm(x, w, 1e-5, r), a.iters, a.warmup, flush)
    report("rmsnorm_residual_fwd", ms, bytes_=4 * T * H * 2)
    xg = x.clone().requires_grad_()
    wg = torch.ones(H, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    y, hsum = E.rms_norm(xg, wg, 1e-5, r)
    dy = torch.randn_like(y)

    def bwd():
        torch.autograd.grad((y, hsum), (xg, wg), (dy, dy), retain_graph=True)

    ms = timeit(bwd, a.iters, a.warmup, flush)
    report("rmsnorm_residual_bwd", ms, bytes_=4 * T * H * 2)
    gu = torch.randn(T, 2 * I, device="cuda").bfloat16()
    ms = timeit(lambda: E.glu(gu), a.iters, a.warmup, flush)
    report("swiglu_fwd", ms, bytes_=3 * T * I * 2)


def probe_adamw(a, flush):
    """Fused AdamW over a flat arena of ``--m * 1e6`` bf16 parameters (fp32 master + two moments, bf16 gradients)."""
    from ..optim.fused_adamw import FusedAdamW

    n = int(a.m) * 1_000_000
    p = torch.nn.Parameter(torch.randn(n, device="cuda").bfloat16())
    opt = FusedAdamW([{"params": [p], "weight_decay": 0.01}], lr=1e-4)
    p.main_grad.normal_()
    ms = timeit(opt.step, a.iters, a.warmup, flush)
    report("adamw", ms, bytes_=30.0 * n, params=n)


def probe_gemm_ar_local(a, flush):
    """The fused GEMM + all-reduce kernel on ONE GPU: rank 0 of an emulated world of 2 whose peer inbox is this
    GPU's own buffer and whose peer flags are pre-set, so that the reducer path can be timed and profiled alone."""
    import ctypes as C

    from ..ops import _native as nat
    from ..parallel import symm  # noqa: F401  (declares the prototype)

    M, N, K = a.m, a.n, a.k
    A_ = torch.randn(M, K, device="cuda").bfloat16()
    B_ = torch.randn(N, K, device="cuda").bfloat16()
    out = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
    slot = M * N
    inbox = torch.zeros(2 * slot, device="cuda", dtype=torch.bfloat16)
    final = torch.zeros(slot, device="cuda", dtype=torch.bfloat16)
    cnt_part = torch.zeros(2 * 512, device="cuda", dtype=torch.int32)
    cnt_final = torch.zeros(2 * 512, device="cuda", dtype=torch.int32)
    cnt_part[512:] = 1 << 30   # the emulated peer has "already delivered" every partial tile of every call
    cnt_final[512:] = 1 << 30  # ... and every final tile
    arr = lambda t: C.cast((C.c_void_p * 2)(t.data_ptr(), t.data_ptr()), C.c_void_p)  # noqa: E731
    st = nat.status_word()
    rb, re, nn = C.c_int(), C.c_int(), C.c_int()
    nat.lib().csb_ar_layout(M, N, 2, 0, 0, C.byref(rb), C.byref(re), C.byref(nn))
    calls = [0]

    def run():
        nat.check(nat.lib().csb_gemm_allreduce_bf16(
            A_.data_ptr(), B_.data_ptr(), out.data_ptr(), M, N, K, K, K, N, 0, 0, 2, 0, arr(inbox), arr(final),
            arr(cnt_part), arr(cnt_final), slot, calls[0] * nn.value, 0, st.data_ptr(), nat.stream()), "gemm_ar")
        calls[0] += 1

    ms = timeit(run, a.iters, a.warmup, flush)
    ref = A_.float() @ B_.float().t()
    own = slice(rb.value, re.value)  # rows owned by the emulated rank 0 hold the sum with the (zero) peer partial
    err = (out.float()[own] - ref[own]).abs().max().item() / ref.abs().max().item()
    report("gemm_allreduce[emulated world 2 on one GPU]", ms, flops=2.0 * M * N * K, M=M, N=N, K=K, reducers=a.reducers,
           rel_err=round(err, 5))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("what", choices=["gemm", "attn_fwd", "attn_bwd", "elementwise", "gemm_ar_local", "adamw", "all"])
    ap.add_argument("--reducers", type=int, default=16)
    ap.add_argument("--m", type=int, default=8192)
    ap.add_argument("--n", type=int, default=4096)
    ap.add_argument("--k", type=int, default=4096)
    ap.add_argument("--seq", type=int, default=8192)
    ap.add_argument("--batch", type=int, default=1)
    ap.add_argument("--heads", type=int, default=32)
    ap.add_argument("--kv-heads", type=int, default=8)
    ap.add_argument("--head-dim", type=int, default=128)
    ap.add_argument("--mask", default="causal", choices=["causal", "full"])
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--no-flush", action="store_true")
    a = ap.parse_args()
    flush = Flusher(not a.no_flush)
    todo = ["gemm", "attn_fwd", "attn_bwd", "elementwise"] if a.what == "all" else [a.what]
    for t in todo:
        {"gemm": probe_gemm, "attn_fwd": probe_attn_fwd, "attn_bwd": probe_attn_bwd, "elementwise": probe_elementwise,
         "gemm_ar_local": probe_gemm_ar_local, "adamw": probe_adamw}[t](a, flush)
    from ..ops import _native as nat

    nat.check_status()


if __name__ == "__main__":
    main()
