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


def probe_gemm_grouped(a, flush):
    """``--groups`` problems of ``--m`` rows each (``--n``, ``--k`` as given; default: the gate / up projection of eight
    Mixtral experts at 2560 rows) as ONE grouped launch against one GEMM launch per group, forward and input-gradient
    forms."""
    from ..ops.gemm import grouped_gemm

    G, R, N, K = a.groups, a.m, a.n, a.k
    x = torch.randn(G * R, K, device="cuda").bfloat16()
    for bmn, tag in ((False, "fwd y=xW^T"), (True, "dx=dyW")):
        bs = [torch.randn((K, N) if bmn else (N, K), device="cuda").bfloat16() for _ in range(G)]
        out = torch.empty(G * R, N, device="cuda", dtype=torch.bfloat16)

        def one_by_one():
            for g in range(G):
                gemm(x[g * R : (g + 1) * R], bs[g], False, bmn, out=out[g * R : (g + 1) * R])

        ms = timeit(lambda: grouped_gemm(x, bs, R, b_mn_major=bmn, out=out), a.iters, a.warmup, flush)
        ms_loop = timeit(one_by_one, a.iters, a.warmup, flush)
        report(f"gemm_grouped[{tag}]", ms, flops=2.0 * G * R * N * K, groups=G, rows_per_group=R, N=N, K=K,
               one_launch_per_group_ms=round(ms_loop, 4), speedup=round(ms_loop / ms, 3))


def probe_gemm_sustained(a, flush):
    """Back-to-back launches for ``--seconds`` (default 3) of this package's GEMM and of ``torch.matmul`` (cuBLAS) on the
    same operands: the throughput both settle at under the power cap, which is what a long training step sees."""
    import time

    M, N, K = a.m, a.n, a.k
    A_ = torch.randn(M, K, device="cuda").bfloat16()
    B_ = torch.randn(N, K, device="cuda").bfloat16()
    out = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
    Bt = B_.t()

    def loop(fn):
        fn()
        torch.cuda.synchronize()
        n, t0 = 0, time.monotonic()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        while time.monotonic() - t0 < a.seconds:
            for _ in range(20):
                fn()
            n += 20
            torch.cuda.synchronize()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / n

    for tag, fn in (("cublas", lambda: torch.matmul(A_, Bt, out=out)), ("native", lambda: gemm(A_, B_, False, False, out=out)),
                    ("cublas", lambda: torch.matmul(A_, Bt, out=out)), ("native", lambda: gemm(A_, B_, False, False, out=out))):
        ms = loop(fn)
        report(f"gemm_sustained[{tag}]", ms, flops=2.0 * M * N * K, M=M, N=N, K=K, seconds=a.seconds)


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


def probe_grad_reduce_local(a, flush):
    """The gradient all-reduce kernel on ONE GPU: rank 0 of an emulated world of 2 whose peer buffer is a second
    buffer of this GPU and whose "gradients complete" counter is pre-set.  ``--m`` = MiB per buffer.  Rank 0 owns the
    first half: it reads that half of both buffers and writes the mean into both."""
    import ctypes as C

    from ..ops import _native as nat
    from ..parallel import dp_fused  # noqa: F401  (declares the prototype)

    n = int(a.m) * (1 << 20) // 2
    mine = torch.randn(n, device="cuda").bfloat16()
    peer = torch.randn(n, device="cuda").bfloat16()
    want = ((mine[: n // 2].float() + peer[: n // 2].float()) * 0.5).bfloat16()
    ready = torch.full((64,), 1 << 30, dtype=torch.int32, device="cuda")
    bufs = (C.c_void_p * 8)(mine.data_ptr(), peer.data_ptr(), 0, 0, 0, 0, 0, 0)
    st = nat.status_word()

    def run():
        nat.check(nat.lib().csb_grad_reduce(C.cast(bufs, C.c_void_p), 2, 0, n, 0.5, 1, ready.data_ptr(), 1, 0, st.data_ptr(),
                                            nat.stream()), "csb_grad_reduce")

    run()
    torch.cuda.synchronize()
    ok = bool(torch.equal(mine[: n // 2], want) and torch.equal(peer[: n // 2], want))
    ms = timeit(run, a.iters, a.warmup, flush)
    # per launch: half a buffer read twice (own + peer copy) and written twice
    report("grad_reduce[emulated world 2 on one GPU]", ms, bytes_=4.0 * (n // 2) * 2, buffer_MiB=a.m, correct=ok)


def probe_moe_push_local(a, flush):
    """The MoE dispatch push on ONE GPU: ``--m`` token rows of width ``--n`` gathered through a random (token, k) order
    and stored into 8 destination buffers that all live on this GPU."""
    import ctypes as C

    from ..ops import _native as nat
    from ..parallel import ep_fused  # noqa: F401  (declares the prototype)

    rows, H, ws = a.m, a.n, 8
    src = torch.randn(rows, H, device="cuda").bfloat16()
    index = torch.randperm(rows, device="cuda").int()
    per = rows // ws
    seg = [min(i * per, rows) for i in range(ws)] + [rows]
    dst = [torch.empty(seg[d + 1] - seg[d], H, device="cuda", dtype=torch.bfloat16) for d in range(ws)]
    seg_arr = (C.c_int * (ws + 1))(*seg)
    dst_arr = (C.c_void_p * ws)(*[t.data_ptr() for t in dst])

    def run():
        nat.check(nat.lib().csb_moe_push(src.data_ptr(), index.data_ptr(), rows, H, C.cast(seg_arr, C.c_void_p),
                                         C.cast(dst_arr, C.c_void_p), ws, rows, nat.stream()), "csb_moe_push")

    run()
    torch.cuda.synchronize()
    ok = bool(torch.equal(torch.cat(dst), src[index.long()]))
    ms = timeit(run, a.iters, a.warmup, flush)
    report("moe_push[8 destinations on one GPU]", ms, bytes_=2.0 * rows * H * 2, rows=rows, H=H, correct=ok)


def probe_attn_fwd_pulled(a, flush):
    """The context-parallel forward on ONE GPU: K / V in two segments, the query rows of the later half; the first
    ``--reducers`` thread blocks copy the other segment, the query tiles read the copy (all memory local)."""
    from ..parallel.cp_fused import attention_segments_local, padded_layout

    B, S, Hq, Hk, D = a.batch, a.seq, a.heads, a.kv_heads, a.head_dim
    half = S // 2
    q = torch.randn(B, half, Hq, D, device="cuda").bfloat16()
    ks = [torch.randn(B, half, Hk, D, device="cuda").bfloat16() for _ in range(2)]
    vs = [torch.randn(B, half, Hk, D, device="cuda").bfloat16() for _ in range(2)]
    _, total = padded_layout([half, half])
    qp = (half + torch.arange(half, dtype=torch.int32, device="cuda"))[None].expand(B, -1).contiguous()
    kp = torch.arange(total, dtype=torch.int32, device="cuda")[None].expand(B, -1).contiguous()
    mask = A.AttnMask(mode=A.MASK_CAUSAL, q_pos=qp, k_pos=kp)
    mask.classes(B, half, total, q.device)
    ms_direct = timeit(lambda: attention_segments_local(q, ks, vs, mask, my_seg=1), a.iters, a.warmup, flush)
    ms = timeit(lambda: attention_segments_local(q, ks, vs, mask, my_seg=1, pull_ctas=a.reducers), a.iters, a.warmup, flush)
    flops = 4.0 * B * Hq * half * D * (half + half / 2)
    report("attn_fwd_seg[2 segments on one GPU, pulled]", ms, flops=flops, S=S, pull_ctas=a.reducers,
           direct_ms=round(ms_direct, 4))


def probe_mma_issue(a, flush):
    """Cycles per tcgen05.mma (128 x N x 16) for a run of 512 issued by one warp: a single lane in a divergent branch
    against the whole converged warp with an elected lane, with idle and with busy (dense FMA) neighbour warps."""
    from ..ops import _native as nat

    lib = nat.lib()
    out = torch.zeros(4, dtype=torch.int64, device="cuda")
    reps = 64
    for busy in (0, 1):
        for n in (64, 128, 256):
            row = {"kernel": "mma_issue", "tile": f"128x{n}x16", "neighbour_warps": "dense FMAs" if busy else "idle",
                   "cycles_at_tensor_peak": 128 * n * 16 * 2 // 8192}
            for whole in (0, 1):
                for _ in range(3):
                    nat.check(lib.csb_mma_issue_probe(n, whole, busy, reps, out.data_ptr(), nat.stream()), "csb_mma_issue_probe")
                torch.cuda.synchronize()
                issued, retired, ok = out[:3].tolist()
                assert ok == 1
                row["one_lane" if whole == 0 else "whole_warp_elected"] = {"issue_cycles_per_mma": round(issued / (reps * 8), 1),
                                                                             "retire_cycles_per_mma": round(retired / (reps * 8), 1)}
            print(json.dumps(row), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--seconds", type=float, default=3.0)
    ap.add_argument("what", choices=["gemm", "gemm_grouped", "gemm_sustained", "attn_fwd", "attn_bwd", "elementwise", "gemm_ar_local", "adamw", "grad_reduce_local",
                                     "moe_push_local", "attn_fwd_pulled", "mma_issue", "all"])
    ap.add_argument("--reducers", type=int, default=16)
    ap.add_argument("--groups", type=int, default=8, help="gemm_grouped: number of groups (experts)")
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
        if t == "gemm_grouped" and (a.m, a.n, a.k) == (8192, 4096, 4096):
            a.m, a.n, a.k = 2560, 28672, 4096  # rows per expert at capacity 1.25 of 8192 tokens; gate | up of Mixtral-8x7B
        {"gemm": probe_gemm, "gemm_grouped": probe_gemm_grouped, "gemm_sustained": probe_gemm_sustained, "attn_fwd": probe_attn_fwd, "attn_bwd": probe_attn_bwd, "elementwise": probe_elementwise,
         "gemm_ar_local": probe_gemm_ar_local, "adamw": probe_adamw, "grad_reduce_local": probe_grad_reduce_local,
         "moe_push_local": probe_moe_push_local, "attn_fwd_pulled": probe_attn_fwd_pulled, "mma_issue": probe_mma_issue}[t](a, flush)
    from ..ops import _native as nat

    nat.check_status()


if __name__ == "__main__":
    main()
