"""The reference's own Triton attention kernels, unmodified, timed next to this package's tcgen05 kernels on the same GPU.

The reference project ships two Triton kernel families (``cornstarch/kernel/bitfield_attention.py``: ``bitfield_attn_func``,
autograd class at :1202-1266; ``cornstarch/kernel/attention.py``: ``flash_attn_func`` at :1126-1147).  They import with
torch + triton alone, so they can run here even though the rest of the reference (model layer, plugins) cannot.  This
module imports them from an installed copy of the reference (``baseline/_ref`` of a checkout, or any ``cornstarch`` on
``sys.path``), runs forward and backward on the shapes of the benchmark workloads, cross-checks outputs and gradients
against this package's kernels and both against an fp32 PyTorch oracle (one KV head and the query heads sharing it; errors are
max |x - oracle| / max |oracle|, the reference's own tolerance is 5e-3), and reports device times.

    python -m cornstarch_b200.utils.reference_kernels            # all cases, one JSON line per case
    python -m cornstarch_b200.utils.reference_kernels --quick    # the two headline shapes only

Timing: CUDA events on the launching stream, warm-up first (it also triggers Triton's compilation and autotuning),
a 256 MB buffer rewritten between timed launches so that inputs do not sit in L2.  FLOPs are counted on the pairs the
mask allows (4 * D per pair forward, 2.5x that backward).
"""

from __future__ import annotations

import argparse
import json
import os
import sys

import torch

from ..ops import attention as A

TOL = 5e-3  # the reference's own tolerance for bf16 outputs and gradients (tests/test_kernel/test_bitfield_attention.py:196-204)


def _import_reference():
    try:
        import cornstarch.kernel.attention as ref_fa
        import cornstarch.kernel.bitfield_attention as ref_bf
    except ImportError:
        root = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
        sys.path.insert(0, os.path.join(root, "baseline", "_ref"))
        import cornstarch.kernel.attention as ref_fa
        import cornstarch.kernel.bitfield_attention as ref_bf
    return ref_bf, ref_fa


def _time(fn, iters, warmup, flush):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    total = 0.0
    for _ in range(iters):
        flush.fill_(1)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize()
        total += e0.elapsed_time(e1)
    return total / iters


def _rel(a, b):
    return float((a.float() - b.float()).abs().max() / b.float().abs().max().clamp(min=1e-6))


def _bits_one_image(B, S, image_tokens, device):
    """Placeholder layout of the headline workload: one image (bit 1) at the start, text after it (text bit + bit 1)."""
    bits = torch.full((B, S), (1 << 62) | 1 | 2, dtype=torch.int64, device=device)
    bits[:, :image_tokens] = 2
    return bits


def _bits_images_at(B, S, image_tokens, starts, device):
    bits = torch.full((B, S), (1 << 62) | 1 | 2, dtype=torch.int64, device=device)
    for s in starts:
        bits[:, s : s + image_tokens] = 2
    return bits


def _case(name, B, S, Hq, Hk, D, bits, iters, warmup, flush, ref_bf, ref_fa):
    """One shape: forward and backward of both implementations; ``bits`` None = no mask (full attention)."""
    dev = "cuda"
    g = torch.Generator(device=dev).manual_seed(0)
    q = torch.randn(B, S, Hq, D, device=dev, generator=g).bfloat16()
    k = torch.randn(B, S, Hk, D, device=dev, generator=g).bfloat16()
    v = torch.randn(B, S, Hk, D, device=dev, generator=g).bfloat16()
    do = torch.randn(B, S, Hq, D, device=dev, generator=g).bfloat16()
    mask = A.AttnMask.full() if bits is None else A.AttnMask.bitfield(bits)
    cls = mask.classes(B, S, S, q.device)
    # allowed pairs, from the tile classes (full tiles) plus the exact count of the mixed tiles' predicate
    if bits is None:
        pairs = float(B) * S * S
    else:
        pairs = float(A.dense_mask(mask, 1, S, S, dev)[0].sum()) * B if S <= 16384 else float((cls != 0).sum()) * 128 * 128
    fwd_flops = 4.0 * pairs * D * Hq
    out = {"case": name, "B": B, "S": S, "Hq": Hq, "Hk": Hk, "D": D, "mask": "none" if bits is None else "bitfield",
           "allowed_pair_fraction": round(pairs / (float(B) * S * S), 4)}

    # ---- this package
    o_n, lse_n = A.attention_forward(q, k, v, mask)
    dq_n, dk_n, dv_n = A.attention_backward(do, q, k, v, o_n, lse_n, mask)
    ms_f = _time(lambda: A.attention_forward(q, k, v, mask), iters, warmup, flush)
    ms_b = _time(lambda: A.attention_backward(do, q, k, v, o_n, lse_n, mask), iters, warmup, flush)
    out["native"] = {"fwd_ms": round(ms_f, 4), "bwd_ms": round(ms_b, 4), "fwd_tflops": round(fwd_flops / ms_f / 1e9, 1),
                     "bwd_tflops": round(2.5 * fwd_flops / ms_b / 1e9, 1)}

    # ---- fp32 oracle (plain PyTorch, dense mask) on the first KV head and the query heads that share it
    g_sz = Hq // Hk
    qo, ko, vo = (t.float().clone().requires_grad_() for t in (q[:, :, :g_sz], k[:, :, :1], v[:, :, :1]))
    o_o, _ = A.attention_reference(qo, ko, vo, mask)
    o_o.backward(do[:, :, :g_sz].float())
    oracle = {"o": o_o.detach(), "dq": qo.grad, "dk": ko.grad, "dv": vo.grad}
    del o_o
    sub = lambda o_, dq_, dk_, dv_: {"o": o_[:, :, :g_sz], "dq": dq_[:, :, :g_sz], "dk": dk_[:, :, :1], "dv": dv_[:, :, :1]}  # noqa: E731
    err_n = {k_: _rel(v_, oracle[k_]) for k_, v_ in sub(o_n, dq_n, dk_n, dv_n).items()}
    out["native"]["max_rel_err_vs_fp32_oracle"] = {k_: round(v_, 5) for k_, v_ in err_n.items()}
    out["native"]["within_5e-3_of_oracle"] = bool(all(v_ <= TOL for v_ in err_n.values()))

    # ---- the reference's Triton kernels through its own autograd function
    try:
        if hasattr(ref_bf, "BitfieldUtils"):
            ref_bf.BitfieldUtils.clear_cache()  # the reference caches ONE compressed mask globally; a new mask needs a clear
        qr, kr, vr = (t.clone().requires_grad_() for t in (q, k, v))
        if bits is None:
            fwd = lambda: ref_fa.flash_attn_func(qr, kr, vr)  # noqa: E731
        else:
            fwd = lambda: ref_bf.bitfield_attn_func(qr, kr, vr, bits)  # noqa: E731
        o_r = fwd()
        o_r.backward(do)
        dq_r, dk_r, dv_r = qr.grad.clone(), kr.grad.clone(), vr.grad.clone()

        def fwd_only():
            with torch.no_grad():
                fwd()

        ms_rf = _time(fwd_only, iters, warmup, flush)

        def fwd_bwd():
            qr.grad = kr.grad = vr.grad = None
            fwd().backward(do)

        ms_rfb = _time(fwd_bwd, iters, warmup, flush)
        ms_rb = max(ms_rfb - ms_rf, 1e-6)
        out["reference_triton"] = {"fwd_ms": round(ms_rf, 4), "bwd_ms": round(ms_rb, 4), "fwd_plus_bwd_ms": round(ms_rfb, 4),
                                   "fwd_tflops": round(fwd_flops / ms_rf / 1e9, 1), "bwd_tflops": round(2.5 * fwd_flops / ms_rb / 1e9, 1)}
        out["speedup"] = {"fwd": round(ms_rf / ms_f, 2), "bwd": round(ms_rb / ms_b, 2),
                          "fwd_plus_bwd": round(ms_rfb / (ms_f + ms_b), 2)}
        err = {"o": _rel(o_n, o_r), "dq": _rel(dq_n, dq_r), "dk": _rel(dk_n, dk_r), "dv": _rel(dv_n, dv_r)}
        out["max_rel_diff_native_vs_reference"] = {k_: round(v_, 5) for k_, v_ in err.items()}
        err_r = {k_: _rel(v_, oracle[k_]) for k_, v_ in sub(o_r, dq_r, dk_r, dv_r).items()}
        out["reference_triton"]["max_rel_err_vs_fp32_oracle"] = {k_: round(v_, 5) for k_, v_ in err_r.items()}
        out["reference_triton"]["within_5e-3_of_oracle"] = bool(all(v_ <= TOL for v_ in err_r.values()))
    except Exception as e:  # noqa: BLE001  (e.g. a Triton compile error for this GPU: reported, not raised)
        out["reference_triton"] = {"error": f"{type(e).__name__}: {e}".replace("\n", " ")[:400]}
    return out


def compare_attention(quick: bool = False, iters: int = 5, warmup: int = 2) -> dict:
    """Run the cases and return ``{"cases": [...], ...}``; ``quick`` keeps the two headline shapes."""
    import triton

    ref_bf, ref_fa = _import_reference()
    flush = torch.empty(256 * 1024 * 1024, dtype=torch.uint8, device="cuda")
    cases = [
        # decoder attention of the headline workload: 8192 tokens, 32 / 8 heads of 128, one 729-token image then text
        ("llm_s8192_one_image", 1, 8192, 32, 8, 128, _bits_one_image(1, 8192, 729, "cuda")),
        # vision tower of the headline workload: 4 images of 729 patch tokens, 16 heads of 72, no mask
        ("siglip_s729_d72", 4, 729, 16, 16, 72, None),
    ]
    if not quick:
        cases.append(("llm_s16384_four_images", 1, 16384, 32, 8, 128,
                      _bits_images_at(1, 16384, 729, [100, 5000, 9000, 14000], "cuda")))
    res = {"torch": torch.__version__, "triton": triton.__version__, "gpu": torch.cuda.get_device_name(0),
           "reference_file": ref_bf.__file__.split("baseline/")[-1], "iters": iters, "warmup": warmup,
           "timing": "CUDA events, 256 MB L2 flush between launches", "cases": []}
    for c in cases:
        res["cases"].append(_case(*c, iters, warmup, flush, ref_bf, ref_fa))
    return res


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--quick", action="store_true")
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    a = ap.parse_args()
    res = compare_attention(a.quick, a.iters, a.warmup)
    cases = res.pop("cases")
    print(json.dumps(res))
    for c in cases:
        print(json.dumps(c), flush=True)


if __name__ == "__main__":
    main()
