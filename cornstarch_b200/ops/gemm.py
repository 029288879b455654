"""bf16 GEMM on the hand-written tcgen05 kernel (``csrc/gemm.cu``) with a plain-PyTorch CPU path.

``gemm(a, b, trans_a, trans_b)`` computes ``op(a) @ op(b).T`` in the kernel's native orientation:

* ``a_mn_major=False``: ``a`` is ``[M, K]`` (K contiguous);  ``True``: ``a`` is ``[K, M]`` (M contiguous)
* ``b_mn_major=False``: ``b`` is ``[N, K]`` (K contiguous);  ``True``: ``b`` is ``[K, N]`` (N contiguous)

so the three GEMMs of a linear layer (``y = x W^T``, ``dx = dy W``, ``dW = dy^T x``) need no transpose
copies.  These are the GEMMs the reference runs through cuBLAS behind ``nn.Linear`` and ColossalAI's
``Linear1D_Col/Row`` (cornstarch/shardformer/policies/llama.py:192-249).
"""

from __future__ import annotations

import torch

from . import _native as nat

ACT = {None: 0, "none": 0, "gelu_tanh": 1, "gelu_pytorch_tanh": 1, "gelu": 2, "gelu_erf": 2, "silu": 3}


def _ref_act(x: torch.Tensor, act) -> torch.Tensor:
    code = ACT[act]
    if code == 0:
        return x
    if code == 1:
        return torch.nn.functional.gelu(x, approximate="tanh")
    if code == 2:
        return torch.nn.functional.gelu(x)
    return torch.nn.functional.silu(x)


def gemm_reference(a, b, a_mn_major=False, b_mn_major=False, bias=None, act=None, out=None, accumulate=False,
                   out_dtype=None):
    """fp32 PyTorch statement of the kernel's contract (CPU path and test oracle)."""
    A = a.float().t() if a_mn_major else a.float()
    B = b.float().t() if b_mn_major else b.float()
    y = A @ B.t()
    if bias is not None:
        y = y + bias.float()
    y = _ref_act(y, act)
    if out is not None:
        if accumulate:
            y = y + out.float()
        out.copy_(y.to(out.dtype))
        return out
    return y.to(out_dtype or a.dtype)


def gemm_library(a, b, a_mn_major=False, b_mn_major=False, bias=None, act=None, out=None, accumulate=False, out_dtype=None):
    """The same contract on cuBLAS (``torch.matmul`` in the operands' dtype): the library baseline."""
    A = a.t() if a_mn_major else a
    B = b if b_mn_major else b.t()
    y = torch.matmul(A, B)
    if bias is not None:
        y = y + bias
    y = _ref_act(y, act)
    if out is not None:
        if accumulate:
            out.add_(y.to(out.dtype))
        else:
            out.copy_(y)
        return out
    return y.to(out_dtype or a.dtype)


def gemm(
    a: torch.Tensor,
    b: torch.Tensor,
    a_mn_major: bool = False,
    b_mn_major: bool = False,
    bias: torch.Tensor | None = None,
    act: str | None = None,
    out: torch.Tensor | None = None,
    accumulate: bool = False,
    out_dtype: torch.dtype | None = None,
    tile_n: int = 0,
    max_ctas: int = 0,
) -> torch.Tensor:
    """``out (+)= act(op(a) @ op(b).T + bias)``; 2-D row-major operands whose row stride may exceed the width."""
    if not a.is_cuda:
        return gemm_reference(a, b, a_mn_major, b_mn_major, bias, act, out, accumulate, out_dtype)
    if nat.LIBRARY_MODE:
        return gemm_library(a, b, a_mn_major, b_mn_major, bias, act, out, accumulate, out_dtype)
    assert a.dtype == torch.bfloat16 and b.dtype == torch.bfloat16, "native GEMM is bf16 x bf16 -> fp32 accumulate"
    assert a.dim() == 2 and b.dim() == 2 and a.stride(1) == 1 and b.stride(1) == 1
    if a_mn_major:
        K, M = a.shape
    else:
        M, K = a.shape
    if b_mn_major:
        Kb, N = b.shape
    else:
        N, Kb = b.shape
    assert K == Kb, f"contraction mismatch {K} vs {Kb}"
    if M == 0 or N == 0 or K == 0:
        # empty operand (an expert that received no token): nothing to launch
        if out is None:
            return torch.zeros((M, N), dtype=out_dtype or torch.bfloat16, device=a.device)
        if not accumulate and K == 0:
            out.zero_()
        return out
    lda, ldb = a.stride(0), b.stride(0)
    if (lda % 8) or (ldb % 8) or (a.data_ptr() % 16) or (b.data_ptr() % 16):
        # TMA needs 16-byte aligned rows; repack the rare odd-sized operand
        if lda % 8 or a.data_ptr() % 16:
            a = _pad_rows(a)
            lda = a.stride(0)
        if ldb % 8 or b.data_ptr() % 16:
            b = _pad_rows(b)
            ldb = b.stride(0)
    if out is None:
        out = torch.empty((M, N), dtype=out_dtype or torch.bfloat16, device=a.device)
        accumulate = False
    assert out.shape == (M, N) and out.stride(1) == 1 and out.dtype in (torch.bfloat16, torch.float32)
    if bias is not None:
        assert bias.dtype == torch.bfloat16 and bias.is_contiguous() and bias.numel() == N
    st = nat.status_word(a.device)
    code = nat.lib().csb_gemm_bf16(
        a.data_ptr(), b.data_ptr(), out.data_ptr(), nat.ptr(bias), M, N, K, lda, ldb, out.stride(0),
        int(a_mn_major), int(b_mn_major), int(out.dtype == torch.float32), int(accumulate), ACT[act],
        tile_n, max_ctas, st.data_ptr(), nat.stream(),
    )
    nat.check(code, "csb_gemm_bf16")
    return out


GROUP_ROW_MULTIPLE = 256  # rows per group of the native grouped GEMM: whole tiles of a pair of thread blocks
MAX_GROUPS = 16


def grouped_gemm_supported(a: torch.Tensor, bs, group_rows: int) -> bool:
    """Whether ``grouped_gemm`` runs these operands as ONE native launch."""
    b0 = bs[0]
    return (a.is_cuda and not nat.LIBRARY_MODE and a.dtype == torch.bfloat16 and a.dim() == 2 and a.stride(1) == 1
            and a.stride(0) % 8 == 0 and a.data_ptr() % 16 == 0 and 1 <= len(bs) <= MAX_GROUPS
            and group_rows > 0 and group_rows % GROUP_ROW_MULTIPLE == 0 and a.shape[0] == len(bs) * group_rows
            and all(b.dtype == torch.bfloat16 and b.dim() == 2 and b.shape == b0.shape and b.stride() == b0.stride()
                    and b.stride(1) == 1 and b.stride(0) % 8 == 0 and b.data_ptr() % 16 == 0 for b in bs))


def grouped_gemm(a: torch.Tensor, bs, group_rows: int, b_mn_major: bool = False, out: torch.Tensor | None = None,
                 accumulate: bool = False) -> torch.Tensor:
    """``out[g] (+)= a[g] @ op(bs[g]).T`` for every group ``g``: rows ``[g * group_rows, (g + 1) * group_rows)`` of ``a`` and
    ``out`` belong to group ``g``, ``bs[g]`` is ``[N, K]`` (``b_mn_major=False``) or ``[K, N]`` (``True``).  One launch of
    the GEMM kernel for all groups when ``grouped_gemm_supported``; one GEMM per group otherwise.  This is the expert MLP
    of a MoE layer whose experts all receive the same number of rows (Mixtral's experts in the reference run one after
    another, cornstarch/shardformer/modeling/mixtral.py:419-430)."""
    G = len(bs)
    assert a.dim() == 2 and a.shape[0] == G * group_rows, (a.shape, G, group_rows)
    N = bs[0].shape[1] if b_mn_major else bs[0].shape[0]
    K = bs[0].shape[0] if b_mn_major else bs[0].shape[1]
    assert a.shape[1] == K, f"contraction mismatch {a.shape[1]} vs {K}"
    if out is None:
        out = torch.empty((a.shape[0], N), dtype=a.dtype, device=a.device)
        accumulate = False
    if not grouped_gemm_supported(a, bs, group_rows) or out.stride(1) != 1 or out.dtype not in (torch.bfloat16, torch.float32):
        for g in range(G):
            rows = slice(g * group_rows, (g + 1) * group_rows)
            gemm(a[rows], bs[g], b_mn_major=b_mn_major, out=out[rows], accumulate=accumulate)
        return out
    import ctypes

    ptrs = (ctypes.c_void_p * G)(*[b.data_ptr() for b in bs])
    st = nat.status_word(a.device)
    code = nat.lib().csb_gemm_grouped_bf16(
        a.data_ptr(), ctypes.cast(ptrs, ctypes.c_void_p), out.data_ptr(), G, group_rows, N, K, a.stride(0), bs[0].stride(0),
        out.stride(0), int(b_mn_major), int(out.dtype == torch.float32), int(accumulate), 0, st.data_ptr(), nat.stream(),
    )
    nat.check(code, "csb_gemm_grouped_bf16")
    return out


def _pad_rows(t: torch.Tensor) -> torch.Tensor:
    """Copy a 2-D tensor into storage whose row stride is a multiple of 8 elements (16 bytes)."""
    r, c = t.shape
    ld = (c + 7) // 8 * 8
    buf = torch.zeros((r, ld), dtype=t.dtype, device=t.device)
    buf[:, :c].copy_(t)
    return buf[:, :c]
