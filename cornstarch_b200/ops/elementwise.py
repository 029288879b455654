"""Autograd wrappers of the fused HBM-bound kernels (``csrc/norm.cu``, ``csrc/elementwise.cu``).

Every function has two paths: the native sm_100a kernel for bf16 CUDA tensors and a plain PyTorch
statement of the same math for everything else (CPU tests, fp32).  The PyTorch statements are also
the oracles of the GPU numerics tests.

* :func:`rms_norm`, :func:`layer_norm` — optional fused residual add (returns the new residual too)
* :func:`rope_` — in-place rotate-half RoPE on the q|k part of a fused projection output
* :func:`glu` — ``act(gate) * up`` on a fused ``[.., 2I]`` gate|up tensor (SwiGLU / GeGLU)
* :func:`activation` — GELU (erf / tanh), quick-GELU, SiLU
* :func:`embed_merge` — token embedding with encoder features scattered in at placeholder positions

These replace apex FusedRMSNorm/LayerNorm (cornstarch/shardformer/policies/llama.py:252-275), HF
``apply_rotary_pos_emb`` / ``ACT2FN`` and the ``masked_scatter`` merge
(cornstarch/models/multimodal_language_model/modeling_multimodal_language_model.py:930-936).
"""

from __future__ import annotations

import torch
import torch.nn.functional as F

from . import _native as nat


def _native_ok(x: torch.Tensor) -> bool:
    return x.is_cuda and x.dtype == torch.bfloat16 and not nat.LIBRARY_MODE


# --------------------------------------------------------------------------------------- norms
def _norm_ref(x, w, b, eps, is_ln, w_offset):
    if nat.LIBRARY_MODE and x.is_cuda:
        wt = w if not w_offset else (w.float() + w_offset).to(w.dtype)
        if is_ln:
            return F.layer_norm(x, (x.shape[-1],), wt, b, eps)
        return F.rms_norm(x, (x.shape[-1],), wt, eps)
    xf = x.float()
    if is_ln:
        mean = xf.mean(-1, keepdim=True)
        var = (xf - mean).pow(2).mean(-1, keepdim=True)
        y = (xf - mean) * torch.rsqrt(var + eps)
    else:
        y = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)
    y = y * (w.float() + w_offset)
    if b is not None:
        y = y + b.float()
    return y.to(x.dtype)


class _NormFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, res, w, b, eps, is_ln, w_offset):
        H = x.shape[-1]
        x2 = x.reshape(-1, H)
        x2 = x2 if x2.is_contiguous() else x2.contiguous()
        rows = x2.shape[0]
        r2 = None
        if res is not None:
            r2 = res.reshape(-1, H)
            r2 = r2 if r2.is_contiguous() else r2.contiguous()
        y = torch.empty_like(x2)
        h = torch.empty_like(x2) if res is not None else None
        rstd = torch.empty(rows, dtype=torch.float32, device=x.device)
        mean = torch.empty(rows, dtype=torch.float32, device=x.device) if is_ln else None
        nat.check(
            nat.lib().csb_norm_fwd(int(is_ln), x2.data_ptr(), nat.ptr(r2), w.data_ptr(), nat.ptr(b), y.data_ptr(),
                                   nat.ptr(h), nat.ptr(mean), rstd.data_ptr(), rows, H, eps, w_offset, nat.stream()),
            "csb_norm_fwd",
        )
        hs = h if h is not None else x2
        ctx.save_for_backward(hs, w, mean, rstd)
        ctx.is_ln, ctx.w_offset, ctx.shape, ctx.has_res, ctx.has_b = is_ln, w_offset, x.shape, res is not None, b is not None
        ctx.w_ref, ctx.b_ref = w, b
        if res is not None:
            return y.view(x.shape), h.view(x.shape)
        return y.view(x.shape), None

    @staticmethod
    def backward(ctx, dy, dh):
        hs, w, mean, rstd = ctx.saved_tensors
        rows, H = hs.shape
        dy2 = dy.reshape(-1, H)
        dy2 = dy2 if dy2.is_contiguous() else dy2.contiguous()
        dres = None
        if dh is not None:
            dres = dh.reshape(-1, H)
            dres = dres if dres.is_contiguous() else dres.contiguous()
        dx = torch.empty_like(hs)
        parts = nat.lib().csb_norm_bwd_parts(rows)
        dw_part = torch.empty(parts * H, dtype=torch.float32, device=hs.device)
        db_part = torch.empty(parts * H, dtype=torch.float32, device=hs.device) if (ctx.is_ln and ctx.has_b) else None
        w_main = getattr(ctx.w_ref, "main_grad", None)
        b_main = getattr(ctx.b_ref, "main_grad", None) if ctx.has_b else None
        use_main = w_main is not None and (not ctx.has_b or b_main is not None)
        if use_main:
            dw_out, db_out, acc = w_main, b_main, 1
        else:
            dw_out = torch.empty(H, dtype=hs.dtype, device=hs.device)
            db_out = torch.empty(H, dtype=hs.dtype, device=hs.device) if db_part is not None else None
            acc = 0
        nat.check(
            nat.lib().csb_norm_bwd(int(ctx.is_ln), dy2.data_ptr(), hs.data_ptr(), w.data_ptr(), nat.ptr(mean),
                                   rstd.data_ptr(), nat.ptr(dres), dx.data_ptr(), dw_part.data_ptr(), nat.ptr(db_part),
                                   dw_out.data_ptr(), nat.ptr(db_out), int(dw_out.dtype == torch.float32), acc, rows, H,
                                   ctx.w_offset, nat.stream()),
            "csb_norm_bwd",
        )
        dx = dx.view(ctx.shape)
        if use_main:
            ctx.w_ref.grad_added_to_main_grad = True
            if ctx.has_b:
                ctx.b_ref.grad_added_to_main_grad = True
            dw_ret, db_ret = None, None
        else:
            dw_ret, db_ret = dw_out, db_out
        # the residual input receives the same gradient as x
        return dx, (dx if ctx.has_res else None), dw_ret, (db_ret if ctx.has_b else None), None, None, None


def _norm(x, w, b, eps, residual, is_ln, w_offset):
    H = x.shape[-1]
    if _native_ok(x) and H % 8 == 0 and H <= 8192:
        y, h = _NormFn.apply(x, residual, w, b, eps, is_ln, w_offset)
        return (y, h) if residual is not None else y
    if residual is not None:
        h = x + residual
        return _norm_ref(h, w, b, eps, is_ln, w_offset), h
    return _norm_ref(x, w, b, eps, is_ln, w_offset)


def rms_norm(x, weight, eps: float = 1e-6, residual=None, weight_offset: float = 0.0):
    """RMSNorm; with ``residual`` returns ``(norm(x + residual), x + residual)``.  ``weight_offset=1`` is Gemma's (1+w)."""
    return _norm(x, weight, None, eps, residual, False, weight_offset)


def layer_norm(x, weight, bias=None, eps: float = 1e-5, residual=None):
    """LayerNorm; with ``residual`` returns ``(norm(x + residual), x + residual)``."""
    return _norm(x, weight, bias, eps, residual, True, 0.0)


# --------------------------------------------------------------------------------------- RoPE
def rope_tables(max_pos: int, dim: int, theta: float = 10000.0, device="cpu", scaling: dict | None = None):
    """fp32 ``cos, sin`` tables ``[max_pos, dim/2]`` (llama3-style frequency scaling when ``scaling`` is given)."""
    inv = 1.0 / (theta ** (torch.arange(0, dim, 2, dtype=torch.float32, device=device) / dim))
    if scaling and scaling.get("rope_type", scaling.get("type")) == "llama3":
        factor = scaling["factor"]
        lo, hi = scaling["low_freq_factor"], scaling["high_freq_factor"]
        old = scaling["original_max_position_embeddings"]
        wavelen = 2 * torch.pi / inv
        smooth = ((old / wavelen) - lo) / (hi - lo)
        scaled = torch.where(wavelen > old / lo, inv / factor, inv)
        mid = (1 - smooth) * inv / factor + smooth * inv
        is_mid = (wavelen <= old / lo) & (wavelen >= old / hi)
        inv = torch.where(is_mid, mid, scaled)
    elif scaling and scaling.get("rope_type", scaling.get("type")) == "linear":
        inv = inv / scaling["factor"]
    t = torch.arange(max_pos, dtype=torch.float32, device=device)
    fr = torch.outer(t, inv)
    return fr.cos().contiguous(), fr.sin().contiguous()


def _rope_ref(x, cos, sin, pos, rot_dim):
    # x: [B, S, H, D]; cos/sin: [P, rot/2]; pos: [B, S] or None
    B, S = x.shape[:2]
    idx = pos.long() if pos is not None else torch.arange(S, device=x.device).expand(B, S)
    c = cos[idx][:, :, None, :].float()
    s = sin[idx][:, :, None, :].float()
    half = rot_dim // 2
    x1, x2, rest = x[..., :half].float(), x[..., half:rot_dim].float(), x[..., rot_dim:]
    o1 = x1 * c - x2 * s
    o2 = x2 * c + x1 * s
    return torch.cat([o1.to(x.dtype), o2.to(x.dtype), rest], dim=-1)


class _RopeFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, buf, cos, sin, pos, n_heads, D, rot_dim):
        B, S, W = buf.shape
        assert buf.stride(2) == 1 and buf.stride(1) % 8 == 0 and buf.stride(0) == S * buf.stride(1)
        p = pos.int().contiguous() if pos is not None else None
        nat.check(
            nat.lib().csb_rope(buf.data_ptr(), cos.data_ptr(), sin.data_ptr(), nat.ptr(p), B * S, S, buf.stride(1),
                               n_heads, D, rot_dim, 1.0, cos.shape[0], nat.stream()),
            "csb_rope",
        )
        ctx.save_for_backward(cos, sin, p)
        ctx.args = (n_heads, D, rot_dim)
        ctx.mark_dirty(buf)
        return buf

    @staticmethod
    def backward(ctx, g):
        cos, sin, p = ctx.saved_tensors
        n_heads, D, rot_dim = ctx.args
        g = g.contiguous() if not (g.stride(2) == 1 and g.stride(0) == g.shape[1] * g.stride(1)) else g
        B, S, W = g.shape
        nat.check(
            nat.lib().csb_rope(g.data_ptr(), cos.data_ptr(), sin.data_ptr(), nat.ptr(p), B * S, S, g.stride(1), n_heads,
                               D, rot_dim, -1.0, cos.shape[0], nat.stream()),
            "csb_rope(bwd)",
        )
        return g, None, None, None, None, None, None


def rope_(fused: torch.Tensor, cos, sin, pos, n_heads: int, head_dim: int, rot_dim: int | None = None):
    """Rotate the first ``n_heads`` heads of each token row of ``fused [B, S, W]`` (the q|k block of a fused
    q|k|v projection).  In place on CUDA/bf16 (the backward also rotates the incoming gradient in place)."""
    rot_dim = rot_dim or head_dim
    if _native_ok(fused) and rot_dim % 16 == 0:
        return _RopeFn.apply(fused, cos, sin, pos, n_heads, head_dim, rot_dim)
    B, S, W = fused.shape
    qk = fused[..., : n_heads * head_dim].reshape(B, S, n_heads, head_dim)
    qk = _rope_ref(qk, cos.to(fused.device), sin.to(fused.device), pos, rot_dim)
    return torch.cat([qk.reshape(B, S, n_heads * head_dim), fused[..., n_heads * head_dim :]], dim=-1)


# --------------------------------------------------------------------------------------- activations
_GLU_ACT = {"silu": 0, "swish": 0, "gelu_pytorch_tanh": 1, "gelu_tanh": 1}
_ACT_KIND = {"gelu_pytorch_tanh": 1, "gelu_tanh": 1, "gelu_new": 1, "gelu": 2, "gelu_erf": 2, "quick_gelu": 3, "silu": 4,
             "swish": 4}


def _act_ref(x, name):
    if name in ("gelu_pytorch_tanh", "gelu_tanh", "gelu_new"):
        return F.gelu(x, approximate="tanh")
    if name in ("gelu", "gelu_erf"):
        return F.gelu(x)
    if name == "quick_gelu":
        return x * torch.sigmoid(1.702 * x)
    if name in ("silu", "swish"):
        return F.silu(x)
    if name == "relu":
        return F.relu(x)
    raise ValueError(f"unknown activation {name}")


class _GluFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, gu, act):
        I = gu.shape[-1] // 2
        g2 = gu.reshape(-1, 2 * I)
        g2 = g2 if g2.is_contiguous() else g2.contiguous()
        y = torch.empty((g2.shape[0], I), dtype=gu.dtype, device=gu.device)
        nat.check(nat.lib().csb_glu_fwd(g2.data_ptr(), y.data_ptr(), g2.shape[0], I, act, nat.stream()), "csb_glu_fwd")
        ctx.save_for_backward(g2)
        ctx.act, ctx.shape = act, gu.shape
        return y.view(*gu.shape[:-1], I)

    @staticmethod
    def backward(ctx, dy):
        (g2,) = ctx.saved_tensors
        I = g2.shape[1] // 2
        d2 = dy.reshape(-1, I)
        d2 = d2 if d2.is_contiguous() else d2.contiguous()
        dgu = torch.empty_like(g2)
        nat.check(nat.lib().csb_glu_bwd(g2.data_ptr(), d2.data_ptr(), dgu.data_ptr(), g2.shape[0], I, ctx.act, nat.stream()),
                  "csb_glu_bwd")
        return dgu.view(ctx.shape), None


def glu(gate_up: torch.Tensor, act: str = "silu") -> torch.Tensor:
    """``act(gate) * up`` where ``gate_up = [gate | up]`` along the last dimension."""
    I = gate_up.shape[-1] // 2
    if _native_ok(gate_up) and I % 8 == 0 and act in _GLU_ACT:
        return _GluFn.apply(gate_up, _GLU_ACT[act])
    return _act_ref(gate_up[..., :I], act) * gate_up[..., I:]


class _ActFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, kind):
        xc = x if x.is_contiguous() else x.contiguous()
        y = torch.empty_like(xc)
        nat.check(nat.lib().csb_act_fwd(xc.data_ptr(), y.data_ptr(), xc.numel(), kind, nat.stream()), "csb_act_fwd")
        ctx.save_for_backward(xc)
        ctx.kind = kind
        return y

    @staticmethod
    def backward(ctx, dy):
        (xc,) = ctx.saved_tensors
        d = dy if dy.is_contiguous() else dy.contiguous()
        dx = torch.empty_like(xc)
        nat.check(nat.lib().csb_act_bwd(xc.data_ptr(), d.data_ptr(), dx.data_ptr(), xc.numel(), ctx.kind, nat.stream()),
                  "csb_act_bwd")
        return dx, None


def activation(x: torch.Tensor, name: str) -> torch.Tensor:
    if _native_ok(x) and name in _ACT_KIND and x.numel() % 8 == 0:
        return _ActFn.apply(x, _ACT_KIND[name])
    return _act_ref(x, name)


# --------------------------------------------------------------------------------------- embedding + merge
class _EmbedMergeFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, weight, feats, src):
        T = src.numel()
        H = weight.shape[1]
        out = torch.empty((T, H), dtype=weight.dtype, device=weight.device)
        f = feats if feats is not None else weight
        nat.check(nat.lib().csb_gather_merge(weight.data_ptr(), f.data_ptr(), src.data_ptr(), out.data_ptr(), T, H,
                                             weight.shape[0], feats.shape[0] if feats is not None else 0, nat.stream()),
                  "csb_gather_merge")
        ctx.n_embed = weight.shape[0]
        ctx.save_for_backward(src)
        ctx.w_ref = weight
        ctx.n_feats = feats.shape[0] if feats is not None else 0
        return out

    @staticmethod
    def backward(ctx, dout):
        (src,) = ctx.saved_tensors
        w = ctx.w_ref
        d = dout if dout.is_contiguous() else dout.contiguous()
        T, H = d.shape
        dfe = torch.zeros((ctx.n_feats, H), dtype=d.dtype, device=d.device) if ctx.n_feats and ctx.needs_input_grad[1] else None
        dw_ret = None
        demb = None
        if ctx.needs_input_grad[0]:
            main = getattr(w, "main_grad", None)
            if main is not None:
                demb = main
                w.grad_added_to_main_grad = True
            else:
                demb = torch.zeros(w.shape, dtype=torch.float32, device=d.device)
        nat.check(
            nat.lib().csb_scatter_merge_bwd(d.data_ptr(), src.data_ptr(), nat.ptr(demb),
                                            int(demb is not None and demb.dtype == torch.float32), nat.ptr(dfe), T, H,
                                            ctx.n_embed, ctx.n_feats, nat.stream()),
            "csb_scatter_merge_bwd",
        )
        if demb is not None and getattr(w, "main_grad", None) is None:
            dw_ret = demb.to(w.dtype)
        return dw_ret, dfe, None


def embed_merge(weight: torch.Tensor, src: torch.Tensor, feats: torch.Tensor | None = None) -> torch.Tensor:
    """Rows ``weight[src]`` where ``src >= 0`` and ``feats[-src-1]`` where ``src < 0``; ``src`` is int32 ``[T]``."""
    if _native_ok(weight) and weight.shape[1] % 8 == 0:
        return _EmbedMergeFn.apply(weight, feats, src.int().contiguous())
    s = src.long()
    emb = F.embedding(s.clamp(min=0), weight)
    if feats is None:
        return emb
    is_feat = s < 0
    # rows that keep their embedding still gather SOME feature row; spread them over the rows (a clamp would put them all
    # on row 0 and make the gather's backward pass a sum of thousands of zero rows into one)
    picked = feats[torch.remainder(-s - 1, feats.shape[0])]
    return torch.where(is_feat[:, None], picked.to(emb.dtype), emb)
