"""EvaCLIP text tower, joint model and ``*WithProjection`` variants against a straightforward fp32 restatement of the
same math (plain ``torch`` ops on the model's own state dict): causal text attention with an optional padding mask,
pooled output at the end-of-text token, pre- and post-norm layers, LayerNorm and RMSNorm, projections, cosine logits and
the contrastive loss.  Also the configuration / checkpoint round trip and the pipeline unit names."""

import math

import pytest
import torch
import torch.nn.functional as F

from cornstarch_b200.models import evaclip as EV

TEXT = dict(vocab_size=99, hidden_size=32, intermediate_size=64, projection_dim=24, num_hidden_layers=2, num_attention_heads=4,
            max_position_embeddings=16)
VIS = dict(hidden_size=48, intermediate_size=96, num_hidden_layers=2, num_attention_heads=4, image_size=28, patch_size=14,
           projection_dim=24)


def _norm(x, sd, pre, rms, eps):
    if rms:
        return x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + eps) * sd[pre + ".weight"]
    return F.layer_norm(x, (x.shape[-1],), sd[pre + ".weight"], sd[pre + ".bias"], eps)


def _layer(x, sd, pre, heads, add_mask, cfg):
    rms, post, eps = cfg.use_rms_norm, cfg.post_layernorm, cfg.layer_norm_eps
    B, S, H = x.shape
    D = H // heads

    def lin(t, name):
        return F.linear(t, sd[f"{pre}.{name}.weight"], sd.get(f"{pre}.{name}.bias"))

    h = x if post else _norm(x, sd, pre + ".layer_norm1", rms, eps)
    q, k, v = (lin(h, f"self_attn.{n}_proj").view(B, S, heads, D).transpose(1, 2) for n in "qkv")
    s = q @ k.transpose(-1, -2) / math.sqrt(D)
    if add_mask is not None:
        s = s + add_mask
    o = (torch.softmax(s, -1) @ v).transpose(1, 2).reshape(B, S, H)
    o = lin(o, "self_attn.out_proj")
    x = x + (_norm(o, sd, pre + ".layer_norm1", rms, eps) if post else o)
    h = x if post else _norm(x, sd, pre + ".layer_norm2", rms, eps)
    m = lin(F.gelu(lin(h, "mlp.fc1")), "mlp.fc2")
    return x + (_norm(m, sd, pre + ".layer_norm2", rms, eps) if post else m)


def _text_oracle(sd, cfg, ids, attn=None, pre="text_model"):
    S = ids.shape[1]
    x = sd[f"{pre}.embeddings.token_embedding.weight"][ids] + sd[f"{pre}.embeddings.position_embedding.weight"][:S]
    mask = torch.full((S, S), float("-inf")).triu(1)[None, None]
    if attn is not None:
        mask = mask + torch.where(attn.bool(), 0.0, float("-inf"))[:, None, None, :]
    for i in range(cfg.num_hidden_layers):
        x = _layer(x, sd, f"{pre}.encoder.layers.{i}", cfg.num_attention_heads, mask, cfg)
    last = _norm(x, sd, f"{pre}.final_layer_norm", cfg.use_rms_norm, cfg.layer_norm_eps)
    return last, last[torch.arange(ids.shape[0]), ids.argmax(-1)]


def _vision_oracle(sd, cfg, pix, pre="vision_model"):
    x = F.conv2d(pix, sd[f"{pre}.embeddings.patch_embedding.weight"], sd[f"{pre}.embeddings.patch_embedding.bias"],
                 stride=cfg.patch_size).flatten(2).transpose(1, 2)
    x = torch.cat([sd[f"{pre}.embeddings.class_embedding"].expand(x.shape[0], 1, -1), x], 1)
    x = x + sd[f"{pre}.embeddings.position_embedding.weight"][: x.shape[1]]
    for i in range(cfg.num_hidden_layers):
        x = _layer(x, sd, f"{pre}.encoder.layers.{i}", cfg.num_attention_heads, None, cfg)
    return x, _norm(x[:, 0], sd, f"{pre}.post_layernorm", cfg.use_rms_norm, cfg.layer_norm_eps)


@pytest.mark.parametrize("variant", ["prenorm_ln", "postnorm_rms", "no_qk_bias"])
def test_text_tower_matches_restatement(variant):
    torch.manual_seed(0)
    extra = {"prenorm_ln": {}, "postnorm_rms": dict(post_layernorm=True, use_rms_norm=True), "no_qk_bias": dict(k_bias=False)}[variant]
    cfg = EV.EvaCLIPTextConfig(**TEXT, **extra)
    model = EV.EvaCLIPTextModelWithProjection(cfg).eval()
    sd = {k: v.detach() for k, v in model.state_dict().items()}
    assert "text_model.embeddings.token_embedding.weight" in sd and "text_projection.weight" in sd
    assert ("text_model.encoder.layers.0.self_attn.k_proj.bias" in sd) == (variant != "no_qk_bias")
    ids = torch.randint(3, 98, (3, 11))
    ids[:, -1] = 98  # end-of-text token: the highest id
    out = model(input_ids=ids)
    last, pooled = _text_oracle(sd, cfg, ids)
    assert torch.allclose(out.last_hidden_state, last, atol=2e-5, rtol=1e-4)
    assert torch.allclose(out.text_embeds, pooled @ sd["text_projection.weight"].t(), atol=2e-5, rtol=1e-4)
    # padded batch: the last three positions of sample 0 are padding, its end-of-text token sits before them
    attn = torch.ones(3, 11, dtype=torch.long)
    attn[0, 8:] = 0
    ids2 = ids.clone()
    ids2[0, 8:] = 1
    ids2[0, 7] = 98
    base = EV.EvaCLIPTextModel(cfg).eval()
    base.load_state_dict({k: v for k, v in sd.items() if k.startswith("text_model.")})
    got = base(input_ids=ids2, attention_mask=attn)
    last2, pooled2 = _text_oracle(sd, cfg, ids2, attn)
    keep = attn.bool()
    assert torch.allclose(got.last_hidden_state[keep], last2[keep], atol=2e-5, rtol=1e-4)
    assert torch.allclose(got.pooler_output, pooled2, atol=2e-5, rtol=1e-4)


def test_joint_model_logits_loss_and_features():
    torch.manual_seed(1)
    cfg = EV.EvaCLIPConfig(text_config=TEXT, vision_config=VIS, projection_dim=24)
    model = EV.EvaCLIPModel(cfg).eval()
    sd = {k: v.detach() for k, v in model.state_dict().items()}
    ids = torch.randint(3, 98, (4, 9))
    ids[:, -1] = 98
    pix = torch.randn(4, 3, 28, 28)
    out = model(input_ids=ids, pixel_values=pix, return_loss=True)
    _, tp = _text_oracle(sd, cfg.text_config, ids)
    _, vp = _vision_oracle(sd, cfg.vision_config, pix)
    te = tp @ sd["text_projection.weight"].t()
    ie = vp @ sd["visual_projection.weight"].t()
    assert torch.allclose(model.encode_text(ids), te, atol=2e-5, rtol=1e-4)
    assert torch.allclose(model.encode_image(pix), ie, atol=2e-5, rtol=1e-4)
    te, ie = te / te.norm(dim=-1, keepdim=True), ie / ie.norm(dim=-1, keepdim=True)
    logits = te @ ie.t() * 100.0
    assert torch.allclose(out.logits_per_text, logits, atol=2e-3, rtol=1e-4)
    assert torch.allclose(out.logits_per_image, logits.t(), atol=2e-3, rtol=1e-4)
    tgt = torch.arange(4)
    want = (F.cross_entropy(logits, tgt) + F.cross_entropy(logits.t(), tgt)) / 2
    assert torch.allclose(out.loss, want, atol=1e-4, rtol=1e-4)
    out.loss.backward()
    assert model.text_projection.weight.grad is not None and model.vision_model.embeddings.class_embedding.grad is not None


def test_vision_with_projection_and_round_trip(tmp_path):
    torch.manual_seed(2)
    vcfg = EV.EvaCLIPVisionConfig(**VIS)
    vis = EV.EvaCLIPVisionModelWithProjection(vcfg).eval()
    sd = {k: v.detach() for k, v in vis.state_dict().items()}
    pix = torch.randn(2, 3, 28, 28)
    _, pooled = _vision_oracle(sd, vcfg, pix)
    assert torch.allclose(vis(pixel_values=pix).image_embeds, pooled @ sd["visual_projection.weight"].t(), atol=2e-5, rtol=1e-4)
    # configuration and checkpoint round trip of the joint model, and the model_type registry
    cfg = EV.EvaCLIPConfig.from_text_vision_configs(EV.EvaCLIPTextConfig(**TEXT), vcfg, projection_dim=24)
    model = EV.EvaCLIPModel(cfg).eval()
    model.save_pretrained(str(tmp_path))
    from cornstarch_b200.models import AutoModel

    again = AutoModel.from_pretrained(str(tmp_path))
    assert isinstance(again, EV.EvaCLIPModel) and again.config == cfg
    for (n, a), (_, b) in zip(model.state_dict().items(), again.state_dict().items()):
        assert torch.equal(a, b), n
    names = EV.EvaCLIPModel.module_names(cfg)
    assert names[0] == "text_model.embeddings" and names[-1] == "visual_projection" and len(names) == 2 * 2 + 6
    assert EV.EvaCLIPTextModel.module_names(cfg.text_config) == [
        "text_model.embeddings", "text_model.encoder.layers.0", "text_model.encoder.layers.1", "text_model.final_layer_norm"]
