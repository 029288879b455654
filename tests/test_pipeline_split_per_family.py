"""Pipeline split per model family, in one process: the model cut into two stages (``PipelineTemplate.even_split`` +
``hold_only``) with the first stage's output handed to the second gives the loss / features and the input gradient of
the whole model.  Checks every family's ``module_names``, stage pruning and stage-to-stage hand-over."""

import copy

import pytest
import torch

from cornstarch_b200.pipeline_template import PipelineTemplate
from tests.test_policy_tp_numerics import _build, _run

FAMILIES = ["llama", "mistral", "qwen2", "qwen3", "gemma", "gemma2", "gemma3", "phi3", "mixtral", "qwen3_moe", "llama4", "gpt2",
            "opt", "bert", "siglip", "clip", "vit", "dinov2", "internvit", "evaclip", "pixtral", "whisper", "qwen2_audio", "phi4_audio", "qwen2_vl"]


def _build_any(family):
    if family == "gpt2":
        from cornstarch_b200.models import text_legacy as T

        return T.GPT2LMHeadModel(T.GPT2Config(n_layer=2, n_embd=64, n_head=4, vocab_size=128, n_positions=64,
                                              tie_word_embeddings=False)), "text"
    return _build(family)


def _input(kind):
    g = torch.Generator().manual_seed(5)
    if kind == "text":
        return torch.randint(0, 128, (2, 24), generator=g)
    if kind == "image":
        return torch.randn(2, 3, 28, 28, generator=g)
    if kind == "image56":
        return torch.randn(2, 3, 56, 56, generator=g)
    if kind == "phi4":
        return torch.randn(2, 64, 16, generator=g)
    if kind == "qwen2vl":
        return torch.randn(32, 3 * 2 * 14 * 14, generator=g)
    return torch.randn(2, 8, 20, generator=g)


@pytest.mark.parametrize("family", FAMILIES)
def test_two_stage_split_matches_whole_model(family):
    torch.manual_seed(0)
    whole, kind = _build_any(family)
    whole.eval()
    x = _input(kind)
    ref = _run(whole, kind, x)

    template = PipelineTemplate.even_split(whole, 2)
    assert template.num_stages == 2 and all(template.modules_per_stage)
    stages = []
    for names in template.modules_per_stage:
        m = copy.deepcopy(whole)
        m.hold_only(list(names))
        stages.append(m)
    assert sum(p.numel() for p in stages[0].parameters()) < sum(p.numel() for p in whole.parameters())

    key = {"text": "input_ids", "image": "pixel_values", "image56": "pixel_values", "audio": "input_features",
           "phi4": "audio_input_features", "qwen2vl": "hidden_states"}[kind]
    extra = {"grid_thw": torch.tensor([[1, 4, 4], [1, 4, 4]])} if kind == "qwen2vl" else {}
    first = stages[0](**{key: x}, **extra)
    passed = {k: v for k, v in first.items() if v is not None} if isinstance(first, dict) else {"hidden_states": first}
    assert "hidden_states" in passed, list(passed)
    if kind == "text":
        out = stages[1](labels=x, **passed)
        got = out.loss
    else:
        out = stages[1](**passed, **extra)
        h = out["last_hidden_state"] if isinstance(out, dict) else out[0]
        got = h.float().square().mean()
    assert abs(got.item() - ref.item()) < 1e-4 * max(1.0, abs(ref.item())), (family, got.item(), ref.item())
