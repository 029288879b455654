"""HF-compatible sharded checkpoints under PP x TP: train -> save -> rebuild -> load -> equal parameters and optimizer
state -> identical next step; directory layout and index schema; frozen modules are not saved
(reference: tests/test_plugins/multimodal_parallel_plugin/test_multimodal_checkpoint_io.py:100-345)."""

import json
import os
import tempfile

import pytest
import torch
import torch.distributed as dist

from tests.dist_utils import run_distributed


def _shared_tmpdir():
    path = [tempfile.mkdtemp() if dist.get_rank() == 0 else None]
    dist.broadcast_object_list(path, src=0)
    return path[0]


def _boost(tp, llm_stages, freeze_vision=False, seed=0, shape="tiny", ep=1):
    from cornstarch_b200.booster import Booster
    from cornstarch_b200.optim.fused_adamw import FusedAdamW, split_decay_groups
    from cornstarch_b200.pipeline_template import PipelineTemplate
    from cornstarch_b200.plugin.modal_parallel_plugin import ModalParallelPlugin
    from cornstarch_b200.plugin.multimodal_parallel_plugin import MultimodalParallelPlugin
    from cornstarch_b200.zoo import build_model

    torch.manual_seed(seed)
    model = build_model(shape)
    if freeze_vision:
        model.train(encoders_mode={"vision": (False, True)}, llm_mode=True)
    plugin = MultimodalParallelPlugin(
        encoder_plugins={"vision": ModalParallelPlugin(tp_size=tp, pipeline_template=PipelineTemplate.even_split(model.vision_encoder, 1))},
        language_model_plugin=ModalParallelPlugin(tp_size=tp, pipeline_template=PipelineTemplate.even_split(model.language_model, llm_stages),
                                                  ep_size=ep),
        num_microbatches=2, device=torch.device("cpu"))
    booster = Booster(plugin=plugin)
    opt = FusedAdamW(split_decay_groups(model, 0.0), lr=1e-2)
    pmodel, popt, crit, *_ = booster.boost(model, opt, criterion=lambda out, b: out.loss)
    return booster, plugin, pmodel, popt, crit


def _step(booster, pmodel, popt, crit, seed, shape="tiny"):
    from cornstarch_b200.zoo import synthetic_batch

    out = booster.execute_pipeline(iter([synthetic_batch(shape, 4, seed=seed)]), pmodel, crit, popt, return_loss=True)
    popt.step()
    popt.zero_grad()
    return out["loss"]


def _mine(pmodel):
    return getattr(pmodel.module, pmodel.my_modal_name)


def _roundtrip_worker(rank, world, tp, llm_stages):
    booster, plugin, pmodel, popt, crit = _boost(tp, llm_stages, seed=0)
    _step(booster, pmodel, popt, crit, 1)
    root = _shared_tmpdir()
    booster.save_model(pmodel, os.path.join(root, "model"), shard=True, size_per_shard=1)
    booster.save_optimizer(popt, os.path.join(root, "optim"), shard=True, size_per_shard=1)
    dist.barrier()
    before = {k: v.detach().clone() for k, v in _mine(pmodel).state_dict().items()}
    loss_a = _step(booster, pmodel, popt, crit, 2)
    after_a = {k: v.detach().clone() for k, v in _mine(pmodel).state_dict().items()}

    # a fresh model with different initial weights, same plan
    from cornstarch_b200.parallel.symm import FusedTensorParallel  # noqa: F401

    booster2, plugin2, pmodel2, popt2, crit2 = _boost(tp, llm_stages, seed=123)
    # reuse the already initialised groups of the first plugin (new_group calls are collective and costly)
    booster2.load_model(pmodel2, os.path.join(root, "model"))
    booster2.load_optimizer(popt2, os.path.join(root, "optim"))
    for k, v in _mine(pmodel2).state_dict().items():
        assert torch.allclose(v, before[k], atol=1e-6), k
    loss_b = _step(booster2, pmodel2, popt2, crit2, 2)
    for k, v in _mine(pmodel2).state_dict().items():
        assert torch.allclose(v, after_a[k], atol=1e-5), (k, (v - after_a[k]).abs().max())
    if loss_a is not None:
        assert abs(loss_a.item() - loss_b.item()) < 1e-5

    dist.barrier()
    if rank == 0:
        # layout: one HF-style directory per module with an index whose weight_map covers the FULL (unsharded) names
        from cornstarch_b200.checkpoint.io import load_state_dict_any
        from cornstarch_b200.zoo import build_model

        ref = build_model("tiny")
        for sub, mod in (("language_model", ref.language_model), ("vision_encoder/module", ref.vision_encoder.module),
                         ("vision_encoder/projector", ref.vision_encoder.projector)):
            d = os.path.join(root, "model", sub)
            assert os.path.isfile(os.path.join(d, "config.json")), d
            sd = load_state_dict_any(d)
            want = mod.state_dict()
            assert set(sd) == set(want), (sub, set(want) ^ set(sd))
            for k in want:
                assert tuple(sd[k].shape) == tuple(want[k].shape), (sub, k)  # un-padded, un-TP-sharded
            idx = [f for f in os.listdir(d) if f.endswith(".index.json")]
            if idx:
                j = json.load(open(os.path.join(d, idx[0])))
                assert set(j) == {"metadata", "weight_map"} and "total_size" in j["metadata"]
            assert not os.path.isdir(os.path.join(d, "tmp_index_files"))
        assert os.path.isdir(os.path.join(root, "optim", "language_model"))
        # the language-model directory is a Hugging Face checkpoint: ``transformers`` loads it and computes the same logits
        try:
            import transformers as tf
        except ImportError:
            tf = None
        if tf is not None:
            from cornstarch_b200.models import AutoModel

            d = os.path.join(root, "model", "language_model")
            ours, theirs = AutoModel.from_pretrained(d).eval(), tf.AutoModelForCausalLM.from_pretrained(d).eval()
            ids = torch.randint(0, 900, (2, 16))
            with torch.no_grad():
                assert torch.allclose(ours(input_ids=ids).logits, theirs(input_ids=ids).logits, atol=1e-4)


@pytest.mark.parametrize("tp,llm_stages,world", [(1, 2, 3), (2, 1, 4)])
def test_checkpoint_roundtrip(tp, llm_stages, world):
    run_distributed(_roundtrip_worker, world, tp, llm_stages, timeout=600)


def _expert_parallel_worker(rank, world):
    """Two replicas of (encoder stage + MoE stage) with the experts sharded over the replicas: every rank of the expert
    group writes the experts it owns, the directory holds ALL experts under their global names, and a rebuilt model
    with the same plan loads weights and optimizer state back and takes the same next step."""
    kw = dict(shape="moe_tiny", ep=2)
    booster, plugin, pmodel, popt, crit = _boost(1, 1, seed=0, **kw)
    _step(booster, pmodel, popt, crit, 1, "moe_tiny")
    root = _shared_tmpdir()
    booster.save_model(pmodel, os.path.join(root, "model"), shard=True, size_per_shard=1)
    booster.save_optimizer(popt, os.path.join(root, "optim"), shard=True, size_per_shard=1)
    dist.barrier()
    before = {k: v.detach().clone() for k, v in _mine(pmodel).state_dict().items()}
    _step(booster, pmodel, popt, crit, 2, "moe_tiny")
    after_a = {k: v.detach().clone() for k, v in _mine(pmodel).state_dict().items()}
    booster2, plugin2, pmodel2, popt2, crit2 = _boost(1, 1, seed=123, **kw)
    booster2.load_model(pmodel2, os.path.join(root, "model"))
    booster2.load_optimizer(popt2, os.path.join(root, "optim"))
    for k, v in _mine(pmodel2).state_dict().items():
        assert torch.allclose(v, before[k], atol=1e-6), k
    _step(booster2, pmodel2, popt2, crit2, 2, "moe_tiny")
    for k, v in _mine(pmodel2).state_dict().items():
        assert torch.allclose(v, after_a[k], atol=1e-5), (k, (v - after_a[k]).abs().max())
    dist.barrier()
    if rank == 0:
        from cornstarch_b200.checkpoint.io import load_state_dict_any
        from cornstarch_b200.zoo import build_model

        want = build_model("moe_tiny").language_model.state_dict()
        sd = load_state_dict_any(os.path.join(root, "model", "language_model"))
        assert set(sd) == set(want), set(want) ^ set(sd)  # experts 0..3 of every layer, although no rank holds them all
        assert any(".experts.3." in k for k in sd)


def test_checkpoint_roundtrip_with_expert_parallelism():
    run_distributed(_expert_parallel_worker, 4, timeout=600)


def _frozen_worker(rank, world):
    booster, plugin, pmodel, popt, crit = _boost(1, 1, freeze_vision=True)
    _step(booster, pmodel, popt, crit, 1)
    root = _shared_tmpdir()
    booster.save_model(pmodel, os.path.join(root, "model"), shard=True)
    dist.barrier()
    if rank == 0:
        assert os.path.isdir(os.path.join(root, "model", "language_model"))
        assert os.path.isdir(os.path.join(root, "model", "vision_encoder", "projector"))
        assert not os.path.exists(os.path.join(root, "model", "vision_encoder", "module"))  # frozen => not saved
    with pytest.raises(NotImplementedError):
        booster.save_model(pmodel, os.path.join(root, "x"), shard=False)


def test_frozen_modules_are_not_saved():
    run_distributed(_frozen_worker, 2)


def test_projector_save_pretrained_roundtrip(tmp_path):
    from cornstarch_b200.models.llama import DecoderConfig
    from cornstarch_b200.models.vision import ViTConfig
    from cornstarch_b200.multimodal.modeling import MultimodalProjector, MultimodalProjectorConfig

    cfg = MultimodalProjectorConfig(encoder_config=ViTConfig(hidden_size=32), text_config=DecoderConfig(hidden_size=64, num_attention_heads=4),
                                    projection_type="mlp", activation="gelu")
    p = MultimodalProjector(cfg)
    p.save_pretrained(str(tmp_path))
    assert sorted(os.listdir(tmp_path)) == ["config.json", "model.safetensors"]
    q = MultimodalProjector.from_pretrained(str(tmp_path))
    assert set(q.state_dict()) == {"projection.in_proj.weight", "projection.in_proj.bias", "projection.out_proj.weight", "projection.out_proj.bias"}
    for k, v in p.state_dict().items():
        assert torch.equal(v, q.state_dict()[k])
    assert q.config.in_features == 32 and q.config.out_features == 64 and q.config.projection_type == "mlp"
    with pytest.raises(ValueError):
        MultimodalProjectorConfig(projection_type="conv")
