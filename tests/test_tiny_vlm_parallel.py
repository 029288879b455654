"""Tiny VLM on CPU / gloo, fp32: data-parallel (world 2) and modality-parallel pipeline (encoder stage + LLM
stage, world 2; encoder stage + 2 LLM stages x TP 2, world 6...) must reproduce the loss and the
post-step weights of the single-process model."""

import copy

import pytest
import torch
import torch.distributed as dist

from tests.dist_utils import run_distributed


def _build(seed=0, shape="tiny"):
    from cornstarch_b200.zoo import build_model

    torch.manual_seed(seed)
    m = build_model(shape)
    m.train()
    return m


def _batch(n, seed=1, shape="tiny"):
    from cornstarch_b200.zoo import synthetic_batch

    return synthetic_batch(shape, n, seed=seed)


def _single_process_reference(n_samples, n_micro, lr=1e-2, steps=2, shape="tiny", eps=1e-8, dense_grads=False):
    from cornstarch_b200.optim.fused_adamw import FusedAdamW, split_decay_groups

    model = _build(shape=shape)
    opt = FusedAdamW(split_decay_groups(model, 0.0), lr=lr, eps=eps)
    batch = _batch(n_samples, shape=shape)
    losses = []
    mb = n_samples // n_micro
    for _ in range(steps):
        total = 0.0
        for i in range(n_micro):
            sub = {k: v[i * mb : (i + 1) * mb] for k, v in batch.items()}
            loss = model(**sub).loss / n_micro
            loss.backward()
            total += loss.item()
        if dense_grads:
            # an expert that received no token has no gradient here and would be skipped by the optimizer; with sharded
            # experts (and in the flat gradient buffer on GPUs) it has a zero gradient and its momentum still moves it
            for p in model.parameters():
                if p.requires_grad and p.grad is None:
                    p.grad = torch.zeros_like(p)
        opt.step()
        opt.zero_grad()
        losses.append(total)
    return losses, {k: v.detach().clone() for k, v in model.state_dict().items()}


def _dp_worker(rank, world):
    from cornstarch_b200.optim.fused_adamw import FusedAdamW, split_decay_groups

    ref_losses, ref_sd = _single_process_reference(4, 2)
    model = _build()
    opt = FusedAdamW(split_decay_groups(model, 0.0), lr=1e-2)
    batch = _batch(4)
    mine = {k: v[rank * 2 : (rank + 1) * 2] for k, v in batch.items()}
    for step in range(2):
        loss = model(**mine).loss
        loss.backward()
        for p in model.parameters():
            if p.grad is not None:
                dist.all_reduce(p.grad)
                p.grad.div_(world)
        opt.step()
        opt.zero_grad()
        tot = loss.detach().clone()
        dist.all_reduce(tot)
        assert abs(tot.item() / world - ref_losses[step]) < 1e-4, (tot.item() / world, ref_losses[step])
    for k, v in model.state_dict().items():
        assert torch.allclose(v, ref_sd[k], atol=1e-5, rtol=1e-4), k


def test_dp2_matches_single_process():
    run_distributed(_dp_worker, 2)


def _pp_worker(rank, world, llm_stages, tp, n_micro):
    from cornstarch_b200.booster import Booster
    from cornstarch_b200.optim.fused_adamw import FusedAdamW, split_decay_groups
    from cornstarch_b200.pipeline_template import PipelineTemplate
    from cornstarch_b200.plugin.modal_parallel_plugin import ModalParallelPlugin
    from cornstarch_b200.plugin.multimodal_parallel_plugin import MultimodalParallelPlugin

    n_samples = 4
    ref_losses, ref_sd = _single_process_reference(n_samples, n_micro)
    model = _build()
    enc_tpl = PipelineTemplate.even_split(model.vision_encoder, 1)
    llm_tpl = PipelineTemplate.even_split(model.language_model, llm_stages)
    plugin = MultimodalParallelPlugin(
        encoder_plugins={"vision": ModalParallelPlugin(tp_size=tp, pipeline_template=enc_tpl)},
        language_model_plugin=ModalParallelPlugin(tp_size=tp, pipeline_template=llm_tpl),
        num_microbatches=n_micro, precision=None, device=torch.device("cpu"))
    booster = Booster(plugin=plugin)
    opt = FusedAdamW(split_decay_groups(model, 0.0), lr=1e-2)
    pmodel, popt, criterion, *_ = booster.boost(model, opt, criterion=lambda out, batch: out.loss)
    batch = _batch(n_samples)
    sm = plugin.stage_manager
    for step in range(2):
        out = booster.execute_pipeline(iter([batch]), pmodel, criterion, popt, return_loss=True)
        popt.step()
        popt.zero_grad()
        if sm.is_last_stage(check_only_in_modal=False):
            assert abs(out["loss"].item() - ref_losses[step]) < 1e-4, (out["loss"].item(), ref_losses[step])
    # post-step weights of the layers this rank holds equal the single-process ones (TP shards compared by slice)
    mine = getattr(pmodel.module, pmodel.my_modal_name)
    from cornstarch_b200 import nn as cnn

    prefix = pmodel.my_modal_name + "."
    tp_rank = dist.get_rank(plugin.tp_group) if tp > 1 else 0
    for name, mod in mine.named_modules():
        for pn, p in mod.named_parameters(recurse=False):
            full = ref_sd[prefix + (name + "." if name else "") + pn]
            if isinstance(mod, cnn.ColumnParallelLinear) and hasattr(mod, "full_vocab_size"):
                local = mod.weight.shape[0]
                full = torch.cat([full, full.new_zeros(local * tp - full.shape[0], full.shape[1])])[tp_rank * local : (tp_rank + 1) * local]
            elif isinstance(mod, cnn.ColumnParallelLinear):
                full = full.chunk(tp, dim=0)[tp_rank]
            elif isinstance(mod, cnn.RowParallelLinear) and pn == "weight":
                full = full.chunk(tp, dim=1)[tp_rank]
            elif isinstance(mod, cnn.VocabParallelEmbedding):
                pad = mod.padded_num_embeddings - full.shape[0]
                full = torch.cat([full, full.new_zeros(pad, full.shape[1])])[mod.vocab_start : mod.vocab_end]
            assert torch.allclose(p.detach(), full, atol=2e-3, rtol=5e-3), (name, pn, (p.detach() - full).abs().max())


@pytest.mark.parametrize("llm_stages,tp,n_micro,world", [(1, 1, 2, 2), (2, 1, 4, 3), (1, 2, 2, 4)])
def test_modality_parallel_pipeline_matches_single_process(llm_stages, tp, n_micro, world):
    run_distributed(_pp_worker, world, llm_stages, tp, n_micro)


def test_pipeline_with_token_sharded_tensor_parallelism(monkeypatch):
    """Encoder stage + 2 LLM stages x TP 2 with token-sharded activations between the tensor-parallel blocks: the LLM
    stages hand only their rank's token rows to the next stage, and loss / weights still match the single process."""
    monkeypatch.setenv("CORNSTARCH_B200_TP_SEQ_SHARD", "1")
    run_distributed(_pp_worker, 6, 2, 2, 4)


def _colocated_worker(rank, world):
    from cornstarch_b200.booster import Booster
    from cornstarch_b200.optim.fused_adamw import FusedAdamW, split_decay_groups
    from cornstarch_b200.pipeline_template import PipelineTemplate
    from cornstarch_b200.plugin.encoders_colocated_plugin import EncodersColocatedMultimodalParallelPlugin
    from cornstarch_b200.plugin.modal_parallel_plugin import ModalParallelPlugin

    n_micro = 2
    ref_losses, ref_sd = _single_process_reference(4, n_micro)
    model = _build()
    plugin = EncodersColocatedMultimodalParallelPlugin(
        encoder_plugins={"vision": ModalParallelPlugin(pipeline_template=PipelineTemplate.even_split(model.vision_encoder, 1))},
        language_model_plugin=ModalParallelPlugin(pipeline_template=PipelineTemplate.even_split(model.language_model, 2)),
        num_microbatches=n_micro, device=torch.device("cpu"))
    booster = Booster(plugin=plugin)
    opt = FusedAdamW(split_decay_groups(model, 0.0), lr=1e-2)
    pmodel, popt, criterion, *_ = booster.boost(model, opt, criterion=lambda out, batch: out.loss)
    batch = _batch(4)
    for step in range(2):
        out = booster.execute_pipeline(iter([batch]), pmodel, criterion, popt, return_loss=True)
        popt.step()
        popt.zero_grad()
        if plugin.stage_manager.is_last_stage(check_only_in_modal=False):
            assert abs(out["loss"].item() - ref_losses[step]) < 1e-4, (out["loss"].item(), ref_losses[step])


def test_encoders_colocated_pipeline_matches_single_process():
    run_distributed(_colocated_worker, 3)


def _valm_worker(rank, world):
    """Vision and audio encoders as parallel pipeline branches feeding one LLM stage (3 ranks)."""
    from cornstarch_b200.booster import Booster
    from cornstarch_b200.optim.fused_adamw import FusedAdamW, split_decay_groups
    from cornstarch_b200.pipeline_template import PipelineTemplate
    from cornstarch_b200.plugin.modal_parallel_plugin import ModalParallelPlugin
    from cornstarch_b200.plugin.multimodal_parallel_plugin import MultimodalParallelPlugin
    from cornstarch_b200.zoo import build_model, synthetic_batch

    n_micro = 2
    torch.manual_seed(0)
    ref = build_model("valm_tiny")
    ref.train()
    batch = synthetic_batch("valm_tiny", 4, seed=1)
    ref_loss = 0.0
    for i in range(n_micro):
        sub = {k: v[2 * i : 2 * i + 2] for k, v in batch.items()}
        ref_loss += (ref(**sub).loss / n_micro).item()
    torch.manual_seed(0)
    model = build_model("valm_tiny")
    model.train()
    plugin = MultimodalParallelPlugin(
        encoder_plugins={"vision": ModalParallelPlugin(pipeline_template=PipelineTemplate.even_split(model.vision_encoder, 1)),
                         "audio": ModalParallelPlugin(pipeline_template=PipelineTemplate.even_split(model.audio_encoder, 1))},
        language_model_plugin=ModalParallelPlugin(pipeline_template=PipelineTemplate.even_split(model.language_model, 1)),
        num_microbatches=n_micro, device=torch.device("cpu"))
    booster = Booster(plugin=plugin)
    opt = FusedAdamW(split_decay_groups(model, 0.0), lr=1e-2)
    pmodel, popt, criterion, *_ = booster.boost(model, opt, criterion=lambda out, b: out.loss)
    out = booster.execute_pipeline(iter([batch]), pmodel, criterion, popt, return_loss=True)
    if plugin.stage_manager.is_last_stage(check_only_in_modal=False):
        assert abs(out["loss"].item() - ref_loss) < 1e-4, (out["loss"].item(), ref_loss)
    popt.step()


def test_two_encoder_branches_match_single_process():
    run_distributed(_valm_worker, 3)


def _phi4_audio_lm(seed=0):
    """Phi-4 audio encoder (its attention bias is computed once, on the encoder's first stage) + a tiny Llama."""
    from cornstarch_b200.models.llama import DecoderConfig, DecoderForCausalLM
    from cornstarch_b200.models.phi4_audio import Phi4MultimodalAudioConfig, Phi4MultimodalAudioModel
    from cornstarch_b200.multimodal.modeling import ModalEncoderModule, MultimodalModel
    from cornstarch_b200.multimodal.modeling import MultimodalProjector, MultimodalProjectorConfig

    torch.manual_seed(seed)
    acfg = Phi4MultimodalAudioConfig(hidden_size=64, intermediate_size=96, num_blocks=2, num_attention_heads=4, input_size=16,
                                     nemo_conv_channels=32, ext_pw_out_channel=64, kernel_size=3, time_reduction=8,
                                     depthwise_separable_out_channel=64)
    lcfg = DecoderConfig(vocab_size=128, hidden_size=64, intermediate_size=128, num_hidden_layers=2, num_attention_heads=4,
                         num_key_value_heads=2, max_position_embeddings=128)
    pcfg = MultimodalProjectorConfig(encoder_config=acfg, text_config=lcfg, projection_type="linear")
    model = MultimodalModel(encoders={"audio": ModalEncoderModule(Phi4MultimodalAudioModel(acfg), MultimodalProjector(pcfg))},
                            language_model=DecoderForCausalLM(lcfg))
    model.set_modality_token_ids({"audio": 127})
    model.train()
    g = torch.Generator().manual_seed(3)
    feats = torch.randn(4, 64, 16, generator=g)  # 64 frames / time_reduction 8 = 8 audio tokens per sample
    ids = torch.randint(0, 127, (4, 32), generator=g)
    ids[:, 2:10] = 127
    return model, {"audio_input_features": feats, "input_ids": ids, "labels": ids.clone()}


def _two_stage_encoder_worker(rank, world, tp):
    from cornstarch_b200.booster import Booster
    from cornstarch_b200.optim.fused_adamw import FusedAdamW, split_decay_groups
    from cornstarch_b200.pipeline_template import PipelineTemplate
    from cornstarch_b200.plugin.modal_parallel_plugin import ModalParallelPlugin
    from cornstarch_b200.plugin.multimodal_parallel_plugin import MultimodalParallelPlugin

    n_micro = 2
    ref, batch = _phi4_audio_lm()
    ref_loss = 0.0
    for i in range(n_micro):
        loss = ref(**{k: v[2 * i : 2 * i + 2] for k, v in batch.items()}).loss / n_micro
        loss.backward()
        ref_loss += loss.item()
    model, _ = _phi4_audio_lm()
    plugin = MultimodalParallelPlugin(
        encoder_plugins={"audio": ModalParallelPlugin(tp_size=tp, pipeline_template=PipelineTemplate.even_split(model.audio_encoder, 2))},
        language_model_plugin=ModalParallelPlugin(tp_size=tp, pipeline_template=PipelineTemplate.even_split(model.language_model, 1)),
        num_microbatches=n_micro, precision=None, device=torch.device("cpu"))
    booster = Booster(plugin=plugin)
    opt = FusedAdamW(split_decay_groups(model, 0.0), lr=1e-2)
    pmodel, popt, criterion, *_ = booster.boost(model, opt, criterion=lambda out, b: out.loss)
    out = booster.execute_pipeline(iter([batch]), pmodel, criterion, popt, return_loss=True)
    sm = plugin.stage_manager
    if sm.is_last_stage(check_only_in_modal=False):
        assert abs(out["loss"].item() - ref_loss) < 1e-4, (out["loss"].item(), ref_loss)
    if pmodel.my_modal_name == "audio_encoder" and sm.is_first_stage(check_only_in_modal=True):
        # the bias table sits on the first encoder stage; its gradient comes back through the second stage's attention
        got = pmodel.module.audio_encoder.module.relative_attention_bias_layer.bias_values.weight.grad
        want = ref.audio_encoder.module.relative_attention_bias_layer.bias_values.weight.grad
        assert got is not None and torch.allclose(got, want, atol=1e-5, rtol=1e-3), (got - want).abs().max()


@pytest.mark.parametrize("tp,world", [(1, 3), (2, 6)])
def test_two_stage_encoder_hands_on_its_attention_bias(tp, world):
    run_distributed(_two_stage_encoder_worker, world, tp)


def _colocated_two_stage_encoder_worker(rank, world):
    """The colocated plugin with a two-stage audio encoder: the attention bias travels beside the encoder's hidden states."""
    from cornstarch_b200.booster import Booster
    from cornstarch_b200.optim.fused_adamw import FusedAdamW, split_decay_groups
    from cornstarch_b200.pipeline_template import PipelineTemplate
    from cornstarch_b200.plugin.encoders_colocated_plugin import EncodersColocatedMultimodalParallelPlugin
    from cornstarch_b200.plugin.modal_parallel_plugin import ModalParallelPlugin

    n_micro = 2
    ref, batch = _phi4_audio_lm()
    ref_loss = sum((ref(**{k: v[2 * i : 2 * i + 2] for k, v in batch.items()}).loss / n_micro).item() for i in range(n_micro))
    model, _ = _phi4_audio_lm()
    plugin = EncodersColocatedMultimodalParallelPlugin(
        encoder_plugins={"audio": ModalParallelPlugin(pipeline_template=PipelineTemplate.even_split(model.audio_encoder, 2))},
        language_model_plugin=ModalParallelPlugin(pipeline_template=PipelineTemplate.even_split(model.language_model, 1)),
        num_microbatches=n_micro, device=torch.device("cpu"))
    booster = Booster(plugin=plugin)
    opt = FusedAdamW(split_decay_groups(model, 0.0), lr=1e-2)
    pmodel, popt, criterion, *_ = booster.boost(model, opt, criterion=lambda out, b: out.loss)
    out = booster.execute_pipeline(iter([batch]), pmodel, criterion, popt, return_loss=True)
    if plugin.stage_manager.is_last_stage(check_only_in_modal=False):
        assert abs(out["loss"].item() - ref_loss) < 1e-4, (out["loss"].item(), ref_loss)


def test_colocated_two_stage_encoder():
    run_distributed(_colocated_two_stage_encoder_worker, 3)


def _ep_plugin_worker(rank, world, capacity, llm_stages=1):
    """Encoder stage + MoE language-model stage, two data-parallel replicas, the experts of every sparse block sharded over
    the two replicas by the plugin (``ModalParallelPlugin(ep_size=2)``): loss and post-step weights equal the
    single-process model with all experts local."""
    from cornstarch_b200.booster import Booster
    from cornstarch_b200.optim.fused_adamw import FusedAdamW, split_decay_groups
    from cornstarch_b200.pipeline_template import PipelineTemplate
    from cornstarch_b200.plugin.modal_parallel_plugin import ModalParallelPlugin
    from cornstarch_b200.plugin.multimodal_parallel_plugin import MultimodalParallelPlugin

    # a larger epsilon than the default: with 1e-8 the first Adam steps move every weight by +-lr whatever the size of its
    # gradient, so elements whose gradient is rounding noise (experts that saw few tokens) differ by whole steps
    ref_losses, ref_sd = _single_process_reference(4, 4, shape="moe_tiny", eps=1e-4, dense_grads=True)
    model = _build(shape="moe_tiny")
    plugin = MultimodalParallelPlugin(
        encoder_plugins={"vision": ModalParallelPlugin(pipeline_template=PipelineTemplate.even_split(model.vision_encoder, 1))},
        language_model_plugin=ModalParallelPlugin(pipeline_template=PipelineTemplate.even_split(model.language_model, llm_stages),
                                                  ep_size=2, ep_capacity_factor=capacity),
        num_microbatches=2, precision=None, device=torch.device("cpu"))
    booster = Booster(plugin=plugin)
    opt = FusedAdamW(split_decay_groups(model, 0.0), lr=1e-2, eps=1e-4)
    pmodel, popt, criterion, *_ = booster.boost(model, opt, criterion=lambda out, batch: out.loss)
    assert plugin.dp_size == 2
    M = plugin.pg_mesh
    replica = M.coords[0][M.dp_axis]
    batch = {k: v[replica * 2 : (replica + 1) * 2] for k, v in _batch(4, shape="moe_tiny").items()}
    sm = plugin.stage_manager
    mine = getattr(pmodel.module, pmodel.my_modal_name)
    if pmodel.my_modal_name == "language_model":
        blocks = [m for m in mine.modules() if getattr(m, "ep", None) is not None]
        assert blocks and all(len(b.experts) == 2 for b in blocks)  # 4 experts over 2 ranks
    for step in range(2):
        out = booster.execute_pipeline(iter([batch]), pmodel, criterion, popt, return_loss=True)
        popt.step()
        popt.zero_grad()
        if sm.is_last_stage(check_only_in_modal=False):
            mean = out["loss"].detach().clone()
            dist.all_reduce(mean, group=plugin.dp_group)
            assert abs(mean.item() / 2 - ref_losses[step]) < 1e-4, (mean.item() / 2, ref_losses[step])
    prefix = pmodel.my_modal_name + "."
    ep_rank = dist.get_rank(plugin.dp_group)
    for name, p in mine.named_parameters():
        key = prefix + name
        if getattr(p, "expert_parallel", False):
            # local expert j of this rank is expert ep_rank * 2 + j of the whole model
            head, j, tail = name.partition(".experts.")[0], int(name.partition(".experts.")[2].split(".")[0]), name.partition(".experts.")[2].split(".", 1)[1]
            key = f"{prefix}{head}.experts.{ep_rank * 2 + j}.{tail}"
        assert torch.allclose(p.detach(), ref_sd[key], atol=2e-3, rtol=5e-3), (name, (p.detach() - ref_sd[key]).abs().max())


@pytest.mark.parametrize("capacity,llm_stages,world", [(4.0, 1, 4), (None, 2, 6)])
def test_plugin_expert_parallelism_matches_single_process(capacity, llm_stages, world):
    run_distributed(_ep_plugin_worker, world, capacity, llm_stages)
