"""Context parallelism: token->rank partitioners (tables for causal and full masks with 4 ranks, as in the
reference's tests/test_shardformer/test_context_parallel.py:30-63), attention over gathered K/V against the
single-device result, and end-to-end loss / gradient parity of a tiny Llama under ring_attn and Ulysses."""

import numpy as np
import pytest
import torch
import torch.distributed as dist

from cornstarch_b200.ops import attention as A
from cornstarch_b200.parallel.cp import ContextParallelBatchSplitUtils as U
from tests.dist_utils import run_distributed

TEXT = (1 << 62) | 1


def causal_assignments(num_blocks):
    """LPT on a causal mask: [..., 2, 1, 0, 0, 1, 2, 3, 3, 2, 1, 0] (heaviest = last block goes to rank 0)."""
    base, tail = [0, 1, 2, 3], [3, 2, 1, 0]
    out = tail[:] if num_blocks >= 4 else tail[:num_blocks]
    toggle = True
    while len(out) < num_blocks:
        need = num_blocks - len(out)
        pre = base[:] if toggle else tail[:]
        if need < 4:
            pre = pre[-need:]
        out = pre + out
        toggle = not toggle
    return np.repeat(np.asarray(out), 128)


def full_assignments(num_blocks):
    pat = [0, 1, 2, 3]
    return np.repeat(np.asarray(pat * (num_blocks // 4) + pat[: num_blocks % 4]), 128)


def _assignment_vector(offsets, S):
    v = np.full(S, -1)
    for r, o in enumerate(offsets):
        v[np.asarray(o)] = r
    return v


@pytest.mark.parametrize("S", [512, 1024, 1152, 2048, 4096])
def test_makespan_causal_and_full_tables(S):
    bits = torch.full((2, S), TEXT, dtype=torch.int64)
    work = U.block_workloads(A.AttnMask.bitfield(bits), 2, S, "cpu")
    offs = U.makespan_min(work, S, 4)
    assert np.array_equal(_assignment_vector(offs, S), causal_assignments(S // 128))
    # one modality covering everything = full attention: equal workloads -> round robin
    bits = torch.full((2, S), 2, dtype=torch.int64)
    work = U.block_workloads(A.AttnMask.bitfield(bits), 2, S, "cpu")
    offs = U.makespan_min(work, S, 4)
    assert np.array_equal(_assignment_vector(offs, S), full_assignments(S // 128))


def test_uniform_zigzag_and_no_split():
    offs = U.uniform(1000, 4)
    assert [len(o) for o in offs] == [250] * 4 and offs[1][0] == 250
    z = U.zigzag(1024, 4)
    assert z[0][0] == 0 and z[0][-1] == 1023 and z[3][0] == 384 and len(set(np.concatenate(z))) == 1024
    # sequences shorter than 128 * sp are not split
    assert U.create_context_parallel_split(torch.full((1, 200), TEXT, dtype=torch.int64), None, "makespan_min") is None


def test_makespan_balances_multimodal_mask_better_than_zigzag():
    S = 4096
    bits = torch.full((1, S), TEXT | 2, dtype=torch.int64)
    bits[0, 100:1900] = 2  # a large bidirectional image block early in the sequence
    work = U.block_workloads(A.AttnMask.bitfield(bits), 1, S, "cpu")

    def makespan(offsets):
        return max(sum(work[b] for b in np.unique(np.asarray(o) // 128)) for o in offsets)

    assert makespan(U.makespan_min(work, S, 4)) <= makespan(U.zigzag(S, 4))


def _cp_attention_worker(rank, world):
    from cornstarch_b200.parallel.cp import ContextParallelState, context_parallel_attention

    torch.manual_seed(0)
    B, S, Hq, Hk, D = 2, 512, 4, 2, 32
    q = torch.randn(B, S, Hq, D)
    k = torch.randn(B, S, Hk, D)
    v = torch.randn(B, S, Hk, D)
    bits = torch.full((B, S), TEXT | 2, dtype=torch.int64)
    bits[:, 40:200] = 2
    bits[:, -7:] = 0
    full = A.AttnMask.bitfield(bits)
    ref_q, ref_k, ref_v = (t.clone().requires_grad_(True) for t in (q, k, v))
    ref, _ = A.attention_reference(ref_q, ref_k, ref_v, full)
    w = torch.randn_like(ref)
    (ref * w).sum().backward()
    group = dist.group.WORLD
    for mode in ("uniform", "zigzag", "makespan_min"):
        offsets = U.create_context_parallel_split(bits, group, mode)
        st = ContextParallelState(group, offsets, full, "cpu")
        lq, lk, lv = (t.index_select(1, st.mine).clone().requires_grad_(True) for t in (q, k, v))
        out = context_parallel_attention(lq, lk, lv, st)
        assert torch.allclose(out, ref.index_select(1, st.mine), atol=1e-5), mode
        (out * w.index_select(1, st.mine)).sum().backward()
        assert torch.allclose(lq.grad, ref_q.grad.index_select(1, st.mine), atol=1e-5), mode
        assert torch.allclose(lk.grad, ref_k.grad.index_select(1, st.mine), atol=1e-5), mode
        assert torch.allclose(lv.grad, ref_v.grad.index_select(1, st.mine), atol=1e-5), mode


    # the entry points at the reference's import paths ([B, heads, S, D] in, [B, S, heads, D] out)
    from cornstarch_b200.shardformer.layers.context_parallel_attention import context_parallel_flash_attention_forward
    from cornstarch_b200.shardformer.layers.context_parallel_bitfield_attention import context_parallel_bitfield_attention_forward

    offsets = U.create_context_parallel_split(bits, group, "makespan_min")
    mine = offsets[rank]
    out, _ = context_parallel_bitfield_attention_forward(
        None, *(t.index_select(1, mine).transpose(1, 2) for t in (q, k, v)), bits, offsets_per_rank=offsets, sp_group=group)
    assert torch.allclose(out, ref.index_select(1, mine), atol=1e-5)
    chunk = torch.tensor_split(torch.arange(S), world)[rank]
    full_ref, _ = A.attention_reference(q, k, v, A.AttnMask.full())
    out, _ = context_parallel_flash_attention_forward(
        None, *(t.index_select(1, chunk).transpose(1, 2) for t in (q, k, v)), sp_group=group)
    assert torch.allclose(out, full_ref.index_select(1, chunk), atol=1e-5)


def test_context_parallel_attention_matches_single_device():
    run_distributed(_cp_attention_worker, 2)


def _llama_sp_worker(rank, world, sp_mode, dist_mode):
    from cornstarch_b200.models.llama import DecoderConfig, DecoderForCausalLM
    from cornstarch_b200.shardformer.shard.shard_config import ShardConfig
    from cornstarch_b200.shardformer.shard.shardformer import ShardFormer

    torch.manual_seed(0)
    cfg = DecoderConfig(vocab_size=512, hidden_size=64, intermediate_size=128, num_hidden_layers=2, num_attention_heads=4,
                        num_key_value_heads=2, max_position_embeddings=1024)
    ref = DecoderForCausalLM(cfg)
    model = DecoderForCausalLM(cfg)
    model.load_state_dict(ref.state_dict())
    S = 512
    ids = torch.randint(0, 512, (2, S))
    bits = torch.full((2, S), TEXT | 2, dtype=torch.int64)
    bits[:, 30:150] = 2
    ref_out = ref(input_ids=ids, attention_mask=bits, labels=ids)
    ref_out.loss.backward()
    sc = ShardConfig(sequence_parallel_process_group=dist.group.WORLD, enable_sequence_parallelism=True,
                     sequence_parallelism_mode=sp_mode, context_parallel_distribution_mode=dist_mode,
                     enable_tensor_parallelism=False, extra_kwargs={"device": "cpu"})
    ShardFormer(sc).optimize(model)
    out = model(input_ids=ids, attention_mask=bits, labels=ids)
    out.loss.backward()
    if sp_mode == "all_to_all":
        assert abs(out.loss.item() - ref_out.loss.item()) < 1e-4
    if sp_mode == "ring_attn":
        # ranks hold token subsets: the mean over sp ranks of (sp * local_sum / total) is the global loss
        tot = out.loss.detach().clone()
        dist.all_reduce(tot)
        assert abs(tot.item() / world - ref_out.loss.item()) < 1e-4
    for (n, p), (_, rp) in zip(model.named_parameters(), ref.named_parameters()):
        g = p.grad.clone()
        dist.all_reduce(g)
        g /= world  # the plugin averages gradients over the dp x sp group
        assert torch.allclose(g, rp.grad, atol=2e-4, rtol=1e-3), (n, (g - rp.grad).abs().max())


@pytest.mark.parametrize("dist_mode", ["uniform", "zigzag", "makespan_min"])
def test_llama_ring_attn_matches_single_device(dist_mode):
    run_distributed(_llama_sp_worker, 2, "ring_attn", dist_mode)


def test_llama_ulysses_matches_single_device():
    run_distributed(_llama_sp_worker, 2, "all_to_all", "uniform")


def _family_sp_worker(rank, world, family, sp_mode):
    """Other decoder families through the same two sequence-parallel modes as Llama above."""
    from cornstarch_b200.shardformer.shard.shard_config import ShardConfig
    from cornstarch_b200.shardformer.shard.shardformer import ShardFormer
    from tests.test_policy_tp_numerics import _build

    torch.manual_seed(0)
    ref, _ = _build(family)
    torch.manual_seed(0)
    model, _ = _build(family)
    model.load_state_dict(ref.state_dict())
    S = 512
    ids = torch.randint(0, 128, (2, S), generator=torch.Generator().manual_seed(3))
    ref.config.max_position_embeddings = model.config.max_position_embeddings = S
    ref_out = ref(input_ids=ids, labels=ids)
    ref_out.loss.backward()
    sc = ShardConfig(sequence_parallel_process_group=dist.group.WORLD, enable_sequence_parallelism=True,
                     sequence_parallelism_mode=sp_mode, context_parallel_distribution_mode="uniform",
                     enable_tensor_parallelism=False, extra_kwargs={"device": "cpu"})
    ShardFormer(sc).optimize(model)
    out = model(input_ids=ids, labels=ids)
    out.loss.backward()
    tot = out.loss.detach().clone()
    dist.all_reduce(tot)
    assert abs(tot.item() / world - ref_out.loss.item()) < 2e-4 * max(1.0, abs(ref_out.loss.item())), (tot.item() / world, ref_out.loss.item())
    for (n, p), (_, rp) in zip(model.named_parameters(), ref.named_parameters()):
        if p.grad is None and rp.grad is None:
            continue
        g = p.grad.clone()
        dist.all_reduce(g)
        g /= world
        err, scale = (g - rp.grad).abs().max().item(), rp.grad.abs().max().item()
        assert err <= 2e-3 * scale + 1e-6, (family, sp_mode, n, err, scale)


def _family_group_worker(rank, world, sp_mode):
    families = ["mistral", "qwen2", "qwen3", "gemma", "gemma2", "gemma3", "phi3", "mixtral", "qwen3_moe", "llama4"]
    for family in families:
        _family_sp_worker(rank, world, family, sp_mode)
        dist.barrier()


@pytest.mark.parametrize("sp_mode", ["ring_attn", "all_to_all"])
def test_decoder_families_sequence_parallel(sp_mode):
    run_distributed(_family_group_worker, 2, sp_mode)


def _two_stage_ring_worker(rank, world):
    """Ring attention across a pipeline cut: the second stage gets this rank's tokens only and recovers the length of
    the whole sequence (and with it the token-to-rank map) from the micro-batch's ``input_ids``."""
    import copy

    from cornstarch_b200.pipeline_template import PipelineTemplate
    from cornstarch_b200.shardformer.shard.shard_config import ShardConfig
    from cornstarch_b200.shardformer.shard.shardformer import ShardFormer
    from tests.test_policy_tp_numerics import _build

    for family in ("llama", "llama4"):
        torch.manual_seed(0)
        whole, _ = _build(family)
        S = 512
        whole.config.max_position_embeddings = S
        ids = torch.randint(0, 128, (2, S), generator=torch.Generator().manual_seed(3))
        want = whole(input_ids=ids, labels=ids).loss
        stages = []
        for names in PipelineTemplate.even_split(whole, 2).modules_per_stage:
            m = copy.deepcopy(whole)
            m.hold_only(list(names))
            sc = ShardConfig(sequence_parallel_process_group=dist.group.WORLD, enable_sequence_parallelism=True,
                             sequence_parallelism_mode="ring_attn", context_parallel_distribution_mode="zigzag",
                             enable_tensor_parallelism=False, extra_kwargs={"device": "cpu"})
            ShardFormer(sc).optimize(m)
            stages.append(m)
        first = stages[0](input_ids=ids)
        assert first["hidden_states"].shape[1] == S // world
        passed = {k: v for k, v in first.items() if isinstance(v, torch.Tensor)}
        out = stages[1](input_ids=ids, labels=ids, **passed)
        tot = out.loss.detach().clone()
        dist.all_reduce(tot)
        assert abs(tot.item() / world - want.item()) < 2e-4 * max(1.0, abs(want.item())), (family, tot.item() / world, want.item())
        dist.barrier()


def test_ring_attention_across_a_pipeline_cut():
    run_distributed(_two_stage_ring_worker, 2)
