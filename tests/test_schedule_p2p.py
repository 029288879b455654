"""1F1B schedule over a modality DAG and the p2p transport, on gloo ranks.

* per-rank forward/backward ORDER for one encoder (1 stage) + LLM (3 stages): rank r runs (4 - r) forwards, then
  (B, F) x (M - 4 + r), then (4 - r) backwards; and for two encoders of 1 and 2 stages + LLM of 2 stages
  (the reference's tests/test_plugins/multimodal_parallel_plugin/test_multimodal_schedule_1f1b.py:272-364);
* numerics: loss and gradients equal the unsharded stack of linears;
* transport: str, tensor, [tensor], {"k": tensor} objects forward and backward, with metadata sent once.
"""

import pytest
import torch
import torch.distributed as dist
import torch.nn as nn

from tests.dist_utils import run_distributed


def _tpl(name, stages):
    from cornstarch_b200.pipeline_template import PipelineTemplate

    return PipelineTemplate(name, [[f"layers.{s}"] for s in range(stages)])


class ToyStage(nn.Module):
    """One linear per stage; the LLM's first stage adds up whatever the encoders sent."""

    def __init__(self, seed, is_last):
        super().__init__()
        torch.manual_seed(seed)
        self.lin = nn.Linear(8, 8)
        self.is_last = is_last

    def forward(self, x=None, hidden_states=None, **kw):
        if hidden_states is None:
            h = x
        elif isinstance(hidden_states, (list, tuple)):
            h = sum(hidden_states)
        else:
            h = hidden_states
        out = torch.tanh(self.lin(h))
        return out if self.is_last else {"hidden_states": out}


def _setup(world, rank, enc_stages, llm_stages):
    from cornstarch_b200.parallel.mesh import MultiModalProcessGroupMesh as Mesh
    from cornstarch_b200.parallel.schedule import MultimodalEncoderTrainingOneForwardOneBackwardSchedule as Sched
    from cornstarch_b200.parallel.stage_manager import MultiModalPipelineStageManager as SM

    encs = {_tpl(f"enc{i}", s): 1 for i, s in enumerate(enc_stages)}
    mesh = Mesh(encs, (_tpl("llm", llm_stages), 1, 1), world_size=world, rank=rank)
    sm = SM(mesh)
    return sm, Sched


def _order_worker(rank, world, enc_stages, llm_stages, M):
    sm, Sched = _setup(world, rank, enc_stages, llm_stages)
    sched = Sched(sm, num_microbatches=M, device=torch.device("cpu"), assume_static_shapes=True)
    sched.order_log = []
    last = sm.is_last_stage(check_only_in_modal=False)
    model = ToyStage(rank, last)
    batch = {"x": torch.randn(M * 2, 8, generator=torch.Generator().manual_seed(0))}
    out = sched.forward_backward_step(model, iter([batch]), lambda o, mb: o.mean(), None, return_loss=True)
    order = "".join(sched.order_log)
    if sm.is_encoder:
        w = sm.num_stages_in_modal + llm_stages - sm.stage_in_modal - 1
    else:
        w = llm_stages - sm.stage_in_modal - 1
    w = min(w, M)
    expected = "F" * w + "FB" * (M - w) + "B" * w
    assert order == expected, (rank, order, expected)
    assert (out["loss"] is not None) == last
    assert model.lin.weight.grad is not None


@pytest.mark.parametrize("enc_stages,llm_stages,M", [((1,), 3, 6), ((1, 2), 2, 4), ((1,), 3, 2)])
def test_1f1b_order(enc_stages, llm_stages, M):
    run_distributed(_order_worker, sum(enc_stages) + llm_stages, enc_stages, llm_stages, M)


def _numerics_worker(rank, world, M):
    enc_stages, llm_stages = (1, 1), 2
    sm, Sched = _setup(world, rank, enc_stages, llm_stages)
    sched = Sched(sm, num_microbatches=M, device=torch.device("cpu"))
    last = sm.is_last_stage(check_only_in_modal=False)
    model = ToyStage(rank, last)
    x = torch.randn(M * 3, 8, generator=torch.Generator().manual_seed(1))
    out = sched.forward_backward_step(model, iter([{"x": x}]), lambda o, mb: o.pow(2).mean(), None, return_loss=True)
    # the same computation in one process: enc0 (rank 0), enc1 (rank 1) -> sum -> llm stage 0 (rank 2) -> stage 1 (rank 3)
    stages = [ToyStage(r, r == 3) for r in range(4)]
    total = 0.0
    mb = x.shape[0] // M
    for i in range(M):
        xi = x[i * mb : (i + 1) * mb]
        h = stages[0](x=xi)["hidden_states"] + stages[1](x=xi)["hidden_states"]
        loss = stages[3](hidden_states=stages[2](hidden_states=h)["hidden_states"]).pow(2).mean() / M
        loss.backward()
        total += loss.item()
    assert torch.allclose(model.lin.weight.grad, stages[rank].lin.weight.grad, atol=1e-6), rank
    if last:
        assert abs(out["loss"].item() - total) < 1e-6


def test_1f1b_numerics_two_encoders():
    run_distributed(_numerics_worker, 4, 3)


def _p2p_worker(rank, world):
    from cornstarch_b200.parallel.p2p import PipelineP2PCommunication

    comm = PipelineP2PCommunication(torch.device("cpu"))
    objs = ["tensor", torch.arange(6.0).view(2, 3), [torch.ones(2), torch.zeros(3)], {"tensor": torch.full((2, 2), 7.0)},
            {"tensor": torch.full((2, 2), 8.0)}, {"a": torch.ones(1, requires_grad=True) * 2, "b": None, "c": 3}]
    nxt, prv = (rank + 1) % world, (rank - 1) % world
    for i, o in enumerate(objs):
        got = comm.communicate([(o, nxt, "fwd")], [(prv, "fwd")])[0]
        if isinstance(o, str):
            assert got == o
        elif isinstance(o, torch.Tensor):
            assert torch.equal(got, o)
        elif isinstance(o, list):
            assert all(torch.equal(a, b) for a, b in zip(got, o))
        else:
            assert got.keys() == o.keys()
            for k in o:
                if isinstance(o[k], torch.Tensor):
                    assert torch.equal(got[k], o[k].detach())
                else:
                    assert got[k] == o[k]
    assert got["a"].requires_grad  # the flag travels with the metadata
    # same layout twice in a row: the second message carried no metadata
    assert comm._sent[(nxt, "fwd")] is not None
    # backward direction uses a separate edge
    g = comm.communicate([({"tensor": torch.ones(2, 2) * rank}, prv, "bwd")], [(nxt, "bwd")])[0]
    assert torch.equal(g["tensor"], torch.ones(2, 2) * nxt)
    # static mode refuses a changed layout
    st = PipelineP2PCommunication(torch.device("cpu"), assume_static=True)
    st.communicate([(torch.ones(2), nxt, "fwd")], [(prv, "fwd")])
    st.communicate([(torch.ones(2) * 2, nxt, "fwd")], [(prv, "fwd")])
    with pytest.raises(RuntimeError):
        st.communicate([(torch.ones(3), nxt, "fwd")], [])


def test_p2p_protocol():
    run_distributed(_p2p_worker, 3)


def _overlap_worker(rank, world, enc_stages, llm_stages, M):
    """Overlapped P2P (asynchronous sends, receives posted ahead): the first step negotiates the message layouts with the
    synchronous protocol, the following steps run overlapped; order, loss and gradients equal the synchronous schedule."""
    from cornstarch_b200.parallel.p2p import make_edge_groups

    sm, Sched = _setup(world, rank, enc_stages, llm_stages)
    last = sm.is_last_stage(check_only_in_modal=False)
    edges = make_edge_groups([] if last else sm.get_next_ranks())
    n_edges = (0 if last else len(sm.get_next_ranks())) + (0 if sm.is_first_stage(check_only_in_modal=False) else len(sm.get_prev_ranks()))
    assert len(edges) == 2 * n_edges
    x = torch.randn(M * 2, 8, generator=torch.Generator().manual_seed(2))
    results = {}
    for mode in ("sync", "overlap"):
        sched = Sched(sm, num_microbatches=M, device=torch.device("cpu"), overlap_p2p=(mode == "overlap"), p2p_edge_groups=edges)
        model = ToyStage(rank, last)
        grads, losses, orders = [], [], []
        for step in range(3):
            model.zero_grad()
            sched.order_log = []
            out = sched.forward_backward_step(model, iter([{"x": x * (step + 1)}]), lambda o, mb: o.pow(2).mean(), None, return_loss=True)
            grads.append(model.lin.weight.grad.clone())
            losses.append(out["loss"].item() if last else None)
            orders.append("".join(sched.order_log))
        results[mode] = (grads, losses, orders)
        assert sched.overlapped_steps == (2 if mode == "overlap" else 0), (mode, sched.overlapped_steps)
        dist.barrier()
    for a, b in zip(results["sync"][0], results["overlap"][0]):
        assert torch.equal(a, b)
    assert results["sync"][1] == results["overlap"][1]
    assert results["sync"][2] == results["overlap"][2]


@pytest.mark.parametrize("enc_stages,llm_stages,M", [((1,), 3, 6), ((1, 2), 2, 4), ((1,), 2, 1)])
def test_overlapped_p2p_matches_synchronous(enc_stages, llm_stages, M):
    run_distributed(_overlap_worker, sum(enc_stages) + llm_stages, enc_stages, llm_stages, M)
