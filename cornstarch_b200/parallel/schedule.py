"""Modality-aware 1F1B pipeline schedule.

Stages form a DAG: encoder branches feed the LLM's first stage.  Each stage runs
``warmup`` forwards, then alternates one forward / one backward, then drains the remaining backwards,
with ``warmup = min(M, llm_stages - stage_in_modal - 1)`` for an LLM stage and
``min(M, my_stages + llm_stages - stage_in_modal - 1)`` for an encoder stage.  The LLM's first stage receives
one object per encoder and merges them key-wise into lists; its backward splits the input gradients
back, one object per encoder.  Same behaviour as the reference schedule
(cornstarch/plugin/multimodal_parallel_plugin/multimodal_1f1b.py:478-877; expected per-rank orders in
tests/test_plugins/multimodal_parallel_plugin/test_multimodal_schedule_1f1b.py:272-364 of the reference).
"""

from __future__ import annotations

from typing import Any, Callable, Iterable

import torch
from torch.utils._pytree import tree_flatten, tree_map

from ..utils.trace import nvtx_range

from .p2p import MultimodalPipelineP2PCommunication


def get_micro_batch(batch: Any, start: int, size: int) -> Any:
    """Slice dim 0 of every tensor of a pytree."""
    return tree_map(lambda x: x[start : start + size] if isinstance(x, torch.Tensor) and x.dim() > 0 else x, batch)


def get_batch_size(batch: Any) -> int:
    for leaf in tree_flatten(batch)[0]:
        if isinstance(leaf, torch.Tensor) and leaf.dim() > 0:
            return leaf.shape[0]
    raise ValueError("no tensor in the batch")


def _to_device(batch: Any, device) -> Any:
    return tree_map(lambda x: x.to(device, non_blocking=True) if isinstance(x, torch.Tensor) else x, batch)


class MultimodalEncoderTrainingOneForwardOneBackwardSchedule:
    def __init__(self, stage_manager, num_microbatches: int | None = None, microbatch_size: int | None = None,
                 device=None, p2p_group=None, assume_static_shapes: bool = True, overlap_p2p: bool = False,
                 p2p_edge_groups: dict | None = None):
        assert num_microbatches is not None or microbatch_size is not None, "Either num_microbatches or microbatch_size should be provided"
        self.stage_manager = stage_manager
        self.comm = MultimodalPipelineP2PCommunication(stage_manager, overlap_p2p=overlap_p2p, device=device, group=p2p_group,
                                                       assume_static=assume_static_shapes, edge_groups=p2p_edge_groups)
        self.overlapped_steps = 0  # steps that ran with asynchronous sends and pre-posted receives
        self.num_microbatches = num_microbatches
        self.microbatch_size = microbatch_size
        self.batch = None
        self.batch_size = None
        self.microbatch_offset = 0
        self.device = device
        self.order_log: list[str] | None = None  # tests set this to [] to record "F"/"B" per micro-batch

    # ------------------------------------------------------------------ data
    def load_batch(self, data_iter: Iterable, device=None) -> None:
        batch = next(data_iter)
        if device is not None:
            batch = _to_device(batch, device)
        self.batch = batch
        self.batch_size = get_batch_size(batch)
        self.microbatch_offset = 0
        if self.microbatch_size is None:
            assert self.batch_size % self.num_microbatches == 0, "Batch size should divided by the number of microbatches"
            self.microbatch_size = self.batch_size // self.num_microbatches
        elif self.num_microbatches is None or self.num_microbatches * self.microbatch_size != self.batch_size:
            assert self.batch_size % self.microbatch_size == 0, "Batch size should divided by the microbatch size"
            self.num_microbatches = self.batch_size // self.microbatch_size

    def load_micro_batch(self) -> Any:
        mb = get_micro_batch(self.batch, self.microbatch_offset, self.microbatch_size)
        self.microbatch_offset += self.microbatch_size
        return mb

    # ------------------------------------------------------------------ fan-in / fan-out
    @staticmethod
    def merge_inputs(objs: list[Any]) -> Any:
        """One object per previous rank -> a single input object (dicts merged key-wise into lists when several)."""
        objs = [o for o in objs if o is not None]
        if not objs:
            return None
        if len(objs) == 1:
            return objs[0]
        if all(isinstance(o, dict) for o in objs):
            keys = []
            for o in objs:
                for k in o:
                    if k not in keys:
                        keys.append(k)
            return {k: [o[k] for o in objs if k in o] for k in keys}
        return list(objs)

    @staticmethod
    def split_input_grads(input_obj: Any, n_prev: int) -> list[Any]:
        """Gradients of a merged input -> one object per previous rank."""
        def grad_of(x):
            return x.grad if isinstance(x, torch.Tensor) else None

        if n_prev == 1:
            return [tree_map(grad_of, input_obj)]
        if isinstance(input_obj, dict):
            outs = []
            for i in range(n_prev):
                outs.append({k: grad_of(v[i]) if isinstance(v, list) and i < len(v) else None for k, v in input_obj.items()})
            return outs
        return [tree_map(grad_of, o) for o in input_obj]

    def recv_forward(self) -> Any:
        sm = self.stage_manager
        if sm.is_first_stage(check_only_in_modal=False):
            return None
        objs = self.comm.recv_forward()
        inp = self.merge_inputs(objs)
        return inp

    def send_forward(self, output_obj: Any) -> None:
        if not self.stage_manager.is_last_stage(check_only_in_modal=False):
            self.comm.send_forward(output_obj)

    def recv_backward(self) -> Any:
        if self.stage_manager.is_last_stage(check_only_in_modal=False):
            return None
        grads = self.comm.recv_backward()
        # a stage that fans out to several identical consumers receives duplicated gradients: keep the first
        return grads[0]

    def send_backward(self, input_obj: Any) -> None:
        sm = self.stage_manager
        if sm.is_first_stage(check_only_in_modal=False) or input_obj is None:
            return
        self.comm.send_backward(self.split_input_grads(input_obj, len(sm.get_prev_ranks())))

    def send_forward_recv_backward(self, output_obj: Any) -> Any:
        if self.stage_manager.is_last_stage(check_only_in_modal=False):
            return None
        return self.comm.send_forward_recv_backward(output_obj)[0]

    def send_backward_recv_forward(self, input_obj: Any) -> Any:
        sm = self.stage_manager
        if sm.is_first_stage(check_only_in_modal=False):
            return None
        grads = self.split_input_grads(input_obj, len(sm.get_prev_ranks()))
        return self.merge_inputs(self.comm.send_backward_recv_forward(grads))

    # ------------------------------------------------------------------ compute
    def forward_step(self, model, input_obj: Any, criterion: Callable | None, accum_loss, outputs: list | None):
        micro_batch = self.load_micro_batch()
        if self.order_log is not None:
            self.order_log.append("F")
        kwargs = dict(micro_batch) if isinstance(micro_batch, dict) else {"inputs": micro_batch}
        if input_obj is not None:
            if isinstance(input_obj, dict):
                kwargs.update(input_obj)
            else:
                kwargs["hidden_states"] = input_obj
        with nvtx_range("pipeline/forward_microbatch"):
            output_obj = model(**kwargs)
        if self.stage_manager.is_last_stage(check_only_in_modal=False):
            loss = criterion(output_obj, micro_batch) / self.num_microbatches
            if accum_loss is not None:
                accum_loss.add_(loss.detach())
            if outputs is not None:
                outputs.append(_detach(output_obj))
            return loss
        return output_obj

    def backward_step(self, optimizer, input_obj: Any, output_obj: Any, output_obj_grad: Any) -> None:
        if self.order_log is not None:
            self.order_log.append("B")
        if input_obj is not None:
            for leaf in tree_flatten(input_obj)[0]:
                if isinstance(leaf, torch.Tensor) and leaf.requires_grad:
                    leaf.retain_grad()
        if output_obj_grad is None:
            with nvtx_range("pipeline/backward_microbatch"):
                _backward(optimizer, output_obj, None)
        else:
            outs, grads = [], []
            o_leaves = tree_flatten(output_obj)[0] if not isinstance(output_obj, dict) else None
            if isinstance(output_obj, dict):
                for k, g in (output_obj_grad.items() if isinstance(output_obj_grad, dict) else []):
                    o = output_obj.get(k)
                    if isinstance(o, torch.Tensor) and isinstance(g, torch.Tensor) and o.requires_grad:
                        outs.append(o)
                        grads.append(g)
            else:
                g_leaves = tree_flatten(output_obj_grad)[0]
                for o, g in zip(o_leaves, g_leaves):
                    if isinstance(o, torch.Tensor) and isinstance(g, torch.Tensor) and o.requires_grad:
                        outs.append(o)
                        grads.append(g)
            if outs:
                with nvtx_range("pipeline/backward_microbatch"):
                    _backward(optimizer, outs, grads)

    # ------------------------------------------------------------------ the schedule
    def num_warmup(self) -> int:
        sm = self.stage_manager
        if sm.is_encoder:
            llm = sm.pg_mesh.llm_template[0] if sm.pg_mesh.llm_template is not None else None
            w = sm.num_stages_in_modal + (llm.num_stages if llm is not None else 0) - sm.stage_in_modal - 1
        else:
            w = sm.num_stages_in_modal - sm.stage_in_modal - 1
        return min(self.num_microbatches, w)

    def _run_overlapped(self, model, criterion, optimizer, accum_loss, outputs) -> None:
        """The same 1F1B order with asynchronous P2P: the receive of the NEXT forward input (and of the next gradient) is
        posted before the current micro-batch is computed, sends are posted and not waited for, and the compute stream
        waits only where it consumes a received tensor.  Runs from the second step on (the first step negotiates the
        message layouts synchronously)."""
        sm, comm = self.stage_manager, self.comm
        first, last = sm.is_first_stage(check_only_in_modal=False), sm.is_last_stage(check_only_in_modal=False)
        M, warmup = self.num_microbatches, self.num_warmup()
        remaining = M - warmup
        n_prev = 0 if first else len(sm.get_prev_ranks())
        input_objs, output_objs = [], []
        fwd_posted = bwd_posted = 0
        fwd_h = bwd_h = None

        def post_fwd():
            nonlocal fwd_h, fwd_posted
            fwd_h = comm.post_recv_forward() if (not first and fwd_posted < M) else None
            fwd_posted += 1

        def post_bwd():
            nonlocal bwd_h, bwd_posted
            bwd_h = comm.post_recv_backward() if (not last and bwd_posted < M) else None
            bwd_posted += 1

        def take_fwd():
            h = fwd_h
            with nvtx_range("pipeline/wait_recv_forward"):
                inp = self.merge_inputs(comm.wait_all(h)) if h is not None else None
            post_fwd()  # the next input travels while this micro-batch is computed
            return inp

        def take_bwd():
            h = bwd_h
            with nvtx_range("pipeline/wait_recv_backward"):
                grad = comm.wait_all(h)[0] if h is not None else None
            post_bwd()
            return grad

        def backward_and_send(grad):
            inp0, out0 = input_objs.pop(0), output_objs.pop(0)
            self.backward_step(optimizer, inp0, out0, grad)
            if not first and inp0 is not None:
                comm.isend_backward(self.split_input_grads(inp0, n_prev))

        post_fwd()
        for _ in range(warmup):
            inp = take_fwd()
            out = self.forward_step(model, inp, criterion, accum_loss, outputs)
            if not last:
                comm.isend_forward(out)
            input_objs.append(inp)
            output_objs.append(out)
        post_bwd()
        for _ in range(remaining):
            inp = take_fwd()
            out = self.forward_step(model, inp, criterion, accum_loss, outputs)
            if not last:
                comm.isend_forward(out)
            input_objs.append(inp)
            output_objs.append(out)
            backward_and_send(take_bwd())
        for _ in range(warmup):
            backward_and_send(take_bwd())
        comm.flush_sends()
        assert not input_objs and not output_objs
        self.overlapped_steps += 1

    def run_forward_backward(self, model, data_iter, criterion, optimizer=None, return_loss=False, return_outputs=False) -> dict:
        sm = self.stage_manager
        self.load_batch(data_iter, self.device)
        last = sm.is_last_stage(check_only_in_modal=False)
        warmup = self.num_warmup()
        remaining = self.num_microbatches - warmup
        input_objs, output_objs = [], []
        accum_loss = None
        if return_loss and last:
            accum_loss = torch.zeros((), device=self.device if self.device is not None else "cpu")
        outputs = [] if return_outputs and last else None
        train = torch.is_grad_enabled() and optimizer is not False
        if train and self.comm.overlap_ready():
            self._run_overlapped(model, criterion, optimizer, accum_loss, outputs)
            return {"loss": accum_loss, "outputs": outputs}

        for _ in range(warmup):
            inp = self.recv_forward()
            out = self.forward_step(model, inp, criterion, accum_loss, outputs)
            self.send_forward(out)
            input_objs.append(inp)
            output_objs.append(out)
        inp = self.recv_forward() if remaining > 0 else None
        for i in range(remaining):
            last_iter = i == remaining - 1
            out = self.forward_step(model, inp, criterion, accum_loss, outputs)
            if not train:
                self.send_forward(out)
                if not last_iter:
                    inp = self.recv_forward()
                continue
            grad = self.send_forward_recv_backward(out)
            input_objs.append(inp)
            output_objs.append(out)
            inp0, out0 = input_objs.pop(0), output_objs.pop(0)
            self.backward_step(optimizer, inp0, out0, grad)
            if last_iter:
                self.send_backward(inp0)
                inp = None
            else:
                inp = self.send_backward_recv_forward(inp0)
        if train:
            for _ in range(warmup):
                inp0, out0 = input_objs.pop(0), output_objs.pop(0)
                grad = self.recv_backward()
                self.backward_step(optimizer, inp0, out0, grad)
                self.send_backward(inp0)
        assert not input_objs and not output_objs
        return {"loss": accum_loss, "outputs": outputs}

    def forward_backward_step(self, model, data_iter, criterion, optimizer=None, return_loss=False, return_outputs=False) -> dict:
        return self.run_forward_backward(model, data_iter, criterion, optimizer, return_loss, return_outputs)


def _detach(obj: Any) -> Any:
    return tree_map(lambda x: x.detach() if isinstance(x, torch.Tensor) else x, obj)


def _backward(optimizer, tensors, grads) -> None:
    if optimizer is not None and hasattr(optimizer, "backward") and grads is None:
        optimizer.backward(tensors)
    elif optimizer is not None and hasattr(optimizer, "backward_by_grad") and grads is not None:
        optimizer.backward_by_grad(tensors, grads)
    elif grads is None:
        tensors.backward()
    else:
        torch.autograd.backward(tensors, grads)
