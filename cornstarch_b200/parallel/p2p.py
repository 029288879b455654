"""Point-to-point transport between pipeline stages (and across modality edges).

An object is any pytree of tensors and picklable leaves (``str``, tensor, ``[tensor]``, ``{"k": tensor}``
are what the reference protocol is tested with, tests/test_plugins/multimodal_parallel_plugin/
test_multimodal_1f1b.py:23-30 in the reference).  The reference sends, for EVERY message, a pickled
metadata size, the pickled metadata, then the tensors (cornstarch/plugin/multimodal_parallel_plugin/
multimodal_1f1b.py:66-397).  Shapes are static in training, so here the metadata travels only when it
changes: each message starts with a 2-element int64 header ``(metadata_bytes_or_0, 0)``; a zero means
"same structure and shapes as last time on this edge" and the receiver reuses its cached buffers' layout.
Tensors go through ``batch_isend_irecv`` (NCCL groups them into one launch; gloo runs them one by one).
"""

from __future__ import annotations

import pickle
from dataclasses import dataclass
from typing import Any

import torch
import torch.distributed as dist
from torch.utils._pytree import tree_flatten, tree_unflatten


@dataclass
class TensorMetadata:
    shape: tuple
    dtype: torch.dtype
    requires_grad: bool


@dataclass
class P2PMetadata:
    tree_spec: Any
    tensor_metadata: list
    non_tensor_obj_idx: list
    non_tensor_objs: list


def create_send_metadata(obj: Any) -> tuple[P2PMetadata, list[torch.Tensor]]:
    leaves, spec = tree_flatten(obj)
    tensors, tmeta, nt_idx, nt_objs = [], [], [], []
    for i, leaf in enumerate(leaves):
        if isinstance(leaf, torch.Tensor):
            tensors.append(leaf)
            tmeta.append(TensorMetadata(tuple(leaf.shape), leaf.dtype, leaf.requires_grad))
        else:
            nt_idx.append(i)
            nt_objs.append(leaf)
    return P2PMetadata(spec, tmeta, nt_idx, nt_objs), tensors


def _same_layout(a: P2PMetadata | None, b: P2PMetadata) -> bool:
    if a is None:
        return False
    return (a.tree_spec == b.tree_spec and a.non_tensor_obj_idx == b.non_tensor_obj_idx
            and a.non_tensor_objs == b.non_tensor_objs
            and [(m.shape, m.dtype) for m in a.tensor_metadata] == [(m.shape, m.dtype) for m in b.tensor_metadata])


class PipelineP2PCommunication:
    """Send/receive pytrees to/from explicit global ranks.

    Every exchange runs in three grouped phases (headers, changed metadata, tensors), each phase being one
    ``batch_isend_irecv`` that contains BOTH directions, so a stage that sends while its neighbour also
    sends cannot deadlock on NCCL (grouped calls) nor on gloo (asynchronous requests).
    """

    def __init__(self, device: torch.device | None = None, group=None, assume_static: bool = False):
        self.group = group
        self.device = device
        # with static shapes the header phase (and its host read) is skipped after the first message of an edge
        self.assume_static = assume_static
        self._sent: dict[tuple[int, str], P2PMetadata] = {}
        self._recv: dict[tuple[int, str], P2PMetadata] = {}

    def _dev(self):
        if self.device is not None:
            return self.device
        if dist.get_backend(self.group) == "nccl":
            return torch.device("cuda", torch.cuda.current_device())
        return torch.device("cpu")

    @staticmethod
    def _run(ops):
        if ops:
            for req in dist.batch_isend_irecv(ops):
                req.wait()

    def communicate(self, sends: list[tuple[Any, int, str]], recvs: list[tuple[int, str]]) -> list[Any]:
        """``sends``: ``(object, dst rank, tag)``; ``recvs``: ``(src rank, tag)``.  Returns the received objects in order."""
        dev = self._dev()
        g = self.group
        # phase 1: headers (skipped on edges already negotiated when shapes are declared static)
        prepared = []
        ops = []
        for obj, dst, tag in sends:
            meta, tensors = create_send_metadata(obj)
            key = (dst, tag)
            same = _same_layout(self._sent.get(key), meta)
            if self.assume_static and key in self._sent:
                if not same:
                    raise RuntimeError(f"p2p edge {key}: message layout changed although shapes were declared static")
                prepared.append((dst, None, None, tensors))
                continue
            payload = None
            if not same:
                raw = pickle.dumps(meta)
                payload = torch.frombuffer(bytearray(raw), dtype=torch.uint8).to(dev)
                self._sent[key] = meta
            header = torch.tensor([0 if payload is None else payload.numel(), 0], dtype=torch.int64, device=dev)
            prepared.append((dst, header, payload, tensors))
            ops.append(dist.P2POp(dist.isend, header, dst, g))
        rheaders = []
        for src, tag in recvs:
            if self.assume_static and (src, tag) in self._recv:
                rheaders.append(None)
                continue
            h = torch.zeros(2, dtype=torch.int64, device=dev)
            rheaders.append(h)
            ops.append(dist.P2POp(dist.irecv, h, src, g))
        self._run(ops)
        # phase 2: metadata that changed
        ops = []
        for dst, _h, payload, _t in prepared:
            if payload is not None:
                ops.append(dist.P2POp(dist.isend, payload, dst, g))
        rbufs = []
        for (src, _tag), h in zip(recvs, rheaders):
            n = int(h[0].item()) if h is not None else 0
            buf = torch.empty(n, dtype=torch.uint8, device=dev) if n > 0 else None
            rbufs.append(buf)
            if buf is not None:
                ops.append(dist.P2POp(dist.irecv, buf, src, g))
        self._run(ops)
        for (src, tag), buf in zip(recvs, rbufs):
            if buf is not None:
                self._recv[(src, tag)] = pickle.loads(buf.cpu().numpy().tobytes())
        # phase 3: tensors
        ops = []
        keep = []
        for dst, _h, _p, tensors in prepared:
            for t in tensors:
                c = t.detach().contiguous().to(dev)
                keep.append(c)
                ops.append(dist.P2POp(dist.isend, c, dst, g))
        rtensors = []
        for src, tag in recvs:
            meta = self._recv[(src, tag)]
            ts = [torch.empty(m.shape, dtype=m.dtype, device=dev) for m in meta.tensor_metadata]
            rtensors.append(ts)
            for t in ts:
                ops.append(dist.P2POp(dist.irecv, t, src, g))
        self._run(ops)
        out = []
        for (src, tag), ts in zip(recvs, rtensors):
            meta = self._recv[(src, tag)]
            for t, m in zip(ts, meta.tensor_metadata):
                if m.requires_grad and t.is_floating_point():
                    t.requires_grad_(True)
            nt = dict(zip(meta.non_tensor_obj_idx, meta.non_tensor_objs))
            leaves, ti = [], 0
            for i in range(len(meta.tensor_metadata) + len(meta.non_tensor_obj_idx)):
                if i in nt:
                    leaves.append(nt[i])
                else:
                    leaves.append(ts[ti])
                    ti += 1
            out.append(tree_unflatten(leaves, meta.tree_spec))
        return out

    def send(self, obj: Any, dst: int, tag: str = "fwd") -> None:
        self.communicate([(obj, dst, tag)], [])

    def recv(self, src: int, tag: str = "fwd") -> Any:
        return self.communicate([], [(src, tag)])[0]


class MultimodalPipelineP2PCommunication(PipelineP2PCommunication):
    """Stage-manager aware wrappers: fan-in from several previous ranks, fan-out to several next ranks.

    Forward sends are broadcasts of one object to every next rank; backward sends carry one object per
    previous rank (the LLM's first stage returns a separate gradient to every encoder).
    """

    def __init__(self, stage_manager, overlap_p2p: bool = False, device=None, group=None, assume_static: bool = False):
        super().__init__(device, group, assume_static)
        self.stage_manager = stage_manager
        self.overlap_p2p = overlap_p2p

    def _fwd_sends(self, obj, ranks, is_broadcast):
        if is_broadcast:
            return [(obj, r, "fwd") for r in ranks]
        assert len(obj) == len(ranks)
        return [(o, r, "fwd") for o, r in zip(obj, ranks)]

    def _bwd_sends(self, obj, ranks, is_broadcast):
        if is_broadcast:
            return [(obj, r, "bwd") for r in ranks]
        assert len(obj) == len(ranks)
        return [(o, r, "bwd") for o, r in zip(obj, ranks)]

    def recv_forward(self, prev_ranks: list[int] | None = None) -> list[Any]:
        prev_ranks = self.stage_manager.get_prev_ranks() if prev_ranks is None else prev_ranks
        return self.communicate([], [(r, "fwd") for r in prev_ranks])

    def recv_backward(self, next_ranks: list[int] | None = None) -> list[Any]:
        next_ranks = self.stage_manager.get_next_ranks() if next_ranks is None else next_ranks
        return self.communicate([], [(r, "bwd") for r in next_ranks])

    def send_forward(self, output_object: Any, next_ranks: list[int] | None = None, is_broadcast: bool = True) -> None:
        next_ranks = self.stage_manager.get_next_ranks() if next_ranks is None else next_ranks
        self.communicate(self._fwd_sends(output_object, next_ranks, is_broadcast), [])

    def send_backward(self, input_object: Any, prev_ranks: list[int] | None = None, is_broadcast: bool = False) -> None:
        prev_ranks = self.stage_manager.get_prev_ranks() if prev_ranks is None else prev_ranks
        self.communicate(self._bwd_sends(input_object, prev_ranks, is_broadcast), [])

    def send_forward_recv_backward(self, output_object: Any, is_broadcast: bool = True, send_first: bool | None = None) -> list[Any]:
        nxt = self.stage_manager.get_next_ranks()
        return self.communicate(self._fwd_sends(output_object, nxt, is_broadcast), [(r, "bwd") for r in nxt])

    def send_backward_recv_forward(self, input_object: Any, is_broadcast: bool = False, send_first: bool | None = None) -> list[Any]:
        prv = self.stage_manager.get_prev_ranks()
        return self.communicate(self._bwd_sends(input_object, prv, is_broadcast), [(r, "fwd") for r in prv])
