"""Point-to-point transport between pipeline stages (and across modality edges).

An object is any pytree of tensors and picklable leaves (``str``, tensor, ``[tensor]``, ``{"k": tensor}``
are what the reference protocol is tested with, tests/test_plugins/multimodal_parallel_plugin/
test_multimodal_1f1b.py:23-30 in the reference).  The reference sends, for EVERY message, a pickled
metadata size, the pickled metadata, then the tensors (cornstarch/plugin/multimodal_parallel_plugin/
multimodal_1f1b.py:66-397).  Shapes are static in training, so here the metadata travels only when it
changes: each message starts with a 2-element int64 header ``(metadata_bytes_or_0, 0)``; a zero means
"same structure and shapes as last time on this edge" and the receiver reuses its cached buffers' layout.
Tensors go through ``batch_isend_irecv`` (NCCL groups them into one launch; gloo runs them one by one).

Overlapped mode (``overlap_p2p=True``): once an edge's layout is known, sends are posted without waiting for them and
receives are posted BEFORE the compute they overlap with (``post_recv`` / ``wait_recv``), so a transfer runs on the
communication library's own stream while the compute stream keeps working; the compute stream only waits when it
needs the received tensors.  The reference's schedule is synchronous (every message is sent and waited for on the
spot, cornstarch/plugin/multimodal_parallel_plugin/multimodal_1f1b.py:339-397).  Un-grouped NCCL operations of one
communicator run on one stream in posting order, so messages that must not wait for one another must not share a
communicator: rank A posting "send forward, receive gradient" while its neighbour posts "send gradient, receive
forward" would wait on each other, and a receive posted early from the previous stage would hold back the send to the
next stage.  Every pipeline edge therefore gets TWO two-rank process groups, one per message direction
(:func:`make_edge_groups`); within one of them both ends post in micro-batch order, so every send meets its receive.
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


def _to_wire(meta: P2PMetadata) -> bytes:
    """Pickle with the tree spec as its JSON string (pickling a ``TreeSpec`` object itself is deprecated and warns)."""
    from torch.utils._pytree import treespec_dumps

    return pickle.dumps(P2PMetadata(treespec_dumps(meta.tree_spec), meta.tensor_metadata, meta.non_tensor_obj_idx, meta.non_tensor_objs))


def _from_wire(raw: bytes) -> P2PMetadata:
    from torch.utils._pytree import treespec_loads

    meta = pickle.loads(raw)
    meta.tree_spec = treespec_loads(meta.tree_spec)
    return meta


def make_edge_groups(next_ranks: list[int], warm_up: bool = True) -> dict:
    """Collective over ALL ranks of the default group.  ``next_ranks``: the ranks this rank sends forward messages to.
    Returns ``{(src, dst, "fwd" | "bwd"): two-rank process group}`` for the edges this rank is part of; ``(src, dst)``
    always names the edge in pipeline order (a "bwd" message of that edge travels from ``dst`` to ``src``).  Every rank
    creates every group in the same order; with ``warm_up`` the two members of a group run one tiny all-reduce in it,
    edge by edge in that same global order, so that communicators which are set up on first use exist before any
    receive is posted ahead of time (their set-up blocks the host until both members call)."""
    world, me = dist.get_world_size(), dist.get_rank()
    gathered = [None] * world
    dist.all_gather_object(gathered, [int(r) for r in next_ranks])
    edges = sorted({(src, dst) for src, nxt in enumerate(gathered) for dst in nxt})
    mine = {}
    dev = torch.device("cuda", torch.cuda.current_device()) if dist.get_backend() == "nccl" else torch.device("cpu")
    for src, dst in edges:
        for direction in ("fwd", "bwd"):
            g = dist.new_group([src, dst])
            if me in (src, dst):
                mine[(src, dst, direction)] = g
                if warm_up:
                    dist.all_reduce(torch.zeros(1, device=dev), group=g)
    return mine


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
                    raise RuntimeError(f"p2p edge {key}: message layout changed although shapes were declared static "
                                       "(build the schedule with assume_static_shapes=False for batches of varying shape)")
                prepared.append((dst, None, None, tensors))
                continue
            payload = None
            if not same:
                raw = _to_wire(meta)
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
                self._recv[(src, tag)] = _from_wire(bytes(buf.cpu().tolist()))
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
        return [self._assemble(self._recv[(src, tag)], ts) for (src, tag), ts in zip(recvs, rtensors)]

    # ------------------------------------------------------------------ overlapped (asynchronous) primitives
    def _group_for(self, tag: str, peer: int, sending: bool):
        """The process group of one message: the edge's own two-rank group when edge groups were made, else ``group``."""
        edge_groups = getattr(self, "edge_groups", None)
        if not edge_groups:
            return self.group
        me = dist.get_rank()
        # a forward message travels src -> dst of its edge, a backward message dst -> src
        src, dst = (me, peer) if (sending == (tag == "fwd")) else (peer, me)
        return edge_groups.get((src, dst, tag), self.group)

    def can_overlap(self, send_keys: list[tuple[int, str]], recv_keys: list[tuple[int, str]]) -> bool:
        """True once every listed edge has been negotiated (its layout is cached on both ends) and shapes are static."""
        return (self.assume_static and all(k in self._sent for k in send_keys) and all(k in self._recv for k in recv_keys))

    def isend(self, obj: Any, dst: int, tag: str) -> None:
        """Post the tensors of ``obj`` to ``dst`` without waiting; ``flush_sends`` (end of step) completes them."""
        meta, tensors = create_send_metadata(obj)
        if not _same_layout(self._sent.get((dst, tag)), meta):
            raise RuntimeError(f"p2p edge {(dst, tag)}: message layout changed although shapes were declared static")
        dev, g = self._dev(), self._group_for(tag, dst, True)
        pending = self.__dict__.setdefault("_pending_sends", [])
        for t in tensors:
            c = t.detach().contiguous().to(dev)
            pending.append((dist.isend(c, dst, group=g), c))

    def flush_sends(self) -> None:
        for req, _t in self.__dict__.get("_pending_sends", []):
            req.wait()
        self.__dict__["_pending_sends"] = []

    def post_recv(self, src: int, tag: str):
        """Post the receives of the next message on edge ``(src, tag)`` into fresh buffers; returns a handle for
        :meth:`wait_recv`.  Call it before the compute that the transfer should overlap with."""
        meta = self._recv[(src, tag)]
        dev, g = self._dev(), self._group_for(tag, src, False)
        ts = [torch.empty(m.shape, dtype=m.dtype, device=dev) for m in meta.tensor_metadata]
        reqs = [dist.irecv(t, src, group=g) for t in ts]
        return (src, tag, ts, reqs)

    def wait_recv(self, handle) -> Any:
        src, tag, ts, reqs = handle
        for r in reqs:
            r.wait()
        return self._assemble(self._recv[(src, tag)], ts)

    @staticmethod
    def _assemble(meta: P2PMetadata, ts: list[torch.Tensor]) -> Any:
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
        return tree_unflatten(leaves, meta.tree_spec)

    def send(self, obj: Any, dst: int, tag: str = "fwd") -> None:
        self.communicate([(obj, dst, tag)], [])

    def recv(self, src: int, tag: str = "fwd") -> Any:
        return self.communicate([], [(src, tag)])[0]


class MultimodalPipelineP2PCommunication(PipelineP2PCommunication):
    """Stage-manager aware wrappers: fan-in from several previous ranks, fan-out to several next ranks.

    Forward sends are broadcasts of one object to every next rank; backward sends carry one object per
    previous rank (the LLM's first stage returns a separate gradient to every encoder).
    """

    def __init__(self, stage_manager, overlap_p2p: bool = False, device=None, group=None, assume_static: bool = False,
                 edge_groups: dict | None = None):
        super().__init__(device, group, assume_static)
        self.stage_manager = stage_manager
        self.overlap_p2p = overlap_p2p
        self.edge_groups = edge_groups or {}  # {(src, dst, "fwd" | "bwd"): two-rank group}, see make_edge_groups

    def overlap_ready(self) -> bool:
        """Overlapped mode can run: it was asked for, and every edge of this rank has been negotiated by an earlier step."""
        if not self.overlap_p2p:
            return False
        if dist.get_backend(self.group) == "nccl" and not self.edge_groups:
            return False  # one communicator for everything could deadlock or serialise (see the module docstring)
        sm = self.stage_manager
        prv = [] if sm.is_first_stage(check_only_in_modal=False) else sm.get_prev_ranks()
        nxt = [] if sm.is_last_stage(check_only_in_modal=False) else sm.get_next_ranks()
        return self.can_overlap([(r, "fwd") for r in nxt] + [(r, "bwd") for r in prv],
                                [(r, "fwd") for r in prv] + [(r, "bwd") for r in nxt])

    def post_recv_forward(self):
        return [self.post_recv(r, "fwd") for r in self.stage_manager.get_prev_ranks()]

    def post_recv_backward(self):
        return [self.post_recv(r, "bwd") for r in self.stage_manager.get_next_ranks()]

    def wait_all(self, handles) -> list[Any]:
        return [self.wait_recv(h) for h in handles]

    def isend_forward(self, output_object: Any, is_broadcast: bool = True) -> None:
        for o, r, tag in self._fwd_sends(output_object, self.stage_manager.get_next_ranks(), is_broadcast):
            self.isend(o, r, tag)

    def isend_backward(self, input_object: Any, is_broadcast: bool = False) -> None:
        for o, r, tag in self._bwd_sends(input_object, self.stage_manager.get_prev_ranks(), is_broadcast):
            self.isend(o, r, tag)

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
