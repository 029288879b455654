"""Symmetric (peer-mapped) device memory and the fused tensor-parallel GEMM + all-reduce built on it.

``SymmetricMemory(nbytes, group)`` allocates the same amount of device memory on every rank of a
single-node group, exchanges CUDA IPC handles through the group and maps every peer's buffer, so a
kernel on any rank can load from / store to any rank's buffer over NVLink (``csrc/symm.cu``).

``FusedTensorParallel`` runs ``csb_gemm_allreduce_bf16``, a two-shot all-reduce folded into the GEMM
epilogue: output tile rows are owned by ranks in contiguous ranges and every rank computes the ranges in
rotated order, its own last.  A tile of a foreign range is pushed as a bf16 partial into the owner's
inbox (posted NVLink stores); a tile of the own range adds the partials that the peers pushed earlier,
stores the sum locally and pushes it into every peer's final buffer.  All 148 SMs keep doing MMA work,
transfers overlap the math tile by tile, and no rank ever waits on a remote load.  This is the row-parallel forward (o_proj / down_proj / fc2) and the column-parallel backward
(dX of q|k|v, gate|up, fc1) of Megatron-1D tensor parallelism, which the reference runs as a cuBLAS GEMM
followed by a blocking NCCL all-reduce (ColossalAI ``Linear1D_Row`` / ``Linear1D_Col``,
cornstarch/shardformer/policies/llama.py:192-249).
"""

from __future__ import annotations

import ctypes as C

import torch
import torch.distributed as dist

from ..ops import _native as nat

vp, i32, i64 = C.c_void_p, C.c_int, C.c_long
nat.declare("csb_symm_alloc", [i64, C.POINTER(vp)])
nat.declare("csb_symm_free", [vp])
nat.declare("csb_ipc_export", [vp, vp])
nat.declare("csb_ipc_import", [vp, C.POINTER(vp)])
nat.declare("csb_ipc_close", [vp])
nat.declare("csb_ipc_handle_size", [])
nat.declare(
    "csb_gemm_allreduce_bf16",
    [vp, vp, vp, i32, i32, i32, i32, i32, i32, i32, i32, i32, i32, vp, vp, vp, vp, i64, i32, i32, vp, vp],
)
nat.declare("csb_ar_layout", [i32, i32, i32, i32, i32, vp, vp, vp])
nat.declare(
    "csb_gemm_reducescatter_bf16",
    [vp, vp, vp, i32, i32, i32, i32, i32, i32, i32, i32, i32, i32, vp, vp, vp, vp, i64, i32, i32, vp, vp],
)
nat.declare("csb_ag_gemm_bf16", [vp, vp, vp, vp, i32, i32, i32, i32, i32, i32, i32, i32, vp, i32, vp, i32, i32, i32, vp, vp])


class _RawCudaBuffer:
    """Exposes a raw device pointer through ``__cuda_array_interface__`` so torch can wrap it without copying."""

    def __init__(self, ptr: int, nbytes: int):
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 3}


class SymmetricMemory:
    """One allocation per rank of ``group`` (single node), every rank holding pointers to all of them."""

    def __init__(self, nbytes: int, group=None):
        self.group = group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self.nbytes = int(nbytes)
        lib = nat.lib()
        own = vp()
        nat.check(lib.csb_symm_alloc(self.nbytes, C.byref(own)), "csb_symm_alloc")
        self._own = own.value
        hsize = lib.csb_ipc_handle_size()
        buf = C.create_string_buffer(hsize)
        nat.check(lib.csb_ipc_export(self._own, C.cast(buf, vp)), "csb_ipc_export")
        handles = [None] * self.world
        dist.all_gather_object(handles, bytes(buf.raw), group=group)
        self.ptrs: list[int] = []
        self._imported: list[int] = []
        for r, h in enumerate(handles):
            if r == self.rank:
                self.ptrs.append(self._own)
                continue
            hb = C.create_string_buffer(h, hsize)
            out = vp()
            nat.check(lib.csb_ipc_import(C.cast(hb, vp), C.byref(out)), "csb_ipc_import")
            self.ptrs.append(out.value)
            self._imported.append(out.value)
        self.ptr_array = (vp * self.world)(*self.ptrs)
        dist.barrier(group)

    def local_tensor(self, dtype=torch.uint8, offset: int = 0, numel: int | None = None) -> torch.Tensor:
        """A torch view of this rank's own buffer."""
        raw = torch.as_tensor(_RawCudaBuffer(self._own + offset, self.nbytes - offset), device="cuda")
        t = raw.view(dtype)
        return t if numel is None else t[:numel]

    def offset_ptr_array(self, offset: int):
        return (vp * self.world)(*[p + offset for p in self.ptrs])

    def close(self):
        lib = nat.lib()
        torch.cuda.synchronize()
        dist.barrier(self.group)
        for p in self._imported:
            lib.csb_ipc_close(p)
        self._imported = []
        if self._own:
            lib.csb_symm_free(self._own)
            self._own = 0


class _ARContext:
    """Symmetric buffers of one output shape: inbox (one slot per source rank), final buffer, arrival counters."""

    ROWS = 512

    def __init__(self, group, M: int, N: int, tile_n: int):
        self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)
        self.M, self.N = M, N
        self.slot = M * N
        cnt_bytes = self.world * self.ROWS * 4
        self.off_final = self.world * self.slot * 2
        self.off_cnt_part = self.off_final + self.slot * 2
        self.off_cnt_final = self.off_cnt_part + cnt_bytes
        total = self.off_cnt_final + cnt_bytes
        self.mem = SymmetricMemory(total, group)
        self.inbox = self.mem.offset_ptr_array(0)
        self.final = self.mem.offset_ptr_array(self.off_final)
        self.cnt_part = self.mem.offset_ptr_array(self.off_cnt_part)
        self.cnt_final = self.mem.offset_ptr_array(self.off_cnt_final)
        self.final_local = self.mem.local_tensor(torch.bfloat16, self.off_final, self.slot).view(M, N)
        rb, re, nn = C.c_int(), C.c_int(), C.c_int()
        nat.lib().csb_ar_layout(M, N, self.world, self.rank, tile_n, C.byref(rb), C.byref(re), C.byref(nn))
        self.row_begin, self.row_end, self.num_n = rb.value, re.value, nn.value
        self.calls = 0


class _AGContext:
    """Symmetric staging of one sharded operand shape ``[M / world, K]``: two staging buffers (a rank may already stage
    call i + 1 while a slower peer still copies call i), the "shard staged" counters the peers write, and the local
    counters of the pulling thread blocks."""

    def __init__(self, group, M: int, K: int):
        self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)
        # thread blocks of the GEMM launch that pull the peers' shards (each keeps 112 KB in flight); they hold their SMs
        # for the whole launch, so no more than the links need
        self.PULL_CTAS = 8 if self.world == 2 else 16
        self.M, self.K = M, K
        assert M % (128 * self.world) == 0, "the row count must split into whole 128-row tiles per rank"
        self.rows = M // self.world
        self.bytes = self.rows * K * 2
        self.mem = SymmetricMemory(2 * self.bytes + 256, group)
        self.stage = [self.mem.local_tensor(torch.bfloat16, i * self.bytes, self.rows * K).view(self.rows, K) for i in range(2)]
        self.shards = [self.mem.offset_ptr_array(i * self.bytes) for i in range(2)]
        flag_off = 2 * self.bytes
        self.flags = self.mem.local_tensor(torch.int32, flag_off, 64)
        self.flags.zero_()
        self.flag_ptrs = torch.tensor([p + flag_off for p in self.mem.ptrs], dtype=torch.int64, device="cuda")
        self.pulled = torch.zeros(64, dtype=torch.int32, device="cuda")
        self.calls = 0
        torch.cuda.synchronize()
        dist.barrier(group)


class FusedTensorParallel:
    """GEMM + all-reduce through peer memory for one tensor-parallel group (world size 2..8, one node)."""

    _by_group: dict = {}

    @classmethod
    def get(cls, group) -> "FusedTensorParallel | None":
        """Cached instance for ``group``; ``None`` when the fused path does not apply (CPU, gloo, world 1 or > 8)."""
        if group is None or not torch.cuda.is_available() or dist.get_backend(group) != "nccl":
            return None
        ws = dist.get_world_size(group)
        if ws < 2 or ws > 8:
            return None
        key = id(group)
        if key not in cls._by_group:
            cls._by_group[key] = cls(group)
        return cls._by_group[key]

    def __init__(self, group):
        self.group = group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self.contexts: dict[tuple[int, int, int], _ARContext] = {}

    def gemm_allreduce(self, a: torch.Tensor, b: torch.Tensor, a_mn_major=False, b_mn_major=False,
                       out: torch.Tensor | None = None, tile_n: int = 0) -> torch.Tensor:
        """``out = sum_ranks op(a) @ op(b).T`` (bf16); every rank of the group must make the same call."""
        if a_mn_major:
            K, M = a.shape
        else:
            M, K = a.shape
        N = b.shape[1] if b_mn_major else b.shape[0]
        key = (M, N, tile_n)
        ctx = self.contexts.get(key)
        if ctx is None:
            ctx = self.contexts[key] = _ARContext(self.group, M, N, tile_n)  # collective: all ranks see the same shapes
        if out is None:
            out = torch.empty((M, N), dtype=torch.bfloat16, device=a.device)
        st = nat.status_word(a.device)
        nat.check(
            nat.lib().csb_gemm_allreduce_bf16(
                a.data_ptr(), b.data_ptr(), out.data_ptr(), M, N, K, a.stride(0), b.stride(0), out.stride(0),
                int(a_mn_major), int(b_mn_major), self.world, self.rank, C.cast(ctx.inbox, vp), C.cast(ctx.final, vp),
                C.cast(ctx.cnt_part, vp), C.cast(ctx.cnt_final, vp), ctx.slot, ctx.calls * ctx.num_n, tile_n,
                st.data_ptr(), nat.stream()),
            "csb_gemm_allreduce_bf16",
        )
        ctx.calls += 1
        # rows owned by the other ranks arrived in the final buffer: move them next to the rows computed here
        if ctx.row_begin > 0:
            out[: ctx.row_begin].copy_(ctx.final_local[: ctx.row_begin])
        if ctx.row_end < M:
            out[ctx.row_end :].copy_(ctx.final_local[ctx.row_end :])
        return out

    # ------------------------------------------------------------------ sequence-sharded activations (Megatron "SP")
    def shard_rows(self, M: int) -> tuple[int, int]:
        """Rows ``[begin, end)`` of an ``M``-row activation that this rank owns (whole 128-row tiles, contiguous ranges)."""
        tiles = (M + 127) // 128
        b = (self.rank * tiles) // self.world * 128
        e = min(M, ((self.rank + 1) * tiles) // self.world * 128)
        return b, e

    def gemm_reducescatter(self, a: torch.Tensor, b: torch.Tensor, a_mn_major=False, b_mn_major=False, tile_n: int = 0) -> torch.Tensor:
        """``sum_ranks op(a) @ op(b).T`` restricted to the rows this rank owns: GEMM with the reduce-scatter in its
        epilogue (a partial tile of a foreign row range is pushed to its owner, the owner adds what arrived to its own
        accumulator; nothing is sent back).  Returns ``[rows owned, N]``."""
        if a_mn_major:
            K, M = a.shape
        else:
            M, K = a.shape
        N = b.shape[1] if b_mn_major else b.shape[0]
        key = ("rs", M, N, tile_n)
        pair = self.contexts.get(key)
        if pair is None:
            # two inbox sets: a rank that runs ahead pushes the partials of call i + 1 while a peer still reads call i
            pair = self.contexts[key] = [_ARContext(self.group, M, N, tile_n), _ARContext(self.group, M, N, tile_n), 0]
        ctx = pair[pair[2] & 1]
        pair[2] += 1
        out = torch.empty((ctx.row_end - ctx.row_begin, N), dtype=torch.bfloat16, device=a.device)
        st = nat.status_word(a.device)
        nat.check(
            nat.lib().csb_gemm_reducescatter_bf16(
                a.data_ptr(), b.data_ptr(), out.data_ptr(), M, N, K, a.stride(0), b.stride(0), out.stride(0),
                int(a_mn_major), int(b_mn_major), self.world, self.rank, C.cast(ctx.inbox, vp), C.cast(ctx.final, vp),
                C.cast(ctx.cnt_part, vp), C.cast(ctx.cnt_final, vp), ctx.slot, ctx.calls * ctx.num_n, tile_n,
                st.data_ptr(), nat.stream()),
            "csb_gemm_reducescatter_bf16",
        )
        ctx.calls += 1
        return out

    def ag_gemm(self, a_shard: torch.Tensor, b: torch.Tensor, b_mn_major=False, tile_n: int = 0):
        """``all_gather(a_shard) @ op(b).T``: the first thread blocks of the GEMM copy the peers' shards once into a local
        full-size operand while the other blocks already compute the tiles of the own rows.  ``a_shard``: this rank's
        ``[M / world, K]`` rows.  Returns ``(out [M, N], a_full [M, K])``; ``a_full`` is a fresh tensor the caller may keep."""
        from . import cp_fused  # noqa: F401  (declares csb_cp_signal)

        rows, K = a_shard.shape
        M = rows * self.world
        N = b.shape[1] if b_mn_major else b.shape[0]
        key = ("ag", M, K)
        ctx = self.contexts.get(key)
        if ctx is None:
            ctx = self.contexts[key] = _AGContext(self.group, M, K)
        cur = ctx.calls & 1
        ctx.calls += 1
        ctx.stage[cur].copy_(a_shard)
        lib, st = nat.lib(), nat.stream()
        nat.check(lib.csb_cp_signal(ctx.flag_ptrs.data_ptr(), self.world, self.rank, ctx.calls, st), "csb_cp_signal")
        a_full = torch.empty((M, K), dtype=torch.bfloat16, device=a_shard.device)
        a_full[self.rank * rows : (self.rank + 1) * rows].copy_(a_shard)  # the kernel reads these rows from the shard in place
        out = torch.empty((M, N), dtype=torch.bfloat16, device=a_shard.device)
        status = nat.status_word(a_shard.device)
        nat.check(
            lib.csb_ag_gemm_bf16(C.cast(ctx.shards[cur], vp), a_full.data_ptr(), b.data_ptr(), out.data_ptr(), M, N, K,
                                 b.stride(0), out.stride(0), int(b_mn_major), self.world, self.rank, ctx.flags.data_ptr(),
                                 ctx.calls, ctx.pulled.data_ptr(), ctx.PULL_CTAS * ctx.calls, ctx.PULL_CTAS, tile_n,
                                 status.data_ptr(), st),
            "csb_ag_gemm_bf16",
        )
        return out, a_full
