"""Symmetric (peer-mapped) device memory and the fused tensor-parallel GEMM + all-reduce built on it.

``SymmetricMemory(nbytes, group)`` allocates the same amount of device memory on every rank of a
single-node group, exchanges CUDA IPC handles through the group and maps every peer's buffer, so a
kernel on any rank can load from / store to any rank's buffer over NVLink (``csrc/symm.cu``).

``FusedTensorParallel`` owns two staging buffers and two flag arrays per rank (alternated call by call)
and runs ``csb_gemm_allreduce_bf16``: the GEMM epilogue publishes this rank's partial tile and raises a
per-tile flag on every rank; reducer CTAs of the same launch add up the partial tiles of all ranks by
peer loads as soon as their flags are up, so the NVLink transfer overlaps the remaining MMA work tile
by tile.  This is the row-parallel forward (o_proj / down_proj / fc2) and the column-parallel backward
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
    [vp, vp, vp, i32, i32, i32, i32, i32, i32, i32, i32, i32, i32, vp, vp, i32, i32, i32, i32, vp, vp],
)


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


class FusedTensorParallel:
    """GEMM + all-reduce through peer memory for one tensor-parallel group (world size 2..8, one node)."""

    MAX_TILES = 16384
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

    def __init__(self, group, elems: int = 8192 * 4096):
        self.group = group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self.elems = 0
        self.mem: SymmetricMemory | None = None
        self.epoch = [0, 0]
        self.calls = 0
        self._alloc(elems)

    def _alloc(self, elems: int):
        if self.mem is not None:
            self.mem.close()
        self.elems = elems
        self.part_bytes = elems * 2
        self.flag_bytes = self.world * self.MAX_TILES * 4
        total = 2 * self.part_bytes + 2 * self.flag_bytes
        self.mem = SymmetricMemory(total, self.group)
        self.part_ptrs = [self.mem.offset_ptr_array(i * self.part_bytes) for i in range(2)]
        self.flag_ptrs = [self.mem.offset_ptr_array(2 * self.part_bytes + i * self.flag_bytes) for i in range(2)]
        self.epoch = [0, 0]

    def gemm_allreduce(self, a: torch.Tensor, b: torch.Tensor, a_mn_major=False, b_mn_major=False,
                       out: torch.Tensor | None = None, n_reducers: int = 16, tile_n: int = 0) -> torch.Tensor:
        """``out = sum_ranks op(a) @ op(b).T`` (bf16); every rank of the group must make the same call."""
        if a_mn_major:
            K, M = a.shape
        else:
            M, K = a.shape
        N = b.shape[1] if b_mn_major else b.shape[0]
        if M * N > self.elems:
            self._alloc(M * N)  # collective: every rank sees the same shapes
        if out is None:
            out = torch.empty((M, N), dtype=torch.bfloat16, device=a.device)
        which = self.calls & 1
        self.calls += 1
        self.epoch[which] += 1
        st = nat.status_word(a.device)
        nat.check(
            nat.lib().csb_gemm_allreduce_bf16(
                a.data_ptr(), b.data_ptr(), out.data_ptr(), M, N, K, a.stride(0), b.stride(0), out.stride(0),
                int(a_mn_major), int(b_mn_major), self.world, self.rank, C.cast(self.part_ptrs[which], vp),
                C.cast(self.flag_ptrs[which], vp), self.MAX_TILES, self.epoch[which], n_reducers, tile_n,
                st.data_ptr(), nat.stream()),
            "csb_gemm_allreduce_bf16",
        )
        return out
