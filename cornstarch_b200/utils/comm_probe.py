"""Multi-GPU micro-benchmarks of the fused compute+collective kernels against the NCCL baseline.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 2 --master-addr 127.0.0.1 --master-port 29533 \
        -m cornstarch_b200.utils.comm_probe gemm_allreduce

For each shape it reports (device-timed with CUDA events, max over ranks): the fused GEMM + all-reduce
kernel, the baseline (same GEMM kernel followed by an NCCL all-reduce), and the roofline of the fused op:
the slower of FLOPs / measured bf16 GEMM peak and NVLink bytes / 770 GB/s (each rank pushes
(world-1)/world of the output as partials and the same amount again as final tiles).
"""

from __future__ import annotations

import argparse
import json
import os
import sys

import torch
import torch.distributed as dist

from ..ops.gemm import gemm
from .kernel_probe import peaks

NVLINK_BPS = 770e9


def timeit(fn, iters=10, warmup=3):
    for _ in range(warmup):
        fn()
    dist.barrier()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        fn()
    e1.record()
    torch.cuda.synchronize()
    t = torch.tensor([e0.elapsed_time(e1) / iters], device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t[0])


def gemm_allreduce(args):
    from ..parallel.symm import FusedTensorParallel

    ftp = FusedTensorParallel.get(dist.group.WORLD)
    world, rank = dist.get_world_size(), dist.get_rank()
    _, flops_peak, src = peaks()
    T, H, I, QKV = 8192, 4096, 14336, 6144
    shapes = [("o_proj fwd", T, H, H // world, 0), ("down_proj fwd", T, H, I // world, 0),
              ("qkv dX", T, H, QKV // world, 1), ("gate_up dX", T, H, 2 * I // world, 1)]
    for name, M, N, K, bmn in shapes:
        a = torch.randn(M, K, device="cuda").bfloat16()
        b = torch.randn((K, N) if bmn else (N, K), device="cuda").bfloat16()
        out = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
        for nred in args.reducers:
            ms_f = timeit(lambda: ftp.gemm_allreduce(a, b, False, bool(bmn), out=out))

            def base():
                gemm(a, b, False, bool(bmn), out=out)
                dist.all_reduce(out)

            ms_b = timeit(base)
            ms_g = timeit(lambda: gemm(a, b, False, bool(bmn), out=out))
            flops = 2.0 * M * N * K
            link_bytes = 2 * (world - 1) / world * M * N * 2
            roof_ms = max(flops / flops_peak, link_bytes / NVLINK_BPS) * 1e3
            if rank == 0:
                print(json.dumps({"op": name, "M": M, "N": N, "K": K, "world": world, "reducer_ctas": nred,
                                  "fused_ms": round(ms_f, 4), "gemm_then_nccl_ms": round(ms_b, 4), "gemm_only_ms": round(ms_g, 4),
                                  "roofline_ms": round(roof_ms, 4), f"frac_of_roofline_{src}": round(roof_ms / ms_f, 3),
                                  "speedup_vs_nccl": round(ms_b / ms_f, 3)}), flush=True)
    from ..ops import _native as nat

    nat.check_status()


def sp_linear(args):
    """Token-sharded tensor parallelism: all-gather -> GEMM (column-parallel forward) and GEMM -> reduce-scatter
    (row-parallel forward) as one kernel each, against NCCL all-gather / reduce-scatter around the same GEMM kernel.
    Roofline: the slower of FLOPs / measured GEMM peak and (world-1)/world of the gathered (or scattered) matrix / 770 GB/s."""
    from ..parallel.symm import FusedTensorParallel

    ftp = FusedTensorParallel.get(dist.group.WORLD)
    world, rank = dist.get_world_size(), dist.get_rank()
    _, flops_peak, src = peaks()
    T, H, I, QKV = 8192, 4096, 14336, 6144
    for name, N, K in [("all-gather -> qkv", QKV // world, H), ("all-gather -> gate_up", 2 * I // world, H)]:
        shard = torch.randn(T // world, K, device="cuda").bfloat16()
        w = torch.randn(N, K, device="cuda").bfloat16()
        full = torch.empty(T, K, device="cuda", dtype=torch.bfloat16)
        ms_f = timeit(lambda: ftp.ag_gemm(shard, w))

        def base():
            dist.all_gather_into_tensor(full, shard)
            gemm(full, w)

        ms_b = timeit(base)
        ms_g = timeit(lambda: gemm(full, w))
        roof_ms = max(2.0 * T * N * K / flops_peak, (world - 1) / world * T * K * 2 / NVLINK_BPS) * 1e3
        if rank == 0:
            print(json.dumps({"op": name, "M": T, "N": N, "K": K, "world": world, "fused_ms": round(ms_f, 4),
                              "nccl_then_gemm_ms": round(ms_b, 4), "gemm_only_ms": round(ms_g, 4), "roofline_ms": round(roof_ms, 4),
                              f"frac_of_roofline_{src}": round(roof_ms / ms_f, 3), "speedup_vs_nccl": round(ms_b / ms_f, 3)}), flush=True)
    for name, N, K in [("o_proj -> reduce-scatter", H, H // world), ("down_proj -> reduce-scatter", H, I // world)]:
        a = torch.randn(T, K, device="cuda").bfloat16()
        w = torch.randn(N, K, device="cuda").bfloat16()
        part = torch.empty(T, N, device="cuda", dtype=torch.bfloat16)
        mine = torch.empty(T // world, N, device="cuda", dtype=torch.bfloat16)
        ms_f = timeit(lambda: ftp.gemm_reducescatter(a, w))

        def base():
            gemm(a, w, out=part)
            dist.reduce_scatter_tensor(mine, part)

        ms_b = timeit(base)
        ms_g = timeit(lambda: gemm(a, w, out=part))
        ms_ar = timeit(lambda: ftp.gemm_allreduce(a, w, False, False, out=part))
        roof_ms = max(2.0 * T * N * K / flops_peak, (world - 1) / world * T * N * 2 / NVLINK_BPS) * 1e3
        if rank == 0:
            print(json.dumps({"op": name, "M": T, "N": N, "K": K, "world": world, "fused_ms": round(ms_f, 4),
                              "gemm_then_nccl_ms": round(ms_b, 4), "gemm_only_ms": round(ms_g, 4),
                              "fused_allreduce_ms": round(ms_ar, 4), "roofline_ms": round(roof_ms, 4),
                              f"frac_of_roofline_{src}": round(roof_ms / ms_f, 3), "speedup_vs_nccl": round(ms_b / ms_f, 3)}), flush=True)
    from ..ops import _native as nat

    nat.check_status()


def cp_attention(args):
    """Context-parallel attention forward + backward: K/V streamed from the peers inside the kernels against
    NCCL all-gather / reduce-scatter around the local kernels.  Llama-8B heads, ``--seq`` tokens per rank."""
    from ..ops import attention as A
    from ..parallel import cp as CP

    world, rank = dist.get_world_size(), dist.get_rank()
    _, flops_peak, src = peaks()
    B, Hq, Hk, D = 1, 32, 8, 128
    S = args.seq * world
    g = torch.Generator().manual_seed(0)
    full = A.AttnMask.causal()
    offs = CP.ContextParallelBatchSplitUtils.create_context_parallel_split(None, dist.group.WORLD, "zigzag", seq_len=S, batch=B, device="cuda")
    state = CP.ContextParallelState(dist.group.WORLD, offs, full, "cuda")
    n = state.mine.numel()
    q = torch.randn(B, n, Hq, D, generator=g).cuda().bfloat16().requires_grad_()
    k = torch.randn(B, n, Hk, D, generator=g).cuda().bfloat16().requires_grad_()
    v = torch.randn(B, n, Hk, D, generator=g).cuda().bfloat16().requires_grad_()
    do = torch.randn(B, n, Hq, D, generator=g).cuda().bfloat16()

    def run():
        q.grad = k.grad = v.grad = None
        CP.context_parallel_attention(q, k, v, state).backward(do)

    res = {}
    for fused in (True, False):
        CP.FUSED_CP_ENABLED = fused
        state.fused_mask = None
        res[fused] = timeit(run, iters=5, warmup=2)
    # causal zigzag: every rank computes 1/world of the S x S / 2 score matrix; forward 4 S^2 H D / 2, backward 2.5x
    flops = 3.5 * 4.0 * S * S * Hq * D * 0.5 / world
    kv_bytes = (world - 1) * n * Hk * D * 2 * 2          # K and V shards of the peers, read once per pass
    link_bytes = 2 * kv_bytes + kv_bytes                  # forward + backward reads, dK/dV tiles written to the owners
    roof_ms = max(flops / flops_peak, link_bytes / NVLINK_BPS) * 1e3
    if rank == 0:
        print(json.dumps({"op": "cp_attention fwd+bwd", "world": world, "tokens_per_rank": n, "S": S,
                          "fused_ms": round(res[True], 3), "nccl_gather_then_kernels_ms": round(res[False], 3),
                          "roofline_ms": round(roof_ms, 3), f"frac_of_roofline_{src}": round(roof_ms / res[True], 3),
                          "speedup_vs_nccl": round(res[False] / res[True], 3)}), flush=True)
    from ..ops import _native as nat

    nat.check_status()


def grad_reduce(args):
    """Flat-gradient all-reduce (mean) of ``--mb`` MiB of bf16: the peer-memory kernel against NCCL all_reduce + div."""
    from ..parallel.dp_fused import FusedGradReducer

    world, rank = dist.get_world_size(), dist.get_rank()
    red = FusedGradReducer.get(dist.group.WORLD)
    n = args.mb * (1 << 20) // 2
    buf = red.allocate(n)
    buf.normal_()
    plain = torch.randn(n, device="cuda").bfloat16()
    ms_f = timeit(lambda: red.reduce([buf]), iters=5, warmup=2)

    def base():
        dist.all_reduce(plain)
        plain.mul_(1.0 / world)

    ms_b = timeit(base, iters=5, warmup=2)
    link_bytes = 2 * (world - 1) / world * n * 2
    roof_ms = link_bytes / NVLINK_BPS * 1e3
    if rank == 0:
        print(json.dumps({"op": "grad all-reduce (mean)", "world": world, "MiB": args.mb, "fused_ms": round(ms_f, 3),
                          "nccl_allreduce_then_scale_ms": round(ms_b, 3), "roofline_ms": round(roof_ms, 3),
                          "frac_of_roofline": round(roof_ms / ms_f, 3), "bus_GBps": round(link_bytes / ms_f / 1e6, 1),
                          "speedup_vs_nccl": round(ms_b / ms_f, 3)}), flush=True)
    from ..ops import _native as nat

    nat.check_status()


def moe_exchange(args):
    """MoE token dispatch: ``--seq`` (token, expert) rows of 4096 bf16 per rank, gathered through a sorted index and sent
    to the expert owners in equal shares.  The peer-memory push kernel (gather fused into the stores, counters instead
    of a collective) against an index gather followed by NCCL ``all_to_all_single``."""
    from ..parallel.ep import all_to_all_uneven
    from ..parallel.ep_fused import FusedExpertExchange

    world, rank = dist.get_world_size(), dist.get_rank()
    rows, H = args.seq, 4096
    per = rows // world
    rows = per * world
    x = torch.randn(rows, H, device="cuda").bfloat16()
    index = torch.randperm(rows, device="cuda")
    counts = [[per] * world for _ in range(world)]
    ex = FusedExpertExchange.get(dist.group.WORLD)
    ex.ensure(rows, H)
    got = ex.exchange(x, index, counts)
    want = all_to_all_uneven(x[index], [per] * world, [per] * world, dist.group.WORLD)
    same = bool(torch.equal(got, want))
    ms_f = timeit(lambda: ex.exchange(x, index, counts), iters=10, warmup=3)
    ms_b = timeit(lambda: all_to_all_uneven(x[index], [per] * world, [per] * world, dist.group.WORLD), iters=10, warmup=3)
    link_bytes = (world - 1) * per * H * 2  # rows that leave this GPU (as many arrive)
    roof_ms = link_bytes / NVLINK_BPS * 1e3
    if rank == 0:
        print(json.dumps({"op": "moe dispatch (gather + all-to-all)", "world": world, "rows_per_rank": rows, "H": H,
                          "fused_ms": round(ms_f, 4), "gather_then_nccl_all_to_all_ms": round(ms_b, 4),
                          "roofline_ms": round(roof_ms, 4), "frac_of_roofline": round(roof_ms / ms_f, 3),
                          "speedup_vs_nccl": round(ms_b / ms_f, 3), "same_rows": same}), flush=True)
    from ..ops import _native as nat

    nat.check_status()


def moe_layer(args):
    """One Mixtral-8x7B-shape MoE block (hidden 4096, intermediate 14336, 8 experts, top 2), experts sharded over the
    ranks, forward + backward on ``--seq`` tokens per rank: exact dispatch (per-expert counts read on the host; NCCL
    all-to-all, and the peer-memory push kernel when there is more than one rank) against capacity mode (static shapes,
    no host read) at two capacity factors.  Device time between two events around the iterations, so launch gaps
    behind a host read are part of it; works on a single GPU too (all exchanges are local then)."""
    import time
    import warnings

    from ..models.moe import MixtralConfig, MixtralSparseMoeBlock
    from ..parallel import ep as EP

    world, rank = dist.get_world_size(), dist.get_rank()
    cfg = MixtralConfig(vocab_size=64, hidden_size=4096, intermediate_size=14336, num_hidden_layers=1, num_attention_heads=32,
                        num_key_value_heads=8, num_local_experts=8, num_experts_per_tok=2)
    torch.manual_seed(0)
    with torch.device("cuda"):
        block = MixtralSparseMoeBlock(cfg).bfloat16()
    EP.shard_experts(block, dist.group.WORLD)
    x = torch.randn(1, args.seq, 4096, device="cuda", generator=torch.Generator("cuda").manual_seed(rank)).bfloat16()
    gy = torch.randn_like(x)

    def step():
        xi = x.detach().requires_grad_()
        y, _ = block(xi)
        y.backward(gy)

    arms = [("exact, NCCL all-to-all", False, None)]
    if world > 1:
        arms.append(("exact, peer-memory push", True, None))
    arms += [("capacity 1.25", False, 1.25), ("capacity 2.0", False, 2.0)]
    rows = []
    for name, fused, cap in arms:
        EP.FUSED_EP_ENABLED = fused
        block.ep.capacity_factor = cap
        ms = timeit(step, iters=10, warmup=3)
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        for _ in range(10):
            step()
        host_ms = (time.perf_counter() - t0) * 100  # time the host needs to ENQUEUE one step (it blocks at host reads)
        torch.cuda.synchronize()
        dropped = int(block.ep.dropped_pairs) if cap is not None else 0
        with warnings.catch_warnings(record=True) as seen:  # PyTorch reports every call that makes the host wait
            warnings.simplefilter("always")
            torch.cuda.set_sync_debug_mode("warn")
            step()
            torch.cuda.set_sync_debug_mode("default")
        torch.cuda.synchronize()
        if rank == 0 and cap is not None:
            for w in seen[:4]:
                print(f"[{name}] host wait: {w.filename}:{w.lineno}", file=sys.stderr, flush=True)
        rows.append({"arm": name, "device_ms": round(ms, 3), "host_enqueue_ms": round(host_ms, 3),
                     "host_waits_per_step": len(seen),
                     "rows_into_local_experts": int(block.ep.last_recv_tokens), "dropped_pairs": dropped})
    if rank == 0:
        print(json.dumps({"op": "MoE block forward + backward", "world": world, "tokens_per_rank": args.seq,
                          "pairs_per_rank": args.seq * 2, "arms": rows}), flush=True)
    from ..ops import _native as nat

    nat.check_status()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("what", choices=["gemm_allreduce", "sp_linear", "cp_attention", "grad_reduce", "moe_exchange", "moe_layer"])
    ap.add_argument("--seq", type=int, default=8192, help="cp_attention: tokens per rank; moe_exchange: rows per rank")
    ap.add_argument("--mb", type=int, default=1024, help="grad_reduce: buffer size in MiB")
    ap.add_argument("--reducers", type=int, nargs="+", default=[16])
    args = ap.parse_args()
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    if "RANK" not in os.environ:  # plain ``python -m``: a group of one on this GPU
        os.environ.update(RANK="0", WORLD_SIZE="1")
        os.environ.setdefault("MASTER_PORT", "29541")
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    {"gemm_allreduce": gemm_allreduce, "sp_linear": sp_linear, "cp_attention": cp_attention, "grad_reduce": grad_reduce,
     "moe_exchange": moe_exchange, "moe_layer": moe_layer}[args.what](args)
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
