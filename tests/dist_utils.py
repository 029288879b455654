"""Multi-process helpers for CPU tests: spawn ``world_size`` gloo ranks on 127.0.0.1 and run a function in each."""

import os
import socket
import sys
import traceback

import torch
import torch.distributed as dist
import torch.multiprocessing as mp


def free_port() -> int:
    with socket.socket(socket.AF_INET, socket.SOCK_STREAM) as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world_size, port, fn, args, errq):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ["RANK"] = str(rank)
    os.environ["WORLD_SIZE"] = str(world_size)
    torch.set_num_threads(1)
    code = 0
    try:
        dist.init_process_group("gloo", rank=rank, world_size=world_size)
        fn(rank, world_size, *args)
        dist.barrier()
    except BaseException:
        errq.put((rank, traceback.format_exc()))
        code = 1
    try:
        if code == 0 and dist.is_initialized():
            dist.destroy_process_group()
    except Exception:
        pass
    # Leave without running C++ static destructors: a gloo / store background thread that is still joinable when the
    # interpreter tears down aborts the process ("terminate called without an active exception", exit -6) although the
    # test body passed.  Everything the parent needs (the error queue) is already written.
    sys.stdout.flush()
    sys.stderr.flush()
    os._exit(code)


def run_distributed(fn, world_size: int, *args, timeout: int = 300):
    """Run ``fn(rank, world_size, *args)`` on ``world_size`` gloo ranks; re-raise the first failure with its traceback."""
    ctx = mp.get_context("spawn")
    errq = ctx.SimpleQueue()
    port = free_port()
    procs = [ctx.Process(target=_worker, args=(r, world_size, port, fn, args, errq)) for r in range(world_size)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout)
    failed = [p for p in procs if p.exitcode != 0]
    for p in procs:
        if p.is_alive():
            p.terminate()
    if failed or not errq.empty():
        msgs = []
        while not errq.empty():
            r, tb = errq.get()
            msgs.append(f"--- rank {r} ---\n{tb}")
        raise AssertionError("distributed test failed:\n" + "\n".join(msgs) + f"\nexit codes: {[p.exitcode for p in procs]}")


def _gpu_worker(rank, world_size, port, fn, args, errq):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world_size),
                      LOCAL_RANK=str(rank), NCCL_NVLS_ENABLE="0")
    code = 0
    try:
        torch.cuda.set_device(rank)
        dist.init_process_group("nccl", rank=rank, world_size=world_size, device_id=torch.device("cuda", rank))
        fn(rank, world_size, *args)
        torch.cuda.synchronize()
        dist.barrier()
        dist.destroy_process_group()
    except BaseException:
        errq.put((rank, traceback.format_exc()))
        code = 1
    sys.stdout.flush()
    sys.stderr.flush()
    os._exit(code)


def run_gpu_ranks(fn, world_size: int, *args, timeout: int = 300):
    """Run ``fn(rank, world_size, *args)`` as ``world_size`` child processes, one GPU each, NCCL for the plumbing
    (NVLS off: a rank that ends early must not leave multicast bindings behind).  Re-raises the first failure."""
    ctx = mp.get_context("spawn")
    errq = ctx.SimpleQueue()
    port = free_port()
    procs = [ctx.Process(target=_gpu_worker, args=(r, world_size, port, fn, args, errq)) for r in range(world_size)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout)
    for p in procs:
        if p.is_alive():
            p.terminate()
    failed = [p for p in procs if p.exitcode != 0]
    if failed or not errq.empty():
        msgs = []
        while not errq.empty():
            r, tb = errq.get()
            msgs.append(f"--- rank {r} ---\n{tb}")
        raise AssertionError("multi-GPU test failed:\n" + "\n".join(msgs) + f"\nexit codes: {[p.exitcode for p in procs]}")
