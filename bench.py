"""Headline benchmark: VLM training tokens/s on N B200s of one node (synthetic data, random-init weights).

Workload: SigLIP-so400m-shaped vision encoder (27 layers, hidden 1152, 729 image tokens from a 384x384
image) + 2-layer GELU MLP projector + Llama-3.1-8B-shaped LLM (32 layers, hidden 4096, 32/8 heads, FFN
14336, vocab 128256); every sample is 1 image + 7463 text tokens = 8192 tokens; 4 samples per GPU per
step (global batch 32 on 8 GPUs); bf16 compute, fp32 master weights and Adam moments; full
forward + backward + optimizer step inside the timed region.

    python bench.py --gpus 1 --steps 5 --warmup 3
    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 --master-port 29511 \
        bench.py --gpus 8 --steps 5 --warmup 3
    python bench.py --impl reference ...      # the unmodified reference, if it can be imported here

Rank 0 prints ONE JSON line.  ``value`` is the whole-job tokens/s with inputs resident on the device,
timed with CUDA events (max over ranks); ``e2e`` repeats the measurement through the public API with
the per-step host->device copy of the inputs from pinned memory and the device->host read of the loss.
"""

from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading

REPO = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, REPO)

SAMPLES_PER_GPU = 4
# the headline metric, spelled as the benchmark definition spells it (one value per GPU count of the 1/2/4/8 series)
METRIC = "VLM training tokens/sec/box (device-timed, max over ranks) at 1/2/4/8 B200"


# ------------------------------------------------------------------------------------------------ clocks
class ClockSampler:
    """Samples SM clocks and throttle reasons of one GPU with nvidia-smi while a region is timed."""

    Q = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index = index
        self.proc = None
        self.lines: list[str] = []

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "200"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._pump, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _pump(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons, power = [], [], set(), []
        for ln in self.lines:
            parts = [p.strip() for p in ln.split(",")]
            if len(parts) < 8:
                continue
            try:
                sm.append(float(parts[0]))
                mx.append(float(parts[1]))
                power.append(float(parts[2]))
            except ValueError:
                continue
            for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), parts[4:8]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        sm.sort()
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "power_w_max": max(power) if power else None, "samples": len(sm), "reasons": sorted(reasons)}


# ------------------------------------------------------------------------------------------------ reference arm
REF_CHAIN = ("cornstarch", "cornstarch.kernel.bitfield_attention", "cornstarch.kernel.attention",
             "cornstarch.models.multimodal_language_model", "cornstarch.plugin.multimodal_parallel_plugin")


def run_reference(args) -> None:
    """The unmodified reference from baseline/_ref through its own public API, or the `unavailable` line.

    The import chain of the reference is tried module by module and the first one that fails is reported.  The
    end-to-end training metric needs the model layer and the plugin (colossalai, peft, timm and transformers-4.5x
    internals, none of which is installed here), so that metric is `unavailable`; what the reference owns as GPU code -
    its Triton attention kernels - imports with torch + triton alone and is timed on this GPU next to this package's
    kernels (`reference_kernels`, rank 0 only), unmodified and through the reference's own `bitfield_attn_func`."""
    ref = os.path.join(REPO, "baseline", "_ref")
    rank0 = int(os.environ.get("RANK", "0")) == 0
    out = {"impl": "reference"}
    if not os.path.isdir(os.path.join(ref, "cornstarch")):
        out["unavailable"] = "baseline/_ref is empty (offline pip install of the reference was not possible)"
        if rank0:
            print(json.dumps(out))
        return
    sys.path.insert(0, ref)
    import importlib

    imported, first_fail = [], None
    for mod in REF_CHAIN:
        try:
            importlib.import_module(mod)
            imported.append(mod)
        except Exception as e:  # missing third-party packages / removed transformers internals
            first_fail = f"{mod}: {type(e).__name__}: {e}".replace("\n", " ")[:240]
            break
    out["imports_ok"] = imported
    out["unavailable"] = ("end-to-end training through the reference's MultimodalModel + MultimodalParallelPlugin cannot run here: "
                          + (f"first failing import {first_fail}" if first_fail else
                             "the modules import but the plugin needs colossalai 0.4.6 and transformers 4.5x internals"))
    if rank0 and "cornstarch.kernel.bitfield_attention" in imported and not args.no_ref_kernels:
        try:
            from cornstarch_b200.utils.reference_kernels import compare_attention

            out["reference_kernels"] = compare_attention(quick=True)
        except Exception as e:  # noqa: BLE001  (a Triton compile error on this GPU is a result, not a crash)
            out["reference_kernels"] = {"error": f"{type(e).__name__}: {e}".replace("\n", " ")[:400]}
    if rank0:
        print(json.dumps(out))


# ------------------------------------------------------------------------------------------------ library baseline arm
def run_baseline_child(args, rank: int, world: int) -> dict | None:
    """Run `bench.py --impl baseline` (same plan, same data, library kernels) as a child process of every rank BEFORE this
    process touches the GPU, and return its JSON record (rank 0).  The children form their own process group on another
    port; when they have exited, all of their memory is free again."""
    env = dict(os.environ)
    env.pop("TORCHELASTIC_USE_AGENT_STORE", None)  # the child group hosts its own store on its own port
    env["MASTER_ADDR"] = "127.0.0.1"
    env["MASTER_PORT"] = str(int(os.environ.get("MASTER_PORT", "29500")) + 23)
    cmd = [sys.executable, os.path.abspath(__file__), "--impl", "baseline", "--gpus", str(world), "--steps", str(args.baseline_steps),
           "--warmup", "3", "--config", str(args.config), "--recompute", args.recompute, "--microbatch", str(args.microbatch)]
    for flag, val, default in (("--shape", args.shape, None), ("--samples-per-gpu", args.samples_per_gpu, None),
                               ("--parallelism", args.parallelism, None)):
        cmd += [flag, str(val)]
    try:
        res = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=args.baseline_timeout)
    except subprocess.TimeoutExpired:
        return {"error": f"baseline arm did not finish within {args.baseline_timeout} s"} if rank == 0 else None
    if rank != 0:
        return None
    rec = None
    for line in res.stdout.splitlines():
        line = line.strip()
        if line.startswith("{") and '"metric"' in line:
            try:
                rec = json.loads(line)
            except ValueError:
                pass
    if rec is None:
        return {"error": f"baseline arm exited {res.returncode}: " + (res.stderr or res.stdout)[-300:].replace("\n", " ")}
    keep = {k: rec.get(k) for k in ("value", "unit", "ms_per_step", "steps", "warmup", "e2e", "gpu_launches")}
    keep["what"] = ("same models, plan, schedule and data with library kernels at every call site (cuBLAS, PyTorch SDPA / norms / "
                    "cross-entropy, torch fused AdamW, NCCL): bench.py --impl baseline, run on this box right before the native steps")
    keep["activation_checkpointing"] = rec.get("config", {}).get("activation_checkpointing")
    keep["peak_memory_gb"] = rec.get("config", {}).get("peak_memory_gb")
    keep["clocks"] = rec.get("clocks")
    return keep


# ------------------------------------------------------------------------------------------------ native arm
def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=4)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--recompute", choices=["auto", "full"], default="auto",
                    help="auto: after the first warm-up step, decoder layers that fit in free memory keep their activations")
    ap.add_argument("--impl", default="native", choices=["native", "reference", "baseline"])
    ap.add_argument("--shape", default="vlm", help="named shape from cornstarch_b200.zoo (default: the headline VLM)")
    ap.add_argument("--samples-per-gpu", type=int, default=SAMPLES_PER_GPU)
    ap.add_argument("--microbatch", type=int, default=1)
    ap.add_argument("--parallelism", default="auto", help="auto | dp | tp | cp | ep | enc<E>+llm<L>xtp<T> (e.g. enc1+llm3xtp2)")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-baseline", action="store_true", help="native arm: skip the library-baseline child run (vs_baseline stays null)")
    ap.add_argument("--baseline-steps", type=int, default=5)
    ap.add_argument("--baseline-timeout", type=int, default=420)
    ap.add_argument("--no-ref-kernels", action="store_true", help="reference arm: skip timing the reference's Triton kernels")
    ap.add_argument("--config", type=int, default=1, choices=[1, 2, 3, 4],
                    help="benchmark configuration: 1 VLM (headline), 2 vision+audio VALM, 3 long-context CP, 4 MoE EP+ZeRO-1")
    args = ap.parse_args()
    # presets of the other configurations (explicit flags win)
    preset = {2: dict(shape="valm", samples_per_gpu=2, parallelism={8: "enc1+llm2xtp2", 4: "enc1+llm2xtp1"}),
              3: dict(shape="long", samples_per_gpu=8, parallelism="cp"),
              4: dict(shape="moe", samples_per_gpu=2, parallelism="ep")}.get(args.config)
    if preset:
        if args.shape == "vlm":
            args.shape = preset["shape"]
        if args.samples_per_gpu == SAMPLES_PER_GPU:
            args.samples_per_gpu = preset["samples_per_gpu"]
        if args.parallelism == "auto":
            plan = preset["parallelism"]
            args.parallelism = plan.get(args.gpus, "auto") if isinstance(plan, dict) else plan
    return args


def main():
    args = parse_args()
    if args.impl == "reference":
        run_reference(args)
        return
    if args.impl == "baseline":
        # same models, plans and schedule with library kernels at every call site (cuBLAS GEMMs, PyTorch SDPA, PyTorch norms /
        # activations / cross-entropy, torch fused AdamW, NCCL collectives): the in-repo stand-in for the reference's stack
        os.environ["CORNSTARCH_B200_LIBRARY_OPS"] = "1"
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    assert world == args.gpus, f"--gpus {args.gpus} but WORLD_SIZE={world}: launch with torch.distributed.run"
    baseline = None
    if args.impl == "native" and not args.no_baseline:
        baseline = run_baseline_child(args, rank, world)
    import torch
    import torch.distributed as dist

    from cornstarch_b200.bench_support import build_trainer

    torch.cuda.set_device(local_rank)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))

    trainer = build_trainer(args, rank, world, local_rank)
    K, W = args.steps, max(args.warmup, 3)

    def sync():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    from cornstarch_b200.ops import _native as nat

    # ---- device-timed region: inputs already on the device
    for i in range(W):
        try:
            trainer.step_device()
        except torch.cuda.OutOfMemoryError:
            # a kept layer cost more than measured: on one GPU (no peer is waiting in a collective) fall back to
            # recomputing every layer and carry on with the warm-up
            if world > 1 or not hasattr(trainer, "recompute_everything"):
                raise
            trainer.recompute_everything()
            args.recompute = "full"
            trainer.step_device()
        if i < 2 and args.recompute == "auto" and hasattr(trainer, "tune_recompute"):
            # the first step ran with every layer recomputed and shows how much memory is left: layers that fit stop
            # being recomputed; the second step shows what a kept layer really costs and may add more.  The remaining
            # warm-up steps run with the final setting.
            trainer.tune_recompute()
    sync()
    sampler = ClockSampler(local_rank)
    sampler.start()
    launches0 = nat.launch_count
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(K):
        trainer.step_device()
    e1.record()
    sync()
    ms = e0.elapsed_time(e1)
    launches = nat.launch_count - launches0
    clocks = sampler.stop()

    # ---- end-to-end region: pinned host inputs copied every step, loss read back every step
    e2e = None
    if not args.no_e2e:
        trainer.step_e2e()
        sync()
        t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0.record()
        last = None
        for _ in range(K):
            last = trainer.step_e2e()
        t1.record()
        sync()
        ms_e2e = t0.elapsed_time(t1)
    else:
        ms_e2e, last = ms, None
    timeline_path = os.environ.get("CORNSTARCH_B200_TIMELINE")
    if timeline_path:
        # untimed extra steps with CUDA events around every schedule range: where each rank's device time goes
        from cornstarch_b200.utils import trace

        sync()
        trace.timeline(True)
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(2):
            trainer.step_device()
        b.record()
        totals = trace.timeline_totals()
        trace.timeline(False)
        rec = {"rank": rank, "role": getattr(trainer, "role", trainer.parallelism), "step_ms": round(a.elapsed_time(b) / 2, 2),
               "ranges": {k: {"count": c // 2, "ms_per_step": round(t / 2, 2)} for k, (c, t) in sorted(totals.items())}}
        covered = sum(v["ms_per_step"] for k, v in rec["ranges"].items())
        rec["other_ms_per_step"] = round(rec["step_ms"] - covered, 2)
        everyone = [rec]
        if world > 1:
            everyone = [None] * world
            dist.all_gather_object(everyone, rec)
        if rank == 0:
            with open(timeline_path, "w") as f:
                json.dump(everyone, f, indent=1)
    if world > 1:
        t = torch.tensor([ms, ms_e2e], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms, ms_e2e = float(t[0]), float(t[1])
        lt = torch.tensor([last if (last is not None and last == last) else -1e30], device="cuda", dtype=torch.float64)
        dist.all_reduce(lt, op=dist.ReduceOp.MAX)  # only the last pipeline stage knows the loss
        last = float(lt[0])
        lc = torch.tensor([launches], device="cuda", dtype=torch.int64)
        dist.all_reduce(lc)
        launches = int(lc[0])
    nat.check_status()
    peak_gb = torch.cuda.max_memory_allocated() / 2**30
    checks = None
    if world > 1:
        pk = torch.tensor([peak_gb], device="cuda", dtype=torch.float64)
        dist.all_reduce(pk, op=dist.ReduceOp.MAX)
        peak_gb = float(pk[0])
        # replicated parameters must agree bit for bit inside every data-parallel / tensor-parallel group
        # (a failure inside the comparison itself is reported in the record instead of costing the timed result)
        try:
            mine = trainer.checks() if hasattr(trainer, "checks") else {}
        except Exception as e:  # noqa: BLE001
            mine = {"error": {"ranks": 0, "params": 0, "mismatched": 1, "what": f"{type(e).__name__}: {e}"[:200]}}
        everyone = [None] * world
        dist.all_gather_object(everyone, mine)
        checks = {}
        for c in everyone:
            for k, v in (c or {}).items():
                agg = checks.setdefault(k, {"ranks": v["ranks"], "params_compared": 0, "mismatched": 0})
                agg["params_compared"] += v["params"]
                agg["mismatched"] += v["mismatched"]
                if "what" in v:
                    agg["what"] = v["what"]
        checks["ok"] = all(v["mismatched"] == 0 for v in checks.values() if isinstance(v, dict))
        # (without the end-to-end steps no loss is read back)
        checks["last_loss_finite"] = None if args.no_e2e else bool(last is not None and last == last and abs(last) < 1e30)
    if world > 1:
        # report the clocks of the busiest GPU (pipeline stages differ a lot in load), with every rank's throttle reasons
        everyone = [None] * world
        dist.all_gather_object(everyone, clocks)
        busiest = max(everyone, key=lambda c: c.get("power_w_max") or 0.0)
        reasons = sorted({r for c in everyone for r in c.get("reasons", [])})
        clocks = dict(busiest, reasons=reasons, sampled_ranks=world)

    tokens_per_step = trainer.tokens_per_step
    value = tokens_per_step * K / (ms / 1e3)
    if not args.no_e2e:
        e2e = {"value": tokens_per_step * K / (ms_e2e / 1e3), "unit": "tokens/s",
               "h2d_bytes_per_step": trainer.h2d_bytes_per_step, "d2h_bytes_per_step": trainer.d2h_bytes_per_step,
               "last_loss": last}
    if rank == 0:
        out = {
            "metric": METRIC, "value": value, "unit": "tokens/s", "n_gpus": world, "steps": K, "warmup": W,
            "ms_per_step": ms / K, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": (value / baseline["value"]) if (baseline and baseline.get("value")) else None, "dtype": "bf16",
            "data": "synthetic (pixels ~N(0,1), token ids uniform), random-init weights",
            "config": {"model": trainer.model_name, "global_batch": trainer.global_batch, "seq_len": trainer.seq_len,
                       "parallelism": trainer.parallelism, "microbatch": args.microbatch,
                       "l2": "no flush needed: every step streams >16 GB of weights and activations, far above the 126 MB L2",
                       "optimizer": ("fused AdamW, fp32 master weights (stored as bf16 parameter + 16-bit remainder) + fp32 moments, bf16 grads" if args.impl == "native"
                                     else "torch.optim.AdamW(fused=True) on bf16 parameters, clip_grad_norm_"),
                       "kernels": ("this package (sm_100a)" if args.impl == "native" else "library: cuBLAS, PyTorch SDPA, PyTorch elementwise, NCCL"), "activation_checkpointing": getattr(trainer, "recompute", "every layer"),
                       "peak_memory_gb": round(peak_gb, 1), "peak_memory_is": "max over ranks"},
            "clocks": clocks, "e2e": e2e, "gpu_launches": launches, "impl": args.impl, "benchmark_config": args.config,
        }
        if baseline is not None:
            out["baseline"] = baseline
            out["vs_baseline_is"] = "native value / library-baseline value measured in this run (the reference publishes no number)"
            if e2e and isinstance(baseline.get("e2e"), dict) and baseline["e2e"].get("value"):
                out["e2e"]["vs_baseline"] = e2e["value"] / baseline["e2e"]["value"]
        if checks is not None:
            out["checks"] = checks
        print(json.dumps(out))
    if nat.KERNEL_TIMES and rank == 0:
        # in-situ breakdown (CORNSTARCH_B200_KERNEL_TIMES=1): device time per native entry point since the process started
        times = nat.kernel_times()  # {entry point: (calls, total ms)}
        rows = sorted(times.items(), key=lambda kv: -kv[1][1])
        print(json.dumps({"kernel_times": {k: {"calls": c, "ms": round(ms, 2)} for k, (c, ms) in rows[:20]},
                          "sum_ms": round(sum(ms for _, ms in times.values()), 1)}))
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
