"""LLM-only hybrid parallelism (tensor x pipeline x data) through the same plugin: a MultimodalModel without encoders
(the reference's examples/distributed/run_llm_hybrid.py uses ColossalAI's HybridParallelPlugin for this).

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 4 --master-addr 127.0.0.1 \
        examples/distributed/run_llm_hybrid.py --tp 2 --pp 2
    ... --backend gloo --tp 1 --pp 2      # on CPU with 2 processes
"""

import os
import sys

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), "../.."))  # run from a source checkout

import argparse

import torch
import torch.distributed as dist

from cornstarch_b200.booster import Booster
from cornstarch_b200.models.llama import DecoderConfig, DecoderForCausalLM
from cornstarch_b200.multimodal import MultimodalModel
from cornstarch_b200.optim.fused_adamw import FusedAdamW
from cornstarch_b200.pipeline_template import PipelineTemplate
from cornstarch_b200.plugin.modal_parallel_plugin import ModalParallelPlugin
from cornstarch_b200.plugin.multimodal_parallel_plugin import MultimodalParallelPlugin


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--tp", type=int, default=1)
    ap.add_argument("--pp", type=int, default=2)
    ap.add_argument("--steps", type=int, default=3)
    ap.add_argument("--backend", default="nccl")
    a = ap.parse_args()
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    if a.backend == "nccl":
        torch.cuda.set_device(int(os.environ["LOCAL_RANK"]))
    dist.init_process_group(a.backend)
    dev = torch.device("cuda", torch.cuda.current_device()) if a.backend == "nccl" else torch.device("cpu")
    dtype = torch.bfloat16 if a.backend == "nccl" else torch.float32
    cfg = DecoderConfig(vocab_size=1024, hidden_size=256, intermediate_size=512, num_hidden_layers=4, num_attention_heads=8,
                        num_key_value_heads=4, max_position_embeddings=512)
    torch.manual_seed(0)
    with torch.device("meta"):
        llm = DecoderForCausalLM(cfg)
    model = MultimodalModel(encoders={}, language_model=llm)
    plugin = MultimodalParallelPlugin(
        encoder_plugins={}, language_model_plugin=ModalParallelPlugin(tp_size=a.tp, pipeline_template=PipelineTemplate.even_split(llm, a.pp)),
        precision="bf16" if a.backend == "nccl" else None, num_microbatches=4, microbatch_size=1, device=dev)
    booster = Booster(plugin=plugin)
    model, opt, criterion, *_ = booster.boost(model, FusedAdamW, criterion=lambda out, batch: out.loss)
    model.train()
    for step in range(a.steps):
        ids = torch.randint(0, 1024, (4, 128), generator=torch.Generator().manual_seed(step)).to(dev)
        out = booster.execute_pipeline(iter([{"input_ids": ids, "labels": ids}]), model, criterion, opt, return_loss=True)
        opt.step()
        opt.zero_grad()
        if out["loss"] is not None:
            print(f"step {step} loss {float(out['loss']):.4f}", flush=True)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
