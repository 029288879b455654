"""Heterogeneous pipelines (Oobleck style) of a small Llama, with a sharded checkpoint written and read back through the
Booster (the reference's examples/pipeline_template/run_llama.py).  3 processes.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 3 --master-addr 127.0.0.1 \
        examples/pipeline_template/run_llama.py --backend gloo --checkpoint /tmp/llama_ckpt
"""

import os
import sys

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), "../.."))  # run from a source checkout
sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))

import torch
import torch.distributed as dist
from data_builder import Tokens, init_distributed, train_heterogeneous
from cornstarch_b200.models.llama import LlamaConfig, LlamaForCausalLM


def main():
    a, dev = init_distributed()
    torch.manual_seed(0)
    model = LlamaForCausalLM(LlamaConfig(vocab_size=1000, hidden_size=128, intermediate_size=256, num_hidden_layers=4,
                                         num_attention_heads=4, num_key_value_heads=2, max_position_embeddings=64))
    train_heterogeneous(model, Tokens(), lambda out, batch: out.loss, dev, checkpoint=a.checkpoint)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
