"""``ShardConfig``: everything a policy needs to know to shard one modality's model.

Field names follow the reference dataclass (cornstarch/shardformer/shard/shard_config.py:12-63).
"""

from __future__ import annotations

from dataclasses import dataclass, field
from enum import Enum
from typing import Any, Optional

import torch.distributed as dist


class ContextParallelDistributionMode(Enum):
    UNIFORM = "uniform"
    ZIGZAG = "zigzag"
    MAKESPAN_MIN = "makespan_min"


SUPPORT_SP_MODE = ["ring_attn", "all_to_all"]


@dataclass
class ShardConfig:
    tensor_parallel_process_group: Optional[Any] = None
    sequence_parallel_process_group: Optional[Any] = None
    pipeline_stage_manager: Optional[Any] = None
    pipeline_template: Optional[Any] = None
    enable_tensor_parallelism: bool = True
    enable_sequence_parallelism: bool = False
    sequence_parallelism_mode: Optional[str] = None  # "ring_attn" | "all_to_all"
    context_parallel_distribution_mode: ContextParallelDistributionMode = ContextParallelDistributionMode.MAKESPAN_MIN
    # The next four switches and gradient_checkpoint_config exist so that the reference's constructor calls keep working
    # (cornstarch/shardformer/shard/shard_config.py:35-38).  They change nothing here: fused norms and flash attention are
    # the only GPU path of this package (CORNSTARCH_B200_LIBRARY_OPS=1 switches ALL ops to library kernels instead), and
    # recomputation is switched on the model (gradient_checkpointing_enable).
    enable_fused_normalization: bool = True
    enable_flash_attention: bool = True
    enable_jit_fused: bool = False
    enable_all_optimization: bool = False
    parallel_output: bool = True
    make_vocab_size_divisible_by: int = 64
    gradient_checkpoint_config: Optional[Any] = None
    expert_parallel_process_group: Optional[Any] = None
    # Tensor parallelism with token-sharded activations between the parallel blocks (norms, residuals and the other
    # token-wise work run on 1/tp of the tokens; the projections gather / scatter inside their GEMMs).  None = decided
    # by the environment variable CORNSTARCH_B200_TP_SEQ_SHARD (default off); decoders without projection biases only.
    tensor_parallel_sequence_sharding: Optional[bool] = None
    extra_kwargs: dict = field(default_factory=dict)

    def __post_init__(self):
        if self.sequence_parallelism_mode is not None:
            assert self.sequence_parallelism_mode in SUPPORT_SP_MODE, (
                f"Sequence parallelism mode {self.sequence_parallelism_mode} is not in the supported list {SUPPORT_SP_MODE}")
            self.enable_sequence_parallelism = True
        if isinstance(self.context_parallel_distribution_mode, str):
            self.context_parallel_distribution_mode = ContextParallelDistributionMode(self.context_parallel_distribution_mode)

    @property
    def tensor_parallel_size(self) -> int:
        g = self.tensor_parallel_process_group
        return 1 if (g is None or not self.enable_tensor_parallelism) else dist.get_world_size(g)

    @property
    def sequence_parallel_size(self) -> int:
        g = self.sequence_parallel_process_group
        return 1 if (g is None or not self.enable_sequence_parallelism) else dist.get_world_size(g)
