"""``ContextParallelBatchSplitUtils`` at the import path of the reference (cornstarch/shardformer/layers/utils.py)."""

from ...parallel.cp import BLOCK_M, BLOCK_N, ContextParallelBatchSplitUtils  # noqa: F401
