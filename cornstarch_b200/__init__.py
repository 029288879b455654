"""cornstarch_b200: multimodal LLM training for NVIDIA B200 (sm_100a).

Sub-packages: ``models`` (LLMs, vision and audio encoders with Hugging Face parameter names), ``multimodal``
(``MultimodalModel``, projector, processor), ``ops`` (entry points of the CUDA kernels in ``csrc``), ``nn`` (linear /
tensor-parallel layers, norms), ``parallel`` (mesh, stage manager, 1F1B schedule, collectives, context / expert
parallelism, peer-memory paths), ``shardformer`` (shard config, policies), ``plugin`` (modality-parallel, encoders-colocated
and heterogeneous plugins, checkpoint IO), ``optim`` (``FusedAdamW``), ``booster`` (``Booster``), ``utils``, ``testing``.

Nothing is imported eagerly: importing a sub-module pulls in what it needs, and the native library is loaded on first use.
"""

__version__ = "0.1.0"
