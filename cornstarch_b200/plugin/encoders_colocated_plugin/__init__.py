"""Encoders-colocated plugin: all encoders share ranks and run one after the other in front of the LLM stages
(the reference's cornstarch/plugin/encoders_colocated_plugin/)."""

from .encoders_colocated_plugin import (
    EncodersColocatedMultimodalParallelModule,
    EncodersColocatedMultimodalParallelPlugin,
    EncodersColocatedPipelineStageManager,
    EncodersColocatedProcessGroupMesh,
)

EncodersColocatedPlugin = EncodersColocatedMultimodalParallelPlugin  # the name the reference's docs use

__all__ = ["EncodersColocatedMultimodalParallelModule", "EncodersColocatedMultimodalParallelPlugin",
           "EncodersColocatedPipelineStageManager", "EncodersColocatedProcessGroupMesh", "EncodersColocatedPlugin"]
