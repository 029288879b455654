"""``cornstarch.models.multimodal_language_model`` under its reference import path
(cornstarch/models/multimodal_language_model/__init__.py:1-14); the classes live in :mod:`cornstarch_b200.multimodal`."""

from ..multimodal.modeling import (
    ModalDecoderModule,
    ModalEncoderModule,
    ModalModuleBase,
    MultimodalModel,
    MultimodalProjector,
    MultimodalProjectorConfig,
)
from ..multimodal.processing import MultimodalProcessor

__all__ = ["MultimodalModel", "ModalEncoderModule", "ModalDecoderModule", "ModalModuleBase", "MultimodalProjector",
           "MultimodalProjectorConfig", "MultimodalProcessor"]
