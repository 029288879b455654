from .modeling import (  # noqa: F401
    ModalDecoderModule,
    ModalEncoderModule,
    ModalModuleBase,
    MultimodalModel,
    MultimodalProjector,
    MultimodalProjectorConfig,
)
from .processing import MultimodalProcessor  # noqa: F401
