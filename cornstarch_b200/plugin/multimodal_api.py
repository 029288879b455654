"""Names exported by the reference's ``cornstarch.plugin.multimodal_parallel_plugin`` package
(cornstarch/plugin/multimodal_parallel_plugin/__init__.py:1-11)."""

from ..parallel.mesh import MultiModalProcessGroupMesh  # noqa: F401
from ..parallel.p2p import MultimodalPipelineP2PCommunication  # noqa: F401
from ..parallel.schedule import MultimodalEncoderTrainingOneForwardOneBackwardSchedule  # noqa: F401
from ..parallel.stage_manager import MultiModalPipelineStageManager  # noqa: F401
from .modal_parallel_plugin import ModalParallelPlugin  # noqa: F401
from .multimodal_parallel_plugin import MultimodalParallelModule, MultimodalParallelPlugin  # noqa: F401
