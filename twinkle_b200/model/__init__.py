"""Model backends.  ``TransformersModel`` / ``MultiLoraTransformersModel`` keep
the reference's names; ``MegatronModel`` is the tensor/pipeline-parallel
backend of the same engine."""
from .base import TwinkleModel
from .multi_lora import LoraConfig, MultiLora
from .native import MultiLoraTransformersModel, TransformersModel
from .optimizer_group import OptimizerGroup, TrainStatus


def __getattr__(name):
    if name in ('MegatronModel', 'MultiLoraMegatronModel'):
        from . import megatron
        return getattr(megatron, name)
    raise AttributeError(name)
