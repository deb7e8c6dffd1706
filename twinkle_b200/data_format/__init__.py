"""Typed records that flow between data, model, sampler and server layers.

Parity: reference ``src/twinkle/data_format/{input_feature,message,trajectory,
output,sampling}.py``.
"""
from .types import (InputFeature, LossOutput, Message, ModelOutput, Tool, ToolCall, Trajectory, to_input_feature)
from .sampling import SampledSequence, SampleResponse, SamplingParams

__all__ = ['InputFeature', 'LossOutput', 'Message', 'ModelOutput', 'Tool', 'ToolCall', 'Trajectory', 'SamplingParams',
           'SampledSequence', 'SampleResponse', 'to_input_feature']
