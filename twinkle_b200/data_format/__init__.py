"""Typed records that flow between data, model, sampler and server layers.

Parity: reference ``src/twinkle/data_format/{input_feature,message,trajectory,
output,sampling}.py``.
"""
from .types import (FunctionCall, FunctionSpec, InputFeature, LossOutput, Message, ModelOutput, Tool, ToolCall, Trajectory, pack_value,
                    to_input_feature, tool_call_to_openai, tool_to_openai, user_data_get, user_data_set)
from .sampling import SampledSequence, SampleResponse, SamplingParams

__all__ = ['InputFeature', 'LossOutput', 'Message', 'ModelOutput', 'Tool', 'ToolCall', 'Trajectory', 'SamplingParams',
           'SampledSequence', 'SampleResponse', 'to_input_feature', 'FunctionCall', 'FunctionSpec', 'pack_value', 'user_data_get',
           'user_data_set', 'tool_to_openai', 'tool_call_to_openai']
