"""Sampler contract.  Parity: reference ``src/twinkle/sampler/base.py:16-114`` and ``base_engine.py:17-106``."""
from __future__ import annotations

from abc import ABC, abstractmethod
from typing import Any, Dict, List, Optional, Sequence, Union

from ..data_format import InputFeature, SampleResponse, SamplingParams, Trajectory


class Sampler(ABC):
    template = None

    @abstractmethod
    def sample(self, inputs, sampling_params: Optional[SamplingParams] = None, adapter_name: Optional[str] = None,
               adapter_path: Optional[str] = None, **kwargs) -> List[SampleResponse]: ...

    def set_template(self, template_cls, **kwargs) -> None:
        from ..template import Template, template_mapping
        if isinstance(template_cls, str):
            template_cls = template_mapping.get(template_cls, Template)
        self.template = template_cls(**kwargs) if isinstance(template_cls, type) else template_cls

    def encode_trajectory(self, trajectory: Trajectory) -> InputFeature:
        if self.template is None:
            raise ValueError('set_template must be called before sampling from trajectories')
        return self.template.encode(trajectory, add_generation_prompt=True)

    def decode_response(self, token_ids: Sequence[int]) -> str:
        return self.template.decode(token_ids) if self.template is not None else ''

    def add_adapter_to_sampler(self, adapter_name: str, config_or_dir, **kwargs) -> None:
        raise NotImplementedError


class BaseSamplerEngine(ABC):

    @abstractmethod
    def generate(self, prompts, params, **kwargs): ...

    def update_weights(self, weights, **kwargs) -> None:
        raise NotImplementedError

    def sleep(self, level: int = 1) -> None:
        pass

    def wake_up(self) -> None:
        pass

    def save_weights_for_sampler(self, path: str) -> None:
        raise NotImplementedError
