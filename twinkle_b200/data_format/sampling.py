"""Sampling request / response records.

Parity: reference ``src/twinkle/data_format/sampling.py:10-186`` — parameter
validation, ``max_tokens == 0`` + ``prompt_logprobs`` = scoring only, and the
response shape consumed by the RL loops.
"""
from __future__ import annotations

from dataclasses import asdict, dataclass, field
from typing import Any, Dict, List, Optional, Tuple, Union


@dataclass
class SamplingParams:
    max_tokens: Optional[int] = None
    seed: Optional[int] = None
    stop: Union[str, List[str], List[int], None] = None
    temperature: float = 1.0
    top_k: int = -1
    top_p: float = 1.0
    repetition_penalty: float = 1.0
    logprobs: Optional[int] = None
    prompt_logprobs: Optional[int] = None
    num_samples: int = 1

    def __post_init__(self):
        if self.max_tokens is not None and self.max_tokens < 0:
            raise ValueError('max_tokens must be >= 0')
        if self.temperature < 0:
            raise ValueError('temperature must be >= 0')
        if not (0.0 < self.top_p <= 1.0):
            raise ValueError('top_p must be in (0, 1]')
        if self.top_k == 0 or self.top_k < -1:
            raise ValueError('top_k must be -1 (off) or >= 1')
        if self.repetition_penalty <= 0:
            raise ValueError('repetition_penalty must be > 0')
        if self.num_samples < 1:
            raise ValueError('num_samples must be >= 1')
        if isinstance(self.stop, str):
            self.stop = [self.stop]

    @property
    def scoring_only(self) -> bool:
        return self.max_tokens == 0

    def stop_token_ids(self) -> List[int]:
        return [s for s in (self.stop or []) if isinstance(s, int)]

    def stop_strings(self) -> List[str]:
        return [s for s in (self.stop or []) if isinstance(s, str)]

    def to_dict(self) -> Dict[str, Any]:
        return asdict(self)

    def __getitem__(self, key: str):
        return getattr(self, key)

    def get(self, key: str, default=None):
        return getattr(self, key, default)

    @classmethod
    def from_dict(cls, d: Union['SampleResponse', Dict[str, Any]]) -> 'SampleResponse':
        """Rebuilds the record from its JSON form (what the sampler routes of the server return)."""
        if isinstance(d, cls):
            return d
        seqs = [s if isinstance(s, SampledSequence) else SampledSequence.from_dict(s) for s in d.get('sequences') or []]
        return cls(sequences=seqs, prompt_logprobs=d.get('prompt_logprobs'), topk_prompt_logprobs=d.get('topk_prompt_logprobs'))

    @classmethod
    def from_dict(cls, d: Optional[Dict[str, Any]]) -> 'SamplingParams':
        d = dict(d or {})
        known = {k: d[k] for k in cls.__dataclass_fields__ if k in d}
        return cls(**known)

    def to_engine(self) -> Dict[str, Any]:
        """Arguments of the native paged-KV engine."""
        return dict(max_new_tokens=self.max_tokens if self.max_tokens is not None else 512, temperature=self.temperature,
                    top_k=self.top_k, top_p=self.top_p, repetition_penalty=self.repetition_penalty, seed=self.seed,
                    stop_token_ids=self.stop_token_ids(), stop_strings=self.stop_strings(),
                    logprobs=self.logprobs, prompt_logprobs=self.prompt_logprobs, n=self.num_samples)


@dataclass
class SampledSequence:
    stop_reason: str  # 'stop' | 'length'
    tokens: List[int]
    logprobs: Optional[List[float]] = None
    topk_logprobs: Optional[List[List[Tuple[int, float]]]] = None
    decoded: Optional[str] = None
    new_input_feature: Optional[Dict[str, Any]] = None
    routed_experts: Any = None

    def __getitem__(self, key: str):  # records that crossed HTTP were dicts once; both spellings keep working
        return getattr(self, key)

    def get(self, key: str, default=None):
        return getattr(self, key, default)

    @classmethod
    def from_dict(cls, d: Dict[str, Any]) -> 'SampledSequence':
        return cls(**{k: d.get(k) for k in ('stop_reason', 'tokens', 'logprobs', 'topk_logprobs', 'decoded', 'new_input_feature', 'routed_experts')})


@dataclass
class SampleResponse:
    sequences: List[SampledSequence] = field(default_factory=list)
    prompt_logprobs: Optional[List[Optional[float]]] = None
    topk_prompt_logprobs: Optional[List[Optional[List[Tuple[int, float]]]]] = None

    def to_dict(self) -> Dict[str, Any]:
        return asdict(self)

    def __getitem__(self, key: str):
        return getattr(self, key)

    def get(self, key: str, default=None):
        return getattr(self, key, default)

    @classmethod
    def from_dict(cls, d: Union['SampleResponse', Dict[str, Any]]) -> 'SampleResponse':
        """Rebuilds the record from its JSON form (what the sampler routes of the server return)."""
        if isinstance(d, cls):
            return d
        seqs = [s if isinstance(s, SampledSequence) else SampledSequence.from_dict(s) for s in d.get('sequences') or []]
        return cls(sequences=seqs, prompt_logprobs=d.get('prompt_logprobs'), topk_prompt_logprobs=d.get('topk_prompt_logprobs'))
