from .base import BaseSamplerEngine, Sampler
from .engine import NativeEngine, PagedKVCache
from .torch_sampler import TorchSampler, vLLMSampler
