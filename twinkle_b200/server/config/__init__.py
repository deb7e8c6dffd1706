"""Typed server configuration.

Parity: reference ``src/twinkle/server/config/server_config.py:28-82``, ``application_spec.py:24-171``,
``persistence.py:21-56``, ``telemetry.py:8-18`` — a strict (``extra='forbid'``) pydantic tree loaded from YAML:
``http_options``, ``telemetry``, ``persistence {mode: memory|file|redis}``, ``task_queue`` and a list of
``applications`` (``import_path`` ∈ server | model | sampler | processor) with typed ``args``.
The reference deploys through Ray Serve; here every application is a FastAPI sub-app mounted at its
``route_prefix`` in one uvicorn process; a model or sampler application whose ``device_group`` has more than one rank
(or ``workers: pool``) builds its backend in a worker-pool device group, one process per rank.
"""
from __future__ import annotations

from typing import Any, Dict, List, Literal, Optional, Union

import yaml
from pydantic import BaseModel, ConfigDict, Field, model_validator


class _Strict(BaseModel):
    model_config = ConfigDict(extra='forbid', protected_namespaces=())


class HttpOptions(_Strict):
    host: str = '127.0.0.1'
    port: int = 8000


class TelemetryConfig(_Strict):
    enabled: bool = False
    debug: bool = False
    otlp_endpoint: Optional[str] = None
    service_name: str = 'twinkle-server'
    metrics_interval_s: float = 15.0


class PersistenceConfig(_Strict):
    mode: Literal['memory', 'file', 'redis'] = 'memory'
    file_path: Optional[str] = None
    redis_url: Optional[str] = None
    key_prefix: str = 'twinkle'

    @model_validator(mode='after')
    def _check(self):
        if self.mode == 'file' and not self.file_path:
            raise ValueError("persistence.mode='file' needs file_path")
        if self.mode == 'redis' and not self.redis_url:
            raise ValueError("persistence.mode='redis' needs redis_url")
        return self


class TaskQueueConfig(_Strict):
    rps_limit: float = 100.0
    tps_limit: float = 16000.0
    window_seconds: float = 1.0
    queue_timeout: float = 300.0
    execution_timeout: float = 120.0
    max_input_tokens: int = 16000
    enabled: bool = True

    @model_validator(mode='after')
    def _check(self):
        for k in ('rps_limit', 'tps_limit', 'window_seconds', 'queue_timeout', 'execution_timeout'):
            if getattr(self, k) <= 0:
                raise ValueError(f'{k} must be > 0')
        return self


class DeviceGroupSpec(_Strict):
    name: str = 'model'
    ranks: Union[int, List[int]] = 1
    device_type: str = 'cuda'
    gpus_per_worker: int = 1


class DeviceMeshSpec(_Strict):
    dp_size: Optional[int] = 1
    fsdp_size: Optional[int] = None
    tp_size: Optional[int] = None
    pp_size: Optional[int] = None
    cp_size: Optional[int] = None
    ep_size: Optional[int] = None
    etp_size: Optional[int] = None
    ulysses_size: Optional[int] = None
    vpp_size: Optional[int] = None
    sequence_parallel: bool = False

    def build(self):
        from ...utils.device_mesh import DeviceMesh
        return DeviceMesh.from_sizes(**self.model_dump())


class ModelArgs(_Strict):
    model_id: str
    nproc_per_node: int = 1
    device_group: DeviceGroupSpec = Field(default_factory=DeviceGroupSpec)
    device_mesh: DeviceMeshSpec = Field(default_factory=DeviceMeshSpec)
    backend: Literal['mock', 'transformers', 'megatron'] = 'transformers'
    workers: Literal['auto', 'pool', 'inline'] = 'auto'  # auto: a worker group when device_group has more than one rank
    adapter_config: Dict[str, Any] = Field(default_factory=dict)
    queue_config: Optional[TaskQueueConfig] = None
    max_loras: int = 5
    max_r: int = 32
    max_length: int = 8192
    adapter_timeout: float = 1800.0
    adapter_max_lifetime: float = 36000.0


class SamplerArgs(_Strict):
    model_id: str
    nproc_per_node: int = 1
    device_group: DeviceGroupSpec = Field(default_factory=lambda: DeviceGroupSpec(name='sampler'))
    device_mesh: DeviceMeshSpec = Field(default_factory=DeviceMeshSpec)
    sampler_type: Literal['mock', 'vllm', 'torch'] = 'torch'
    workers: Literal['auto', 'pool', 'inline'] = 'auto'
    engine_args: Dict[str, Any] = Field(default_factory=dict)
    queue_config: Optional[TaskQueueConfig] = None
    max_loras: int = 4


class ServerArgs(_Strict):
    supported_models: List[str] = Field(default_factory=list)
    per_token_model_limit: int = 30
    session_timeout: float = 1800.0


class ProcessorArgs(_Strict):
    nproc_per_node: int = 1
    device_group: DeviceGroupSpec = Field(default_factory=lambda: DeviceGroupSpec(name='processor', device_type='cpu'))


_ARGS = {'server': ServerArgs, 'model': ModelArgs, 'sampler': SamplerArgs, 'processor': ProcessorArgs}


class ApplicationSpec(_Strict):
    name: str
    route_prefix: str = '/'
    import_path: Literal['server', 'model', 'sampler', 'processor']
    args: Dict[str, Any] = Field(default_factory=dict)
    deployments: List[Dict[str, Any]] = Field(default_factory=list)

    @model_validator(mode='after')
    def _typed_args(self):
        self._typed = _ARGS[self.import_path](**self.args)
        if not self.route_prefix.startswith('/'):
            raise ValueError('route_prefix must start with /')
        return self

    @property
    def typed_args(self):
        return self._typed


class ServerConfig(_Strict):
    ray_namespace: Optional[str] = None  # accepted for compatibility; unused without Ray
    proxy_location: Optional[str] = None
    http_options: HttpOptions = Field(default_factory=HttpOptions)
    telemetry: TelemetryConfig = Field(default_factory=TelemetryConfig)
    persistence: PersistenceConfig = Field(default_factory=PersistenceConfig)
    task_queue: TaskQueueConfig = Field(default_factory=TaskQueueConfig)
    applications: List[ApplicationSpec] = Field(default_factory=list)

    @classmethod
    def from_yaml(cls, path: str) -> 'ServerConfig':
        from ..exceptions import ConfigParseError
        with open(path) as f:
            try:
                doc = yaml.safe_load(f)
            except yaml.YAMLError as e:
                raise ConfigParseError(f'{path}: not valid YAML: {e}') from e
        if doc is not None and not isinstance(doc, dict):
            raise ConfigParseError(f'{path}: the top level must be a mapping, found {type(doc).__name__}')
        return cls(**(doc or {}))

    @model_validator(mode='after')
    def _unique(self):
        names = [a.name for a in self.applications]
        if len(set(names)) != len(names):
            raise ValueError('application names must be unique')
        prefixes = [a.route_prefix for a in self.applications]
        if len(set(prefixes)) != len(prefixes):
            raise ValueError('route prefixes must be unique')
        return self

    def to_yaml(self) -> str:
        return yaml.safe_dump(self.model_dump(), sort_keys=False)
