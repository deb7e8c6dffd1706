"""Typed request and response records of the Twinkle-native HTTP routes, shared by the client twins and the server's
handlers. Requests allow extra keys (method keyword arguments travel beside the named fields); the named fields are the
ones a route cannot work without, so a missing one is reported as a 400 with the field's name instead of failing deep
inside the model call.

The request records are built from one table (route → required / optional fields); ``REQUESTS[route]`` gives the
record type and :func:`validate_request` applies it to a JSON body.

Parity: reference ``src/twinkle_client/types/{model,sampler,processor,session,server,training,checkpoint}.py``."""
from __future__ import annotations

from typing import Any, Dict, List, Optional, Tuple, Type, Union

from pydantic import BaseModel, ConfigDict, ValidationError, create_model, field_validator


class _Request(BaseModel):
    model_config = ConfigDict(extra='allow', protected_namespaces=())


class _Record(BaseModel):
    model_config = ConfigDict(extra='allow', protected_namespaces=())


_REQ = ...  # marks a required field in the table below

# route name → {field: (type, default | _REQ)}
_MODEL_ROUTES: Dict[str, Dict[str, Tuple[Any, Any]]] = {
    'create': {},
    'forward': {'inputs': (Any, _REQ), 'adapter_name': (str, _REQ)},
    'forward_only': {'inputs': (Any, _REQ), 'adapter_name': (Optional[str], None)},
    'forward_backward': {'inputs': (Any, _REQ), 'adapter_name': (str, _REQ)},
    'calculate_loss': {'adapter_name': (str, _REQ)},
    'backward': {'adapter_name': (str, _REQ)},
    'clip_grad_norm': {'adapter_name': (str, _REQ), 'max_grad_norm': (float, 1.0), 'norm_type': (int, 2)},
    'step': {'adapter_name': (str, _REQ)},
    'zero_grad': {'adapter_name': (str, _REQ)},
    'lr_step': {'adapter_name': (str, _REQ)},
    'clip_grad_and_step': {'adapter_name': (str, _REQ), 'max_grad_norm': (float, 1.0), 'norm_type': (int, 2)},
    'get_train_configs': {'adapter_name': (str, _REQ)},
    'set_loss': {'loss_cls': (str, _REQ), 'adapter_name': (str, _REQ)},
    'set_optimizer': {'optimizer_cls': (str, _REQ), 'adapter_name': (str, _REQ)},
    'set_lr_scheduler': {'scheduler_cls': (str, _REQ), 'adapter_name': (str, _REQ)},
    'set_template': {'template_cls': (str, _REQ), 'adapter_name': (str, _REQ)},
    'set_processor': {'processor_cls': (str, _REQ), 'adapter_name': (str, _REQ)},
    'apply_patch': {'patch_cls': (str, _REQ), 'adapter_name': (str, _REQ)},
    'add_metric': {'metric_cls': (str, _REQ), 'adapter_name': (str, _REQ), 'is_training': (Optional[bool], None)},
    'calculate_metric': {'adapter_name': (str, _REQ), 'is_training': (bool, True)},
    'get_state_dict': {'adapter_name': (str, _REQ)},
    'save': {'adapter_name': (str, _REQ), 'save_optimizer': (bool, False), 'name': (Optional[str], None), 'is_sampler': (bool, False)},
    'load': {'adapter_name': (str, _REQ), 'name': (str, _REQ), 'load_optimizer': (bool, False)},
    'resume_from_checkpoint': {'name': (str, _REQ), 'adapter_name': (str, ''), 'resume_only_model': (bool, False)},
    'add_adapter_to_model': {'adapter_name': (str, _REQ), 'config': (Union[str, Dict[str, Any]], _REQ), 'save_dir': (Optional[str], None)},
}
_SAMPLER_ROUTES: Dict[str, Dict[str, Tuple[Any, Any]]] = {
    'sample': {'inputs': (Any, _REQ), 'sampling_params': (Optional[Dict[str, Any]], None), 'adapter_name': (Optional[str], None),
               'adapter_path': (Optional[str], None)},
    'add_adapter_to_sampler': {'adapter_name': (str, _REQ), 'config': (Optional[Union[str, Dict[str, Any]]], None), 'adapter_path': (Optional[str], None)},
}
_OTHER_ROUTES: Dict[str, Dict[str, Tuple[Any, Any]]] = {
    'processor/create': {'class_name': (str, _REQ), 'args': (List[Any], []), 'kwargs': (Dict[str, Any], {}), 'session_id': (Optional[str], None)},
    'processor/call': {'object_id': (str, _REQ), 'method': (str, _REQ), 'args': (List[Any], []), 'kwargs': (Dict[str, Any], {})},
    'processor/heartbeat': {'object_id': (str, _REQ)},
    'create_session': {'metadata': (Optional[Dict[str, Any]], None)},
    'session_heartbeat': {'session_id': (str, _REQ)},
    'weights_info': {'path': (str, _REQ)},
}


def _camel(route: str) -> str:
    return ''.join(p.capitalize() for p in route.replace('/', '_').split('_')) + 'Request'


def _build(table: Dict[str, Dict[str, Tuple[Any, Any]]]) -> Dict[str, Type[_Request]]:
    return {route: create_model(_camel(route), __base__=_Request, **{k: (t, d) for k, (t, d) in fields.items()}) for route, fields in table.items()}


REQUESTS: Dict[str, Type[_Request]] = {**_build(_MODEL_ROUTES), **_build(_SAMPLER_ROUTES), **_build(_OTHER_ROUTES)}


class UploadToHubRequest(_Request):
    """``checkpoint_dir`` may be the record a save call returned; its ``twinkle_path`` is then used."""
    checkpoint_dir: Union[str, Dict[str, Any]]
    hub_model_id: str
    hub_token: Optional[str] = None
    async_upload: bool = False

    @field_validator('checkpoint_dir', mode='before')
    @classmethod
    def _path_of_record(cls, v):
        if isinstance(v, dict):
            if 'twinkle_path' not in v:
                raise ValueError("a checkpoint record needs 'twinkle_path'")
            return v['twinkle_path']
        return v


REQUESTS['upload_to_hub'] = UploadToHubRequest


class RequestError(ValueError):
    """A body that lacks a required field or has one of the wrong type; ``status_code`` 400."""
    status_code = 400


def validate_request(route: str, body: Dict[str, Any], aliases: Optional[Dict[str, str]] = None) -> Dict[str, Any]:
    """Body checked against ``REQUESTS[route]`` (routes without a record pass through): defaults filled in, extra keys
    kept. ``aliases`` maps an accepted alternative key to the record's field (``{'model_id': 'adapter_name'}``)."""
    model = REQUESTS.get(route)
    if model is None:
        return dict(body)
    body = dict(body)
    for alt, name in (aliases or {}).items():
        if name not in body and alt in body:
            body[name] = body[alt]
    try:
        return model(**body).model_dump()
    except ValidationError as e:
        problems = '; '.join(f"{'.'.join(str(x) for x in err['loc'])}: {err['msg']}" for err in e.errors())
        raise RequestError(f'/{route}: {problems}') from None


# ------------------------------------------------------------------------------------------------------- responses
class OkResponse(_Record):
    status: str = 'ok'


class ModelResult(_Record):
    status: str = 'ok'
    result: Any = None


class SaveResponse(_Record):
    twinkle_path: str
    checkpoint_dir: Optional[str] = None


class AddAdapterResponse(OkResponse):
    adapter_name: str


class UploadToHubResponse(_Record):
    request_id: str


class UploadStatusResponse(_Record):
    request_id: str
    status: str  # pending | queued | running | completed | failed
    error: Optional[str] = None


class SampledSequenceModel(_Record):
    stop_reason: str
    tokens: List[int]
    logprobs: Optional[List[float]] = None
    topk_logprobs: Optional[List[Any]] = None
    decoded: Optional[str] = None
    new_input_feature: Optional[Dict[str, Any]] = None
    routed_experts: Any = None


class SampleResponseModel(_Record):
    sequences: List[SampledSequenceModel] = []
    prompt_logprobs: Optional[List[Optional[float]]] = None
    topk_prompt_logprobs: Optional[List[Any]] = None


class SampleResponseModelList(_Record):
    status: str = 'ok'
    result: List[SampleResponseModel] = []


class CreateSessionResponse(_Record):
    session_id: str


class SessionHeartbeatResponse(_Record):
    status: str = 'ok'
    alive: bool = True


class SupportedModel(_Record):
    model_name: str
    max_loras: Optional[int] = None


class GetServerCapabilitiesResponse(_Record):
    supported_models: List[SupportedModel] = []


class HealthResponse(_Record):
    status: str = 'ok'


class ErrorResponse(_Record):
    detail: Any


class Cursor(_Record):
    offset: int = 0
    limit: int = 100
    total_count: int = 0


class Checkpoint(_Record):
    checkpoint_id: str
    checkpoint_type: str = 'training'  # training | sampler
    time: Optional[Union[str, float]] = None
    size_bytes: Optional[int] = None
    public: bool = False
    twinkle_path: Optional[str] = None


class TrainingRun(_Record):
    training_run_id: str
    base_model: Optional[str] = None
    model_owner: Optional[str] = None
    is_lora: bool = True
    lora_rank: Optional[int] = None
    corrupted: bool = False
    last_request_time: Optional[Union[str, float]] = None
    last_checkpoint: Optional[Checkpoint] = None
    last_sampler_checkpoint: Optional[Checkpoint] = None
    user_metadata: Optional[Dict[str, Any]] = None


class TrainingRunsResponse(_Record):
    training_runs: List[TrainingRun] = []
    cursor: Optional[Cursor] = None


class CheckpointsListResponse(_Record):
    checkpoints: List[Checkpoint] = []
    cursor: Optional[Cursor] = None


class WeightsInfoResponse(_Record):
    base_model: Optional[str] = None
    is_lora: bool = True
    lora_rank: Optional[int] = None


class ParsedCheckpointTwinklePath(_Record):
    """Parts of ``twinkle://<training_run_id>/<weights|sampler_weights>/<checkpoint_id>``."""
    path: str
    training_run_id: str
    checkpoint_type: str
    checkpoint_id: str

    @classmethod
    def parse(cls, path: str) -> 'ParsedCheckpointTwinklePath':
        for scheme in ('twinkle://', 'tinker://'):
            if path.startswith(scheme):
                parts = path[len(scheme):].strip('/').split('/')
                if len(parts) == 3 and parts[1] in ('weights', 'sampler_weights') and all(parts):
                    return cls(path=path, training_run_id=parts[0], checkpoint_type='training' if parts[1] == 'weights' else 'sampler',
                               checkpoint_id=parts[2])
        raise ValueError(f'not a checkpoint path: {path!r} (expected twinkle://<run>/<weights|sampler_weights>/<name>)')


class ResolvedLoadPath(_Record):
    """What a ``load`` argument resolved to: a registered checkpoint (``twinkle_path`` + directory) or a plain directory."""
    checkpoint_name: str
    checkpoint_dir: Optional[str] = None
    twinkle_path: Optional[str] = None


__all__ = [n for n, v in list(globals().items()) if isinstance(v, type) and issubclass(v, (_Request, _Record, RequestError)) and not n.startswith('_')] + [
    'REQUESTS', 'validate_request']
