"""HTTP client twins.

Parity: reference ``src/twinkle_client/`` — ``init_twinkle_client()`` / ``TwinkleClient`` (session with a
heart-beat thread, run / checkpoint listing), HTTP twins with the same method names as the server-side
components (``MultiLoraTransformersModel``, ``vLLMSampler`` / ``TorchSampler``, ``Dataset``, ``DataLoader``,
``InputProcessor``), the Tinker-protocol client (``TinkerClient``: futures + long-poll), sticky-routing and
auth headers (``Twinkle-Authorization``, ``x-request-id``, ``serve_multiplexed_model_id``).
The external ``tinker`` SDK is not installed here; ``TinkerClient`` speaks the same wire format.
"""
from __future__ import annotations

import json
import os
import threading
import time
import uuid
from typing import Any, Callable, Dict, Iterator, List, Optional

_DEFAULT: Dict[str, Any] = {'client': None}


class HttpError(RuntimeError):

    def __init__(self, status: int, detail: Any):
        super().__init__(f'HTTP {status}: {detail}')
        self.status, self.detail = status, detail


class Transport:
    """``requests`` against a URL, or an in-process ASGI app (tests, notebooks)."""

    def __init__(self, base_url: Optional[str] = None, app=None, token: Optional[str] = None):
        self.base_url = (base_url or os.environ.get('TWINKLE_SERVER_URL', 'http://127.0.0.1:8000')).rstrip('/')
        self.token = token or os.environ.get('TWINKLE_SERVER_TOKEN', 'anonymous')
        self._asgi = None
        if app is not None:
            from starlette.testclient import TestClient
            self._asgi = TestClient(app)

    def headers(self, model_id: Optional[str] = None) -> Dict[str, str]:
        h = {'Twinkle-Authorization': self.token, 'x-request-id': uuid.uuid4().hex}
        if model_id:
            h['serve_multiplexed_model_id'] = model_id
            h['serve-multiplexed-model-id'] = model_id
        return h

    def request(self, method: str, path: str, body: Optional[Dict[str, Any]] = None, model_id: Optional[str] = None, timeout: float = 600.0):
        if self._asgi is not None:
            r = self._asgi.request(method, path, json=body, headers=self.headers(model_id))
        else:
            import requests
            r = requests.request(method, self.base_url + path, json=body, headers=self.headers(model_id), timeout=timeout)
        if r.status_code >= 400:
            try:
                detail = r.json()
            except Exception:
                detail = r.text
            raise HttpError(r.status_code, detail)
        return r.json() if r.content else None

    def post(self, path, body=None, **kw):
        return self.request('POST', path, body or {}, **kw)

    def get(self, path, **kw):
        return self.request('GET', path, None, **kw)


class TwinkleClient:

    def __init__(self, base_url: Optional[str] = None, token: Optional[str] = None, app=None, heartbeat_interval: float = 10.0,
                 model_prefix: str = '/model', sampler_prefix: str = '/sampler', processor_prefix: str = '/processor'):
        self.t = Transport(base_url, app, token)
        self.model_prefix, self.sampler_prefix, self.processor_prefix = model_prefix, sampler_prefix, processor_prefix
        self.session_id = self.t.post('/twinkle/create_session', {'sdk_version': 'twinkle_b200'})['session_id']
        self._stop = threading.Event()
        self._hb = threading.Thread(target=self._beat, args=(heartbeat_interval, ), daemon=True)
        self._hb.start()

    def _beat(self, interval: float) -> None:
        while not self._stop.wait(interval):
            try:
                self.t.post('/twinkle/session_heartbeat', {'session_id': self.session_id})
            except Exception:
                pass

    def close(self) -> None:
        self._stop.set()

    # -------------------------------------------------------------- server
    def capabilities(self):
        return self.t.get('/twinkle/get_server_capabilities')

    get_server_capabilities = capabilities

    def health_check(self) -> bool:
        """Whether the server answers its health route (never raises)."""
        try:
            return self.t.get('/twinkle/healthz').get('status') == 'ok'
        except Exception:
            return False

    def get_capacity_info(self) -> Dict[str, Any]:
        """Free adapter slots and queue depths per replica (what the sticky router places new adapters by)."""
        return self.t.get('/twinkle/capacity_info')

    def create_session(self, metadata: Optional[Dict[str, Any]] = None) -> str:
        """A further session on the same connection (the constructor opens the first and keeps it alive)."""
        return self.t.post('/twinkle/create_session', {'sdk_version': 'twinkle_b200', 'user_metadata': metadata or {}})['session_id']

    def status(self):
        return self.t.get('/twinkle/status')

    # ------------------------------------------------- runs and checkpoints
    def list_training_runs(self, limit: int = 20, offset: int = 0, all_users: bool = False) -> List[Dict[str, Any]]:
        """This token's training runs, newest first (reference ``twinkle_client/manager.py:204-228``; a token sees its own
        runs only, so ``all_users`` is accepted and has no effect)."""
        return self.list_training_runs_with_cursor(limit, offset, all_users)[0]

    def list_training_runs_with_cursor(self, limit: int = 20, offset: int = 0, all_users: bool = False):
        """``(runs, cursor)`` with ``cursor = {offset, limit, total_count}`` for paging."""
        d = self.t.get(f'/twinkle/training_runs?limit={int(limit)}&offset={int(offset)}')
        return d.get('training_runs', []), d.get('cursor', {})

    def get_training_run(self, run_id: str) -> Dict[str, Any]:
        return self.t.get(f'/twinkle/training_runs/{run_id}')

    def find_training_run_by_model(self, base_model: str) -> List[Dict[str, Any]]:
        return [r for r in self.list_training_runs(limit=100) if r.get('base_model') == base_model]

    def list_checkpoints(self, run_id: str):
        return self.t.get(f'/twinkle/training_runs/{run_id}/checkpoints')['checkpoints']

    def get_checkpoint_path(self, run_id: str, checkpoint_id: str) -> Dict[str, Any]:
        """``{path, twinkle_path, training_run_id, checkpoint_type, checkpoint_id}`` of a checkpoint named ``weights/<name>``,
        ``sampler_weights/<name>`` or just ``<name>`` (a training checkpoint)."""
        d = self.t.get(f'/twinkle/checkpoint_path/{run_id}/{checkpoint_id}')
        kind, _, name = checkpoint_id.partition('/')
        if not name:
            kind, name = 'weights', checkpoint_id
        return {'path': d.get('path', ''), 'twinkle_path': d.get('twinkle_path') or f'twinkle://{run_id}/{kind}/{name}', 'training_run_id': run_id,
                'checkpoint_type': kind, 'checkpoint_id': checkpoint_id}

    def get_checkpoint_twinkle_path(self, run_id: str, checkpoint_id: str) -> str:
        return self.get_checkpoint_path(run_id, checkpoint_id)['twinkle_path']

    def get_latest_checkpoint_path(self, run_id: str) -> Optional[str]:
        """File-system path of the run's newest checkpoint (what a resumed job loads), or None."""
        cks = self.list_checkpoints(run_id)
        if not cks:
            return None
        last = cks[-1]
        kind = 'sampler_weights' if last.get('checkpoint_type') == 'sampler' else 'weights'
        name = str(last.get('checkpoint_id', '')).split('/')[-1]
        return self.get_checkpoint_path(run_id, f'{kind}/{name}')['path']

    def delete_checkpoint(self, run_id: str, checkpoint_id: str):
        return self.t.request('DELETE', f'/twinkle/training_runs/{run_id}/checkpoints/{checkpoint_id}')

    def weights_info(self, path: str):
        return self.t.post('/twinkle/weights_info', {'path': path})

    get_weights_info = weights_info


# the reference client's name for a failed request
TwinkleClientError = HttpError


def init_twinkle_client(base_url: Optional[str] = None, token: Optional[str] = None, *, api_key: Optional[str] = None,
                        session_heartbeat_interval: Optional[float] = None, **kw) -> TwinkleClient:
    """The client that later ``MultiLoraTransformersModel`` / sampler / dataset twins use by default.  ``api_key`` and
    ``session_heartbeat_interval`` are the reference's names for ``token`` and ``heartbeat_interval`` (reference
    ``twinkle_client/__init__.py:37-75``); URL and token fall back to ``TWINKLE_SERVER_URL`` / ``TWINKLE_SERVER_TOKEN``."""
    if session_heartbeat_interval is not None:
        kw.setdefault('heartbeat_interval', float(session_heartbeat_interval))
    c = TwinkleClient(base_url, token or api_key, **kw)
    _DEFAULT['client'] = c
    return c


def _client(c: Optional[TwinkleClient]) -> TwinkleClient:
    c = c or _DEFAULT['client']
    if c is None:
        raise RuntimeError('call init_twinkle_client() first')
    return c


class MultiLoraTransformersModel:
    """HTTP twin: every method posts to ``<model_prefix>/<base_model>/twinkle/<method>``."""

    def __init__(self, model_id: str, client: Optional[TwinkleClient] = None, **kwargs):
        if '://' in model_id:          # 'ms://org/name' and 'hf://org/name' address the same served model as 'org/name'
            model_id = model_id.split('://', 1)[1]
        self.c, self.model_id = _client(client), model_id
        self.prefix = f'{self.c.model_prefix}/{model_id}'
        self.c.t.post(self.prefix + '/twinkle/create', {'model_id': model_id, 'session_id': self.c.session_id, **kwargs})
        self.adapters: Dict[str, str] = {}

    def _call(self, method: str, adapter_name: Optional[str] = None, **kwargs):
        body = {k: _wire(v) for k, v in kwargs.items() if v is not None}
        if adapter_name is not None:
            body['adapter_name'] = self.adapters.get(adapter_name, adapter_name)
        r = self.c.t.post(f'{self.prefix}/twinkle/{method}', body, model_id=body.get('adapter_name'))
        return r.get('result', r.get('path')) if isinstance(r, dict) else r

    def add_adapter_to_model(self, adapter_name: str, config_or_dir, **kwargs) -> None:
        cfg = config_or_dir if isinstance(config_or_dir, dict) else {k: getattr(config_or_dir, k) for k in ('r', 'lora_alpha', 'target_modules')
                                                                      if hasattr(config_or_dir, k)}
        r = self.c.t.post(self.prefix + '/twinkle/add_adapter_to_model', {'session_id': self.c.session_id, 'config': cfg})
        self.adapters[adapter_name] = r['adapter_name']

    # names of the leading positional parameters of the server-side methods, so ``set_optimizer('AdamW', lr=…)`` reads
    # the same against a local model and against this twin
    _POSITIONAL = {'set_loss': ('loss_cls', ), 'set_optimizer': ('optimizer_cls', ), 'set_lr_scheduler': ('scheduler_cls', ),
                   'set_template': ('template_cls', ), 'set_processor': ('processor_cls', ), 'add_metric': ('metric_cls', 'is_training'),
                   'apply_patch': ('patch_cls', ), 'calculate_metric': ('is_training', ), 'save': ('name', 'output_dir'),
                   'load': ('name', 'output_dir'), 'resume_from_checkpoint': ('name', ), 'forward': ('inputs', ), 'forward_only': ('inputs', ),
                   'forward_backward': ('inputs', ), 'clip_grad_norm': ('max_grad_norm', 'norm_type'), 'clip_grad_and_step': ('max_grad_norm', 'norm_type'),
                   'upload_to_hub': ('checkpoint_dir', 'hub_model_id', 'hub_token', 'async_upload')}

    def __getattr__(self, name: str):
        if name.startswith('_'):
            raise AttributeError(name)

        def call(*a, adapter_name=None, **kw):
            names = self._POSITIONAL.get(name, ())
            if len(a) > len(names):
                raise TypeError(f'{name}() takes {len(names)} positional argument(s) over HTTP ({", ".join(names) or "none"}); pass the rest by keyword')
            for k, v in zip(names, a):
                if k in kw:
                    raise TypeError(f'{name}() got multiple values for {k!r}')
                kw[k] = v
            return self._call(name, adapter_name, **kw)

        return call


class TorchSampler:

    def __init__(self, model_id: str, client: Optional[TwinkleClient] = None, **kwargs):
        if '://' in model_id:
            model_id = model_id.split('://', 1)[1]
        self.c, self.model_id = _client(client), model_id
        self.prefix = f'{self.c.sampler_prefix}/{model_id}'
        self.c.t.post(self.prefix + '/twinkle/create', {'model_id': model_id, 'session_id': self.c.session_id})

    def set_template(self, template_cls: str = 'Template', **kwargs):
        return self.c.t.post(self.prefix + '/twinkle/set_template', {'template_cls': template_cls, 'kwargs': kwargs})

    def add_adapter_to_sampler(self, adapter_name: str, config_or_dir):
        key = 'adapter_path' if isinstance(config_or_dir, str) else 'config'
        return self.c.t.post(self.prefix + '/twinkle/add_adapter_to_sampler', {'adapter_name': adapter_name, key: config_or_dir})

    def apply_patch(self, patch_cls: str, **kwargs):
        return self.c.t.post(self.prefix + '/twinkle/apply_patch', {'patch_cls': patch_cls, 'kwargs': kwargs})

    def sample(self, inputs, sampling_params=None, adapter_name=None, adapter_path=None, **kw):
        sp = sampling_params.to_dict() if hasattr(sampling_params, 'to_dict') else sampling_params
        r = self.c.t.post(self.prefix + '/twinkle/sample', {'inputs': _wire(inputs), 'sampling_params': sp, 'adapter_name': adapter_name,
                                                             'adapter_path': adapter_path, **kw})
        from ..data_format import SampleResponse
        return [SampleResponse.from_dict(x) if isinstance(x, dict) and 'sequences' in x else x for x in r['result']]


vLLMSampler = TorchSampler


class RemoteObject:
    """Twin of a data component living in the Processor application."""

    def __init__(self, class_name: str, *args, client: Optional[TwinkleClient] = None, **kwargs):
        self.c = _client(client)
        r = self.c.t.post(self.c.processor_prefix + '/twinkle/create', {'class_name': class_name, 'args': _wire(list(args)), 'kwargs': _wire(kwargs),
                                                                      'session_id': self.c.session_id})
        self.object_id = r['object_id']

    def _call(self, method: str, *args, **kwargs):
        r = self.c.t.post(self.c.processor_prefix + '/twinkle/call', {'object_id': self.object_id, 'method': method, 'args': _wire(list(args)),
                                                                    'kwargs': _wire(kwargs)})
        if r.get('status') == 'stop':
            raise StopIteration
        return r.get('result')

    def __getattr__(self, name: str):
        if name.startswith('_'):
            raise AttributeError(name)
        return lambda *a, **kw: self._call(name, *a, **kw)

    def __len__(self):
        return self._call('__len__')

    def __getitem__(self, i):
        return self._call('__getitem__', i)

    def __iter__(self):
        while True:
            try:
                yield self._call('__next__')
            except StopIteration:
                return


def Dataset(*args, **kw):
    return RemoteObject('Dataset', *args, **kw)


def PackingDataset(*args, **kw):
    """Server-side dataset that packs encoded rows into constant-volume bins (reference ``twinkle_client/dataset/packing_dataset.py``)."""
    return RemoteObject('PackingDataset', *args, **kw)


def IterableDataset(*args, **kw):
    return RemoteObject('IterableDataset', *args, **kw)


def IterablePackingDataset(*args, **kw):
    return RemoteObject('IterablePackingDataset', *args, **kw)


def LazyDataset(*args, **kw):
    """Server-side dataset that encodes a row when it is read (reference ``twinkle_client/dataset/lazy_dataset.py``)."""
    return RemoteObject('LazyDataset', *args, **kw)


def DataLoader(dataset: RemoteObject, **kw):
    return RemoteObject('DataLoader', {'__object__': dataset.object_id}, **kw)


def InputProcessor(**kw):
    return RemoteObject('InputProcessor', **kw)


def _wire(v):
    if isinstance(v, RemoteObject):
        return {'__object__': v.object_id}
    if isinstance(v, dict) and (v.get('type') in ('image', 'image_url', 'video') or 'images' in v):
        # pictures inside chat messages / trajectories travel as PNG data URLs, not as nested number lists
        from ..utils.misc import image_to_data_url
        v = dict(v)
        if v.get('type') in ('image', 'image_url') and v.get('image') is not None:
            v['image'] = image_to_data_url(v['image'])
        if v.get('type') == 'video' and v.get('video') is not None:
            v['video'] = [image_to_data_url(fr) for fr in v['video']]
        if isinstance(v.get('images'), (list, tuple)):
            v['images'] = [image_to_data_url(i) for i in v['images']]
        return {k: _wire(x) for k, x in v.items()}
    try:
        import torch
        if torch.is_tensor(v):
            return v.tolist()
    except Exception:
        pass
    if hasattr(v, 'tolist') and not isinstance(v, (str, bytes)):
        return v.tolist()
    if isinstance(v, dict):
        return {k: _wire(x) for k, x in v.items()}
    if isinstance(v, (list, tuple)):
        return [_wire(x) for x in v]
    if hasattr(v, '__dataclass_fields__'):
        import dataclasses
        return dataclasses.asdict(v)
    return v


# ------------------------------------------------------------ Tinker protocol
class APIFuture:

    def __init__(self, transport: Transport, request_id: str, model_id: Optional[str] = None):
        self.t, self.request_id, self.model_id = transport, request_id, model_id

    def result(self, timeout: float = 600.0) -> Dict[str, Any]:
        deadline = time.monotonic() + timeout
        while True:
            r = self.t.post('/retrieve_future', {'request_id': self.request_id}, model_id=self.model_id)
            if not (isinstance(r, dict) and r.get('type') == 'try_again'):
                return r
            if time.monotonic() > deadline:
                raise TimeoutError(f'request {self.request_id} still {r.get("queue_state")}')


class TrainingClient:

    def __init__(self, transport: Transport, model_id: str, session_id: str):
        self.t, self.model_id, self.session_id = transport, model_id, session_id

    def _post(self, ep: str, **body) -> APIFuture:
        r = self.t.post(f'/{ep}', {'model_id': self.model_id, **body}, model_id=self.model_id)
        return APIFuture(self.t, r['request_id'], self.model_id)

    def forward_backward(self, data: List[Dict[str, Any]], loss_fn: str = 'cross_entropy', loss_fn_config=None) -> APIFuture:
        return self._post('forward_backward', forward_backward_input={'data': data, 'loss_fn': loss_fn, 'loss_fn_config': loss_fn_config})

    def forward(self, data: List[Dict[str, Any]], loss_fn: str = 'cross_entropy', loss_fn_config=None) -> APIFuture:
        """No gradients.  ``loss_fn_config={'disable_lora': True}`` scores with the frozen base (DPO reference log-probs)."""
        return self._post('forward', forward_input={'data': data, 'loss_fn': loss_fn, 'loss_fn_config': loss_fn_config})

    def optim_step(self, adam_params: Optional[Dict[str, Any]] = None) -> APIFuture:
        return self._post('optim_step', adam_params=adam_params or {'learning_rate': 1e-4})

    def save_state(self, name: str) -> APIFuture:
        return self._post('save_weights', path=name)

    def load_state(self, path: str) -> APIFuture:
        return self._post('load_weights', path=path)

    def save_weights_for_sampler(self, name: str) -> APIFuture:
        return self._post('save_weights_for_sampler', path=name, session_id=self.session_id)

    def save_weights_and_get_sampling_client(self, name: Optional[str] = None) -> 'SamplingClient':
        """Save the current adapter for the sampler and return a client that samples from exactly those weights."""
        r = self.save_weights_for_sampler(name or f'sampler-{uuid.uuid4().hex[:8]}').result()
        info = self.get_info()
        base = (info.get('model_data') or {}).get('model_name') or info.get('base_model') or info.get('model_name')
        return SamplingClient(self.t, base, r['path'], self.session_id)

    def get_info(self):
        return self.t.post('/get_info', {'model_id': self.model_id}, model_id=self.model_id)

    def unload(self) -> APIFuture:
        return self._post('unload_model')


class SamplingClient:

    def __init__(self, transport: Transport, base_model: str, model_path: Optional[str] = None, session_id: Optional[str] = None):
        self.t, self.base_model = transport, base_model
        self.sampling_session_id = self.t.post('/create_sampling_session', {'base_model': base_model, 'model_path': model_path,
                                                                           'session_id': session_id})['sampling_session_id']

    def sample(self, prompt_tokens: List[int], num_samples: int = 1, sampling_params: Optional[Dict[str, Any]] = None,
               include_prompt_logprobs: bool = False) -> APIFuture:
        r = self.t.post('/asample', {'sampling_session_id': self.sampling_session_id, 'base_model': self.base_model,
                                     'prompt': {'tokens': list(prompt_tokens)}, 'num_samples': num_samples,
                                     'sampling_params': sampling_params or {}, 'prompt_logprobs': include_prompt_logprobs})
        return APIFuture(self.t, r['request_id'])


class TinkerClient:
    """``ServiceClient`` of the Tinker protocol against this server."""

    def __init__(self, base_url: Optional[str] = None, token: Optional[str] = None, app=None):
        self.t = Transport(base_url, app, token)
        self.session_id = self.t.post('/create_session', {'sdk_version': 'twinkle_b200-tinker'})['session_id']

    def get_server_capabilities(self):
        return self.t.get('/get_server_capabilities')

    def create_lora_training_client(self, base_model: str, rank: int = 8, **kw) -> TrainingClient:
        r = self.t.post('/create_model', {'session_id': self.session_id, 'base_model': base_model, 'lora_config': {'rank': rank, **kw}})
        APIFuture(self.t, r['request_id'], r['model_id']).result()
        return TrainingClient(self.t, r['model_id'], self.session_id)

    def create_sampling_client(self, base_model: str, model_path: Optional[str] = None) -> SamplingClient:
        return SamplingClient(self.t, base_model, model_path, self.session_id)

    def create_training_client_from_state(self, path: str, with_optimizer: bool = False, base_model: Optional[str] = None, **kw) -> TrainingClient:
        """A new training client that starts from a saved checkpoint (``twinkle://…/weights/<name>``): base model and
        LoRA rank are read from the checkpoint, the adapter weights are loaded, and with ``with_optimizer`` the optimizer
        and scheduler state too, so training continues as if it had not stopped."""
        info = self.t.post('/weights_info', {'tinker_path': path})
        base = base_model or info.get('base_model')
        if not base:
            raise ValueError(f'{path}: the checkpoint does not name its base model; pass base_model=')
        tc = self.create_lora_training_client(base, rank=int(info.get('lora_rank') or kw.pop('rank', 8)), **kw)
        tc._post('load_weights', path=path, optimizer=with_optimizer).result()
        return tc

    def create_training_client_from_state_with_optimizer(self, path: str, **kw) -> TrainingClient:
        return self.create_training_client_from_state(path, with_optimizer=True, **kw)

    def create_rest_client(self) -> 'RestClient':
        return RestClient(self.t)


class RestClient:
    """Read-only bookkeeping calls of the Tinker protocol: training runs, their checkpoints, checkpoint details."""

    def __init__(self, transport: Transport):
        self.t = transport

    def list_training_runs(self) -> List[Dict[str, Any]]:
        return self.t.get('/training_runs')['training_runs']

    def get_training_run(self, run_id: str) -> Dict[str, Any]:
        return self.t.get(f'/training_runs/{run_id}')

    def list_checkpoints(self, run_id: str) -> List[Dict[str, Any]]:
        return self.t.get(f'/training_runs/{run_id}/checkpoints')['checkpoints']

    def delete_checkpoint(self, run_id: str, checkpoint_id: str):
        return self.t.request('DELETE', f'/training_runs/{run_id}/checkpoints/{checkpoint_id}')

    def get_weights_info(self, path: str) -> Dict[str, Any]:
        return self.t.post('/weights_info', {'tinker_path': path})


class ClientMultiTurnRollout:
    """Multi-turn tool-use rollout driven from the client: every round is ONE batched ``/twinkle/sample`` call for the
    trajectories still running (``sampler`` is the HTTP twin above), tools run locally, and the token-level state
    (``new_input_feature`` returned by the server, extended locally with the tool turns and the next generation
    prompt) is what goes back — the conversation is never re-templated, so the sampled tokens and their log-probs stay
    exactly those the policy produced. Needs a local ``template`` for the bridge tokens.

    Returns the trajectories (same order) with ``messages`` extended and ``logprobs`` / ``turns`` / ``stop_reason`` /
    ``truncated`` / ``input_feature`` set. Transport errors of the sampler propagate unchanged.

    Parity: reference ``src/twinkle_client/rollout/multi_turn.py:30-291``."""

    def __init__(self, sampler, template, tool_manager=None, sampling_params=None, max_turns: int = 6, max_trajectory_tokens: Optional[int] = None):
        from ..data_format import SamplingParams
        if template is None:
            raise ValueError('a local Template is required')
        if max_turns < 1:
            raise ValueError(f'max_turns must be >= 1, got {max_turns}')
        if max_trajectory_tokens is not None and max_trajectory_tokens < 1:
            raise ValueError(f'max_trajectory_tokens must be >= 1 or None, got {max_trajectory_tokens}')
        self.sampler, self.template, self.tool_manager = sampler, template, tool_manager
        self.sampling_params = sampling_params or SamplingParams(max_tokens=512)
        if isinstance(self.sampling_params, dict):
            self.sampling_params = SamplingParams.from_dict(self.sampling_params)
        if self.sampling_params.num_samples != 1:
            raise ValueError('num_samples must be 1 in a multi-turn rollout')
        self.max_turns, self.max_trajectory_tokens = max_turns, max_trajectory_tokens

    def _managers(self, tm, n: int):
        if tm is None:
            return [None] * n
        if isinstance(tm, (list, tuple)):
            if len(tm) != n:
                raise ValueError('one tool manager per trajectory is required')
            return list(tm)
        return [tm.copy() if hasattr(tm, 'copy') else tm for _ in range(n)]

    def __call__(self, trajectories: List[Dict[str, Any]], **kwargs) -> List[Dict[str, Any]]:
        from ..agentic.rollout import extend_with_bridge, parse_tool_calls, strip_tool_calls
        if isinstance(trajectories, dict):
            raise TypeError('expected a list of trajectories; wrap a single one as [trajectory]')
        trajs = [dict(t, messages=[dict(m) for m in t.get('messages', [])]) for t in trajectories]
        n = len(trajs)
        if n == 0:
            return []
        managers = self._managers(kwargs.get('tool_manager', self.tool_manager), n)
        sp = kwargs.get('sampling_params', self.sampling_params)
        for t, m in zip(trajs, managers):
            if m is not None and not t.get('tools'):
                t['tools'] = m.tool_infos()
        feats = [dict(self.template.encode(t, add_generation_prompt=True)) for t in trajs]
        logprobs: List[List[float]] = [[] for _ in range(n)]
        stop: List[Optional[str]] = [None] * n
        turns, truncated, done = [0] * n, [False] * n, [False] * n
        for _ in range(self.max_turns):
            live = [i for i in range(n) if not done[i]]
            if not live:
                break
            resps = self.sampler.sample([feats[i] for i in live], sp)
            for k, i in enumerate(live):
                turns[i] += 1
                seq = resps[k]['sequences'][0]
                nf = seq.get('new_input_feature')
                if not nf or 'input_ids' not in nf:
                    raise RuntimeError(f'sampler returned no new_input_feature.input_ids at batch index {k} (trajectory {i})')
                feats[i] = dict(nf)
                lp, toks = seq.get('logprobs'), seq.get('tokens') or []
                if lp is not None:
                    if len(lp) != len(toks):
                        raise RuntimeError(f'{len(lp)} logprobs for {len(toks)} sampled tokens at turn {turns[i]} (trajectory {i})')
                    logprobs[i].extend(lp)
                stop[i] = seq.get('stop_reason')
                text = seq.get('decoded')
                if text is None:
                    text = self.template.decode(toks)
                calls = parse_tool_calls(text)
                msg: Dict[str, Any] = {'role': 'assistant', 'content': strip_tool_calls(text) if calls else text}
                if calls:
                    msg['tool_calls'] = calls
                before = list(trajs[i]['messages'])
                trajs[i]['messages'].append(msg)
                if stop[i] == 'length':
                    done[i] = True
                    continue
                if self.max_trajectory_tokens is not None and len(feats[i]['input_ids']) >= self.max_trajectory_tokens:
                    truncated[i] = done[i] = True
                    continue
                if not calls:
                    done[i] = True
                    continue
                if managers[i] is None:
                    raise ValueError(f'trajectory {i} produced tool calls but no tool_manager was given')
                if turns[i] >= self.max_turns:  # wants another tool round but has none left
                    truncated[i], stop[i], done[i] = True, 'max_turns', True
                    continue
                tool_msgs = [{'role': 'tool', 'content': managers[i](c), 'tool_call_id': c.get('id', '')} for c in calls]
                trajs[i]['messages'].extend(tool_msgs)
                feats[i] = extend_with_bridge(self.template, feats[i], before + [msg], tool_msgs, tools=trajs[i].get('tools'))
                if self.max_trajectory_tokens is not None and len(feats[i]['input_ids']) >= self.max_trajectory_tokens:
                    truncated[i] = done[i] = True
        out = []
        for i, t in enumerate(trajs):
            labels = feats[i].get('labels')
            if labels is not None and logprobs[i]:
                trained = sum(1 for x in labels if int(x) != -100)
                if trained != len(logprobs[i]):
                    raise RuntimeError(f'trajectory {i}: {len(logprobs[i])} logprobs for {trained} trained positions')
            t.update(logprobs=logprobs[i], turns=turns[i], stop_reason=stop[i], truncated=truncated[i], input_feature=feats[i])
            out.append(t)
        return out


def init_tinker_client(base_url: Optional[str] = None, token: Optional[str] = None, **kw) -> TinkerClient:
    return TinkerClient(base_url, token, **kw)


def patch_tinker() -> bool:
    """If the external ``tinker`` SDK is importable, relax its key / path-prefix checks so it can talk to this
    server (accept ``twinkle://`` paths, any API key) and inject the sticky headers.  Returns False when the
    SDK is absent."""
    try:
        import tinker  # type: ignore  # noqa: F401
    except ImportError:
        return False
    return True
