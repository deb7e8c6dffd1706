"""The four HTTP applications: Gateway, Model, Sampler, Processor.

Parity: reference ``src/twinkle/server/{gateway,model,sampler,processor}/`` and ``server/deployment.py`` —
the same route set as the reference's frozen HTTP contract (``tests/server/contract/
client_api_baseline.json``): Tinker-public routes on the gateway root, native routes under ``/twinkle``,
OpenAI-compatible ``/chat/completions`` + ``/models``; compute routes of the Tinker family return
``{request_id, model_id}`` at once and complete through ``/retrieve_future`` long-polling
(``TWINKLE_LONG_POLL_TIMEOUT`` 30 s, ``TWINKLE_POLL_INTERVAL`` 0.5 s, ``{'type': 'try_again'}`` while
pending); native routes block.  Middleware order: replica-id header → metrics → tracing → token check
(``Twinkle-Authorization`` or ``Authorization: Bearer``; ``x-request-id`` mandatory on compute routes) →
exception boundary → handler.  The reference hosts each app as a Ray Serve deployment and proxies over
httpx; here the apps are FastAPI sub-applications of one process and the gateway calls the model / sampler
apps in-process (an httpx transport is used when they are mounted elsewhere).
"""
from __future__ import annotations

import asyncio
import json
import os
import time
import uuid
from typing import Any, Dict, List, Optional

from fastapi import FastAPI, HTTPException, Request
from fastapi.responses import JSONResponse, PlainTextResponse, StreamingResponse

from ..backends import BackendSelector
from ..checkpoint import CheckpointManager
from ...client.types import validate_request
from ..exceptions import TwinkleServerError, status_code_of
from ..queue import PreflightError, TaskQueueMixin
from ..state import ServerState
from ..telemetry import get_registry, get_tracer

LONG_POLL = lambda: float(os.environ.get('TWINKLE_LONG_POLL_TIMEOUT', '30'))
POLL_INTERVAL = lambda: float(os.environ.get('TWINKLE_POLL_INTERVAL', '0.5'))


def get_token(request: Request) -> str:
    t = request.headers.get('Twinkle-Authorization') or request.headers.get('Authorization') or request.headers.get('X-API-Key') or ''
    if t.lower().startswith('bearer '):
        t = t[7:]
    return t.strip() or 'anonymous'


def is_token_valid(token: str) -> bool:
    """Authentication stub (the reference accepts every token as well)."""
    return True


def install_middleware(app: FastAPI, name: str, replica_id: str, require_request_id: bool = False) -> None:
    reg, tracer = get_registry(), get_tracer()

    @app.middleware('http')
    async def pipeline(request: Request, call_next):
        start = time.monotonic()
        path = request.url.path
        token = get_token(request)
        request.state.token = token
        request.state.request_id = request.headers.get('x-request-id') or uuid.uuid4().hex
        status = 500
        try:
            with tracer.span(f'{request.method} {path}', parent=request.headers.get('traceparent'), app=name, replica_id=replica_id):
                if not is_token_valid(token):
                    resp = JSONResponse({'detail': 'invalid token'}, status_code=401)
                elif require_request_id and request.method == 'POST' and not request.headers.get('x-request-id') and '/tinker/' in path:
                    resp = JSONResponse({'detail': 'x-request-id header is required'}, status_code=400)
                else:
                    try:
                        resp = await call_next(request)
                    except PreflightError as e:
                        resp = JSONResponse({'detail': str(e)}, status_code=e.status_code)
                    except HTTPException as e:
                        resp = JSONResponse({'detail': e.detail}, status_code=e.status_code)
                    except (TwinkleServerError, KeyError, ValueError, PermissionError, FileNotFoundError) as e:
                        resp = JSONResponse({'detail': f'{type(e).__name__}: {e}'}, status_code=status_code_of(e))
                    except Exception as e:  # exception boundary: never leak a traceback, always answer
                        resp = JSONResponse({'detail': f'internal error: {type(e).__name__}: {e}'}, status_code=500)
                status = resp.status_code
        finally:
            reg.inc('twinkle_http_requests_total', app=name, path=path, status=status)
            reg.observe('twinkle_http_request_seconds', time.monotonic() - start, app=name)
        resp.headers['x-replica-id'] = replica_id
        return resp


async def body_of(request: Request) -> Dict[str, Any]:
    try:
        b = await request.json()
        return b if isinstance(b, dict) else {'value': b}
    except Exception:
        return {}


# =============================================================== Model app
class ModelApp(TaskQueueMixin):

    def __init__(self, args, state: ServerState, queue_cfg, checkpoints: CheckpointManager, name: str = 'model',
                 remote_group: Optional[str] = None):
        """``remote_group``: name of the worker-pool device group that hosts the backend (one worker per rank of the
        application's ``device_group``); ``None`` keeps the backend inside the server process."""
        self.args, self.checkpoints, self.name = args, checkpoints, name
        self.replica_id = f'{name}-{uuid.uuid4().hex[:8]}'
        self._init_task_queue(state, args.queue_config or queue_cfg, get_registry())
        kw = dict(model_id=args.model_id, max_loras=args.max_loras)
        if args.backend != 'mock':
            kw.update(device_mesh=args.device_mesh.build(), max_r=args.max_r, max_length=args.max_length)
            if remote_group is not None:
                kw['remote_group'] = remote_group
        self.backend = BackendSelector.model(args.backend, **kw)
        self.adapters: Dict[str, Dict[str, Any]] = {}  # model_id → {adapter, token, session, created, last_used}
        self.uploads: Dict[str, str] = {}
        self.app = FastAPI(title='twinkle-model')
        install_middleware(self.app, name, self.replica_id, require_request_id=True)
        self._routes()
        state.register_replica(self.replica_id, args.model_id, args.max_loras, 0)

    # ---------------------------------------------------------- adapters
    def adapter_of(self, model_id: str, token: str) -> str:
        a = self.adapters.get(model_id)
        if a is None:
            raise KeyError(f'model {model_id!r} is not loaded on this replica')
        if a['token'] != token:
            raise PermissionError('model belongs to another token')
        a['last_used'] = time.time()
        return a['adapter']

    def create_adapter(self, token: str, session_id: Optional[str], lora_config: Optional[Dict[str, Any]], model_id: Optional[str] = None,
                       save_dir: Optional[str] = None, user_metadata: Optional[Dict[str, Any]] = None) -> str:
        model_id = model_id or uuid.uuid4().hex
        if model_id in self.adapters:  # a client-chosen id must not take over another tenant's (or its own live) entry
            raise HTTPException(409, f'model {model_id!r} already exists on this replica')
        adapter = f'{session_id or "nosession"}-{model_id[:12]}'
        cfg = dict(self.args.adapter_config or {})
        cfg.update({k: v for k, v in (lora_config or {}).items() if v is not None})
        if 'rank' in cfg:
            cfg['r'] = cfg.pop('rank')
        cfg.setdefault('r', 8)
        cfg.setdefault('lora_alpha', cfg.get('alpha', 2 * cfg['r']))
        cfg.pop('alpha', None)
        self.state.register_model(model_id, token, self.args.model_id, session_id, self.replica_id)
        try:
            self.backend.add_adapter_to_model(adapter, {k: v for k, v in cfg.items() if k in ('r', 'lora_alpha', 'target_modules', 'use_rslora')})
        except Exception:
            self.state.unregister_model(model_id)
            raise
        self.adapters[model_id] = {'adapter': adapter, 'token': token, 'session_id': session_id, 'created': time.time(), 'last_used': time.time(),
                                   'lora_config': cfg}
        self.state.register_replica(self.replica_id, self.args.model_id, self.args.max_loras, len(self.adapters))
        self.checkpoints.create_run(token, model_id, self.args.model_id, lora_config={**cfg, 'rank': cfg['r']}, is_lora=True,
                                    save_dir=save_dir, user_metadata=user_metadata)
        return model_id

    def unload(self, model_id: str) -> None:
        a = self.adapters.pop(model_id, None)
        if a:
            self.backend.remove_adapter(a['adapter'])
        self.state.unregister_model(model_id)
        self.state.register_replica(self.replica_id, self.args.model_id, self.args.max_loras, len(self.adapters))

    def expire_adapters(self) -> List[str]:
        """Drop adapters whose session stopped heart-beating or that outlived ``adapter_max_lifetime``."""
        now, gone = time.time(), []
        for mid, a in list(self.adapters.items()):
            age = self.state.session_age(a['session_id']) if a['session_id'] else None
            stale = (age is None and a['session_id'] is not None) or (age is not None and age > self.args.adapter_timeout)
            if stale or now - a['created'] > self.args.adapter_max_lifetime:
                self.unload(mid)
                gone.append(mid)
        return gone

    # ------------------------------------------------------------ routes
    def _routes(self) -> None:
        app = self.app

        @app.get('/healthz')
        async def healthz():
            try:  # with a worker group behind the backend this is a round trip to every worker
                ok = bool(self.backend.ping())
            except Exception:
                ok = False
            return JSONResponse({'status': 'ok' if ok else 'unhealthy', 'replica_id': self.replica_id, 'queue_depth': self.worker.depth(),
                                 'adapters': len(self.adapters)}, status_code=200 if ok else 503)

        @app.post('/tinker/create_model')
        async def create_model(request: Request):
            b = await body_of(request)
            token = request.state.token
            mid = b.get('model_id') or uuid.uuid4().hex
            if mid in self.adapters:
                raise HTTPException(409, f'model {mid!r} already exists on this replica')

            def work():
                self.create_adapter(token, b.get('session_id'), b.get('lora_config'), mid, b.get('save_dir'), b.get('user_metadata'))
                return {'model_id': mid, 'type': 'create_model'}

            return self.schedule_task(work, token=token, model_id=mid, request_id=request.state.request_id)

        @app.post('/tinker/get_info')
        async def get_info(request: Request):
            b = await body_of(request)
            a = self.adapters.get(b.get('model_id', ''))
            if a is None:
                raise HTTPException(404, 'unknown model')
            self.adapter_of(b['model_id'], request.state.token)
            return {'model_id': b['model_id'], 'model_data': {'model_name': self.args.model_id, 'arch': 'decoder'}, 'is_lora': True,
                    'lora_rank': a['lora_config'].get('r')}

        @app.post('/tinker/unload_model')
        async def unload_model(request: Request):
            b = await body_of(request)
            token, mid = request.state.token, b.get('model_id', '')
            self.adapter_of(mid, token)
            return self.schedule_task(lambda: (self.unload(mid), {'model_id': mid, 'type': 'unload_model'})[1], token=token, model_id=mid,
                                      request_id=request.state.request_id)

        def _fb(backward: bool):
            async def handler(request: Request):
                b = await body_of(request)
                token, mid = request.state.token, b.get('model_id', '')
                adapter = self.adapter_of(mid, token)
                inp = b.get('forward_backward_input') or b.get('forward_input') or b
                datums = inp.get('data') or []
                loss_fn = inp.get('loss_fn', 'cross_entropy')
                n_tok = sum(len((d.get('model_input') or {}).get('tokens', []) or [t for c in (d.get('model_input') or {}).get('chunks', [])
                                                                                     for t in c.get('tokens', [])]) for d in datums)
                dws = self.backend.data_world_size()
                return self.schedule_task(lambda: self.backend.tinker_forward_backward(datums, adapter, loss_fn, backward, inp.get('loss_fn_config')),
                                          token=token, model_id=mid, input_tokens=n_tok, batch_size=len(datums), data_world_size=dws,
                                          request_id=request.state.request_id)
            return handler

        app.post('/tinker/forward_backward')(_fb(True))
        app.post('/tinker/forward')(_fb(False))

        @app.post('/tinker/optim_step')
        async def optim_step(request: Request):
            b = await body_of(request)
            token, mid = request.state.token, b.get('model_id', '')
            adapter = self.adapter_of(mid, token)
            return self.schedule_task(lambda: self.backend.tinker_step(adapter, b.get('adam_params')), token=token, model_id=mid,
                                      request_id=request.state.request_id)

        def _save(kind: str):
            async def handler(request: Request):
                b = await body_of(request)
                token, mid = request.state.token, b.get('model_id', '')
                adapter = self.adapter_of(mid, token)
                name = b.get('path') or b.get('name') or f'ckpt-{int(time.time())}'

                def work():
                    out_dir = os.path.dirname(self.checkpoints.path_for(token, mid, name, kind))
                    self.backend.save(name, out_dir, adapter_name=adapter, save_optimizer=(kind == 'weights'))
                    meta = self.checkpoints.register(token, mid, name, kind, base_model=self.args.model_id)
                    res = {'path': meta['path'], 'type': 'save_weights' if kind == 'weights' else 'save_weights_for_sampler'}
                    if kind == 'sampler_weights':
                        res['sampling_session_id'] = self.state.create_sampling_session(token, self.args.model_id, meta['path'], b.get('session_id'))
                    return res

                return self.schedule_task(work, token=token, model_id=mid, request_id=request.state.request_id)
            return handler

        app.post('/tinker/save_weights')(_save('weights'))
        app.post('/tinker/save_weights_for_sampler')(_save('sampler_weights'))

        @app.post('/tinker/load_weights')
        async def load_weights(request: Request):
            b = await body_of(request)
            token, mid = request.state.token, b.get('model_id', '')
            adapter = self.adapter_of(mid, token)
            path = self.checkpoints.resolve_load_path(token, b.get('path', ''))
            return self.schedule_task(lambda: (self.backend.load(None, path, adapter_name=adapter, load_optimizer=b.get('optimizer', True)),
                                               {'path': b.get('path'), 'type': 'load_weights'})[1], token=token, model_id=mid,
                                      request_id=request.state.request_id)

        # ------------------------------------------------ native (blocking) routes
        @app.post('/twinkle/create')
        async def tw_create(request: Request):
            b = await body_of(request)
            return {'status': 'ok', 'model_id': self.args.model_id, 'replica_id': self.replica_id, 'max_loras': self.args.max_loras}

        @app.post('/twinkle/add_adapter_to_model')
        async def tw_add_adapter(request: Request):
            b = await body_of(request)
            token = request.state.token
            mid = await self.schedule_task_and_wait(lambda: self.create_adapter(token, b.get('session_id'), b.get('config') or b.get('lora_config'),
                                                                               b.get('adapter_name'), b.get('save_dir'), b.get('user_metadata')),
                                                    token=token)
            return {'status': 'ok', 'adapter_name': mid}

        generic = ['forward', 'forward_only', 'calculate_loss', 'backward', 'forward_backward', 'clip_grad_norm', 'step', 'zero_grad', 'lr_step',
                   'clip_grad_and_step', 'get_train_configs', 'set_loss', 'set_optimizer', 'set_lr_scheduler',
                   'apply_patch', 'add_metric', 'set_template', 'set_processor', 'calculate_metric', 'get_state_dict']

        def _generic(method: str):
            async def handler(request: Request):
                b = await body_of(request)
                token = request.state.token
                validate_request(method, b, aliases={'model_id': 'adapter_name'})  # a missing field is a 400 naming it
                name = b.pop('adapter_name', None) or b.pop('model_id', None)
                b.pop('model_id', None)
                # every named adapter resolves through the ownership table: an unknown name is a 404, another token's a
                # 403 — the backend's internal adapter names are never accepted from a client
                adapter = self.adapter_of(name, token) if name else None
                kwargs = {k: v for k, v in b.items() if k not in ('session_id', )}
                n_inputs = len(kwargs.get('inputs') or []) if isinstance(kwargs.get('inputs'), list) else None
                res = await self.schedule_task_and_wait(lambda: self.backend.generic_call(method, adapter_name=adapter, **kwargs), token=token,
                                                        model_id=name or '', batch_size=n_inputs if method.startswith('forward') else None,
                                                        data_world_size=self.backend.data_world_size())
                return {'status': 'ok', 'result': res}
            return handler

        for m in generic:
            app.post(f'/twinkle/{m}')(_generic(m))

        @app.post('/twinkle/save')
        async def tw_save(request: Request):
            b = await body_of(request)
            token, name = request.state.token, b.get('adapter_name') or b.get('model_id')
            adapter = self.adapter_of(name, token)
            ck = b.get('name') or f'ckpt-{int(time.time())}'

            def work():
                out_dir = os.path.dirname(self.checkpoints.path_for(token, name, ck, 'weights'))
                self.backend.save(ck, out_dir, adapter_name=adapter, save_optimizer=b.get('save_optimizer', False))
                return self.checkpoints.register(token, name, ck, 'weights', base_model=self.args.model_id)['path']

            return {'status': 'ok', 'path': await self.schedule_task_and_wait(work, token=token, model_id=name)}

        @app.post('/twinkle/load')
        async def tw_load(request: Request):
            b = await body_of(request)
            token, name = request.state.token, b.get('adapter_name') or b.get('model_id')
            adapter = self.adapter_of(name, token)
            path = self.checkpoints.resolve_load_path(token, b.get('path') or b.get('name', ''))
            await self.schedule_task_and_wait(lambda: self.backend.load(None, path, adapter_name=adapter), token=token, model_id=name)
            return {'status': 'ok'}

        @app.post('/twinkle/resume_from_checkpoint')
        async def tw_resume(request: Request):
            """Weights + optimizer / scheduler / RNG / progress counters of a checkpoint this token saved.  The body names
            it as ``name`` (the field of the request record) or ``checkpoint_dir``; a ``twinkle://`` path returned by
            ``save`` resolves to the token's own directory (reference ``server/model/twinkle_handlers.py`` resume route)."""
            b = await body_of(request)
            token, name = request.state.token, b.get('adapter_name') or b.get('model_id')
            ck = b.get('name') or b.get('checkpoint_dir')
            if not ck:
                raise HTTPException(400, "resume_from_checkpoint needs 'name' (or 'checkpoint_dir')")
            adapter = self.adapter_of(name, token) if name else None
            path = self.checkpoints.resolve_load_path(token, ck)
            res = await self.schedule_task_and_wait(lambda: self.backend.generic_call('resume_from_checkpoint', checkpoint_dir=path, adapter_name=adapter,
                                                                                      resume_only_model=bool(b.get('resume_only_model', False))),
                                                    token=token, model_id=name or '')
            return {'status': 'ok', 'result': res}

        @app.post('/twinkle/upload_to_hub')
        async def tw_upload(request: Request):
            b = await body_of(request)
            token = request.state.token
            path = self.checkpoints.resolve_load_path(token, b.get('checkpoint_dir') or b.get('path', ''))

            def work():
                from ...hub import HubOperation
                return str(HubOperation.push_to_hub(b['hub_model_id'], path, token=b.get('hub_token')))

            rid = self.schedule_background_task(work, 'upload_to_hub')
            return {'status': 'ok', 'request_id': rid}

        @app.get('/twinkle/upload_status/{request_id}')
        async def tw_upload_status(request_id: str):
            f = self.state.get_future(request_id)
            if f is None:
                raise HTTPException(404, 'unknown upload')
            return {'status': f['status'], 'error': f.get('error')}


# ============================================================= Sampler app
class SamplerApp(TaskQueueMixin):

    def __init__(self, args, state: ServerState, queue_cfg, checkpoints: CheckpointManager, name: str = 'sampler',
                 remote_group: Optional[str] = None):
        self.args, self.checkpoints, self.name = args, checkpoints, name
        self.replica_id = f'{name}-{uuid.uuid4().hex[:8]}'
        self._init_task_queue(state, args.queue_config or queue_cfg, get_registry())
        kw: Dict[str, Any] = dict(model_id=args.model_id)
        if args.sampler_type != 'mock':
            kw.update(engine_args=args.engine_args, max_loras=args.max_loras)
            if remote_group is not None:
                kw.update(remote_group=remote_group, device_mesh=args.device_mesh.build())
        self.backend = BackendSelector.sampler(args.sampler_type, **kw)
        self.app = FastAPI(title='twinkle-sampler')
        install_middleware(self.app, name, self.replica_id, require_request_id=True)
        self._routes()

    def _adapter_path(self, token: str, b: Dict[str, Any]) -> Optional[str]:
        path = b.get('model_path') or b.get('adapter_path')
        sid = b.get('sampling_session_id')
        if not path and sid:
            s = self.state.get_sampling_session(sid)
            if s is None:
                raise KeyError(f'unknown sampling session {sid}')
            path = s.get('model_path')
        return self.checkpoints.resolve_load_path(token, path) if path else None

    @staticmethod
    def _to_wire(responses) -> List[Dict[str, Any]]:
        out = []
        for r in responses:
            out.append({'sequences': [{'stop_reason': s.stop_reason, 'tokens': s.tokens, 'logprobs': s.logprobs, 'decoded': s.decoded,
                                       'new_input_feature': s.new_input_feature} for s in r.sequences],
                        'prompt_logprobs': r.prompt_logprobs, 'topk_prompt_logprobs': r.topk_prompt_logprobs})
        return out

    def _routes(self) -> None:
        app = self.app

        @app.post('/tinker/asample')
        async def asample(request: Request):
            b = await body_of(request)
            token = request.state.token
            prompt = b.get('prompt') or {}
            ids = prompt.get('tokens') or [t for c in prompt.get('chunks', []) for t in c.get('tokens', [])]
            sp = dict(b.get('sampling_params') or {})
            sp['num_samples'] = b.get('num_samples', sp.get('num_samples', 1))
            if b.get('prompt_logprobs'):
                sp['prompt_logprobs'] = sp.get('prompt_logprobs', 0)
            path = self._adapter_path(token, b)

            def work():
                res = self.backend.sample([{'input_ids': ids}], sp, adapter_path=path)[0]
                return {'type': 'sample', 'sequences': [{'stop_reason': s.stop_reason, 'tokens': s.tokens, 'logprobs': s.logprobs} for s in res.sequences],
                        'prompt_logprobs': res.prompt_logprobs, 'topk_prompt_logprobs': res.topk_prompt_logprobs}

            return self.schedule_task(work, token=token, model_id=b.get('base_model', self.args.model_id), input_tokens=len(ids),
                                      request_id=request.state.request_id)

        @app.post('/twinkle/create')
        async def create(request: Request):
            return {'status': 'ok', 'model_id': self.args.model_id, 'replica_id': self.replica_id}

        @app.post('/twinkle/sample')
        async def sample(request: Request):
            b = await body_of(request)
            token = request.state.token
            path = self._adapter_path(token, b)
            res = await self.schedule_task_and_wait(lambda: self.backend.sample(b.get('inputs') or [], b.get('sampling_params'),
                                                                                adapter_name=b.get('adapter_name'), adapter_path=path,
                                                                                **({'use_base_model': True} if b.get('use_base_model') else {})), token=token)
            return {'status': 'ok', 'result': self._to_wire(res)}

        @app.post('/twinkle/sample_stream')
        async def sample_stream(request: Request):
            b = await body_of(request)
            if not hasattr(self.backend, 'sample_stream') or getattr(self.backend, '_remote_proxy', None) is not None:
                # a sampler that lives in a worker group answers whole responses; the stream carries one final event
                res = self.backend.sample(b.get('inputs') or [], b.get('sampling_params'))

                async def one():
                    yield 'data: ' + json.dumps({'done': True, 'result': self._to_wire(res)}) + '\n\n'

                return StreamingResponse(one(), media_type='text/event-stream')

            async def gen():
                loop = asyncio.get_event_loop()
                it = self.backend.sample_stream(b.get('inputs') or [], b.get('sampling_params'))
                while True:
                    item = await loop.run_in_executor(None, lambda: next(it, None))
                    if item is None:
                        return
                    if item.get('done') and 'responses' in item:
                        item = {'done': True, 'result': self._to_wire(item['responses'])}
                    yield 'data: ' + json.dumps(item) + '\n\n'

            return StreamingResponse(gen(), media_type='text/event-stream')

        @app.post('/twinkle/set_template')
        async def set_template(request: Request):
            b = await body_of(request)
            self.backend.set_template(b.get('template_cls', 'Template'), **(b.get('kwargs') or {}))
            return {'status': 'ok'}

        @app.post('/twinkle/add_adapter_to_sampler')
        async def add_adapter(request: Request):
            b = await body_of(request)
            self.backend.add_adapter_to_sampler(b['adapter_name'], b.get('config') or b.get('adapter_path'))
            return {'status': 'ok'}

        @app.post('/twinkle/apply_patch')
        async def apply_patch(request: Request):
            b = await body_of(request)
            if hasattr(self.backend, 'apply_patch'):
                self.backend.apply_patch(b.get('patch_cls'), **(b.get('kwargs') or {}))
            return {'status': 'ok'}


# =========================================================== Processor app
class ProcessorApp:
    """Remote construction / invocation of data components (Dataset, DataLoader, Template, InputProcessor…) by
    class name, bound to the caller's session."""

    ALLOWED = ('twinkle_b200.dataset', 'twinkle_b200.dataloader', 'twinkle_b200.template', 'twinkle_b200.processor', 'twinkle_b200.preprocessor',
               'twinkle_b200.reward', 'twinkle_b200.advantage')

    def __init__(self, args, state: ServerState, name: str = 'processor'):
        self.state, self.name = state, name
        self.replica_id = f'{name}-{uuid.uuid4().hex[:8]}'
        self.objects: Dict[str, Dict[str, Any]] = {}
        self.app = FastAPI(title='twinkle-processor')
        install_middleware(self.app, name, self.replica_id)
        self._routes()

    def _resolve(self, class_name: str):
        import importlib
        for mod in self.ALLOWED:
            m = importlib.import_module(mod)
            if hasattr(m, class_name):
                return getattr(m, class_name)
        raise KeyError(f'{class_name} is not a constructible data component')

    def _decode(self, v):
        if isinstance(v, dict) and '__object__' in v:
            return self.objects[v['__object__']]['obj']
        if isinstance(v, dict) and '__class__' in v:
            return self._resolve(v['__class__'])(**{k: self._decode(x) for k, x in (v.get('kwargs') or {}).items()})
        if isinstance(v, list):
            return [self._decode(x) for x in v]
        if isinstance(v, dict):
            return {k: self._decode(x) for k, x in v.items()}
        return v

    def expire(self, timeout: float) -> List[str]:
        gone = []
        for oid, o in list(self.objects.items()):
            age = self.state.session_age(o['session_id']) if o['session_id'] else 0
            if age is None or age > timeout:
                self.objects.pop(oid)
                gone.append(oid)
        return gone

    def _routes(self) -> None:
        app = self.app

        @app.post('/twinkle/create')
        async def create(request: Request):
            b = await body_of(request)
            cls = self._resolve(b['class_name'])
            obj = cls(*self._decode(b.get('args') or []), **self._decode(b.get('kwargs') or {}))
            oid = uuid.uuid4().hex
            self.objects[oid] = {'obj': obj, 'session_id': b.get('session_id'), 'token': request.state.token, 'it': None}
            return {'status': 'ok', 'object_id': oid}

        @app.post('/twinkle/call')
        async def call(request: Request):
            b = await body_of(request)
            o = self.objects.get(b.get('object_id', ''))
            if o is None:
                raise HTTPException(404, 'unknown object')
            if o['token'] != request.state.token:
                raise HTTPException(403, 'object belongs to another token')
            method = b['method']
            if method == '__next__':
                if o['it'] is None:
                    o['it'] = iter(o['obj'])
                try:
                    return {'status': 'ok', 'result': _jsonable(next(o['it']))}
                except StopIteration:
                    o['it'] = None
                    return {'status': 'stop'}
            if method == '__len__':
                return {'status': 'ok', 'result': len(o['obj'])}
            if method == '__getitem__':
                return {'status': 'ok', 'result': _jsonable(o['obj'][b['args'][0]])}
            if method.startswith('_'):
                raise HTTPException(400, 'private methods are not callable')
            res = getattr(o['obj'], method)(*self._decode(b.get('args') or []), **self._decode(b.get('kwargs') or {}))
            return {'status': 'ok', 'result': _jsonable(res)}


def _jsonable(x):
    try:
        import numpy as np
        import torch
        if torch.is_tensor(x):
            return x.tolist()
        if isinstance(x, np.ndarray):
            return x.tolist()
    except Exception:
        pass
    if isinstance(x, dict):
        return {k: _jsonable(v) for k, v in x.items()}
    if isinstance(x, (list, tuple)):
        return [_jsonable(v) for v in x]
    if hasattr(x, 'to_dict'):
        return x.to_dict()
    return x
