"""Gateway: sessions, futures, training-run / checkpoint listing, OpenAI-compatible chat, and routing of
compute calls to the model / sampler applications.

Parity: reference ``src/twinkle/server/gateway/{app,tinker_handlers,twinkle_handlers,openai_handlers,
openai_bridge,proxy}.py``.
"""
from __future__ import annotations

import asyncio
import json
import time
import uuid
from typing import Any, Callable, Dict, List, Optional

from fastapi import FastAPI, HTTPException, Request
from fastapi.responses import JSONResponse, PlainTextResponse, StreamingResponse

from ..checkpoint import CheckpointManager
from ..state import ServerState
from ..telemetry import get_registry
from . import LONG_POLL, POLL_INTERVAL, ModelApp, SamplerApp, body_of, install_middleware


class Router:
    """Sticky routing: a model id goes to the replica that holds its adapter; new models go to the replica
    of that base model with the most free LoRA slots (reference ``server/common/router.py:13-78``)."""

    def __init__(self):
        self.models: Dict[str, List[ModelApp]] = {}
        self.samplers: Dict[str, List[SamplerApp]] = {}

    def add_model(self, app: ModelApp) -> None:
        self.models.setdefault(app.args.model_id, []).append(app)

    def add_sampler(self, app: SamplerApp) -> None:
        self.samplers.setdefault(app.args.model_id, []).append(app)

    def model_for(self, base_model: Optional[str], model_id: Optional[str] = None) -> ModelApp:
        if model_id:
            for apps in self.models.values():
                for a in apps:
                    if model_id in a.adapters:
                        return a
        apps = self.models.get(base_model or '') or (next(iter(self.models.values())) if len(self.models) == 1 and not base_model else None)
        if not apps:
            raise KeyError(f'no model deployment serves {base_model!r}')
        return max(apps, key=lambda a: a.args.max_loras - len(a.adapters))

    def sampler_for(self, base_model: Optional[str]) -> SamplerApp:
        apps = self.samplers.get(base_model or '') or (next(iter(self.samplers.values())) if self.samplers else None)
        if not apps:
            raise KeyError(f'no sampler deployment serves {base_model!r}')
        return min(apps, key=lambda a: a.worker.depth())


async def _call(sub_app: FastAPI, path: str, request: Request, body: Dict[str, Any]) -> Any:
    """In-process proxy: run the sub-application's ASGI handler with the caller's headers (keeps the
    sticky-routing / auth / trace headers exactly as an HTTP hop would)."""
    import httpx
    headers = {k: v for k, v in request.headers.items() if k.lower() in ('twinkle-authorization', 'authorization', 'x-request-id',
                                                                         'traceparent', 'serve_multiplexed_model_id')}
    headers.setdefault('x-request-id', getattr(request.state, 'request_id', uuid.uuid4().hex))
    transport = httpx.ASGITransport(app=sub_app)
    async with httpx.AsyncClient(transport=transport, base_url='http://inproc') as c:
        r = await c.post(path, json=body, headers=headers, timeout=None)
    if r.status_code >= 400:
        raise HTTPException(r.status_code, r.json().get('detail', r.text) if r.headers.get('content-type', '').startswith('application/json') else r.text)
    return r.json()


class GatewayApp:

    def __init__(self, args, state: ServerState, checkpoints: CheckpointManager, router: Router, name: str = 'server'):
        self.args, self.state, self.checkpoints, self.router, self.name = args, state, checkpoints, router, name
        self.replica_id = f'{name}-{uuid.uuid4().hex[:8]}'
        self.app = FastAPI(title='twinkle-gateway')
        install_middleware(self.app, name, self.replica_id)
        self._routes()

    def supported_models(self) -> List[str]:
        return sorted(set(self.args.supported_models) | set(self.router.models) | set(self.router.samplers))

    def _routes(self) -> None:
        app, st = self.app, self.state

        # ---------------------------------------------------- sessions
        async def create_session(request: Request):
            b = await body_of(request)
            sid = st.create_session(request.state.token, {'tags': b.get('tags'), 'sdk_version': b.get('sdk_version'), 'user_metadata': b.get('user_metadata')})
            return {'type': 'create_session', 'session_id': sid, 'info_message': None, 'warning_message': None, 'error_message': None}

        async def session_heartbeat(request: Request):
            b = await body_of(request)
            if not st.heartbeat(b.get('session_id', '')):
                raise HTTPException(404, 'unknown session')
            return {'type': 'session_heartbeat'}

        async def capabilities(request: Request):
            return {'supported_models': [{'model_name': m} for m in self.supported_models()]}

        for prefix in ('', '/twinkle'):
            app.post(prefix + '/create_session')(create_session)
            app.post(prefix + '/session_heartbeat')(session_heartbeat)
            app.get(prefix + '/get_server_capabilities')(capabilities)

        @app.get('/healthz')
        async def healthz():
            return {'status': 'ok'}

        @app.get('/twinkle/healthz')
        async def tw_healthz():
            return {'status': 'ok', 'replica_id': self.replica_id}

        @app.get('/twinkle/healthz/deep')
        async def deep():
            parts, ok = {}, True
            for base, apps in list(self.router.models.items()) + list(self.router.samplers.items()):
                for a in apps:
                    try:
                        good = bool(a.backend.ping()) if hasattr(a.backend, 'ping') else True
                    except Exception:
                        good = False
                    parts[a.replica_id] = 'ok' if good else 'unhealthy'
                    ok = ok and good
            return JSONResponse({'status': 'ok' if ok else 'degraded', 'components': parts}, status_code=200 if ok else 503)

        @app.get('/twinkle/status')
        async def status():
            return {'gauges': st.gauges(), 'leader': st.is_leader(), 'replica_id': self.replica_id,
                    'queues': {a.replica_id: a.worker.depth() for apps in self.router.models.values() for a in apps}}

        @app.get('/twinkle/capacity_info')
        async def capacity():
            return {'replicas': st.replica_capacity()}

        @app.post('/telemetry')
        async def telemetry(request: Request):
            b = await body_of(request)
            get_registry().inc('twinkle_client_telemetry_events_total', len(b.get('events') or [1]))
            return {'status': 'accepted'}

        @app.get('/metrics')
        async def metrics():
            for k, v in st.gauges().items():
                get_registry().set_gauge(f'twinkle_active_{k}', v)
            return PlainTextResponse(get_registry().render_prometheus())

        # ---------------------------------------------------- futures
        @app.post('/retrieve_future')
        async def retrieve_future(request: Request):
            b = await body_of(request)
            rid = b.get('request_id', '')
            deadline = time.monotonic() + LONG_POLL()
            while True:
                f = st.get_future(rid)
                if f is None:
                    raise HTTPException(404, f'unknown request {rid}')
                if f['status'] == 'completed':
                    res = f.get('result')
                    return res if isinstance(res, dict) else {'result': res}
                if f['status'] == 'failed':
                    return JSONResponse({'type': 'request_failed', 'error': f.get('error', 'failed'), 'category': 'server'}, status_code=400)
                if time.monotonic() >= deadline:
                    return {'type': 'try_again', 'request_id': rid, 'queue_state': f['status'], 'queue_depth': f.get('queue_depth')}
                await asyncio.sleep(POLL_INTERVAL())

        # ------------------------------------------ model compute (proxied)
        def _to_model(endpoint: str, new_model: bool = False):
            async def handler(request: Request):
                b = await body_of(request)
                if new_model:
                    sess = st.get_session(b.get('session_id', '')) if b.get('session_id') else None
                    if b.get('session_id') and sess is None:
                        raise HTTPException(404, 'unknown session')
                    target = self.router.model_for(b.get('base_model'))
                    b.setdefault('model_id', uuid.uuid4().hex)
                else:
                    info = st.get_model(b.get('model_id', ''))
                    if info is None:
                        raise HTTPException(404, f"unknown model {b.get('model_id')!r}")
                    if info['token'] != request.state.token:
                        raise HTTPException(403, 'model belongs to another token')
                    target = self.router.model_for(info['base_model'], b['model_id'])
                return await _call(target.app, f'/tinker/{endpoint}', request, b)
            return handler

        app.post('/create_model')(_to_model('create_model', new_model=True))
        for ep in ('get_info', 'unload_model', 'forward', 'forward_backward', 'optim_step', 'save_weights', 'load_weights', 'save_weights_for_sampler'):
            app.post(f'/{ep}')(_to_model(ep))

        # ---------------------------------------------------- sampling
        @app.post('/create_sampling_session')
        async def create_sampling_session(request: Request):
            b = await body_of(request)
            sid = st.create_sampling_session(request.state.token, b.get('base_model') or '', b.get('model_path'), b.get('session_id'))
            return {'type': 'create_sampling_session', 'sampling_session_id': sid}

        @app.post('/asample')
        async def asample(request: Request):
            b = await body_of(request)
            base = b.get('base_model')
            if not base and b.get('sampling_session_id'):
                s = st.get_sampling_session(b['sampling_session_id'])
                base = (s or {}).get('base_model')
            return await _call(self.router.sampler_for(base).app, '/tinker/asample', request, b)

        # ---------------------------------------------- runs / checkpoints
        async def list_runs(request: Request, limit: int = 20, offset: int = 0):
            return self.checkpoints.runs.list_runs(request.state.token, limit, offset)

        async def get_run(run_id: str, request: Request):
            r = self.checkpoints.get_run(request.state.token, run_id)
            if r is None:
                raise HTTPException(404, 'unknown training run')
            return r

        async def list_ckpt(run_id: str, request: Request):
            return {'checkpoints': self.checkpoints.list_checkpoints(request.state.token, run_id)}

        async def del_ckpt(run_id: str, checkpoint_id: str, request: Request):
            if not self.checkpoints.delete(request.state.token, run_id, checkpoint_id.replace(':', '/')):
                raise HTTPException(404, 'unknown checkpoint')
            return {'status': 'deleted'}

        async def weights_info(request: Request):
            b = await body_of(request)
            return self.checkpoints.weights_info(request.state.token, b.get('tinker_path') or b.get('path', ''))

        for prefix in ('', '/twinkle'):
            app.get(prefix + '/training_runs')(list_runs)
            app.get(prefix + '/training_runs/{run_id}')(get_run)
            app.get(prefix + '/training_runs/{run_id}/checkpoints')(list_ckpt)
            app.delete(prefix + '/training_runs/{run_id}/checkpoints/{checkpoint_id:path}')(del_ckpt)
            app.post(prefix + '/weights_info')(weights_info)

        @app.post('/training_runs/{run_id}/checkpoints/{checkpoint_id:path}/publish')
        async def publish(run_id: str, checkpoint_id: str, request: Request):
            b = await body_of(request)
            kind, _, name = checkpoint_id.replace(':', '/').partition('/')
            path = self.checkpoints.path_for(request.state.token, run_id, name or kind, kind if name else 'weights')
            from ...hub import HubOperation
            fut = HubOperation.push_to_hub(b.get('hub_model_id', f'{run_id}-{name}'), path, token=b.get('hub_token'), async_upload=True)
            return {'status': 'publishing'}

        @app.get('/twinkle/checkpoint_path/{run_id}/{checkpoint_id:path}')
        async def checkpoint_path(run_id: str, checkpoint_id: str, request: Request):
            kind, _, name = checkpoint_id.replace(':', '/').partition('/')
            kind, name = (kind, name) if name else ('weights', kind)
            return {'path': self.checkpoints.path_for(request.state.token, run_id, name, kind), 'twinkle_path': f'twinkle://{run_id}/{kind}/{name}'}

        # ------------------------------------------------ OpenAI-compatible
        @app.get('/models')
        async def models():
            return {'object': 'list', 'data': [{'id': m, 'object': 'model', 'owned_by': 'twinkle'} for m in self.supported_models()]}

        @app.post('/chat/completions')
        async def chat(request: Request):
            b = await body_of(request)
            sampler = self.router.sampler_for(b.get('model'))
            sp = {'max_tokens': b.get('max_tokens') or b.get('max_completion_tokens') or 256, 'temperature': b.get('temperature', 1.0),
                  'top_p': b.get('top_p', 1.0), 'seed': b.get('seed'), 'stop': b.get('stop'), 'num_samples': b.get('n', 1)}
            from ...agentic.quality import normalize_messages
            from ...data_format import tool_call_to_openai
            tools = [{'tool_name': (t.get('function') or t).get('name'), 'description': (t.get('function') or t).get('description', ''),
                      'parameters': (t.get('function') or t).get('parameters', {})} for t in (b.get('tools') or [])]
            # OpenAI wire messages (function-style tool calls, list-of-parts contents) → the internal message form
            traj = normalize_messages({'messages': b.get('messages') or []})
            if tools:
                traj['tools'] = tools
            want_lp = bool(b.get('logprobs'))
            if want_lp:
                sp['logprobs'] = int(b.get('top_logprobs') or 1)
            if sampler.backend.template is None:
                sampler.backend.set_template('Template', model_id=sampler.args.model_id)
            tpl = sampler.backend.template
            created, cid = int(time.time()), 'chatcmpl-' + uuid.uuid4().hex[:24]
            if b.get('stream') and hasattr(sampler.backend, 'sample_stream'):
                async def gen():
                    loop = asyncio.get_event_loop()
                    it = sampler.backend.sample_stream([traj], sp)
                    base = {'id': cid, 'object': 'chat.completion.chunk', 'created': created, 'model': b.get('model')}
                    yield 'data: ' + json.dumps({**base, 'choices': [{'index': 0, 'delta': {'role': 'assistant', 'content': ''}, 'finish_reason': None}]}) + '\n\n'
                    final = None
                    while True:
                        item = await loop.run_in_executor(None, lambda: next(it, None))
                        if item is None:
                            break
                        if item.get('done'):
                            final = item
                            break
                        yield 'data: ' + json.dumps({**base, 'choices': [{'index': item['index'], 'delta': {'content': item['text']},
                                                                           'finish_reason': None}]}) + '\n\n'
                    reasons = {}
                    for r in (final or {}).get('responses') or []:
                        for i, q in enumerate(getattr(r, 'sequences', None) or (r.get('sequences') if isinstance(r, dict) else []) or []):
                            reasons[i] = (getattr(q, 'stop_reason', None) if not isinstance(q, dict) else q.get('stop_reason')) or 'stop'
                    for i, why in sorted(reasons.items()) or [(0, 'stop')]:
                        yield 'data: ' + json.dumps({**base, 'choices': [{'index': i, 'delta': {}, 'finish_reason': 'stop' if why == 'stop' else 'length'}]}) + '\n\n'
                    yield 'data: [DONE]\n\n'
                return StreamingResponse(gen(), media_type='text/event-stream')
            res = await sampler.schedule_task_and_wait(lambda: sampler.backend.sample([traj], sp), token=request.state.token)
            seqs = res[0].sequences
            n_prompt = len(seqs[0].new_input_feature['input_ids']) - len(seqs[0].tokens) if seqs else 0
            choices = []
            for i, q in enumerate(seqs):
                text = q.decoded or ''
                reasoning = ''
                if text.lstrip().startswith('<think>') and '</think>' in text:
                    head, text = text.split('</think>', 1)
                    reasoning, text = head.split('<think>', 1)[1].strip(), text.lstrip('\n')
                msg = tpl.response_message(text) if hasattr(tpl, 'response_message') else {'role': 'assistant', 'content': text}
                out = {'role': 'assistant', 'content': msg['content'] or (None if msg.get('tool_calls') else '')}
                if reasoning:
                    out['reasoning_content'] = reasoning
                if msg.get('tool_calls'):
                    out['tool_calls'] = [tool_call_to_openai(c) for c in msg['tool_calls']]
                choice = {'index': i, 'message': out,
                          'finish_reason': 'tool_calls' if msg.get('tool_calls') and q.stop_reason == 'stop' else ('stop' if q.stop_reason == 'stop' else 'length')}
                if want_lp and q.logprobs is not None:
                    dec = (lambda t: tpl.decode([t], skip_special_tokens=False)) if hasattr(tpl, 'decode') else str
                    content = []
                    for k, (t, lp) in enumerate(zip(q.tokens, q.logprobs)):
                        ent = {'token': dec(t), 'logprob': lp, 'bytes': None}
                        if q.topk_logprobs and k < len(q.topk_logprobs) and q.topk_logprobs[k]:
                            ent['top_logprobs'] = [{'token': dec(a), 'logprob': b_, 'bytes': None} for a, b_ in q.topk_logprobs[k]]
                        content.append(ent)
                    choice['logprobs'] = {'content': content}
                choices.append(choice)
            return {'id': cid, 'object': 'chat.completion', 'created': created, 'model': b.get('model'), 'choices': choices,
                    'usage': {'prompt_tokens': n_prompt, 'completion_tokens': sum(len(s.tokens) for s in seqs),
                              'total_tokens': n_prompt + sum(len(s.tokens) for s in seqs)}}
