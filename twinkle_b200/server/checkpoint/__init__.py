"""Server-side checkpoint registry.

Parity: reference ``src/twinkle/server/checkpoint/{paths,checkpoint_manager,training_run_manager}.py`` — a
filesystem registry under ``TWINKLE_DEFAULT_SAVE_DIR``: ``<root>/<hmac(token)>/<run_id>/{weights|
sampler_weights}/<name>`` addressed as ``twinkle://<run_id>/weights/<name>`` (``tinker://`` accepted as an
alias), with per-checkpoint ``metadata.json``, listing / deletion / ``weights_info`` / ``resolve_load_path``
/ ``parse_adapter_uri``; a token can only see its own runs.
"""
from __future__ import annotations

import hashlib
import hmac
import json
import os
import shutil
import time
from typing import Any, Dict, List, Optional, Tuple

SCHEMES = ('twinkle://', 'tinker://')


def save_root() -> str:
    return os.environ.get('TWINKLE_DEFAULT_SAVE_DIR', './output')


def token_dir(token: str) -> str:
    salt = os.environ.get('TWINKLE_TOKEN_SALT', 'twinkle')
    return hmac.new(salt.encode(), (token or 'anonymous').encode(), hashlib.sha256).hexdigest()[:24]


def parse_uri(uri: str) -> Tuple[str, str, str]:
    """``twinkle://run/weights/name`` → (run, kind, name)."""
    for s in SCHEMES:
        if uri.startswith(s):
            parts = uri[len(s):].strip('/').split('/')
            if len(parts) == 3 and parts[1] in ('weights', 'sampler_weights'):
                return parts[0], parts[1], parts[2]
            if len(parts) == 2:
                return parts[0], 'weights', parts[1]
            raise ValueError(f'malformed checkpoint uri {uri!r}')
    raise ValueError(f'unknown scheme in {uri!r}')


class CheckpointManager:

    def __init__(self, root: Optional[str] = None):
        self.root = root or save_root()

    def run_dir(self, token: str, run_id: str) -> str:
        return os.path.join(self.root, token_dir(token), run_id)

    def path_for(self, token: str, run_id: str, name: str, kind: str = 'weights') -> str:
        if kind not in ('weights', 'sampler_weights'):
            raise ValueError(kind)
        if any(x in ('..', '') or '/' in x for x in (run_id, name)):
            raise ValueError('invalid run or checkpoint name')
        return os.path.join(self.run_dir(token, run_id), kind, name)

    def uri_for(self, run_id: str, name: str, kind: str = 'weights', scheme: str = 'twinkle://') -> str:
        return f'{scheme}{run_id}/{kind}/{name}'

    # ---------------------------------------------------------------- runs
    def create_run(self, token: str, run_id: str, base_model: str, **info) -> Dict[str, Any]:
        d = self.run_dir(token, run_id)
        os.makedirs(d, exist_ok=True)
        meta = {'training_run_id': run_id, 'base_model': base_model, 'created': time.time(), 'last_request_time': time.time(), **info}
        with open(os.path.join(d, 'run.json'), 'w') as f:
            json.dump(meta, f)
        return meta

    def touch_run(self, token: str, run_id: str) -> None:
        p = os.path.join(self.run_dir(token, run_id), 'run.json')
        if os.path.isfile(p):
            with open(p) as f:
                meta = json.load(f)
            meta['last_request_time'] = time.time()
            with open(p, 'w') as f:
                json.dump(meta, f)

    def list_runs(self, token: str) -> List[Dict[str, Any]]:
        base = os.path.join(self.root, token_dir(token))
        out = []
        if os.path.isdir(base):
            for r in sorted(os.listdir(base)):
                p = os.path.join(base, r, 'run.json')
                if os.path.isfile(p):
                    with open(p) as f:
                        out.append(json.load(f))
        return out

    def get_run(self, token: str, run_id: str) -> Optional[Dict[str, Any]]:
        p = os.path.join(self.run_dir(token, run_id), 'run.json')
        if not os.path.isfile(p):
            return None
        with open(p) as f:
            return json.load(f)

    # --------------------------------------------------------- checkpoints
    def register(self, token: str, run_id: str, name: str, kind: str = 'weights', **info) -> Dict[str, Any]:
        d = self.path_for(token, run_id, name, kind)
        os.makedirs(d, exist_ok=True)
        meta = {'checkpoint_id': f'{kind}/{name}', 'name': name, 'kind': kind, 'time': time.time(), 'path': self.uri_for(run_id, name, kind),
                'is_lora': os.path.isfile(os.path.join(d, 'adapter_model.safetensors')), **info}
        with open(os.path.join(d, 'metadata.json'), 'w') as f:
            json.dump(meta, f)
        return meta

    def list_checkpoints(self, token: str, run_id: str) -> List[Dict[str, Any]]:
        out = []
        for kind in ('weights', 'sampler_weights'):
            d = os.path.join(self.run_dir(token, run_id), kind)
            if os.path.isdir(d):
                for n in sorted(os.listdir(d)):
                    m = os.path.join(d, n, 'metadata.json')
                    if os.path.isfile(m):
                        with open(m) as f:
                            out.append(json.load(f))
        return out

    def delete(self, token: str, run_id: str, checkpoint_id: str) -> bool:
        kind, _, name = checkpoint_id.partition('/')
        if not name:
            kind, name = 'weights', kind
        d = self.path_for(token, run_id, name, kind)
        if os.path.isdir(d):
            shutil.rmtree(d)
            return True
        return False

    def _allowed_roots(self, token: str) -> List[str]:
        roots = [os.path.join(self.root, token_dir(token))]
        roots += [r for r in os.environ.get('TWINKLE_ALLOWED_LOAD_DIRS', '').split(os.pathsep) if r]
        return [os.path.realpath(r) for r in roots]

    def resolve_load_path(self, token: str, path: str) -> str:
        """URI → local directory of the token's own run.  A plain directory is accepted only when, after resolving
        symlinks, it lies under the token's own root or under a root the operator listed in
        ``TWINKLE_ALLOWED_LOAD_DIRS``: a served instance must not read (and un-pickle optimizer state from) arbitrary
        server-local paths a client names (the reference takes ``twinkle://`` URIs checked per token, or hub ids).
        Anything that is not a local path is treated as a hub id."""
        if not path:
            raise ValueError('empty checkpoint path')
        if path.startswith(SCHEMES):
            run, kind, name = parse_uri(path)
            d = self.path_for(token, run, name, kind)
            if not os.path.isdir(d):
                raise FileNotFoundError(f'checkpoint {path} not found for this token')
            return d
        if os.path.exists(path) or os.path.isabs(path) or path.startswith('.'):
            real = os.path.realpath(path)
            if not os.path.isdir(real):
                raise FileNotFoundError(f'checkpoint directory {path!r} not found')
            if not any(real == r or real.startswith(r + os.sep) for r in self._allowed_roots(token)):
                raise PermissionError(f'{path!r} is outside this token\'s checkpoint root; use the twinkle:// path returned by save')
            return real
        from ...hub import HubOperation
        return HubOperation.download_model(path)

    def weights_info(self, token: str, path: str) -> Dict[str, Any]:
        d = self.resolve_load_path(token, path)
        info: Dict[str, Any] = {'path': path, 'is_lora': False}
        ac = os.path.join(d, 'adapter_config.json')
        if os.path.isfile(ac):
            with open(ac) as f:
                cfg = json.load(f)
            info.update(is_lora=True, lora_rank=cfg.get('r'), base_model=cfg.get('base_model_name_or_path'))
        m = os.path.join(d, 'metadata.json')
        if os.path.isfile(m):
            with open(m) as f:
                info.update({k: v for k, v in json.load(f).items() if info.get(k) is None})
        return info

    parse_adapter_uri = staticmethod(parse_uri)
