"""Server-side checkpoint registry.

Parity: reference ``src/twinkle/server/checkpoint/{paths,checkpoint_manager,training_run_manager}.py`` — a
filesystem registry under ``TWINKLE_DEFAULT_SAVE_DIR``: ``<root>/<hmac(token)>/<run_id>/{weights|
sampler_weights}/<name>`` addressed as ``twinkle://<run_id>/weights/<name>`` (``tinker://`` accepted as an
alias), with per-checkpoint ``metadata.json``, listing / deletion / ``weights_info`` / ``resolve_load_path``
/ ``parse_adapter_uri``; a token can only see its own runs.

Two cooperating classes, as in the reference: :class:`TrainingRunManager` owns the per-run record (``run.json``: base
model, owner digest, LoRA settings, user metadata, last request time, last training / sampler checkpoint, an optional
client-chosen ``save_dir`` reached through a pointer file in the default location, paged listing newest first) and
:class:`CheckpointManager` owns the per-checkpoint records (``metadata.json``: type, time, size on disk, visibility and
the run's training settings, so that a published checkpoint is self-describing) and keeps the run record's
``last_checkpoint`` fields current.  Sampler weights are transient: registering a new set removes the earlier ones.
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


def dir_size(path: str) -> int:
    """Bytes of the regular files under ``path`` (symlinks are not followed)."""
    total = 0
    for dirpath, _, files in os.walk(path):
        for fn in files:
            fp = os.path.join(dirpath, fn)
            if not os.path.islink(fp):
                try:
                    total += os.path.getsize(fp)
                except OSError:
                    pass
    return total


def _write_json(path: str, data: Dict[str, Any]) -> None:
    tmp = f'{path}.{os.getpid()}.part'
    with open(tmp, 'w') as f:
        json.dump(data, f, indent=1)
    os.replace(tmp, path)           # readers never see a half-written record


def _read_json(path: str) -> Optional[Dict[str, Any]]:
    try:
        with open(path) as f:
            d = json.load(f)
        return d if isinstance(d, dict) else None
    except (OSError, ValueError):
        return None


RUN_FILE = 'run.json'
POINTER_KEY = '_save_dir_pointer'


class TrainingRunManager:
    """Run records under ``<root>/<digest(token)>/<run_id>/run.json``.  A client may ask for its run to live under its
    own ``save_dir`` (``<save_dir>/<digest(token)>/<run_id>``); the default location then holds a pointer record so
    that the run is still found by id (reference ``server/checkpoint/training_run_manager.py:101-262``)."""

    FIELDS = ('training_run_id', 'base_model', 'model_owner', 'save_dir', 'is_lora', 'corrupted', 'lora_rank', 'train_unembed', 'train_mlp',
              'train_attn', 'created', 'last_request_time', 'last_checkpoint', 'last_sampler_checkpoint', 'user_metadata')

    def __init__(self, root: Optional[str] = None):
        self.root = root or save_root()

    def base_dir(self, token: str, save_dir: Optional[str] = None) -> str:
        return os.path.join(os.path.abspath(save_dir) if save_dir else self.root, token_dir(token))

    def check_save_dir(self, save_dir: str) -> str:
        """A client-chosen directory must exist on the server and lie under the default root or under a root the
        operator listed in ``TWINKLE_ALLOWED_SAVE_DIRS``: a request must not make the server write wherever it names
        (the reference accepts any existing server directory, ``checkpoint/paths.py:34-42``)."""
        real = os.path.realpath(os.path.expanduser(save_dir))
        if not os.path.isdir(real):
            raise ValueError(f'save_dir is not a directory on the server: {save_dir!r}')
        roots = [os.path.realpath(self.root)] + [os.path.realpath(r) for r in os.environ.get('TWINKLE_ALLOWED_SAVE_DIRS', '').split(os.pathsep) if r]
        if not any(real == r or real.startswith(r + os.sep) for r in roots):
            raise PermissionError(f'save_dir {save_dir!r} is outside the roots this server may write to (TWINKLE_ALLOWED_SAVE_DIRS)')
        return real

    def _pointer(self, token: str, run_id: str) -> Optional[Dict[str, Any]]:
        d = _read_json(os.path.join(self.base_dir(token), run_id, RUN_FILE))
        return d if d and d.get(POINTER_KEY) else None

    def run_dir(self, token: str, run_id: str, save_dir: Optional[str] = None) -> str:
        if any(x in ('..', '') or '/' in x or os.sep in x for x in (run_id, )):
            raise ValueError('invalid run id')
        if save_dir is None:
            ptr = self._pointer(token, run_id)
            save_dir = ptr.get('save_dir') if ptr else None
        return os.path.join(self.base_dir(token, save_dir), run_id)

    def save(self, token: str, run_id: str, base_model: str, lora_config: Optional[Dict[str, Any]] = None, save_dir: Optional[str] = None,
             user_metadata: Optional[Dict[str, Any]] = None, **info) -> Dict[str, Any]:
        lc = lora_config or {}
        save_dir = save_dir or (user_metadata or {}).get('save_dir')
        if save_dir:
            save_dir = self.check_save_dir(save_dir)
        rank = lc.get('rank', lc.get('r', info.pop('lora_rank', None)))
        now = time.time()
        rec = {'training_run_id': run_id, 'base_model': base_model, 'model_owner': token_dir(token),
               'save_dir': os.path.abspath(save_dir) if save_dir else None, 'is_lora': bool(info.pop('is_lora', bool(lc) or rank is not None)),
               'corrupted': False, 'lora_rank': rank, 'train_unembed': lc.get('train_unembed'), 'train_mlp': lc.get('train_mlp'),
               'train_attn': lc.get('train_attn'), 'created': now, 'last_request_time': now, 'last_checkpoint': None,
               'last_sampler_checkpoint': None, 'user_metadata': user_metadata, **info}
        self._write(token, run_id, rec)
        return rec

    def _write(self, token: str, run_id: str, rec: Dict[str, Any]) -> None:
        d = self.run_dir(token, run_id, rec.get('save_dir'))
        os.makedirs(d, exist_ok=True)
        _write_json(os.path.join(d, RUN_FILE), rec)
        default = os.path.join(self.base_dir(token), run_id)
        if rec.get('save_dir') and os.path.realpath(default) != os.path.realpath(d):
            os.makedirs(default, exist_ok=True)
            _write_json(os.path.join(default, RUN_FILE), {POINTER_KEY: True, 'training_run_id': run_id, 'save_dir': rec['save_dir']})

    def get(self, token: str, run_id: str) -> Optional[Dict[str, Any]]:
        try:
            path = os.path.join(self.run_dir(token, run_id), RUN_FILE)
        except ValueError:
            return None
        if not os.path.isfile(path):
            return None
        rec = _read_json(path)
        if rec is None:     # the record exists but cannot be read: the run is listed as corrupted, not hidden
            return {'training_run_id': run_id, 'base_model': '', 'model_owner': token_dir(token), 'corrupted': True}
        return rec

    def update(self, token: str, run_id: str, updates: Dict[str, Any]) -> Optional[Dict[str, Any]]:
        rec = self.get(token, run_id)
        if rec is None or rec.get('corrupted'):
            return None
        rec.update(updates)
        self._write(token, run_id, rec)
        return rec

    def touch(self, token: str, run_id: str) -> None:
        self.update(token, run_id, {'last_request_time': time.time()})

    def list_runs(self, token: str, limit: int = 20, offset: int = 0) -> Dict[str, Any]:
        """Newest first (by the record's modification time), one page of it."""
        base = self.base_dir(token)
        cands = []
        if os.path.isdir(base):
            for r in os.listdir(base):
                f = os.path.join(base, r, RUN_FILE)
                if os.path.isfile(f):
                    ptr = _read_json(f)
                    real = os.path.join(self.run_dir(token, r), RUN_FILE) if (ptr and ptr.get(POINTER_KEY)) else f
                    cands.append((os.path.getmtime(real) if os.path.isfile(real) else 0.0, r))
        cands.sort(reverse=True)
        runs = [x for x in (self.get(token, r) for _, r in cands) if x]
        limit = max(int(limit), 0)
        offset = max(int(offset), 0)
        return {'training_runs': runs[offset:offset + limit], 'cursor': {'offset': offset, 'limit': limit, 'total_count': len(runs)}}


class CheckpointManager:

    def __init__(self, root: Optional[str] = None, runs: Optional[TrainingRunManager] = None):
        self.root = root or save_root()
        self.runs = runs or TrainingRunManager(self.root)

    def run_dir(self, token: str, run_id: str) -> str:
        return self.runs.run_dir(token, run_id)

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
        return self.runs.save(token, run_id, base_model, **info)

    def touch_run(self, token: str, run_id: str) -> None:
        self.runs.touch(token, run_id)

    def list_runs(self, token: str, limit: int = 1 << 30, offset: int = 0) -> List[Dict[str, Any]]:
        return self.runs.list_runs(token, limit, offset)['training_runs']

    def get_run(self, token: str, run_id: str) -> Optional[Dict[str, Any]]:
        return self.runs.get(token, run_id)

    # --------------------------------------------------------- checkpoints
    def register(self, token: str, run_id: str, name: str, kind: str = 'weights', public: bool = False, **info) -> Dict[str, Any]:
        """Record a checkpoint whose files are already in place.  Sampler weights replace the run's earlier sampler
        weights on disk (they exist to be loaded by a sampler once, reference ``checkpoint_manager.py:289-311``)."""
        d = self.path_for(token, run_id, name, kind)
        os.makedirs(d, exist_ok=True)
        if kind == 'sampler_weights':
            self._drop_other_sampler_weights(token, run_id, keep=name)
        run = self.runs.get(token, run_id) or {}
        is_lora = os.path.isfile(os.path.join(d, 'adapter_model.safetensors')) or bool(run.get('is_lora'))
        meta = {'checkpoint_id': f'{kind}/{name}', 'checkpoint_type': 'sampler' if kind == 'sampler_weights' else 'training', 'name': name,
                'kind': kind, 'time': time.time(), 'path': self.uri_for(run_id, name, kind), 'size_bytes': dir_size(d), 'public': bool(public),
                'base_model': run.get('base_model'), 'is_lora': is_lora, 'lora_rank': run.get('lora_rank'),
                'train_unembed': run.get('train_unembed'), 'train_mlp': run.get('train_mlp'), 'train_attn': run.get('train_attn'),
                'user_metadata': run.get('user_metadata'), **info}
        _write_json(os.path.join(d, 'metadata.json'), meta)
        self.runs.update(token, run_id, {('last_sampler_checkpoint' if kind == 'sampler_weights' else 'last_checkpoint'): meta,
                                         'last_request_time': time.time()})
        return meta

    def _drop_other_sampler_weights(self, token: str, run_id: str, keep: str) -> None:
        d = os.path.join(self.run_dir(token, run_id), 'sampler_weights')
        if not os.path.isdir(d):
            return
        for n in os.listdir(d):
            p = os.path.join(d, n)
            if n == keep:
                continue
            if os.path.islink(p):
                os.unlink(p)        # never follow a link into somebody else's files
            elif os.path.isdir(p):
                shutil.rmtree(p)

    def get(self, token: str, run_id: str, checkpoint_id: str) -> Optional[Dict[str, Any]]:
        kind, _, name = checkpoint_id.partition('/')
        if not name:
            kind, name = 'weights', kind
        try:
            return _read_json(os.path.join(self.path_for(token, run_id, name, kind), 'metadata.json'))
        except ValueError:
            return None

    def list_checkpoints(self, token: str, run_id: str) -> List[Dict[str, Any]]:
        """Oldest first."""
        out = []
        for kind in ('weights', 'sampler_weights'):
            d = os.path.join(self.run_dir(token, run_id), kind)
            if os.path.isdir(d):
                for n in os.listdir(d):
                    m = _read_json(os.path.join(d, n, 'metadata.json'))
                    if m:
                        out.append(m)
        out.sort(key=lambda m: (m.get('time', 0.0), m.get('checkpoint_id', '')))
        return out

    def delete(self, token: str, run_id: str, checkpoint_id: str) -> bool:
        kind, _, name = checkpoint_id.partition('/')
        if not name:
            kind, name = 'weights', kind
        try:
            d = self.path_for(token, run_id, name, kind)
        except ValueError:
            return False
        if not os.path.isdir(d):
            return False
        shutil.rmtree(d)
        left = [m for m in self.list_checkpoints(token, run_id) if m.get('kind') == kind]
        self.runs.update(token, run_id, {('last_sampler_checkpoint' if kind == 'sampler_weights' else 'last_checkpoint'): left[-1] if left else None})
        return True

    def parse_path(self, path: str) -> Optional[Dict[str, str]]:
        """``twinkle://run/weights/name`` → its parts, ``None`` for anything else."""
        try:
            run, kind, name = parse_uri(path)
        except ValueError:
            return None
        return {'path': path, 'training_run_id': run, 'checkpoint_type': 'sampler' if kind == 'sampler_weights' else 'training',
                'checkpoint_id': f'{kind}/{name}'}

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
        m = _read_json(os.path.join(d, 'metadata.json'))
        if m:
            info.update({k: v for k, v in m.items() if info.get(k) is None})
        parsed = self.parse_path(path)
        if parsed:
            run = self.runs.get(token, parsed['training_run_id']) or {}
            info.setdefault('training_run_id', parsed['training_run_id'])
            for k in ('base_model', 'model_owner', 'lora_rank'):
                if info.get(k) is None and run.get(k) is not None:
                    info[k] = run[k]
        return info

    parse_adapter_uri = staticmethod(parse_uri)
