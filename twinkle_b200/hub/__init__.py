"""Model / dataset hub access.

Parity: reference ``src/twinkle/hub/hub.py:31-657`` — ``ms://`` and ``hf://``
prefixes, ``download_model``, ``download_file``, ``load_dataset``, ``create_model_repo``,
``push_to_hub`` (optionally on a background thread with ``wait_for``), ``try_login`` and the
server's model-alias table.  The network is optional: a local directory always resolves to
itself, and remote ids are looked up in the local HF / ModelScope caches before any client
library is asked to download.

A third hub needs no network at all: ``dir://<repo>`` addresses repositories kept as plain
directories under ``TWINKLE_DIR_HUB`` (a shared file system of an air-gapped cluster).  It
implements the whole interface — create, push (synchronous or queued), download with ignore
patterns into a cache, single-file download — and is what the hub tests run against.
"""
from __future__ import annotations

import os
import threading
from concurrent.futures import Future, ThreadPoolExecutor
from typing import Any, Dict, Optional

_POOL = ThreadPoolExecutor(max_workers=2, thread_name_prefix='hub-upload')
_UPLOADS: Dict[str, Future] = {}
MODEL_ALIASES: Dict[str, str] = {}


LARGE_FILE_PATTERNS = ('*.bin', '*.safetensors', '*.pth', '*.pt', '*.h5', '*.ckpt', '*.onnx', '*.gguf', '*.msgpack')


def _strip(model_id: str):
    for p, hub in (('ms://', 'ms'), ('hf://', 'hf'), ('dir://', 'dir')):
        if model_id.startswith(p):
            return model_id[len(p):], hub
    return model_id, os.environ.get('TWINKLE_DEFAULT_HUB', 'ms')


class DirHub:
    """Repositories as directories under one root (``TWINKLE_DIR_HUB``).  ``token`` is checked against the optional
    ``<root>/.tokens`` file (one accepted token per line) so that the login path can be exercised too."""

    @staticmethod
    def root() -> str:
        r = os.environ.get('TWINKLE_DIR_HUB')
        if not r:
            raise FileNotFoundError('dir:// ids need TWINKLE_DIR_HUB (the directory that holds the repositories)')
        return r

    @classmethod
    def _repo(cls, name: str) -> str:
        if not name or name.startswith(('/', '.')) or '..' in name.split('/'):
            raise ValueError(f'invalid repository id {name!r}')
        return os.path.join(cls.root(), name)

    @classmethod
    def try_login(cls, token: Optional[str]) -> bool:
        f = os.path.join(cls.root(), '.tokens')
        if not os.path.isfile(f):
            return True
        with open(f) as fh:
            return (token or '') in {l.strip() for l in fh if l.strip()}

    @classmethod
    def create_repo(cls, name: str, token: Optional[str] = None, private: bool = True) -> str:
        if not cls.try_login(token):
            raise PermissionError('hub token rejected')
        d = cls._repo(name)
        os.makedirs(d, exist_ok=True)
        return d

    @classmethod
    def upload_folder(cls, name: str, folder: str, token: Optional[str] = None, ignore_patterns=()) -> str:
        import fnmatch
        import shutil
        d = cls.create_repo(name, token)
        for dirpath, _, files in os.walk(folder):
            rel = os.path.relpath(dirpath, folder)
            for fn in files:
                if any(fnmatch.fnmatch(fn, p) for p in ignore_patterns or ()):
                    continue
                dst = os.path.join(d, rel, fn) if rel != '.' else os.path.join(d, fn)
                os.makedirs(os.path.dirname(dst), exist_ok=True)
                shutil.copy2(os.path.join(dirpath, fn), dst + '.part')
                os.replace(dst + '.part', dst)       # a reader never sees a half-written file
        return d

    @classmethod
    def snapshot_download(cls, name: str, ignore_patterns=(), cache_dir: Optional[str] = None) -> str:
        import fnmatch
        import shutil
        src = cls._repo(name)
        if not os.path.isdir(src):
            raise FileNotFoundError(f'no repository {name!r} under {cls.root()}')
        cache = os.path.join(cache_dir or os.environ.get('TWINKLE_HUB_CACHE', os.path.expanduser('~/.cache/twinkle_b200/hub')), name)
        for dirpath, _, files in os.walk(src):
            rel = os.path.relpath(dirpath, src)
            for fn in files:
                if fn == '.tokens' or any(fnmatch.fnmatch(fn, p) for p in ignore_patterns or ()):
                    continue
                dst = os.path.join(cache, rel, fn) if rel != '.' else os.path.join(cache, fn)
                s_ = os.path.join(dirpath, fn)
                if os.path.isfile(dst) and os.path.getmtime(dst) >= os.path.getmtime(s_) and os.path.getsize(dst) == os.path.getsize(s_):
                    continue
                os.makedirs(os.path.dirname(dst), exist_ok=True)
                shutil.copy2(s_, dst)
        return cache


class HubOperation:

    @staticmethod
    def resolve_alias(model_id: str) -> str:
        return MODEL_ALIASES.get(model_id, model_id)

    @staticmethod
    def try_login(token: Optional[str] = None, hub: str = 'dir') -> bool:
        if hub == 'dir':
            return DirHub.try_login(token)
        if hub == 'hf':
            from huggingface_hub import login
            login(token=token)
            return True
        from modelscope.hub.api import HubApi  # type: ignore
        HubApi().login(token)
        return True

    @staticmethod
    def create_model_repo(hub_model_id: str, token: Optional[str] = None, private: bool = True) -> str:
        name, hub = _strip(hub_model_id)
        if hub == 'dir':
            return DirHub.create_repo(name, token, private)
        if hub == 'hf':
            from huggingface_hub import HfApi
            return str(HfApi(token=token).create_repo(name, private=private, exist_ok=True))
        from modelscope.hub.api import HubApi  # type: ignore
        api = HubApi()
        if token:
            api.login(token)
        return str(api.create_model(name))

    @staticmethod
    def download_file(repo_id: str, allow_patterns=None, token: Optional[str] = None, **kwargs) -> str:
        """The repository with only the files that match ``allow_patterns`` (a pattern or a list)."""
        import fnmatch
        pats = [allow_patterns] if isinstance(allow_patterns, str) else list(allow_patterns or ['*'])
        name, hub = _strip(repo_id)
        if hub == 'dir':
            src = DirHub._repo(name)
            every = {fn for _, _, fs in os.walk(src) for fn in fs}
            skip = [fn for fn in every if not any(fnmatch.fnmatch(fn, p) for p in pats)]
            return DirHub.snapshot_download(name, ignore_patterns=skip, cache_dir=kwargs.get('cache_dir'))
        if hub == 'hf':
            from huggingface_hub import snapshot_download
            return snapshot_download(name, allow_patterns=pats, token=token)
        from modelscope import snapshot_download  # type: ignore
        return snapshot_download(name, allow_patterns=pats)

    @staticmethod
    def download_model(model_id: str, revision: Optional[str] = None, ignore_model: bool = False, ignore_patterns=(), **kwargs) -> str:
        """``ignore_model=True`` leaves the weight files out (tokenizer / config only)."""
        model_id = HubOperation.resolve_alias(model_id)
        if os.path.isdir(model_id):
            return model_id
        name, hub = _strip(model_id)
        if os.path.isdir(name):
            return name
        if hub == 'dir':
            pats = tuple(ignore_patterns or ()) + (LARGE_FILE_PATTERNS if ignore_model else ())
            return DirHub.snapshot_download(name, ignore_patterns=pats, cache_dir=kwargs.get('cache_dir'))
        for root in (os.environ.get('MODELSCOPE_CACHE', os.path.expanduser('~/.cache/modelscope/hub')),
                     os.path.join(os.environ.get('HF_HOME', os.path.expanduser('~/.cache/huggingface')), 'hub')):
            for cand in (os.path.join(root, name), os.path.join(root, 'models', name),
                         os.path.join(root, 'models--' + name.replace('/', '--'))):
                if os.path.isdir(cand):
                    snap = os.path.join(cand, 'snapshots')
                    if os.path.isdir(snap) and os.listdir(snap):
                        return os.path.join(snap, sorted(os.listdir(snap))[-1])
                    return cand
        try:
            if hub == 'hf':
                from huggingface_hub import snapshot_download
                return snapshot_download(name, revision=revision)
            from modelscope import snapshot_download  # type: ignore
            return snapshot_download(name, revision=revision)
        except Exception as e:
            raise FileNotFoundError(f'model {model_id!r} is not a local directory, not cached, and could not be '
                                    f'downloaded ({type(e).__name__}: {e})') from e

    @staticmethod
    def load_dataset(dataset_id: str, subset_name: Optional[str] = None, split: str = 'train', **kwargs):
        import datasets
        name, hub = _strip(dataset_id)
        if os.path.exists(name):
            ext = os.path.splitext(name)[1].lstrip('.')
            if os.path.isdir(name):
                return datasets.load_dataset(name, subset_name, split=split, **kwargs)
            fmt = {'jsonl': 'json', 'json': 'json', 'csv': 'csv', 'parquet': 'parquet', 'txt': 'text'}.get(ext, 'json')
            return datasets.load_dataset(fmt, data_files=name, split=split, **kwargs)
        if hub == 'ms':
            try:
                from modelscope import MsDataset  # type: ignore
                return MsDataset.load(name, subset_name=subset_name, split=split).to_hf_dataset()
            except ImportError:
                pass
        return datasets.load_dataset(name, subset_name, split=split, **kwargs)

    @staticmethod
    def push_to_hub(hub_model_id: str, folder: str, token: Optional[str] = None, private: bool = True,
                    async_upload: bool = False, **kwargs):
        name, hub = _strip(hub_model_id)

        def work():
            if hub == 'dir':
                return DirHub.upload_folder(name, folder, token, kwargs.get('ignore_patterns', ()))
            if hub == 'hf':
                from huggingface_hub import HfApi
                api = HfApi(token=token)
                api.create_repo(name, private=private, exist_ok=True)
                return api.upload_folder(repo_id=name, folder_path=folder)
            from modelscope.hub.api import HubApi  # type: ignore
            api = HubApi()
            if token:
                api.login(token)
            return api.upload_folder(repo_id=name, folder_path=folder)

        if async_upload:
            fut = _POOL.submit(work)
            _UPLOADS[hub_model_id] = fut
            return fut
        return work()

    @staticmethod
    def wait_for(hub_model_id: Optional[str] = None, timeout: Optional[float] = None):
        targets = [hub_model_id] if hub_model_id else list(_UPLOADS)
        return {k: _UPLOADS[k].result(timeout) for k in targets if k in _UPLOADS}

    @staticmethod
    def upload_status(hub_model_id: str) -> str:
        f = _UPLOADS.get(hub_model_id)
        if f is None:
            return 'unknown'
        if not f.done():
            return 'running'
        return 'failed' if f.exception() else 'completed'


MSHub = HFHub = HubOperation
