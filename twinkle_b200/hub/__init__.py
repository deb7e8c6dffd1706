"""Model / dataset hub access.

Parity: reference ``src/twinkle/hub/hub.py:31-657`` — ``ms://`` and ``hf://``
prefixes, ``download_model``, ``load_dataset``, ``push_to_hub`` (optionally on a
background thread with ``wait_for``) and the server's model-alias table.  The
network is optional: a local directory always resolves to itself, and remote
ids are looked up in the local HF / ModelScope caches before any client
library is asked to download.
"""
from __future__ import annotations

import os
import threading
from concurrent.futures import Future, ThreadPoolExecutor
from typing import Any, Dict, Optional

_POOL = ThreadPoolExecutor(max_workers=2, thread_name_prefix='hub-upload')
_UPLOADS: Dict[str, Future] = {}
MODEL_ALIASES: Dict[str, str] = {}


def _strip(model_id: str):
    for p, hub in (('ms://', 'ms'), ('hf://', 'hf')):
        if model_id.startswith(p):
            return model_id[len(p):], hub
    return model_id, os.environ.get('TWINKLE_DEFAULT_HUB', 'ms')


class HubOperation:

    @staticmethod
    def resolve_alias(model_id: str) -> str:
        return MODEL_ALIASES.get(model_id, model_id)

    @staticmethod
    def download_model(model_id: str, revision: Optional[str] = None, **kwargs) -> str:
        model_id = HubOperation.resolve_alias(model_id)
        if os.path.isdir(model_id):
            return model_id
        name, hub = _strip(model_id)
        if os.path.isdir(name):
            return name
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
