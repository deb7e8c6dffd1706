"""Tools the auto agent may call, with their JSON schemas and a dispatcher.

Parity: reference ``src/twinkle_client/auto/agent/tools.py`` (``ToolExecutor``: list / status / start / select /
pause / resume / stop / update_script, start_server / shutdown_server with a generated config, list supported
models, hub search, cluster info).  Differences by design: the server started here is this package's own
(``python -m twinkle_b200.server.launcher launch``), there is no Ray cluster to bring up, and hub search looks
only at what is cached locally because training hosts are commonly offline.
"""
from __future__ import annotations

import json
import os
import signal
import subprocess
import sys
import time
from pathlib import Path
from typing import Any, Callable, Dict, List, Optional

from .runs import RunStore, pid_state


def _fn(name: str, description: str, props: Dict[str, Any], required: List[str]) -> Dict[str, Any]:
    return dict(type='function', function=dict(name=name, description=description,
                                               parameters=dict(type='object', properties=props, required=required)))


_S, _I = dict(type='string'), dict(type='integer')
TOOL_SCHEMAS: List[Dict[str, Any]] = [
    _fn('list_training_runs', 'All known runs, newest first, with status and last step.', {}, []),
    _fn('get_training_status', 'Status, recent metrics and the log tail of one run.', dict(run_id=_S), ['run_id']),
    _fn('start_training', 'Store a complete Python training script as a new run and launch it.',
        dict(run_id=dict(type='string', description='short name; a timestamp is appended'), script_content=_S, model_id=_S), ['run_id', 'script_content']),
    _fn('select_run', 'Make a run the one shown in the panels and watched by the monitor.', dict(run_id=_S), ['run_id']),
    _fn('pause_training', 'Kill the script process; the server keeps model and optimizer state.', dict(run_id=_S), ['run_id']),
    _fn('resume_training', 'Relaunch the stored script of a paused, stopped or crashed run.', dict(run_id=_S), ['run_id']),
    _fn('stop_training', 'SIGTERM: the script saves a checkpoint and exits.', dict(run_id=_S), ['run_id']),
    _fn('update_script', 'Replace the stored script (the old one is archived); does not relaunch.', dict(run_id=_S, script_content=_S), ['run_id', 'script_content']),
    _fn('start_server', 'Start a local training server for a base model, optionally with sampler GPUs.',
        dict(model_id=_S, train_gpus=_I, sampler_gpus=_I, port=_I, max_loras=_I, max_lora_rank=_I), ['model_id']),
    _fn('shutdown_server', 'Stop the server this agent started.', {}, []),
    _fn('list_supported_models', 'Ask a running server which base models it serves.', dict(base_url=_S), []),
    _fn('search_models', 'Search locally cached models by substring.', dict(query=_S, limit=_I), ['query']),
    _fn('search_datasets', 'Search locally cached datasets by substring.', dict(query=_S, limit=_I), ['query']),
    _fn('get_cluster_info', 'GPUs (name, memory, utilisation) and CPU/RAM of this host.', {}, []),
]


def split_gpus(total: int, train: Optional[int] = None, sampler: Optional[int] = None) -> Dict[str, List[int]]:
    """Device ids for trainer and sampler.  Unspecified: everything trains on ≤ 2 GPUs; otherwise a quarter
    (at least one) samples.  Requests are clamped to what exists; the trainer keeps at least one GPU."""
    total = max(int(total), 0)
    if total == 0:
        return dict(train=[], sampler=[])
    if sampler is None:
        sampler = 0 if (train is not None and train >= total) or total <= 2 else max(1, total // 4)
    sampler = max(0, min(int(sampler), total - 1))
    train = total - sampler if train is None else max(1, min(int(train), total - sampler))
    ids = list(range(total))
    return dict(train=ids[:train], sampler=ids[train:train + sampler])


def server_config(model_id: str, gpus: Dict[str, List[int]], port: int = 8000, max_loras: int = 4, max_lora_rank: int = 32,
                  persistence_path: Optional[str] = None) -> Dict[str, Any]:
    """The YAML document (as a dict) for ``twinkle-server launch``: one model application on the training GPUs,
    one sampler application when sampler GPUs are given, the Tinker-compatible gateway, file persistence."""
    short = model_id.rstrip('/').split('/')[-1]
    n_train, n_samp = max(len(gpus['train']), 1), len(gpus['sampler'])
    apps: List[Dict[str, Any]] = [
        dict(name=f'models-{short}', route_prefix=f'/model/{model_id}', import_path='model',
             args=dict(model_id=model_id, nproc_per_node=n_train, device_group=dict(name='model', ranks=gpus['train'] or 1),
                       device_mesh=dict(dp_size=n_train), max_loras=max_loras, max_r=max_lora_rank)),
        dict(name='processor', route_prefix='/processor', import_path='processor', args={}),
    ]
    if n_samp:
        apps.append(dict(name=f'sampler-{short}', route_prefix=f'/sampler/{model_id}', import_path='sampler',
                         args=dict(model_id=model_id, sampler_type='torch', nproc_per_node=n_samp,
                                   device_group=dict(name='sampler', ranks=gpus['sampler']), device_mesh=dict(dp_size=n_samp), max_loras=max_loras)))
    apps.append(dict(name='server', route_prefix='/api/v1', import_path='server', args=dict(supported_models=[model_id])))
    return dict(http_options=dict(host='127.0.0.1', port=int(port)), applications=apps,
                persistence=dict(mode='file', file_path=persistence_path or str(Path.home() / '.cache' / 'twinkle_b200' / 'server_state.json')))


class ToolExecutor:

    def __init__(self, store: RunStore, on_select: Optional[Callable[[str], None]] = None):
        self.store = store
        self.on_select = on_select
        self.server_url = os.environ.get('TWINKLE_SERVER_URL', '')
        self._server: Optional[subprocess.Popen] = None
        self._server_log: Optional[Path] = None

    # ---- dispatch ---------------------------------------------------------------------------------------------------
    def execute(self, name: str, arguments: Dict[str, Any]) -> str:
        """Always returns a JSON string: the tool's result or ``{'error': ...}``; a tool never raises into the
        conversation loop."""
        fn = getattr(self, f'tool_{name}', None)
        if fn is None:
            return json.dumps(dict(error=f'unknown tool {name!r}', available=[t['function']['name'] for t in TOOL_SCHEMAS]))
        try:
            return json.dumps(fn(**(arguments or {})), default=str, ensure_ascii=False)
        except TypeError as e:
            return json.dumps(dict(error=f'bad arguments for {name}: {e}'))
        except Exception as e:
            return json.dumps(dict(error=f'{type(e).__name__}: {e}'))

    # ---- runs -------------------------------------------------------------------------------------------------------
    def tool_list_training_runs(self):
        return self.store.list_runs()

    def tool_get_training_status(self, run_id: str):
        meta = self.store.meta(run_id)
        if not meta:
            return dict(error=f'unknown run {run_id}')
        return dict(run_id=run_id, status=self.store.status(run_id), process=pid_state(meta.get('pid')), model_id=meta.get('model_id', ''),
                    script_version=meta.get('script_version', 1), recent_metrics=self.store.metrics(run_id, 10), log_tail=self.store.log_tail(run_id, 1500))

    def _select(self, run_id: str) -> None:
        self.store.selected = run_id
        if self.on_select:
            self.on_select(run_id)

    def tool_start_training(self, run_id: str, script_content: str, model_id: str = ''):
        try:
            compile(script_content, 'train.py', 'exec')           # refuse what cannot even parse
        except SyntaxError as e:
            return dict(status='error', error=f'script does not parse: line {e.lineno}: {e.msg}')
        res = self.store.start(run_id, script_content, model_id)
        if res.get('run_id'):
            self._select(res['run_id'])
        return res

    def tool_select_run(self, run_id: str):
        if not self.store.meta(run_id):
            return dict(error=f'unknown run {run_id}')
        self._select(run_id)
        return dict(selected=run_id)

    def tool_pause_training(self, run_id: str):
        return self.store.pause(run_id)

    def tool_resume_training(self, run_id: str):
        return self.store.resume(run_id)

    def tool_stop_training(self, run_id: str):
        return self.store.stop(run_id)

    def tool_update_script(self, run_id: str, script_content: str):
        try:
            compile(script_content, 'train.py', 'exec')
        except SyntaxError as e:
            return dict(status='error', error=f'script does not parse: line {e.lineno}: {e.msg}')
        return self.store.update_script(run_id, script_content)

    # ---- server -----------------------------------------------------------------------------------------------------
    def _healthy(self, url: str, timeout: float = 2.0) -> bool:
        try:
            import requests
            return requests.get(url.rstrip('/') + '/healthz', timeout=timeout).status_code == 200
        except Exception:
            return False

    def tool_start_server(self, model_id: str, train_gpus: Optional[int] = None, sampler_gpus: Optional[int] = None, port: int = 8000,
                          max_loras: int = 4, max_lora_rank: int = 32, wait_seconds: float = 600.0):
        url = f'http://127.0.0.1:{int(port)}'
        if self._healthy(url):
            self.server_url = url
            return dict(status='already_running', base_url=url)
        import yaml
        gpus = split_gpus(self.gpu_count(), train_gpus, sampler_gpus)
        cfg_dir = self.store.base / '_server'
        cfg_dir.mkdir(parents=True, exist_ok=True)
        cfg_path, self._server_log = cfg_dir / 'server.yaml', cfg_dir / 'server.log'
        cfg_path.write_text(yaml.safe_dump(server_config(model_id, gpus, port, max_loras, max_lora_rank, str(cfg_dir / 'state.json')), sort_keys=False))
        with open(self._server_log, 'ab') as out:
            self._server = subprocess.Popen([sys.executable, '-m', 'twinkle_b200.server.launcher', 'launch', '--config', str(cfg_path)],
                                            stdout=out, stderr=subprocess.STDOUT, stdin=subprocess.DEVNULL, start_new_session=True)
        end = time.time() + wait_seconds
        while time.time() < end:
            if self._server.poll() is not None:
                return dict(status='error', error='server exited during start-up', log_tail=self._tail(self._server_log))
            if self._healthy(url):
                self.server_url = url
                return dict(status='running', base_url=url, pid=self._server.pid, gpus=gpus, config=str(cfg_path))
            time.sleep(1.0)
        return dict(status='error', error=f'server not healthy after {wait_seconds:.0f}s', log_tail=self._tail(self._server_log))

    @staticmethod
    def _tail(path: Optional[Path], n: int = 1500) -> str:
        try:
            return path.read_text(errors='replace')[-n:] if path else ''
        except OSError:
            return ''

    def tool_shutdown_server(self):
        if self._server is None or self._server.poll() is not None:
            return dict(status='not_running')
        pid = self._server.pid
        os.kill(pid, signal.SIGTERM)                              # the one process this executor started
        try:
            self._server.wait(timeout=30)
        except subprocess.TimeoutExpired:
            os.kill(pid, signal.SIGKILL)
            self._server.wait(timeout=10)
        self._server = None
        return dict(status='stopped', pid=pid)

    def tool_list_supported_models(self, base_url: Optional[str] = None):
        import requests
        url = (base_url or self.server_url or 'http://127.0.0.1:8000').rstrip('/')
        r = requests.get(url + '/api/v1/get_server_capabilities', timeout=10, headers={'Twinkle-Authorization': os.environ.get('TWINKLE_SERVER_TOKEN', 'anonymous')})
        r.raise_for_status()
        return dict(base_url=url, supported_models=r.json().get('supported_models', []))

    # ---- hub (local caches only) -----------------------------------------------------------------------------------
    @staticmethod
    def _cache_roots(kind: str) -> List[Path]:
        home = Path.home()
        sub = 'models' if kind == 'model' else 'datasets'
        roots = [Path(os.environ.get('MODELSCOPE_CACHE', str(home / '.cache' / 'modelscope'))) / 'hub' / sub,
                 Path(os.environ.get('HF_HOME', str(home / '.cache' / 'huggingface'))) / 'hub']
        extra = os.environ.get('TWINKLE_LOCAL_HUB')
        return ([Path(extra) / sub] if extra else []) + roots

    def _search(self, kind: str, query: str, limit: int) -> Dict[str, Any]:
        q, hits = query.lower(), []
        for root in self._cache_roots(kind):
            if not root.is_dir():
                continue
            for org in sorted(root.iterdir()):
                if not org.is_dir():
                    continue
                if org.name.startswith(f'{kind}s--'):             # huggingface layout: models--org--name
                    ident, path = org.name.split('--', 1)[1].replace('--', '/'), org
                    cands = [(ident, path)]
                else:
                    cands = [(f'{org.name}/{d.name}', d) for d in sorted(org.iterdir()) if d.is_dir()]
                hits += [dict(id=i, path=str(p)) for i, p in cands if q in i.lower()]
        return dict(query=query, source='local caches', results=hits[:max(int(limit), 1)])

    def tool_search_models(self, query: str, limit: int = 5):
        return self._search('model', query, limit)

    def tool_search_datasets(self, query: str, limit: int = 5):
        return self._search('dataset', query, limit)

    # ---- host -------------------------------------------------------------------------------------------------------
    @staticmethod
    def _nvidia_smi() -> List[Dict[str, Any]]:
        try:
            out = subprocess.run(['nvidia-smi', '--query-gpu=index,name,memory.total,memory.used,utilization.gpu', '--format=csv,noheader,nounits'],
                                 capture_output=True, text=True, timeout=10)
        except (OSError, subprocess.TimeoutExpired):
            return []
        gpus = []
        for ln in out.stdout.splitlines() if out.returncode == 0 else []:
            f = [x.strip() for x in ln.split(',')]
            if len(f) == 5:
                gpus.append(dict(index=int(f[0]), name=f[1], memory_total_mib=int(f[2]), memory_used_mib=int(f[3]), utilization_pct=int(f[4])))
        return gpus

    def gpu_count(self) -> int:
        vis = os.environ.get('CUDA_VISIBLE_DEVICES')
        if vis is not None:
            return len([v for v in vis.split(',') if v.strip() and v.strip() != '-1'])
        return len(self._nvidia_smi())

    def tool_get_cluster_info(self):
        import psutil
        vm = psutil.virtual_memory()
        return dict(gpus=self._nvidia_smi(), gpu_count=self.gpu_count(), cpu_count=os.cpu_count(), ram_total_gib=round(vm.total / 2**30, 1),
                    ram_available_gib=round(vm.available / 2**30, 1), server_url=self.server_url or None)
