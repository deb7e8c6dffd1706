"""Filesystem store of training runs and control of the script processes behind them.

Parity: reference ``src/twinkle_client/auto/connection.py`` (``LocalConnection``: run directory with ``train.py``,
archived ``train_vN.py``, ``meta.json``, ``metrics.jsonl``, ``output.log``; pause = kill the stateless client,
resume = relaunch the stored script, stop = SIGTERM so the script checkpoints first).

A run is a directory ``<base>/<run_id>/``.  Training scripts are *clients* of a training server, so the server
keeps weights and optimizer state while the script process comes and goes; that is what makes "pause" a plain
kill.  Every signal goes to the one PID that this store started and recorded, never to a pattern.
"""
from __future__ import annotations

import json
import os
import re
import shutil
import signal
import subprocess
import sys
import time
from dataclasses import dataclass
from pathlib import Path
from typing import Any, Dict, List, Optional

META, SCRIPT, METRICS, OUTPUT, PROGRESS = 'meta.json', 'train.py', 'metrics.jsonl', 'output.log', 'progress.json'


def default_base_dir() -> Path:
    return Path(os.environ.get('TWINKLE_AUTO_HOME', str(Path.home() / '.cache' / 'twinkle_b200' / 'runs')))


def pid_state(pid: Optional[int]) -> str:
    """'alive', 'zombie', 'exited' or 'unknown' for a PID recorded in a run's metadata."""
    if not pid:
        return 'unknown'
    try:
        with open(f'/proc/{pid}/stat') as f:
            state = f.read().rsplit(')', 1)[1].split()[0]
        return 'zombie' if state == 'Z' else 'alive'
    except FileNotFoundError:
        return 'exited'
    except Exception:
        try:
            os.kill(pid, 0)
            return 'alive'
        except ProcessLookupError:
            return 'exited'
        except PermissionError:
            return 'alive'


@dataclass
class RunPaths:
    root: Path

    def __getattr__(self, name: str) -> Path:
        table = dict(meta=META, script=SCRIPT, metrics=METRICS, output=OUTPUT, progress=PROGRESS)
        if name in table:
            return self.root / table[name]
        raise AttributeError(name)


class RunStore:

    def __init__(self, base_dir: Optional[os.PathLike] = None, python: Optional[str] = None):
        self.base = Path(base_dir) if base_dir else default_base_dir()
        self.python = python or sys.executable
        self.selected: Optional[str] = None
        self._children: Dict[int, subprocess.Popen] = {}

    def paths(self, run_id: str) -> RunPaths:
        return RunPaths(self.base / run_id)

    # ---- metadata -------------------------------------------------------------------------------------------------
    def meta(self, run_id: str) -> Optional[Dict[str, Any]]:
        try:
            return json.loads(self.paths(run_id).meta.read_text())
        except (OSError, ValueError):
            return None

    def _write_meta(self, run_id: str, meta: Dict[str, Any]) -> None:
        p = self.paths(run_id)
        p.root.mkdir(parents=True, exist_ok=True)
        tmp = p.meta.with_suffix('.tmp')
        tmp.write_text(json.dumps(meta, indent=1, default=str))
        os.replace(tmp, p.meta)                                   # a reader never sees half a file

    def _reap(self) -> None:
        for pid, proc in list(self._children.items()):
            if proc.poll() is not None:
                del self._children[pid]

    def status(self, run_id: str) -> str:
        """The recorded status corrected by what the process is actually doing."""
        self._reap()
        meta = self.meta(run_id)
        if not meta:
            return 'unknown'
        st = meta.get('status', 'unknown')
        if st in ('running', 'starting', 'stopping') and pid_state(meta.get('pid')) != 'alive':
            st = 'stopped' if st == 'stopping' else ('completed' if meta.get('finished') else 'crashed')
            meta['status'] = st
            self._write_meta(run_id, meta)
        return st

    def list_runs(self) -> List[Dict[str, Any]]:
        out = []
        if self.base.is_dir():
            for d in sorted(self.base.iterdir()):
                meta = self.meta(d.name) if d.is_dir() else None
                if meta:
                    last = self.metrics(d.name, 1)
                    out.append(dict(run_id=d.name, model_id=meta.get('model_id', ''), status=self.status(d.name),
                                    script_version=meta.get('script_version', 1), start_time=meta.get('start_time'),
                                    last_step=last[-1].get('step') if last else None))
        return sorted(out, key=lambda r: r.get('start_time') or 0, reverse=True)

    # ---- telemetry ------------------------------------------------------------------------------------------------
    def metrics(self, run_id: str, last_n: int = 200) -> List[Dict[str, Any]]:
        try:
            lines = self.paths(run_id).metrics.read_text().splitlines()
        except OSError:
            return []
        rows = []
        for ln in lines[-last_n:]:
            try:
                rows.append(json.loads(ln))
            except ValueError:
                continue                                          # a line still being written
        return rows

    def log_tail(self, run_id: str, max_chars: int = 2000) -> str:
        p = self.paths(run_id).output
        try:
            with open(p, 'rb') as f:
                f.seek(0, 2)
                f.seek(max(0, f.tell() - max_chars))
                return f.read().decode('utf-8', 'replace')
        except OSError:
            return ''

    def script(self, run_id: str) -> str:
        try:
            return self.paths(run_id).script.read_text()
        except OSError:
            return ''

    # ---- process control ------------------------------------------------------------------------------------------
    def _launch(self, run_id: str) -> Dict[str, Any]:
        meta = self.meta(run_id)
        p = self.paths(run_id)
        if not meta or not p.script.exists():
            return dict(status='error', run_id=run_id, error=f'no script stored for run {run_id}')
        if meta.get('status') in ('running', 'starting') and pid_state(meta.get('pid')) == 'alive':
            return dict(status='error', run_id=run_id, error=f'run {run_id} is already running (pid {meta["pid"]})')
        env = dict(os.environ, TWINKLE_RUN_ID=run_id, TWINKLE_AUTO_HOME=str(self.base), PYTHONUNBUFFERED='1')
        with open(p.output, 'ab') as out:
            out.write(f'\n===== launch v{meta.get("script_version", 1)} at {time.strftime("%F %T")} =====\n'.encode())
            out.flush()
            try:
                proc = subprocess.Popen([self.python, '-u', str(p.script)], cwd=str(p.root), env=env, stdout=out,
                                        stderr=subprocess.STDOUT, stdin=subprocess.DEVNULL, start_new_session=True)
            except OSError as e:
                return dict(status='error', run_id=run_id, error=f'launch failed: {e}')
        self._children[proc.pid] = proc
        time.sleep(0.05)
        if proc.poll() is not None and proc.returncode != 0:      # syntax error, missing import …
            meta.update(status='crashed', pid=None)
            self._write_meta(run_id, meta)
            return dict(status='error', run_id=run_id, error=self.log_tail(run_id, 600) or f'exit code {proc.returncode}')
        meta.update(status='running', pid=proc.pid, finished=False, launches=meta.get('launches', 0) + 1)
        self._write_meta(run_id, meta)
        return dict(status='running', run_id=run_id, pid=proc.pid, script_path=str(p.script))

    def start(self, name: str, script: str, model_id: str = '', unique: bool = True) -> Dict[str, Any]:
        run_id = f'{re.sub(r"[^A-Za-z0-9_.-]+", "-", name).strip("-") or "run"}' + (time.strftime('_%Y%m%d_%H%M%S') if unique else '')
        n = 1
        base_id = run_id
        while (self.base / run_id).exists():
            n += 1
            run_id = f'{base_id}-{n}'
        p = self.paths(run_id)
        p.root.mkdir(parents=True)
        p.script.write_text(script)
        self._write_meta(run_id, dict(run_id=run_id, model_id=model_id, status='starting', script_version=1, start_time=time.time()))
        self.selected = run_id
        return self._launch(run_id)

    def _signal(self, run_id: str, sig: int, new_status: str) -> Dict[str, Any]:
        meta = self.meta(run_id)
        if not meta:
            return dict(status='error', run_id=run_id, error='unknown run')
        pid = meta.get('pid')
        if pid and pid_state(pid) == 'alive':
            try:
                os.kill(pid, sig)                                 # exactly the PID this store launched
            except (ProcessLookupError, PermissionError):
                pass
        meta['status'] = new_status
        self._write_meta(run_id, meta)
        return dict(status=new_status, run_id=run_id, pid=pid)

    def pause(self, run_id: str) -> Dict[str, Any]:
        return self._signal(run_id, signal.SIGKILL, 'paused')

    def stop(self, run_id: str) -> Dict[str, Any]:
        return self._signal(run_id, signal.SIGTERM, 'stopping')

    def resume(self, run_id: str) -> Dict[str, Any]:
        return self._launch(run_id)

    def wait(self, run_id: str, timeout: float = 30.0) -> str:
        """Block until the run's process is gone (tests and scripted use)."""
        end = time.time() + timeout
        while time.time() < end:
            self._reap()
            meta = self.meta(run_id) or {}
            if pid_state(meta.get('pid')) != 'alive':
                break
            time.sleep(0.05)
        return self.status(run_id)

    def update_script(self, run_id: str, script: str) -> Dict[str, Any]:
        p = self.paths(run_id)
        p.root.mkdir(parents=True, exist_ok=True)
        version = 1
        if p.script.exists():
            taken = [int(m.group(1)) for f in p.root.glob('train_v*.py') if (m := re.fullmatch(r'train_v(\d+)\.py', f.name))]
            archive = max(taken, default=0) + 1
            shutil.copy2(p.script, p.root / f'train_v{archive}.py')
            version = archive + 1
        p.script.write_text(script)
        meta = self.meta(run_id) or dict(run_id=run_id, start_time=time.time(), status='created')
        meta['script_version'] = version
        self._write_meta(run_id, meta)
        return dict(run_id=run_id, script_version=version, script_path=str(p.script))
