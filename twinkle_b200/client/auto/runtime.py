"""What a generated training script imports to be observable and controllable by the auto agent.

Parity: reference ``src/twinkle_client/auto/runtime.py`` (``TrainingRuntime``: ``start`` / ``log_metrics`` / ``log``
/ ``get_resume_info`` / ``finish`` / ``register_graceful_shutdown``).

    rt = TrainingRuntime()                    # run id comes from the launcher's environment
    rt.start(model_id='Qwen/Qwen3-8B', config={...})
    step0 = rt.get_resume_info()['global_step']
    rt.register_graceful_shutdown(lambda: model.save('last'))
    for step in range(step0, n):
        ...
        rt.log_metrics(step=step, loss=loss, lr=lr)
    rt.finish()
"""
from __future__ import annotations

import json
import math
import os
import signal
import sys
import time
from pathlib import Path
from typing import Any, Callable, Dict, Optional

from .runs import META, METRICS, PROGRESS, default_base_dir


class TrainingRuntime:

    def __init__(self, run_id: Optional[str] = None, base_dir: Optional[os.PathLike] = None):
        self.run_id = run_id or os.environ.get('TWINKLE_RUN_ID') or f'run_{time.strftime("%Y%m%d_%H%M%S")}'
        self.root = (Path(base_dir) if base_dir else default_base_dir()) / self.run_id
        self.root.mkdir(parents=True, exist_ok=True)
        self._progress: Dict[str, int] = {}
        self._t0 = time.time()

    # ---- metadata ---------------------------------------------------------------------------------------------------
    def _meta(self) -> Dict[str, Any]:
        try:
            return json.loads((self.root / META).read_text())
        except (OSError, ValueError):
            return dict(run_id=self.run_id)

    def _write_meta(self, meta: Dict[str, Any]) -> None:
        tmp = self.root / (META + '.tmp')
        tmp.write_text(json.dumps(meta, indent=1, default=str))
        os.replace(tmp, self.root / META)

    def start(self, model_id: str = '', config: Optional[Dict[str, Any]] = None, **extra: Any) -> None:
        meta = self._meta()
        meta.update(model_id=model_id or meta.get('model_id', ''), config=config or {}, status='running', pid=os.getpid(),
                    finished=False, **extra)
        meta.setdefault('start_time', time.time())
        self._write_meta(meta)
        self.log(f'run {self.run_id} started (model={model_id or "?"})')

    # ---- telemetry --------------------------------------------------------------------------------------------------
    def log_metrics(self, **values: Any) -> None:
        """One JSON line per step.  Tensors and numpy scalars become floats; NaN/inf become strings so the file
        stays strict JSON and the monitor can still see them."""
        row: Dict[str, Any] = dict(time=time.time())
        for k, v in values.items():
            if hasattr(v, 'item'):
                try:
                    v = v.item()
                except Exception:
                    v = str(v)
            if isinstance(v, float) and not math.isfinite(v):
                v = str(v)
            row[k] = v
        with open(self.root / METRICS, 'a') as f:
            f.write(json.dumps(row, default=str) + '\n')
        step = row.get('step')
        if isinstance(step, int):
            self._progress['global_step'] = step + 1
            for k in ('consumed_samples', 'epoch'):
                if isinstance(row.get(k), int):
                    self._progress[k] = row[k]
            self._save_progress()

    def log(self, message: str) -> None:
        print(f'[{time.strftime("%T")}] {message}', flush=True)

    # ---- resume -----------------------------------------------------------------------------------------------------
    def _save_progress(self) -> None:
        tmp = self.root / (PROGRESS + '.tmp')
        tmp.write_text(json.dumps(self._progress))
        os.replace(tmp, self.root / PROGRESS)

    def get_resume_info(self) -> Dict[str, int]:
        """Where a relaunched script continues: the step after the last logged one, and the samples consumed."""
        info = dict(global_step=0, consumed_samples=0, epoch=0)
        try:
            info.update({k: int(v) for k, v in json.loads((self.root / PROGRESS).read_text()).items()})
        except (OSError, ValueError):
            pass
        self._progress.update(info)
        return info

    # ---- lifecycle --------------------------------------------------------------------------------------------------
    def finish(self, status: str = 'completed') -> None:
        meta = self._meta()
        meta.update(status=status, finished=True, end_time=time.time(), wall_seconds=round(time.time() - self._t0, 1))
        self._write_meta(meta)
        self.log(f'run {self.run_id} {status}')

    def register_graceful_shutdown(self, save: Optional[Callable[[], Any]] = None, model: Any = None, dataloader: Any = None,
                                   checkpoint_name: str = 'interrupted') -> None:
        """SIGTERM → save a checkpoint (``save()``, or ``model.save(checkpoint_name)``), record the dataloader
        position, mark the run stopped, exit 0."""

        def handler(signum, frame):
            self.log('SIGTERM: saving before exit')
            try:
                if save is not None:
                    save()
                elif model is not None:
                    model.save(checkpoint_name)
                if dataloader is not None and hasattr(dataloader, 'get_state'):
                    state = dataloader.get_state()
                    if isinstance(state, dict) and 'consumed_samples' in state:
                        self._progress['consumed_samples'] = int(state['consumed_samples'])
                        self._save_progress()
            except Exception as e:                                  # the exit must still happen
                self.log(f'save on shutdown failed: {e!r}')
            self.finish('stopped')
            sys.exit(0)

        signal.signal(signal.SIGTERM, handler)
