"""Periodic health check of the selected run: gather every signal, ask the model, act on its verdict.

Parity: reference ``src/twinkle_client/auto/agent/monitor.py`` (``TrainingMonitor``: snapshot of process state,
log tail, metrics, stall time and the script; verdict LGTM / WARNING / FIX with a complete fixed script that is
applied and relaunched; at most three automatic fixes per run; unchanged snapshots are not re-analysed).
Added here: cheap local findings (non-finite loss, dead process, stall) are computed before the model is asked
and handed to it as facts, and a healthy, progressing run with nothing new in its log costs no model call.
"""
from __future__ import annotations

import hashlib
import json
import re
import threading
import time
from typing import Any, Callable, Dict, List, Optional, Tuple

from .runs import RunStore, pid_state

MAX_FIX_ATTEMPTS = 3
ERROR_MARKERS = ('Traceback (most recent call last)', 'Error:', 'CUDA out of memory', 'HTTP 4', 'HTTP 5', 'Connection refused')

MONITOR_PROMPT = """\
You watch one LLM training run. You receive a snapshot: process state, seconds since the last new metric, local \
findings, the tail of the combined stdout/stderr, recent metrics, and the current train.py. Answer in exactly one \
of three forms.

LGTM
  when the process is alive, metrics advance and nothing in the log needs attention (a stall under three minutes \
is normal).

A one-to-three sentence observation with a suggestion
  when something deserves the user's attention but the script itself is not broken: plateau, exploding KL or \
gradient norm, collapsing entropy, reward hacking, a slow step rate.

```diagnosis
<root cause in one or two sentences>
```
```python
<the complete corrected train.py>
```
  when the script crashed or cannot make progress because of its own code. Change only what causes the failure; \
keep the resume logic (rt.get_resume_info(), dataloader.skip_consumed_samples) and the metric reporting intact. \
Do not propose a fix for a transient condition such as a brief network error.
"""


def local_findings(snapshot: Dict[str, Any]) -> List[str]:
    out = []
    if snapshot['process'] in ('exited', 'zombie') and snapshot['status'] not in ('completed', 'stopped', 'paused'):
        out.append(f'process is {snapshot["process"]} but the run never reported completion')
    rows = snapshot['metrics']
    for key in ('loss', 'grad_norm', 'kl'):
        vals = [r.get(key) for r in rows if key in r]
        if vals and isinstance(vals[-1], str) and vals[-1].lower() in ('nan', 'inf', '-inf'):
            out.append(f'{key} is {vals[-1]} at step {rows[-1].get("step")}')
    losses = [r['loss'] for r in rows if isinstance(r.get('loss'), (int, float))]
    if len(losses) >= 8 and min(losses[-4:]) > 2.0 * max(min(losses[:-4]), 1e-8):
        out.append(f'loss rose from a low of {min(losses[:-4]):.4g} to {losses[-1]:.4g}')
    if snapshot['process'] == 'alive' and snapshot['stall_seconds'] > 600:
        out.append(f'no new metric for {snapshot["stall_seconds"]:.0f} s')
    if any(m in snapshot['log_tail'] for m in ERROR_MARKERS):
        out.append('the log tail contains an error marker')
    return out


def parse_verdict(response: str) -> Tuple[str, str, str]:
    """('lgtm' | 'warning' | 'fix', text, script)."""
    text = (response or '').strip()
    code = re.search(r'```python\s*\n(.*?)```', text, re.S)
    if code and code.group(1).strip():
        diag = re.search(r'```diagnosis\s*\n(.*?)```', text, re.S)
        if diag:
            why = diag.group(1).strip()
        else:
            before = [ln.strip() for ln in text[:code.start()].splitlines() if ln.strip() and not ln.startswith('```')]
            why = before[-1] if before else 'automatic fix'
        return 'fix', why, code.group(1).strip() + '\n'
    if text.upper().startswith('LGTM') or not text:
        return 'lgtm', '', ''
    return 'warning', text, ''


class TrainingMonitor:

    def __init__(self, store: RunStore, llm, on_message: Callable[[str], None], poll_interval: float = 30.0, max_metrics: int = 30,
                 clock: Callable[[], float] = time.time):
        self.store, self.llm, self.on_message = store, llm, on_message
        self.poll_interval, self.max_metrics, self.clock = poll_interval, max_metrics, clock
        self.fix_attempts: Dict[str, int] = {}
        self._run: Optional[str] = None
        self._last_step: Any = None
        self._last_progress = clock()
        self._last_hash = ''
        self._stop = threading.Event()
        self._thread: Optional[threading.Thread] = None

    # ---- thread -----------------------------------------------------------------------------------------------------
    def start(self) -> None:
        self._stop.clear()
        self._thread = threading.Thread(target=self._loop, name='twinkle-auto-monitor', daemon=True)
        self._thread.start()

    def stop(self) -> None:
        self._stop.set()
        if self._thread is not None:
            self._thread.join(timeout=5)

    def _loop(self) -> None:
        while not self._stop.wait(self.poll_interval):
            try:
                self.check()
            except Exception as e:                                # the monitor must outlive a bad cycle
                self.on_message(f'[monitor] cycle failed: {e!r}')

    # ---- one cycle --------------------------------------------------------------------------------------------------
    def snapshot(self, run_id: str) -> Dict[str, Any]:
        """Everything known about the run.  The log is cut at the latest launch banner so that a traceback from a
        previous version of the script is not held against the current one."""
        meta = self.store.meta(run_id) or {}
        rows = self.store.metrics(run_id, self.max_metrics)
        step = rows[-1].get('step') if rows else None
        if run_id != self._run:
            self._run, self._last_step, self._last_progress, self._last_hash = run_id, step, self.clock(), ''
        elif step != self._last_step:
            self._last_step, self._last_progress = step, self.clock()
        snap = dict(run_id=run_id, status=self.store.status(run_id), process=pid_state(meta.get('pid')), model_id=meta.get('model_id', ''),
                    script_version=meta.get('script_version', 1), metrics=rows, stall_seconds=self.clock() - self._last_progress,
                    log_tail=self.store.log_tail(run_id, 3000).rsplit('===== launch ', 1)[-1], script=self.store.script(run_id), fix_attempts=self.fix_attempts.get(run_id, 0))
        snap['findings'] = local_findings(snap)
        return snap

    @staticmethod
    def fingerprint(snap: Dict[str, Any]) -> str:
        """Equal while nothing observable changed: stall time is bucketed to whole minutes on purpose."""
        key = (snap['status'], snap['process'], snap['script_version'], snap['metrics'][-1].get('step') if snap['metrics'] else None,
               snap['log_tail'][-500:], int(snap['stall_seconds'] // 60), tuple(snap['findings']))
        return hashlib.sha1(repr(key).encode()).hexdigest()

    @staticmethod
    def render(snap: Dict[str, Any]) -> str:
        parts = [f'## Run {snap["run_id"]} (model {snap["model_id"] or "?"}, script v{snap["script_version"]})',
                 f'- recorded status: {snap["status"]}\n- process: {snap["process"]}\n- seconds since last new metric: {snap["stall_seconds"]:.0f}',
                 '## Local findings\n' + ('\n'.join(f'- {f}' for f in snap['findings']) or '- none'),
                 '## output.log (tail)\n```\n' + (snap['log_tail'] or '(empty)') + '\n```',
                 '## Recent metrics\n' + ('\n'.join(json.dumps({k: v for k, v in r.items() if k != 'time'}) for r in snap['metrics'][-15:]) or '(none yet)')]
        if snap['script']:
            parts.append('## Current train.py\n```python\n' + snap['script'] + '\n```')
        return '\n\n'.join(parts)

    def check(self) -> str:
        """Run one cycle; returns what was done: 'idle', 'unchanged', 'healthy', 'lgtm', 'warning', 'fix',
        'fix-refused' or 'llm-error'."""
        run_id = self.store.selected
        if not run_id or not self.store.meta(run_id):
            return 'idle'
        snap = self.snapshot(run_id)
        if snap['status'] in ('completed', 'stopped', 'paused') and not snap['findings']:
            return 'idle'
        fp = self.fingerprint(snap)
        if fp == self._last_hash:
            return 'unchanged'
        self._last_hash = fp
        if snap['process'] == 'alive' and not snap['findings'] and snap['stall_seconds'] < 180 and snap['metrics']:
            return 'healthy'
        note = '\n\nAutomatic fixes are used up for this run: do not answer with a fixed script.' if snap['fix_attempts'] >= MAX_FIX_ATTEMPTS else ''
        try:
            reply = self.llm.chat([dict(role='system', content=MONITOR_PROMPT + note), dict(role='user', content=self.render(snap))],
                                  temperature=0.3, max_tokens=4096)
        except Exception as e:
            self.on_message(f'[monitor] model call failed: {e!r}')
            return 'llm-error'
        kind, text, script = parse_verdict(reply.get('content', ''))
        if kind == 'warning':
            self.on_message(f'[monitor] {text}')
        elif kind == 'fix':
            return self._apply_fix(run_id, text, script)
        return kind

    def _apply_fix(self, run_id: str, diagnosis: str, script: str) -> str:
        n = self.fix_attempts.get(run_id, 0)
        if n >= MAX_FIX_ATTEMPTS:
            self.on_message(f'[monitor] {MAX_FIX_ATTEMPTS} automatic fixes already tried on {run_id}; leaving it to you. Last diagnosis: {diagnosis}')
            return 'fix-refused'
        try:
            compile(script, 'train.py', 'exec')
        except SyntaxError as e:
            self.fix_attempts[run_id] = n + 1
            self.on_message(f'[monitor] proposed fix does not parse (line {e.lineno}: {e.msg}); not applied')
            return 'fix-refused'
        self.fix_attempts[run_id] = n + 1
        self.on_message(f'[monitor] fixing {run_id} (attempt {n + 1}/{MAX_FIX_ATTEMPTS}): {diagnosis}')
        if pid_state((self.store.meta(run_id) or {}).get('pid')) == 'alive':
            self.store.pause(run_id)
            self.store.wait(run_id, 10)
        up = self.store.update_script(run_id, script)
        res = self.store.resume(run_id)
        if res.get('status') == 'error':
            self.on_message(f'[monitor] relaunch failed: {res.get("error", "?")[:500]}')
        else:
            self.on_message(f'[monitor] script v{up["script_version"]} relaunched (pid {res.get("pid")})')
            self._last_progress, self._last_step, self._last_hash = self.clock(), None, ''
        return 'fix'
