"""Terminal front end of the auto agent.

Parity: reference ``src/twinkle_client/auto/app.py`` (a full-screen app with a chat pane, a run/metrics pane and a
log pane) and ``auto/__main__.py``.  The ``textual`` toolkit is not a dependency of this package, so the screen is
built with ``rich``: a status header (selected run, state, last metrics, a loss sparkline) is printed before each
prompt, the conversation scrolls below it, and monitor messages are queued by the monitor thread and shown at the next
prompt.  Slash commands cover what the panes did: ``/runs``, ``/select``, ``/log``, ``/metrics``, ``/skills``,
``/pause``, ``/resume``, ``/stop``, ``/quit``.  ``--once TEXT`` runs a single turn without a terminal.
"""
from __future__ import annotations

import argparse
import queue
import sys
from typing import List, Optional

from ..skills import default_manager
from .agent import AgentLoop
from .llm import ChatLLM, ScriptedLLM
from .monitor import TrainingMonitor
from .runs import RunStore
from .tools import ToolExecutor

BARS = ' ▁▂▃▄▅▆▇█'


def sparkline(values: List[float], width: int = 40) -> str:
    vals = [v for v in values if isinstance(v, (int, float)) and v == v and abs(v) != float('inf')][-width:]
    if not vals:
        return ''
    lo, hi = min(vals), max(vals)
    return ''.join(BARS[1 + int((v - lo) / (hi - lo) * (len(BARS) - 2))] if hi > lo else BARS[4] for v in vals)


def header_lines(store: RunStore) -> List[str]:
    rid = store.selected
    if not rid:
        return ['no run selected  (/runs to list, or ask for a training run)']
    rows = store.metrics(rid, 60)
    last = {k: v for k, v in (rows[-1] if rows else {}).items() if k != 'time'}
    fmt = ' '.join(f'{k}={v:.4g}' if isinstance(v, float) else f'{k}={v}' for k, v in last.items())
    return [f'run {rid}  [{store.status(rid)}]  {fmt}'.rstrip(), 'loss ' + sparkline([r.get('loss') for r in rows])]


class AutoApp:

    def __init__(self, store: RunStore, llm, monitor_llm=None, poll_interval: float = 30.0, skills_dirs: Optional[List[str]] = None,
                 out=None, monitor: bool = True):
        self.store = store
        self.out = out or sys.stdout
        self.pending: 'queue.Queue[str]' = queue.Queue()
        self.executor = ToolExecutor(store)
        self.agent = AgentLoop(llm, self.executor, on_tool=self._on_tool)
        self.skills = default_manager(skills_dirs)
        self.skills.load_all()
        self.agent.inject_skills(self.skills.format_for_prompt())
        self.monitor = TrainingMonitor(store, monitor_llm or llm, self._on_monitor, poll_interval) if monitor else None

    # ---- output -----------------------------------------------------------------------------------------------------
    def say(self, text: str = '', end: str = '\n') -> None:
        self.out.write(text + end)
        self.out.flush()
        if text + end:
            self._bol = (text + end).endswith('\n')

    def fresh_line(self) -> None:
        if not getattr(self, '_bol', True):
            self.say()

    def _on_tool(self, name, arguments, result) -> None:
        self.fresh_line()
        brief = {k: (v if len(str(v)) < 60 else f'<{len(str(v))} chars>') for k, v in arguments.items()}
        self.say(f'  · {name}({brief}) → {result[:160]}{"…" if len(result) > 160 else ""}')

    def _on_monitor(self, text: str) -> None:
        self.pending.put(text)
        self.agent.note(text)

    def drain(self) -> None:
        while not self.pending.empty():
            self.say(self.pending.get_nowait())

    # ---- commands ---------------------------------------------------------------------------------------------------
    def command(self, line: str) -> bool:
        """Handle a slash command; False means quit."""
        cmd, _, arg = line[1:].partition(' ')
        arg = arg.strip() or (self.store.selected or '')
        if cmd in ('quit', 'exit', 'q'):
            return False
        if cmd == 'runs':
            for r in self.store.list_runs() or [dict(run_id='(none)', status='', last_step='', model_id='')]:
                mark = '*' if r['run_id'] == self.store.selected else ' '
                self.say(f' {mark} {r["run_id"]:<40} {r["status"]:<10} step={r.get("last_step")} {r.get("model_id", "")}')
        elif cmd == 'select':
            self.say(self.executor.execute('select_run', dict(run_id=arg)))
        elif cmd == 'log':
            self.say(self.store.log_tail(arg, 4000) or '(no output yet)')
        elif cmd == 'metrics':
            for r in self.store.metrics(arg, 15):
                self.say('  ' + ' '.join(f'{k}={v}' for k, v in r.items() if k != 'time'))
        elif cmd == 'skills':
            for s in self.skills.skills:
                self.say(f'  {s.name:<24} [{s.source}] {s.description[:90]}')
            for k, v in self.skills.errors.items():
                self.say(f'  ! {k}: {v}')
        elif cmd in ('pause', 'resume', 'stop'):
            self.say(self.executor.execute(f'{cmd}_training', dict(run_id=arg)))
        elif cmd == 'check' and self.monitor:
            self.say(f'monitor: {self.monitor.check()}')
            self.drain()
        else:
            self.say('commands: /runs /select ID /log [ID] /metrics [ID] /skills /pause /resume /stop /check /quit')
        return True

    def turn(self, text: str) -> str:
        streamed: List[str] = []

        def on_text(piece: str) -> None:
            if getattr(self, '_bol', True):
                self.say('agent> ', end='')
            streamed.append(piece)
            self.say(piece, end='')

        reply = self.agent.send(text, on_text=on_text)
        if streamed:
            self.fresh_line()
        else:
            self.say(f'agent> {reply}')
        return reply

    # ---- main loop --------------------------------------------------------------------------------------------------
    def run(self, inp=None) -> None:
        reader = inp or sys.stdin
        if self.monitor:
            self.monitor.start()
        self.say(f'twinkle-auto — runs in {self.store.base}; skills: {", ".join(self.skills.names()) or "none"}; /help for commands')
        try:
            while True:
                self.drain()
                for ln in header_lines(self.store):
                    self.say(f'│ {ln}')
                self.say('you> ', end='')
                line = reader.readline()
                if not line:
                    break
                line = line.strip()
                if not line:
                    continue
                if line.startswith('/'):
                    if not self.command(line):
                        break
                    continue
                try:
                    self.turn(line)
                except KeyboardInterrupt:
                    self.say('\n(interrupted)')
                except Exception as e:
                    self.say(f'\n! model call failed: {e}')
        finally:
            if self.monitor:
                self.monitor.stop()
            self.executor.tool_shutdown_server()


def main(argv: Optional[List[str]] = None) -> int:
    ap = argparse.ArgumentParser(prog='twinkle-auto', description='Conversational agent that writes, launches and watches training scripts.')
    ap.add_argument('--base-dir', default=None, help='directory of run folders (default: $TWINKLE_AUTO_HOME or ~/.cache/twinkle_b200/runs)')
    ap.add_argument('--llm-url', default=None, help='OpenAI-compatible endpoint, e.g. http://127.0.0.1:8000/v1')
    ap.add_argument('--llm-key', default=None)
    ap.add_argument('--llm-model', default=None)
    ap.add_argument('--monitor-model', default=None, help='a different (cheaper) model for the health monitor')
    ap.add_argument('--poll-interval', type=float, default=30.0)
    ap.add_argument('--skills', action='append', default=[], help='extra skill directory or hub repository (repeatable)')
    ap.add_argument('--no-monitor', action='store_true')
    ap.add_argument('--once', default=None, help='run one turn with this text and exit')
    ap.add_argument('--dry-run', action='store_true', help='no model endpoint: a stand-in that answers every message with a fixed line')
    a = ap.parse_args(argv)
    if a.dry_run:
        llm = mon = ScriptedLLM([], default='(dry run: no model endpoint configured)')
    else:
        llm = ChatLLM(a.llm_url, a.llm_key, a.llm_model)
        mon = ChatLLM(a.llm_url, a.llm_key, a.monitor_model) if a.monitor_model else llm
    app = AutoApp(RunStore(a.base_dir), llm, mon, a.poll_interval, a.skills, monitor=not a.no_monitor and a.once is None)
    if a.once is not None:
        app.turn(a.once)
        return 0
    app.run()
    return 0


if __name__ == '__main__':
    sys.exit(main())
