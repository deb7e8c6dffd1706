"""Conversation loop of the auto agent: user text → model → tool calls → tool results → … → final text.

Parity: reference ``src/twinkle_client/auto/agent/core.py`` (``AgentLoop``: system prompt with injected skills,
tool-call rounds with a cap, history pruning that never separates a tool result from the call it answers) and
``agent/prompts.py``.
"""
from __future__ import annotations

import json
import threading
from typing import Any, Callable, Dict, List, Optional

from .tools import TOOL_SCHEMAS, ToolExecutor

SYSTEM_PROMPT = """\
You are twinkle-auto, an assistant that runs LLM post-training experiments on this machine with the twinkle_b200 \
framework. You act only through the tools you are given.

How to work:
- Find out what exists first (get_cluster_info, list_training_runs, list_supported_models) instead of assuming.
- A training run is a complete Python script. Write it in full, start it with start_training, and read its \
status before you claim anything about it. Scripts use `from twinkle_b200.client.auto.runtime import TrainingRuntime` \
to report metrics, resume from `rt.get_resume_info()`, and save on SIGTERM via `rt.register_graceful_shutdown(...)`.
- Scripts talk to a training server. If none is running, start one with start_server before starting a run.
- To change a running experiment: update_script, then pause_training and resume_training. The server keeps the \
adapter and optimizer state across that restart.
- Keep answers short. Report numbers you read from tools, never numbers you expect.
"""


class AgentLoop:

    def __init__(self, llm, executor: ToolExecutor, system_prompt: str = SYSTEM_PROMPT, max_tool_rounds: int = 12,
                 max_history_chars: int = 120_000, on_tool: Optional[Callable[[str, Dict[str, Any], str], None]] = None):
        self.llm, self.executor = llm, executor
        self.base_prompt = system_prompt
        self.skills_prompt = ''
        self.max_tool_rounds, self.max_history_chars = max_tool_rounds, max_history_chars
        self.on_tool = on_tool
        self.history: List[Dict[str, Any]] = []
        self._lock = threading.Lock()                             # one conversation turn at a time

    def inject_skills(self, skills_prompt: str) -> None:
        self.skills_prompt = skills_prompt or ''

    def system_message(self) -> Dict[str, str]:
        text = self.base_prompt + (('\n\n' + self.skills_prompt) if self.skills_prompt else '')
        if self.executor.store.selected:
            text += f'\n\nCurrently selected run: {self.executor.store.selected}'
        return dict(role='system', content=text)

    def note(self, text: str) -> None:
        """Put an out-of-band observation (e.g. from the monitor) where the next turn will see it."""
        with self._lock:
            self.history.append(dict(role='user', content=f'[system note] {text}'))

    def send(self, user_text: str, on_text: Optional[Callable[[str], None]] = None) -> str:
        with self._lock:
            self.history.append(dict(role='user', content=user_text))
            final = ''
            for _ in range(self.max_tool_rounds):
                self._prune()
                reply = self.llm.chat([self.system_message()] + self.history, tools=TOOL_SCHEMAS, on_text=on_text)
                calls = reply.get('tool_calls') or []
                msg: Dict[str, Any] = dict(role='assistant', content=reply.get('content') or '')
                if calls:
                    msg['tool_calls'] = [dict(id=c['id'], type='function', function=dict(name=c['name'], arguments=json.dumps(c['arguments'], ensure_ascii=False)))
                                         for c in calls]
                self.history.append(msg)
                final = msg['content']
                if not calls:
                    return final
                for c in calls:
                    result = self.executor.execute(c['name'], c['arguments'])
                    if self.on_tool:
                        self.on_tool(c['name'], c['arguments'], result)
                    self.history.append(dict(role='tool', tool_call_id=c['id'], content=result[:20_000]))
            self.history.append(dict(role='assistant', content='(stopped: too many tool rounds in one turn)'))
            return final or self.history[-1]['content']

    def _prune(self) -> None:
        """Drop the oldest whole exchanges until the history fits.  A cut only ever lands in front of a user
        message, so an assistant tool call and its tool results leave together."""
        size = lambda: sum(len(m.get('content') or '') + len(json.dumps(m.get('tool_calls') or '')) for m in self.history)
        while size() > self.max_history_chars:
            cut = next((i for i in range(1, len(self.history)) if self.history[i]['role'] == 'user'), None)
            if cut is None:
                break
            del self.history[:cut]
