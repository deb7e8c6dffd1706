"""Tools and environments for multi-turn rollouts.

What it covers: reference ``src/twinkle_agentic/tools/{base,tool_manager}.py``, ``envs/{base,env_tool}.py``.
A ``Tool`` is a callable ``(tool_name, arguments) -> str`` that describes itself with a ``Tool`` record
(``data_format.types.Tool``); a ``ToolManager`` dispatches the assistant's tool calls; an ``Env`` is a stateful
episode (reset / step / evaluate) whose actions are exposed to the policy as tools through ``EnvTool``.
"""
from __future__ import annotations

import copy
import json
from abc import ABC, abstractmethod
from dataclasses import dataclass, field
from typing import Any, Callable, Dict, List, Optional, Sequence, Union

from ..data_format.types import Tool as ToolInfo
from ..data_format.types import ToolCall, Trajectory


class Tool(ABC):

    @abstractmethod
    def __call__(self, tool_name: str, arguments: Dict[str, Any]) -> str:
        ...

    @abstractmethod
    def tool_info(self) -> ToolInfo:
        ...


class FunctionTool(Tool):
    """Wraps a plain Python function; the parameter schema is taken from its signature."""

    def __init__(self, fn: Callable[..., Any], name: Optional[str] = None, description: Optional[str] = None):
        import inspect
        self.fn, self.name = fn, name or fn.__name__
        self.description = description or (fn.__doc__ or '').strip()
        props, required = {}, []
        for p in inspect.signature(fn).parameters.values():
            ann = {int: 'integer', float: 'number', bool: 'boolean', str: 'string'}.get(p.annotation, 'string')
            props[p.name] = {'type': ann}
            if p.default is inspect.Parameter.empty:
                required.append(p.name)
        self.parameters = {'type': 'object', 'properties': props, 'required': required}

    def __call__(self, tool_name: str, arguments: Dict[str, Any]) -> str:
        out = self.fn(**arguments)
        return out if isinstance(out, str) else json.dumps(out, ensure_ascii=False, default=str)

    def tool_info(self) -> ToolInfo:
        return ToolInfo(tool_name=self.name, description=self.description, parameters=self.parameters)


class ToolManager:
    """Name → tool registry.  Calling it with a tool call returns the observation text; errors come back as text too
    (the policy sees them), never as exceptions that would end the rollout."""

    def __init__(self, tools: Optional[Sequence[Tool]] = None, max_observation_chars: int = 8000):
        self._tools: Dict[str, Tool] = {}
        self.max_observation_chars = max_observation_chars
        for t in tools or ():
            self.register(t)

    def register(self, tool: Tool) -> None:
        name = tool.tool_info().get('tool_name')
        if not name:
            raise ValueError('a tool must name itself in tool_info()')
        self._tools[name] = tool

    def unregister(self, name: str) -> Optional[Tool]:
        return self._tools.pop(name, None)

    def names(self) -> List[str]:
        return list(self._tools)

    def copy(self) -> 'ToolManager':
        m = ToolManager(max_observation_chars=self.max_observation_chars)
        m._tools = {k: copy.copy(v) for k, v in self._tools.items()}
        return m

    def tool_infos(self) -> List[ToolInfo]:
        return [t.tool_info() for t in self._tools.values()]

    def __call__(self, tool_call: Union[ToolCall, Dict[str, Any]]) -> str:
        name = tool_call.get('tool_name') or (tool_call.get('function') or {}).get('name')
        args = tool_call.get('arguments')
        if args is None:
            args = (tool_call.get('function') or {}).get('arguments', {})
        if isinstance(args, str):
            try:
                args = json.loads(args) if args.strip() else {}
            except json.JSONDecodeError as e:
                return f'Error: arguments of {name!r} are not valid JSON ({e})'
        tool = self._tools.get(name)
        if tool is None:
            return f'Error: unknown tool {name!r}; available: {", ".join(self._tools) or "none"}'
        try:
            out = tool(name, args or {})
        except Exception as e:  # noqa: BLE001 — reported to the policy
            out = f'Error: {type(e).__name__}: {e}'
        out = out if isinstance(out, str) else str(out)
        if len(out) > self.max_observation_chars:
            out = out[:self.max_observation_chars] + f'\n… [{len(out) - self.max_observation_chars} characters cut]'
        return out


# ------------------------------------------------------------------------------------------------------ environments
@dataclass
class StepResult:
    observation: str = ''
    reward: float = 0.0
    done: bool = False
    info: Dict[str, Any] = field(default_factory=dict)


class Env(ABC):
    """One episode at a time.  ``tools()`` lists the actions; ``step`` applies one."""

    @abstractmethod
    def reset(self, trajectory: Optional[Trajectory] = None) -> StepResult:
        ...

    @abstractmethod
    def step(self, tool_name: str, arguments: Dict[str, Any]) -> StepResult:
        ...

    @abstractmethod
    def tools(self) -> List[ToolInfo]:
        ...

    def evaluate(self, trajectories: List[Trajectory], **kwargs) -> List[float]:
        return [0.0 for _ in trajectories]

    def close(self) -> None:
        pass

    def __enter__(self):
        return self

    def __exit__(self, *args):
        self.close()


class EnvTool(Tool):
    """One action of an ``Env`` as a tool; remembers the reward and whether the episode ended."""

    def __init__(self, env: Env, info: ToolInfo, state: Optional[Dict[str, Any]] = None):
        self.env, self.info = env, info
        self.state = state if state is not None else {'done': False, 'reward': 0.0}

    def __call__(self, tool_name: str, arguments: Dict[str, Any]) -> str:
        if self.state['done']:
            return 'Error: the episode is over'
        r = self.env.step(tool_name, arguments)
        self.state['reward'] += r.reward
        self.state['done'] = r.done
        return r.observation

    def tool_info(self) -> ToolInfo:
        return self.info

    @property
    def done(self) -> bool:
        return bool(self.state['done'])

    @property
    def episode_reward(self) -> float:
        return float(self.state['reward'])

    @classmethod
    def from_env(cls, env: Env) -> List['EnvTool']:
        shared = {'done': False, 'reward': 0.0}
        return [cls(env, info, shared) for info in env.tools()]


class EnvPool:
    """A fixed set of environments handed out to trajectories of a batch (one each), reset on acquire."""

    def __init__(self, factory: Callable[[], Env], size: int):
        self.envs = [factory() for _ in range(size)]

    def managers(self, trajectories: Sequence[Trajectory]) -> List[ToolManager]:
        if len(trajectories) > len(self.envs):
            raise ValueError(f'{len(trajectories)} trajectories for a pool of {len(self.envs)} environments')
        out = []
        for env, traj in zip(self.envs, trajectories):
            env.reset(traj)
            out.append(ToolManager(EnvTool.from_env(env)))
        return out

    def close(self) -> None:
        for e in self.envs:
            e.close()
