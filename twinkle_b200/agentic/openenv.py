"""Adapters for third-party episodic environments (the OpenEnv convention: ``reset()`` and ``step(action)`` returning an
object or mapping with ``observation`` / ``reward`` / ``done``) and a pool of them sharded over worker processes.

* :class:`OpenEnv` wraps one such environment object as this package's :class:`Env` — in process, no HTTP server.
* :class:`ShardedEnvPool` is a ``@remote_class``: every worker of its device group owns a contiguous range of slots;
  calls carry slot indices and each worker answers for the slots it owns.
* :class:`EnvPoolAdapter` presents one slot of a pool as an :class:`Env`, so rollouts need not know about the pool.

Parity: reference ``src/twinkle_agentic/envs/openenv.py:27-355``."""
from __future__ import annotations

import importlib
import json
import math
import os
import pkgutil
from typing import Any, Callable, Dict, List, Optional, Sequence, Tuple, Union

from ..infra import remote_class, remote_function
from ..utils.device_mesh import DeviceMesh
from ..utils.logger import get_logger
from .tools import Env, StepResult, ToolInfo

logger = get_logger()


def import_class(path: str):
    """``'pkg.module:Class'`` or ``'pkg.module.Class'`` → the class."""
    if ':' in path:
        mod, name = path.rsplit(':', 1)
    elif '.' in path:
        mod, name = path.rsplit('.', 1)
    else:
        raise ValueError(f"expected 'module.Class' or 'module:Class', got {path!r}")
    module = importlib.import_module(mod)
    if not hasattr(module, name):
        raise ImportError(f'module {mod!r} has no attribute {name!r}')
    return getattr(module, name)


def observation_text(obs: Any) -> str:
    """Observation as text: strings pass, mappings give their ``result`` / ``output`` / ``content`` / ``text`` /
    ``message`` entry (else JSON), pydantic-like objects their dumped JSON, anything else ``str()``."""
    if obs is None:
        return ''
    if isinstance(obs, str):
        return obs
    if isinstance(obs, dict):
        for k in ('result', 'output', 'content', 'text', 'message'):
            if k in obs:
                return str(obs[k])
        return json.dumps(obs, ensure_ascii=False, default=str)
    if hasattr(obs, 'model_dump'):
        try:
            return json.dumps(obs.model_dump(), ensure_ascii=False, default=str)
        except (TypeError, ValueError):
            pass
    return str(obs)


def normalize_result(result: Any) -> Dict[str, Any]:
    """``{'observation': str, 'reward': float, 'done': bool}`` from a mapping, an object with those attributes, or a
    bare observation."""
    if isinstance(result, dict):
        obs, reward, done = result.get('observation', ''), result.get('reward'), result.get('done')
    elif hasattr(result, 'observation'):
        obs, reward, done = result.observation, getattr(result, 'reward', None), getattr(result, 'done', None)
    else:
        obs, reward, done = result, getattr(result, 'reward', None), getattr(result, 'done', None)
    return {'observation': observation_text(obs), 'reward': float(reward or 0.0), 'done': bool(done)}


def discover_env_classes(env_name: str) -> Tuple[type, Optional[type]]:
    """Environment and action classes of an installed OpenEnv package: the ``*Environment`` class of a
    ``*_environment`` module under ``<env_name>.server`` and, when present, the ``*Action`` class of
    ``<env_name>.models``."""
    importlib.import_module(env_name)
    server = importlib.import_module(env_name + '.server')
    env_cls = None
    for info in pkgutil.iter_modules(server.__path__):
        if info.name.endswith('_environment'):
            mod = importlib.import_module(f'{env_name}.server.{info.name}')
            for name in dir(mod):
                obj = getattr(mod, name)
                if isinstance(obj, type) and name.endswith('Environment') and obj.__module__ == mod.__name__:
                    env_cls = obj
    if env_cls is None:
        raise ImportError(f"no '*Environment' class in a '*_environment' module under {env_name}.server")
    action_cls = None
    try:
        models = importlib.import_module(env_name + '.models')
        for name in dir(models):
            obj = getattr(models, name)
            if isinstance(obj, type) and name.endswith('Action') and obj.__module__ == models.__name__:
                action_cls = obj
    except ModuleNotFoundError:
        pass
    return env_cls, action_cls


class OpenEnv(Env):
    """One embedded environment. ``env_cls`` (class or import path) or ``env_name`` (installed package, classes
    discovered) selects it; ``env_kwargs`` go to its constructor. A tool call becomes the action: ``action_mapper
    (tool_name, arguments)`` when given, else the arguments themselves; a mapping is passed through ``action_cls``
    when there is one. ``tool_infos`` lists the actions offered to the policy (default: one free-form ``act`` tool)."""

    def __init__(self, env_name: Optional[str] = None, env_cls: Union[str, type, None] = None, env_kwargs: Optional[Dict[str, Any]] = None,
                 action_cls: Union[str, type, None] = None, action_mapper: Optional[Callable[[str, Dict[str, Any]], Any]] = None,
                 tool_infos: Optional[Sequence[ToolInfo]] = None, **_ignored):
        if env_cls is None and env_name is None:
            raise ValueError("give 'env_cls' (class or 'module:Class') or 'env_name' (an installed environment package)")
        if env_cls is None:
            cls, found_action = discover_env_classes(env_name)
            action_cls = action_cls or found_action
        else:
            cls = import_class(env_cls) if isinstance(env_cls, str) else env_cls
        self.env = cls(**(env_kwargs or {}))
        self.action_cls = import_class(action_cls) if isinstance(action_cls, str) else action_cls
        self.action_mapper = action_mapper
        self._tools = list(tool_infos) if tool_infos else [
            {'tool_name': 'act', 'description': 'Take one action in the environment.',
             'parameters': {'type': 'object', 'properties': {}, 'additionalProperties': True}}]

    def _result(self, raw) -> StepResult:
        n = normalize_result(raw)
        return StepResult(n['observation'], n['reward'], n['done'])

    def reset(self, trajectory=None) -> StepResult:
        return self._result(self.env.reset())

    def step(self, tool_name: str, arguments: Optional[Dict[str, Any]] = None) -> StepResult:
        action = self.action_mapper(tool_name, arguments or {}) if self.action_mapper is not None else (arguments or {})
        if self.action_cls is not None and isinstance(action, dict):
            action = self.action_cls(**action)
        return self._result(self.env.step(action))

    def tools(self) -> List[ToolInfo]:
        return list(self._tools)

    def close(self) -> None:
        if hasattr(self.env, 'close'):
            self.env.close()


def _first_answer(results, device_mesh=None):
    for r in results:
        if r is not None:
            return r
    return None


def _merge_by_slot(results, device_mesh=None):
    merged = [pair for part in results if part for pair in part]
    merged.sort(key=lambda p: p[0])
    return [p[1] for p in merged]


@remote_class(execute='all')
class ShardedEnvPool:
    """``pool_size`` environments split over the workers of a device group: worker ``r`` of ``w`` owns slots
    ``[r·ceil(n/w), (r+1)·ceil(n/w))``. Every call reaches every worker; a worker answers only for its own slots, and
    the driver keeps the one answer (``reset`` / ``step``) or merges the answers in slot order (``*_batch``). The
    running sum of rewards per slot is kept beside the environment and returned with every result."""

    def __init__(self, pool_size: int = 32, device_mesh: Optional[DeviceMesh] = None, env_kwargs: Optional[Dict[str, Any]] = None,
                 env_factory: Optional[Callable[[], Env]] = None, **_ignored):
        self._pool_size = pool_size
        rank, world = int(os.environ.get('RANK', 0)), int(os.environ.get('WORLD_SIZE', 1))
        if device_mesh is not None and getattr(device_mesh, 'world_size', world) < world:
            world = device_mesh.world_size  # a pool on a sub-group of the job
            rank = rank % world
        shard = math.ceil(pool_size / max(world, 1))
        self._start = min(rank * shard, pool_size)
        self._end = min(self._start + shard, pool_size)
        make = env_factory or (lambda: OpenEnv(**(env_kwargs or {})))
        self._envs: List[Env] = [make() for _ in range(self._end - self._start)]
        self._totals: List[float] = [0.0] * len(self._envs)
        logger.info(f'ShardedEnvPool: {pool_size} slots, this worker owns [{self._start}, {self._end})')

    def _owns(self, idx: int) -> bool:
        return self._start <= idx < self._end

    def _reset(self, idx: int) -> Dict[str, Any]:
        k = idx - self._start
        self._totals[k] = 0.0
        r = self._envs[k].reset()
        return {'observation': r.observation, 'reward': r.reward, 'done': r.done, 'episode_reward': 0.0}

    def _step(self, idx: int, tool_name: str, arguments: Dict[str, Any]) -> Dict[str, Any]:
        k = idx - self._start
        r = self._envs[k].step(tool_name, arguments)
        self._totals[k] += r.reward
        return {'observation': r.observation, 'reward': r.reward, 'done': r.done, 'episode_reward': self._totals[k]}

    @remote_function(dispatch='all', collect=_first_answer)
    def reset(self, idx: int) -> Optional[Dict[str, Any]]:
        return self._reset(idx) if self._owns(idx) else None

    @remote_function(dispatch='all', collect=_first_answer)
    def step(self, idx: int, tool_name: str, arguments: Dict[str, Any]) -> Optional[Dict[str, Any]]:
        return self._step(idx, tool_name, arguments) if self._owns(idx) else None

    @remote_function(dispatch='all', collect=_merge_by_slot)
    def reset_batch(self, indices: List[int]) -> List:
        return [(i, self._reset(i)) for i in indices if self._owns(i)]

    @remote_function(dispatch='all', collect=_merge_by_slot)
    def step_batch(self, indices: List[int], tool_names: List[str], arguments_list: List[Dict[str, Any]]) -> List:
        return [(i, self._step(i, t, a)) for i, t, a in zip(indices, tool_names, arguments_list) if self._owns(i)]

    @remote_function(dispatch='all', collect=_first_answer)
    def tool_infos(self) -> Optional[List[ToolInfo]]:
        return self._envs[0].tools() if self._envs else None

    @remote_function(dispatch='all', collect='first')
    def close(self) -> None:
        for e in self._envs:
            e.close()
        self._envs.clear()

    @property
    def pool_size(self) -> int:
        return self._pool_size

    def get_adapters(self, n: int) -> List['EnvPoolAdapter']:
        """Driver side: adapters for slots ``0 … n−1``."""
        if n > self._pool_size:
            raise ValueError(f'{n} adapters requested from a pool of {self._pool_size} slots')
        return [EnvPoolAdapter(self, i) for i in range(n)]


class EnvPoolAdapter(Env):
    """Slot ``idx`` of a :class:`ShardedEnvPool` as an :class:`Env`. A failing step ends the episode with the error as
    the observation instead of raising into the rollout loop."""

    def __init__(self, pool, idx: int):
        self.pool, self.idx, self._episode_reward, self._tools = pool, idx, 0.0, None

    def reset(self, trajectory=None) -> StepResult:
        self._episode_reward = 0.0
        r = self.pool.reset(self.idx) or {}
        return StepResult(r.get('observation', ''), 0.0, False, dict(r))

    def step(self, tool_name: str, arguments: Optional[Dict[str, Any]] = None) -> StepResult:
        try:
            r = self.pool.step(self.idx, tool_name, arguments or {})
        except Exception as e:
            logger.warning(f'environment slot {self.idx}: step failed: {e}')
            return StepResult(f'Error: {e}', 0.0, True, {'error': str(e)})
        self._episode_reward = float(r.get('episode_reward', 0.0))
        return StepResult(r.get('observation', ''), float(r.get('reward', 0.0)), bool(r.get('done', False)),
                          {'episode_reward': self._episode_reward})

    def tools(self) -> List[ToolInfo]:
        if self._tools is None:
            self._tools = self.pool.tool_infos() or []
        return list(self._tools)

    @property
    def episode_reward(self) -> float:
        return self._episode_reward

    def close(self) -> None:  # the pool owns the environment
        pass
