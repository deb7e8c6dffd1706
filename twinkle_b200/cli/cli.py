"""Training-script argument system.

Parity: reference ``src/twinkle/cli/cli.py:14-643`` — dataclass argument groups (Model, Lora, Dataset,
Template, Training, Optimizer, Scheduler, Loss, Sampler, Sampling, Infra, Server, RL, Checkpoint) filled from
layered sources with increasing priority ``.env`` file < environment variables (``TWINKLE_<FIELD>``) < YAML
file (``--config``) < command-line flags; short aliases (``--lr``); unknown flags are kept in ``args.extra``.
"""
from __future__ import annotations

import dataclasses
import os
import sys
from dataclasses import dataclass, field, fields
from typing import Any, Dict, List, Optional, Sequence, Type, get_args, get_origin, Union


@dataclass
class ArgGroup:
    pass


@dataclass
class ModelArgs(ArgGroup):
    model_id: str = 'qwen3-8b'
    backend: str = 'transformers'  # transformers | megatron
    mixed_precision: str = 'bf16'
    max_length: int = 8192


@dataclass
class LoraArgs(ArgGroup):
    use_lora: bool = False
    lora_rank: int = 8
    lora_alpha: int = 32
    target_modules: str = 'all-linear'
    max_loras: int = 5
    max_r: int = 32


@dataclass
class DatasetArgs(ArgGroup):
    dataset: str = ''
    subset_name: str = 'default'
    split: str = 'train'
    preprocessor: str = ''
    packing: bool = False
    streaming: bool = False
    num_proc: int = 1


@dataclass
class TemplateArgs(ArgGroup):
    template: str = 'Template'
    truncation_strategy: str = 'raise'
    default_system: str = ''
    enable_thinking: bool = True


@dataclass
class TrainingArgs(ArgGroup):
    batch_size: int = 8
    micro_batch_size: int = 1
    gradient_accumulation_steps: int = 1
    num_epochs: int = 1
    max_steps: int = -1
    max_grad_norm: float = 1.0
    log_interval: int = 1
    seed: int = 42


@dataclass
class OptimizerArgs(ArgGroup):
    optimizer: str = 'AdamW'
    learning_rate: float = 1e-5
    weight_decay: float = 0.01
    adam_beta1: float = 0.9
    adam_beta2: float = 0.999
    adam_eps: float = 1e-8


@dataclass
class SchedulerArgs(ArgGroup):
    lr_scheduler: str = 'cosine'
    warmup_steps: int = 0
    min_lr_ratio: float = 0.0


@dataclass
class LossArgs(ArgGroup):
    loss: str = 'cross_entropy'
    beta: float = 0.0
    epsilon: float = 0.2
    epsilon_high: float = 0.2


@dataclass
class SamplerArgs(ArgGroup):
    sampler_type: str = 'torch'
    sampler_gpus: int = 0
    gpu_memory_utilization: float = 0.85
    kv_block_size: int = 16


@dataclass
class SamplingArgs(ArgGroup):
    max_tokens: int = 1024
    temperature: float = 1.0
    top_p: float = 1.0
    top_k: int = -1
    num_generations: int = 8


@dataclass
class InfraArgs(ArgGroup):
    mode: str = 'local'
    nproc_per_node: int = 1
    dp_size: int = 1
    fsdp_size: int = 0
    tp_size: int = 0
    pp_size: int = 0
    cp_size: int = 0
    ep_size: int = 0
    ulysses_size: int = 0
    vpp_size: int = 0
    sequence_parallel: bool = False


@dataclass
class ServerArgs(ArgGroup):
    server_url: str = ''
    server_token: str = ''
    server_config: str = ''


@dataclass
class RLArgs(ArgGroup):
    advantage: str = 'grpo'
    advantage_scale: str = 'group'
    kl_coef: float = 0.0
    reward: str = ''
    sync_interval: int = 1
    merge_and_sync: bool = False


@dataclass
class CheckpointArgs(ArgGroup):
    output_dir: str = './output'
    save_interval: int = 500
    resume_from_checkpoint: str = ''
    save_optimizer: bool = True
    hub_model_id: str = ''


GROUPS: Dict[str, Type[ArgGroup]] = {
    'model': ModelArgs, 'lora': LoraArgs, 'dataset': DatasetArgs, 'template': TemplateArgs, 'training': TrainingArgs,
    'optimizer': OptimizerArgs, 'scheduler': SchedulerArgs, 'loss': LossArgs, 'sampler': SamplerArgs, 'sampling': SamplingArgs,
    'infra': InfraArgs, 'server': ServerArgs, 'rl': RLArgs, 'checkpoint': CheckpointArgs,
}
ALIASES = {'lr': 'learning_rate', 'wd': 'weight_decay', 'bs': 'batch_size', 'mbs': 'micro_batch_size', 'model': 'model_id',
           'epochs': 'num_epochs', 'ga': 'gradient_accumulation_steps', 'rank': 'lora_rank', 'n': 'num_generations'}


def _coerce(value: Any, typ) -> Any:
    if get_origin(typ) is Union:
        typ = [a for a in get_args(typ) if a is not type(None)][0]
    if typ is bool:
        if isinstance(value, bool):
            return value
        return str(value).lower() in ('1', 'true', 'yes', 'on')
    if typ in (int, float, str):
        return typ(value)
    return value


class Args:
    """Holds one instance of every group; fields are also reachable flat (``args.learning_rate``)."""

    def __init__(self):
        for name, cls in GROUPS.items():
            setattr(self, name, cls())
        self.extra: Dict[str, Any] = {}
        self._index = {f.name: (g, f) for g, cls in GROUPS.items() for f in fields(cls)}

    def __getattr__(self, item):
        idx = self.__dict__.get('_index', {})
        if item in idx:
            return getattr(getattr(self, idx[item][0]), item)
        raise AttributeError(item)

    def set(self, key: str, value: Any) -> bool:
        key = ALIASES.get(key, key)
        if key not in self._index:
            return False
        g, f = self._index[key]
        setattr(getattr(self, g), key, _coerce(value, f.type if not isinstance(f.type, str) else type(f.default)))
        return True

    def to_dict(self) -> Dict[str, Any]:
        return {g: dataclasses.asdict(getattr(self, g)) for g in GROUPS}

    def device_mesh(self):
        from ..utils.device_mesh import DeviceMesh
        i = self.infra
        kw = {k: (getattr(i, k) or None) for k in ('fsdp_size', 'tp_size', 'pp_size', 'cp_size', 'ep_size', 'ulysses_size', 'vpp_size')}
        return DeviceMesh.from_sizes(dp_size=i.dp_size or 1, sequence_parallel=i.sequence_parallel, **kw)


class CLI:

    @staticmethod
    def _read_env_file(path: str) -> Dict[str, str]:
        out = {}
        if os.path.isfile(path):
            with open(path) as f:
                for line in f:
                    line = line.strip()
                    if line and not line.startswith('#') and '=' in line:
                        k, v = line.split('=', 1)
                        out[k.strip()] = v.strip().strip('"').strip("'")
        return out

    @staticmethod
    def from_args(argv: Optional[Sequence[str]] = None, env_file: str = '.env') -> Args:
        argv = list(sys.argv[1:] if argv is None else argv)
        args = Args()
        # 1. .env file, 2. environment
        for source in (CLI._read_env_file(env_file), dict(os.environ)):
            for k, v in source.items():
                if k.startswith('TWINKLE_'):
                    args.set(k[len('TWINKLE_'):].lower(), v)
        # parse flags first to find --config
        flags: Dict[str, Any] = {}
        i = 0
        while i < len(argv):
            a = argv[i]
            if a.startswith('--'):
                key = a[2:].replace('-', '_')
                if '=' in key:
                    key, val = key.split('=', 1)
                elif i + 1 < len(argv) and not argv[i + 1].startswith('--'):
                    val = argv[i + 1]
                    i += 1
                else:
                    val = True
                flags[key] = val
            i += 1
        # 3. YAML
        cfg = flags.pop('config', None)
        if cfg:
            import yaml
            with open(cfg) as f:
                y = yaml.safe_load(f) or {}
            for k, v in y.items():
                if isinstance(v, dict) and k in GROUPS:
                    for kk, vv in v.items():
                        if not args.set(kk, vv):
                            args.extra[kk] = vv
                elif not args.set(k, v):
                    args.extra[k] = v
        # 4. flags
        for k, v in flags.items():
            if not args.set(k, v):
                args.extra[k] = v
        return args
