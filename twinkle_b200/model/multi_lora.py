"""Tenant → LoRA-slot bookkeeping on top of the physical slot pools.

Parity: reference ``src/twinkle/model/multi_lora.py:209-287, 558-754`` — a fixed
pool of ``max_loras`` adapters of rank ``max_r`` lives on every LoRA-able
module; ``acquire_lora`` binds a tenant to a free slot (errors: duplicate
tenant, pool exhausted, ``r > max_r``), ``release_lora`` restores the slot's
initial ``A`` and zeroes ``B``; state dicts are sliced to the tenant's rank on
save (PEFT key names) and padded back on load.
"""
from __future__ import annotations

import json
import math
import os
import re
from dataclasses import asdict, dataclass, field
from typing import Any, Dict, Iterator, List, Optional, Tuple, Union

import torch

from ..models.bridge import lora_expert_to_peft, lora_internal_to_peft
from ..models.decoder import DecoderModel, Experts
from ..models.layers import Linear, LoraBatch, TargetFilter


@dataclass
class LoraConfig:
    """Subset of PEFT's ``LoraConfig`` that the engine honours."""
    r: int = 8
    lora_alpha: int = 16
    target_modules: Union[str, List[str], None] = 'all-linear'
    lora_dropout: float = 0.0
    use_rslora: bool = False
    bias: str = 'none'
    task_type: str = 'CAUSAL_LM'
    target_parameters: Optional[List[str]] = None  # e.g. ['experts.gate_up_proj', 'experts.down_proj']
    exclude_modules: Union[str, List[str], None] = None  # PEFT: module-name suffixes (or a full-match regex) kept out of ``target_modules``
    base_model_name_or_path: Optional[str] = None

    _UNSUPPORTED = ('use_dora', 'rank_pattern', 'alpha_pattern', 'modules_to_save', 'layers_to_transform', 'layers_pattern', 'use_qalora',
                    'trainable_token_indices', 'layer_replication', 'megatron_config')

    @property
    def scaling(self) -> float:
        return self.lora_alpha / math.sqrt(self.r) if self.use_rslora else self.lora_alpha / self.r

    @classmethod
    def from_any(cls, obj) -> 'LoraConfig':
        if isinstance(obj, cls):
            return obj
        if isinstance(obj, str):  # directory with adapter_config.json
            with open(os.path.join(obj, 'adapter_config.json')) as f:
                obj = json.load(f)
        if not isinstance(obj, dict):
            obj = {k: getattr(obj, k) for k in tuple(cls.__dataclass_fields__) + cls._UNSUPPORTED if hasattr(obj, k)}
        # PEFT options that change the adapter's arithmetic or its set of trained tensors and are not implemented here: refused
        # rather than dropped (a run that silently trained something else is worse than one that does not start)
        for k in cls._UNSUPPORTED:
            v = obj.get(k)
            if v not in (None, False, 0, 0.0, '', [], {}, (), 'none') and not (k == 'init_lora_weights' and v is True) and not (k == 'bias' and v == 'none'):
                raise NotImplementedError(f'LoRA option {k}={v!r} is not supported (plain LoRA / rsLoRA with target_modules, exclude_modules and '
                                          'target_parameters are)')
        known = {k: obj[k] for k in cls.__dataclass_fields__ if k in obj and obj[k] is not None}
        if float(known.get('lora_dropout') or 0.0) > 0.0:
            import logging
            logging.getLogger('twinkle_b200').warning('lora_dropout=%s is recorded in the adapter config but not applied: the slot pools serve several '
                                                      'tenants from one deterministic kernel path', known['lora_dropout'])
        for k in ('target_modules', 'exclude_modules'):
            if isinstance(known.get(k), (set, tuple)):
                known[k] = sorted(known[k])
        return cls(**known)

    def to_peft_dict(self) -> Dict[str, Any]:
        d = asdict(self)
        d.update(peft_type='LORA', inference_mode=False, fan_in_fan_out=False, init_lora_weights=True, modules_to_save=None)
        return d


@dataclass
class _Tenant:
    name: str
    slot: int
    config: LoraConfig
    target: TargetFilter


def _interleave_gate(bq: torch.Tensor, bg: torch.Tensor, d: int) -> torch.Tensor:
    """Rows of the query part and of the output-gate part ``[H·d, r]`` each → the checkpoint's q_proj row order
    ``[head 0: query (d) | gate (d), head 1: …]``."""
    h = bq.shape[0] // d
    return torch.cat([bq.reshape(h, d, -1), bg.reshape(h, d, -1)], 1).reshape(2 * h * d, -1)


def _split_gate(b: torch.Tensor, d: int):
    h = b.shape[0] // (2 * d)
    x = b.reshape(h, 2 * d, -1)
    return x[:, :d].reshape(h * d, -1), x[:, d:].reshape(h * d, -1)


class MultiLora:

    def __init__(self, model: DecoderModel, max_loras: int = 5, max_r: int = 32, expert_lora: bool = True, seed: Optional[int] = None):
        """``seed``: the pool's ``A`` matrices are drawn from their own random stream, so two models built with the same
        seed hold the same pool whatever else consumed random numbers before (and the caller's stream is left alone)."""
        self.model, self.max_loras, self.max_r = model, max_loras, max_r
        self.tenants: Dict[str, _Tenant] = {}
        self.modules: List[Tuple[str, Any]] = []
        dev = next(model.parameters()).device
        with torch.random.fork_rng(devices=[dev] if dev.type == 'cuda' else [], enabled=seed is not None):
            if seed is not None:
                torch.manual_seed(0x10A5EED + int(seed))
            self._build_pools(model, max_loras, max_r, expert_lora)
        # base weights are frozen once a pool exists; only pool tensors train
        for n, p in model.named_parameters():
            p.requires_grad_('lora' in n)
        self._initial_A: Dict[str, torch.Tensor] = {n: p.detach().clone() for n, p in self.pool_parameters() if self._is_A(n)}

    def _build_pools(self, model, max_loras: int, max_r: int, expert_lora: bool) -> None:
        for name, m in model.lora_modules():
            if isinstance(m, Linear):
                if name == 'lm_head' or name.endswith('.gate'):
                    continue
                m.add_lora_pool(max_loras, max_r)
                self.modules.append((name, m))
            elif isinstance(m, Experts) and expert_lora:
                m.add_lora_pool(max_loras, max_r)
                self.modules.append((name, m))

    def sync_initial(self, comm) -> None:
        """Make the saved initial ``A`` values (what a released slot is reset to) the first rank's on every rank of a
        data-parallel group, so that a re-used slot starts equal everywhere."""
        if comm is None or comm.world_size <= 1:
            return
        for n in sorted(self._initial_A):
            comm.broadcast(self._initial_A[n], 0)

    @staticmethod
    def _is_A(name: str) -> bool:
        return 'lora_A' in name or name.endswith('_A')

    def pool_parameters(self) -> Iterator[Tuple[str, torch.nn.Parameter]]:
        for n, p in self.model.named_parameters():
            if 'lora' in n:
                yield n, p

    # ------------------------------------------------------------- tenants
    def acquire_lora(self, tenant: str, config) -> int:
        cfg = LoraConfig.from_any(config)
        if tenant in self.tenants:
            raise ValueError(f'adapter {tenant!r} already exists')
        if cfg.r > self.max_r:
            raise ValueError(f'adapter rank {cfg.r} exceeds the pool rank {self.max_r}')
        used = {t.slot for t in self.tenants.values()}
        free = [s for s in range(self.max_loras) if s not in used]
        if not free:
            raise RuntimeError(f'no free LoRA slot (max_loras={self.max_loras})')
        self.tenants[tenant] = _Tenant(tenant, free[0], cfg, TargetFilter(cfg.target_modules, cfg.exclude_modules))
        return free[0]

    def release_lora(self, tenant: str) -> None:
        t = self.tenants.pop(tenant)
        with torch.no_grad():
            for n, p in self.pool_parameters():
                if self._is_A(n):
                    p[t.slot].copy_(self._initial_A[n][t.slot])
                else:
                    p[t.slot].zero_()

    def has(self, tenant: str) -> bool:
        return tenant in self.tenants

    def free_slots(self) -> int:
        return self.max_loras - len(self.tenants)

    def batch_for(self, tenant: Optional[str], num_tokens: int, device, disable: bool = False) -> Optional[LoraBatch]:
        if tenant is None or disable:
            return None
        t = self.tenants[tenant]
        return LoraBatch.single(num_tokens, t.slot, t.config.r, t.config.scaling, device, t.target)

    def batch_for_segments(self, segments: List[Tuple[Optional[str], int]], device) -> LoraBatch:
        """Several tenants in one packed row: ``segments`` = (tenant|None, n_tokens) in order."""
        segs, targets, lo = [], [], 0
        for name, n in segments:
            if name is None:
                segs.append((lo, lo + n, -1, 0, 0.0))
                targets.append(None)
            else:
                t = self.tenants[name]
                segs.append((lo, lo + n, t.slot, t.config.r, t.config.scaling))
                targets.append(t.target)
            lo += n
        return LoraBatch(segs, device, targets)

    # ------------------------------------------------ per-tenant parameters
    def tenant_slices(self, tenant: str) -> List[Tuple[str, torch.nn.Parameter, int]]:
        """(pool parameter name, pool parameter, slot) for every pool tensor the
        tenant trains (modules outside its ``target_modules`` are skipped)."""
        t = self.tenants[tenant]
        out = []
        for mod_name, m in self.modules:
            prefix = mod_name.rsplit('.', 1)[0] if '.' in mod_name else ''
            if isinstance(m, Linear):
                for pname, _ in m.parts:
                    full = f'{prefix}.{pname}' if prefix else pname
                    if t.target.matches(full, pname):
                        if not (pname == 'q_gate' and m.lora_A[pname] is m.lora_A.get('q_proj')):   # the gate shares q_proj's A: listed once
                            out.append((f'{mod_name}.lora_A.{pname}', m.lora_A[pname], t.slot))
                        out.append((f'{mod_name}.lora_B.{pname}', m.lora_B[pname], t.slot))
            else:
                for which in ('gate_up', 'down'):
                    if t.target.matches(f'{mod_name}.{which}', which) or (t.config.target_parameters and any(
                            which in tp for tp in t.config.target_parameters)):
                        out.append((f'{mod_name}.lora.{which}_A', m.lora[which + '_A'], t.slot))
                        out.append((f'{mod_name}.lora.{which}_B', m.lora[which + '_B'], t.slot))
        return out

    def _rope_perm(self, pname: str, rows: int, to_hf: bool):
        cfg = getattr(self.model, 'cfg', None)
        if cfg is None or not getattr(cfg, 'rope_interleaved', False) or pname not in ('q_proj', 'k_proj'):
            return None
        from ..models.bridge import rope_row_perm
        return rope_row_perm(cfg, rows // cfg.head_dim, to_hf)

    # ------------------------------------------------------------ state dict
    def get_state_dict(self, tenant: str) -> Dict[str, torch.Tensor]:
        """PEFT-named tensors sliced to the tenant's rank."""
        t = self.tenants[tenant]
        r = t.config.r
        sd: Dict[str, torch.Tensor] = {}
        for mod_name, m in self.modules:
            prefix = mod_name.rsplit('.', 1)[0] if '.' in mod_name else ''
            if isinstance(m, Linear):
                for pname, _ in m.parts:
                    full = f'{prefix}.{pname}' if prefix else pname
                    if pname == 'q_gate' or not t.target.matches(full, pname):
                        continue            # the gate's rows travel inside q_proj's B (below)
                    b = m.lora_B[pname][t.slot, :, :r].detach().clone()
                    perm = self._rope_perm(pname, b.shape[0], True)
                    if perm is not None:
                        b = b[perm]             # the checkpoint's rotary pairing: rows of q / k move with it
                    if pname == 'q_proj' and m.gate_head_dim:
                        b = _interleave_gate(b, m.lora_B['q_gate'][t.slot, :, :r].detach(), m.gate_head_dim)
                    sd[lora_internal_to_peft(mod_name, pname, 'A')] = m.lora_A[pname][t.slot, :r].detach().clone()
                    sd[lora_internal_to_peft(mod_name, pname, 'B')] = b
            else:
                for which in ('gate_up', 'down'):
                    sd[lora_expert_to_peft(mod_name, which, 'A')] = m.lora[which + '_A'][t.slot, :, :r].detach().clone()
                    sd[lora_expert_to_peft(mod_name, which, 'B')] = m.lora[which + '_B'][t.slot, :, :, :r].detach().clone()
        return sd

    @torch.no_grad()
    def set_state_dict(self, tenant: str, sd: Dict[str, torch.Tensor]) -> List[str]:
        """Load PEFT-named tensors (rank ≤ max_r, zero-padded).  Returns unused keys."""
        t = self.tenants[tenant]
        used = set()
        for mod_name, m in self.modules:
            if isinstance(m, Linear):
                for pname, _ in m.parts:
                    ka, kb = lora_internal_to_peft(mod_name, pname, 'A'), lora_internal_to_peft(mod_name, pname, 'B')
                    if ka in sd and kb in sd and pname != 'q_gate':
                        a, b = sd[ka], sd[kb]
                        r = a.shape[0]
                        if pname == 'q_proj' and m.gate_head_dim:      # [query | gate] rows interleaved per head → two parts
                            b, bg = _split_gate(b, m.gate_head_dim)
                            m.lora_B['q_gate'][t.slot].zero_()
                            m.lora_B['q_gate'][t.slot, :, :r].copy_(bg)
                        perm = self._rope_perm(pname, b.shape[0], False)
                        if perm is not None:
                            b = b[perm.to(b.device)]
                        m.lora_A[pname][t.slot].zero_()
                        m.lora_B[pname][t.slot].zero_()
                        m.lora_A[pname][t.slot, :r].copy_(a)
                        m.lora_B[pname][t.slot, :, :r].copy_(b)
                        used.update((ka, kb))
            else:
                for which in ('gate_up', 'down'):
                    ka, kb = lora_expert_to_peft(mod_name, which, 'A'), lora_expert_to_peft(mod_name, which, 'B')
                    if ka in sd and kb in sd:
                        r = sd[ka].shape[-2]
                        m.lora[which + '_A'][t.slot].zero_()
                        m.lora[which + '_B'][t.slot].zero_()
                        m.lora[which + '_A'][t.slot, :, :r].copy_(sd[ka])
                        m.lora[which + '_B'][t.slot, :, :, :r].copy_(sd[kb])
                        used.update((ka, kb))
        return [k for k in sd if k not in used]

    @torch.no_grad()
    def merged_delta(self, tenant: str, mod_name: str, pname: str) -> torch.Tensor:
        """``scale · B A`` of one projection (for merge-and-sync to a sampler)."""
        t = self.tenants[tenant]
        m = dict(self.modules)[mod_name]
        r = t.config.r
        return (m.lora_B[pname][t.slot, :, :r].float() @ m.lora_A[pname][t.slot, :r].float()) * t.config.scaling
