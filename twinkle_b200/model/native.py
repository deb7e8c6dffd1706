"""The native training backend: one engine behind the Twinkle model API.

Parity: reference ``src/twinkle/model/transformers/transformers.py:150-1616``
(``TransformersModel``) and ``multi_lora_transformers.py:22-340``
(``MultiLoraTransformersModel``).  Same public methods and the same numerical
contracts (pre-shifted labels, ``logps`` outputs, the ``num_tokens``
normalisation at clip time, per-adapter optimizer groups, HF / PEFT checkpoint
layout) on top of the owned decoder + flat-bucket FSDP engine instead of Hugging
Face modules + ``fully_shard``.
"""
from __future__ import annotations

import json
import math
import os
import time
from contextlib import contextmanager, nullcontext
from typing import Any, Callable, Dict, List, Optional, Sequence, Tuple, Type, Union

import torch
import torch.distributed as dist

from .. import ops
from ..data_format import InputFeature, LossOutput, ModelOutput
from ..infra import remote_class, remote_function, collect_tensor_dict
from ..loss import Loss, torch_loss_mapping
from ..metric import Metric, metric_mapping
from ..models.bridge import hf_to_internal, internal_to_hf
from ..models.config import PRESETS, DecoderConfig, preset
from ..models.decoder import DecoderModel, PackedBatch, build_model
from ..models.layers import lora_batch
from ..module.scheduler import scheduler_mapping
from ..parallel.comm import Communicator
from ..parallel.fsdp import FSDPEngine
from ..processor import InputProcessor, MicroBatch
from ..utils.device_mesh import DeviceMesh
from ..utils.logger import get_logger
from ..utils.nccl_safe import collective_safe
from ..utils.platform import Platform
from ..utils.safetensors_io import SafetensorLazyLoader, StreamingSafetensorSaver
from ..checkpoint_engine import CheckpointEngineMixin
from .base import TwinkleModel
from .multi_lora import LoraConfig, MultiLora
from .optimizer_group import AdamHyper, OptimizerGroup, TrainStatus

logger = get_logger()
_DEFAULT = ''
DEFAULT_LEARNING_RATE = 1e-5
DEFAULT_WEIGHT_DECAY = 0.01
_NO_DECAY_MARKERS = ('bias', 'layernorm', 'rmsnorm', 'norm', '_norm')


def _no_decay(name: str) -> bool:
    low = name.lower()
    return any(m in low for m in _NO_DECAY_MARKERS)


class EngineOptimizer(torch.optim.Optimizer):
    """``torch.optim.Optimizer``-shaped facade so stock LR schedulers can drive
    the fused AdamW of the engine.  Two groups as in the reference (decay /
    no-decay, ``transformers.py:787-832``) carrying ``param_names``."""

    def __init__(self, hyper: AdamHyper, decay_names: List[str], no_decay_names: List[str]):
        self._dummies = [torch.nn.Parameter(torch.zeros(1)), torch.nn.Parameter(torch.zeros(1))]
        groups = [dict(params=[self._dummies[0]], weight_decay=hyper.weight_decay, param_names=decay_names),
                  dict(params=[self._dummies[1]], weight_decay=0.0, param_names=no_decay_names)]
        super().__init__(groups, dict(lr=hyper.lr, betas=tuple(hyper.betas), eps=hyper.eps, weight_decay=hyper.weight_decay))
        self.step_fn: Optional[Callable[[], None]] = None

    def step(self, closure=None):  # type: ignore[override]
        if self.step_fn is not None:
            self.step_fn()

    def zero_grad(self, set_to_none: bool = True):  # type: ignore[override]
        pass


@remote_class()
class TransformersModel(TwinkleModel, CheckpointEngineMixin):
    """Full-parameter or single-adapter training on the owned decoder.

    ``model_id`` is a directory with ``config.json`` + safetensors, or the name
    of an architecture preset (``'qwen3-8b'``, ``'tiny-dense'`` …) for random
    initialisation; ``config`` (``DecoderConfig`` or HF dict) overrides it.
    """

    def __init__(self, model_id: Optional[str] = None, config: Union[DecoderConfig, Dict[str, Any], None] = None,
                 device_mesh: DeviceMesh = None, mixed_precision: str = 'bf16', strategy: str = 'native_fsdp',
                 task: str = 'causal_lm', seed: int = 0, grad_dtype: Optional[str] = None, comm_backend: str = 'auto',
                 gradient_accumulation_steps: int = 1, max_loras: int = 0, max_r: int = 0, device=None,
                 fsdp_group_dims: Optional[Sequence[str]] = None, keep_attention: bool = True, **kwargs):
        self._try_init_process_group()
        self.keep_attention = keep_attention
        self.device_mesh = device_mesh or DeviceMesh.from_sizes(dp_size=Platform.get_world_size())
        self.task = task
        self.model_id = model_id
        self.seed = seed
        self.strategy_name = strategy
        self.fsdp_group_dims = tuple(fsdp_group_dims) if fsdp_group_dims else None
        self.comm_backend = comm_backend
        self.device = torch.device(device) if device is not None else Platform.current_device()
        if self.device.type == 'cuda' and self.device.index is None:
            self.device = torch.device('cuda', torch.cuda.current_device())
        on_gpu = self.device.type == 'cuda'
        if on_gpu:
            torch.cuda.set_device(self.device)
        self.compute_dtype = {'bf16': torch.bfloat16, 'fp16': torch.float16, 'no': torch.float32, 'fp32': torch.float32}.get(
            mixed_precision, torch.bfloat16) if on_gpu else torch.float32
        self.grad_dtype = {'bf16': torch.bfloat16, 'fp32': torch.float32, None: torch.float32}[grad_dtype]
        # ---- architecture + weights
        if isinstance(config, DecoderConfig):
            self.config = config
        elif isinstance(config, dict):
            self.config = DecoderConfig.from_hf(config)
        elif model_id and model_id.lower() in PRESETS:
            self.config = preset(model_id)
        elif model_id and os.path.isdir(model_id):
            self.config = DecoderConfig.from_pretrained(model_id)
        else:
            from ..hub import HubOperation
            path = HubOperation.download_model(model_id)
            self.model_id = path
            self.config = DecoderConfig.from_pretrained(path)
        load_dir = self.model_id if self.model_id and os.path.isdir(str(self.model_id)) else None
        self.model: DecoderModel = build_model(self.config, device=self.device, dtype=self.compute_dtype, seed=seed,
                                               init=load_dir is None)
        if load_dir is not None:
            self._load_hf_weights(load_dir)
        # vision-language models: ``freeze_vision=True`` keeps the tower as it is in a full-parameter run (it is frozen
        # anyway under LoRA); ``freeze_llm=True`` trains the tower and its mergers only (connector alignment)
        if kwargs.get('freeze_vision') and getattr(self.model, 'visual', None) is not None:
            self.model.visual.requires_grad_(False)
        if kwargs.get('freeze_llm'):
            for n, p in self.model.named_parameters():
                if not n.startswith('visual.'):
                    p.requires_grad_(False)
        self.multi_lora: Optional[MultiLora] = None
        self._pool_cfg = (max_loras, max_r)
        self.engine: Optional[FSDPEngine] = None
        self.optimizer_groups: Dict[str, OptimizerGroup] = {
            _DEFAULT: OptimizerGroup(adapter_name=_DEFAULT, gradient_accumulation_steps=gradient_accumulation_steps)}
        self._patches: List[Any] = []
        self._forward_ran = self._backward_ran = False
        self._pending_scale: Dict[str, float] = {}
        self._lora_state: Dict[str, Dict[str, Any]] = {}  # tenant → {pool name: {master, exp_avg, exp_avg_sq}}
        self.active_adapter: Optional[str] = None
        self.step_timer_ms: Optional[float] = None

    # ------------------------------------------------------------ plumbing
    def _load_hf_weights(self, directory: str) -> None:
        loader = SafetensorLazyLoader(directory)
        with torch.no_grad():
            for name, p in self.model.named_parameters():
                if 'lora' in name:
                    continue
                try:
                    t = hf_to_internal(name, self.config, loader.get)
                except KeyError:
                    if name == 'lm_head.weight' and 'model.embed_tokens.weight' in loader:
                        t = loader.get('model.embed_tokens.weight')
                    else:
                        raise
                p.copy_(t.to(p.dtype))
        loader.close()

    def _dp_comm(self) -> Communicator:
        if not hasattr(self, '_comm'):
            group = None
            if dist.is_available() and dist.is_initialized():
                # context-parallel ranks hold different tokens of the same sequences: for parameters and gradients they
                # are data ranks like any other
                dims = [d for d in ('dp', 'fsdp', 'cp') if self.device_mesh.has_dim(d)]
                if dims and self.device_mesh.world_size == dist.get_world_size() and len(dims) < len(self.device_mesh.mesh_dim_names):
                    group = self.device_mesh.get_dim_group(tuple(dims))
            self._comm = Communicator(group, self.device, single=self.device_mesh.world_size == 1)
        return self._comm

    @property
    def sp_size(self) -> int:
        return self.device_mesh.ulysses_size or 1

    def _hybrid_shard_dims(self) -> Optional[Tuple[str, ...]]:
        """Axes the parameters are sharded over when that is NOT the whole data group.  ``fsdp_group_dims=('fsdp',)``
        asks for it outright; ``strategy='accelerate'`` on a mesh with both ``dp`` and ``fsdp`` larger than one means
        the same thing, as in the reference (``strategy/accelerate.py:106-110``: replicate over ``dp``, shard over
        ``fsdp``); ``native_fsdp`` shards over the flattened mesh (``strategy/native_fsdp.py:445-451``)."""
        m = self.device_mesh
        data_dims = [d for d in ('dp', 'fsdp', 'cp') if m.has_dim(d)]
        dims = tuple(self.fsdp_group_dims) if self.fsdp_group_dims else None
        if dims is None and self.strategy_name == 'accelerate' and (m.dp_world_size or 1) > 1 and (m.fsdp_world_size or 1) > 1:
            dims = ('fsdp', )
        if dims is None or set(dims) >= set(data_dims) or not (dist.is_available() and dist.is_initialized()):
            return None
        if (m.ep_size or 1) > 1 or self.sp_size > 1:
            raise NotImplementedError('hybrid sharding combines with neither expert nor sequence parallelism here; use the flat sharding of native_fsdp')
        for d in dims:
            if not m.has_dim(d):
                raise ValueError(f"fsdp_group_dims names axis '{d}' that the mesh {m.mesh_dim_names} does not have")
        return dims

    def _lazy_wrap_model(self) -> None:
        """First use: LoRA pool (if any) → expert parallel → sequence parallel →
        sharding engine.  Mirrors the order of the reference's
        ``_lazy_wrap_model`` (``transformers.py:316-339``)."""
        if self.engine is not None:
            return
        comm = self._dp_comm()
        if self.device_mesh.ep_size and self.device_mesh.ep_size > 1 and self.config.is_moe:
            from ..parallel.expert import apply_expert_parallel
            apply_expert_parallel(self.model, self.device_mesh, self.config, self.comm_backend)
        if self.sp_size > 1:
            from ..parallel.ulysses import apply_ulysses
            apply_ulysses(self.model, self.device_mesh, self.config, self.comm_backend)
        if (self.device_mesh.cp_world_size or 1) > 1:
            from ..parallel.context import apply_context_parallel
            apply_context_parallel(self.model, self.device_mesh)
        if comm.world_size > 1 and self.comm_backend in ('auto', 'symm') and self.device.type == 'cuda':
            try:
                from ..parallel.symm import SymmCommunicator
                comm = SymmCommunicator(comm.group, self.device)
                self._comm = comm
            except Exception as e:  # the NCCL path stays correct
                if self.comm_backend == 'symm':
                    raise
                logger.warning(f'peer-memory communicator unavailable ({e}); using NCCL collectives')
        ignored = None
        if self.device_mesh.ep_size and self.device_mesh.ep_size > 1 and self.config.is_moe:
            ignored = lambda n: '.mlp.experts.' in n  # experts are EP-local, not FSDP-sharded over the dp group
        replica = None
        shard_dims = self._hybrid_shard_dims()
        if shard_dims is not None:
            # hybrid sharding: shard inside the listed axes, replicate (and all-reduce gradients) over the other data axes
            other = tuple(d for d in ('dp', 'fsdp', 'cp') if self.device_mesh.has_dim(d) and d not in shard_dims)
            shard = Communicator(self.device_mesh.get_dim_group(shard_dims), self.device)
            replica = Communicator(self.device_mesh.get_dim_group(other), self.device)
            if shard.world_size > 1 and self.comm_backend in ('auto', 'symm') and self.device.type == 'cuda':
                try:
                    from ..parallel.symm import SymmCommunicator
                    shard = SymmCommunicator(shard.group, self.device)
                except Exception as e:
                    if self.comm_backend == 'symm':
                        raise
                    logger.warning(f'peer-memory communicator unavailable ({e}); using NCCL collectives')
            comm = shard
        self.engine = FSDPEngine(self.model, comm, self.compute_dtype, self.device, grad_dtype=self.grad_dtype, ignored=ignored,
                                 keep_attention=self.keep_attention, replica_comm=replica)
        if self.multi_lora is not None:
            self.multi_lora.sync_initial(comm)

    def data_plane(self) -> Dict[str, str]:
        """Which transport each sharded path resolved to at run time: ``'symm'`` (peer-memory kernels over NVLink),
        ``'nccl'`` / ``'gloo'`` (library collectives) or ``'local'`` (one rank).  ``comm_backend='auto'`` falls back
        to the library path when the peer-memory communicator cannot be built; this makes that visible."""
        self._lazy_wrap_model()

        def kind(c) -> str:
            if c is None or getattr(c, 'world_size', 1) <= 1:
                return 'local'
            if hasattr(c, 'peer_ptrs'):
                return 'symm'
            return 'nccl' if getattr(c, 'cuda', False) else 'gloo'

        out = {'fsdp': kind(self.engine.comm)}
        for layer in self.model.layers:
            strat = getattr(getattr(layer, 'self_attn', None), 'attn_parallel', None)
            if strat is not None and hasattr(strat, 'comm'):
                out['ulysses'] = kind(strat.comm)
                break
        for layer in self.model.layers:
            ep = getattr(getattr(layer, 'mlp', None), 'moe_parallel', None)
            if ep is not None:
                out['expert'] = 'symm' if type(ep).__name__ == 'SymmExpertParallel' else kind(getattr(ep, 'comm', None))
                break
        return out

    def _group(self, adapter_name: Optional[str]) -> OptimizerGroup:
        name = adapter_name or _DEFAULT
        if name not in self.optimizer_groups:
            raise KeyError(f'unknown adapter {name!r}; call add_adapter_to_model first')
        return self.optimizer_groups[name]

    # ------------------------------------------------------------- inputs
    def _encode(self, inputs, og: OptimizerGroup) -> List[InputFeature]:
        if isinstance(inputs, dict):
            inputs = [inputs]
        inputs = list(inputs)
        if inputs and isinstance(inputs[0], dict) and 'input_ids' not in inputs[0]:
            if og.template is None:
                raise ValueError('inputs are trajectories but no template is set (set_template)')
            inputs = og.template.batch_encode(inputs)
        return inputs

    def _processor(self, og: OptimizerGroup, micro_batch_size: Optional[int]) -> InputProcessor:
        proc = og.processor
        if proc is None:
            proc = InputProcessor(device_mesh=self.device_mesh, pad_token_id=self.config.pad_token_id or 0)
            og.processor = proc
        proc.micro_batch_size = micro_batch_size
        return proc

    @staticmethod
    def _slice_kwargs(kwargs: Dict[str, Any], lo: int, hi: int, n: int) -> Dict[str, Any]:
        out = {}
        for k, v in kwargs.items():
            if isinstance(v, (list, tuple)) and len(v) == n:
                out[k] = v[lo:hi]
            elif torch.is_tensor(v) and v.dim() >= 1 and v.shape[0] == n:
                out[k] = v[lo:hi]
            elif isinstance(v, dict):
                out[k] = TransformersModel._slice_kwargs(v, lo, hi, n)
            else:
                out[k] = v
        return out

    # ------------------------------------------------------------ forward
    def _forward_micro(self, mb: MicroBatch, og: OptimizerGroup, need_grad: bool, temperature: float = 1.0,
                       return_logits: bool = False, disable_lora: bool = False) -> Dict[str, Any]:
        self._lazy_wrap_model()
        mb = mb.to(self.device)
        extras = mb.extras or {}
        batch = PackedBatch(mb.input_ids, mb.position_ids, mb.cu_seqlens, mb.max_seqlen, mb.labels,
                            routed_experts=self._routed_for(extras, mb), seq_lens=list(mb.seq_lens))
        if extras.get('pixel_values') is not None:  # vision-language batch: patches, grids and three-component positions
            dt = next(self.model.parameters()).dtype
            batch.pixel_values = extras['pixel_values'].to(self.device, dt)
            batch.image_grid_thw = extras['image_grid_thw'].to(self.device)
            batch.position_ids = extras['mrope_position_ids'].to(self.device)
            if extras.get('vision_rows') is not None:
                batch.vision_rows = extras['vision_rows'].to(self.device)
        loss_obj = og.loss_instance
        want_entropy = bool(getattr(loss_obj, 'require_entropy', False))
        want_logits = return_logits or bool(getattr(loss_obj, 'require_logits', False))
        want_hidden = bool(getattr(loss_obj, 'require_hidden', False)) or self.task == 'embedding'
        lb = None
        if self.multi_lora is not None and og.adapter_name in self.multi_lora.tenants and not disable_lora:
            lb = self.multi_lora.batch_for(og.adapter_name, int(mb.input_ids.numel()), self.device)
        grad_ctx = nullcontext() if need_grad else torch.no_grad()
        with grad_ctx, lora_batch(lb):
            self.engine.begin_step(need_grad)
            self.engine.aux_values.clear()
            hidden = self.model(batch)
            out: Dict[str, Any] = {}
            if self.task == 'embedding':
                out['embeddings'] = self._pool_embeddings(hidden, mb)
            elif want_hidden:
                out['hidden_states'] = hidden
                out['lm_head_weight'] = self.model.head_weight()
            if self.task != 'embedding':
                logps, ent = self.model.token_logprobs(hidden, mb.labels, temperature, want_entropy)
                out['logps'], out['entropies'] = logps, ent
                if want_logits:
                    out['logits'] = self.model.logits(hidden) / temperature if temperature != 1.0 else self.model.logits(hidden)
            aux = self.model.aux_loss()
            if self.engine.aux_values:
                aux_val = torch.stack(self.engine.aux_values).mean() * self.config.router_aux_loss_coef
                out['aux_loss'] = aux_val if aux is None else aux + aux_val
            elif aux is not None:
                out['aux_loss'] = aux
        routed = self.model.collect_routed_experts()
        if routed is not None:
            out['routed_experts'] = routed
        return self._gather_sequence_parallel(out, mb)

    def _routed_for(self, extras, mb):
        r = extras.get('routed_experts') if extras else None
        if not r or any(x is None for x in r):
            return None
        # per-feature [L, T_i, k] → per-layer [ΣT, k].  A sampler records one row per token it fed through the model,
        # which is one fewer than the feature holds (the last sampled token is never fed; reference
        # processor/base.py:826-850 pads the same gap): missing rows become -1 = route freely, extra rows are cut.
        per_layer = []
        n_layers = len(r[0])
        lens = list(mb.seq_lens) if len(mb.seq_lens) == len(r) else [None] * len(r)

        def fit(t, n):
            t = torch.as_tensor(t).long()
            if n is None or t.shape[0] == n:
                return t
            if t.shape[0] > n:
                return t[:n]
            return torch.cat([t, torch.full((n - t.shape[0], t.shape[1]), -1, dtype=torch.long)], 0)

        for l in range(n_layers):
            per_layer.append(torch.cat([fit(x[l], n) for x, n in zip(r, lens)], 0).to(self.device))
        if mb.local_index is not None:
            per_layer = [p[mb.local_index.to(p.device)] for p in per_layer]
        return per_layer

    def _pool_embeddings(self, hidden: torch.Tensor, mb: MicroBatch) -> torch.Tensor:
        """Last-token pooling per sequence (sum over SP ranks places it on all)."""
        ends = torch.tensor([sum(mb.seq_lens[:i + 1]) - 1 for i in range(len(mb.seq_lens))], device=hidden.device)
        if mb.local_index is None:
            return hidden[ends]
        li = mb.local_index.to(hidden.device)
        emb = hidden.new_zeros(len(mb.seq_lens), hidden.shape[-1])
        pos = torch.searchsorted(li, ends)
        ok = (pos < li.numel()) & (li[pos.clamp_max(li.numel() - 1)] == ends)
        emb[ok] = hidden[pos[ok]]
        self._sp_comm().all_reduce(emb)
        return emb

    def _sp_comm(self) -> Communicator:
        if not hasattr(self, '_sp'):
            from ..parallel.ulysses import sp_group_for
            self._sp = Communicator(sp_group_for(self.device_mesh), self.device)
        return self._sp

    def _gather_sequence_parallel(self, out: Dict[str, Any], mb: MicroBatch) -> Dict[str, Any]:
        """Per-token outputs of the SP peers are concatenated (each rank holds a
        contiguous chunk of the packed row), differentiable for ``logps``, then
        cut into ``[n_seq, max_len]``."""
        labels = mb.labels
        if self.sp_size > 1:
            from ..parallel.ulysses import gather_tokens
            comm = self._sp_comm()
            for k in ('logps', 'entropies'):
                if out.get(k) is not None:
                    out[k] = gather_tokens(out[k], comm)
            if out.get('logits') is not None:
                out['logits'] = gather_tokens(out['logits'], comm)
            labels = comm.all_gather_tensor(labels)
        cp = self.device_mesh.cp_world_size or 1
        if cp > 1:
            # zig-zag shards: concatenate the peers' pieces (differentiable for this rank's own piece) and put every
            # token back at its position in the full packed row, so the loss sees whole sequences on every rank
            from ..parallel.context import cp_group_for, gather_zigzag_rows
            if not hasattr(self, '_cp'):
                self._cp = Communicator(cp_group_for(self.device_mesh), self.device)
            comm = self._cp

            def full_row(x, fill, differentiable):
                return gather_zigzag_rows(x, comm, mb.seq_lens, fill, differentiable)

            for k in ('logps', 'entropies', 'logits'):
                if out.get(k) is not None:
                    out[k] = full_row(out[k], 0, True)
            labels = full_row(labels, -100, False)
        out['packed_labels'] = labels
        for k in ('logps', 'entropies', 'logits'):
            if out.get(k) is not None:
                out[k] = InputProcessor.unpack_packed_sequences(out[k], mb.seq_lens, 0)
        out['labels'] = InputProcessor.unpack_packed_sequences(labels, mb.seq_lens, -100)
        return out

    def _loss_micro(self, og: OptimizerGroup, out: Dict[str, Any], loss_kwargs: Dict[str, Any], is_training: bool = True):
        st = og.status(is_training)
        inputs = {'labels': out['labels']}
        res = og.loss_instance(inputs, out, **loss_kwargs)
        loss = res['loss'] if isinstance(res, dict) else res
        nt = res.get('num_tokens', 0) if isinstance(res, dict) else 0
        nt_f = float(nt) if nt is not None else 0.0
        contrib = (nt_f if nt_f > 0 else 1.0) / (self.sp_size * (self.device_mesh.cp_world_size or 1))
        if out.get('aux_loss') is not None and torch.is_tensor(out['aux_loss']):
            # scale so that after the later division by the denominator the aux term is O(coef)
            loss = loss + out['aux_loss'] * (nt_f if nt_f > 0 else 1.0)
        st.num_tokens += contrib
        st.loss_value = loss
        st.loss_sum += float(loss.detach())
        st.outputs = out
        if self.engine is not None:
            self.engine.aux_grad_weight = self.config.router_aux_loss_coef * (nt_f if nt_f > 0 else 1.0) / max(
                1, sum(1 for l in self.model.layers if getattr(l, 'is_moe', False)))
        return loss, nt_f

    # ----------------------------------------------------- public: forward
    @remote_function(dispatch='slice_dp', collect=collect_tensor_dict)
    def forward(self, *, inputs, adapter_name: Optional[str] = None, temperature: float = 1.0, return_logits: bool = False,
                disable_lora: bool = False, **kwargs) -> ModelOutput:
        og = self._group(adapter_name)
        feats = self._encode(inputs, og)
        mbs = self._processor(og, None)(feats)
        out = self._forward_micro(mbs[0], og, True, temperature, return_logits, disable_lora)
        og.train_status.inputs, og.train_status.outputs, og.train_status.forward_kwargs = feats, out, kwargs
        self._forward_ran = True
        og.last_forward_training = True
        return self._public_outputs(out)

    @remote_function(dispatch='slice_dp', collect=collect_tensor_dict)
    def forward_only(self, *, inputs, adapter_name: Optional[str] = None, temperature: float = 1.0, return_logits: bool = False,
                     disable_lora: bool = False, micro_batch_size: Optional[int] = None, **kwargs) -> ModelOutput:
        og = self._group(adapter_name)
        feats = self._encode(inputs, og)
        outs, raw = [], []
        for mb in self._processor(og, micro_batch_size)(feats):
            o = self._forward_micro(mb, og, False, temperature, return_logits, disable_lora)
            self.engine.end_forward_only()
            raw.append(o)
            outs.append(self._public_outputs(o))
        # what calculate_loss evaluates next: every micro-batch of this call, with the caller's loss arguments
        og.eval_status.inputs, og.eval_status.outputs, og.eval_status.forward_kwargs = feats, raw, kwargs
        og.last_forward_training = False
        return collect_tensor_dict(outs) if len(outs) > 1 else outs[0]

    @staticmethod
    def _public_outputs(out: Dict[str, Any]) -> Dict[str, Any]:
        pub = {}
        for k in ('logps', 'entropies', 'logits', 'embeddings', 'routed_experts', 'labels'):
            v = out.get(k)
            if v is None:
                continue
            pub[k] = v.detach() if torch.is_tensor(v) else v
        return pub

    @remote_function(collect='mean')
    def calculate_loss(self, adapter_name: Optional[str] = None, **kwargs) -> float:
        """Loss of the latest forward.  After ``forward`` it is the training loss that ``backward`` will differentiate;
        after ``forward_only`` it is an evaluation loss over every micro-batch of that call, accumulated into the
        evaluation metrics (reference ``transformers.py:620-665`` picks the status by the module's train/eval mode)."""
        og = self._group(adapter_name)
        if getattr(og, 'last_forward_training', True):
            st = og.train_status
            kw = dict(st.forward_kwargs or {})
            kw.update(kwargs)
            loss, _ = self._loss_micro(og, st.outputs, kw)
            return float(loss.detach())
        st = og.eval_status
        kw = dict(st.forward_kwargs or {})
        kw.update(kwargs)
        outs = st.outputs if isinstance(st.outputs, list) else [st.outputs]
        total, tokens = 0.0, 0.0
        with torch.no_grad():
            for o in outs:
                loss, nt = self._loss_micro(og, o, kw, is_training=False)
                total += float(loss.detach())
                tokens += nt
                for m in st.metrics:
                    m.accumulate({'labels': o.get('labels')}, {'loss': float(loss.detach()), 'num_tokens': nt, 'logps': o.get('logps')},
                                 step_done=False, loss_instance=getattr(og.loss_instance, 'loss', og.loss_instance))
        st.loss_value = None
        st.outputs = outs  # _loss_micro leaves the last micro-batch there
        return total / tokens if tokens > 0 else total / max(len(outs), 1)

    @remote_function()
    def backward(self, adapter_name: Optional[str] = None, **kwargs) -> None:
        og = self._group(adapter_name)
        loss = og.train_status.loss_value
        if loss is None:
            raise RuntimeError('backward called before calculate_loss')
        loss.backward()
        self.engine.end_backward()
        og.train_status.loss_value = None
        og.cur_step += 1
        og.grad_ready = True
        self._backward_ran = True

    def _force_zero_backward(self) -> None:
        """Keep collectives aligned after a failure between forward and backward."""
        for og in self.optimizer_groups.values():
            out = og.train_status.outputs
            if out and torch.is_tensor(out.get('logps')) and out['logps'].requires_grad:
                (torch.nan_to_num(out['logps']).sum() * 0.0).backward()
                self.engine.end_backward()
                return

    @remote_function(dispatch='slice_dp', collect=collect_tensor_dict)
    @collective_safe
    def forward_backward(self, *, inputs, adapter_name: Optional[str] = None, micro_batch_size: Optional[int] = None,
                         temperature: float = 1.0, gradient_accumulation_steps: Optional[int] = None,
                         disable_lora: bool = False, **kwargs) -> ModelOutput:
        """Forward + loss + backward over every micro-batch of ``inputs``;
        gradients accumulate in the fp32 shards.  Loss keyword arguments whose
        first dimension equals the number of features are sliced alongside."""
        og = self._group(adapter_name)
        feats = self._encode(inputs, og)
        n = len(feats)
        proc = self._processor(og, micro_batch_size)
        groups = proc.split_micro_batches(proc.normalize(feats))
        results, lo = [], 0
        total_loss, total_tok = 0.0, 0.0
        for g in groups:
            hi = lo + len(g)
            mb = proc._pack(g)
            from ..utils.profiling import PHASES
            with PHASES('forward'):
                out = self._forward_micro(mb, og, True, temperature, False, disable_lora)
                self._forward_ran = True
                loss, nt = self._loss_micro(og, out, self._slice_kwargs(kwargs, lo, hi, n))
            with PHASES('backward'):
                loss.backward()
                self.engine.end_backward()
            self._backward_ran = True
            og.train_status.loss_value = None
            total_loss += float(loss.detach())
            total_tok += nt
            pub = self._public_outputs(out)
            results.append(pub)
            lo = hi
        og.cur_step += 1
        og.grad_ready = True
        og.consumed_train_samples += n * max(self.device_mesh.data_world_size, 1)
        merged = collect_tensor_dict(results) if len(results) > 1 else results[0]
        merged['loss'] = total_loss / total_tok if total_tok > 0 else total_loss / max(len(groups), 1)
        merged['num_tokens'] = total_tok
        for m in og.train_status.metrics:
            m.accumulate({'labels': merged.get('labels')}, {'loss': total_loss, 'num_tokens': total_tok, 'logps': merged.get('logps')},
                         step_done=False, **{k: v for k, v in kwargs.items() if k in ('old_logps', 'advantages')},
                         loss_instance=getattr(og.loss_instance, 'loss', og.loss_instance))
        return merged

    # ------------------------------------------------------ optimiser side
    def _trainable_lora_slices(self, og: OptimizerGroup):
        if self.multi_lora is None or og.adapter_name not in self.multi_lora.tenants:
            return []
        return self.multi_lora.tenant_slices(og.adapter_name)

    @remote_function(collect='first')
    def clip_grad_norm(self, max_grad_norm: float = 1.0, norm_type=2, adapter_name: Optional[str] = None, **kwargs) -> float:
        """Divide by the global denominator (Σ tokens for sum-losses, number of
        loss evaluations for mean-losses), measure the global L2 norm and clip.
        The division and the clip coefficient are folded into one scale that the
        fused AdamW applies while reading the gradient."""
        og = self._group(adapter_name)
        if not og.do_grad_sync(kwargs.get('gradient_accumulation_steps')):
            return og._last_grad_norm or 0.0
        comm = self._dp_comm()
        if self.engine is not None:
            self.engine.finish_grads()
        denom = comm.all_reduce_scalar(og.train_status.num_tokens, 'sum')
        denom = denom if denom > 0 else 1.0
        sq = torch.zeros((), dtype=torch.float32, device=self.device)
        sq_ep = torch.zeros((), dtype=torch.float32, device=self.device)  # expert-parallel tensors: distinct per EP rank
        has_ep = False
        slices = self._trainable_lora_slices(og)
        if slices:
            for _, p, slot in slices:
                if p.grad is not None:
                    v = ops.sumsq(p.grad[slot].contiguous())
                    if getattr(p, '_ep_local', False):
                        sq_ep, has_ep = sq_ep + v, True
                    else:
                        sq = sq + v
        elif self.engine is not None:
            sq_sh = self.engine.grad_norm_sq()
            self.engine.comm.all_reduce(sq_sh)  # over the shard group: under hybrid sharding the replicas hold equal shards
            sq = sq + sq_sh
            for _, p in self.engine.replicated:
                if p.requires_grad and p.grad is not None:
                    v = ops.sumsq(p.grad)
                    if getattr(p, '_ep_local', False):
                        sq_ep, has_ep = sq_ep + v, True
                    else:
                        sq = sq + v
        ep_comm = getattr(self.model, '_ep_comm', None)
        if ep_comm is not None and ep_comm.world_size > 1:  # every EP rank joins, with or without local expert grads
            sq_ep = sq_ep.reshape(1)
            ep_comm.all_reduce(sq_ep)
            sq = sq + sq_ep[0]
        elif has_ep:
            sq = sq + sq_ep
        norm = float(sq.sqrt()) / denom
        if self.device.type == 'cuda':
            code = ops.ext().read_and_clear_error()
            if code:
                raise RuntimeError(f'a device-side bounded wait expired (code {code}): a peer rank is missing or a pipeline stalled')
        coef = 1.0
        if max_grad_norm is not None and max_grad_norm > 0:
            coef = min(1.0, max_grad_norm / (norm + 1e-6))
        self._pending_scale[og.adapter_name] = coef / denom
        og._last_grad_norm = norm
        og.train_status.num_tokens = 0.0
        return norm

    @remote_function()
    def step(self, adapter_name: Optional[str] = None, optim_params: Optional[Dict[str, Any]] = None, **kwargs) -> None:
        og = self._group(adapter_name)
        if not og.do_grad_sync(kwargs.get('gradient_accumulation_steps')):
            return
        if og.optimizer is None:
            self.set_optimizer('AdamW', adapter_name=adapter_name)
        opt = og.optimizer
        if optim_params:
            for g in opt.param_groups:
                if 'lr' in optim_params:
                    g['lr'] = optim_params['lr']
                if 'betas' in optim_params:
                    g['betas'] = tuple(optim_params['betas'])
                if 'eps' in optim_params:
                    g['eps'] = optim_params['eps']
                if 'weight_decay' in optim_params and g['weight_decay'] > 0:
                    g['weight_decay'] = optim_params['weight_decay']
        og.optim_steps += 1
        if self.engine is not None:
            self.engine.finish_grads()
        opt._opt_called = True  # the fused update below is this optimizer's step; stock LR schedulers check the flag
        scale = self._pending_scale.pop(og.adapter_name, 1.0)
        fence = getattr(self._dp_comm(), 'step_barrier', None)
        if fence is not None:
            fence()  # peers have finished reading my parameter shards and gradient buffers
        gd, gn = opt.param_groups[0], opt.param_groups[1]
        lr, betas, eps = gd['lr'], gd['betas'], gd['eps']
        wd_for = lambda name: 0.0 if _no_decay(name) else gd['weight_decay']
        slices = self._trainable_lora_slices(og)
        if slices:
            st = self._lora_state.setdefault(og.adapter_name, {})
            for name, p, slot in slices:
                if p.grad is None:
                    continue
                view = p.data[slot]
                s = st.get(name)
                if s is None:
                    s = dict(master=view.float().clone(), exp_avg=torch.zeros_like(view, dtype=torch.float32),
                             exp_avg_sq=torch.zeros_like(view, dtype=torch.float32))
                    st[name] = s
                ops.adamw_step(s['master'].view(-1), s['exp_avg'].view(-1), s['exp_avg_sq'].view(-1),
                               p.grad[slot].contiguous().view(-1), view.view(-1), lr, betas[0], betas[1], eps,
                               gd['weight_decay'], og.optim_steps, scale)
        else:
            for b in self.engine.trainable_buckets():
                b.adamw(lr, betas, eps, wd_for, og.optim_steps, scale)
            for name, p in self.engine.replicated:
                if p.requires_grad and p.grad is not None:
                    s = self._lora_state.setdefault('#replicated', {}).setdefault(name, None)
                    if s is None:
                        s = dict(master=p.data.float().clone(), exp_avg=torch.zeros_like(p.data, dtype=torch.float32),
                                 exp_avg_sq=torch.zeros_like(p.data, dtype=torch.float32))
                        self._lora_state['#replicated'][name] = s
                    ops.adamw_step(s['master'].view(-1), s['exp_avg'].view(-1), s['exp_avg_sq'].view(-1),
                                   p.grad.contiguous().view(-1), p.data.view(-1), lr, betas[0], betas[1], eps,
                                   wd_for(name), og.optim_steps, scale)
        if fence is not None:
            fence()  # nobody gathers the shards before every rank has updated its own
        og.grad_ready = False

    @remote_function()
    def zero_grad(self, adapter_name: Optional[str] = None, **kwargs) -> None:
        og = self._group(adapter_name)
        if not og.do_grad_sync(kwargs.get('gradient_accumulation_steps')):
            return
        slices = self._trainable_lora_slices(og)
        if slices:
            for _, p, slot in slices:
                if p.grad is not None:
                    p.grad[slot].zero_()
        elif self.engine is not None:
            self.engine.zero_grad()
        og.train_status.num_tokens = 0.0

    @remote_function()
    def lr_step(self, adapter_name: Optional[str] = None, **kwargs) -> None:
        og = self._group(adapter_name)
        if not og.do_grad_sync(kwargs.get('gradient_accumulation_steps')):
            return
        if og.lr_scheduler is not None:
            og.lr_scheduler.step()

    @remote_function(collect='first')
    def clip_grad_and_step(self, max_grad_norm: float = 1.0, norm_type=2, adapter_name: Optional[str] = None, **kwargs):
        from ..utils.profiling import PHASES
        with PHASES('grad_norm'):
            norm = self.clip_grad_norm(max_grad_norm, norm_type, adapter_name=adapter_name, **kwargs)
        with PHASES('optimizer'):
            self.step(adapter_name=adapter_name, **kwargs)
            self.zero_grad(adapter_name=adapter_name, **kwargs)
        self.lr_step(adapter_name=adapter_name, **kwargs)
        og = self._group(adapter_name)
        for m in og.train_status.metrics:
            if type(m).__name__ in ('LossMetric', ):
                m.grad_norm = max(m.grad_norm or 0.0, norm) if hasattr(m, 'grad_norm') else norm
            if type(m).__name__ == 'TrainMetric':
                m.accumulate(None, None, lr=og.current_lr()[0])
        return norm

    # ------------------------------------------------------------ setters
    @remote_function()
    def set_loss(self, loss_cls, adapter_name: Optional[str] = None, **kwargs) -> None:
        og = self._group(adapter_name)
        if isinstance(loss_cls, str):
            loss_cls = torch_loss_mapping[loss_cls]
        loss = loss_cls(**kwargs) if isinstance(loss_cls, type) else loss_cls
        og.set_loss(loss)

    def _param_names(self, og: OptimizerGroup) -> List[str]:
        slices = self._trainable_lora_slices(og)
        if slices:
            return [n for n, _, _ in slices]
        return [n for n, p in self.model.named_parameters() if p.requires_grad]

    @remote_function()
    def set_optimizer(self, optimizer_cls='AdamW', adapter_name: Optional[str] = None, **kwargs) -> None:
        """Only Adam-family optimisers exist in the engine (fused AdamW kernel);
        ``optimizer_cls`` may be ``'AdamW'``/``torch.optim.AdamW``/``'Adam'``."""
        og = self._group(adapter_name)
        name = optimizer_cls if isinstance(optimizer_cls, str) else getattr(optimizer_cls, '__name__', 'AdamW')
        if name.lower() not in ('adamw', 'adam', 'fusedadam', 'default'):
            raise ValueError(f'optimizer {name!r} is not available; the engine implements AdamW')
        h = AdamHyper(lr=kwargs.get('lr', DEFAULT_LEARNING_RATE), betas=tuple(kwargs.get('betas', (0.9, 0.999))),
                      eps=kwargs.get('eps', 1e-8),
                      weight_decay=kwargs.get('weight_decay', DEFAULT_WEIGHT_DECAY if name.lower() != 'adam' else 0.0))
        og.hyper = h
        names = self._param_names(og)
        og.optimizer = EngineOptimizer(h, [n for n in names if not _no_decay(n)], [n for n in names if _no_decay(n)])

    @remote_function()
    def set_lr_scheduler(self, scheduler_cls, adapter_name: Optional[str] = None, **kwargs) -> None:
        og = self._group(adapter_name)
        if og.optimizer is None:
            self.set_optimizer('AdamW', adapter_name=adapter_name)
        if isinstance(scheduler_cls, str):
            from ..module.scheduler import resolve_scheduler
            scheduler_cls = resolve_scheduler(scheduler_cls)
        og.lr_scheduler = scheduler_cls(og.optimizer, **kwargs) if isinstance(scheduler_cls, type) else scheduler_cls

    @remote_function()
    def set_template(self, template_cls, adapter_name: Optional[str] = None, **kwargs) -> None:
        from ..template import template_mapping, Template
        og = self._group(adapter_name)
        if isinstance(template_cls, str):
            template_cls = template_mapping.get(template_cls, Template)
        kwargs.setdefault('model_id', self.model_id)
        from ..template.base import Qwen2VLTemplate
        if isinstance(template_cls, type) and issubclass(template_cls, Qwen2VLTemplate) and self.config.vision:
            kwargs.setdefault('vision_config', self.config.vision)      # image parts are cut into this model's own patch grid
        og.template = template_cls(**kwargs) if isinstance(template_cls, type) else template_cls

    @remote_function()
    def set_processor(self, processor_cls, adapter_name: Optional[str] = None, **kwargs) -> None:
        og = self._group(adapter_name)
        if isinstance(processor_cls, str):
            processor_cls = InputProcessor
        kwargs.setdefault('device_mesh', self.device_mesh)
        og.processor = processor_cls(**kwargs) if isinstance(processor_cls, type) else processor_cls

    @remote_function()
    def add_metric(self, metric_cls, is_training: Optional[bool] = None, adapter_name: Optional[str] = None, **kwargs) -> None:
        og = self._group(adapter_name)
        if isinstance(metric_cls, str):
            metric_cls = metric_mapping[metric_cls]
        m = metric_cls(device_mesh=self.device_mesh, **kwargs) if isinstance(metric_cls, type) else metric_cls
        if is_training in (None, True):
            og.train_status.metrics.append(m)
        if is_training in (None, False):
            og.eval_status.metrics.append(m)

    @remote_function(collect='first')
    def calculate_metric(self, is_training: bool = True, adapter_name: Optional[str] = None, **kwargs) -> Dict[str, Any]:
        og = self._group(adapter_name)
        out: Dict[str, Any] = {}
        for m in og.status(is_training).metrics:
            out.update(m.calculate())
        return out

    @remote_function()
    def apply_patch(self, patch_cls, **kwargs) -> None:
        from ..patch import apply_patch
        self._patches.append(apply_patch(self, patch_cls, **kwargs))

    # ------------------------------------------------------------- adapters
    @remote_function()
    def add_adapter_to_model(self, adapter_name: str, config_or_dir, **kwargs) -> None:
        """Bind ``adapter_name`` to a LoRA slot.  The pool is created on the
        first call (rank = the adapter's rank unless ``max_r`` was given)."""
        if self.engine is not None and self.multi_lora is None:
            raise RuntimeError('add_adapter_to_model must precede the first forward')
        cfg = LoraConfig.from_any(config_or_dir)
        if self.multi_lora is None:
            max_loras, max_r = self._pool_cfg
            self.multi_lora = MultiLora(self.model, max_loras or 1, max_r or cfg.r, seed=self.seed)
        self.multi_lora.acquire_lora(adapter_name, cfg)
        og = OptimizerGroup(adapter_name=adapter_name, adapter_config=cfg,
                            gradient_accumulation_steps=kwargs.get('gradient_accumulation_steps', 1))
        self.optimizer_groups[adapter_name] = og
        if isinstance(config_or_dir, str) and os.path.isfile(os.path.join(config_or_dir, 'adapter_model.safetensors')):
            self._load_adapter_file(adapter_name, config_or_dir)
        if self.active_adapter is None:
            self.active_adapter = adapter_name

    @remote_function()
    def remove_adapter(self, adapter_name: str, **kwargs) -> None:
        if self.multi_lora is not None and self.multi_lora.has(adapter_name):
            self.multi_lora.release_lora(adapter_name)
        self.optimizer_groups.pop(adapter_name, None)
        self._lora_state.pop(adapter_name, None)
        self._pending_scale.pop(adapter_name, None)

    @remote_function(collect='first')
    def get_peft_config_dict(self, adapter_name: Optional[str] = None) -> Dict[str, Any]:
        og = self._group(adapter_name)
        return og.adapter_config.to_peft_dict() if og.adapter_config is not None else {}

    # ---- trainer end of a weight sync across worker groups (reference transformers.py:1507-1616)
    @remote_function(collect='first')
    def prepare_checkpoint_engine(self, role: str = 'send', **kwargs) -> Dict[str, Any]:
        return CheckpointEngineMixin.prepare_checkpoint_engine(self, role, **kwargs)

    @remote_function(collect='first', lazy_collect=True)
    def send_weights(self, adapter_name: Optional[str] = None, merge_and_sync: bool = False, lora_only: bool = False, **kwargs) -> Dict[str, float]:
        """Runs on every rank of the model group (gathering sharded parameters is collective); the first rank feeds
        the engine.  Returns to the driver at once so that the sampler's ``receive_weights`` can run alongside."""
        return self._send_weights(adapter_name, merge_and_sync, lora_only)

    @remote_function()
    def finalize_checkpoint_engine(self) -> None:
        CheckpointEngineMixin.finalize_checkpoint_engine(self)

    def _load_adapter_file(self, adapter_name: str, directory: str) -> None:
        from safetensors.torch import load_file
        sd = load_file(os.path.join(directory, 'adapter_model.safetensors'))
        unused = self.multi_lora.set_state_dict(adapter_name, {k: v.to(self.device) for k, v in sd.items()})
        if unused:
            logger.warning(f'{len(unused)} adapter tensors not used, e.g. {unused[:3]}')

    # ----------------------------------------------------------- state dict
    @remote_function(collect='first')
    def get_state_dict(self, adapter_name: Optional[str] = None, hf_format: bool = True, **kwargs) -> Dict[str, torch.Tensor]:
        """Adapter tensors (PEFT names) when ``adapter_name`` is a tenant, else
        the full model in HF naming.  Collective across the sharding group."""
        if adapter_name and self.multi_lora is not None and self.multi_lora.has(adapter_name):
            return self.multi_lora.get_state_dict(adapter_name)
        sd = self._internal_state_dict()
        if not hf_format:
            return sd
        out = {}
        for k, v in sd.items():
            for hk, hv in internal_to_hf(k, v, self.config):
                out[hk] = hv
        return out

    def _internal_state_dict(self) -> Dict[str, torch.Tensor]:
        if self.engine is None:
            return {n: p.detach() for n, p in self.model.named_parameters() if 'lora' not in n}
        sd = self.engine.full_state_dict()
        for n, p in self.engine.replicated:
            if 'lora' not in n:
                sd[n] = self._gather_replicated(n, p)
        return sd

    def _gather_replicated(self, name: str, p: torch.Tensor) -> torch.Tensor:
        """EP-local expert tensors are concatenated over the expert-parallel group."""
        if '.mlp.experts.' in name and (self.device_mesh.ep_size or 1) > 1:
            from ..parallel.expert import ep_group_for
            comm = Communicator(ep_group_for(self.device_mesh), self.device)
            return comm.all_gather_tensor(p.detach())
        return p.detach()

    # ------------------------------------------------------------ save/load
    def _ckpt_dir(self, name: Optional[str], output_dir: Optional[str]) -> str:
        output_dir = output_dir or os.environ.get('TWINKLE_DEFAULT_SAVE_DIR', './output')
        return os.path.join(output_dir, name) if name else output_dir

    @remote_function(collect='first')
    def save(self, name: Optional[str] = None, output_dir: Optional[str] = None, adapter_name: Optional[str] = None,
             save_optimizer: bool = False, interval: int = 1, **kwargs) -> str:
        """Full model: ``config.json`` + sharded ``model-*.safetensors`` in HF
        naming.  Adapter: ``adapter_config.json`` + ``adapter_model.safetensors``
        in PEFT naming.  Optionally the training state (optimizer shards per
        rank, scheduler, RNG, ``trainer_state.json``)."""
        og = self._group(adapter_name)
        path = self._ckpt_dir(name, output_dir)
        is_writer = Platform.is_master()
        if is_writer:
            os.makedirs(path, exist_ok=True)
        if adapter_name and self.multi_lora is not None and self.multi_lora.has(adapter_name):
            sd = self.multi_lora.get_state_dict(adapter_name)
            saver = StreamingSafetensorSaver(path, peft=True, is_writer=is_writer)
            saver.add_many(sd.items())
            saver.finalize()
            if is_writer:
                with open(os.path.join(path, 'adapter_config.json'), 'w') as f:
                    json.dump(og.adapter_config.to_peft_dict(), f, indent=2)
        else:
            sd = self.get_state_dict(hf_format=True)
            saver = StreamingSafetensorSaver(path, is_writer=is_writer)
            saver.add_many(sd.items())
            saver.finalize()
            if is_writer:
                self.config.save_pretrained(path)
        if is_writer and og.template is not None and getattr(og.template, 'tokenizer', None) is not None:
            try:
                og.template.tokenizer.save_pretrained(path)
            except Exception:
                pass
        if save_optimizer:
            self._save_training_state(path, og)
        if dist.is_available() and dist.is_initialized():
            dist.barrier()
        return path

    def _save_training_state(self, path: str, og: OptimizerGroup) -> None:
        rank = Platform.get_rank()
        os.makedirs(path, exist_ok=True)
        state: Dict[str, Any] = {'hyper': og.optimizer.state_dict()['param_groups'] if og.optimizer else None,
                                 'optim_steps': og.optim_steps}
        if self._trainable_lora_slices(og):
            state['lora'] = {k: {kk: vv.cpu() for kk, vv in v.items()} for k, v in self._lora_state.get(og.adapter_name, {}).items()}
        elif self.engine is not None:
            state['buckets'] = {b.name: b.optimizer_state() for b in self.engine.trainable_buckets()}
        torch.save(state, os.path.join(path, f'optimizer_rank{rank}.pt' if Platform.get_world_size() > 1 else 'optimizer.pt'))
        if Platform.is_master():
            if og.lr_scheduler is not None:
                torch.save(og.lr_scheduler.state_dict(), os.path.join(path, 'scheduler.pt'))
            with open(os.path.join(path, 'trainer_state.json'), 'w') as f:
                json.dump({'checkpoint_version': 1, 'cur_step': og.cur_step,
                           'gradient_accumulation_steps': og.gradient_accumulation_steps,
                           'consumed_train_samples': og.consumed_train_samples, 'optim_steps': og.optim_steps}, f)
        torch.save(Platform.get_rng_state(), os.path.join(path, f'rng_state_rank{rank}.pt' if Platform.get_world_size() > 1
                                                          else 'rng_state.pt'))

    @remote_function()
    def load(self, name: Optional[str] = None, output_dir: Optional[str] = None, adapter_name: Optional[str] = None,
             load_optimizer: bool = False, **kwargs) -> None:
        og = self._group(adapter_name)
        path = self._ckpt_dir(name, output_dir)
        if os.path.isfile(os.path.join(path, 'adapter_model.safetensors')):
            if self.multi_lora is None or not self.multi_lora.has(adapter_name or ''):
                self.add_adapter_to_model(adapter_name or 'default', path)
            else:
                self._load_adapter_file(adapter_name, path)
        else:
            loader = SafetensorLazyLoader(path)
            names = [n for n, _ in self.model.named_parameters() if 'lora' not in n]
            for n in names:
                t = hf_to_internal(n, self.config, loader.get)       # a head the file does not carry comes from the embedding
                if self.engine is None or not self.engine.load_full_tensor(n, t):
                    dict(self.model.named_parameters())[n].data.copy_(t.to(self.device))
            loader.close()
        if load_optimizer:
            self._load_training_state(path, og)

    def _load_training_state(self, path: str, og: OptimizerGroup) -> Dict[str, Any]:
        rank = Platform.get_rank()
        f = os.path.join(path, f'optimizer_rank{rank}.pt' if Platform.get_world_size() > 1 else 'optimizer.pt')
        if os.path.isfile(f):
            state = torch.load(f, map_location='cpu', weights_only=True)
            og.optim_steps = state.get('optim_steps', 0)
            if og.optimizer is None:
                self.set_optimizer('AdamW', adapter_name=og.adapter_name or None)
            if state.get('hyper'):
                for g, s in zip(og.optimizer.param_groups, state['hyper']):
                    for k in ('lr', 'betas', 'eps', 'weight_decay'):
                        if k in s:
                            g[k] = s[k] if k != 'betas' else tuple(s[k])
            if 'lora' in state:
                self._lora_state[og.adapter_name] = {k: {kk: vv.to(self.device) for kk, vv in v.items()}
                                                     for k, v in state['lora'].items()}
            if 'buckets' in state:
                self._lazy_wrap_model()
                by_name = {b.name: b for b in self.engine.trainable_buckets()}
                for k, v in state['buckets'].items():
                    by_name[k].load_optimizer_state(v)
        sched = os.path.join(path, 'scheduler.pt')
        if os.path.isfile(sched) and og.lr_scheduler is not None:
            og.lr_scheduler.load_state_dict(torch.load(sched, map_location='cpu', weights_only=True))
        rng = os.path.join(path, f'rng_state_rank{rank}.pt' if Platform.get_world_size() > 1 else 'rng_state.pt')
        if os.path.isfile(rng):
            Platform.set_rng_state(torch.load(rng, map_location='cpu', weights_only=True))
        ts = os.path.join(path, 'trainer_state.json')
        info = {'cur_step': 0, 'consumed_train_samples': 0, 'gradient_accumulation_steps': og.gradient_accumulation_steps}
        if os.path.isfile(ts):
            with open(ts) as fh:
                info.update(json.load(fh))
            og.cur_step = info['cur_step']
            og.consumed_train_samples = info['consumed_train_samples']
            og.gradient_accumulation_steps = info['gradient_accumulation_steps']
        return info

    @remote_function(collect='first')
    def resume_from_checkpoint(self, checkpoint_dir: str, *, resume_only_model: bool = False, adapter_name: Optional[str] = None,
                               **kwargs) -> Dict[str, Any]:
        self.load(None, checkpoint_dir, adapter_name=adapter_name)
        og = self._group(adapter_name)
        if resume_only_model:
            return {'cur_step': 0, 'consumed_train_samples': 0, 'gradient_accumulation_steps': og.gradient_accumulation_steps}
        info = self._load_training_state(checkpoint_dir, og)
        return {k: info[k] for k in ('cur_step', 'consumed_train_samples', 'gradient_accumulation_steps')}

    @remote_function(collect='first')
    def get_train_configs(self, adapter_name: Optional[str] = None, **kwargs) -> str:
        og = self._group(adapter_name)
        n_total = self.config.num_params()
        if self.multi_lora is not None and og.adapter_name in self.multi_lora.tenants:
            r = og.adapter_config.r
            n_train = sum(p[slot].numel() // self.multi_lora.max_r * r for _, p, slot in self._trainable_lora_slices(og))
        else:
            n_train = sum(p.numel() for p in self.model.parameters() if p.requires_grad) if self.engine is None else sum(
                b.numel for b in self.engine.trainable_buckets())
        lines = [f'model: {self.model_id or self.config.model_type} ({n_total / 1e9:.3f}B params)',
                 f'trainable: {n_train:,} ({100.0 * n_train / max(n_total, 1):.4f}%)',
                 f'mesh: dims={self.device_mesh.mesh_dim_names} shape={tuple(self.device_mesh.mesh.shape)} '
                 f'ulysses={self.device_mesh.ulysses_size} ep={self.device_mesh.ep_size}',
                 f'dtype: {self.compute_dtype}, loss: {type(getattr(og.loss_instance, "loss", og.loss_instance)).__name__}',
                 f'optimizer: AdamW lr={og.hyper.lr} wd={og.hyper.weight_decay}, grad_accum={og.gradient_accumulation_steps}']
        if og.adapter_config is not None:
            lines.append(f'adapter: {og.adapter_name} r={og.adapter_config.r} alpha={og.adapter_config.lora_alpha} '
                         f'targets={og.adapter_config.target_modules}')
        return '\n'.join(lines)

    # ------------------------------------------------------ weight export
    def weight_iterator(self, adapter_name: Optional[str] = None, merge_and_sync: bool = False, lora_only: bool = False):
        """(hf_name, tensor) stream for the trainer→sampler sync: LoRA-only
        (PEFT names), merged (base + scaled BA) or plain base weights."""
        if lora_only and adapter_name and self.multi_lora is not None:
            yield from self.multi_lora.get_state_dict(adapter_name).items()
            return
        sd = self._internal_state_dict()
        mods = dict(self.multi_lora.modules) if self.multi_lora is not None else {}
        for k, v in sd.items():
            if merge_and_sync and adapter_name and k.endswith('.weight') and k[:-7] in mods:
                m = mods[k[:-7]]
                parts, off = [], 0
                t = self.multi_lora.tenants[adapter_name]
                for pname, n in m.parts:
                    parts.append(self.multi_lora.merged_delta(adapter_name, k[:-7], pname))
                v = (v.float() + torch.cat(parts, 0)).to(v.dtype)
            for hk, hv in internal_to_hf(k, v, self.config):
                yield hk, hv


@remote_class()
class MultiLoraTransformersModel(TransformersModel):
    """Several tenants on one frozen base.  Every call names its
    ``adapter_name``; each tenant has its own optimizer group."""

    def __init__(self, model_id: Optional[str] = None, config=None, device_mesh: DeviceMesh = None, max_loras: int = 5,
                 max_r: int = 32, max_length: int = 8192, **kwargs):
        super().__init__(model_id=model_id, config=config, device_mesh=device_mesh, max_loras=max_loras, max_r=max_r, **kwargs)
        self.max_length = max_length
        self.multi_lora = MultiLora(self.model, max_loras, max_r, seed=self.seed)

    def _group(self, adapter_name: Optional[str]) -> OptimizerGroup:
        if not adapter_name:
            raise ValueError('adapter_name is required on a multi-LoRA model')
        return super()._group(adapter_name)

    @remote_function()
    def add_adapter_to_model(self, adapter_name: str, config_or_dir, **kwargs) -> None:
        cfg = LoraConfig.from_any(config_or_dir)
        cfg.bias, cfg.lora_dropout = 'none', 0.0  # server-side sanitisation: no bias / modules_to_save / custom init
        self.multi_lora.acquire_lora(adapter_name, cfg)
        self.optimizer_groups[adapter_name] = OptimizerGroup(adapter_name=adapter_name, adapter_config=cfg,
                                                             gradient_accumulation_steps=kwargs.get('gradient_accumulation_steps', 1))
        if isinstance(config_or_dir, str) and os.path.isfile(os.path.join(config_or_dir, 'adapter_model.safetensors')):
            self._load_adapter_file(adapter_name, config_or_dir)

    def check_length(self, inputs, max_length: Optional[int] = None) -> None:
        limit = max_length or self.max_length
        for f in ([inputs] if isinstance(inputs, dict) else inputs):
            n = len(f['input_ids']) if 'input_ids' in f else 0
            if n > limit:
                raise ValueError(f'input of {n} tokens exceeds max_length {limit}')

    @contextmanager
    def adapter(self, adapter_name: str, disable_lora: bool = False):
        prev = self.active_adapter
        self.active_adapter = None if disable_lora else adapter_name
        try:
            yield
        finally:
            self.active_adapter = prev
