"""The tensor- / pipeline-parallel backend ("Megatron-style" path) on the same decoder and kernels.

Parity: reference ``src/twinkle/model/megatron/megatron.py:99-1748`` (``MegatronModel``),
``strategy/megatron.py:14-326`` and ``multi_lora_megatron.py:34-451``.  The reference delegates to
megatron-core, TransformerEngine and ``mcore_bridge``; here the pieces are owned:

* mesh order innermost→outermost ``tp - (cp) - dp - pp`` (the reference's ``'tp-cp-ep-dp-pp'``);
* TP linears with sequence-parallel activations (``parallel.tensor``), vocab-parallel embedding and
  log-prob;
* 1F1B / interleaved-VPP schedule over NCCL p2p (``parallel.pipeline``); micro-batches come from the
  ``InputProcessor``; the last stage computes logps → pluggable ``Loss``; the loss is broadcast from the last
  stage and averaged over dp;
* per-token loss: gradients are divided by the global token count at clip time (same contract as the
  sharded backend);
* weights are saved / loaded in Hugging Face safetensors naming through ``models.bridge`` (TP shards
  gathered per tensor, pipeline stages contribute their layers) — bitwise round trip;
* replicated AdamW state per rank on its own shards (fused AdamW kernel), data-parallel gradient
  all-reduce.
"""
from __future__ import annotations

import json
import math
import os
import re
from typing import Any, Dict, List, Optional, Tuple

import torch
import torch.distributed as dist

from .. import ops
from ..infra import collect_tensor_dict, remote_class, remote_function
from ..loss import torch_loss_mapping
from ..models.bridge import hf_names_for, hf_to_internal, internal_to_hf, tp_rule, tp_shard, tp_unshard
from ..models.config import PRESETS, DecoderConfig, preset
from ..models.decoder import DecoderModel, PackedBatch, build_model
from ..module.scheduler import scheduler_mapping
from ..parallel.comm import Communicator
from ..parallel.pipeline import PipelineRunner
from ..parallel.tensor import SliceTokens, apply_tensor_parallel, make_fused_tp
from ..processor import InputProcessor
from ..utils.device_mesh import DeviceMesh
from ..utils.platform import Platform
from ..utils.safetensors_io import SafetensorLazyLoader, StreamingSafetensorSaver
from .base import TwinkleModel
from .native import EngineOptimizer, _no_decay
from .optimizer_group import AdamHyper, OptimizerGroup


def split_layers(num_layers: int, pp: int, vpp: int) -> List[List[Tuple[int, int]]]:
    """``result[rank][chunk] = (first_layer, last_layer_exclusive)``; virtual stage ``chunk·pp + rank``."""
    stages = pp * vpp
    base, extra = divmod(num_layers, stages)
    bounds, lo = [], 0
    for s in range(stages):
        n = base + (1 if s < extra else 0)
        bounds.append((lo, lo + n))
        lo += n
    return [[bounds[c * pp + r] for c in range(vpp)] for r in range(pp)]


@remote_class()
class _AttachAux(torch.autograd.Function):
    """Passes a pipeline chunk's activations through and gives ``aux`` (a scalar loss term of the chunk's own layers) a
    unit gradient when the activations' gradient arrives, so the term needs no pass of its own through the schedule."""

    @staticmethod
    def forward(ctx, h, aux):
        return h.view_as(h)

    @staticmethod
    def backward(ctx, g):
        return g, (g if g.dim() == 0 else torch.ones((), dtype=g.dtype, device=g.device))


class MegatronModel(TwinkleModel):

    def __init__(self, model_id: Optional[str] = None, config=None, device_mesh: DeviceMesh = None, mixed_precision: str = 'bf16',
                 seed: int = 0, device=None, comm_backend: str = 'auto', recompute: Optional[str] = None,
                 use_distributed_optimizer: bool = True, **kwargs):
        """``recompute='full'`` re-runs every decoder layer in backward instead of keeping its activations (reference
        ``recompute_granularity='full'``, ``megatron/strategy/megatron.py:90-107``).  ``use_distributed_optimizer``
        shards the fp32 master weights and Adam moments of every parameter over the data-parallel ranks (each rank
        updates its slice, the updated slices are all-gathered), as megatron-core's distributed optimizer does."""
        self._try_init_process_group()
        self.recompute = recompute if recompute in ('full', 'selective') else None
        self.use_distributed_optimizer = bool(use_distributed_optimizer)
        self.device_mesh = device_mesh or DeviceMesh.from_sizes(dp_size=Platform.get_world_size())
        self.comm_backend = comm_backend
        mesh = self.device_mesh
        self.device = torch.device(device) if device is not None else Platform.current_device()
        on_gpu = self.device.type == 'cuda'
        if on_gpu:
            torch.cuda.set_device(self.device)
        self.compute_dtype = torch.bfloat16 if (on_gpu and mixed_precision == 'bf16') else torch.float32
        if isinstance(config, DecoderConfig):
            self.config = config
        elif isinstance(config, dict):
            self.config = DecoderConfig.from_hf(config)
        elif model_id and model_id.lower() in PRESETS:
            self.config = preset(model_id)
        else:
            self.config = DecoderConfig.from_pretrained(model_id)
        self.model_id = model_id
        cfg = self.config
        self.tp_size, self.pp_size = mesh.tp_world_size or 1, mesh.pp_world_size or 1
        self.vpp = mesh.vpp_size or 1
        self.tp_rank, self.pp_rank = mesh.tp_rank or 0, mesh.pp_rank or 0
        multi = dist.is_available() and dist.is_initialized() and mesh.world_size > 1
        self.tp_comm = Communicator(mesh.get_dim_group('tp') if multi and mesh.has_dim('tp') else None, self.device, single=self.tp_size == 1)
        self.pp_group = mesh.get_dim_group('pp') if multi and mesh.has_dim('pp') else None
        # context-parallel ranks hold different tokens of the same sequences: for parameters and gradients they are data
        # ranks like any other
        self.cp_size = mesh.cp_world_size or 1
        dp_dims = tuple(d for d in ('dp', 'fsdp', 'cp') if mesh.has_dim(d))
        dp_world = 1
        for d in dp_dims:
            dp_world *= mesh.get_dim_size(d)
        self.dp_comm = Communicator(mesh.get_dim_group(dp_dims) if multi and dp_dims and dp_world > 1 else None, self.device,
                                    single=dp_world == 1)
        # ---- model chunks of this pipeline rank
        self.layer_plan = split_layers(cfg.num_hidden_layers, self.pp_size, self.vpp)
        self.chunks: List[DecoderModel] = []
        fused_tp = make_fused_tp(self.tp_comm, self.device, bool(mesh.sequence_parallel), comm_backend) if self.tp_size > 1 else None
        # expert tensor parallelism: 1 (experts whole on a rank, the default here) or the tensor-parallel degree
        self.etp_size = int(mesh.etp_size or 1) if (cfg.is_moe and self.tp_size > 1) else 1
        if self.etp_size not in (1, self.tp_size):
            raise ValueError(f'etp_size={self.etp_size}: experts are either whole (1) or split over the whole tensor-parallel group ({self.tp_size})')
        if self.etp_size > 1:
            if cfg.moe_intermediate_size % self.tp_size:
                raise ValueError('moe_intermediate_size must divide over the tensor-parallel group')
            cfg.expert_tensor_parallel = True   # read by the sharding rules (models/bridge.py::tp_rule)
        load_dir = model_id if model_id and os.path.isdir(str(model_id)) else None
        for c, (lo, hi) in enumerate(self.layer_plan[self.pp_rank]):
            first = self.pp_rank == 0 and c == 0
            last = self.pp_rank == self.pp_size - 1 and c == self.vpp - 1
            need_embed = first or (last and cfg.tie_word_embeddings)
            m = build_model(cfg, device=self.device, dtype=self.compute_dtype, seed=seed, init=load_dir is None, layer_range=(lo, hi),
                            has_embed=need_embed, has_head=last)
            # parameter names carry GLOBAL layer indices so that seeds / bridge names agree across layouts
            self._rename_for_init(m, lo, seed, load_dir)
            apply_tensor_parallel(m, cfg, self.tp_comm, mesh.sequence_parallel, fused_tp)
            if self.cp_size > 1:
                from ..parallel.context import apply_context_parallel
                apply_context_parallel(m, mesh)  # zig-zag shards, keys / values gathered per layer (``parallel/context.py``)
            self.chunks.append(m)
        self.sequence_parallel = bool(mesh.sequence_parallel and self.tp_size > 1)
        self._n_moe_layers = max(1, cfg.num_hidden_layers if cfg.is_moe else 1)
        self.ep_comm, self.ep_rank, self.ep_size = None, 0, 1
        if (mesh.ep_size or 1) > 1 and cfg.is_moe:
            self._apply_expert_parallel(mesh, comm_backend)
        self.cp_comm = None
        if self.cp_size > 1:
            from ..parallel.context import cp_group_for
            self.cp_comm = Communicator(cp_group_for(mesh), self.device)
        self.runner = PipelineRunner(self.pp_group, self.pp_rank, self.pp_size, self.vpp, self.compute_dtype, self.device)
        self.optimizer_groups: Dict[str, OptimizerGroup] = {'': OptimizerGroup(adapter_name='')}
        self._state: Dict[str, Dict[str, torch.Tensor]] = {}
        self._pending_scale = 1.0

    # ------------------------------------------------------------ expert parallel
    def _apply_expert_parallel(self, mesh: DeviceMesh, backend: str) -> None:
        """Experts split over ``ep`` consecutive data-parallel ranks (same tp / pp / cp coordinates); attention and router
        stay as they are (reference ``megatron/strategy/megatron.py:90-107``: ``expert_model_parallel_size``).  A rank's expert tensors are shared with every rank
        that holds the same experts of the same layers: the other data-parallel blocks, the context-parallel peers and,
        under sequence parallelism, the tensor-parallel peers (they route different tokens); gradients are summed over
        exactly that set.  With expert tensor parallelism the tensor-parallel peers hold different slices of the same
        experts instead: they are not in that set, and every rank of a tensor-parallel group sends the group's whole token
        set to its own expert-parallel line."""
        from ..parallel.expert import ExpertParallel, shard_experts
        ep = int(mesh.ep_size)
        if self.tp_size > 1 and not self.sequence_parallel:
            raise NotImplementedError('expert parallel with tensor parallel needs sequence_parallel=True (each tp rank then routes its own tokens)')
        names = list(mesh.mesh_dim_names)
        data_dims = [d for d in ('dp', 'fsdp') if d in names]
        coords = {r: mesh.coord_of(r) for r in mesh.mesh.reshape(-1).tolist()}

        def key_of(r, dims):
            return tuple(coords[r][names.index(d)] for d in dims if d in names)

        me = dist.get_rank()
        lines: Dict[tuple, List[int]] = {}
        for r in sorted(coords):
            lines.setdefault(key_of(r, [d for d in names if d not in data_dims]), []).append(r)
        ep_group, my_pos, pos_of = None, 0, {}
        for other in sorted(lines):
            line = sorted(lines[other], key=lambda r: key_of(r, data_dims))
            if len(line) % ep != 0:
                raise ValueError(f'ep_size={ep} does not divide the {len(line)} data-parallel ranks')
            for i in range(0, len(line), ep):
                block = line[i:i + ep]
                g = dist.new_group(ranks=block)
                for j, r in enumerate(block):
                    pos_of[r] = j
                if me in block:
                    ep_group, my_pos = g, block.index(me)
        rep_group = None
        pp_i = names.index('pp') if 'pp' in names else None
        tp_i = names.index('tp') if ('tp' in names and self.etp_size > 1) else None
        for stage in sorted({coords[r][pp_i] if pp_i is not None else 0 for r in coords}):
            for slice_ in sorted({coords[r][tp_i] if tp_i is not None else 0 for r in coords}):
                for j in range(ep):
                    members = sorted(r for r in coords if pos_of[r] == j and (coords[r][pp_i] if pp_i is not None else 0) == stage
                                     and (coords[r][tp_i] if tp_i is not None else 0) == slice_)
                    g = dist.new_group(ranks=members)
                    if me in members:
                        rep_group = g if len(members) > 1 else None
        self.ep_comm = Communicator(ep_group, self.device)
        strat = None
        if self.device.type == 'cuda' and backend in ('auto', 'symm'):
            try:
                from ..parallel.expert_symm import SymmExpertParallel
                from ..parallel.symm import SymmCommunicator
                strat = SymmExpertParallel(SymmCommunicator(ep_group, self.device), self.config.num_experts)
            except Exception:
                if backend == 'symm':
                    raise
        if strat is None:
            strat = ExpertParallel(self.ep_comm, self.config.num_experts)
        rep_comm = Communicator(rep_group, self.device) if rep_group is not None else None
        for m in self.chunks:
            shard_experts(m, strat, my_pos, rep_comm)
        self.ep_rank, self.ep_size = my_pos, ep

    # ------------------------------------------------------------ weights
    def _rename_for_init(self, m: DecoderModel, lo: int, seed: int, load_dir: Optional[str]) -> None:
        """Re-initialise (or load) with global layer names: ``layers.<local>`` → ``layers.<lo+local>``."""
        from ..utils.seed import stable_seed
        loader = SafetensorLazyLoader(load_dir) if load_dir else None
        with torch.no_grad():
            for name, p in m.named_parameters():
                g = self._global_name(name, lo)
                if loader is not None:
                    t = hf_to_internal(g, self.config, loader.get)       # a head the file does not carry comes from the embedding
                    p.copy_(t.to(p.dtype))
                elif p.dim() > 1:
                    # the same rule as ``DecoderModel.init_weights``: one stream per (global) parameter name, drawn on the
                    # host for small tensors and on the device for large ones, so every layout starts from the same values
                    if p.numel() <= 2**24 or p.device.type == 'cpu':
                        gen = torch.Generator(device='cpu').manual_seed(stable_seed(seed, g))
                        p.copy_(torch.randn(p.shape, generator=gen, dtype=torch.float32).mul_(self.config.initializer_range))
                    else:
                        gd = torch.Generator(device=p.device).manual_seed(stable_seed(seed, g))
                        p.normal_(0.0, self.config.initializer_range, generator=gd)
        m._layer_offset = lo

    @staticmethod
    def _global_name(name: str, lo: int) -> str:
        if name.startswith('layers.'):
            parts = name.split('.')
            parts[1] = str(int(parts[1]) + lo)
            return '.'.join(parts)
        return name

    def named_parameters(self):
        for m in self.chunks:
            for n, p in m.named_parameters():
                yield self._global_name(n, m._layer_offset), p

    def _group(self, adapter_name=None) -> OptimizerGroup:
        return self.optimizer_groups['']

    # ------------------------------------------------------------ forward
    def _micro_batches(self, inputs, micro_batch_size: Optional[int]):
        og = self._group()
        if isinstance(inputs, dict):
            inputs = [inputs]
        feats = list(inputs)
        if feats and 'input_ids' not in feats[0]:
            feats = og.template.batch_encode(feats)
        proc = og.processor or InputProcessor(pad_token_id=self.config.pad_token_id or 0)
        og.processor = proc
        proc.micro_batch_size = micro_batch_size or 1
        proc.sp_size = 1
        proc.cp_size, proc.cp_rank = self.cp_size, (self.device_mesh.cp_rank or 0)
        items = proc.normalize(feats)
        # a rank's share of the row (1/cp of every sequence, in two zig-zag halves) must divide over the tp group
        mult = (self.tp_size if self.sequence_parallel else 1) * (2 * self.cp_size if self.cp_size > 1 else 1)
        mbs = []
        for g in proc.split_micro_batches(items):
            mbs.append(proc._pack(g, pad_multiple=mult, split=self.cp_size > 1))
        return feats, mbs

    def _forward_chunk(self, mbs, og, loss_kwargs, results, aux_report: Optional[List[float]] = None):
        aux_report = aux_report if aux_report is not None else []

        def run(chunk: int, micro: int, x: Optional[torch.Tensor]) -> torch.Tensor:
            m = self.chunks[chunk]
            mb = mbs[micro].to(self.device)
            batch = PackedBatch(mb.input_ids, mb.position_ids, mb.cu_seqlens, mb.max_seqlen, mb.labels, seq_lens=list(mb.seq_lens))
            if x is None:
                h = m.embed(batch)
                if m.tp is not None and not m.tp.sp:
                    pass
            else:
                h = x
            cos, sin = ops.rope_tables(batch.position_ids, self.config.rotary_dim, self.config.rope_theta, self.config.rope_scaling)
            if self.config.rope_local_theta:
                batch.rope_local = ops.rope_tables(batch.position_ids, self.config.rotary_dim, self.config.rope_local_theta, None)
            if self.recompute is not None and torch.is_grad_enabled():
                from torch.utils.checkpoint import checkpoint
                for layer in m.layers:
                    h = checkpoint(layer, h, cos, sin, batch, use_reentrant=False)
            else:
                for layer in m.layers:
                    h = layer(h, cos, sin, batch)
            # router load-balance loss of this chunk's layers: per token of the micro-batch it weighs
            # coef / (number of mixture layers) like on the sharded backend; its gradient enters with the chunk's backward
            aux_term = None
            if self.config.is_moe and self.config.router_aux_loss_coef > 0 and torch.is_grad_enabled():
                auxes = [l.mlp.last_aux for l in m.layers if getattr(l, 'is_moe', False) and l.mlp.last_aux is not None]
                for l in m.layers:
                    if getattr(l, 'is_moe', False):
                        l.mlp.last_aux = None
                if auxes:
                    nt_mb = float((mb.labels != -100).sum()) or 1.0
                    # sequence-parallel peers each hold 1/tp of these tokens; context-parallel peers count their own labels
                    share = self.tp_size if self.sequence_parallel else 1
                    aux_term = torch.stack(auxes).sum() * (self.config.router_aux_loss_coef * nt_mb / (self._n_moe_layers * share))
                    aux_report.append(float(aux_term.detach()))
            if not m.has_head:
                return h if aux_term is None else _AttachAux.apply(h, aux_term)
            h = m.norm(h)
            logps, _ = m.token_logprobs(h, mb.labels)
            labels = mb.labels
            if self.cp_comm is not None:  # whole sequences for the loss on every context-parallel rank
                from ..parallel.context import gather_zigzag_rows
                logps = gather_zigzag_rows(logps, self.cp_comm, mb.seq_lens, 0, True)
                labels = gather_zigzag_rows(labels, self.cp_comm, mb.seq_lens, -100, False)
            out = {'logps': InputProcessor.unpack_packed_sequences(logps, mb.seq_lens, 0),
                   'labels': InputProcessor.unpack_packed_sequences(labels, mb.seq_lens, -100)}
            res = og.loss_instance({'labels': out['labels']}, out, **loss_kwargs(micro))
            loss = res['loss'] if isinstance(res, dict) else res
            nt = float(res.get('num_tokens', 0) or 0) if isinstance(res, dict) else 0.0
            nt /= self.cp_size                      # every context-parallel peer reports the same rows
            results.append({'logps': out['logps'].detach(), 'labels': out['labels'], 'num_tokens': nt, 'loss': float(loss.detach()) / self.cp_size})
            # the reported loss stays the language-model loss (as on the sharded backend); the term only adds its gradient
            return loss if aux_term is None else _AttachAux.apply(loss, aux_term)

        return run

    def _hidden_shape(self, mbs):
        def shape(micro: int):
            t = int(mbs[micro].input_ids.numel())
            if self.sequence_parallel:
                t //= self.tp_size
            return (t, self.config.hidden_size)
        return shape

    @remote_function(dispatch='slice_dp', collect=collect_tensor_dict)
    def forward_backward(self, *, inputs, micro_batch_size: Optional[int] = 1, adapter_name: Optional[str] = None, **kwargs):
        og = self._group()
        feats, mbs = self._micro_batches(inputs, micro_batch_size)
        n = len(feats)
        per = micro_batch_size or 1

        def loss_kwargs(micro: int):
            from .native import TransformersModel
            return TransformersModel._slice_kwargs(kwargs, micro * per, min((micro + 1) * per, n), n)

        results: List[Dict[str, Any]] = []
        aux_report: List[float] = []
        self.runner.run(len(mbs), self._forward_chunk(mbs, og, loss_kwargs, results, aux_report), self._hidden_shape(mbs))
        # loss / token count live on the last stage: share them with the whole pipeline group
        stats = torch.zeros(3, dtype=torch.float64, device=self.device if self.device.type == 'cuda' else 'cpu')
        if results:
            stats[0] = sum(r['loss'] for r in results)
            stats[1] = sum(r['num_tokens'] for r in results)
            stats[2] = len(results)
        if self.pp_size > 1:
            dist.all_reduce(stats, group=self.pp_group)  # only last-stage ranks contribute non-zeros
        loss_sum, tokens, calls = (float(x) for x in stats)
        og.train_status.num_tokens += tokens if tokens > 0 else calls
        og.cur_step += 1
        og.grad_ready = True
        og.consumed_train_samples += n * max(self.dp_comm.world_size, 1)
        out: Dict[str, Any] = {'loss': loss_sum / tokens if tokens > 0 else loss_sum / max(calls, 1), 'num_tokens': tokens}
        if results:
            merged = collect_tensor_dict([{'logps': r['logps'], 'labels': r['labels']} for r in results])
            out.update(merged)
        return out

    @remote_function(dispatch='slice_dp', collect=collect_tensor_dict)
    def forward_only(self, *, inputs, micro_batch_size: Optional[int] = 1, **kwargs):
        with torch.no_grad():
            og = self._group()
            feats, mbs = self._micro_batches(inputs, micro_batch_size)
            results: List[Dict[str, Any]] = []
            fc = self._forward_chunk(mbs, og, lambda m: {}, results)
            # forward-only pipeline: every micro-batch flows through all stages in order
            P, V = self.pp_size, self.vpp
            for micro in range(len(mbs)):
                for chunk in range(V):
                    x = None
                    if not self.runner.is_first(chunk):
                        x = self.runner._recv(self._hidden_shape(mbs)(micro), self.runner.prev, 7_000_000 + chunk * 1024 + micro)
                    y = fc(chunk, micro, x)
                    if not self.runner.is_last(chunk):
                        nxt_chunk = chunk if self.pp_rank < P - 1 else chunk + 1
                        self.runner._send(y, self.runner.next, 7_000_000 + nxt_chunk * 1024 + micro)
                        self.runner._flush()
            for h in self.runner._pending:
                h.wait()
            self.runner._pending.clear()
        return collect_tensor_dict([{'logps': r['logps'], 'labels': r['labels']} for r in results]) if results else {}

    forward = forward_only

    def calculate_loss(self, **kwargs):
        raise NotImplementedError('the pipeline backend fuses loss into forward_backward')

    def backward(self, **kwargs):
        raise NotImplementedError('the pipeline backend fuses backward into forward_backward')

    # ------------------------------------------------------------ optimiser
    def _params(self) -> List[Tuple[str, torch.nn.Parameter]]:
        return [(n, p) for n, p in self.named_parameters() if p.requires_grad]

    @remote_function(collect='first')
    def clip_grad_norm(self, max_grad_norm: float = 1.0, norm_type=2, **kwargs) -> float:
        og = self._group()
        # 1. data-parallel gradient sum; sequence-parallel: norm weights saw different tokens on each tp rank
        for n, p in self._params():
            if p.grad is None:
                continue
            if getattr(p, '_ep_local', False):  # experts: summed over the ranks that hold the same experts, nobody else
                rc = getattr(p, '_ep_replica_comm', None)
                if rc is not None and rc.world_size > 1:
                    rc.all_reduce(p.grad)
                continue
            if self.dp_comm.world_size > 1:
                self.dp_comm.all_reduce(p.grad)
            if self.tp_size > 1 and tp_rule(n, self.config) is None and (
                    self.sequence_parallel or n.endswith(('self_attn.q_norm.weight', 'self_attn.k_norm.weight'))):
                # replicated tensors whose gradient is a partial sum on each tp rank: under sequence parallelism all of
                # them (every rank saw different tokens); always the per-head q / k norm weights (every rank applied them
                # to its own heads)
                self.tp_comm.all_reduce(p.grad)
        denom = self.dp_comm.all_reduce_scalar(og.train_status.num_tokens, 'sum') or 1.0
        # 2. global norm: tp-sharded tensors are disjoint (sum over tp), replicated ones counted once; sum over pp
        sq = torch.zeros((), dtype=torch.float32, device=self.device)
        sq_ep = torch.zeros((), dtype=torch.float32, device=self.device)
        tied_dup = self.config.tie_word_embeddings and self.pp_size > 1 and self.pp_rank == self.pp_size - 1
        for n, p in self._params():
            if p.grad is None or (tied_dup and n == 'embed_tokens.weight'):
                continue
            s = ops.sumsq(p.grad)
            if self.tp_size > 1 and tp_rule(n, self.config) is None:
                s = s / self.tp_size
            if getattr(p, '_ep_local', False):
                sq_ep = sq_ep + s
            else:
                sq = sq + s
        if self.ep_comm is not None:  # each EP rank holds different experts: their squared norms add up over the group
            sq_ep = sq_ep.reshape(1)
            self.ep_comm.all_reduce(sq_ep)
            sq = sq + sq_ep[0]
        if self.tp_size > 1:
            self.tp_comm.all_reduce(sq)
        if self.pp_size > 1:
            dist.all_reduce(sq, group=self.pp_group)
        norm = float(sq.sqrt()) / denom
        coef = min(1.0, max_grad_norm / (norm + 1e-6)) if max_grad_norm and max_grad_norm > 0 else 1.0
        self._pending_scale = coef / denom
        og._last_grad_norm = norm
        og.train_status.num_tokens = 0.0
        return norm

    def _sync_tied_embedding_grads(self) -> None:
        """Tied embedding/head across the first and last pipeline stage: sum the two gradients."""
        if not (self.config.tie_word_embeddings and self.pp_size > 1):
            return
        if self.pp_rank in (0, self.pp_size - 1):
            for m in self.chunks:
                if m.embed_tokens is not None and m.embed_tokens.weight.grad is not None:
                    g = m.embed_tokens.weight.grad
                    other = self.runner._globals[self.pp_size - 1 if self.pp_rank == 0 else 0]
                    buf = torch.empty_like(g)
                    ops_ = [dist.P2POp(dist.isend, g.contiguous(), other, group=self.pp_group), dist.P2POp(dist.irecv, buf, other, group=self.pp_group)]
                    for w in dist.batch_isend_irecv(ops_):
                        w.wait()
                    g.add_(buf)
                    return

    @remote_function()
    def step(self, optim_params: Optional[Dict[str, Any]] = None, **kwargs) -> None:
        og = self._group()
        if og.optimizer is None:
            self.set_optimizer('AdamW')
        if optim_params:
            for g in og.optimizer.param_groups:
                for k in ('lr', 'eps'):
                    if k in optim_params:
                        g[k] = optim_params[k]
                if 'betas' in optim_params:
                    g['betas'] = tuple(optim_params['betas'])
                if 'weight_decay' in optim_params and g['weight_decay'] > 0:
                    g['weight_decay'] = optim_params['weight_decay']
        og.optim_steps += 1
        gd = og.optimizer.param_groups[0]
        scale, self._pending_scale = self._pending_scale, 1.0
        dp, r = self.dp_comm.world_size, self.dp_comm.rank
        zero1 = self.use_distributed_optimizer and dp > 1
        for n, p in self._params():
            if p.grad is None:
                continue
            numel = p.numel()
            ep_local = bool(getattr(p, '_ep_local', False))  # differs per EP rank: never sliced over the data-parallel group
            lo, hi = (0, numel) if ep_local else self._state_range(numel)
            st = self._state.get(n)
            if st is None:
                flat = p.data.view(-1)[lo:hi]
                st = {'master': flat.float().clone(), 'exp_avg': torch.zeros(hi - lo, dtype=torch.float32, device=p.device),
                      'exp_avg_sq': torch.zeros(hi - lo, dtype=torch.float32, device=p.device)}
                self._state[n] = st
            wd = 0.0 if _no_decay(n) else gd['weight_decay']
            if hi > lo:
                ops.adamw_step(st['master'], st['exp_avg'], st['exp_avg_sq'], p.grad.contiguous().view(-1)[lo:hi], p.data.view(-1)[lo:hi],
                               gd['lr'], gd['betas'][0], gd['betas'][1], gd['eps'], wd, og.optim_steps, scale)
            if zero1 and not ep_local:
                # every rank updated its slice of the parameter; the slices are exchanged so all ranks hold the whole tensor
                chunk = -(-numel // dp)
                mine = torch.zeros(chunk, dtype=p.dtype, device=p.device)
                mine[:hi - lo].copy_(p.data.view(-1)[lo:hi])
                full = torch.empty(chunk * dp, dtype=p.dtype, device=p.device)
                dist.all_gather_into_tensor(full, mine, group=self.dp_comm.group)
                p.data.view(-1).copy_(full[:numel])
        og.grad_ready = False

    def _state_range(self, numel: int) -> Tuple[int, int]:
        """Slice of a flattened parameter whose optimizer state this rank keeps: the whole tensor, or one of ``dp``
        contiguous chunks under the distributed optimizer."""
        dp, r = self.dp_comm.world_size, self.dp_comm.rank
        if not (self.use_distributed_optimizer and dp > 1):
            return 0, numel
        chunk = -(-numel // dp)
        return min(r * chunk, numel), min((r + 1) * chunk, numel)

    @remote_function()
    def zero_grad(self, **kwargs) -> None:
        for _, p in self._params():
            p.grad = None

    @remote_function()
    def lr_step(self, **kwargs) -> None:
        og = self._group()
        if og.lr_scheduler is not None:
            og.lr_scheduler.step()

    @remote_function(collect='first')
    def clip_grad_and_step(self, max_grad_norm: float = 1.0, norm_type=2, **kwargs):
        self._sync_tied_embedding_grads()
        norm = self.clip_grad_norm(max_grad_norm, norm_type)
        self.step(**kwargs)
        self.zero_grad()
        self.lr_step()
        return norm

    @remote_function()
    def set_loss(self, loss_cls, **kwargs) -> None:
        if isinstance(loss_cls, str):
            loss_cls = torch_loss_mapping[loss_cls]
        self._group().set_loss(loss_cls(**kwargs) if isinstance(loss_cls, type) else loss_cls)

    @remote_function()
    def set_optimizer(self, optimizer_cls='AdamW', **kwargs) -> None:
        og = self._group()
        h = AdamHyper(lr=kwargs.get('lr', 1e-5), betas=tuple(kwargs.get('betas', (0.9, 0.999))), eps=kwargs.get('eps', 1e-8),
                      weight_decay=kwargs.get('weight_decay', 0.01))
        og.hyper = h
        names = [n for n, _ in self._params()]
        og.optimizer = EngineOptimizer(h, [n for n in names if not _no_decay(n)], [n for n in names if _no_decay(n)])

    @remote_function()
    def set_lr_scheduler(self, scheduler_cls, **kwargs) -> None:
        og = self._group()
        if og.optimizer is None:
            self.set_optimizer('AdamW')
        if isinstance(scheduler_cls, str):
            from ..module.scheduler import resolve_scheduler
            scheduler_cls = resolve_scheduler(scheduler_cls)
        og.lr_scheduler = scheduler_cls(og.optimizer, **kwargs) if isinstance(scheduler_cls, type) else scheduler_cls

    @remote_function()
    def set_template(self, template_cls, **kwargs) -> None:
        from ..template import Template, template_mapping
        if isinstance(template_cls, str):
            template_cls = template_mapping.get(template_cls, Template)
        self._group().template = template_cls(**kwargs) if isinstance(template_cls, type) else template_cls

    @remote_function()
    def set_processor(self, processor_cls, **kwargs) -> None:
        self._group().processor = processor_cls(**kwargs) if isinstance(processor_cls, type) else processor_cls

    def apply_patch(self, patch_cls, **kwargs) -> None:
        from ..patch import apply_patch
        apply_patch(self, patch_cls, **kwargs)

    def add_metric(self, metric_cls, is_training=None, **kwargs) -> None:
        from ..metric import metric_mapping
        m = metric_mapping[metric_cls](**kwargs) if isinstance(metric_cls, str) else metric_cls
        self._group().train_status.metrics.append(m)

    def calculate_metric(self, is_training: bool = True, **kwargs) -> Dict[str, Any]:
        out: Dict[str, Any] = {}
        for m in self._group().status(is_training).metrics:
            out.update(m.calculate())
        return out

    def add_adapter_to_model(self, adapter_name: str, config_or_dir, **kwargs) -> None:
        raise NotImplementedError('use MultiLoraMegatronModel for adapters')

    def get_train_configs(self, **kwargs) -> str:
        n = sum(p.numel() for _, p in self._params())
        return (f'model: {self.model_id or self.config.model_type}; this rank holds {n:,} parameters\n'
                f'layout: tp={self.tp_size} pp={self.pp_size} vpp={self.vpp} dp={self.dp_comm.world_size} '
                f'sequence_parallel={self.sequence_parallel}; layers of this rank: {self.layer_plan[self.pp_rank]}')

    # ---------------------------------------------------------- save / load
    def _gather_full(self, name: str, p: torch.Tensor) -> torch.Tensor:
        t = p.detach()
        if getattr(p, '_ep_local', False) and self.ep_comm is not None:  # all experts, in expert order
            parts = [torch.empty_like(t) for _ in range(self.ep_comm.world_size)]
            dist.all_gather(parts, t.contiguous(), group=self.ep_comm.group)
            t = torch.cat(parts, 0)
        if self.tp_size == 1 or tp_rule(name, self.config) is None:
            return t
        parts = [torch.empty_like(t) for _ in range(self.tp_size)]
        dist.all_gather(parts, t.contiguous(), group=self.tp_comm.group)
        return tp_unshard(name, parts, self.config)

    @remote_function(collect='first')
    def get_state_dict(self, **kwargs) -> Dict[str, torch.Tensor]:
        """HF-named tensors held by this pipeline stage (TP shards gathered)."""
        out = {}
        for n, p in self.named_parameters():
            if n == 'embed_tokens.weight' and self.config.tie_word_embeddings and self.pp_rank != 0:
                continue
            full = self._gather_full(n, p)
            for hk, hv in internal_to_hf(n, full, self.config):
                out[hk] = hv
        return out

    def get_hf_state_dict(self):
        yield from self.get_state_dict().items()

    @remote_function(collect='first')
    def save(self, name: Optional[str] = None, output_dir: Optional[str] = None, **kwargs) -> str:
        """Every pipeline stage writes its own shard files (``model-ppXX-….safetensors``); rank 0 merges the
        indices so the directory is a standard HF checkpoint."""
        path = os.path.join(output_dir or './output', name) if name else (output_dir or './output')
        sd = self.get_state_dict()
        writer = (self.tp_rank == 0) and (self.dp_comm.rank == 0)
        os.makedirs(path, exist_ok=True)
        if writer:
            from safetensors.torch import save_file
            fn = f'model-pp{self.pp_rank:02d}-of-{self.pp_size:02d}.safetensors'
            save_file({k: v.detach().cpu().contiguous() for k, v in sd.items()}, os.path.join(path, fn), metadata={'format': 'pt'})
            with open(os.path.join(path, f'.index-pp{self.pp_rank:02d}.json'), 'w') as f:
                json.dump({k: fn for k in sd}, f)
        if dist.is_available() and dist.is_initialized():
            dist.barrier()
        if Platform.is_master():
            weight_map: Dict[str, str] = {}
            for r in range(self.pp_size):
                pth = os.path.join(path, f'.index-pp{r:02d}.json')
                with open(pth) as f:
                    weight_map.update(json.load(f))
                os.remove(pth)
            with open(os.path.join(path, 'model.safetensors.index.json'), 'w') as f:
                json.dump({'metadata': {}, 'weight_map': weight_map}, f)
            self.config.save_pretrained(path)
        if kwargs.get('save_optimizer'):
            self._save_training_state(path)
        if dist.is_available() and dist.is_initialized():
            dist.barrier()
        return path

    @remote_function()
    def load(self, name: Optional[str] = None, output_dir: Optional[str] = None, **kwargs) -> None:
        path = os.path.join(output_dir or './output', name) if name else (output_dir or './output')
        loader = SafetensorLazyLoader(path)
        with torch.no_grad():
            for n, p in self.named_parameters():
                full = hf_to_internal(n, self.config, loader.get)
                if getattr(p, '_ep_local', False) and self.ep_comm is not None:
                    el = p.shape[0]
                    full = full[self.ep_rank * el:(self.ep_rank + 1) * el]
                p.copy_(tp_shard(n, full, self.config, self.tp_rank, self.tp_size).to(p.device, p.dtype))
                st = self._state.get(n)
                if st is not None:
                    lo, hi = (0, p.numel()) if getattr(p, '_ep_local', False) else self._state_range(p.numel())
                    st['master'].copy_(p.data.view(-1)[lo:hi].float())
        if kwargs.get('load_optimizer'):
            self._load_training_state(path)

    # Training state.  Weights go through the bridge into one HF checkpoint; what the optimizer holds is layout-specific
    # (a tensor-parallel shard of a pipeline stage, possibly one data-parallel slice of it), so every rank writes its
    # own file ``optimizer_tpXX_ppXX_dpXX.pt`` (the reference's megatron-core distributed checkpoint does the same,
    # ``megatron/megatron.py:1078-1243``).  A run of the same layout reads its own file back; a run of another tensor /
    # pipeline / data-parallel layout reassembles every tensor it needs from the files that hold its pieces
    # (``_load_resharded_state``).
    def _rank_tag(self) -> str:
        return f'tp{self.tp_rank:02d}_pp{self.pp_rank:02d}_dp{self.dp_comm.rank:02d}'

    def _layout(self) -> Dict[str, Any]:
        return {'tp': self.tp_size, 'pp': self.pp_size, 'vpp': self.vpp, 'dp': self.dp_comm.world_size,
                'distributed_optimizer': bool(self.use_distributed_optimizer and self.dp_comm.world_size > 1),
                'ep': int(getattr(self, 'ep_size', 1) or 1), 'etp': int(getattr(self, 'etp_size', 1) or 1)}

    def _save_training_state(self, path: str) -> None:
        og = self._group()
        os.makedirs(path, exist_ok=True)
        shapes = {n: tuple(p.shape) for n, p in self._params()}
        state = {'layout': self._layout(), 'ep_rank': int(getattr(self, 'ep_rank', 0) or 0), 'shapes': {n: shapes[n] for n in self._state if n in shapes},
                 'optim_steps': og.optim_steps, 'hyper': og.optimizer.state_dict()['param_groups'] if og.optimizer else None,
                 'params': {n: {k: v.detach().cpu() for k, v in st.items()} for n, st in self._state.items()}}
        torch.save(state, os.path.join(path, f'optimizer_{self._rank_tag()}.pt'))
        torch.save(Platform.get_rng_state(), os.path.join(path, f'rng_state_{self._rank_tag()}.pt'))
        if Platform.is_master():
            if og.lr_scheduler is not None:
                torch.save(og.lr_scheduler.state_dict(), os.path.join(path, 'scheduler.pt'))
            with open(os.path.join(path, 'trainer_state.json'), 'w') as f:
                json.dump({'checkpoint_version': 1, 'cur_step': og.cur_step, 'gradient_accumulation_steps': og.gradient_accumulation_steps,
                           'consumed_train_samples': og.consumed_train_samples, 'optim_steps': og.optim_steps}, f)

    def _apply_saved_hyper(self, state: Dict[str, Any]) -> None:
        og = self._group()
        og.optim_steps = int(state.get('optim_steps', 0))
        if og.optimizer is None:
            self.set_optimizer('AdamW')
        if state.get('hyper'):
            for g, sv in zip(og.optimizer.param_groups, state['hyper']):
                for k in ('lr', 'betas', 'eps', 'weight_decay'):
                    if k in sv:
                        g[k] = sv[k] if k != 'betas' else tuple(sv[k])

    def _load_resharded_state(self, path: str, files: Dict[Tuple[int, int, int], str]) -> None:
        """Optimizer state written under another tensor / pipeline / data-parallel layout.  For every parameter this rank
        holds: the saved data-parallel slices of each saved tensor-parallel rank are joined into that rank's shard, the
        shards into the full tensor (the same rule that splits weights, ``models/bridge.py::tp_unshard``), and the full
        tensor is cut again for this rank's shard and data-parallel slice.  Expert tensors written under expert parallelism
        are put together from the saved expert-parallel ranks in expert order first.  Files are memory-mapped, so only the
        tensors a rank needs are read."""
        wanted = dict(self._params())
        found: Dict[str, Dict[Tuple[int, int], Dict[str, torch.Tensor]]] = {}
        found_ep: Dict[str, Dict[Tuple[int, int], Dict[str, torch.Tensor]]] = {}     # expert tensors: (saved ep rank, tp rank) → state
        shapes: Dict[str, Dict[int, Tuple[int, ...]]] = {}
        first = None
        for (t, pstage, d), fn in sorted(files.items(), key=lambda kv: (kv[0][1], kv[0][0], kv[0][2])):
            st = torch.load(fn, map_location='cpu', weights_only=True, mmap=True)
            if first is None:
                first = st
            if 'shapes' not in st:
                raise ValueError(f'{fn} has no shard shapes: it was written by a version that could only resume into the same layout')
            if st.get('layout', {}).get('ep', 1) != 1 and 'ep_rank' not in st:
                raise ValueError(f'{fn} does not say which experts it holds: it loads only into the layout that wrote it')
            for n, tensors in st['params'].items():
                if n not in wanted:
                    continue
                if st['layout'].get('ep', 1) != 1 and n.endswith(('mlp.experts.gate_up_proj', 'mlp.experts.down_proj')):   # written per expert-parallel rank
                    found_ep.setdefault(n, {}).setdefault((int(st.get('ep_rank', 0)), t), tensors)     # replicas hold the same values
                    shapes.setdefault(n, {})[t] = tuple(st['shapes'][n])
                elif (t, d) not in found.setdefault(n, {}):      # a tied embedding sits on two stages: the first one wins
                    found[n][(t, d)] = tensors
                    shapes.setdefault(n, {})[t] = tuple(st['shapes'][n])
        if first is None:
            raise FileNotFoundError(f'no optimizer_tp*_pp*_dp*.pt files under {path}')
        self._apply_saved_hyper(first)
        sharded_dp = bool(first['layout'].get('distributed_optimizer'))
        state: Dict[str, Dict[str, torch.Tensor]] = {}
        for n, p in wanted.items():
            entry = {}
            if n in found_ep:
                # expert tensors are never sliced by the distributed optimizer: every saved expert-parallel rank holds whole
                # tensors of its own experts.  All experts are put together in expert order, then cut for this rank.
                eps, tps = sorted({j for j, _ in found_ep[n]}), sorted({t for _, t in found_ep[n]})
                for key in ('master', 'exp_avg', 'exp_avg_sq'):
                    blocks = [tp_unshard(n, [found_ep[n][(j, t)][key].reshape(shapes[n][t]) for t in tps], self.config) for j in eps]
                    full = torch.cat(blocks, 0)
                    if getattr(p, '_ep_local', False) and self.ep_size > 1:
                        el = full.shape[0] // self.ep_size
                        full = full[self.ep_rank * el:(self.ep_rank + 1) * el]
                        mine = tp_shard(n, full, self.config, self.tp_rank, self.tp_size).reshape(-1)
                    else:
                        lo, hi = self._state_range(p.numel())
                        mine = tp_shard(n, full, self.config, self.tp_rank, self.tp_size).reshape(-1)[lo:hi]
                    entry[key] = mine.to(self.device, torch.float32).clone()
                state[n] = entry
                continue
            if n not in found:
                raise KeyError(f'optimizer state of {n} is not in the checkpoint under {path}')
            tps = sorted({t for t, _ in found[n]})
            ep_local = bool(getattr(p, '_ep_local', False)) and self.ep_size > 1
            lo, hi = (0, p.numel()) if ep_local else self._state_range(p.numel())
            for key in ('master', 'exp_avg', 'exp_avg_sq'):
                shards = []
                for t in tps:
                    ds = sorted(d for tt, d in found[n] if tt == t)
                    flat = torch.cat([found[n][(t, d)][key] for d in ds]) if sharded_dp else found[n][(t, ds[0])][key]
                    shape = shapes[n][t]
                    shards.append(flat[:math.prod(shape)].reshape(shape))
                full = tp_unshard(n, shards, self.config)
                if ep_local:      # written with whole experts everywhere, read into an expert-parallel layout
                    el = full.shape[0] // self.ep_size
                    full = full[self.ep_rank * el:(self.ep_rank + 1) * el]
                mine = tp_shard(n, full, self.config, self.tp_rank, self.tp_size).reshape(-1)[lo:hi]
                entry[key] = mine.to(self.device, torch.float32).clone()
            state[n] = entry
        self._state = state

    def _load_training_state(self, path: str) -> Dict[str, Any]:
        og = self._group()
        f = os.path.join(path, f'optimizer_{self._rank_tag()}.pt')
        same_layout = False
        if os.path.isfile(f):
            state = torch.load(f, map_location='cpu', weights_only=True)
            want = self._layout()
            same_layout = all(state.get('layout', {}).get(k, want[k] if k in ('ep', 'etp') else None) == v for k, v in want.items())
            if same_layout:
                self._apply_saved_hyper(state)
                self._state = {n: {k: v.to(self.device) for k, v in st.items()} for n, st in state['params'].items()}
        if not same_layout:
            import glob
            files = {}
            for fn in glob.glob(os.path.join(path, 'optimizer_tp*_pp*_dp*.pt')):
                m = re.match(r'optimizer_tp(\d+)_pp(\d+)_dp(\d+)\.pt$', os.path.basename(fn))
                if m:
                    files[(int(m.group(1)), int(m.group(2)), int(m.group(3)))] = fn
            if files:
                self._load_resharded_state(path, files)
        sched = os.path.join(path, 'scheduler.pt')
        if os.path.isfile(sched) and og.lr_scheduler is not None:
            og.lr_scheduler.load_state_dict(torch.load(sched, map_location='cpu', weights_only=True))
        rng = os.path.join(path, f'rng_state_{self._rank_tag()}.pt')
        if same_layout and os.path.isfile(rng):       # generator states belong to the ranks of the layout that wrote them
            Platform.set_rng_state(torch.load(rng, map_location='cpu', weights_only=True))
        info = {'cur_step': 0, 'consumed_train_samples': 0, 'gradient_accumulation_steps': og.gradient_accumulation_steps}
        ts = os.path.join(path, 'trainer_state.json')
        if os.path.isfile(ts):
            with open(ts) as fh:
                info.update(json.load(fh))
            og.cur_step, og.consumed_train_samples = info['cur_step'], info['consumed_train_samples']
            og.gradient_accumulation_steps = info['gradient_accumulation_steps']
        return info

    @remote_function(collect='first')
    def resume_from_checkpoint(self, checkpoint_dir: str, *, resume_only_model: bool = False, **kwargs) -> Dict[str, Any]:
        """Weights, then (unless ``resume_only_model``) optimizer / scheduler / RNG state and the progress counters."""
        self.load(None, checkpoint_dir)
        og = self._group()
        if resume_only_model:
            return {'cur_step': 0, 'consumed_train_samples': 0, 'gradient_accumulation_steps': og.gradient_accumulation_steps}
        info = self._load_training_state(checkpoint_dir)
        return {k: info[k] for k in ('cur_step', 'consumed_train_samples', 'gradient_accumulation_steps')}


@remote_class()
class MultiLoraMegatronModel(MegatronModel):
    """Tenants' adapters on the tensor- / pipeline-parallel backend over one frozen base (reference
    ``src/twinkle/model/megatron/multi_lora_megatron.py:34-451``).

    Every chunk of this rank carries a slot pool.  On tensor-parallel linears the pools follow the shards: ``A``
    replicated and ``B`` row-sharded on column-parallel linears, ``A`` column-sharded and ``B`` replicated on
    row-parallel ones; gradients of the replicated halves are partial sums and are all-reduced over the TP group.
    Expert pools (target-parameter LoRA on the fused expert tensors) are whole on every rank while the experts are, and
    follow the expert shards under expert tensor parallelism (``gate_up``: ``B`` rows of this rank's gate and up slices;
    ``down``: ``A`` columns of this rank's slice of the intermediate dimension); under expert parallelism a rank keeps the
    pools of its own experts, with gradients summed over the ranks that hold the same experts and all experts gathered on save.
    Each tenant has its own optimizer state (fp32 master + Adam moments of its slot slices), gradient norm, progress
    counters and scheduler (``multi_lora_megatron.py:213-291``); adapters are saved and loaded in PEFT format with the
    TP shards and pipeline stages merged into one ``adapter_model.safetensors``."""

    def __init__(self, *args, max_loras: int = 5, max_r: int = 32, max_length: int = 8192, **kwargs):
        kwargs.setdefault('use_distributed_optimizer', False)  # adapter state is small: every data-parallel rank keeps it whole
        super().__init__(*args, **kwargs)
        from .multi_lora import MultiLora
        self.max_length = max_length
        seed = kwargs.get('seed', 0)
        self.pools = [MultiLora(m, max_loras, max_r, seed=seed * 1000 + self.pp_rank * 16 + c) for c, m in enumerate(self.chunks)]
        self._sync_pools()
        self.optimizer_groups = {}
        self._tenant_state: Dict[str, Dict[str, Dict[str, torch.Tensor]]] = {}
        self._tenant_scale: Dict[str, float] = {}

    # ------------------------------------------------------------ pool plumbing
    def _pool_params(self):
        """(global parameter name, parameter, tp_mode of its module) for every pool tensor of this rank."""
        for m, pool in zip(self.chunks, self.pools):
            mods = dict(pool.modules)
            for n, p in pool.pool_parameters():
                mod_name = n.split('.lora')[0]
                yield self._global_name(n, m._layer_offset), p, getattr(mods.get(mod_name), 'tp_mode', None)

    def _expert_replicas(self):
        """Communicator over the ranks that hold the same experts as this one (None: nobody else does), when experts are
        split over an expert-parallel group; the pools on the expert tensors follow the experts."""
        if self.ep_size <= 1:
            return None
        for m in self.chunks:
            for layer in m.layers:
                if getattr(layer, 'is_moe', False):
                    return getattr(layer.mlp.experts.gate_up_proj, '_ep_replica_comm', None)
        return None

    def _is_ep_pool(self, name: str) -> bool:
        return self.ep_size > 1 and '.lora.' in name

    def _sync_pools(self) -> None:
        """Replicated pool tensors start equal: over the TP group for the replicated halves, over the data-parallel
        group for everything (each process drew its pool from its own stream position).  Pools on expert-parallel
        experts belong to this rank's experts: they are made equal only among the ranks that hold the same ones."""
        from ..parallel.tensor import lora_param_is_replicated
        rc = self._expert_replicas()
        with torch.no_grad():
            for pool in self.pools:
                init = pool._initial_A
                for n, p, mode in self._pool_params_of(pool):
                    if self._is_ep_pool(n):
                        if rc is not None and rc.world_size > 1:
                            rc.broadcast(p.data, 0)
                        if n in init:
                            init[n].copy_(p.data)
                        continue
                    if self.tp_size > 1 and lora_param_is_replicated(n, mode, self.etp_size > 1):
                        self.tp_comm.broadcast(p.data, 0)
                    if self.dp_comm.world_size > 1:
                        self.dp_comm.broadcast(p.data, 0)
                    if n in init:
                        init[n].copy_(p.data)

    def _pool_params_of(self, pool):
        mods = dict(pool.modules)
        for n, p in pool.pool_parameters():
            yield n, p, getattr(mods.get(n.split('.lora')[0]), 'tp_mode', None)

    def _tenant_slices(self, adapter_name: str):
        """(global name, pool parameter, slot, tp_mode) of every pool tensor the tenant trains on this rank."""
        out = []
        for m, pool in zip(self.chunks, self.pools):
            mods = dict(pool.modules)
            for n, p, slot in pool.tenant_slices(adapter_name):
                out.append((self._global_name(n, m._layer_offset), p, slot, getattr(mods.get(n.split('.lora')[0]), 'tp_mode', None)))
        return out

    def _group(self, adapter_name=None) -> OptimizerGroup:
        if adapter_name is None:
            adapter_name = getattr(self, '_active', None)
        if adapter_name not in self.optimizer_groups:
            raise KeyError(f'unknown adapter {adapter_name!r}; call add_adapter_to_model first')
        return self.optimizer_groups[adapter_name]

    @remote_function()
    def add_adapter_to_model(self, adapter_name: str, config_or_dir, **kwargs) -> None:
        from .multi_lora import LoraConfig
        cfg = LoraConfig.from_any(config_or_dir)
        for pool in self.pools:
            pool.acquire_lora(adapter_name, cfg)
        self.optimizer_groups[adapter_name] = OptimizerGroup(adapter_name=adapter_name, adapter_config=cfg)
        self._active = adapter_name
        if isinstance(config_or_dir, str) and os.path.isfile(os.path.join(config_or_dir, 'adapter_model.safetensors')):
            self._load_adapter(adapter_name, config_or_dir)

    @remote_function()
    def remove_adapter(self, adapter_name: str, **kwargs) -> None:
        for pool in self.pools:
            pool.release_lora(adapter_name)
        self.optimizer_groups.pop(adapter_name, None)
        self._tenant_state.pop(adapter_name, None)

    def check_length(self, inputs, max_length=None) -> None:
        limit = max_length or self.max_length
        for f in ([inputs] if isinstance(inputs, dict) else inputs):
            if len(f.get('input_ids', [])) > limit:
                raise ValueError(f'input exceeds max_length {limit}')

    # ------------------------------------------------------------ training
    def _lora_scope(self, adapter_name: str):
        from ..models.layers import LoraBatch, lora_batch
        t = self.pools[0].tenants[adapter_name]
        # one tenant per call: a single segment that covers every token of every micro-batch
        return lora_batch(LoraBatch.single(1 << 30, t.slot, t.config.r, t.config.scaling, self.device, t.target))

    @remote_function(dispatch='slice_dp', collect=collect_tensor_dict)
    def forward_backward(self, *, inputs, adapter_name: Optional[str] = None, **kwargs):
        self._active = adapter_name = adapter_name or getattr(self, '_active', None)
        self._group(adapter_name)
        with self._lora_scope(adapter_name):
            return MegatronModel.forward_backward.__wrapped__(self, inputs=inputs, adapter_name=adapter_name, **kwargs)

    @remote_function(dispatch='slice_dp', collect=collect_tensor_dict)
    def forward_only(self, *, inputs, adapter_name: Optional[str] = None, disable_lora: bool = False, **kwargs):
        self._active = adapter_name = adapter_name or getattr(self, '_active', None)
        if disable_lora:
            return MegatronModel.forward_only.__wrapped__(self, inputs=inputs, **kwargs)
        with self._lora_scope(adapter_name):
            return MegatronModel.forward_only.__wrapped__(self, inputs=inputs, **kwargs)

    forward = forward_only

    @remote_function(collect='first')
    def clip_grad_norm(self, max_grad_norm: float = 1.0, norm_type=2, adapter_name: Optional[str] = None, **kwargs) -> float:
        from ..parallel.tensor import lora_param_is_replicated
        adapter_name = adapter_name or self._active
        og = self._group(adapter_name)
        sq = torch.zeros((), dtype=torch.float32, device=self.device)
        sq_ep = torch.zeros((), dtype=torch.float32, device=self.device)
        rc = self._expert_replicas()
        for n, p, slot, mode in self._tenant_slices(adapter_name):
            if p.grad is None:
                continue
            g = p.grad[slot]
            rep = lora_param_is_replicated(n, mode, self.etp_size > 1)
            if self._is_ep_pool(n):
                # this rank's experts: gradients summed over the ranks that hold the same experts (other data blocks and, with
                # whole experts, the tensor-parallel peers — they are in that group already); under expert tensor
                # parallelism the replicated halves are partial sums over the tensor-parallel group as well
                g = g.contiguous()
                if rc is not None and rc.world_size > 1:
                    rc.all_reduce(g)
                if self.etp_size > 1 and rep:
                    self.tp_comm.all_reduce(g)
                p.grad[slot].copy_(g)
                v = ops.sumsq(g)
                sq_ep = sq_ep + (v / self.tp_size if (self.tp_size > 1 and rep) else v)
                continue
            if self.dp_comm.world_size > 1 or (self.tp_size > 1 and rep):
                g = g.contiguous()
                if self.dp_comm.world_size > 1:
                    self.dp_comm.all_reduce(g)
                if self.tp_size > 1 and rep:
                    self.tp_comm.all_reduce(g)  # the ranks' partial sums of a replicated tensor's gradient
                p.grad[slot].copy_(g)
            v = ops.sumsq(p.grad[slot].contiguous())
            sq = sq + (v / self.tp_size if (self.tp_size > 1 and rep) else v)
        if self.ep_comm is not None:       # every expert-parallel rank holds other experts: their squared norms add up
            sq_ep = sq_ep.reshape(1)
            self.ep_comm.all_reduce(sq_ep)
            sq = sq + sq_ep[0]
        if self.tp_size > 1:
            self.tp_comm.all_reduce(sq)
        if self.pp_size > 1:
            dist.all_reduce(sq, group=self.pp_group)
        denom = self.dp_comm.all_reduce_scalar(og.train_status.num_tokens, 'sum') or 1.0
        norm = float(sq.sqrt()) / denom
        coef = min(1.0, max_grad_norm / (norm + 1e-6)) if max_grad_norm and max_grad_norm > 0 else 1.0
        self._tenant_scale[adapter_name] = coef / denom
        og._last_grad_norm = norm
        og.train_status.num_tokens = 0.0
        return norm

    @remote_function()
    def step(self, adapter_name: Optional[str] = None, optim_params: Optional[Dict[str, Any]] = None, **kwargs) -> None:
        adapter_name = adapter_name or self._active
        og = self._group(adapter_name)
        if og.optimizer is None:
            self.set_optimizer('AdamW', adapter_name=adapter_name)
        gd = og.optimizer.param_groups[0]
        if optim_params:
            for k in ('lr', 'eps', 'weight_decay'):
                if k in optim_params:
                    gd[k] = optim_params[k]
            if 'betas' in optim_params:
                gd['betas'] = tuple(optim_params['betas'])
        og.optim_steps += 1
        scale = self._tenant_scale.pop(adapter_name, 1.0)
        state = self._tenant_state.setdefault(adapter_name, {})
        for n, p, slot, _ in self._tenant_slices(adapter_name):
            if p.grad is None:
                continue
            view = p.data[slot]
            st = state.get(n)
            if st is None:
                st = {'master': view.float().clone(), 'exp_avg': torch.zeros_like(view, dtype=torch.float32),
                      'exp_avg_sq': torch.zeros_like(view, dtype=torch.float32)}
                state[n] = st
            ops.adamw_step(st['master'].view(-1), st['exp_avg'].view(-1), st['exp_avg_sq'].view(-1), p.grad[slot].contiguous().view(-1),
                           view.view(-1), gd['lr'], gd['betas'][0], gd['betas'][1], gd['eps'], gd['weight_decay'], og.optim_steps, scale)
        og.grad_ready = False

    @remote_function()
    def zero_grad(self, adapter_name: Optional[str] = None, **kwargs) -> None:
        adapter_name = adapter_name or self._active
        for _, p, slot, _ in self._tenant_slices(adapter_name):
            if p.grad is not None:
                p.grad[slot].zero_()

    @remote_function()
    def lr_step(self, adapter_name: Optional[str] = None, **kwargs) -> None:
        og = self._group(adapter_name or self._active)
        if og.lr_scheduler is not None:
            og.lr_scheduler.step()

    @remote_function(collect='first')
    def clip_grad_and_step(self, max_grad_norm: float = 1.0, norm_type=2, adapter_name: Optional[str] = None, **kwargs):
        norm = self.clip_grad_norm(max_grad_norm, norm_type, adapter_name=adapter_name)
        self.step(adapter_name=adapter_name, **kwargs)
        self.zero_grad(adapter_name=adapter_name)
        self.lr_step(adapter_name=adapter_name)
        return norm

    @remote_function()
    def set_loss(self, loss_cls, adapter_name: Optional[str] = None, **kwargs) -> None:
        if isinstance(loss_cls, str):
            loss_cls = torch_loss_mapping[loss_cls]
        self._group(adapter_name).set_loss(loss_cls(**kwargs) if isinstance(loss_cls, type) else loss_cls)

    @remote_function()
    def set_optimizer(self, optimizer_cls='AdamW', adapter_name: Optional[str] = None, **kwargs) -> None:
        og = self._group(adapter_name)
        h = AdamHyper(lr=kwargs.get('lr', 1e-4), betas=tuple(kwargs.get('betas', (0.9, 0.999))), eps=kwargs.get('eps', 1e-8),
                      weight_decay=kwargs.get('weight_decay', 0.0))
        og.hyper = h
        og.optimizer = EngineOptimizer(h, [n for n, *_ in self._tenant_slices(og.adapter_name)], [])

    @remote_function()
    def set_lr_scheduler(self, scheduler_cls, adapter_name: Optional[str] = None, **kwargs) -> None:
        og = self._group(adapter_name)
        if og.optimizer is None:
            self.set_optimizer('AdamW', adapter_name=og.adapter_name)
        if isinstance(scheduler_cls, str):
            from ..module.scheduler import resolve_scheduler
            scheduler_cls = resolve_scheduler(scheduler_cls)
        og.lr_scheduler = scheduler_cls(og.optimizer, **kwargs) if isinstance(scheduler_cls, type) else scheduler_cls

    def calculate_metric(self, is_training: bool = True, adapter_name: Optional[str] = None, **kwargs) -> Dict[str, Any]:
        out: Dict[str, Any] = {}
        for m in self._group(adapter_name).status(is_training).metrics:
            out.update(m.calculate())
        return out

    def add_metric(self, metric_cls, is_training=None, adapter_name: Optional[str] = None, **kwargs) -> None:
        from ..metric import metric_mapping
        m = metric_mapping[metric_cls](**kwargs) if isinstance(metric_cls, str) else metric_cls
        self._group(adapter_name).train_status.metrics.append(m)

    # ---------------------------------------------------------- adapters on disk
    def _adapter_state_dict(self, adapter_name: str) -> Dict[str, torch.Tensor]:
        """PEFT-named tensors of the tenant for the layers of this pipeline stage, TP shards merged (collective over the
        TP group)."""
        from ..models.bridge import lora_expert_to_peft, lora_internal_to_peft
        t = self.pools[0].tenants[adapter_name]
        r = t.config.r
        sd: Dict[str, torch.Tensor] = {}
        for m, pool in zip(self.chunks, self.pools):
            for mod_name, mod in pool.modules:
                gname = self._global_name(mod_name, m._layer_offset)
                prefix = gname.rsplit('.', 1)[0] if '.' in gname else ''
                mode = getattr(mod, 'tp_mode', None)
                if not hasattr(mod, 'parts'):           # fused expert tensors
                    for which in ('gate_up', 'down'):
                        if not (t.target.matches(f'{gname}.{which}', which) or (t.config.target_parameters and any(
                                which in tpn for tpn in t.config.target_parameters))):
                            continue
                        a = mod.lora[which + '_A'][t.slot, :, :r].detach().contiguous()           # [E, r, in]
                        b = mod.lora[which + '_B'][t.slot, :, :, :r].detach().contiguous()        # [E, out, r]
                        if self.ep_size > 1:       # all experts, in expert order
                            pa, pb = [torch.empty_like(a) for _ in range(self.ep_size)], [torch.empty_like(b) for _ in range(self.ep_size)]
                            dist.all_gather(pa, a, group=self.ep_comm.group)
                            dist.all_gather(pb, b, group=self.ep_comm.group)
                            a, b = torch.cat(pa, 0), torch.cat(pb, 0)
                        if self.etp_size > 1 and which == 'gate_up':      # B: this rank's gate rows, then its up rows
                            parts = [torch.empty_like(b) for _ in range(self.tp_size)]
                            dist.all_gather(parts, b, group=self.tp_comm.group)
                            half = b.shape[1] // 2
                            b = torch.cat([x[:, :half] for x in parts] + [x[:, half:] for x in parts], 1)
                        elif self.etp_size > 1:                            # A: this rank's columns of the intermediate dimension
                            parts = [torch.empty_like(a) for _ in range(self.tp_size)]
                            dist.all_gather(parts, a, group=self.tp_comm.group)
                            a = torch.cat(parts, 2)
                        sd[lora_expert_to_peft(gname, which, 'A')] = a.clone()
                        sd[lora_expert_to_peft(gname, which, 'B')] = b.clone()
                    continue
                for pname, _ in mod.parts:
                    if not t.target.matches(f'{prefix}.{pname}' if prefix else pname, pname):
                        continue
                    a = mod.lora_A[pname][t.slot, :r].detach().contiguous()
                    b = mod.lora_B[pname][t.slot, :, :r].detach().contiguous()
                    if self.tp_size > 1 and mode == 'col':      # B rows are sharded
                        parts = [torch.empty_like(b) for _ in range(self.tp_size)]
                        dist.all_gather(parts, b, group=self.tp_comm.group)
                        b = torch.cat(parts, 0)
                    elif self.tp_size > 1 and mode == 'row':    # A columns are sharded
                        parts = [torch.empty_like(a) for _ in range(self.tp_size)]
                        dist.all_gather(parts, a, group=self.tp_comm.group)
                        a = torch.cat(parts, 1)
                    sd[lora_internal_to_peft(gname, pname, 'A')] = a.clone()
                    sd[lora_internal_to_peft(gname, pname, 'B')] = b.clone()
        return sd

    @remote_function(collect='first')
    def get_state_dict(self, adapter_name: Optional[str] = None, **kwargs) -> Dict[str, torch.Tensor]:
        if adapter_name is None:
            return MegatronModel.get_state_dict.__wrapped__(self, **kwargs)
        return self._adapter_state_dict(adapter_name)

    @remote_function(collect='first')
    def save(self, name: Optional[str] = None, output_dir: Optional[str] = None, adapter_name: Optional[str] = None,
             save_optimizer: bool = False, **kwargs) -> str:
        """``adapter_model.safetensors`` + ``adapter_config.json`` of one tenant (all pipeline stages and TP shards
        merged); with ``save_optimizer`` also the tenant's optimizer slices per rank, scheduler and counters."""
        if adapter_name is None:
            return MegatronModel.save.__wrapped__(self, name, output_dir, save_optimizer=save_optimizer, **kwargs)
        og = self._group(adapter_name)
        path = os.path.join(output_dir or './output', name) if name else (output_dir or './output')
        os.makedirs(path, exist_ok=True)
        sd = {k: v.cpu() for k, v in self._adapter_state_dict(adapter_name).items()}
        if self.pp_size > 1:
            gathered = [None] * self.pp_size
            dist.all_gather_object(gathered, sd, group=self.pp_group)
            sd = {k: v for part in gathered for k, v in part.items()}
        if Platform.is_master():
            from safetensors.torch import save_file
            save_file({k: v.contiguous() for k, v in sd.items()}, os.path.join(path, 'adapter_model.safetensors'), metadata={'format': 'pt'})
            with open(os.path.join(path, 'adapter_config.json'), 'w') as f:
                json.dump(og.adapter_config.to_peft_dict(), f, indent=2)
        if save_optimizer:
            st = {'optim_steps': og.optim_steps, 'hyper': og.optimizer.state_dict()['param_groups'] if og.optimizer else None,
                  'params': {n: {k: v.cpu() for k, v in d.items()} for n, d in self._tenant_state.get(adapter_name, {}).items()}}
            torch.save(st, os.path.join(path, f'optimizer_{self._rank_tag()}.pt'))
            if Platform.is_master():
                if og.lr_scheduler is not None:
                    torch.save(og.lr_scheduler.state_dict(), os.path.join(path, 'scheduler.pt'))
                with open(os.path.join(path, 'trainer_state.json'), 'w') as f:
                    json.dump({'checkpoint_version': 1, 'cur_step': og.cur_step, 'gradient_accumulation_steps': og.gradient_accumulation_steps,
                               'consumed_train_samples': og.consumed_train_samples, 'optim_steps': og.optim_steps}, f)
        if dist.is_available() and dist.is_initialized():
            dist.barrier()
        return path

    @torch.no_grad()
    def _load_adapter(self, adapter_name: str, path: str) -> None:
        """Every rank reads the PEFT file and keeps the shards of the layers it holds."""
        from ..models.bridge import lora_expert_to_peft, lora_internal_to_peft
        loader = SafetensorLazyLoader(path)
        t = self.pools[0].tenants[adapter_name]
        for m, pool in zip(self.chunks, self.pools):
            for mod_name, mod in pool.modules:
                gname = self._global_name(mod_name, m._layer_offset)
                mode = getattr(mod, 'tp_mode', None)
                if not hasattr(mod, 'parts'):           # fused expert tensors
                    for which in ('gate_up', 'down'):
                        ka, kb = lora_expert_to_peft(gname, which, 'A'), lora_expert_to_peft(gname, which, 'B')
                        if ka not in loader or kb not in loader:
                            continue
                        a, b = loader.get(ka), loader.get(kb)
                        if self.ep_size > 1:
                            el = a.shape[0] // self.ep_size
                            a, b = a[self.ep_rank * el:(self.ep_rank + 1) * el], b[self.ep_rank * el:(self.ep_rank + 1) * el]
                        if self.etp_size > 1 and which == 'gate_up':
                            half = b.shape[1] // 2
                            n = half // self.tp_size
                            b = torch.cat([b[:, self.tp_rank * n:(self.tp_rank + 1) * n], b[:, half + self.tp_rank * n:half + (self.tp_rank + 1) * n]], 1)
                        elif self.etp_size > 1:
                            n = a.shape[2] // self.tp_size
                            a = a[:, :, self.tp_rank * n:(self.tp_rank + 1) * n]
                        r = a.shape[1]
                        mod.lora[which + '_A'][t.slot].zero_()
                        mod.lora[which + '_B'][t.slot].zero_()
                        mod.lora[which + '_A'][t.slot, :, :r].copy_(a)
                        mod.lora[which + '_B'][t.slot, :, :, :r].copy_(b)
                    continue
                for pname, _ in mod.parts:
                    ka, kb = lora_internal_to_peft(gname, pname, 'A'), lora_internal_to_peft(gname, pname, 'B')
                    if ka not in loader or kb not in loader:
                        continue
                    a, b = loader.get(ka), loader.get(kb)
                    if self.tp_size > 1 and mode == 'col':
                        n = b.shape[0] // self.tp_size
                        b = b[self.tp_rank * n:(self.tp_rank + 1) * n]
                    elif self.tp_size > 1 and mode == 'row':
                        n = a.shape[1] // self.tp_size
                        a = a[:, self.tp_rank * n:(self.tp_rank + 1) * n]
                    r = a.shape[0]
                    mod.lora_A[pname][t.slot].zero_()
                    mod.lora_B[pname][t.slot].zero_()
                    mod.lora_A[pname][t.slot, :r].copy_(a)
                    mod.lora_B[pname][t.slot, :, :r].copy_(b)
        loader.close()

    @remote_function()
    def load(self, name: Optional[str] = None, output_dir: Optional[str] = None, adapter_name: Optional[str] = None,
             load_optimizer: bool = False, **kwargs) -> None:
        path = os.path.join(output_dir or './output', name) if name else (output_dir or './output')
        if adapter_name is None or not os.path.isfile(os.path.join(path, 'adapter_model.safetensors')):
            return MegatronModel.load.__wrapped__(self, name, output_dir, load_optimizer=load_optimizer, **kwargs)
        if adapter_name not in self.optimizer_groups:
            self.add_adapter_to_model(adapter_name, path)
        else:
            self._load_adapter(adapter_name, path)
        # the fp32 masters of the tenant's optimizer follow the loaded values
        for n, p, slot, _ in self._tenant_slices(adapter_name):
            st = self._tenant_state.get(adapter_name, {}).get(n)
            if st is not None:
                st['master'].copy_(p.data[slot].float())
        if load_optimizer:
            self._load_tenant_state(adapter_name, path)

    def _load_tenant_state(self, adapter_name: str, path: str) -> Dict[str, Any]:
        og = self._group(adapter_name)
        f = os.path.join(path, f'optimizer_{self._rank_tag()}.pt')
        if os.path.isfile(f):
            st = torch.load(f, map_location='cpu', weights_only=True)
            og.optim_steps = int(st.get('optim_steps', 0))
            if og.optimizer is None:
                self.set_optimizer('AdamW', adapter_name=adapter_name)
            if st.get('hyper'):
                for g, sv in zip(og.optimizer.param_groups, st['hyper']):
                    for k in ('lr', 'betas', 'eps', 'weight_decay'):
                        if k in sv:
                            g[k] = sv[k] if k != 'betas' else tuple(sv[k])
            self._tenant_state[adapter_name] = {n: {k: v.to(self.device) for k, v in d.items()} for n, d in st['params'].items()}
        sched = os.path.join(path, 'scheduler.pt')
        if os.path.isfile(sched) and og.lr_scheduler is not None:
            og.lr_scheduler.load_state_dict(torch.load(sched, map_location='cpu', weights_only=True))
        info = {'cur_step': 0, 'consumed_train_samples': 0, 'gradient_accumulation_steps': og.gradient_accumulation_steps}
        ts = os.path.join(path, 'trainer_state.json')
        if os.path.isfile(ts):
            with open(ts) as fh:
                info.update(json.load(fh))
            og.cur_step, og.consumed_train_samples = info['cur_step'], info['consumed_train_samples']
        return info

    @remote_function(collect='first')
    def resume_from_checkpoint(self, checkpoint_dir: str, *, adapter_name: Optional[str] = None, resume_only_model: bool = False,
                               **kwargs) -> Dict[str, Any]:
        if adapter_name is None:
            return MegatronModel.resume_from_checkpoint.__wrapped__(self, checkpoint_dir, resume_only_model=resume_only_model, **kwargs)
        self.load(None, checkpoint_dir, adapter_name=adapter_name)
        og = self._group(adapter_name)
        if resume_only_model:
            return {'cur_step': 0, 'consumed_train_samples': 0, 'gradient_accumulation_steps': og.gradient_accumulation_steps}
        info = self._load_tenant_state(adapter_name, checkpoint_dir)
        return {k: info[k] for k in ('cur_step', 'consumed_train_samples', 'gradient_accumulation_steps')}
