"""Native generation engine: paged KV cache + continuous batched decode on the owned decoder.

Fills the role vLLM plays for the reference (``src/twinkle/sampler/vllm_sampler/vllm_engine.py:47-863``):
per-token logprobs of the *processed* distribution (after temperature / top-k / top-p), prompt logprobs
and their top-k for distillation, ``max_tokens = 0`` scoring, stop tokens / strings, per-request LoRA (a
batch may mix adapters — the segmented LoRA kernel serves them in one launch), routed-expert capture for
MoE router replay, weight updates from tensors (no reload).

Prefill runs the training forward kernels (varlen flash attention) with a sink that writes K/V into the
paged cache; decode runs one token per live sequence through ``ops.paged_attention_decode``.
"""
from __future__ import annotations

import math
import os
from dataclasses import dataclass, field
from typing import Any, Callable, Dict, Iterator, List, Optional, Sequence, Tuple

import torch

from .. import ops
from ..data_format import SampledSequence, SampleResponse, SamplingParams
from ..models.config import DecoderConfig
from ..models.decoder import DecoderModel, PackedBatch
from ..models.layers import LoraBatch, lora_batch


class PagedKVCache:
    """``[layers][num_blocks, block_size, Hkv, D]`` K and V pools + a free list.  Block 0 is never handed
    out so that an all-zero block table row is harmless."""

    def __init__(self, cfg: DecoderConfig, num_blocks: int, block_size: int, device, dtype):
        self.cfg, self.block_size, self.num_blocks = cfg, block_size, num_blocks
        shape = (cfg.num_hidden_layers, num_blocks, block_size, cfg.num_key_value_heads, cfg.head_dim)
        self.k = torch.zeros(shape, device=device, dtype=dtype)
        self.v = torch.zeros(shape, device=device, dtype=dtype)
        self.free: List[int] = list(range(num_blocks - 1, 0, -1))

    def allocate(self, n: int) -> List[int]:
        if n > len(self.free):
            raise RuntimeError(f'KV cache exhausted: need {n} blocks, {len(self.free)} free')
        return [self.free.pop() for _ in range(n)]

    def release(self, blocks: Sequence[int]) -> None:
        self.free.extend(reversed(list(blocks)))

    def blocks_for(self, n_tokens: int) -> int:
        return (n_tokens + self.block_size - 1) // self.block_size

    def write(self, layer: int, blocks: Sequence[int], start: int, k: torch.Tensor, v: torch.Tensor) -> None:
        """Store ``k, v [n, Hkv, D]`` at token positions ``start .. start+n`` of a sequence."""
        n = k.shape[0]
        pos = torch.arange(start, start + n, device=k.device)
        blk = torch.as_tensor(blocks, device=k.device)[pos // self.block_size]
        off = pos % self.block_size
        self.k[layer, blk, off] = k
        self.v[layer, blk, off] = v


@dataclass
class _Seq:
    request: int
    prompt: List[int]
    params: SamplingParams
    slot: int = -1          # LoRA slot (−1 = base)
    lora_rank: int = 0
    lora_scale: float = 0.0
    lora_target: Any = None
    blocks: List[int] = field(default_factory=list)
    tokens: List[int] = field(default_factory=list)
    logprobs: List[float] = field(default_factory=list)
    topk: List[List[Tuple[int, float]]] = field(default_factory=list)
    done: bool = False
    stop_reason: str = 'length'
    generator: Optional[torch.Generator] = None
    routed: Optional[List[torch.Tensor]] = None
    text_tail: str = ''
    vision: Optional[Dict[str, Any]] = None   # pixel_values, image_grid_thw, mrope_position_ids [3, L] of a prompt with images
    rope_delta: int = 0                        # rotary position − token index for the tokens after the prompt (images compress positions)
    linear: Dict[int, Tuple[torch.Tensor, torch.Tensor]] = field(default_factory=dict)  # layer → (conv rows, recurrent state) of linear-attention layers

    @property
    def length(self) -> int:
        return len(self.prompt) + len(self.tokens)


class NativeEngine:

    def __init__(self, model: DecoderModel, cfg: DecoderConfig, device=None, num_blocks: Optional[int] = None, block_size: int = 16,
                 max_batch: int = 256, gpu_memory_utilization: float = 0.85, decode: Optional[Callable[[List[int]], str]] = None):
        self.model, self.cfg = model, cfg
        self.device = device or next(model.parameters()).device
        self.dtype = next(model.parameters()).dtype
        if num_blocks is None:
            per_block = 2 * cfg.num_hidden_layers * block_size * cfg.num_key_value_heads * cfg.head_dim * (2 if self.dtype != torch.float32 else 4)
            if self.device.type == 'cuda':
                free, _ = torch.cuda.mem_get_info(self.device)
                num_blocks = max(int(free * gpu_memory_utilization * 0.9 // per_block), 64)
            else:
                num_blocks = 1024
        self.cache = PagedKVCache(cfg, num_blocks, block_size, self.device, self.dtype)
        self.max_batch = max_batch
        self.decode_text = decode
        self.capture_routing = False
        self.use_cuda_graphs = bool(int(os.environ.get('TWINKLE_SAMPLER_CUDA_GRAPHS', '1')))
        self._graphs: Dict[Tuple[int, int], Dict[str, Any]] = {}

    # --------------------------------------------------------------- LoRA
    def _lora_for(self, seqs: Sequence[_Seq], lens: Sequence[int]) -> Optional[LoraBatch]:
        if all(s.slot < 0 for s in seqs):
            return None
        segs, lo = [], 0
        for s, n in zip(seqs, lens):
            segs.append((lo, lo + n, s.slot, s.lora_rank, s.lora_scale))
            lo += n
        return LoraBatch(segs, self.device, [s.lora_target for s in seqs])

    # ------------------------------------------------------------- prefill
    @torch.no_grad()
    def prefill(self, seqs: List[_Seq]) -> torch.Tensor:
        """Runs all prompts as one packed row; fills the KV cache; returns the final-norm hidden state of
        every prompt token ``[ΣL, H]`` (the caller picks last tokens / scores prompts)."""
        lens = [len(s.prompt) for s in seqs]
        ids = torch.tensor([t for s in seqs for t in s.prompt], dtype=torch.long, device=self.device)
        pos = torch.cat([torch.arange(n, device=self.device) for n in lens])
        cu = torch.tensor([0] + list(torch.tensor(lens).cumsum(0)), dtype=torch.int32, device=self.device)
        for s, n in zip(seqs, lens):
            s.blocks = self.cache.allocate(self.cache.blocks_for(n + (s.params.max_tokens or 0) + 1))
        bounds = cu.tolist()

        def sink(layer: int, k: torch.Tensor, v: torch.Tensor) -> None:
            for s, a, b in zip(seqs, bounds[:-1], bounds[1:]):
                self.cache.write(layer, s.blocks, 0, k[a:b], v[a:b])

        def linear_state(layer: int, conv: torch.Tensor, state: torch.Tensor) -> None:  # hybrid stacks: what decode continues from
            for i, s in enumerate(seqs):
                s.linear[layer] = (conv[i], state[i])

        sink.linear_state = linear_state
        batch = PackedBatch(ids, pos, cu, max(lens))
        if any(s.vision for s in seqs):  # prompts with images: patches, grids and (time, height, width) positions beside the row
            p3, pix, grids = [], [], []
            for s, n in zip(seqs, lens):
                if s.vision:
                    m = torch.as_tensor(s.vision['mrope_position_ids']).long()
                    pix.append(torch.as_tensor(s.vision['pixel_values']))
                    grids.append(torch.as_tensor(s.vision['image_grid_thw']).long().view(-1, 3))
                    s.rope_delta = int(m.max()) + 1 - n
                else:
                    m = torch.arange(n).expand(3, -1)
                p3.append(m)
            batch.position_ids = torch.cat(p3, 1).to(self.device)
            batch.pixel_values = torch.cat(pix, 0).to(self.device, self.dtype)
            batch.image_grid_thw = torch.cat(grids, 0).to(self.device)
        self.model.set_record_routing(self.capture_routing)
        with lora_batch(self._lora_for(seqs, lens)):
            hidden = self.model(batch, kv_sink=sink)
        if self.capture_routing:
            routed = self.model.collect_routed_experts()
            if routed is not None:
                for s, a, b in zip(seqs, bounds[:-1], bounds[1:]):
                    s.routed = [r[a:b].cpu() for r in routed]
        return hidden

    # --------------------------------------------------------------- decode
    def _decode_body(self, tokens, positions, table, seq_lens, lora: Optional[LoraBatch], seqs: Optional[List[_Seq]] = None,
                     rope_positions: Optional[torch.Tensor] = None) -> torch.Tensor:
        """One decode token per row from device tensors only (what a CUDA graph captures). Linear-attention layers of
        hybrid stacks keep their state on the sequences (``seqs``) and always run eagerly."""
        cfg, B = self.cfg, tokens.shape[0]
        # ``positions`` index the KV cache; the rotary position differs from it after a prompt with images
        cos, sin = ops.rope_tables(positions if rope_positions is None else rope_positions, cfg.rotary_dim, cfg.rope_theta, cfg.rope_scaling)
        local = None
        if cfg.rope_local_theta:       # sliding-window layers of Gemma-3 rotate with a base of their own
            local = ops.rope_tables(positions if rope_positions is None else rope_positions, cfg.rotary_dim, cfg.rope_local_theta, None)
        x = self.model.embed_ids(tokens)
        blk = table.gather(1, (positions // self.cache.block_size).unsqueeze(1)).squeeze(1).long()
        off = positions % self.cache.block_size
        with lora_batch(lora):
            for li, layer in enumerate(self.model.layers):
                at = layer.self_attn
                h = layer.pre(x)
                if getattr(layer, 'is_linear', False):
                    conv = torch.stack([s.linear[li][0] for s in seqs])
                    st = torch.stack([s.linear[li][1] for s in seqs])
                    y, conv, st = at.step(h, conv, st)
                    for i, s in enumerate(seqs):
                        s.linear[li] = (conv[i], st[i])
                    n, x = layer.after_attention(x, y)
                    x = x + layer.feed_forward(n)
                    continue
                q, k, v, gate = at.heads_from(h, *(local if (local is not None and getattr(at, 'local_rope', False)) else (cos, sin)))
                self.cache.k[li, blk, off], self.cache.v[li, blk, off] = at.cache_entry(k, v)
                o = ops.paged_attention_decode(q, self.cache.k[li], self.cache.v[li], table, seq_lens, at.scale,
                                               window=getattr(at, 'window', None), softcap=getattr(at, 'softcap', None), sinks=getattr(at, 'sinks', None))
                n, x = layer.after_attention(x, at.project_out(o, gate))
                x = x + layer.feed_forward(n)
            x = self.model.norm(x)
        return self.model.logits(x).float()

    def _graph_for(self, B: int, max_blocks: int):
        """A captured decode step for batch bucket ``B`` and block-table width ``max_blocks`` (both powers of two).
        Inputs live in static tensors that ``decode_step`` fills before every replay; rows beyond the live batch have
        length 0 and write their K/V into block 0, which no sequence owns."""
        key = (B, max_blocks)
        ent = self._graphs.get(key)
        if ent is not None:
            return ent
        dev = self.device
        st = {'tokens': torch.zeros(B, dtype=torch.long, device=dev), 'positions': torch.zeros(B, dtype=torch.long, device=dev),
              'table': torch.zeros(B, max_blocks, dtype=torch.int32, device=dev), 'seq_lens': torch.zeros(B, dtype=torch.int32, device=dev)}
        side = torch.cuda.Stream(device=dev)
        side.wait_stream(torch.cuda.current_stream(dev))
        with torch.cuda.stream(side):  # warm-up outside the capture: one-time kernel attribute set-up, allocator warm-up
            for _ in range(2):
                self._decode_body(st['tokens'], st['positions'], st['table'], st['seq_lens'], None)
        torch.cuda.current_stream(dev).wait_stream(side)
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            st['logits'] = self._decode_body(st['tokens'], st['positions'], st['table'], st['seq_lens'], None)
        st['graph'] = graph
        self._graphs[key] = st
        return st

    @torch.no_grad()
    def decode_step(self, seqs: List[_Seq], last_tokens: torch.Tensor) -> torch.Tensor:
        """One token for every sequence; returns logits ``[B, V]`` (fp32).  On a GPU the per-token work of a whole
        layer stack is a few dozen short kernels, so the step is replayed from a CUDA graph (one per batch-size
        bucket) unless adapters or routing capture need the eager path."""
        B = len(seqs)
        positions = torch.tensor([s.length - 1 for s in seqs], device=self.device)
        max_blocks = max(len(s.blocks) for s in seqs)
        lora = self._lora_for(seqs, [1] * B)
        use_graph = (self.use_cuda_graphs and self.device.type == 'cuda' and lora is None and not self.capture_routing and not self.cfg.is_moe
                     and not any(getattr(l, 'is_linear', False) for l in self.model.layers) and not any(s.rope_delta for s in seqs)
                     # windows, score caps and latent attention decode through the PyTorch form, which reads lengths on the host
                     and not self.cfg.sliding_window and not self.cfg.attn_logit_softcapping and not self.cfg.is_mla and not self.cfg.attn_sinks)
        if use_graph:
            Bb = 1 << max(B - 1, 0).bit_length()
            Mb = 1 << max(max_blocks - 1, 0).bit_length()
            try:
                st = self._graph_for(Bb, Mb)
            except Exception as e:  # capture is an optimisation: the eager path below is always valid
                self.use_cuda_graphs = False
                import logging
                logging.getLogger('twinkle_b200').warning(f'CUDA-graph capture of the decode step failed ({type(e).__name__}: {e}); running eagerly')
                st = None
            if st is not None:
                table = torch.zeros(Bb, Mb, dtype=torch.int32)
                for i, s in enumerate(seqs):
                    table[i, :len(s.blocks)] = torch.tensor(s.blocks, dtype=torch.int32)
                lens = torch.zeros(Bb, dtype=torch.int32)
                lens[:B] = torch.tensor([s.length for s in seqs], dtype=torch.int32)
                st['table'].copy_(table, non_blocking=True)
                st['seq_lens'].copy_(lens, non_blocking=True)
                st['tokens'].zero_()
                st['tokens'][:B].copy_(last_tokens)
                st['positions'].zero_()
                st['positions'][:B].copy_(positions)
                st['graph'].replay()
                return st['logits'][:B]
        table = torch.zeros(B, max_blocks, dtype=torch.int32, device=self.device)
        for i, s in enumerate(seqs):
            table[i, :len(s.blocks)] = torch.tensor(s.blocks, dtype=torch.int32)
        seq_lens = torch.tensor([s.length for s in seqs], dtype=torch.int32, device=self.device)
        self.model.set_record_routing(self.capture_routing)
        deltas = [s.rope_delta for s in seqs]
        rope_pos = positions + torch.tensor(deltas, device=self.device) if any(deltas) else None
        logits = self._decode_body(last_tokens, positions, table, seq_lens, lora, seqs, rope_pos)
        if self.capture_routing:
            routed = self.model.collect_routed_experts()  # per layer [B, k]: the experts of the token just fed
            if routed is not None:
                for i, s in enumerate(seqs):
                    rows = [r[i:i + 1].cpu() for r in routed]
                    s.routed = rows if s.routed is None else [torch.cat([a, b], 0) for a, b in zip(s.routed, rows)]
        return logits

    # ------------------------------------------------------------- sampling
    def _sample(self, seqs: List[_Seq], logits: torch.Tensor) -> Tuple[List[int], List[float], List[Optional[List[Tuple[int, float]]]]]:
        toks, lps, tops = [], [], []
        groups: Dict[Tuple, List[int]] = {}
        for i, s in enumerate(seqs):
            p = s.params
            groups.setdefault((p.temperature, p.top_k, p.top_p, p.repetition_penalty != 1.0 or s.generator is not None, i if (
                p.repetition_penalty != 1.0 or s.generator is not None) else -1), []).append(i)
        out_tok = [0] * len(seqs)
        out_lp = [0.0] * len(seqs)
        out_top: List[Optional[List[Tuple[int, float]]]] = [None] * len(seqs)
        for (temp, tk, tp, _special, _), idxs in groups.items():
            lg = logits[idxs]
            for j, i in enumerate(idxs):
                rp = seqs[i].params.repetition_penalty
                if rp != 1.0:
                    seen = torch.tensor(sorted(set(seqs[i].prompt + seqs[i].tokens)), device=lg.device)
                    vals = lg[j, seen]
                    lg[j, seen] = torch.where(vals > 0, vals / rp, vals * rp)
            gen = seqs[idxs[0]].generator if len(idxs) == 1 else None
            tok, lp = ops.ref.sample_tokens(lg, temp, tk, tp, gen) if not lg.is_cuda else ops.sample_tokens(lg, temp, tk, tp, gen)
            for j, i in enumerate(idxs):
                out_tok[i], out_lp[i] = int(tok[j]), float(lp[j])
                k = seqs[i].params.logprobs
                if k and k > 1:
                    proc = torch.log_softmax(lg[j] / max(temp, 1e-6), -1) if temp > 0 else torch.log_softmax(lg[j], -1)
                    v, ix = proc.topk(min(k, proc.numel()))
                    out_top[i] = [(int(a), float(b)) for a, b in zip(ix, v)]
        return out_tok, out_lp, out_top

    def _check_stop(self, s: _Seq, tok: int, eos: Optional[int]) -> None:
        p = s.params
        if (eos is not None and tok == eos) or tok in p.stop_token_ids():
            s.done, s.stop_reason = True, 'stop'
            return
        strs = p.stop_strings()
        if strs and self.decode_text is not None:
            s.text_tail = (s.text_tail + self.decode_text([tok]))[-256:]
            if any(x in s.text_tail for x in strs):
                s.done, s.stop_reason = True, 'stop'
                return
        if p.max_tokens is not None and len(s.tokens) >= p.max_tokens:
            s.done, s.stop_reason = True, 'length'

    # ----------------------------------------------------------------- API
    @torch.no_grad()
    def generate(self, prompts: List[List[int]], params: List[SamplingParams], lora: Optional[List[Optional[Dict[str, Any]]]] = None,
                 eos_token_id: Optional[int] = None, on_token: Optional[Callable[[int, int, float], None]] = None,
                 vision: Optional[List[Optional[Dict[str, Any]]]] = None) -> List[SampleResponse]:
        """``prompts[i]`` is sampled ``params[i].num_samples`` times.  ``lora[i]`` = ``{slot, rank, scale, target}`` or None."""
        responses = [SampleResponse() for _ in prompts]
        seqs: List[_Seq] = []
        for i, (pr, sp) in enumerate(zip(prompts, params)):
            lo = (lora[i] if lora else None) or {}
            for n in range(sp.num_samples):
                g = None
                if sp.seed is not None:
                    g = torch.Generator(device=self.device).manual_seed(sp.seed + n)
                seqs.append(_Seq(i, list(pr), sp, lo.get('slot', -1), lo.get('rank', 0), lo.get('scale', 0.0), lo.get('target'), generator=g,
                                 vision=vision[i] if vision else None))
        for lo_i in range(0, len(seqs), self.max_batch):
            self._run_group(seqs[lo_i:lo_i + self.max_batch], responses, eos_token_id, on_token)
        return responses

    def _run_group(self, seqs: List[_Seq], responses, eos, on_token) -> None:
        hidden = self.prefill(seqs)
        lens = [len(s.prompt) for s in seqs]
        ends = torch.tensor(lens, device=self.device).cumsum(0) - 1
        # prompt scoring (teacher logprobs for distillation / max_tokens == 0)
        need_prompt = [s.params.prompt_logprobs is not None for s in seqs]
        if any(need_prompt):
            off = 0
            for s, n, need in zip(seqs, lens, need_prompt):
                if need and responses[s.request].prompt_logprobs is None:
                    h = hidden[off:off + n]
                    ids = torch.tensor(s.prompt[1:] + [0], device=self.device)
                    temp = s.params.temperature if s.params.temperature > 0 else 1.0
                    lp, _ = ops.fused_linear_logprob(h, self.model.head_weight(), ids, temp)
                    responses[s.request].prompt_logprobs = [None] + [float(x) for x in lp[:-1]]
                    k = s.params.prompt_logprobs
                    if k and k > 0:
                        lg = torch.log_softmax(self.model.logits(h[:-1]).float() / temp, -1)
                        v, ix = lg.topk(min(k, lg.shape[-1]), -1)
                        responses[s.request].topk_prompt_logprobs = [None] + [[(int(a), float(b)) for a, b in zip(r_i, r_v)]
                                                                             for r_i, r_v in zip(ix.tolist(), v.tolist())]
                off += n
        live = [s for s in seqs if not s.params.scoring_only]
        for s in seqs:
            if s.params.scoring_only:
                s.done = True
        if live:
            idx = [i for i, s in enumerate(seqs) if not s.params.scoring_only]
            logits = self.model.logits(hidden[ends[idx]]).float()
            while live:
                toks, lps, tops = self._sample(live, logits)
                for s, t, lp, tp in zip(live, toks, lps, tops):
                    s.tokens.append(t)
                    s.logprobs.append(lp)
                    if tp is not None:
                        s.topk.append(tp)
                    if on_token is not None:
                        on_token(s.request, t, lp)
                    self._check_stop(s, t, eos)
                nxt = [s for s in live if not s.done]
                if not nxt:
                    break
                last = torch.tensor([s.tokens[-1] for s in nxt], device=self.device)
                for s in nxt:  # grow the block list when a sequence crosses a block boundary
                    need = self.cache.blocks_for(s.length + 1) - len(s.blocks)
                    if need > 0:
                        s.blocks += self.cache.allocate(need)
                logits = self.decode_step(nxt, last)
                live = nxt
        for s in seqs:
            self.cache.release(s.blocks)
            s.blocks, s.linear = [], {}
            if not s.params.scoring_only:
                responses[s.request].sequences.append(SampledSequence(stop_reason=s.stop_reason, tokens=s.tokens, logprobs=s.logprobs,
                                                                      topk_logprobs=s.topk or None, routed_experts=s.routed))

    def reset_prefix_cache(self) -> None:
        """No cross-request prefix reuse is kept, so there is nothing stale to drop after a weight update."""
        return None
