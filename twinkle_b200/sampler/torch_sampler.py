"""The native sampler component.

Parity: reference ``src/twinkle/sampler/vllm_sampler/vllm_sampler.py:39-516`` (``vLLMSampler``): ``sample``
(dispatch ``slice_dp``, collect ``flatten``) turns trajectories or features into prompts, runs the engine and
returns one ``SampleResponse`` per input whose sequences carry ``new_input_feature`` (prompt ⊕ sampled tokens
with labels on the sampled part, ready for ``forward_backward``); ``max_tokens == 0`` scores prompts only;
``sample_stream``; ``sleep / wake_up``; ``reset_prefix_cache``; ``receive_weights`` / ``update_weights`` take
tensors straight from the trainer (peer-copy weight sync) without a reload; LoRA adapters come from a
directory (``adapter_path``), from a previous ``add_adapter_to_sampler`` or from synced tensors.
``vLLMSampler`` is kept as an alias so reference scripts keep working.
"""
from __future__ import annotations

import os
from typing import Any, Dict, Iterator, List, Optional, Sequence, Union

import torch

from ..data_format import SampleResponse, SamplingParams
from ..infra import remote_class, remote_function
from ..model.multi_lora import LoraConfig, MultiLora
from ..models.bridge import hf_names_for, hf_to_internal
from ..models.config import PRESETS, DecoderConfig, preset
from ..models.decoder import build_model
from ..template import Template
from ..utils.device_mesh import DeviceMesh
from ..utils.platform import Platform
from ..checkpoint_engine import CheckpointEngineMixin
from .base import Sampler
from .engine import NativeEngine


@remote_class()
class TorchSampler(Sampler, CheckpointEngineMixin):

    def __init__(self, model_id: Optional[str] = None, config: Union[DecoderConfig, Dict[str, Any], None] = None,
                 device_mesh: DeviceMesh = None, engine_args: Optional[Dict[str, Any]] = None, seed: int = 42, device=None,
                 max_loras: int = 4, max_r: int = 32, enable_lora: bool = True, **kwargs):
        self.device_mesh = device_mesh
        self.device = torch.device(device) if device is not None else Platform.current_device()
        if self.device.type == 'cuda':
            torch.cuda.set_device(self.device)
        if isinstance(config, DecoderConfig):
            self.config = config
        elif isinstance(config, dict):
            self.config = DecoderConfig.from_hf(config)
        elif model_id and model_id.lower() in PRESETS:
            self.config = preset(model_id)
        else:
            from ..hub import HubOperation
            model_id = HubOperation.download_model(model_id)
            self.config = DecoderConfig.from_pretrained(model_id)
        self.model_id = model_id
        dtype = torch.bfloat16 if self.device.type == 'cuda' else torch.float32
        load_dir = model_id if model_id and os.path.isdir(str(model_id)) else None
        self.model = build_model(self.config, device=self.device, dtype=dtype, seed=kwargs.get('weight_seed', 0), init=load_dir is None)
        if load_dir:
            self._load_dir(load_dir)
        self.model.requires_grad_(False)
        self.multi_lora = MultiLora(self.model, max_loras, max_r) if enable_lora else None
        if self.multi_lora is not None:
            self.model.requires_grad_(False)
        ea = dict(engine_args or {})
        self.engine = NativeEngine(self.model, self.config, self.device, num_blocks=ea.get('num_blocks'),
                                   block_size=ea.get('block_size', 16), max_batch=ea.get('max_batch', 256),
                                   gpu_memory_utilization=ea.get('gpu_memory_utilization', 0.85), decode=self._decode_tokens)
        self.seed = seed + Platform.get_rank()
        self._synced_adapter = '__synced__'
        self._path_adapters: Dict[str, str] = {}
        self._asleep = False

    def _decode_tokens(self, ids: List[int]) -> str:
        return self.template.decode(ids, skip_special_tokens=False) if self.template is not None else ''

    def _load_dir(self, directory: str) -> None:
        from ..utils.safetensors_io import SafetensorLazyLoader
        loader = SafetensorLazyLoader(directory)
        with torch.no_grad():
            for n, p in self.model.named_parameters():
                if 'lora' in n:
                    continue
                if n == 'lm_head.weight' and 'lm_head.weight' not in loader:
                    p.copy_(loader.get('model.embed_tokens.weight'))
                else:
                    p.copy_(hf_to_internal(n, self.config, loader.get).to(p.dtype))

    # ------------------------------------------------------------ adapters
    @remote_function()
    def add_adapter_to_sampler(self, adapter_name: str, config_or_dir, **kwargs) -> None:
        if self.multi_lora is None:
            raise RuntimeError('sampler was created with enable_lora=False')
        if self.multi_lora.has(adapter_name):
            self.multi_lora.release_lora(adapter_name)
        self.multi_lora.acquire_lora(adapter_name, LoraConfig.from_any(config_or_dir))
        if isinstance(config_or_dir, str) and os.path.isfile(os.path.join(config_or_dir, 'adapter_model.safetensors')):
            from safetensors.torch import load_file
            sd = load_file(os.path.join(config_or_dir, 'adapter_model.safetensors'))
            self.multi_lora.set_state_dict(adapter_name, {k: v.to(self.device) for k, v in sd.items()})

    def _resolve_adapter(self, adapter_name: Optional[str], adapter_path: Optional[str]) -> Optional[str]:
        if adapter_path:
            key = os.path.abspath(adapter_path)
            name = self._path_adapters.get(key)
            if name is None:
                name = f'__path_{len(self._path_adapters)}__'
                if self.multi_lora.free_slots() == 0:  # evict the oldest path adapter
                    old_key, old = next(iter(self._path_adapters.items()))
                    self.multi_lora.release_lora(old)
                    del self._path_adapters[old_key]
                self.add_adapter_to_sampler(name, adapter_path)
                self._path_adapters[key] = name
            return name
        if adapter_name and self.multi_lora is not None and self.multi_lora.has(adapter_name):
            return adapter_name
        if self.multi_lora is not None and self.multi_lora.has(self._synced_adapter):
            return self._synced_adapter
        return None

    # -------------------------------------------------------------- sample
    def _prompts(self, inputs) -> List[Dict[str, Any]]:
        if isinstance(inputs, dict):
            inputs = [inputs]
        feats = []
        for x in inputs:
            if 'input_ids' in x:
                feats.append(x)
            else:
                feats.append(self.encode_trajectory(x))
        return feats

    @remote_function(dispatch='slice_dp', collect='flatten')
    def sample(self, inputs, sampling_params: Union[SamplingParams, Dict[str, Any], None] = None, adapter_name: Optional[str] = None,
               adapter_path: Optional[str] = None, **kwargs) -> List[SampleResponse]:
        if self._asleep:
            self.wake_up()
        sp = sampling_params if isinstance(sampling_params, SamplingParams) else SamplingParams.from_dict(sampling_params)
        if sp.seed is None and self.seed is not None and kwargs.get('deterministic', False):
            sp.seed = self.seed
        feats = self._prompts(inputs)
        prompts = [[int(t) for t in f['input_ids']] for f in feats]
        # ``use_base_model=True`` bypasses every adapter, the synced policy adapter included (a condenser or judge that shares
        # the sampler with the policy under training must not see half-trained weights)
        name = self._resolve_adapter(adapter_name, adapter_path) if self.multi_lora is not None and not kwargs.get('use_base_model') else None
        lora = None
        if name is not None:
            t = self.multi_lora.tenants[name]
            lora = [{'slot': t.slot, 'rank': t.config.r, 'scale': t.config.scaling, 'target': t.target}] * len(prompts)
        eos = self.template.eos_token_id if self.template is not None else self.config.eos_token_id
        self.engine.capture_routing = bool(kwargs.get('return_routed_experts', self.config.is_moe))
        vision = [{k: f[k] for k in ('pixel_values', 'image_grid_thw', 'mrope_position_ids')} if f.get('pixel_values') is not None else None for f in feats]
        responses = self.engine.generate(prompts, [sp] * len(prompts), lora, eos, vision=vision if any(vision) else None)
        for f, r in zip(feats, responses):
            for s in r.sequences:
                s.new_input_feature = Template.concat_input_feature(f, s.tokens)
                if s.routed_experts is not None:
                    s.new_input_feature['routed_experts'] = s.routed_experts
                if self.template is not None:
                    s.decoded = self.template.decode(s.tokens)
        return responses

    def sample_stream(self, inputs, sampling_params=None, adapter_name: Optional[str] = None, **kwargs) -> Iterator[Dict[str, Any]]:
        """Yields ``{'index', 'token', 'logprob', 'text'}`` per generated token, then ``{'done': True, 'responses': [...]}``."""
        import queue
        import threading
        q: 'queue.Queue' = queue.Queue()
        sp = sampling_params if isinstance(sampling_params, SamplingParams) else SamplingParams.from_dict(sampling_params)
        feats = self._prompts(inputs)
        prompts = [[int(t) for t in f['input_ids']] for f in feats]
        eos = self.template.eos_token_id if self.template is not None else self.config.eos_token_id

        def work():
            try:
                res = self.engine.generate(prompts, [sp] * len(prompts), None, eos, on_token=lambda i, t, lp: q.put(
                    {'index': i, 'token': t, 'logprob': lp, 'text': self._decode_tokens([t])}))
                q.put({'done': True, 'responses': res})
            except Exception as e:  # surfaced to the consumer
                q.put({'done': True, 'error': repr(e)})

        threading.Thread(target=work, daemon=True).start()
        while True:
            item = q.get()
            yield item
            if item.get('done'):
                return

    # ------------------------------------------------------- weight updates
    @remote_function()
    def update_weights(self, weights, peft_config: Optional[Dict[str, Any]] = None, **kwargs) -> None:
        """``weights``: iterable of (HF or PEFT name, tensor).  PEFT names update the synced adapter slot;
        HF names overwrite base weights (fused tensors are reassembled from their parts)."""
        base: Dict[str, torch.Tensor] = {}
        lora: Dict[str, torch.Tensor] = {}
        if isinstance(weights, dict):
            weights = weights.items()
        for k, v in weights:
            (lora if 'lora_' in k else base)[k] = v
        if base:
            with torch.no_grad():
                for n, p in self.model.named_parameters():
                    if 'lora' in n:
                        continue
                    names = hf_names_for(n, self.config)
                    if all(x in base for x in names):
                        p.copy_(hf_to_internal(n, self.config, base.__getitem__).to(p.device, p.dtype))
        if lora:
            # a named tenant keeps its own slot (multi-tenant RL); without a name the single "synced" slot is used
            name = kwargs.get('adapter_name') or self._synced_adapter
            if not self.multi_lora.has(name):
                cfg = LoraConfig.from_any(peft_config or {'r': next(iter(lora.values())).shape[0] if lora else 8})
                self.multi_lora.acquire_lora(name, cfg)
            self.multi_lora.set_state_dict(name, {k: v.to(self.device) for k, v in lora.items()})
        self.engine.reset_prefix_cache()

    # ---- sampler end of a weight sync across worker groups (reference vllm_sampler.py:439-487)
    @remote_function(collect='first')
    def prepare_checkpoint_engine(self, role: str = 'recv', **kwargs) -> Dict[str, Any]:
        return CheckpointEngineMixin.prepare_checkpoint_engine(self, role, **kwargs)

    @remote_function(collect='first')
    def receive_weights(self, weights=None, peft_config: Optional[Dict[str, Any]] = None, **kwargs):
        """With ``weights``: same as ``update_weights``.  Without: take them from the prepared checkpoint engine;
        returns the number of bytes received."""
        if weights is not None:
            return self.update_weights(weights, peft_config=peft_config, **kwargs)
        return self._receive_weights(peft_config=peft_config, **kwargs)

    @remote_function()
    def finalize_checkpoint_engine(self) -> None:
        CheckpointEngineMixin.finalize_checkpoint_engine(self)

    @remote_function(collect='first')
    def get_state_keys(self) -> List[str]:
        keys = []
        for n, _ in self.model.named_parameters():
            if 'lora' not in n:
                keys += hf_names_for(n, self.config)
        return keys

    @remote_function()
    def reset_prefix_cache(self) -> None:
        self.engine.reset_prefix_cache()

    @remote_function()
    def sleep(self, level: int = 1) -> None:
        """Level 1 drops the KV pools (they are rebuilt on wake-up); level 2 also moves weights to the host."""
        self.engine.cache.k = self.engine.cache.v = None
        if level >= 2:
            self.model.to('cpu')
        if self.device.type == 'cuda':
            torch.cuda.empty_cache()
        self._asleep = True

    @remote_function()
    def wake_up(self) -> None:
        if not self._asleep:
            return
        self.model.to(self.device)
        c = self.engine.cache
        shape = (self.config.num_hidden_layers, c.num_blocks, c.block_size, self.config.num_key_value_heads, self.config.head_dim)
        c.k = torch.zeros(shape, device=self.device, dtype=self.engine.dtype)
        c.v = torch.zeros(shape, device=self.device, dtype=self.engine.dtype)
        c.free = list(range(c.num_blocks - 1, 0, -1))
        self._asleep = False

    @remote_function()
    def apply_patch(self, patch_cls, **kwargs) -> None:
        from ..patch import apply_patch
        apply_patch(self, patch_cls, **kwargs)


vLLMSampler = TorchSampler
