"""Model / sampler back ends behind the server apps.

Parity: reference ``src/twinkle/server/model/backends/{common,transformers_model,mock_model}.py``,
``server/common/datum.py`` and ``server/sampler/backends/mock_sampler.py``:

* ``datum_to_input_feature`` — Tinker ``Datum`` → ``InputFeature`` (``target_tokens`` + ``weights`` → labels
  with −100 where the weight is 0; without weights token id 0 → −100; ``logprobs`` → ``old_logps``,
  ``advantages``, ``ref_logps``);
* ``loss_fn`` routing: ``cross_entropy`` → CrossEntropyLoss, ``importance_sampling`` → DPO when any datum
  carries ``ref_logps`` else GRPO;
* per-datum ``{'logprobs', 'elementwise_loss'}`` TensorData outputs + numeric ``metrics``;
* ``MockModel`` / ``MockSampler``: deterministic numpy outputs keyed by a stable hash of the request, so
  the whole HTTP stack is testable without a GPU;
* ``BackendSelector`` validates the requested kind before constructing.
"""
from __future__ import annotations

import hashlib
import json
from typing import Any, Dict, List, Optional, Sequence

import numpy as np

from ...utils.seed import stable_seed
from ..exceptions import ConfigError


# ----------------------------------------------------------------- datum I/O
def tensor_data(values: Sequence[float], dtype: str = 'float32') -> Dict[str, Any]:
    v = list(values)
    return {'data': v, 'dtype': dtype, 'shape': [len(v)]}


def from_tensor_data(td: Any) -> List[Any]:
    if td is None:
        return []
    if isinstance(td, dict):
        return list(td.get('data', []))
    return list(td)


def _tensor_of(td: Any):
    """A ``TensorData`` record (flat ``data`` + ``shape``) as a torch tensor."""
    import torch
    t = torch.tensor(from_tensor_data(td), dtype=torch.int64 if isinstance(td, dict) and str(td.get('dtype', '')).startswith('int') else torch.float32)
    shape = td.get('shape') if isinstance(td, dict) else None
    return t.view(*shape) if shape else t


def datum_to_input_feature(datum: Dict[str, Any], model_config: Any = None) -> Dict[str, Any]:
    """Tinker datum → input feature. Vision-language clients send preprocessed ``pixel_values`` and ``image_grid_thw`` in
    ``loss_fn_inputs`` (the tokens already hold one placeholder per merged patch); with the model's config at hand the
    three-row positions are rebuilt here (reference ``server/common/datum.py:11-60``)."""
    mi = datum.get('model_input') or {}
    if 'chunks' in mi:
        ids = [t for c in mi['chunks'] for t in c.get('tokens', [])]
    else:
        ids = list(mi.get('tokens', mi.get('input_ids', [])))
    lf = datum.get('loss_fn_inputs') or {}
    targets = from_tensor_data(lf.get('target_tokens'))
    weights = from_tensor_data(lf.get('weights'))
    feat: Dict[str, Any] = {'input_ids': [int(t) for t in ids]}
    if targets:
        if weights:
            labels = [int(t) if w != 0 else -100 for t, w in zip(targets, weights)]
        else:
            labels = [int(t) if int(t) != 0 else -100 for t in targets]
        labels = (labels + [-100] * len(ids))[:len(ids)]
        feat['labels'] = labels
    for src, dst in (('logprobs', 'old_logps'), ('advantages', 'advantages'), ('ref_logps', 'ref_logps')):
        if lf.get(src) is not None:
            feat[dst] = [float(x) for x in from_tensor_data(lf[src])]
    if lf.get('pixel_values') is not None and lf.get('image_grid_thw') is not None:
        feat['pixel_values'] = _tensor_of(lf['pixel_values'])
        grid = _tensor_of(lf['image_grid_thw']).long().view(-1, 3)
        feat['image_grid_thw'] = grid.tolist()
        image_id = getattr(model_config, 'image_token_id', None)
        if image_id is None:
            raise ValueError('this datum carries images but the model behind the endpoint is not a vision-language model')
        from ...models.vision import rope_index
        vision = getattr(model_config, 'vision', None) or {}
        feat['mrope_position_ids'] = rope_index(feat['input_ids'], feat['image_grid_thw'], image_id, int(vision.get('spatial_merge_size', 2)),
                                                video_token_id=getattr(model_config, 'video_token_id', None))
        feat['placeholder_ids'] = [t for t in (image_id, getattr(model_config, 'video_token_id', None)) if t is not None]
    return feat


def split_loss_inputs(features: List[Dict[str, Any]]) -> Dict[str, Any]:
    """Collect per-datum RL extras into loss keyword arguments (ragged lists are aligned by the loss)."""
    kw: Dict[str, Any] = {}
    n = len(features)
    for key in ('old_logps', 'advantages'):
        if any(key in f for f in features):
            rows = []
            for f in features:
                v = f.get(key)
                if v is None:
                    v = [0.0]
                lab = f.get('labels')
                if lab is not None and len(v) == len(lab):  # full-length: keep only target positions
                    v = [x for x, l in zip(v, lab) if l != -100] or [0.0]
                rows.append(v)
            kw[key] = rows
    if any('ref_logps' in f for f in features):
        import torch
        width = max(len(f.get('ref_logps', [])) for f in features)
        kw['ref_outputs'] = {'logps': torch.tensor([(f.get('ref_logps', []) + [0.0] * width)[:width] for f in features])}
    return kw


FORWARD_OPTIONS = ('disable_lora', )  # keys of ``loss_fn_config`` that steer the forward pass, not the loss


def forward_options(loss_fn_config: Optional[Dict[str, Any]]) -> Dict[str, Any]:
    """``{'disable_lora': True}`` runs the frozen base model: how a client gets reference log-probs for DPO from the same
    server-side model (reference ``server/model/backends/common.py:120-150``)."""
    return {k: bool(v) for k, v in (loss_fn_config or {}).items() if k in FORWARD_OPTIONS}


def choose_loss(loss_fn: str, features: List[Dict[str, Any]], loss_fn_config: Optional[Dict[str, Any]] = None):
    from ...loss import CrossEntropyLoss, DPOLoss, GRPOLoss, torch_loss_mapping
    cfg = {k: v for k, v in (loss_fn_config or {}).items() if k not in FORWARD_OPTIONS}
    if loss_fn == 'cross_entropy':
        return CrossEntropyLoss(**cfg)
    if loss_fn in ('importance_sampling', 'ppo'):
        if any('ref_logps' in f for f in features):
            # the wire names carry a dpo_ prefix (dpo_beta, dpo_loss_type, dpo_sft_weight); plain names are accepted too
            return DPOLoss(**{(k[4:] if k.startswith('dpo_') else k): v for k, v in cfg.items()})
        return GRPOLoss(**{k: v for k, v in cfg.items() if not k.startswith('dpo_')})
    if loss_fn in torch_loss_mapping:
        return torch_loss_mapping[loss_fn](**cfg)
    raise ValueError(f'unknown loss_fn {loss_fn!r}')


def clean_metrics(metrics: Dict[str, Any]) -> Dict[str, float]:
    """Metric objects report strings (``'0.03 iters/s'``); Tinker wants numbers."""
    out = {}
    for k, v in (metrics or {}).items():
        if isinstance(v, (int, float)):
            out[k] = float(v)
            continue
        try:
            out[k] = float(str(v).split()[0].rstrip('s%'))
        except (ValueError, IndexError):
            continue
    return out


def build_fwdbwd_output(features: List[Dict[str, Any]], out: Dict[str, Any], metrics: Dict[str, Any]) -> Dict[str, Any]:
    """Tinker ``ForwardBackwardOutput``: per datum the logprobs and element-wise loss of its target positions."""
    import torch
    results = []
    logps = out.get('logps')
    for i, f in enumerate(features):
        n = len(f['input_ids'])
        lab = f.get('labels') or [-100] * n
        row = logps[i, :n].tolist() if torch.is_tensor(logps) and logps.dim() == 2 and i < logps.shape[0] else [0.0] * n
        lp = [x if l != -100 else 0.0 for x, l in zip(row, lab)]
        results.append({'logprobs': tensor_data(lp), 'elementwise_loss': tensor_data([-x for x in lp])})
    m = clean_metrics(metrics)
    if 'loss' in out:
        m.setdefault('loss:sum' if out.get('num_tokens') else 'loss', float(out['loss']))
    return {'loss_fn_output_type': 'per_datum', 'loss_fn_outputs': results, 'metrics': m}


# -------------------------------------------------------------------- mocks
class MockModel:
    """Deterministic stand-in for the training backend (numpy only)."""

    def __init__(self, model_id: str = 'mock', max_loras: int = 5, **kwargs):
        self.model_id, self.max_loras = model_id, max_loras
        self.adapters: Dict[str, Dict[str, Any]] = {}
        self.steps: Dict[str, int] = {}
        self.saved: Dict[str, str] = {}

    def ping(self) -> bool:
        return True

    def data_world_size(self) -> int:
        return 1

    def add_adapter_to_model(self, adapter_name: str, config_or_dir=None, **kw) -> None:
        if adapter_name in self.adapters:
            raise ValueError(f'adapter {adapter_name!r} already exists')
        if len(self.adapters) >= self.max_loras:
            raise RuntimeError('no free LoRA slot')
        self.adapters[adapter_name] = {'config': config_or_dir, 'grad_ready': False}
        self.steps[adapter_name] = 0

    def remove_adapter(self, adapter_name: str, **kw) -> None:
        self.adapters.pop(adapter_name, None)
        self.steps.pop(adapter_name, None)

    def _rng(self, *key) -> np.random.Generator:
        return np.random.default_rng(stable_seed(self.model_id, *key))

    def tinker_forward_backward(self, datums: List[Dict[str, Any]], adapter_name: str, loss_fn: str = 'cross_entropy', backward: bool = True,
                                loss_fn_config: Optional[Dict[str, Any]] = None) -> Dict[str, Any]:
        if adapter_name not in self.adapters:
            raise KeyError(f'unknown adapter {adapter_name!r}')
        outs, total, ntok = [], 0.0, 0
        for d in datums:
            f = datum_to_input_feature(d)
            rng = self._rng(f['input_ids'], self.steps[adapter_name])
            lp = (-np.abs(rng.normal(2.0, 0.5, size=len(f['input_ids'])))).round(6)
            lab = f.get('labels') or [-100] * len(lp)
            lp = [float(x) if l != -100 else 0.0 for x, l in zip(lp, lab)]
            outs.append({'logprobs': tensor_data(lp), 'elementwise_loss': tensor_data([-x for x in lp])})
            total += -sum(lp)
            ntok += sum(1 for l in lab if l != -100)
        if backward:
            self.adapters[adapter_name]['grad_ready'] = True
        return {'loss_fn_output_type': 'per_datum', 'loss_fn_outputs': outs, 'metrics': {'loss:sum': total, 'num_tokens': float(ntok)}}

    def tinker_step(self, adapter_name: str, adam_params: Optional[Dict[str, Any]] = None) -> Dict[str, Any]:
        a = self.adapters[adapter_name]
        if not a['grad_ready']:
            raise RuntimeError('optim_step without a preceding forward_backward')
        a['grad_ready'] = False
        self.steps[adapter_name] += 1
        return {'metrics': {'step': float(self.steps[adapter_name]), 'learning_rate': float((adam_params or {}).get('learning_rate', 1e-4))}}

    def save(self, name: str, output_dir: str, adapter_name: Optional[str] = None, **kw) -> str:
        import os
        path = os.path.join(output_dir, name)
        os.makedirs(path, exist_ok=True)
        with open(os.path.join(path, 'mock_state.json'), 'w') as f:
            json.dump({'adapter': adapter_name, 'steps': self.steps.get(adapter_name or '', 0)}, f)
        with open(os.path.join(path, 'adapter_config.json'), 'w') as f:
            json.dump({'r': 8, 'lora_alpha': 16, 'peft_type': 'LORA', 'base_model_name_or_path': self.model_id}, f)
        return path

    def load(self, name: Optional[str], output_dir: str, adapter_name: Optional[str] = None, **kw) -> None:
        import os
        p = os.path.join(output_dir, name, 'mock_state.json') if name else os.path.join(output_dir, 'mock_state.json')
        if os.path.isfile(p):
            with open(p) as f:
                self.steps[adapter_name or ''] = json.load(f).get('steps', 0)

    def generic_call(self, method: str, **kwargs) -> Any:
        if method in ('forward', 'forward_only', 'forward_backward'):
            n = len(kwargs.get('inputs') or [])
            return {'loss': round(float(self._rng(method, n).uniform(1, 3)), 6), 'num_tokens': float(n)}
        if method == 'calculate_loss':
            return 2.0
        if method == 'clip_grad_norm' or method == 'clip_grad_and_step':
            return 1.0
        if method == 'calculate_metric':
            return {'loss': '2.0000'}
        if method == 'get_train_configs':
            return f'mock model {self.model_id}'
        if method == 'get_state_dict':
            return {}
        return None


class MockSampler:
    """Scriptable generation: tokens derive from a hash of the prompt; ``script`` entries (per call) can force
    ``stop_reason`` or a literal completion (used by tool-call turn tests)."""

    def __init__(self, model_id: str = 'mock', script: Optional[List[Dict[str, Any]]] = None, **kwargs):
        self.model_id = model_id
        self.script = list(script or [])
        self.calls = 0
        self.template = None

    def set_template(self, template_cls, **kw) -> None:
        from ...template import Template, template_mapping
        if isinstance(template_cls, str):
            template_cls = template_mapping.get(template_cls, Template)
        self.template = template_cls(**kw) if isinstance(template_cls, type) else template_cls

    def add_adapter_to_sampler(self, adapter_name: str, config_or_dir=None, **kw) -> None:
        pass

    def sample(self, inputs, sampling_params=None, adapter_name=None, adapter_path=None, **kw):
        from ...data_format import SampledSequence, SampleResponse, SamplingParams
        from ...template import Template
        sp = sampling_params if isinstance(sampling_params, SamplingParams) else SamplingParams.from_dict(sampling_params)
        out = []
        for x in ([inputs] if isinstance(inputs, dict) else inputs):
            if 'input_ids' not in x and self.template is not None:
                x = self.template.encode(x, add_generation_prompt=True)
            ids = list(x.get('input_ids', []))
            step = self.script[self.calls % len(self.script)] if self.script else {}
            self.calls += 1
            resp = SampleResponse()
            n_new = min(sp.max_tokens if sp.max_tokens is not None else 16, 64)
            for s in range(sp.num_samples):
                rng = np.random.default_rng(stable_seed(self.model_id, ids, s, sp.seed))
                if 'text' in step and self.template is not None:
                    toks = self.template.tokenizer.encode(step['text'])
                else:
                    toks = [int(t) for t in rng.integers(1, 255, size=n_new)]
                lps = [float(-abs(v)) for v in rng.normal(1.0, 0.3, size=len(toks))]
                seq = SampledSequence(stop_reason=step.get('stop_reason', 'length' if len(toks) >= n_new else 'stop'), tokens=toks, logprobs=lps)
                seq.new_input_feature = Template.concat_input_feature({'input_ids': ids}, toks)
                if self.template is not None:
                    seq.decoded = self.template.decode(toks)
                resp.sequences.append(seq)
            if sp.prompt_logprobs is not None:
                rng = np.random.default_rng(stable_seed(self.model_id, ids, 'prompt'))
                resp.prompt_logprobs = [None] + [float(-abs(v)) for v in rng.normal(2.0, 0.5, size=max(len(ids) - 1, 0))]
            out.append(resp)
        return out


class BackendSelector:
    MODEL = ('mock', 'transformers', 'megatron')
    SAMPLER = ('mock', 'torch', 'vllm')

    @staticmethod
    def model(kind: str, **kwargs):
        if kind not in BackendSelector.MODEL:
            raise ConfigError('backend', kind, BackendSelector.MODEL)
        if kind == 'mock':
            return MockModel(**kwargs)
        from .native import NativeModelBackend
        return NativeModelBackend(kind=kind, **kwargs)

    @staticmethod
    def sampler(kind: str, **kwargs):
        if kind not in BackendSelector.SAMPLER:
            raise ConfigError('sampler_type', kind, BackendSelector.SAMPLER)
        if kind == 'mock':
            return MockSampler(**kwargs)
        from ...sampler import TorchSampler
        kwargs.pop('script', None)
        return TorchSampler(**kwargs)
