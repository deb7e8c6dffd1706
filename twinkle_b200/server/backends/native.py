"""The real training backend behind the Model app: the multi-LoRA engine plus the Tinker-shaped methods.

Parity: reference ``src/twinkle/server/model/backends/transformers_model.py:22-112`` and
``common.py:125-362`` (``tinker_forward_only``, ``tinker_forward_backward``, ``tinker_step``,
``tinker_calculate_metric``, ``tinker_load``, ``ping``).
"""
from __future__ import annotations

from typing import Any, Dict, List, Optional

from . import build_fwdbwd_output, choose_loss, clean_metrics, datum_to_input_feature, forward_options, split_loss_inputs


class NativeModelBackend:

    def __init__(self, kind: str = 'transformers', model_id: str = 'tiny-dense', device_mesh=None, max_loras: int = 5, max_r: int = 32,
                 max_length: int = 8192, **kwargs):
        if kind == 'megatron':
            from ...model.megatron import MultiLoraMegatronModel as Cls
        else:
            from ...model import MultiLoraTransformersModel as Cls
        self.model = Cls(model_id=model_id, device_mesh=device_mesh, max_loras=max_loras, max_r=max_r, max_length=max_length, **kwargs)
        self.model_id = model_id

    def ping(self) -> bool:
        return True

    def data_world_size(self) -> int:
        return self.model.device_mesh.data_world_size

    def add_adapter_to_model(self, adapter_name: str, config_or_dir=None, **kw) -> None:
        self.model.add_adapter_to_model(adapter_name, config_or_dir or {'r': 8, 'lora_alpha': 16}, **kw)

    def remove_adapter(self, adapter_name: str, **kw) -> None:
        self.model.remove_adapter(adapter_name)

    def tinker_forward_backward(self, datums: List[Dict[str, Any]], adapter_name: str, loss_fn: str = 'cross_entropy', backward: bool = True,
                                loss_fn_config: Optional[Dict[str, Any]] = None) -> Dict[str, Any]:
        feats = [datum_to_input_feature(d, getattr(self.model, 'config', None)) for d in datums]
        self.model.check_length(feats)
        loss = choose_loss(loss_fn, feats, loss_fn_config)
        self.model.set_loss(loss, adapter_name=adapter_name)
        if type(loss).__name__ == 'DPOLoss':
            self._ensure_metric(adapter_name, 'DPOMetric')      # reward margins / accuracies come back with the step's metrics
        kw = split_loss_inputs(feats)
        opts = forward_options(loss_fn_config)
        clean = [{k: v for k, v in f.items() if k in ('input_ids', 'labels', 'position_ids')} for f in feats]
        if backward:
            out = self.model.forward_backward(inputs=clean, adapter_name=adapter_name, **opts, **kw)
        else:
            out = self.model.forward_only(inputs=clean, adapter_name=adapter_name, **opts)
        metrics = self.model.calculate_metric(True, adapter_name=adapter_name) if backward else {}
        if backward:
            # calculating drains the accumulators; the step that follows reports the same window (loss statistics such as
            # the DPO reward margins) together with its own gradient norm
            self._window_metrics = getattr(self, '_window_metrics', {})
            self._window_metrics[adapter_name] = clean_metrics(metrics)
        return build_fwdbwd_output(clean, out, metrics)

    def _ensure_metric(self, adapter_name: str, metric: str) -> None:
        og = self.model._group(adapter_name)
        if not any(type(m).__name__ == metric for m in og.train_status.metrics):
            self.model.add_metric(metric, is_training=True, adapter_name=adapter_name)

    def tinker_step(self, adapter_name: str, adam_params: Optional[Dict[str, Any]] = None) -> Dict[str, Any]:
        og = self.model._group(adapter_name)
        if not og.grad_ready:
            raise RuntimeError('optim_step without a preceding forward_backward')
        p = adam_params or {}
        norm = self.model.clip_grad_norm(p.get('grad_clip_norm', 1.0) or 0.0, adapter_name=adapter_name)
        optim = {k2: p[k1] for k1, k2 in (('learning_rate', 'lr'), ('eps', 'eps'), ('weight_decay', 'weight_decay')) if k1 in p}
        if 'beta1' in p or 'beta2' in p:
            optim['betas'] = (p.get('beta1', 0.9), p.get('beta2', 0.999))
        self.model.step(adapter_name=adapter_name, optim_params=optim)
        self.model.zero_grad(adapter_name=adapter_name)
        self.model.lr_step(adapter_name=adapter_name)
        window = getattr(self, '_window_metrics', {}).pop(adapter_name, {})
        return {'metrics': {**window, 'grad_norm': float(norm), **clean_metrics(self.model.calculate_metric(True, adapter_name=adapter_name))}}

    def save(self, name: str, output_dir: str, adapter_name: Optional[str] = None, **kw) -> str:
        return self.model.save(name, output_dir, adapter_name=adapter_name, **kw)

    def load(self, name: Optional[str], output_dir: str, adapter_name: Optional[str] = None, **kw) -> None:
        self.model.load(name, output_dir, adapter_name=adapter_name, **kw)

    def generic_call(self, method: str, **kwargs) -> Any:
        fn = getattr(self.model, method)
        out = fn(**kwargs)
        import torch
        if isinstance(out, dict):
            return {k: (v.tolist() if torch.is_tensor(v) else v) for k, v in out.items() if k not in ('routed_experts', )}
        return out
