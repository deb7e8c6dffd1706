"""The real training backend behind the Model app: the multi-LoRA engine plus the Tinker-shaped methods.

Parity: reference ``src/twinkle/server/model/backends/transformers_model.py:22-112`` and
``common.py:125-362`` (``tinker_forward_only``, ``tinker_forward_backward``, ``tinker_step``,
``tinker_calculate_metric``, ``tinker_load``, ``ping``).
"""
from __future__ import annotations

from typing import Any, Dict, List, Optional

from ...infra import collect_results, dispatch_args, remote_class, remote_function
from ...utils.device_mesh import DeviceMesh
from . import build_fwdbwd_output, choose_loss, clean_metrics, datum_to_input_feature, forward_options, split_loss_inputs


def _collect_fwdbwd(results: List[Dict[str, Any]], device_mesh: Optional[DeviceMesh] = None) -> Dict[str, Any]:
    """Per-datum outputs of the data-parallel workers back in request order; sums add up, other metrics average.
    Sequence / tensor / pipeline peers of a data rank return the same rows, so only the mesh's collect ranks count."""
    if device_mesh is not None and len(results) > 1:
        keep = set(device_mesh.get_collect_ranks())
        results = [r for i, r in enumerate(results) if i in keep] or results
    results = [r for r in results if r]
    out = dict(results[0])
    if len(results) > 1:
        out['loss_fn_outputs'] = [x for r in results for x in r.get('loss_fn_outputs', [])]
        metrics: Dict[str, Any] = {}
        for k in results[0].get('metrics', {}):
            vals = [float(r['metrics'][k]) for r in results if k in r.get('metrics', {})]
            metrics[k] = sum(vals) if k.endswith(':sum') else sum(vals) / len(vals)
        out['metrics'] = metrics
    return out


def _generic_dispatch(n_workers: int, args: tuple, kwargs: dict, device_mesh: Optional[DeviceMesh] = None):
    """``generic_call(method, **kw)`` is cut the way ``method`` itself asks for (``forward_backward`` slices its inputs
    over the data ranks, ``set_optimizer`` goes to every worker unchanged …)."""
    from ...model import MultiLoraTransformersModel
    method = args[0] if args else kwargs.get('method')
    spec = getattr(getattr(MultiLoraTransformersModel, str(method), None), '_remote_spec', None) or {}
    rule = spec.get('dispatch', 'all')
    if rule == 'all' or device_mesh is None:
        return [(args, kwargs) for _ in range(n_workers)]
    rest = {k: v for k, v in kwargs.items() if k != 'method'}
    per = dispatch_args(rule, n_workers, (), rest, device_mesh=device_mesh)
    return [(args, dict(kw, **({'method': kwargs['method']} if 'method' in kwargs else {}))) for _, kw in per]


def _generic_collect(results: List[Any], device_mesh: Optional[DeviceMesh] = None):
    from ...model import MultiLoraTransformersModel
    method = results[0][0]
    spec = getattr(getattr(MultiLoraTransformersModel, str(method), None), '_remote_spec', None) or {}
    rule = spec.get('collect', 'first')
    vals = [r[1] for r in results]
    if rule == 'none':
        rule = 'first'
    merged = collect_results(rule, vals, device_mesh, list(range(len(vals)))) if not callable(rule) else rule(
        vals, device_mesh=device_mesh, worker_ranks=list(range(len(vals))))
    return _plain(merged)


def _plain(out):
    import torch
    if isinstance(out, dict):
        return {k: (v.tolist() if torch.is_tensor(v) else v) for k, v in out.items() if k not in ('routed_experts', )}
    return out


@remote_class()
class NativeModelBackend:
    """In-process when the application's device group has one rank; with ``remote_group=`` (pool mode) one instance
    lives in every worker of the group and this object is the driver-side proxy: datums are cut over the data ranks,
    every worker joins every collective, per-datum results come back in request order (reference
    ``src/twinkle/server/model/app.py:50-234`` builds the backend as ``@remote_class`` workers on the configured device
    group)."""

    def __init__(self, kind: str = 'transformers', model_id: str = 'tiny-dense', device_mesh: Optional[DeviceMesh] = None, max_loras: int = 5,
                 max_r: int = 32, max_length: int = 8192, **kwargs):
        if kind == 'megatron':
            from ...model.megatron import MultiLoraMegatronModel as Cls
        else:
            from ...model import MultiLoraTransformersModel as Cls
        self.model = Cls(model_id=model_id, device_mesh=device_mesh, max_loras=max_loras, max_r=max_r, max_length=max_length, **kwargs)
        self.model_id = model_id

    @remote_function(collect='first', sync=True, timeout=30.0)
    def ping(self) -> bool:
        return True

    @remote_function(collect='first', sync=True)
    def data_world_size(self) -> int:
        return self.model.device_mesh.data_world_size

    @remote_function(collect='first', sync=True)
    def add_adapter_to_model(self, adapter_name: str, config_or_dir=None, **kw) -> None:
        self.model.add_adapter_to_model(adapter_name, config_or_dir or {'r': 8, 'lora_alpha': 16}, **kw)

    @remote_function(collect='first', sync=True)
    def remove_adapter(self, adapter_name: str, **kw) -> None:
        self.model.remove_adapter(adapter_name)

    @remote_function(dispatch='slice_dp', collect=_collect_fwdbwd, sync=True)
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

    @remote_function(collect='first', sync=True)
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

    @remote_function(collect='first', sync=True)
    def save(self, name: str, output_dir: str, adapter_name: Optional[str] = None, **kw) -> str:
        return self.model.save(name, output_dir, adapter_name=adapter_name, **kw)

    @remote_function(collect='first', sync=True)
    def load(self, name: Optional[str], output_dir: str, adapter_name: Optional[str] = None, **kw) -> None:
        self.model.load(name, output_dir, adapter_name=adapter_name, **kw)

    def generic_call(self, method: str, **kwargs) -> Any:
        if getattr(self, '_remote_proxy', None) is None:
            return _plain(getattr(self.model, method)(**kwargs))
        return self._generic_remote(method, **kwargs)

    @remote_function(dispatch=_generic_dispatch, collect=_generic_collect, sync=True)
    def _generic_remote(self, method: str, **kwargs):
        return method, getattr(self.model, method)(**kwargs)
