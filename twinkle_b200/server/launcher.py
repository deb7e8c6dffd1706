"""Builds and runs the whole server from a ``ServerConfig``.

Parity: reference ``src/twinkle/server/launcher/server_launcher.py:30-319`` (+ ``builder_registry``,
``env_propagation``) and ``server/cli/app.py`` (``twinkle-server launch | check-config | print-config |
clear persistence``).  The reference starts Ray Serve and one deployment per application; this launcher
builds one FastAPI root application, mounts every configured application at its ``route_prefix``
(``…/model/<base_model>``, ``…/sampler/<base_model>``, ``…/processor``), starts the lifecycle loop
(heart-beat expiry, leader lease renewal, resource gauges) and serves with uvicorn until SIGINT / SIGTERM.
"""
from __future__ import annotations

import argparse
import asyncio
import contextlib
import os
import signal
import sys
from typing import Any, Dict, List, Optional, Union

from fastapi import FastAPI

from .apps import ModelApp, ProcessorApp, SamplerApp
from .apps.gateway import GatewayApp, Router
from .checkpoint import CheckpointManager
from .config import ServerConfig
from .state import LEASE_RENEW, ServerState, build_backend
from .telemetry import ResourceMetricsCollector, get_registry


class ServerLauncher:

    def __init__(self, config: Union[ServerConfig, str, Dict[str, Any]]):
        if isinstance(config, str):
            config = ServerConfig.from_yaml(config)
        elif isinstance(config, dict):
            config = ServerConfig(**config)
        self.config = config
        self.state = ServerState(build_backend(config.persistence))
        self.checkpoints = CheckpointManager()
        self.router = Router()
        self.root = FastAPI(title='twinkle-b200-server', lifespan=self._lifespan)
        self.model_apps: List[ModelApp] = []
        self.sampler_apps: List[SamplerApp] = []
        self.processor_apps: List[ProcessorApp] = []
        self.gateway: Optional[GatewayApp] = None
        self._lifecycle_task: Optional[asyncio.Task] = None
        self._export_env()
        self._build()

    def _export_env(self) -> None:
        """Worker processes rebuild persistence / telemetry from the environment."""
        p = self.config.persistence
        os.environ['TWINKLE_PERSISTENCE_MODE'] = p.mode
        if p.file_path:
            os.environ['TWINKLE_PERSISTENCE_FILE'] = p.file_path
        os.environ['TWINKLE_TELEMETRY_ENABLED'] = '1' if self.config.telemetry.enabled else '0'
        os.environ.setdefault('TWINKLE_FAIL_FAST', '0')  # a bad request must not wedge the collectives of the model workers

    def _worker_groups(self) -> Dict[str, Any]:
        """Applications whose ``device_group`` has more than one rank (or that ask for ``workers: pool``) get a group of
        worker processes — one per rank, devices assigned by the group's position — and their backend is built there
        (reference ``src/twinkle/server/model/app.py:50-234``, ``server/utils/device_utils.py:1-40``).  Returns
        application name → ``DeviceGroup``; starts the pool when there is at least one."""
        from ..utils.device_mesh import DeviceGroup
        groups: Dict[str, Any] = {}
        for spec in self.config.applications:
            if spec.import_path not in ('model', 'sampler'):
                continue
            a = spec.typed_args
            if getattr(a, 'backend', getattr(a, 'sampler_type', '')) == 'mock':
                continue
            g = a.device_group
            n = g.ranks if isinstance(g.ranks, int) else len(g.ranks)
            mode = getattr(a, 'workers', 'auto')
            if mode == 'inline' or (mode == 'auto' and n <= 1):
                continue
            mesh_world = a.device_mesh.build().world_size
            if mesh_world != n // max(g.gpus_per_worker, 1):
                raise ValueError(f"application '{spec.name}': device_mesh spans {mesh_world} ranks but device_group has "
                                 f'{n} ranks / {g.gpus_per_worker} per worker')
            groups[spec.name] = DeviceGroup(name=f'{spec.name}', ranks=g.ranks, device_type=g.device_type, gpus_per_worker=g.gpus_per_worker)
        if groups:
            from .. import infra
            if infra.get_mode() == 'pool':
                raise RuntimeError('a worker pool is already running in this process; the server starts its own')
            infra.initialize(mode='pool', groups=list(groups.values()), lazy_collect=False)
            self._owns_pool = True
        return groups

    def _build(self) -> None:
        gateway_spec = None
        self._owns_pool = False
        groups = self._worker_groups()
        for spec in self.config.applications:
            a = spec.typed_args
            rg = spec.name if spec.name in groups else None
            if spec.import_path == 'model':
                m = ModelApp(a, self.state, self.config.task_queue, self.checkpoints, spec.name, remote_group=rg)
                self.model_apps.append(m)
                self.router.add_model(m)
                self.root.mount(spec.route_prefix.rstrip('/'), m.app)
            elif spec.import_path == 'sampler':
                s = SamplerApp(a, self.state, self.config.task_queue, self.checkpoints, spec.name, remote_group=rg)
                self.sampler_apps.append(s)
                self.router.add_sampler(s)
                self.root.mount(spec.route_prefix.rstrip('/'), s.app)
            elif spec.import_path == 'processor':
                p = ProcessorApp(a, self.state, spec.name)
                self.processor_apps.append(p)
                self.root.mount(spec.route_prefix.rstrip('/'), p.app)
            else:
                gateway_spec = spec
        if gateway_spec is not None:
            self.state.per_token_model_limit = gateway_spec.typed_args.per_token_model_limit
            self.gateway = GatewayApp(gateway_spec.typed_args, self.state, self.checkpoints, self.router, gateway_spec.name)
            prefix = gateway_spec.route_prefix.rstrip('/')
            self.root.mount(prefix or '/', self.gateway.app)

        self._otlp_stop = None

    @contextlib.asynccontextmanager
    async def _lifespan(self, app):
        """Start-up: the lifecycle loop and, when configured, the OTLP exporter. Shut-down: stop both, push what is left,
        give up the cleanup lease."""
        self._lifecycle_task = asyncio.get_event_loop().create_task(self._lifecycle())
        t = self.config.telemetry
        if t.enabled and t.otlp_endpoint and not t.debug:
            from .telemetry import get_tracer
            from .telemetry.otlp import OTLPExporter
            self._otlp_stop = OTLPExporter(t.otlp_endpoint, t.service_name).start(get_registry(), get_tracer(), t.metrics_interval_s)
        try:
            yield
        finally:
            if self._lifecycle_task:
                self._lifecycle_task.cancel()
            if self._otlp_stop is not None:
                self._otlp_stop.set()  # one last push of metrics and spans
            self.state.release_leadership()

    async def _lifecycle(self) -> None:
        """10-second countdown loop: expire adapters / processors whose session went silent, renew the
        cleanup lease, sweep (leader only), publish gauges."""
        collector = ResourceMetricsCollector(get_registry())
        timeout = self.gateway.args.session_timeout if self.gateway else 1800.0
        while True:
            try:
                for m in self.model_apps:
                    m.expire_adapters()
                for p in self.processor_apps:
                    p.expire(timeout)
                if self.state.try_acquire_leadership():
                    self.state.sweep(timeout)
                    for k, v in self.state.gauges().items():
                        get_registry().set_gauge(f'twinkle_active_{k}', v)
                collector.collect()
            except Exception:
                pass
            await asyncio.sleep(LEASE_RENEW)

    def launch(self, block: bool = True) -> None:
        import uvicorn
        # images in requests of a served instance: inline data only, unless the operator widens it (no file reads or URL
        # fetches on a tenant's behalf); in-process use of the launcher leaves the process environment alone
        os.environ.setdefault('TWINKLE_MM_SOURCES', 'data')
        h = self.config.http_options
        cfg = uvicorn.Config(self.root, host=h.host, port=h.port, log_level='warning')
        server = uvicorn.Server(cfg)
        if block:
            server.run()
        else:
            import threading
            t = threading.Thread(target=server.run, daemon=True)
            t.start()
            self._server, self._thread = server, t

    def shutdown(self) -> None:
        s = getattr(self, '_server', None)
        if s is not None:
            s.should_exit = True
            self._thread.join(timeout=10)
        if getattr(self, '_owns_pool', False):
            from .. import infra
            infra.shutdown()
            self._owns_pool = False


def launch_server(config: Union[ServerConfig, Dict[str, Any], None] = None, config_path: Optional[str] = None, block: bool = True) -> ServerLauncher:
    launcher = ServerLauncher(config if config is not None else config_path)
    launcher.launch(block)
    return launcher


def main(argv: Optional[List[str]] = None) -> int:
    ap = argparse.ArgumentParser(prog='twinkle-server')
    sub = ap.add_subparsers(dest='cmd', required=True)
    for name in ('launch', 'check-config', 'print-config'):
        sp = sub.add_parser(name)
        sp.add_argument('--config', '-c', required=True)
    clr = sub.add_parser('clear')
    clr.add_argument('what', choices=['persistence'])
    clr.add_argument('--config', '-c', required=True)
    a = ap.parse_args(argv)
    try:
        cfg = ServerConfig.from_yaml(a.config)
    except Exception as e:
        print(f'invalid config: {e}', file=sys.stderr)
        return 2
    if a.cmd == 'check-config':
        print('config ok:', len(cfg.applications), 'applications')
        return 0
    if a.cmd == 'print-config':
        print(cfg.to_yaml())
        return 0
    if a.cmd == 'clear':
        if cfg.persistence.mode == 'file' and os.path.exists(cfg.persistence.file_path):
            os.remove(cfg.persistence.file_path)
        print('persistence cleared')
        return 0
    launch_server(cfg)
    return 0


if __name__ == '__main__':
    sys.exit(main())
