"""OTLP over HTTP with JSON bodies (``POST <endpoint>/v1/metrics`` and ``/v1/traces``) for the in-process metrics registry
and span buffer — what an OpenTelemetry collector accepts on port 4318 — written on the standard protocol's JSON mapping so
that no OpenTelemetry SDK is needed. Counters go out as monotonic cumulative sums, gauges as gauges, the value series as
summaries (count, sum, quantiles). A span is sent once.

Parity: reference ``src/twinkle/server/telemetry/*`` exports through the OpenTelemetry SDK's OTLP exporter
(``telemetry.otlp_endpoint`` in the server config); the same config key switches this exporter on."""
from __future__ import annotations

import threading
import time
from typing import Any, Callable, Dict, List, Optional, Tuple


def _attrs(labels) -> List[Dict[str, Any]]:
    out = []
    for k, v in (labels.items() if isinstance(labels, dict) else labels):
        if isinstance(v, bool):
            val = {'boolValue': v}
        elif isinstance(v, int):
            val = {'intValue': str(v)}
        elif isinstance(v, float):
            val = {'doubleValue': v}
        else:
            val = {'stringValue': str(v)}
        out.append({'key': str(k), 'value': val})
    return out


def _nanos(t: float) -> str:
    return str(int(t * 1e9))


class OTLPExporter:

    def __init__(self, endpoint: str, service_name: str = 'twinkle-server', post: Optional[Callable[[str, Dict[str, Any]], Any]] = None,
                 timeout: float = 5.0, headers: Optional[Dict[str, str]] = None):
        ep = endpoint.rstrip('/')
        if ep.endswith(':4317'):  # the gRPC port of a collector: its HTTP receiver listens next door
            ep = ep[:-5] + ':4318'
        self.endpoint, self.timeout, self.headers = ep, timeout, dict(headers or {})
        self.resource = {'attributes': _attrs({'service.name': service_name})}
        self._post = post or self._http_post
        self._start = time.time()
        self._sent_spans: set = set()
        self.failures = 0

    def _http_post(self, url: str, body: Dict[str, Any]) -> None:
        import requests
        requests.post(url, json=body, headers={'Content-Type': 'application/json', **self.headers}, timeout=self.timeout).raise_for_status()

    # ------------------------------------------------------------------ metrics
    def metrics_payload(self, registry) -> Dict[str, Any]:
        now, start = _nanos(time.time()), _nanos(self._start)
        by_name: Dict[Tuple[str, str], List[Dict[str, Any]]] = {}
        with registry._lock:
            counters, gauges = dict(registry.counters), dict(registry.gauges)
            hist = {k: list(v) for k, v in registry.hist.items() if v}
        for (name, labels), v in counters.items():
            by_name.setdefault((name, 'sum'), []).append({'attributes': _attrs(labels), 'startTimeUnixNano': start, 'timeUnixNano': now, 'asDouble': float(v)})
        for (name, labels), v in gauges.items():
            by_name.setdefault((name, 'gauge'), []).append({'attributes': _attrs(labels), 'timeUnixNano': now, 'asDouble': float(v)})
        for (name, labels), vals in hist.items():
            s = sorted(vals)
            by_name.setdefault((name, 'summary'), []).append({
                'attributes': _attrs(labels), 'startTimeUnixNano': start, 'timeUnixNano': now, 'count': str(len(s)), 'sum': float(sum(s)),
                'quantileValues': [{'quantile': q, 'value': s[min(int(q * len(s)), len(s) - 1)]} for q in (0.5, 0.9, 0.99)]})
        metrics = []
        for (name, kind), points in sorted(by_name.items()):
            if kind == 'sum':
                metrics.append({'name': name, 'sum': {'dataPoints': points, 'aggregationTemporality': 2, 'isMonotonic': True}})
            elif kind == 'gauge':
                metrics.append({'name': name, 'gauge': {'dataPoints': points}})
            else:
                metrics.append({'name': name, 'unit': 's', 'summary': {'dataPoints': points}})
        return {'resourceMetrics': [{'resource': self.resource, 'scopeMetrics': [{'scope': {'name': 'twinkle_b200.server'}, 'metrics': metrics}]}]}

    # ------------------------------------------------------------------- traces
    def traces_payload(self, spans) -> Tuple[Dict[str, Any], List[str]]:
        out, ids = [], []
        for s in list(spans):
            if s['span_id'] in self._sent_spans or 'duration_s' not in s:
                continue
            trace = ''.join(c for c in str(s['trace_id']) if c in '0123456789abcdef')[:32].rjust(32, '0')
            rec = {'traceId': trace, 'spanId': s['span_id'][:16].rjust(16, '0'), 'name': s['name'], 'kind': 2,
                   'startTimeUnixNano': _nanos(s['start']), 'endTimeUnixNano': _nanos(s['start'] + s['duration_s']),
                   'attributes': _attrs(s.get('attributes') or {}),
                   'status': {'code': 2, 'message': s.get('error', '')} if s.get('status') == 'error' else {'code': 1}}
            out.append(rec)
            ids.append(s['span_id'])
        return {'resourceSpans': [{'resource': self.resource, 'scopeSpans': [{'scope': {'name': 'twinkle_b200.server'}, 'spans': out}]}]}, ids

    # ------------------------------------------------------------------- export
    def export(self, registry=None, tracer=None) -> bool:
        """One push of everything new; returns False (and counts a failure) when the collector cannot be reached —
        telemetry never takes the server down."""
        ok = True
        try:
            if registry is not None:
                self._post(self.endpoint + '/v1/metrics', self.metrics_payload(registry))
            if tracer is not None:
                body, ids = self.traces_payload(tracer.spans)
                if ids:
                    self._post(self.endpoint + '/v1/traces', body)
                    self._sent_spans.update(ids)
                    if len(self._sent_spans) > 4 * (tracer.spans.maxlen or 2048):  # forget ids that left the ring buffer
                        self._sent_spans &= {s['span_id'] for s in tracer.spans}
        except Exception:
            self.failures += 1
            ok = False
        return ok

    def start(self, registry, tracer, interval_s: float = 15.0) -> threading.Event:
        """Background pushes every ``interval_s`` until the returned event is set (one last push follows)."""
        stop = threading.Event()

        def loop():
            while not stop.wait(interval_s):
                self.export(registry, tracer)
            self.export(registry, tracer)

        threading.Thread(target=loop, name='otlp-export', daemon=True).start()
        return stop
