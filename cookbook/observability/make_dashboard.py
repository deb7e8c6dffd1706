"""Writes ``grafana/dashboards/twinkle-overview.json`` from the panel table below (run after changing it):

    python cookbook/observability/make_dashboard.py

Every expression uses the metric names the server exposes at ``GET /metrics`` (Prometheus text format)."""
import json
import os

PANELS = [
    # title, unit, [(legend, expr)]
    ('HTTP requests / s by app', 'reqps', [('{{app}}', 'sum by (app) (rate(twinkle_http_requests_total[1m]))')]),
    ('HTTP errors / s by status', 'reqps', [('{{status}}', 'sum by (status) (rate(twinkle_http_requests_total{status=~"4..|5.."}[1m]))')]),
    ('HTTP latency p90 by app', 's', [('{{app}}', 'twinkle_http_request_seconds{quantile="0.9"}')]),
    ('Active resources (cleanup leader)', 'short', [(k, f'max(twinkle_active_{k})') for k in ('sessions', 'models', 'sampling_sessions', 'futures')]),
    ('Task queue depth', 'short', [('depth', 'max(twinkle_queue_depth)')]),
    ('Task execution / wait p90', 's', [('execution', 'twinkle_task_execution_seconds{quantile="0.9"}'), ('wait', 'twinkle_task_wait_seconds{quantile="0.9"}')]),
    ('Tasks finished / s by status', 'ops', [('{{status}}', 'sum by (status) (rate(twinkle_tasks_total[1m]))')]),
    ('Rate-limit rejections / s', 'ops', [('rejected', 'sum(rate(twinkle_rate_limit_rejections_total[1m]))')]),
    ('GPU utilisation', 'percent', [('gpu {{gpu}}', 'twinkle_gpu_utilization')]),
    ('GPU memory used', 'bytes', [('gpu {{gpu}}', 'twinkle_gpu_memory_used_bytes')]),
    ('Host CPU / memory', 'percent', [('cpu', 'twinkle_host_cpu_percent'), ('memory', 'twinkle_host_memory_percent')]),
    ('Client telemetry events / s', 'ops', [('events', 'sum(rate(twinkle_client_telemetry_events_total[1m]))')]),
]


def dashboard():
    panels = []
    for i, (title, unit, targets) in enumerate(PANELS):
        panels.append({
            'id': i + 1, 'type': 'timeseries', 'title': title, 'datasource': {'type': 'prometheus', 'uid': 'twinkle-prometheus'},
            'gridPos': {'h': 8, 'w': 12, 'x': 12 * (i % 2), 'y': 8 * (i // 2)},
            'fieldConfig': {'defaults': {'unit': unit}, 'overrides': []},
            'targets': [{'refId': chr(ord('A') + j), 'expr': expr, 'legendFormat': legend} for j, (legend, expr) in enumerate(targets)],
        })
    return {'uid': 'twinkle-overview', 'title': 'Twinkle server overview', 'tags': ['twinkle'], 'timezone': 'browser', 'schemaVersion': 39,
            'version': 1, 'refresh': '10s', 'time': {'from': 'now-30m', 'to': 'now'}, 'panels': panels}


if __name__ == '__main__':
    out = os.path.join(os.path.dirname(os.path.abspath(__file__)), 'grafana', 'dashboards', 'twinkle-overview.json')
    with open(out, 'w') as f:
        json.dump(dashboard(), f, indent=1)
    print('wrote', out)
