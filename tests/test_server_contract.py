"""API contract freeze: the four apps of an all-mock server must serve exactly the paths (and methods) recorded in
``tests/fixtures/client_api_baseline.json``. A route that appears or disappears fails this test; after a deliberate
change, regenerate the file with ``python -m tests.test_server_contract`` from the repository root."""
import json
import os

BASELINE = os.path.join(os.path.dirname(os.path.abspath(__file__)), 'fixtures', 'client_api_baseline.json')
PREFIXES = {'gateway': '/api/v1', 'model': '/api/v1/model/mock-base', 'sampler': '/api/v1/sampler/mock-base', 'processor': '/api/v1/processor'}


def current_contract():
    from starlette.routing import Mount
    from twinkle_b200.server.config import ServerConfig
    from twinkle_b200.server.launcher import ServerLauncher
    cfg = ServerConfig(applications=[
        {'name': 'gw', 'route_prefix': PREFIXES['gateway'], 'import_path': 'server', 'args': {}},
        {'name': 'm', 'route_prefix': PREFIXES['model'], 'import_path': 'model', 'args': {'model_id': 'mock-base', 'backend': 'mock'}},
        {'name': 's', 'route_prefix': PREFIXES['sampler'], 'import_path': 'sampler', 'args': {'model_id': 'mock-base', 'sampler_type': 'mock'}},
        {'name': 'p', 'route_prefix': PREFIXES['processor'], 'import_path': 'processor', 'args': {}}])
    root = ServerLauncher(cfg).root
    mounts = {r.path: r.app for r in root.routes if isinstance(r, Mount)}
    out = {}
    for name, prefix in PREFIXES.items():
        routes = {}
        for r in mounts[prefix].routes:
            methods = sorted(m for m in (getattr(r, 'methods', None) or []) if m not in ('HEAD', 'OPTIONS'))
            if methods and not r.path.startswith(('/docs', '/openapi', '/redoc')):
                routes[r.path] = sorted(set(routes.get(r.path, [])) | set(methods))
        out[name] = dict(sorted(routes.items()))
    return out


def test_served_paths_match_the_frozen_contract():
    with open(BASELINE) as f:
        frozen = json.load(f)
    now = current_contract()
    for app in PREFIXES:
        added = sorted(set(now[app]) - set(frozen[app]))
        removed = sorted(set(frozen[app]) - set(now[app]))
        assert not added and not removed, f'{app}: added {added}, removed {removed}'
        changed = {p: (frozen[app][p], now[app][p]) for p in now[app] if frozen[app][p] != now[app][p]}
        assert not changed, f'{app}: methods changed {changed}'


def test_contract_covers_the_protocol_routes():
    """The Tinker-compatible and native routes a client of the reference server relies on."""
    with open(BASELINE) as f:
        frozen = json.load(f)
    gw, model, sampler = set(frozen['gateway']), set(frozen['model']), set(frozen['sampler'])
    assert {'/create_session', '/session_heartbeat', '/create_model', '/forward_backward', '/optim_step', '/retrieve_future', '/asample',
            '/save_weights_for_sampler', '/chat/completions', '/models', '/healthz', '/training_runs', '/weights_info',
            '/twinkle/capacity_info', '/twinkle/healthz/deep'} <= gw
    assert {'/tinker/forward_backward', '/tinker/optim_step', '/twinkle/forward_backward', '/twinkle/clip_grad_and_step', '/twinkle/save',
            '/twinkle/load', '/twinkle/add_adapter_to_model', '/twinkle/get_state_dict', '/twinkle/upload_to_hub', '/healthz'} <= model
    assert {'/tinker/asample', '/twinkle/sample', '/twinkle/sample_stream', '/twinkle/set_template', '/twinkle/add_adapter_to_sampler'} <= sampler


if __name__ == '__main__':
    os.makedirs(os.path.dirname(BASELINE), exist_ok=True)
    with open(BASELINE, 'w') as f:
        json.dump(current_contract(), f, indent=1)
    print('wrote', BASELINE)
