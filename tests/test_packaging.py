"""Entry points named in pyproject.toml resolve, and the server CLI validates / prints a config."""
import importlib
import tomllib

import yaml


def test_console_scripts_resolve(tmp_path, capsys):
    with open('pyproject.toml', 'rb') as f:
        meta = tomllib.load(f)
    for target in meta['project']['scripts'].values():
        mod, fn = target.split(':')
        assert callable(getattr(importlib.import_module(mod), fn))
    cfg = {'applications': [{'name': 'gateway', 'route_prefix': '/', 'import_path': 'server', 'args': {'supported_models': ['mock-base']}},
                            {'name': 'model', 'route_prefix': '/model/mock-base', 'import_path': 'model', 'args': {'model_id': 'mock-base', 'backend': 'mock'}}]}
    p = tmp_path / 'server.yaml'
    p.write_text(yaml.safe_dump(cfg))
    from twinkle_b200.server.launcher import main
    assert main(['check-config', '-c', str(p)]) == 0
    assert main(['print-config', '-c', str(p)]) == 0
    assert 'mock-base' in capsys.readouterr().out
    bad = tmp_path / 'bad.yaml'
    bad.write_text(yaml.safe_dump({'applications': [], 'no_such_key': 1}))
    assert main(['check-config', '-c', str(bad)]) == 2
