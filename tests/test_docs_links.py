"""Relative links and referenced source paths in the user-facing Markdown files must exist."""
import glob
import os
import re

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
DOCS = ['README.md', 'cookbook/README.md', 'cookbook/observability/README.md'] + sorted(
    os.path.relpath(p, ROOT) for p in glob.glob(os.path.join(ROOT, 'docs', '**', '*.md'), recursive=True))
LINK = re.compile(r'\[[^\]]*\]\(([^)#\s]+)(?:#[^)]*)?\)')


def test_relative_markdown_links_resolve():
    broken = []
    for doc in DOCS:
        path = os.path.join(ROOT, doc)
        if not os.path.exists(path):
            continue
        text = open(path, encoding='utf-8').read()
        for target in LINK.findall(text):
            if re.match(r'^[a-z]+://|^mailto:', target):
                continue
            if not os.path.exists(os.path.normpath(os.path.join(os.path.dirname(path), target))):
                broken.append(f'{doc}: {target}')
    assert not broken, broken


def test_cookbook_readme_lists_every_script():
    text = open(os.path.join(ROOT, 'cookbook', 'README.md'), encoding='utf-8').read()
    scripts = sorted(os.path.basename(p) for p in glob.glob(os.path.join(ROOT, 'cookbook', '*.py')))
    missing = [s for s in scripts if s not in text]
    assert not missing, f'cookbook/README.md does not mention {missing}'
