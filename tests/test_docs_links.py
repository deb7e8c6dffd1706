"""Relative links and file references in the user-facing Markdown resolve (reference ``tests/docs/test_markdown_links.py``)."""
import os
import re

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
PAGES = ['README.md', 'cookbook/README.md', 'cookbook/observability/README.md'] + sorted(
    os.path.join('docs', f) for f in os.listdir(os.path.join(ROOT, 'docs')) if f.endswith('.md'))
LINK = re.compile(r'\[[^\]]*\]\(([^)#\s]+)(?:#[^)]*)?\)')


def test_relative_links_point_at_files():
    bad = []
    for page in PAGES:
        path = os.path.join(ROOT, page)
        if not os.path.isfile(path):
            continue
        text = open(path).read()
        for target in LINK.findall(text):
            if re.match(r'^[a-z]+://|^mailto:', target):
                continue
            if not os.path.exists(os.path.normpath(os.path.join(os.path.dirname(path), target))):
                bad.append((page, target))
    assert not bad, bad


def test_cookbook_table_lists_every_script_and_only_scripts_that_exist():
    text = open(os.path.join(ROOT, 'cookbook', 'README.md')).read()
    listed = set(re.findall(r'^\| `([a-z0-9_]+\.py)` \|', text, flags=re.M))
    present = {f for f in os.listdir(os.path.join(ROOT, 'cookbook')) if f.endswith('.py')}
    assert listed == present, (sorted(listed - present), sorted(present - listed))


def test_docs_index_lists_every_page():
    text = open(os.path.join(ROOT, 'docs', 'index.md')).read()
    pages = {f for f in os.listdir(os.path.join(ROOT, 'docs')) if f.endswith('.md') and f != 'index.md'}
    assert pages == set(re.findall(r'\]\(([a-z0-9-]+\.md)\)', text)), pages
