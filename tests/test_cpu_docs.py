"""The documentation site builds strictly: every page is in ``nav``, every ``nav`` entry exists, every relative link in a
page points at a file that exists.  (``mkdocs build --strict`` enforces the same in CI; this test needs no mkdocs.)"""

import os
import re

import yaml

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
DOCS = os.path.join(ROOT, "docs")


def _nav_files(node):
    if isinstance(node, str):
        yield node
    elif isinstance(node, list):
        for item in node:
            yield from _nav_files(item)
    elif isinstance(node, dict):
        for value in node.values():
            yield from _nav_files(value)


def _pages():
    for base, _dirs, files in os.walk(DOCS):
        for name in files:
            if name.endswith(".md"):
                yield os.path.relpath(os.path.join(base, name), DOCS)


def test_nav_and_pages_agree():
    with open(os.path.join(ROOT, "mkdocs.yaml")) as f:
        cfg = yaml.safe_load(f)
    assert cfg["strict"] is True and cfg["docs_dir"] == "docs"
    nav = list(_nav_files(cfg["nav"]))
    assert len(nav) == len(set(nav)), "a page is listed twice in nav"
    missing = [p for p in nav if not os.path.isfile(os.path.join(DOCS, p))]
    assert not missing, f"nav entries without a file: {missing}"
    orphans = sorted(set(_pages()) - set(nav))
    assert not orphans, f"pages that are not in nav: {orphans}"


def test_relative_links_resolve():
    link = re.compile(r"\[[^\]]*\]\(([^)\s]+)\)")
    broken = []
    for page in _pages():
        text = open(os.path.join(DOCS, page)).read()
        text = re.sub(r"```.*?```", "", text, flags=re.S)  # code blocks hold example syntax, not links
        for target in link.findall(text):
            if re.match(r"^[a-z]+:", target) or target.startswith("#"):
                continue
            path = os.path.normpath(os.path.join(DOCS, os.path.dirname(page), target.split("#")[0]))
            if not os.path.exists(path):
                broken.append(f"{page} -> {target}")
    assert not broken, f"broken relative links: {broken}"


def test_import_lines_in_code_blocks_resolve():
    """Every ``from rl_engine... import name`` / ``import rl_engine...`` line inside a ``python`` block of the pages and
    of the README names a module and attributes that exist, so a snippet cannot outlive the API it shows."""
    import ast
    import importlib

    pages = [os.path.join(DOCS, page) for page in _pages()] + [os.path.join(ROOT, "README.md")]
    problems, checked = [], 0
    for path in pages:
        with open(path) as f:
            blocks = re.findall(r"```python\n(.*?)```", f.read(), re.S)
        for block in blocks:
            for line in block.splitlines():
                line = line.split("#")[0].strip()
                if not line.startswith(("from rl_engine", "import rl_engine")) or line.endswith("("):
                    continue
                node = ast.parse(line).body[0]
                checked += 1
                if isinstance(node, ast.Import):
                    for alias in node.names:
                        importlib.import_module(alias.name)
                    continue
                module = importlib.import_module(node.module)
                for alias in node.names:
                    if hasattr(module, alias.name):
                        continue
                    try:
                        importlib.import_module(f"{node.module}.{alias.name}")
                    except ImportError:
                        problems.append(f"{os.path.relpath(path, ROOT)}: {node.module} has no {alias.name}")
    assert not problems, problems
    assert checked >= 10
