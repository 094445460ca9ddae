"""The documentation names things that exist: relative links resolve, `python -m kern_b200 <command>` names a command of
the CLI, `python -m kern_b200.<module>` names a module, and paths in backticks that look like files of this tree are there."""
import importlib.util
import re
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parents[1]
PAGES = sorted((ROOT / "docs").glob("*.md")) + [ROOT / "README.md"]
COMMANDS = {"verify", "cut", "kernels", "schema", "gate", "run", "test", "bench", "workload", "server", "e2e-logits", "capture"}


@pytest.mark.parametrize("page", PAGES, ids=lambda p: p.name)
def test_page_names_things_that_exist(page):
    text = page.read_text()
    for target in re.findall(r"\]\(([^)#]+)(?:#[^)]*)?\)", text):
        if "://" not in target:
            assert (page.parent / target).exists(), f"{page.name}: link to {target}"
    for cmd in re.findall(r"python -m kern_b200 ([a-z0-9-]+)", text) + re.findall(r"`kern ([a-z0-9-]+)[ `]", text):
        assert cmd in COMMANDS, f"{page.name}: `kern {cmd}` is not a command"
    for mod in re.findall(r"python -m (kern_b200(?:\.\w+)+)", text):
        assert importlib.util.find_spec(mod) is not None, f"{page.name}: module {mod}"
    for path in re.findall(r"`((?:kern_b200|csrc|tests|examples|schema|profiles|kernel_index)/[\w./\-]+\.(?:py|cpp|hpp|cu|cuh|json|toml|md|jsonl))`", text):
        if "<" in path or "*" in path:
            continue
        assert (ROOT / path).exists(), f"{page.name}: {path}"
