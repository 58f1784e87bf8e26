"""The Python snippets of the tutorials run as written (CPU)."""
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
RUNNABLE = ["docs/tutorials/working_with_tensors.md", "docs/tutorials/write_first_model.md"]


def _blocks(path):
    text = open(os.path.join(ROOT, path)).read()
    return re.findall(r"```python\n(.*?)```", text, re.S)


@pytest.mark.parametrize("path", RUNNABLE)
def test_tutorial_snippets_run(path, tmp_path, monkeypatch):
    blocks = _blocks(path)
    assert blocks, path
    monkeypatch.chdir(tmp_path)
    for i, code in enumerate(blocks):
        try:
            exec(compile(code, f"{path}[{i}]", "exec"), {"__name__": "__docs__"})
        except Exception as e:      # noqa: BLE001
            raise AssertionError(f"{path}, block {i}: {type(e).__name__}: {e}\n{code}") from e


def test_every_dotted_name_in_the_docs_resolves():
    """`zml_b200.a.b.c` written anywhere in the docs or the README names something that exists."""
    import importlib
    import re
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    pages = [os.path.join(root, "README.md")]
    for d, _, fs in os.walk(os.path.join(root, "docs")):
        pages += [os.path.join(d, f) for f in fs if f.endswith(".md")]
    for d, _, fs in os.walk(os.path.join(root, "examples")):
        pages += [os.path.join(d, f) for f in fs if f.endswith(".md")]
    missing = []
    for page in pages:
        for name in sorted(set(re.findall(r"\bzml_b200(?:\.[A-Za-z_][A-Za-z0-9_]*)+", open(page).read()))):
            parts = name.split(".")
            obj, i = None, len(parts)
            while i > 0 and obj is None:                     # the longest importable module prefix
                try:
                    obj = importlib.import_module(".".join(parts[:i]))
                except ImportError:
                    i -= 1
            for attr in parts[i:]:
                if attr in ("py", "md", "so"):               # a file name, e.g. zml_b200.vfs.py never appears; guard anyway
                    break
                if not hasattr(obj, attr):
                    missing.append(f"{os.path.relpath(page, root)}: {name}")
                    break
                obj = getattr(obj, attr)
    assert not missing, "\n".join(missing)
