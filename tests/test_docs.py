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
