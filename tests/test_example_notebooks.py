"""Every example notebook runs top to bottom on CPU (code cells executed in one namespace, in order)."""

from __future__ import annotations

import json
from pathlib import Path

import pytest

NOTEBOOKS = sorted((Path(__file__).resolve().parents[1] / "examples" / "notebooks").glob("*.ipynb"))


def test_the_six_notebooks_are_present_and_stripped():
    assert [p.name[:2] for p in NOTEBOOKS] == ["01", "02", "03", "04", "05", "06"]
    for path in NOTEBOOKS:
        nb = json.loads(path.read_text())
        assert nb["nbformat"] == 4
        first = "".join(nb["cells"][0]["source"])
        assert all(word in first for word in ("Objectives", "Requirements", "Runtime")), path.name
        assert all(not c.get("outputs") for c in nb["cells"] if c["cell_type"] == "code"), f"{path.name} has stored outputs"


@pytest.mark.parametrize("path", NOTEBOOKS, ids=lambda p: p.stem)
def test_notebook_runs_on_cpu(path, monkeypatch, tmp_path):
    monkeypatch.setenv("CUDA_VISIBLE_DEVICES", "")
    monkeypatch.chdir(path.parent)
    nb = json.loads(path.read_text())
    namespace: dict = {"__name__": "__notebook__"}
    for i, cell in enumerate(nb["cells"]):
        if cell["cell_type"] != "code":
            continue
        source = "".join(cell["source"])
        exec(compile(source, f"{path.name}[cell {i}]", "exec"), namespace)
