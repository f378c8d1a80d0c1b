"""Shared fixtures.  GPU tests carry the ``gpu`` marker; everything else runs on the CPU."""

from __future__ import annotations

import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT))
sys.path.insert(0, str(ROOT / "tests"))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on the GPU box)")


def pytest_collection_modifyitems(config, items):
    import torch

    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


@pytest.fixture(scope="session")
def model_folders(tmp_path_factory):
    """Tiny model folders (random weights, made by the plain implementation's own writer)."""
    import torch

    import plain_llama as plain

    base = tmp_path_factory.mktemp("models")
    made = {}

    def get(which: str, dtype: str = "float32", std: float | None = None) -> Path:
        key = (which, dtype, std)
        if key not in made:
            raw, seed, default_std = {"a": (plain.TINY_A, 0, 0.05), "b": (plain.TINY_B, 1, 0.08)}[which]
            made[key] = plain.write_model_folder(
                base / f"tiny_{which}_{dtype}_{std}", raw, seed, std=std or default_std,
                dtype={"float32": torch.float32, "bfloat16": torch.bfloat16}[dtype])
        return made[key]

    return get
