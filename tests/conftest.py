"""pytest configuration: the ``gpu`` marker and shared fixture helpers."""

from __future__ import annotations

import sys
from pathlib import Path

import numpy as np
import pytest

ROOT = Path(__file__).resolve().parent.parent
GOLDEN = ROOT / "tests" / "golden"
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


def pytest_collection_modifyitems(config, items):
    import torch

    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


ATTENTION_GOLDEN = sorted(p.stem[len("attention_"):] for p in GOLDEN.glob("attention_*.npz"))


def load_attention_golden(name: str) -> dict:
    """Load one ``tests/golden/attention_<name>.npz`` into tensors + meta dict."""

    import torch

    raw = np.load(GOLDEN / f"attention_{name}.npz")
    meta = raw["meta"].tolist()
    keys = ("hidden", "heads", "d", "buckets", "max_pos", "share", "rel", "c2p", "p2c")
    case = dict(zip(keys, meta))
    types = tuple(t for t in ("c2p", "p2c") if case[t])
    params = {k[len("param/"):]: torch.from_numpy(raw[k]) for k in raw.files if k.startswith("param/")}
    return dict(
        case=case,
        types=types,
        params=params,
        hidden_states=torch.from_numpy(raw["hidden"]),
        rel_embeddings=torch.from_numpy(raw["rel_embeddings"]),
        mask=torch.from_numpy(raw["mask"]),
        ctx_original=torch.from_numpy(raw["ctx_original"]),
        ctx_torch=torch.from_numpy(raw["ctx_torch"]),
    )


@pytest.fixture(scope="session")
def position_golden():
    return np.load(GOLDEN / "position_plans.npz")
