"""Host-side helpers of ``bench.py``: the executed-tile fraction that scales the counted FLOPs of the attention
kernel must mirror the kernel's rule (128 x 128 tiles; fully padded query tiles take no tile; a query tile without a
padded row walks the key tiles between the first and the last kept key; a mixed query tile walks every key tile)."""

import importlib.util
import sys
from pathlib import Path

import torch

ROOT = Path(__file__).resolve().parent.parent


def _bench():
    spec = importlib.util.spec_from_file_location("bench_under_test", ROOT / "bench.py")
    module = importlib.util.module_from_spec(spec)
    argv, sys.argv = sys.argv, ["bench.py"]
    try:
        spec.loader.exec_module(module)
    finally:
        sys.argv = argv
    return module


def test_executed_tile_fraction_follows_the_kernel_rule():
    bench = _bench()
    length = 512
    def mask_of(*valid):
        return torch.arange(length)[None, :] < torch.tensor(valid)[:, None]

    assert bench.executed_tile_fraction(mask_of(512)) == 1.0
    # 384 valid: three full query tiles x three key tiles, the fourth query tile is padding
    assert bench.executed_tile_fraction(mask_of(384)) == 9 / 16
    # 300 valid: two full query tiles x three key tiles, one mixed tile x four key tiles, one padded tile
    assert bench.executed_tile_fraction(mask_of(300)) == (2 * 3 + 4) / 16
    # one valid row: a single mixed query tile that walks every key tile
    assert bench.executed_tile_fraction(mask_of(1)) == 4 / 16
    assert bench.executed_tile_fraction(mask_of(512, 384)) == (16 + 9) / 32
    # a left-padded row: kept keys 200..511 -> key tiles 1..3; query tile 1 is mixed, 2 and 3 are full
    left = torch.arange(length)[None, :] >= 200
    assert bench.executed_tile_fraction(left) == (4 + 2 * 3) / 16


def test_workload_registry_matches_the_benchmark_configurations():
    bench = _bench()
    assert bench.WORKLOAD["batch"] == 32 and bench.WORKLOAD["seq_len"] == 512 and bench.WORKLOAD["min_len"] == 256
    assert bench.GEOMETRY["v3-base"] == dict(layers=12, hidden=768, heads=12, head_dim=64, ffn=3072, conv=3)
    assert bench.GEOMETRY["v2-xlarge"]["hidden"] == 1536 and bench.GEOMETRY["v2-xlarge"]["layers"] == 24
    assert sum(bench.MIXED["buckets"].values()) == 512 and sorted(bench.MIXED["buckets"]) == [128, 256, 512]
