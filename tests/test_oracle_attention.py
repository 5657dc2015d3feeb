"""The torch-CPU attention oracle against outputs of the real reference.

Golden data: ``tests/golden/attention_*.npz`` (inputs, parameters, and the
context tensors produced by the reference's ``original`` and ``torch``
backends in fp32).  Tolerance 2e-5 absolute: both sides are fp32 chains of
the same operations, differing only in summation order.
"""

import pytest
import torch

from conftest import ATTENTION_GOLDEN, load_attention_golden
from oracle import attention_module_forward

FP32_TOL = 2e-5


def run_oracle(g, dtype=torch.float32, storage_dtype=None):
    case, p = g["case"], g["params"]
    get = lambda k: p[k].to(dtype) if k in p else None  # noqa: E731
    with torch.no_grad():
        return attention_module_forward(
            g["hidden_states"].to(dtype),
            g["mask"],
            wq=get("query_proj.weight"), wk=get("key_proj.weight"), wv=get("value_proj.weight"),
            bq=get("query_proj.bias"), bk=get("key_proj.bias"), bv=get("value_proj.bias"),
            rel_embeddings=g["rel_embeddings"].to(dtype),
            num_heads=case["heads"],
            position_buckets=case["buckets"],
            max_relative_positions=case["max_pos"],
            pos_att_type=g["types"],
            relative_attention=bool(case["rel"]),
            share_att_key=bool(case["share"]),
            w_pos_key=get("pos_key_proj.weight"), b_pos_key=get("pos_key_proj.bias"),
            w_pos_query=get("pos_query_proj.weight"), b_pos_query=get("pos_query_proj.bias"),
            storage_dtype=storage_dtype,
        )


@pytest.mark.parametrize("name", ATTENTION_GOLDEN)
def test_oracle_matches_reference_backends(name):
    g = load_attention_golden(name)
    out = run_oracle(g)
    assert out.shape == g["ctx_torch"].shape
    assert (out - g["ctx_torch"]).abs().max().item() <= FP32_TOL
    assert (out - g["ctx_original"]).abs().max().item() <= FP32_TOL


@pytest.mark.parametrize("name", ATTENTION_GOLDEN)
def test_padded_query_rows_are_uniform_mean_of_values(name):
    # reference kernel.py:253-256 / _reference.py:308-312: a padded query attends uniformly to all L keys.
    g = load_attention_golden(name)
    mask = g["mask"]
    if mask.all():
        pytest.skip("no padded rows in this case")
    out = run_oracle(g, torch.float64)
    p = g["params"]
    v = torch.nn.functional.linear(g["hidden_states"].double(), p["value_proj.weight"].double(),
                                   p["value_proj.bias"].double())
    mean_v = v.mean(dim=1, keepdim=True).expand_as(v)
    assert (out[~mask] - mean_v[~mask]).abs().max().item() < 1e-9
