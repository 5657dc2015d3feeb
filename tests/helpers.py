"""Shared builders for the parity tests (seeded inputs + oracle evaluation)."""

from __future__ import annotations

import math

import numpy as np
import torch

import oracle

MASK_PATTERNS = ("none", "right", "left", "heavy", "all")


def make_mask(pattern: str, batch: int, length: int, gen: torch.Generator) -> torch.Tensor:
    """Mask patterns of the reference's validation matrix (validation/validate_cuda.py:42-82)."""

    mask = torch.ones(batch, length, dtype=torch.bool)
    if pattern == "none":
        return mask
    if pattern == "all":
        mask[-1] = False
        return mask
    lengths = torch.randint(max(1, length // 4), length + 1, (batch,), generator=gen)
    pos = torch.arange(length)[None, :]
    if pattern == "right":
        return pos < lengths[:, None]
    if pattern == "left":
        return pos >= (length - lengths)[:, None]
    if pattern == "heavy":
        keep = torch.rand(batch, length, generator=gen) < 0.3
        keep[:, 0] = True
        return keep
    raise ValueError(pattern)


def plan_for(length: int, buckets: int = 256, max_pos: int = 512, uses_bias: bool = True):
    span = buckets if buckets > 0 else max_pos
    return oracle.compact_position_plan(
        length, position_buckets=buckets, max_relative_positions=max_pos, position_embedding_size=span,
        uses_position_bias=uses_bias,
    ), span


def make_core_case(batch, heads, length, d, dtype, seed, *, mode="both", mask="right", buckets=256, max_pos=512,
                   std=1.0):
    """Seeded Q/K/V/posK/posQ (already pruned to active slots), LUT and mask, as CPU tensors of ``dtype``."""

    gen = torch.Generator().manual_seed(seed)
    plan, span = plan_for(length, buckets, max_pos)
    q, k, v = (torch.randn(batch, heads, length, d, generator=gen).mul_(std).to(dtype) for _ in range(3))
    active = torch.from_numpy(plan.active_slots)
    pos_key = pos_query = None
    if mode in ("both", "c2p"):
        pos_key = torch.randn(heads, 2 * span, d, generator=gen).mul_(std).to(dtype)[:, active].contiguous()
    if mode in ("both", "p2c"):
        pos_query = torch.randn(heads, 2 * span, d, generator=gen).mul_(std).to(dtype)[:, active].contiguous()
    m = make_mask(mask, batch, length, gen)
    lut = torch.from_numpy(plan.delta_to_local)
    return dict(q=q, k=k, v=v, pos_key=pos_key, pos_query=pos_query, lut=lut, mask=m, plan=plan,
                scale=1.0 / math.sqrt(d * (1 + int(pos_key is not None) + int(pos_query is not None))))


def oracle_core(case, compute=torch.float32):
    """fp32 (or fp64) oracle on the same, already rounded, inputs.

    For 16-bit cases the C2P/P2C scores are rounded once to the input dtype,
    as the reference's position-score GEMMs do; nothing else is rounded.
    """

    up = lambda t: None if t is None else t.to(compute)  # noqa: E731
    in_dtype = case["q"].dtype
    with torch.no_grad():
        return oracle.attention_core(up(case["q"]), up(case["k"]), up(case["v"]), up(case["pos_key"]),
                                     up(case["pos_query"]), case["plan"].delta_to_local, case["mask"],
                                     score_dtype=None if in_dtype == torch.float32 else in_dtype)


def tolerance(dtype: torch.dtype, ref: torch.Tensor) -> torch.Tensor:
    """Element-wise bound used by every floating-point parity test.

    FP32: 1e-5 absolute plus 1e-5 relative (the strict-FP32 target).  FP16/BF16: 2e-3 absolute
    plus one rounding step of the output dtype at the reference magnitude
    (2^-11 relative for FP16, 2^-8 for BF16): an output of magnitude ~1 cannot
    be stored in BF16 to better than 3.9e-3, whatever computes it.
    """

    ref = ref.abs().to(torch.float64)
    if dtype == torch.float32:
        # 1e-5 absolute for outputs up to magnitude 1 (the reference's benchmark regime has |out| << 1);
        # larger outputs get the same bound relative to their size (fp32 has 24 bits at any magnitude).
        return torch.full_like(ref, 1e-5) + ref * 1e-5
    ulp = 2.0 ** -11 if dtype == torch.float16 else 2.0 ** -8
    return torch.full_like(ref, 2e-3) + ref * ulp


def assert_close(got: torch.Tensor, ref: torch.Tensor, dtype: torch.dtype, what: str = "") -> float:
    got64 = got.detach().cpu().to(torch.float64)
    ref64 = ref.detach().cpu().to(torch.float64)
    assert got64.shape == ref64.shape, (what, got64.shape, ref64.shape)
    assert torch.isfinite(got64).all(), f"{what}: non-finite output"
    err = (got64 - ref64).abs()
    bound = tolerance(dtype, ref64)
    worst = (err - bound).max().item()
    assert worst <= 0, f"{what}: max abs err {err.max().item():.3e} exceeds bound by {worst:.3e}"
    return err.max().item()


from oracle.encoder import oracle_encoder_forward  # noqa: E402,F401  (re-exported for the tests)
