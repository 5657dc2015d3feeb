"""PyTorch-on-CPU restatement of the reference's prepared attention forward.

TEST INFRASTRUCTURE ONLY (see ``oracle/__init__.py``).

The reference's ``torch`` backend (README: "PyTorch impl.") is itself a chain
of PyTorch tensor ops, so the faithful CPU restatement is the same chain of
ops, written against plain tensors instead of an ``nn.Module``:

* ``fuse_qkv``               <- ``_prepare_fused_qkv``        (``_torch.py:112-123``)
* ``split_heads``            <- ``_reshape_heads``            (``_torch.py:299-314``)
* ``project_positions``      <- ``prepare_for_inference`` + ``transpose_for_scores``
                                (``_torch.py:143-158``, ``_reference.py:243-250``)
* ``attention_core``         <- the score/softmax/PV part of ``forward_prepared``
                                (``_torch.py:337-387``) with the mask rule of
                                ``_prepare_attention_mask`` (``_reference.py:189-191``)
* ``attention_module_forward`` <- the whole of ``forward_prepared``
                                (``_torch.py:316-387``) after ``prepare_shape``
                                (``_torch.py:171-219``).

Everything materialises ``[B, H, L, L]`` exactly like the reference's CPU
path does; that is what makes it a fair host-CPU baseline.
"""

from __future__ import annotations

import math

import numpy as np
import torch
from torch.nn import functional as F

from .position import PositionPlan, compact_position_plan, dense_pair_map


def fuse_qkv(wq, wk, wv, bq=None, bk=None, bv=None):
    """Concatenate the three projections; bias only if all three exist."""

    weight = torch.cat((wq, wk, wv), dim=0).contiguous()
    biases = (bq, bk, bv)
    bias = torch.cat(biases, dim=0).contiguous() if all(b is not None for b in biases) else None
    return weight, bias


def split_heads(tensor: torch.Tensor, num_heads: int) -> torch.Tensor:
    """``[B, L, H*d] -> [B, H, L, d]`` contiguous."""

    b, l, hd = tensor.shape
    return tensor.view(b, l, num_heads, hd // num_heads).permute(0, 2, 1, 3).contiguous()


def project_positions(rel_embeddings, weight, bias, num_heads: int, span: int) -> torch.Tensor:
    """Relative embedding table through a content projection: ``[H, 2*span, d]``.

    ``share_att_key=True`` passes ``key_proj``/``query_proj`` (bias included);
    otherwise ``pos_key_proj``/``pos_query_proj`` (``_torch.py:146-158``).
    """

    rel = rel_embeddings[: 2 * span]
    projected = F.linear(rel, weight, bias)  # [2*span, H*d]
    d = projected.shape[-1] // num_heads
    return projected.view(2 * span, num_heads, d).permute(1, 0, 2).contiguous()


def attention_core(
    q: torch.Tensor,
    k: torch.Tensor,
    v: torch.Tensor,
    pos_key: torch.Tensor | None,
    pos_query: torch.Tensor | None,
    delta_to_local,
    mask: torch.Tensor,
    *,
    scale_factor: int | None = None,
    score_dtype: torch.dtype | None = None,
) -> torch.Tensor:
    """Scores + C2P/P2C gathers + mask + softmax + PV.

    ``score_dtype``: when the model runs in FP16/BF16 the reference's two
    position-score GEMMs return tensors of that dtype (``kernel.py:577,583``),
    i.e. every C2P/P2C score is rounded to 16 bits before it is added to the
    fp32 content score.  Passing the dtype here reproduces that one rounding
    while everything else stays in the precision of ``q``.

    ``q, k, v``: ``[B, H, L, d]``; ``pos_key``/``pos_query``: ``[H, A, d]``
    already pruned to the active slots (or ``None`` when the term is off);
    ``delta_to_local``: int ``[2L-1]``; ``mask``: ``[B, L]`` (non-zero = keep).
    Returns ``[B, L, H*d]`` in the dtype of ``q``.

    Mask rule (``_reference.py:189-191``, ``_torch.py:371-379``): pair (i, j)
    is attended iff both tokens are kept; every other score is replaced by the
    most negative finite value, so a padded query row becomes uniform over
    all L keys.
    """

    bsz, heads, length, d = q.shape
    has_c2p = pos_key is not None
    has_p2c = pos_query is not None
    if scale_factor is None:
        scale_factor = 1 + int(has_c2p) + int(has_p2c)
    scale = math.sqrt(d * scale_factor)

    scores = torch.matmul(q, k.transpose(-1, -2) / scale)
    if has_c2p or has_p2c:
        lut = torch.as_tensor(np.asarray(delta_to_local), dtype=torch.long)
        idx = torch.arange(length)
        pair = lut[idx[:, None] - idx[None, :] + length - 1]
        pair = pair.view(1, 1, length, length).expand(bsz, heads, length, length)
    if has_c2p:
        c2p = torch.matmul(q, pos_key.transpose(-1, -2))
        if score_dtype is not None:
            c2p = c2p.to(score_dtype).to(q.dtype)
        c2p = c2p / scale
        scores = scores + torch.gather(c2p, dim=-1, index=pair)
    if has_p2c:
        p2c = torch.matmul(k, pos_query.transpose(-1, -2))
        if score_dtype is not None:
            p2c = p2c.to(score_dtype).to(q.dtype)
        p2c = p2c / scale
        scores = scores + torch.gather(p2c.transpose(-1, -2), dim=-2, index=pair)

    keep = mask.to(torch.bool)
    pair_keep = keep[:, None, :, None] & keep[:, None, None, :]
    scores = scores.masked_fill(~pair_keep, torch.finfo(q.dtype).min)
    probs = torch.softmax(scores, dim=-1)
    ctx = torch.matmul(probs, v)
    return ctx.permute(0, 2, 1, 3).contiguous().view(bsz, length, heads * d)


def attention_module_forward(
    hidden: torch.Tensor,
    mask: torch.Tensor,
    *,
    wq, wk, wv, bq=None, bk=None, bv=None,
    rel_embeddings: torch.Tensor | None = None,
    num_heads: int,
    position_buckets: int = 256,
    max_relative_positions: int = 512,
    pos_att_type=("p2c", "c2p"),
    relative_attention: bool = True,
    share_att_key: bool = True,
    w_pos_key=None, b_pos_key=None, w_pos_query=None, b_pos_query=None,
    plan: PositionPlan | None = None,
    storage_dtype: torch.dtype | None = None,
) -> torch.Tensor:
    """Whole attention sub-module: hidden ``[B, L, hid]`` -> context ``[B, L, H*d]``.

    ``storage_dtype``: a model running in FP16/BF16 stores every tensor that
    passes between two kernels in that type: Q/K/V after the projection, the
    projected position tables, and the C2P/P2C scores.  Passing the dtype
    reproduces exactly those roundings (arithmetic stays in the dtype of
    ``hidden``), so a 16-bit implementation can be compared tightly.

    ``max_relative_positions`` must already be resolved (values < 1 mean
    ``max_position_embeddings``, ``_reference.py:223-225``).
    """

    length = hidden.shape[1]
    weight, bias = fuse_qkv(wq, wk, wv, bq, bk, bv)
    hd = wq.shape[0]
    rnd = (lambda t: t.to(storage_dtype).to(hidden.dtype)) if storage_dtype is not None else (lambda t: t)
    q, k, v = F.linear(hidden, weight, bias).split(hd, dim=-1)
    q, k, v = (rnd(split_heads(t, num_heads)) for t in (q, k, v))

    has_c2p = relative_attention and "c2p" in pos_att_type
    has_p2c = relative_attention and "p2c" in pos_att_type
    span = position_buckets if position_buckets > 0 else max_relative_positions
    if plan is None:
        plan = compact_position_plan(
            length,
            position_buckets=position_buckets,
            max_relative_positions=max_relative_positions,
            position_embedding_size=span,
            uses_position_bias=has_c2p or has_p2c,
        )
    active = torch.as_tensor(plan.active_slots, dtype=torch.long)
    pos_key = pos_query = None
    if has_c2p:
        w, b = (wk, bk) if share_att_key else (w_pos_key, b_pos_key)
        pos_key = rnd(project_positions(rel_embeddings, w, b, num_heads, span)).index_select(1, active).contiguous()
    if has_p2c:
        w, b = (wq, bq) if share_att_key else (w_pos_query, b_pos_query)
        pos_query = rnd(project_positions(rel_embeddings, w, b, num_heads, span)).index_select(1, active).contiguous()

    # The reference scales by 1 + [c2p in type] + [p2c in type] even when
    # relative attention is off (``_torch.py:337``).
    scale_factor = 1 + int("c2p" in pos_att_type) + int("p2c" in pos_att_type)
    return attention_core(q, k, v, pos_key, pos_query, plan.delta_to_local, mask, scale_factor=scale_factor,
                          score_dtype=storage_dtype)


__all__ = [
    "attention_core",
    "attention_module_forward",
    "compact_position_plan",
    "dense_pair_map",
    "fuse_qkv",
    "project_positions",
    "split_heads",
]
