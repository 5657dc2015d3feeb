"""numpy restatement of the reference's relative-position index builder.

TEST INFRASTRUCTURE ONLY (see ``oracle/__init__.py``).

Follows, function by function:

* ``log_bucket_position``   <- ``make_log_bucket_position``
  (reference ``src/disentangled_flash/_reference.py:115-136``)
* ``compact_position_plan`` <- ``SharedPositionPlanCache.compact``
  (reference ``src/disentangled_flash/position.py:89-128``)
* ``dense_pair_map``        <- ``SharedPositionPlanCache.dense``
  (reference ``src/disentangled_flash/position.py:130-156``)

The reference evaluates the bucket formula in float32 on the CPU.  The same
float32 steps are taken here (numpy float32 scalars and arrays), and the
result is pinned against the reference's own output for every delta in
[-2047, 2047] by ``tests/test_oracle_position.py``.
"""

from __future__ import annotations

from typing import NamedTuple

import numpy as np


class PositionPlan(NamedTuple):
    """Mirror of the reference ``SharedPositionIndexPlan`` (position.py:17-22)."""

    sequence_length: int
    active_slots: np.ndarray  # int64 [A], sorted global slots that occur
    delta_to_local: np.ndarray  # int32 [2L-1], delta index -> local slot


def log_bucket_position(relative_pos: np.ndarray, bucket_size: int, max_position: int) -> np.ndarray:
    """Signed log bucket of integer distances; float32 result like the reference.

    reference ``_reference.py:115-136``: distances with ``|d| < mid`` keep
    their value, larger ones are compressed logarithmically into
    ``(mid, bucket_size)`` with the sign re-applied.
    """

    rel = np.asarray(relative_pos, dtype=np.int64)
    sign = np.sign(rel).astype(np.float32)
    mid = bucket_size // 2
    inside = (rel < mid) & (rel > -mid)
    abs_pos = np.where(inside, np.int64(mid - 1), np.abs(rel))
    # int64 / python int -> float32 in the reference (torch default dtype).
    ratio = abs_pos.astype(np.float32) / np.float32(mid)
    denom = np.log(np.float32((max_position - 1) / mid))
    log_pos = np.ceil(np.log(ratio) / denom * np.float32(mid - 1)) + np.float32(mid)
    return np.where(abs_pos <= mid, rel.astype(np.float32), log_pos * sign).astype(np.float32)


def compact_position_plan(
    sequence_length: int,
    *,
    position_buckets: int,
    max_relative_positions: int,
    position_embedding_size: int,
    uses_position_bias: bool = True,
) -> PositionPlan:
    """O(L) plan: pruned slot list plus delta -> local-slot table.

    reference ``position.py:103-120``.
    """

    if sequence_length < 1:
        raise ValueError("sequence_length must be positive")
    length = int(sequence_length)
    if not uses_position_bias:
        return PositionPlan(length, np.empty(0, np.int64), np.zeros(2 * length - 1, np.int32))

    deltas = np.arange(-(length - 1), length, dtype=np.int64)
    if position_buckets > 0:
        deltas = log_bucket_position(deltas, position_buckets, max_relative_positions).astype(np.int64)
    span = position_embedding_size
    global_slots = np.clip(deltas + span, 0, 2 * span - 1)
    active = np.unique(global_slots)
    local = np.searchsorted(active, global_slots).astype(np.int32)
    return PositionPlan(length, active.astype(np.int64), local)


def dense_pair_map(plan: PositionPlan) -> np.ndarray:
    """``pair_to_local[i, j] = delta_to_local[i - j + L - 1]`` (position.py:145-150)."""

    length = plan.sequence_length
    idx = np.arange(length)
    return plan.delta_to_local[idx[:, None] - idx[None, :] + length - 1].astype(np.int64)
