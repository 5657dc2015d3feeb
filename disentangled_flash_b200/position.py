"""Model-wide relative-position index plans, built on the GPU.

Mirror of the reference's ``SharedPositionPlanCache``
(``src/disentangled_flash/position.py:52-128``): one cache per encoder, one
immutable plan per (sequence length, device).  The reference evaluates the
log-bucket formula, ``unique`` and ``searchsorted`` with CPU tensors and then
copies the result to the device; here the same tables are produced directly
on the device by ``dfl_build_position_lut`` (bit-exact with the CPU result).
Only the compact ``O(L)`` plan exists: the dense ``L x L`` gather map of the
reference's PyTorch backend is never needed by the fused kernel.
"""

from __future__ import annotations

from typing import NamedTuple

import torch

from . import _cabi


class SharedPositionIndexPlan(NamedTuple):
    """Compact ``O(L)`` position plan consumed by the fused kernel."""

    sequence_length: int
    active_slots: torch.Tensor  # int64 [A]
    delta_to_local: torch.Tensor  # int32 [2L-1]


def canonical_device(requested: torch.device | str | None, resident: torch.device) -> torch.device:
    """Resolve ``"cuda"`` to the device the module already lives on."""

    resolved = torch.device(requested) if requested is not None else resident
    if resolved.type == resident.type and resolved.index is None:
        return resident
    return resolved


class SharedPositionPlanCache:
    """Cache of immutable position-index tensors shared by all encoder layers."""

    def __init__(self, *, position_buckets: int, max_relative_positions: int, position_embedding_size: int,
                 uses_position_bias: bool = True) -> None:
        self.position_buckets = position_buckets
        self.max_relative_positions = max_relative_positions
        self.position_embedding_size = position_embedding_size
        self.uses_position_bias = uses_position_bias
        self._compact: dict[tuple[int, str], SharedPositionIndexPlan] = {}

    def clear(self) -> None:
        self._compact.clear()

    @torch.no_grad()
    def compact(self, sequence_length: int, device: torch.device | str) -> SharedPositionIndexPlan:
        """Return (building on first use) the delta LUT for one sequence length."""

        if sequence_length < 1:
            raise ValueError("sequence_length must be positive")
        resolved = torch.device(device)
        if resolved.type != "cuda":
            raise ValueError("B200 position plans must be prepared on CUDA")
        if resolved.index is None:
            resolved = torch.device("cuda", torch.cuda.current_device())
        key = (int(sequence_length), str(resolved))
        cached = self._compact.get(key)
        if cached is not None:
            return cached
        active, lut = _cabi.build_position_lut(
            int(sequence_length), int(self.position_buckets), int(self.max_relative_positions),
            int(self.position_embedding_size), bool(self.uses_position_bias), resolved,
        )
        plan = SharedPositionIndexPlan(int(sequence_length), active, lut)
        self._compact[key] = plan
        return plan


__all__ = ["SharedPositionIndexPlan", "SharedPositionPlanCache", "canonical_device"]
