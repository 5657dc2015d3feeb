"""Stand-alone attention configuration (subset of Hugging Face ``DebertaV2Config``).

Same field names and defaults as the reference's ``DebertaAttentionConfig``
(``src/disentangled_flash/_reference.py:37-59``), so scripts written against
the reference keep working; any object with these attributes (for instance
a real ``DebertaV2Config``) is accepted wherever a config is expected.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any


@dataclass(frozen=True)
class DebertaAttentionConfig:
    hidden_size: int = 768
    num_attention_heads: int = 12
    attention_head_size: int | None = None
    num_hidden_layers: int = 12
    intermediate_size: int = 3072
    hidden_act: Any = "gelu"
    attention_probs_dropout_prob: float = 0.1
    hidden_dropout_prob: float = 0.1
    layer_norm_eps: float = 1e-7
    relative_attention: bool = True
    max_relative_positions: int = -1
    max_position_embeddings: int = 512
    position_buckets: int = 256
    share_att_key: bool = True
    pos_att_type: Any = ("p2c", "c2p")
    norm_rel_ebd: str = "layer_norm"
    conv_kernel_size: int = 0
    conv_groups: int = 1
    conv_act: str = "tanh"


def normalise_pos_att_type(value: Any) -> tuple[str, ...]:
    """``"p2c|c2p"`` / list / tuple / None -> tuple of lower-case names."""

    if value is None:
        return ()
    if isinstance(value, str):
        return tuple(part.strip().lower() for part in value.split("|") if part.strip())
    return tuple(str(part).strip().lower() for part in value)
