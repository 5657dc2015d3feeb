"""B200-native DeBERTa-v2/v3 disentangled self-attention inference.

Drop-in for the attention path of ``disentangled_flash``: the same
``optimize_deberta()`` / ``enable_deberta_inference()`` entry points and
Hugging Face parameter names, with the hot path running in hand-written
sm_100a CUDA kernels behind a C ABI (``include/dfl_b200.h``).
"""

from .attention import B200PreparedPositionPlan, DisentangledFlashAttention
from .config import DebertaAttentionConfig
from .embeddings import fuse_deberta_embeddings
from .encoder import (
    DebertaV2InferenceEncoder,
    capture_deberta_buckets,
    compile_deberta_buckets,
    enable_deberta_inference,
    enable_deberta_v2_inference,
    optimize_deberta,
)
from .position import SharedPositionIndexPlan, SharedPositionPlanCache

__version__ = "0.1.0"

__all__ = [
    "B200PreparedPositionPlan",
    "DebertaAttentionConfig",
    "DebertaV2InferenceEncoder",
    "DisentangledFlashAttention",
    "SharedPositionIndexPlan",
    "SharedPositionPlanCache",
    "capture_deberta_buckets",
    "compile_deberta_buckets",
    "enable_deberta_inference",
    "enable_deberta_v2_inference",
    "fuse_deberta_embeddings",
    "optimize_deberta",
]
