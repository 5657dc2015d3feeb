"""Inference-only DeBERTa-v2/v3 disentangled self-attention on B200 kernels.

Host-side mirror of the reference's Triton attention module
(``TritonInferenceDisentangledSelfAttention``, reference
``src/disentangled_flash/kernel.py:471-638``, whose preparation logic lives in
``src/disentangled_flash/_torch.py:112-219``).  Parameter names are the
Hugging Face ones (``query_proj``, ``key_proj``, ``value_proj`` and, without
``share_att_key``, ``pos_key_proj`` / ``pos_query_proj``) so checkpoints load
with ``strict=True``.

The hot function is :meth:`forward_prepared`.  On the current CUDA stream it
issues ``dfl_qkv_proj`` (fused QKV projection, written head-major
``[B,H,L,d]``) followed by

* ``dfl_attention_rel_fwd`` where it applies (FP16/BF16, head dim 32/64,
  length up to 2048): one persistent kernel that computes the C2P/P2C scores
  on the tensor cores from the plan's relative-distance tables and consumes
  them in place (QK^T + relative gathers + mask + softmax + PV), or otherwise
* ``dfl_pos_scores`` (the two score GEMMs) and ``dfl_attention_fwd`` (the
  fused kernel fed with their output), the reference's operator boundary.

There is no PyTorch, Triton or CPU implementation behind them.
"""

from __future__ import annotations

import math
from typing import Any, NamedTuple, Optional

import torch
from torch import nn

from . import _cabi
from .config import normalise_pos_att_type
from .position import SharedPositionPlanCache, canonical_device

SUPPORTED_HEAD_DIMS = (32, 64, 128)


class B200PreparedPositionPlan(NamedTuple):
    """Layer projections plus one shared compact position LUT.

    Same fields as the reference's ``TritonPreparedPositionPlan``
    (``kernel.py:461-468``).
    """

    sequence_length: int
    active_slots: torch.Tensor
    delta_to_local: torch.Tensor
    pos_key: torch.Tensor | None
    pos_query: torch.Tensor | None
    # B200 additions: the pruned tables expanded by relative distance, [H, 2L-1, d], when the
    # single-launch attention kernel covers the configuration (else None)
    rel_key: torch.Tensor | None = None
    rel_query: torch.Tensor | None = None


# --------------------------------------------------------------------------
# Operator boundary.  The reference registers its fused kernel as a torch
# custom op so that torch.compile can trace the encoder around it
# (kernel.py:431-438); this op plays the same role for the C-ABI calls of one layer:
# dfl_qkv_proj, then dfl_attention_rel_fwd where the plan carries relative-distance
# tables, else dfl_pos_scores + dfl_attention_fwd.
# --------------------------------------------------------------------------
def _attention_forward(   # the plain function: what an eager forward calls

    hidden_states: torch.Tensor,
    attention_mask: torch.Tensor,
    qkv_weight: torch.Tensor,
    qkv_bias: Optional[torch.Tensor],
    pos_key: Optional[torch.Tensor],
    pos_query: Optional[torch.Tensor],
    delta_to_local: Optional[torch.Tensor],
    rel_key: Optional[torch.Tensor],
    rel_query: Optional[torch.Tensor],
    num_heads: int,
    head_dim: int,
    scale: float,
    algo: int,
    status: Optional[torch.Tensor],
) -> torch.Tensor:
    length = hidden_states.shape[1]
    query, key, value = _cabi.linear_heads(
        hidden_states, qkv_weight, qkv_bias, n_out=3, heads=num_heads, head_dim=head_dim, rows_per_seq=length,
        algo=algo, status=status,
    )
    if rel_key is not None or rel_query is not None:
        # relative scores are produced inside the attention kernel: no [B,H,L,A] tensor in memory
        return _cabi.attention_rel_fwd(query, key, value, rel_key, rel_query, attention_mask, scale, status=status)
    c2p = p2c = None
    ld_slots = 0
    if pos_key is not None or pos_query is not None:
        c2p, p2c, ld_slots = _cabi.pos_scores(query, key, pos_key, pos_query, algo=algo, status=status)
    return _cabi.attention_fwd(query, key, value, c2p, p2c, delta_to_local, attention_mask, scale,
                               ld_slots=ld_slots, algo=algo, status=status)


# The same function as a custom operator, for a forward that is being traced (``compile_deberta_buckets``): the
# dispatcher's way into a Python operator costs more host time than some of the kernels run, so an eager forward
# calls the function directly.
_attention_forward_op = torch.library.custom_op("disentangled_flash_b200::attention_forward", mutates_args=("status",),
                                                device_types="cuda")(_attention_forward)


@_attention_forward_op.register_fake
def _attention_forward_fake(hidden_states, attention_mask, qkv_weight, qkv_bias, pos_key, pos_query,
                            delta_to_local, rel_key, rel_query, num_heads, head_dim, scale, algo, status):
    return hidden_states.new_empty(hidden_states.shape[0], hidden_states.shape[1], num_heads * head_dim)


def _require_2d_padding_mask(attention_mask: torch.Tensor, batch_size: int, sequence_length: int) -> torch.Tensor:
    """Validate the factorised per-token padding-mask contract (reference kernel.py:441-458).

    Bool and integer masks are handed to the kernel as they are (it tests
    each element for non-zero); anything else is converted to bool once.
    """

    if attention_mask.dim() != 2:
        raise ValueError(
            "the fused path requires a factorized padding mask with shape [B, L]; "
            "arbitrary pairwise masks are not supported"
        )
    if attention_mask.shape != (batch_size, sequence_length):
        raise ValueError(
            f"attention_mask shape {tuple(attention_mask.shape)} does not match [{batch_size}, {sequence_length}]"
        )
    if attention_mask.dtype.is_floating_point or attention_mask.element_size() not in (1, 4, 8):
        attention_mask = attention_mask.bool()
    return attention_mask.contiguous()


def _invalidate_attention_cache_after_load(module: nn.Module, _incompatible_keys: Any) -> None:
    module.clear_inference_cache()


class DisentangledFlashAttention(nn.Module):
    """Forward-only CUDA DeBERTa-v2/v3 self-attention for head dims 32, 64 and 128.

    FP16/BF16 run on the tcgen05 tensor-core kernels.  FP32 always runs the
    IEEE-fp32 CUDA-core kernels: ``fp32_precision="strict"`` is what they
    implement, and ``"fast"`` (TF32 in the reference) is accepted and served by
    the same, more accurate, kernels.
    """

    def __init__(self, config: Any, *, position_plan_cache: SharedPositionPlanCache | None = None,
                 fp32_precision: str = "strict") -> None:
        super().__init__()
        if config.hidden_size % config.num_attention_heads != 0 and not getattr(config, "attention_head_size", None):
            raise ValueError(
                f"The hidden size ({config.hidden_size}) is not a multiple of the number "
                f"of attention heads ({config.num_attention_heads})"
            )
        if fp32_precision not in {"strict", "fast"}:
            raise ValueError("fp32_precision must be 'strict' or 'fast'")
        self.fp32_precision = fp32_precision
        self.num_attention_heads = config.num_attention_heads
        default_head = config.hidden_size // config.num_attention_heads
        self.attention_head_size = getattr(config, "attention_head_size", None) or default_head
        self.all_head_size = self.num_attention_heads * self.attention_head_size
        self.query_proj = nn.Linear(config.hidden_size, self.all_head_size, bias=True)
        self.key_proj = nn.Linear(config.hidden_size, self.all_head_size, bias=True)
        self.value_proj = nn.Linear(config.hidden_size, self.all_head_size, bias=True)

        self.share_att_key = bool(getattr(config, "share_att_key", False))
        self.pos_att_type = normalise_pos_att_type(getattr(config, "pos_att_type", None))
        self.relative_attention = bool(getattr(config, "relative_attention", False))
        self.position_buckets = getattr(config, "position_buckets", -1)
        self.max_relative_positions = getattr(config, "max_relative_positions", -1)
        if self.max_relative_positions < 1:
            self.max_relative_positions = config.max_position_embeddings
        self.pos_ebd_size = self.position_buckets if self.position_buckets > 0 else self.max_relative_positions
        if self.relative_attention and not self.share_att_key:
            if "c2p" in self.pos_att_type:
                self.pos_key_proj = nn.Linear(config.hidden_size, self.all_head_size, bias=True)
            if "p2c" in self.pos_att_type:
                self.pos_query_proj = nn.Linear(config.hidden_size, self.all_head_size)

        self.position_plan_cache = position_plan_cache or SharedPositionPlanCache(
            position_buckets=self.position_buckets,
            max_relative_positions=self.max_relative_positions,
            position_embedding_size=self.pos_ebd_size,
            uses_position_bias=self.has_c2p or self.has_p2c,
        )
        self.register_buffer("_cached_pos_key", None, persistent=False)
        self.register_buffer("_cached_pos_query", None, persistent=False)
        self.register_buffer("_cached_qkv_weight", None, persistent=False)
        self.register_buffer("_cached_qkv_bias", None, persistent=False)
        # device int32 that the kernels of this layer write if one of their bounded waits expires; an encoder
        # shares one word between its layers (set_status_word) and reads it in check_device_status()
        self.register_buffer("_status_word", None, persistent=False)
        self._position_projection_cache: dict[tuple[int, str], B200PreparedPositionPlan] = {}
        self._algo = _cabi.ALGO_AUTO
        self.register_load_state_dict_post_hook(_invalidate_attention_cache_after_load)

    # ------------------------------------------------------------ properties
    @property
    def has_c2p(self) -> bool:
        return self.relative_attention and "c2p" in self.pos_att_type

    @property
    def has_p2c(self) -> bool:
        return self.relative_attention and "p2c" in self.pos_att_type

    def _scale(self, scale_factor: int) -> float:
        return math.sqrt(self.attention_head_size * scale_factor)

    # ---------------------------------------------------- cache invalidation
    def set_position_plan_cache(self, cache: SharedPositionPlanCache) -> "DisentangledFlashAttention":
        self.position_plan_cache = cache
        self._position_projection_cache.clear()
        return self

    def set_status_word(self, status: torch.Tensor | None) -> "DisentangledFlashAttention":
        """Use ``status`` (a zeroed CUDA int32 with one element, e.g. shared by all layers of an encoder)."""

        self._status_word = status
        return self

    def check_device_status(self) -> None:
        """Raise ``DflError(DFL_ERR_DEVICE_TIMEOUT)`` if a bounded device-side wait of this layer's kernels expired.

        Synchronises the current stream; call it after a batch, not between layers.
        """

        if self._status_word is not None:
            _cabi.check_status(self._status_word)

    def clear_inference_cache(self) -> None:
        """Invalidate every tensor derived from this layer's parameters."""

        self._cached_pos_key = None
        self._cached_pos_query = None
        self._cached_qkv_weight = None
        self._cached_qkv_bias = None
        if hasattr(self, "_position_projection_cache"):
            self._position_projection_cache.clear()

    def train(self, mode: bool = True) -> "DisentangledFlashAttention":
        if mode:
            self.clear_inference_cache()
        return super().train(mode)

    def _apply(self, fn: Any, recurse: bool = True) -> "DisentangledFlashAttention":
        result = super()._apply(fn, recurse=recurse)
        self.clear_inference_cache()
        return result

    # ------------------------------------------------------------ preparation
    def _validate_device_dtype(self, tensor: torch.Tensor) -> None:
        if tensor.device.type != "cuda":
            raise RuntimeError("DisentangledFlashAttention requires CUDA")
        if tensor.dtype not in (torch.float16, torch.bfloat16, torch.float32):
            raise TypeError("the B200 path supports FP16, BF16, and FP32")
        if self.attention_head_size not in SUPPORTED_HEAD_DIMS:
            raise ValueError("the B200 path supports attention head dimensions 32, 64, and 128")

    @torch.no_grad()
    def _prepare_fused_qkv(self) -> None:
        self._cached_qkv_weight = torch.cat(
            (self.query_proj.weight, self.key_proj.weight, self.value_proj.weight), dim=0
        ).contiguous()
        biases = (self.query_proj.bias, self.key_proj.bias, self.value_proj.bias)
        self._cached_qkv_bias = (
            torch.cat(biases, dim=0).contiguous() if all(b is not None for b in biases) else None
        )

    def _project_relative(self, relative: torch.Tensor, projection: nn.Linear) -> torch.Tensor:
        """``[2*span, hid] -> [H, 2*span, d]`` through ``dfl_qkv_proj`` with ``n_out=1``."""

        (projected,) = _cabi.linear_heads(
            relative, projection.weight.contiguous(), projection.bias, n_out=1, heads=self.num_attention_heads,
            head_dim=self.attention_head_size, rows_per_seq=relative.shape[0], algo=self._algo,
            status=self._status_word,
        )
        return projected[0]

    @torch.no_grad()
    def prepare_for_inference(self, rel_embeddings: torch.Tensor | None) -> "DisentangledFlashAttention":
        """Cache the fused QKV weight and the projected relative-position tables."""

        if self.training:
            raise RuntimeError("prepare_for_inference() requires module.eval()")
        self._validate_device_dtype(self.query_proj.weight)
        self.clear_inference_cache()
        self._prepare_fused_qkv()
        if self._status_word is None or self._status_word.device != self.query_proj.weight.device:
            self._status_word = _cabi.new_status_word(self.query_proj.weight.device)
        if not (self.has_c2p or self.has_p2c):
            return self
        if rel_embeddings is None:
            raise ValueError("rel_embeddings is required for relative attention")
        span = self.pos_ebd_size
        relative = rel_embeddings[: span * 2].to(self.query_proj.weight.dtype).contiguous()
        if self.has_c2p:
            projection = self.key_proj if self.share_att_key else self.pos_key_proj
            self._cached_pos_key = self._project_relative(relative, projection)
        if self.has_p2c:
            projection = self.query_proj if self.share_att_key else self.pos_query_proj
            self._cached_pos_query = self._project_relative(relative, projection)
        return self

    def _plan_device(self) -> torch.device:
        if self._cached_pos_key is not None:
            return self._cached_pos_key.device
        if self._cached_pos_query is not None:
            return self._cached_pos_query.device
        return self.query_proj.weight.device

    def _project_active_positions(self, active_slots: torch.Tensor):
        pos_key = pos_query = None
        if self.has_c2p:
            if self._cached_pos_key is None:
                raise RuntimeError("call prepare_for_inference() before prepare_shape()")
            pos_key = _cabi.gather_slots(self._cached_pos_key, active_slots)
        if self.has_p2c:
            if self._cached_pos_query is None:
                raise RuntimeError("call prepare_for_inference() before prepare_shape()")
            pos_query = _cabi.gather_slots(self._cached_pos_query, active_slots)
        return pos_key, pos_query

    @torch.no_grad()
    def prepare_shape(self, sequence_length: int, device: torch.device | str | None = None) -> B200PreparedPositionPlan:
        """Prepare the per-length plan: shared LUT plus this layer's pruned tables."""

        if self.training:
            raise RuntimeError("prepare_shape() requires module.eval()")
        resident = self._plan_device()
        resolved = canonical_device(device, resident)
        if resolved.type != "cuda":
            raise ValueError("B200 shape plans must be prepared on CUDA")
        key = (sequence_length, str(resolved))
        cached = self._position_projection_cache.get(key)
        if cached is not None:
            return cached
        indices = self.position_plan_cache.compact(sequence_length, resolved)
        pos_key, pos_query = self._project_active_positions(indices.active_slots)
        rel_key = rel_query = None
        dtype = self.query_proj.weight.dtype
        if _cabi.attention_rel_supported(dtype, sequence_length, self.attention_head_size, self.has_c2p, self.has_p2c,
                                         self._algo):
            if pos_key is not None:
                rel_key = _cabi.expand_rel_tables(pos_key, indices.delta_to_local, sequence_length)
            if pos_query is not None:
                rel_query = _cabi.expand_rel_tables(pos_query, indices.delta_to_local, sequence_length)
        plan = B200PreparedPositionPlan(
            sequence_length=sequence_length,
            active_slots=indices.active_slots,
            delta_to_local=indices.delta_to_local,
            pos_key=pos_key,
            pos_query=pos_query,
            rel_key=rel_key,
            rel_query=rel_query,
        )
        self._position_projection_cache[key] = plan
        return plan

    # ---------------------------------------------------------------- forward
    def _validate_inference_call(self) -> None:
        if self.training:
            raise RuntimeError("DisentangledFlashAttention requires module.eval()")
        if torch.is_grad_enabled():
            raise RuntimeError("DisentangledFlashAttention requires torch.no_grad() or torch.inference_mode()")

    def _project_qkv(self, hidden_states: torch.Tensor):
        """Fused QKV projection; returns ``q, k, v`` head-major ``[B, H, L, d]``.

        The reference returns ``[B, L, H*d]`` views and transposes afterwards
        (``_torch.py:284-314``); here the transpose is part of the GEMM epilogue.
        """

        if self._cached_qkv_weight is None:
            raise RuntimeError("fused QKV projection is not prepared; call prepare_for_inference() first")
        self._validate_device_dtype(hidden_states)
        return _cabi.linear_heads(
            hidden_states.contiguous(), self._cached_qkv_weight, self._cached_qkv_bias, n_out=3,
            heads=self.num_attention_heads, head_dim=self.attention_head_size,
            rows_per_seq=hidden_states.shape[1], algo=self._algo, status=self._status_word,
        )

    def forward_prepared(self, hidden_states: torch.Tensor, attention_mask: torch.Tensor,
                         plan: B200PreparedPositionPlan) -> tuple[torch.Tensor, None]:
        """Pure forward using a plan prepared completely outside the hot path."""

        self._validate_device_dtype(hidden_states)
        self._validate_inference_call()
        batch_size, sequence_length = hidden_states.shape[:2]
        if sequence_length != plan.sequence_length:
            raise ValueError(
                f"prepared length {plan.sequence_length} does not match input length {sequence_length}"
            )
        if self._cached_qkv_weight is None:
            raise RuntimeError("fused QKV projection is not prepared; call prepare_for_inference() first")
        if hidden_states.dtype != self._cached_qkv_weight.dtype:
            raise TypeError("hidden_states dtype does not match the module's parameters")
        base_mask = _require_2d_padding_mask(attention_mask, batch_size, sequence_length)
        if self.has_c2p and plan.pos_key is None:
            raise ValueError("prepared plan has no content-to-position keys")
        if self.has_p2c and plan.pos_query is None:
            raise ValueError("prepared plan has no position-to-content queries")

        # Hugging Face counts the configured position terms in the scale even
        # when relative attention is switched off (_reference.py:277-286).
        scale_factor = 1 + int("c2p" in self.pos_att_type) + int("p2c" in self.pos_att_type)
        uses_lut = self.has_c2p or self.has_p2c
        output = (_attention_forward_op if torch.compiler.is_compiling() else _attention_forward)(
            hidden_states.contiguous(),
            base_mask,
            self._cached_qkv_weight,
            self._cached_qkv_bias,
            plan.pos_key if self.has_c2p else None,
            plan.pos_query if self.has_p2c else None,
            plan.delta_to_local if uses_lut else None,
            plan.rel_key if self.has_c2p else None,
            plan.rel_query if self.has_p2c else None,
            self.num_attention_heads,
            self.attention_head_size,
            1.0 / self._scale(scale_factor),
            self._algo,
            self._status_word,
        )
        return output, None

    def forward_packed_rows(self, hidden_states: torch.Tensor, attention_mask: torch.Tensor,
                            plan: B200PreparedPositionPlan,
                            packed_rows: tuple[torch.Tensor, torch.Tensor, int],
                            packed_input: tuple[torch.Tensor, tuple[torch.Tensor, ...]] | None = None) -> torch.Tensor:
        """``forward_prepared`` with the context written as packed rows ``[T, H*d]``: sequence ``b`` owns rows
        ``row_base[b] .. + row_count[b]`` (``packed_rows = (row_base, row_count, T)``); positions beyond
        ``row_count[b]`` are not stored.  Only on the single-launch attention path (FP16/BF16, head dim 32/64, a
        relative term); no counterpart in the reference, which keeps padded positions in every tensor.

        With ``packed_input = (row_groups, (q, k, v))`` the hidden states are packed rows ``[T, hid]`` as well
        (``attention_mask`` still gives batch and length): the projection writes group ``g`` of 32 rows to rows
        ``row_groups[g] .. +31`` of the caller's ``[B, H, L, d]`` buffers, whose remaining rows must hold finite
        values (masked keys get probability zero, and zero times a stale NaN would still be NaN)."""

        self._validate_device_dtype(hidden_states)
        self._validate_inference_call()
        batch_size, sequence_length = (attention_mask if packed_input is not None else hidden_states).shape[:2]
        if sequence_length != plan.sequence_length:
            raise ValueError(f"prepared length {plan.sequence_length} does not match input length {sequence_length}")
        if self._cached_qkv_weight is None:
            raise RuntimeError("fused QKV projection is not prepared; call prepare_for_inference() first")
        rel_key = plan.rel_key if self.has_c2p else None
        rel_query = plan.rel_query if self.has_p2c else None
        if rel_key is None and rel_query is None:
            raise NotImplementedError("packed rows need the single-launch attention path (expanded position tables)")
        base_mask = _require_2d_padding_mask(attention_mask, batch_size, sequence_length)
        scale_factor = 1 + int("c2p" in self.pos_att_type) + int("p2c" in self.pos_att_type)
        row_groups, buffers = packed_input if packed_input is not None else (None, None)
        query, key, value = _cabi.linear_heads(
            hidden_states.contiguous(), self._cached_qkv_weight, self._cached_qkv_bias, n_out=3,
            heads=self.num_attention_heads, head_dim=self.attention_head_size, rows_per_seq=sequence_length,
            algo=self._algo, status=self._status_word, row_groups=row_groups, outs=buffers)
        return _cabi.attention_rel_fwd(query, key, value, rel_key, rel_query, base_mask,
                                       1.0 / self._scale(scale_factor), status=self._status_word,
                                       packed_rows=packed_rows)

    def forward(self, hidden_states: torch.Tensor, attention_mask: torch.Tensor, output_attentions: bool = False,
                query_states: torch.Tensor | None = None, relative_pos: torch.Tensor | None = None,
                rel_embeddings: torch.Tensor | None = None) -> tuple[torch.Tensor, None]:
        """Convenience wrapper with lazy preparation outside the pure hot path."""

        self._validate_device_dtype(hidden_states)
        self._validate_inference_call()
        if output_attentions:
            raise ValueError("output_attentions=True is not supported by the fused path")
        if query_states is not None:
            raise ValueError("the fused path supports self-attention only")
        if relative_pos is not None:
            raise ValueError("custom relative_pos tensors are not supported by the fused path")
        needs_key = self.has_c2p and self._cached_pos_key is None
        needs_query = self.has_p2c and self._cached_pos_query is None
        if needs_key or needs_query or self._cached_qkv_weight is None:
            self.prepare_for_inference(rel_embeddings)
        plan = self.prepare_shape(hidden_states.size(1), hidden_states.device)
        return self.forward_prepared(hidden_states, attention_mask, plan)


__all__ = ["B200PreparedPositionPlan", "DisentangledFlashAttention", "SUPPORTED_HEAD_DIMS"]
