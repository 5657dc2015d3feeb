"""Encoder-level drop-in: ``optimize_deberta`` / ``enable_deberta_inference``.

Mirror of the reference's encoder wrapper and public API
(``src/disentangled_flash/deberta.py:38-447``).  The wrapper keeps the
Hugging Face layer list, ``rel_embeddings``, ``LayerNorm`` and ``conv`` by
reference (checkpoint keys do not change), swaps every
``layer.attention.self`` for :class:`DisentangledFlashAttention`, prepares one
tuple of per-layer plans per sequence-length bucket, and runs the layer loop
with the 2-D padding mask and the prepared plans: no ``[B,1,L,L]`` mask and no
``[L,L]`` relative-position tensor is ever built.

Everything outside ``attention.self`` (attention output projection, FFN,
layer norms, the layer-0 convolution) stays the caller's PyTorch modules.
There is a single backend; ``backend="triton"`` is accepted as the legacy name
of the fused backend, ``backend="torch"`` is refused because no CPU/PyTorch
attention ships with this package.
"""

from __future__ import annotations

import inspect
import types
from collections.abc import Callable, Iterable, Mapping
from dataclasses import dataclass
from typing import Any

import torch
from torch import nn

from .attention import B200PreparedPositionPlan, DisentangledFlashAttention
from .config import normalise_pos_att_type
from .position import SharedPositionPlanCache

FUSED_BACKENDS = ("b200", "triton")


@dataclass
class BaseModelOutput:
    """Minimal stand-in for Transformers' ``BaseModelOutput`` (indexable like a tuple)."""

    last_hidden_state: torch.Tensor
    hidden_states: tuple[torch.Tensor, ...] | None = None
    attentions: tuple[torch.Tensor, ...] | None = None

    def __getitem__(self, index: int) -> Any:
        present = tuple(v for v in (self.last_hidden_state, self.hidden_states, self.attentions) if v is not None)
        return present[index]


def _invalidate_encoder_cache_after_load(module: nn.Module, _incompatible_keys: Any) -> None:
    module.clear_inference_cache()


class DebertaV2InferenceEncoder(nn.Module):
    """Inference-only replacement for a Hugging Face ``DebertaV2Encoder``.

    Call :meth:`prepare_for_inference` with every production bucket length,
    then :meth:`activate_shape` before running a bucket.  ``forward`` touches
    only the active immutable tuple of plans.
    """

    def __init__(self, source_encoder: nn.Module, config: Any, *, backend: str = "b200",
                 fp32_precision: str = "strict") -> None:
        super().__init__()
        if backend in ("torch", "optimized"):
            raise ValueError(
                f"backend={backend!r} is not available: this package ships only the fused CUDA backend "
                f"(use one of {FUSED_BACKENDS})"
            )
        if backend not in FUSED_BACKENDS:
            raise ValueError(f"backend must be one of {FUSED_BACKENDS}")
        if not hasattr(source_encoder, "layer"):
            raise TypeError("source_encoder does not look like a DebertaV2Encoder")

        self.backend = backend
        self.fp32_precision = fp32_precision
        self.relative_attention = getattr(source_encoder, "relative_attention", False)
        self.max_relative_positions = getattr(
            source_encoder, "max_relative_positions", getattr(config, "max_position_embeddings", 512)
        )
        self.position_buckets = getattr(source_encoder, "position_buckets", -1)
        self.norm_rel_ebd = list(getattr(source_encoder, "norm_rel_ebd", ["none"]))
        self.gradient_checkpointing = False

        # Same attribute names as Hugging Face: checkpoint keys stay stable.
        self.layer = source_encoder.layer
        if self.relative_attention:
            self.rel_embeddings = source_encoder.rel_embeddings
        if hasattr(source_encoder, "LayerNorm"):
            self.LayerNorm = source_encoder.LayerNorm
        self.conv = getattr(source_encoder, "conv", None)

        span = self.position_buckets if self.position_buckets > 0 else self.max_relative_positions
        types_ = normalise_pos_att_type(getattr(config, "pos_att_type", ()) or ())
        self.position_plan_cache = SharedPositionPlanCache(
            position_buckets=self.position_buckets,
            max_relative_positions=self.max_relative_positions,
            position_embedding_size=span,
            uses_position_bias=self.relative_attention and bool({"c2p", "p2c"} & set(types_)),
        )

        for layer in self.layer:
            original = layer.attention.self
            if isinstance(original, DisentangledFlashAttention):
                replacement = original.set_position_plan_cache(self.position_plan_cache)
            else:
                replacement = DisentangledFlashAttention(
                    config, position_plan_cache=self.position_plan_cache, fp32_precision=fp32_precision
                )
                replacement.load_state_dict(original.state_dict(), strict=True)
                replacement.to(device=original.query_proj.weight.device, dtype=original.query_proj.weight.dtype)
                replacement.train(original.training)
            layer.attention.self = replacement

        self._prepared_plans: dict[int, tuple[B200PreparedPositionPlan, ...]] = {}
        self._active_sequence_length: int | None = None
        self._active_plans: tuple[B200PreparedPositionPlan, ...] | None = None
        self.register_load_state_dict_post_hook(_invalidate_encoder_cache_after_load)

    # ----------------------------------------------------------- HF-like API
    def get_rel_embedding(self) -> torch.Tensor | None:
        relative = self.rel_embeddings.weight if self.relative_attention else None
        if relative is not None and "layer_norm" in self.norm_rel_ebd:
            relative = self.LayerNorm(relative)
        return relative

    def get_attention_mask(self, attention_mask: torch.Tensor) -> torch.Tensor:
        if attention_mask.dim() != 2:
            raise ValueError("the inference encoder requires attention_mask with shape [B, L]")
        return attention_mask

    def get_rel_pos(self, *args: Any, **kwargs: Any) -> None:
        return None

    def _attention_modules(self) -> tuple[DisentangledFlashAttention, ...]:
        return tuple(layer.attention.self for layer in self.layer)

    # ---------------------------------------------------- cache invalidation
    def clear_inference_cache(self) -> None:
        self._prepared_plans.clear()
        self._active_sequence_length = None
        self._active_plans = None
        self.position_plan_cache.clear()
        for attention in self._attention_modules():
            attention.clear_inference_cache()

    def train(self, mode: bool = True) -> "DebertaV2InferenceEncoder":
        if mode and hasattr(self, "_prepared_plans"):
            self.clear_inference_cache()
        return super().train(mode)

    def _apply(self, fn: Any, recurse: bool = True) -> "DebertaV2InferenceEncoder":
        result = super()._apply(fn, recurse=recurse)
        if hasattr(self, "_prepared_plans"):
            self.clear_inference_cache()
        return result

    # ------------------------------------------------------------ preparation
    @torch.no_grad()
    def prepare_for_inference(self, sequence_lengths: int | Iterable[int]) -> "DebertaV2InferenceEncoder":
        """Prepare every layer and every selected production bucket."""

        if self.training:
            raise RuntimeError("prepare_for_inference() requires encoder.eval()")
        if isinstance(sequence_lengths, int):
            lengths: tuple[int, ...] = (sequence_lengths,)
        else:
            lengths = tuple(dict.fromkeys(int(length) for length in sequence_lengths))
        if not lengths or any(length < 1 for length in lengths):
            raise ValueError("sequence_lengths must contain positive integers")

        self.clear_inference_cache()
        rel_embeddings = self.get_rel_embedding()
        attentions = self._attention_modules()
        for attention in attentions:
            attention.eval().prepare_for_inference(rel_embeddings)
        device = attentions[0].query_proj.weight.device
        for length in lengths:
            self._prepared_plans[length] = tuple(a.prepare_shape(length, device) for a in attentions)
        self.activate_shape(lengths[0])
        return self

    def activate_shape(self, sequence_length: int) -> "DebertaV2InferenceEncoder":
        """Select a prebuilt bucket outside the hot path."""

        try:
            plans = self._prepared_plans[sequence_length]
        except KeyError as error:
            raise ValueError(
                f"sequence length {sequence_length} was not prepared; available buckets: "
                f"{sorted(self._prepared_plans)}"
            ) from error
        self._active_sequence_length = sequence_length
        self._active_plans = plans
        return self

    # ---------------------------------------------------------------- forward
    def _validate_forward(self, hidden_states, attention_mask, output_attentions, query_states, relative_pos):
        if self.training:
            raise RuntimeError("DebertaV2InferenceEncoder requires model.eval()")
        if torch.is_grad_enabled():
            raise RuntimeError("DebertaV2InferenceEncoder requires torch.no_grad() or inference_mode()")
        if output_attentions:
            raise ValueError("output_attentions=True is not supported")
        if query_states is not None:
            raise ValueError("query_states/z_steps are not supported by the inference path")
        if relative_pos is not None:
            raise ValueError("custom relative_pos is not supported by the inference path")
        if attention_mask.dim() != 2:
            raise ValueError("attention_mask must have shape [B, L]")
        if attention_mask.shape[:2] != hidden_states.shape[:2]:
            raise ValueError("attention_mask and hidden_states must have matching [B, L]")
        if self._active_plans is None or self._active_sequence_length is None:
            raise RuntimeError("call prepare_for_inference() before forward()")
        if hidden_states.size(1) != self._active_sequence_length:
            raise ValueError(
                f"active bucket length {self._active_sequence_length} does not match "
                f"input length {hidden_states.size(1)}; call activate_shape() first"
            )
        return self._active_plans

    def forward_prepared(self, hidden_states: torch.Tensor, attention_mask: torch.Tensor,
                         plans: tuple[B200PreparedPositionPlan, ...], *, output_hidden_states: bool = True,
                         return_dict: bool = True) -> Any:
        """Layer loop with the 2-D mask and prepared plans."""

        all_hidden_states = (hidden_states,) if output_hidden_states else None
        next_kv = hidden_states
        input_mask = attention_mask
        # One dtype conversion per forward instead of one per layer: the kernel
        # reads bool / integer masks directly.
        kernel_mask = attention_mask
        if attention_mask.dtype.is_floating_point:
            kernel_mask = attention_mask.bool()
        output_states = hidden_states
        for index, (layer, plan) in enumerate(zip(self.layer, plans)):
            self_output, _ = layer.attention.self.forward_prepared(next_kv, kernel_mask, plan)
            attention_output = layer.attention.output(self_output, next_kv)
            intermediate_output = layer.intermediate(attention_output)
            output_states = layer.output(intermediate_output, attention_output)
            if index == 0 and self.conv is not None:
                output_states = self.conv(hidden_states, output_states, input_mask)
            if output_hidden_states:
                all_hidden_states = all_hidden_states + (output_states,)
            next_kv = output_states

        if not return_dict:
            return tuple(v for v in (output_states, all_hidden_states, None) if v is not None)
        return BaseModelOutput(last_hidden_state=output_states, hidden_states=all_hidden_states, attentions=None)

    def forward(self, hidden_states: torch.Tensor, attention_mask: torch.Tensor, output_hidden_states: bool = True,
                output_attentions: bool = False, query_states: torch.Tensor | None = None,
                relative_pos: torch.Tensor | None = None, return_dict: bool = True) -> Any:
        plans = self._validate_forward(hidden_states, attention_mask, output_attentions, query_states, relative_pos)
        return self.forward_prepared(hidden_states, attention_mask, plans,
                                     output_hidden_states=output_hidden_states, return_dict=return_dict)


def enable_deberta_inference(model: nn.Module, *, backend: str = "b200",
                             sequence_lengths: Iterable[int] | int | None = None,
                             fp32_precision: str = "strict") -> nn.Module:
    """Replace a HF DeBERTa-v2/v3 encoder in place without changing checkpoint keys.

    ``model`` must be the backbone (the object with ``embeddings`` and
    ``encoder``).  Same contract as the reference's function of this name
    (``deberta.py:313-346``).
    """

    if not hasattr(model, "encoder") or not hasattr(model, "embeddings"):
        raise TypeError("model must be a Hugging Face DeBERTa-v2/v3 backbone")
    if getattr(model, "z_steps", 0) > 1:
        raise ValueError("DeBERTa z_steps > 1 is not supported by the inference path")
    if isinstance(model.encoder, DebertaV2InferenceEncoder):
        raise TypeError("the model already uses DebertaV2InferenceEncoder")
    was_training = model.training
    if sequence_lengths is not None and was_training:
        raise RuntimeError("call model.eval() before preparing inference buckets")
    model.encoder = DebertaV2InferenceEncoder(model.encoder, model.config, backend=backend,
                                              fp32_precision=fp32_precision)
    model.train(was_training)
    if sequence_lengths is not None:
        model.encoder.prepare_for_inference(sequence_lengths)
    return model


def optimize_deberta(model: nn.Module, *, sequence_lengths: Iterable[int] | int | None = None,
                     fp32_precision: str = "strict") -> nn.Module:
    """Enable the fused B200 backend on a Hugging Face DeBERTa backbone."""

    return enable_deberta_inference(model, backend="b200", sequence_lengths=sequence_lengths,
                                    fp32_precision=fp32_precision)


def compile_deberta_buckets(
    encoder: DebertaV2InferenceEncoder,
    sequence_lengths: Iterable[int] | None = None,
    *,
    mode: str = "max-autotune-no-cudagraphs",
    fullgraph: bool = True,
    dynamic_batch: bool = True,
    examples: Mapping[int, tuple[torch.Tensor, torch.Tensor]] | None = None,
) -> dict[int, Callable[[torch.Tensor, torch.Tensor], torch.Tensor]]:
    """One ``torch.compile``-d callable per prepared bucket (reference ``deberta.py:349-427``).

    Compilation only concerns the PyTorch modules around the attention; the
    attention itself is the opaque custom op
    ``disentangled_flash_b200::attention_forward`` and is never traced into.
    """

    if sequence_lengths is None:
        lengths = tuple(sorted(encoder._prepared_plans))
    else:
        lengths = tuple(dict.fromkeys(int(length) for length in sequence_lengths))
    missing = [length for length in lengths if length not in encoder._prepared_plans]
    if missing:
        raise ValueError(f"unprepared bucket lengths: {missing}")

    isolate = "isolate_recompiles" in inspect.signature(torch.compile).parameters
    compiled: dict[int, Callable[[torch.Tensor, torch.Tensor], torch.Tensor]] = {}

    def make_forward(plans):
        def bucket_forward(hidden_states: torch.Tensor, attention_mask: torch.Tensor) -> torch.Tensor:
            return encoder.forward_prepared(hidden_states, attention_mask, plans,
                                            output_hidden_states=False).last_hidden_state
        return bucket_forward

    for length in lengths:
        function = make_forward(encoder._prepared_plans[length])
        kwargs: dict[str, Any] = {"mode": mode, "fullgraph": fullgraph, "dynamic": dynamic_batch}
        if isolate:
            kwargs["isolate_recompiles"] = True
        else:
            # Distinct code object per bucket so that buckets do not share one recompile budget.
            clone = types.FunctionType(function.__code__.replace(), function.__globals__,
                                       name=f"deberta_bucket_{length}", argdefs=function.__defaults__,
                                       closure=function.__closure__)
            clone.__kwdefaults__ = function.__kwdefaults__
            function = clone
        compiled[length] = torch.compile(function, **kwargs)

    if examples is not None:
        with torch.inference_mode():
            for length, function in compiled.items():
                if length not in examples:
                    raise ValueError(f"missing compilation example for bucket {length}")
                hidden_states, attention_mask = examples[length]
                if hidden_states.size(1) != length:
                    raise ValueError(f"bucket {length} example has sequence length {hidden_states.size(1)}")
                function(hidden_states, attention_mask)
    return compiled


enable_deberta_v2_inference = enable_deberta_inference

__all__ = [
    "BaseModelOutput",
    "DebertaV2InferenceEncoder",
    "compile_deberta_buckets",
    "enable_deberta_inference",
    "enable_deberta_v2_inference",
    "optimize_deberta",
]
