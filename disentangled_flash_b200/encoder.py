"""Encoder-level drop-in: ``optimize_deberta`` / ``enable_deberta_inference``.

Plays the role of the reference's encoder wrapper and public API
(``src/disentangled_flash/deberta.py:38-447``): the names, signatures,
exception classes and messages a user of the reference relies on are kept, the
implementation is this package's own.

The wrapper adopts a Hugging Face ``DebertaV2Encoder`` without changing a
checkpoint key: the layer list, ``rel_embeddings``, ``LayerNorm`` and ``conv``
are the caller's modules, only ``layer.attention.self`` is exchanged for
:class:`DisentangledFlashAttention`.  Per sequence-length bucket it keeps one
tuple of per-layer position plans (a ``_BucketTable``); a forward pass walks the
layers with the 2-D padding mask and the active tuple.  No ``[B,1,L,L]`` mask
and no ``[L,L]`` relative-position tensor exists at any point.

Outside ``attention.self`` the dense projections, the activation and the
layer-0 convolution stay the caller's PyTorch modules; the tail of the two
output blocks of a layer, ``LayerNorm(dense(x) + residual)``, runs the add and
the norm as one kernel (``dfl_add_layernorm``) when the block has the Hugging
Face shape (``dense`` / ``LayerNorm`` / ``dropout``), and a 16-bit
``gelu(dense(x))`` intermediate block runs as one GEMM with the bias and the
GELU in its epilogue (``dfl_dense``); the layer-0 convolution branch runs as a
GEMM over the taps (``dfl_conv1d``) plus the masked add-and-norm when it is a
plain ``nn.Conv1d`` with ``tanh`` or ``gelu`` in a 16-bit type and the bucket has
at least 256 positions.  There is one backend;
``backend="triton"`` is accepted as the legacy name of the fused backend and
``backend="torch"`` is refused because no CPU/PyTorch attention ships here.
"""

from __future__ import annotations

from collections.abc import Callable, Iterable, Mapping
from dataclasses import dataclass
from typing import Any, Optional

import torch
from torch import nn
from torch.nn import functional as F

from . import _cabi
from .attention import B200PreparedPositionPlan, DisentangledFlashAttention
from .config import normalise_pos_att_type
from .position import SharedPositionPlanCache

FUSED_BACKENDS = ("b200", "triton")
_REFUSED_BACKENDS = ("torch", "optimized")

Plans = tuple[B200PreparedPositionPlan, ...]


@dataclass
class BaseModelOutput:
    """Minimal stand-in for Transformers' ``BaseModelOutput`` (indexable like a tuple)."""

    last_hidden_state: torch.Tensor
    hidden_states: tuple[torch.Tensor, ...] | None = None
    attentions: tuple[torch.Tensor, ...] | None = None

    def __getitem__(self, index: int) -> Any:
        fields = (self.last_hidden_state, self.hidden_states, self.attentions)
        return [field for field in fields if field is not None][index]


def _add_layernorm(x: torch.Tensor, residual: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor],
                   eps: float) -> torch.Tensor:
    """``LayerNorm(x + residual)`` in one pass; sum and statistics in fp32 (``dfl_add_layernorm``)."""

    return _cabi.add_layernorm(x.contiguous(), residual.contiguous(), weight, bias, eps)


_add_layernorm_op = torch.library.custom_op("disentangled_flash_b200::add_layernorm", mutates_args=(),
                                            device_types="cuda")(_add_layernorm)


@_add_layernorm_op.register_fake
def _add_layernorm_fake(x, residual, weight, bias, eps):
    return torch.empty_like(x, memory_format=torch.contiguous_format)


def _dense_gelu(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor],
                status: Optional[torch.Tensor]) -> torch.Tensor:
    """``gelu(x @ weight^T + bias)`` (erf form) with bias and activation in the GEMM epilogue (``dfl_dense``)."""

    return _cabi.dense(x.contiguous(), weight, bias, activation=_cabi.ACT_GELU, status=status)


_dense_gelu_op = torch.library.custom_op("disentangled_flash_b200::dense_gelu", mutates_args=("status",),
                                         device_types="cuda")(_dense_gelu)


@_dense_gelu_op.register_fake
def _dense_gelu_fake(x, weight, bias, status):
    return x.new_empty(*x.shape[:-1], weight.shape[0])


def _conv_branch(hidden_states: torch.Tensor, residual: torch.Tensor, attention_mask: torch.Tensor,
                 conv_weight: torch.Tensor, conv_bias: Optional[torch.Tensor], norm_weight: torch.Tensor,
                 norm_bias: Optional[torch.Tensor], eps: float, activation: int,
                 status: Optional[torch.Tensor]) -> torch.Tensor:
    """The layer-0 convolution branch, ``keep * LayerNorm(residual + act(keep * conv1d(hidden_states)))``
    (``_reference.py:534-568``), as two kernels: ``dfl_conv1d`` (GEMM over the taps with bias, mask and activation in
    its epilogue) and ``dfl_add_layernorm`` (with the mask)."""

    keep = attention_mask
    if keep.dtype not in (torch.bool, torch.uint8, torch.int32, torch.int64):
        keep = keep != 0
    keep = keep.contiguous()
    out = _cabi.conv1d(hidden_states.contiguous(), conv_weight, conv_bias, keep, activation=activation, status=status)
    return _cabi.add_layernorm(out, residual.contiguous(), norm_weight, norm_bias, eps, out=out, row_mask=keep)


_conv_branch_op = torch.library.custom_op("disentangled_flash_b200::conv_branch", mutates_args=("status",),
                                          device_types="cuda")(_conv_branch)


@_conv_branch_op.register_fake
def _conv_branch_fake(hidden_states, residual, attention_mask, conv_weight, conv_bias, norm_weight, norm_bias, eps,
                      activation, status):
    return torch.empty_like(residual, memory_format=torch.contiguous_format)


_CONV_ACTIVATIONS = {"tanh": _cabi.ACT_TANH, "gelu": _cabi.ACT_GELU}


def _conv_activation(module: nn.Module) -> int | None:
    """Activation code of a Hugging Face ``ConvLayer`` if the branch has the shape the fused kernels cover."""

    conv, norm = getattr(module, "conv", None), getattr(module, "LayerNorm", None)
    if not (isinstance(conv, nn.Conv1d) and isinstance(norm, nn.LayerNorm) and norm.weight is not None):
        return None
    if not {name for name, _ in module.named_children()} <= {"conv", "LayerNorm", "dropout"}:
        return None
    taps = conv.kernel_size[0]
    plain = (conv.groups == 1 and conv.stride == (1,) and conv.dilation == (1,) and conv.padding_mode == "zeros"
             and taps % 2 == 1 and conv.padding == ((taps - 1) // 2,))
    if not plain or not conv.weight.is_cuda or conv.weight.dtype != norm.weight.dtype:
        return None
    return _CONV_ACTIVATIONS.get(getattr(module, "conv_act", None))


def _is_erf_gelu(fn: Any) -> bool:
    """``torch.nn.functional.gelu`` in its erf form, as a function, an ``nn.GELU`` or a wrapper module around it."""

    if fn is F.gelu:
        return True
    if isinstance(fn, nn.GELU):
        return fn.approximate == "none"
    return isinstance(fn, nn.Module) and getattr(fn, "act", None) is F.gelu   # Transformers' GELUActivation


def _intermediate_is_fusable(block: nn.Module) -> bool:
    """Whether ``block`` is ``gelu(dense(x))`` in the Hugging Face shape (``_reference.py:461-471``) in a 16-bit type
    on a CUDA device, with row lengths the tensor-core GEMM takes."""

    dense = getattr(block, "dense", None)
    if not isinstance(dense, nn.Linear) or not _is_erf_gelu(getattr(block, "intermediate_act_fn", None)):
        return False
    if not {name for name, _ in block.named_children()} <= {"dense", "intermediate_act_fn"}:
        return False
    weight = dense.weight
    return (weight.is_cuda and weight.dtype in (torch.float16, torch.bfloat16)
            and weight.shape[0] % 8 == 0 and weight.shape[1] % 8 == 0
            and (dense.bias is None or dense.bias.dtype == weight.dtype))


def _op(operator, function):
    """The custom operator while a forward is being traced, the plain function otherwise: the dispatcher's way into
    a Python operator costs more host time than the smaller kernels run."""

    return operator if torch.compiler.is_compiling() else function


_OUTPUT_BLOCK_CHILDREN = frozenset(("dense", "LayerNorm", "dropout"))


def _output_block_is_fusable(block: nn.Module) -> bool:
    """Whether ``block`` is ``LayerNorm(dropout(dense(x)) + residual)`` in the Hugging Face shape
    (``_reference.py:101-112``, ``474-485``) at a size and type ``dfl_add_layernorm`` covers.  Decided when a bucket
    is prepared, not in the forward pass."""

    dense, norm = getattr(block, "dense", None), getattr(block, "LayerNorm", None)
    if not (isinstance(dense, nn.Linear) and isinstance(norm, nn.LayerNorm) and norm.weight is not None):
        return False
    if not {name for name, _ in block.named_children()} <= _OUTPUT_BLOCK_CHILDREN:
        return False
    weight = norm.weight
    return (weight.is_cuda and len(norm.normalized_shape) == 1 and dense.weight.dtype == weight.dtype
            and _cabi.add_layernorm_supported(weight.dtype, norm.normalized_shape[0]))


def _output_block(block: nn.Module, fused: bool, projected: torch.Tensor, residual: torch.Tensor) -> torch.Tensor:
    """A layer's output block; with ``fused`` the add and the norm are one kernel (the encoder runs in eval mode,
    so the block's dropout is the identity)."""

    if not fused or projected.dtype != block.LayerNorm.weight.dtype or residual.dtype != projected.dtype:
        return block(projected, residual)
    dense, norm = block.dense, block.LayerNorm
    return _op(_add_layernorm_op, _add_layernorm)(F.linear(projected, dense.weight, dense.bias), residual, norm.weight, norm.bias,
                             float(norm.eps))


class _BucketTable:
    """Prepared plans per sequence length, and which of them is active."""

    def __init__(self) -> None:
        self.by_length: dict[int, Plans] = {}
        self.active_length: int | None = None
        self.active: Plans | None = None

    def reset(self) -> None:
        self.by_length.clear()
        self.active_length = None
        self.active = None

    def select(self, sequence_length: int) -> None:
        plans = self.by_length.get(sequence_length)
        if plans is None:
            raise ValueError(
                f"sequence length {sequence_length} was not prepared; available buckets: {sorted(self.by_length)}"
            )
        self.active_length, self.active = sequence_length, plans

    def require(self, lengths: Iterable[int]) -> tuple[int, ...]:
        wanted = _unique_lengths(lengths)
        absent = [length for length in wanted if length not in self.by_length]
        if absent:
            raise ValueError(f"unprepared bucket lengths: {absent}")
        return wanted


def _unique_lengths(lengths: int | Iterable[int]) -> tuple[int, ...]:
    items = [lengths] if isinstance(lengths, int) else list(lengths)
    seen: list[int] = []
    for item in items:
        value = int(item)
        if value not in seen:
            seen.append(value)
    return tuple(seen)


def _adopt_attention(layer: nn.Module, config: Any, cache: SharedPositionPlanCache, fp32_precision: str) -> None:
    """Exchange ``layer.attention.self`` for the fused module, carrying parameters, placement and mode over."""

    current = layer.attention.self
    if isinstance(current, DisentangledFlashAttention):
        current.set_position_plan_cache(cache)
        return
    fused = DisentangledFlashAttention(config, position_plan_cache=cache, fp32_precision=fp32_precision)
    fused.load_state_dict(current.state_dict(), strict=True)
    anchor = current.query_proj.weight
    fused.to(device=anchor.device, dtype=anchor.dtype)
    fused.train(current.training)
    layer.attention.self = fused


def _drop_plans_after_load(module: nn.Module, _incompatible_keys: Any) -> None:
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
        if backend in _REFUSED_BACKENDS:
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
        self.gradient_checkpointing = False

        # geometry of the relative-position scheme, as the source encoder states it
        self.relative_attention = bool(getattr(source_encoder, "relative_attention", False))
        fallback_positions = getattr(config, "max_position_embeddings", 512)
        self.max_relative_positions = getattr(source_encoder, "max_relative_positions", fallback_positions)
        self.position_buckets = getattr(source_encoder, "position_buckets", -1)
        self.norm_rel_ebd = list(getattr(source_encoder, "norm_rel_ebd", ["none"]))

        # the caller's modules under their Hugging Face names: checkpoint keys do not move
        self.layer = source_encoder.layer
        for name in ("rel_embeddings", "LayerNorm"):
            if (name != "rel_embeddings" or self.relative_attention) and hasattr(source_encoder, name):
                setattr(self, name, getattr(source_encoder, name))
        self.conv = getattr(source_encoder, "conv", None)

        terms = set(normalise_pos_att_type(getattr(config, "pos_att_type", ()) or ()))
        self.position_plan_cache = SharedPositionPlanCache(
            position_buckets=self.position_buckets,
            max_relative_positions=self.max_relative_positions,
            position_embedding_size=self.position_buckets if self.position_buckets > 0 else self.max_relative_positions,
            uses_position_bias=self.relative_attention and not terms.isdisjoint(("c2p", "p2c")),
        )
        for layer in self.layer:
            _adopt_attention(layer, config, self.position_plan_cache, fp32_precision)

        self._buckets = _BucketTable()
        self._fused_output_blocks: list[tuple[bool, bool]] = [(False, False)] * len(self.layer)
        self._fused_intermediates: list[bool] = [False] * len(self.layer)
        self._conv_fused: dict[int, bool] = {}       # per bucket length: the fused convolution branch covers it
        self._packed_qkv: dict[Any, tuple[torch.Tensor, ...]] = {}   # head-major Q/K/V buffers of forward_packed
        self._conv_weight: torch.Tensor | None = None   # nn.Conv1d weight as [taps, out, in]
        self._conv_activation_code = 0
        self._status_word: torch.Tensor | None = None
        self.register_load_state_dict_post_hook(_drop_plans_after_load)

    # ----------------------------------------------------------- HF-like API
    def get_rel_embedding(self) -> torch.Tensor | None:
        if not self.relative_attention:
            return None
        table = self.rel_embeddings.weight
        return self.LayerNorm(table) if "layer_norm" in self.norm_rel_ebd else table

    def get_attention_mask(self, attention_mask: torch.Tensor) -> torch.Tensor:
        if attention_mask.dim() != 2:
            raise ValueError("the inference encoder requires attention_mask with shape [B, L]")
        return attention_mask

    def get_rel_pos(self, *args: Any, **kwargs: Any) -> None:
        return None

    def _attention_modules(self) -> list[DisentangledFlashAttention]:
        return [layer.attention.self for layer in self.layer]

    # the reference's tests and tooling look these up
    @property
    def _prepared_plans(self) -> dict[int, Plans]:
        return self._buckets.by_length

    @property
    def _active_sequence_length(self) -> int | None:
        return self._buckets.active_length

    @property
    def _active_plans(self) -> Plans | None:
        return self._buckets.active

    # ---------------------------------------------------- cache invalidation
    def clear_inference_cache(self) -> None:
        """Forget every bucket and everything derived from the parameters (three triggers: ``train()``,
        ``_apply`` i.e. ``.to()/.half()/...``, and ``load_state_dict``)."""

        self._buckets.reset()
        self._conv_fused, self._conv_weight = {}, None
        self._packed_qkv = {}
        self.position_plan_cache.clear()
        for attention in self._attention_modules():
            attention.clear_inference_cache()

    def train(self, mode: bool = True) -> "DebertaV2InferenceEncoder":
        if mode and "_buckets" in self.__dict__:
            self.clear_inference_cache()
        return super().train(mode)

    def _apply(self, fn: Any, recurse: bool = True) -> "DebertaV2InferenceEncoder":
        applied = super()._apply(fn, recurse=recurse)
        if "_buckets" in self.__dict__:
            self.clear_inference_cache()
        return applied

    # ------------------------------------------------------------ preparation
    @torch.no_grad()
    def prepare_for_inference(self, sequence_lengths: int | Iterable[int]) -> "DebertaV2InferenceEncoder":
        """Prepare every layer and every selected production bucket."""

        if self.training:
            raise RuntimeError("prepare_for_inference() requires encoder.eval()")
        lengths = _unique_lengths(sequence_lengths)
        if not lengths or min(lengths) < 1:
            raise ValueError("sequence_lengths must contain positive integers")
        self.clear_inference_cache()
        relative = self.get_rel_embedding()
        modules = self._attention_modules()
        device = modules[0].query_proj.weight.device
        # one status word for all layers: a bounded device-side wait that expires anywhere in the encoder shows up in
        # check_device_status()
        self._status_word = _cabi.new_status_word(device) if device.type == "cuda" else None
        for module in modules:
            module.eval()
            module.prepare_for_inference(relative)
            module.set_status_word(self._status_word)
        for length in lengths:
            self._buckets.by_length[length] = tuple(module.prepare_shape(length, device) for module in modules)
        self._buckets.select(lengths[0])
        self._fused_output_blocks = [
            (_output_block_is_fusable(layer.attention.output), _output_block_is_fusable(layer.output))
            for layer in self.layer
        ] if device.type == "cuda" else [(False, False)] * len(self.layer)
        self._fused_intermediates = [device.type == "cuda" and _intermediate_is_fusable(layer.intermediate)
                                     for layer in self.layer]
        self._conv_fused, self._conv_weight = {}, None
        activation = _conv_activation(self.conv) if self.conv is not None and device.type == "cuda" else None
        if activation is not None:
            weight = self.conv.conv.weight   # [out, in, taps]
            c_out, c_in, taps = weight.shape
            self._conv_activation_code = activation
            self._conv_fused = {length: _cabi.conv1d_supported(weight.dtype, length, c_in, c_out, taps, activation)
                                for length in lengths}
            if any(self._conv_fused.values()):
                self._conv_weight = weight.detach().permute(2, 0, 1).contiguous()
        return self

    def activate_shape(self, sequence_length: int) -> "DebertaV2InferenceEncoder":
        """Select a prebuilt bucket outside the hot path."""

        self._buckets.select(sequence_length)
        return self

    def check_device_status(self) -> None:
        """Raise ``DflError`` (``DFL_ERR_DEVICE_TIMEOUT``) if a bounded device-side wait expired in any layer since the
        last check.  Synchronises the current stream: for the end of a batch, not for the hot path."""

        if self._status_word is not None:
            _cabi.check_status(self._status_word)

    # ---------------------------------------------------------------- forward
    def _validate_forward(self, hidden_states, attention_mask, output_attentions, query_states, relative_pos) -> Plans:
        refusals = (
            (self.training, RuntimeError, "DebertaV2InferenceEncoder requires model.eval()"),
            (torch.is_grad_enabled(), RuntimeError,
             "DebertaV2InferenceEncoder requires torch.no_grad() or inference_mode()"),
            (bool(output_attentions), ValueError, "output_attentions=True is not supported"),
            (query_states is not None, ValueError, "query_states/z_steps are not supported by the inference path"),
            (relative_pos is not None, ValueError, "custom relative_pos is not supported by the inference path"),
            (attention_mask.dim() != 2, ValueError, "attention_mask must have shape [B, L]"),
        )
        for refused, error, message in refusals:
            if refused:
                raise error(message)
        if tuple(attention_mask.shape) != tuple(hidden_states.shape[:2]):
            raise ValueError("attention_mask and hidden_states must have matching [B, L]")
        table = self._buckets
        if table.active is None:
            raise RuntimeError("call prepare_for_inference() before forward()")
        if hidden_states.size(1) != table.active_length:
            raise ValueError(
                f"active bucket length {table.active_length} does not match "
                f"input length {hidden_states.size(1)}; call activate_shape() first"
            )
        return table.active

    def forward_prepared(self, hidden_states: torch.Tensor, attention_mask: torch.Tensor,
                         plans: Plans, *, output_hidden_states: bool = True, return_dict: bool = True) -> Any:
        """Layer loop with the 2-D mask and prepared plans."""

        # The kernels test bool / integer mask elements for non-zero themselves; a floating-point mask is turned
        # into bool here, once per forward and not once per layer.
        keep = attention_mask.bool() if attention_mask.dtype.is_floating_point else attention_mask
        trace = [hidden_states] if output_hidden_states else None
        state = hidden_states
        for depth, layer in enumerate(self.layer):
            context, _ = layer.attention.self.forward_prepared(state, keep, plans[depth])
            fuse_attention_output, fuse_output = self._fused_output_blocks[depth]
            mixed = _output_block(layer.attention.output, fuse_attention_output, context, state)
            if self._fused_intermediates[depth] and mixed.dtype == layer.intermediate.dense.weight.dtype:
                dense = layer.intermediate.dense
                inner = _op(_dense_gelu_op, _dense_gelu)(mixed, dense.weight, dense.bias, self._status_word)
            else:
                inner = layer.intermediate(mixed)
            state = _output_block(layer.output, fuse_output, inner, mixed)
            if depth == 0 and self.conv is not None:
                # the convolution branch sees the encoder input and the padding mask as the caller gave it
                if self._conv_fused.get(hidden_states.size(1), False) and hidden_states.dtype == state.dtype:
                    norm = self.conv.LayerNorm
                    state = _op(_conv_branch_op, _conv_branch)(hidden_states, state, attention_mask, self._conv_weight,
                                            self.conv.conv.bias, norm.weight, norm.bias, float(norm.eps),
                                            self._conv_activation_code, self._status_word)
                else:
                    state = self.conv(hidden_states, state, attention_mask)
            if trace is not None:
                trace.append(state)
        collected = None if trace is None else tuple(trace)
        if return_dict:
            return BaseModelOutput(last_hidden_state=state, hidden_states=collected, attentions=None)
        return (state,) if collected is None else (state, collected)

    def forward_packed(self, hidden_states: torch.Tensor, attention_mask: torch.Tensor,
                       lengths: Iterable[int]) -> BaseModelOutput:
        """Forward of a right-padded batch without the padding: between the attention kernels the layers run on the
        valid positions only, packed into consecutive rows (each sequence rounded up to 32 rows).

        ``lengths`` are the valid lengths on the host (what a tokenizer returns); ``attention_mask`` must be the
        matching prefix mask.  The result equals ``forward`` at the valid positions; padded positions of
        ``last_hidden_state`` are unspecified (zero beyond each sequence's 32-row block), where the reference carries
        values through every layer - the reason this is a method of its own and not the default.  Needs every layer's
        blocks fused (a 16-bit Hugging Face shaped encoder on the single-launch attention path)."""

        plans = self._validate_forward(hidden_states, attention_mask, False, None, None)
        if not (all(a and b for a, b in self._fused_output_blocks) and all(self._fused_intermediates)):
            raise NotImplementedError("forward_packed needs the fused output and intermediate blocks in every layer")
        batch, length, hidden = hidden_states.shape
        valid = [int(n) for n in lengths]
        if len(valid) != batch or min(valid) < 0 or max(valid) > length:
            raise ValueError("lengths must hold one length in [0, L] per sequence")
        counts = [min(length, -(-n // 32) * 32) for n in valid]
        bases = [0] * batch
        for b in range(1, batch):
            bases[b] = bases[b - 1] + counts[b - 1]
        total = bases[-1] + counts[-1]
        if total == 0:
            raise ValueError("forward_packed needs at least one valid position")
        device = hidden_states.device
        source_rows = torch.cat([torch.arange(b * length, b * length + counts[b], dtype=torch.int32)
                                 for b in range(batch)])
        pack_rows = source_rows.to(device, non_blocking=True)
        row_base = torch.tensor(bases, dtype=torch.int32).to(device, non_blocking=True)
        row_count = torch.tensor(counts, dtype=torch.int32).to(device, non_blocking=True)
        packed = (row_base, row_count, total)

        keep = attention_mask.bool() if attention_mask.dtype.is_floating_point else attention_mask
        state_u = hidden_states.contiguous()
        state_p = _cabi.copy_rows(state_u.view(batch * length, hidden), pack_rows)
        # With a bucket length in multiples of 32 the QKV projection reads the packed rows too and writes each group
        # of 32 rows to its place in head-major buffers that are kept from call to call (rows no call has written
        # yet are zero, later ones hold finite leftovers: masked keys must not be NaN).  The unpacked state is then
        # needed only by the layer-0 convolution and as the result.
        project_packed = length % 32 == 0
        packed_input = None
        if project_packed:
            group_rows = torch.cat([torch.arange(b * length, b * length + counts[b], 32, dtype=torch.int32)
                                    for b in range(batch)]).to(device, non_blocking=True)
            first = self.layer[0].attention.self
            key = (batch, length, first.num_attention_heads, first.attention_head_size, hidden_states.dtype, device)
            buffers = self._packed_qkv.get(key)
            if buffers is None:
                buffers = tuple(torch.zeros(batch, first.num_attention_heads, length, first.attention_head_size,
                                            dtype=hidden_states.dtype, device=device) for _ in range(3))
                self._packed_qkv = {key: buffers}      # one shape at a time: 3 x B x L x hidden elements
            packed_input = (group_rows, buffers)
        unpacked = [torch.zeros(batch * length, hidden, dtype=hidden_states.dtype, device=device)
                    for _ in range(1 if project_packed else 2)]
        last = len(self.layer) - 1
        for depth, layer in enumerate(self.layer):
            if project_packed:
                context = layer.attention.self.forward_packed_rows(state_p, keep, plans[depth], packed,
                                                                   packed_input=packed_input)
            else:
                context = layer.attention.self.forward_packed_rows(state_u, keep, plans[depth], packed)
            block = layer.attention.output
            projected = F.linear(context, block.dense.weight, block.dense.bias)
            mixed = _cabi.add_layernorm(projected, state_p, block.LayerNorm.weight, block.LayerNorm.bias,
                                        float(block.LayerNorm.eps), out=projected)
            dense = layer.intermediate.dense
            inner = _cabi.dense(mixed, dense.weight, dense.bias, activation=_cabi.ACT_GELU, status=self._status_word)
            block = layer.output
            projected = F.linear(inner, block.dense.weight, block.dense.bias)
            convolve = depth == 0 and self.conv is not None
            scatter = None
            if not project_packed or convolve or depth == last:
                target = unpacked[depth % len(unpacked)]
                scatter = (target, pack_rows)
                state_u = target.view(batch, length, hidden)
            state_p = _cabi.add_layernorm(projected, mixed, block.LayerNorm.weight, block.LayerNorm.bias,
                                          float(block.LayerNorm.eps), out=projected, scatter=scatter)
            if convolve:
                # the convolution runs along the sequence: on the unpacked layout, once per forward
                if self._conv_fused.get(length, False):
                    norm = self.conv.LayerNorm
                    state_u = _conv_branch(hidden_states, state_u, attention_mask, self._conv_weight,
                                              self.conv.conv.bias, norm.weight, norm.bias, float(norm.eps),
                                              self._conv_activation_code, self._status_word)
                else:
                    state_u = self.conv(hidden_states, state_u, attention_mask).contiguous()
                if depth != last:
                    state_p = _cabi.copy_rows(state_u.view(batch * length, hidden), pack_rows)
        return BaseModelOutput(last_hidden_state=state_u, hidden_states=None, attentions=None)

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

    if not (hasattr(model, "encoder") and hasattr(model, "embeddings")):
        raise TypeError("model must be a Hugging Face DeBERTa-v2/v3 backbone")
    if getattr(model, "z_steps", 0) > 1:
        raise ValueError("DeBERTa z_steps > 1 is not supported by the inference path")
    if isinstance(model.encoder, DebertaV2InferenceEncoder):
        raise TypeError("the model already uses DebertaV2InferenceEncoder")
    training = model.training
    if training and sequence_lengths is not None:
        raise RuntimeError("call model.eval() before preparing inference buckets")
    model.encoder = DebertaV2InferenceEncoder(model.encoder, model.config, backend=backend,
                                              fp32_precision=fp32_precision)
    model.train(training)   # the new sub-modules follow the model's mode
    if sequence_lengths is not None:
        model.encoder.prepare_for_inference(sequence_lengths)
    return model


def optimize_deberta(model: nn.Module, *, sequence_lengths: Iterable[int] | int | None = None,
                     fp32_precision: str = "strict") -> nn.Module:
    """Enable the fused B200 backend on a Hugging Face DeBERTa backbone."""

    return enable_deberta_inference(model, backend="b200", sequence_lengths=sequence_lengths,
                                    fp32_precision=fp32_precision)


_BUCKET_SOURCE = (
    "def deberta_bucket_{length}(hidden_states, attention_mask):\n"
    "    return _layers(hidden_states, attention_mask, _plans, output_hidden_states=False).last_hidden_state\n"
)


def _bucket_function(encoder: DebertaV2InferenceEncoder, length: int, plans: Plans) -> Callable:
    """A function of its own per bucket (own code object, so that ``torch.compile`` keeps one recompile budget per
    bucket), closed over the bucket's plans."""

    scope: dict[str, Any] = {"_layers": encoder.forward_prepared, "_plans": plans}
    exec(compile(_BUCKET_SOURCE.format(length=length), f"<deberta bucket {length}>", "exec"), scope)  # noqa: S102
    return scope[f"deberta_bucket_{length}"]


def compile_deberta_buckets(
    encoder: DebertaV2InferenceEncoder,
    sequence_lengths: Iterable[int] | None = None,
    *,
    mode: str = "max-autotune-no-cudagraphs",
    fullgraph: bool = True,
    dynamic_batch: bool = True,
    examples: Mapping[int, tuple[torch.Tensor, torch.Tensor]] | None = None,
) -> dict[int, Callable[[torch.Tensor, torch.Tensor], torch.Tensor]]:
    """One ``torch.compile``-d callable per prepared bucket (the reference's function of this name,
    ``deberta.py:349-427``).

    Compilation concerns the PyTorch modules around the attention only; the attention is the opaque custom op
    ``disentangled_flash_b200::attention_forward`` and is never traced into.  With ``examples`` every bucket is run
    once (under ``inference_mode``) so that compilation happens here and not on the first request.
    """

    table = encoder._buckets
    lengths = tuple(sorted(table.by_length)) if sequence_lengths is None else table.require(sequence_lengths)
    programs: dict[int, Callable[[torch.Tensor, torch.Tensor], torch.Tensor]] = {}
    for length in lengths:
        function = _bucket_function(encoder, length, table.by_length[length])
        options: dict[str, Any] = {"mode": mode, "fullgraph": fullgraph, "dynamic": dynamic_batch}
        try:   # newer PyTorch can keep recompiles of different callables apart by itself
            programs[length] = torch.compile(function, isolate_recompiles=True, **options)
        except TypeError:
            programs[length] = torch.compile(function, **options)
    if examples is not None:
        for length in lengths:
            if length not in examples:
                raise ValueError(f"missing compilation example for bucket {length}")
            hidden_states, attention_mask = examples[length]
            if hidden_states.size(1) != length:
                raise ValueError(f"bucket {length} example has sequence length {hidden_states.size(1)}")
        with torch.inference_mode():
            for length in lengths:
                programs[length](*examples[length])
    return programs


class CapturedBucket:
    """One prepared bucket at one batch size as a CUDA graph: a whole encoder forward is one graph launch.

    Calling it copies ``hidden_states`` and ``attention_mask`` into the graph's input buffers, replays the graph and
    returns the graph's output buffer - the same tensor on every call, overwritten by the next one (clone it to
    keep it).  Everything is enqueued on the current stream; nothing synchronises with the host.
    """

    def __init__(self, graph: "torch.cuda.CUDAGraph", hidden: torch.Tensor, mask: torch.Tensor, out: torch.Tensor):
        self.graph, self.hidden_states, self.attention_mask, self.last_hidden_state = graph, hidden, mask, out

    def __call__(self, hidden_states: torch.Tensor, attention_mask: torch.Tensor) -> torch.Tensor:
        if hidden_states.shape != self.hidden_states.shape or attention_mask.shape != self.attention_mask.shape:
            raise ValueError(
                f"captured for hidden_states {tuple(self.hidden_states.shape)} and attention_mask "
                f"{tuple(self.attention_mask.shape)}, got {tuple(hidden_states.shape)} and {tuple(attention_mask.shape)}"
            )
        self.hidden_states.copy_(hidden_states, non_blocking=True)
        self.attention_mask.copy_(attention_mask, non_blocking=True)
        self.graph.replay()
        return self.last_hidden_state


def capture_deberta_buckets(
    encoder: DebertaV2InferenceEncoder,
    batch_size: int | Mapping[int, int],
    sequence_lengths: Iterable[int] | None = None,
    *,
    mask_dtype: torch.dtype = torch.bool,
    warmup: int = 2,
) -> dict[int, CapturedBucket]:
    """One CUDA graph per prepared bucket at a fixed batch size (one size for all buckets, or ``{length: size}``,
    which also selects the buckets).

    A forward of a small batch is bound by the rate at which the host can launch kernels (some twenty per layer);
    a captured bucket is launched once.  The reference reaches for ``torch.compile`` here
    (``compile_deberta_buckets``, ``deberta.py:349-427``); this is the same idea with a stream capture of the
    prepared forward instead of a tracing compiler.  Each bucket is run ``warmup`` times on a side stream before it is
    captured, so that every one-time kernel configuration and lazy module load happens outside the capture.
    """

    table = encoder._buckets
    if isinstance(batch_size, Mapping):
        sizes = {int(length): int(size) for length, size in batch_size.items()}
        lengths = table.require(sorted(sizes) if sequence_lengths is None else sequence_lengths)
        if any(length not in sizes for length in lengths):
            raise ValueError("batch_size has no entry for a requested bucket")
    else:
        if int(batch_size) < 1:
            raise ValueError("batch_size must be positive")
        lengths = tuple(sorted(table.by_length)) if sequence_lengths is None else table.require(sequence_lengths)
        sizes = {length: int(batch_size) for length in lengths}
    if any(size < 1 for size in sizes.values()):
        raise ValueError("batch_size must be positive")
    anchor = encoder._attention_modules()[0].query_proj.weight
    if anchor.device.type != "cuda":
        raise RuntimeError("capture_deberta_buckets needs the encoder on a CUDA device")
    hidden_size = anchor.shape[1]
    captured: dict[int, CapturedBucket] = {}
    # the input buffers are ordinary tensors (callers copy into them outside inference mode)
    buffers = {length: (torch.zeros(sizes[length], length, hidden_size, dtype=anchor.dtype, device=anchor.device),
                        torch.ones(sizes[length], length, dtype=mask_dtype, device=anchor.device)) for length in lengths}
    with torch.cuda.device(anchor.device), torch.inference_mode():
        for length in lengths:
            plans = table.by_length[length]
            hidden, mask = buffers[length]
            side = torch.cuda.Stream(anchor.device)
            side.wait_stream(torch.cuda.current_stream(anchor.device))
            with torch.cuda.stream(side):
                for _ in range(max(1, warmup)):
                    encoder.forward_prepared(hidden, mask, plans, output_hidden_states=False)
            torch.cuda.current_stream(anchor.device).wait_stream(side)
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                out = encoder.forward_prepared(hidden, mask, plans, output_hidden_states=False).last_hidden_state
            captured[length] = CapturedBucket(graph, hidden, mask, out)
    return captured


enable_deberta_v2_inference = enable_deberta_inference

__all__ = [
    "BaseModelOutput",
    "CapturedBucket",
    "DebertaV2InferenceEncoder",
    "capture_deberta_buckets",
    "compile_deberta_buckets",
    "enable_deberta_inference",
    "enable_deberta_v2_inference",
    "optimize_deberta",
]
