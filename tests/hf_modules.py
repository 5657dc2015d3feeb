"""Minimal DeBERTa-v2/v3 encoder stack with Hugging Face module names (test and benchmark harness).

The fused kernels replace only ``layer.attention.self``; everything else in a
layer stays ordinary PyTorch.  Real deployments pass a Transformers
``DebertaV2Model``.  This file provides the same module tree (same attribute
and parameter names, same arithmetic) without depending on Transformers, so
that benchmarks and tests can build a random-initialised encoder of any
geometry offline.  ``AttentionParameters`` only holds the projection weights:
it has no forward of its own and must be replaced through
``enable_deberta_inference`` / ``DebertaV2InferenceEncoder``.
"""

from __future__ import annotations

from typing import Any

import torch
from torch import nn
from torch.nn import functional as F

from disentangled_flash_b200.config import normalise_pos_att_type

_ACTIVATIONS = {"gelu": F.gelu, "relu": F.relu, "silu": F.silu, "swish": F.silu, "tanh": torch.tanh,
                "gelu_new": lambda x: F.gelu(x, approximate="tanh")}


class AttentionParameters(nn.Module):
    """Parameter holder with the names of HF ``DisentangledSelfAttention``."""

    def __init__(self, config: Any) -> None:
        super().__init__()
        heads = config.num_attention_heads
        head_dim = getattr(config, "attention_head_size", None) or config.hidden_size // heads
        all_head = heads * head_dim
        self.query_proj = nn.Linear(config.hidden_size, all_head, bias=True)
        self.key_proj = nn.Linear(config.hidden_size, all_head, bias=True)
        self.value_proj = nn.Linear(config.hidden_size, all_head, bias=True)
        types_ = normalise_pos_att_type(getattr(config, "pos_att_type", None))
        if getattr(config, "relative_attention", False) and not getattr(config, "share_att_key", False):
            if "c2p" in types_:
                self.pos_key_proj = nn.Linear(config.hidden_size, all_head, bias=True)
            if "p2c" in types_:
                self.pos_query_proj = nn.Linear(config.hidden_size, all_head)

    def forward(self, *args: Any, **kwargs: Any):
        raise RuntimeError("AttentionParameters has no forward; wrap the encoder with enable_deberta_inference()")


class SelfOutput(nn.Module):
    def __init__(self, config: Any) -> None:
        super().__init__()
        self.dense = nn.Linear(config.hidden_size, config.hidden_size)
        self.LayerNorm = nn.LayerNorm(config.hidden_size, config.layer_norm_eps)
        self.dropout = nn.Dropout(config.hidden_dropout_prob)

    def forward(self, hidden_states: torch.Tensor, input_tensor: torch.Tensor) -> torch.Tensor:
        return self.LayerNorm(self.dropout(self.dense(hidden_states)) + input_tensor)


class Attention(nn.Module):
    def __init__(self, config: Any) -> None:
        super().__init__()
        self.self = AttentionParameters(config)
        self.output = SelfOutput(config)


class Intermediate(nn.Module):
    def __init__(self, config: Any) -> None:
        super().__init__()
        self.dense = nn.Linear(config.hidden_size, config.intermediate_size)
        act = config.hidden_act
        self.intermediate_act_fn = _ACTIVATIONS[act] if isinstance(act, str) else act

    def forward(self, hidden_states: torch.Tensor) -> torch.Tensor:
        return self.intermediate_act_fn(self.dense(hidden_states))


class Output(nn.Module):
    def __init__(self, config: Any) -> None:
        super().__init__()
        self.dense = nn.Linear(config.intermediate_size, config.hidden_size)
        self.LayerNorm = nn.LayerNorm(config.hidden_size, config.layer_norm_eps)
        self.dropout = nn.Dropout(config.hidden_dropout_prob)

    def forward(self, hidden_states: torch.Tensor, input_tensor: torch.Tensor) -> torch.Tensor:
        return self.LayerNorm(self.dropout(self.dense(hidden_states)) + input_tensor)


class Layer(nn.Module):
    def __init__(self, config: Any) -> None:
        super().__init__()
        self.attention = Attention(config)
        self.intermediate = Intermediate(config)
        self.output = Output(config)


class ConvLayer(nn.Module):
    """Layer-0 convolution branch of DeBERTa-v2 (HF ``ConvLayer``)."""

    def __init__(self, config: Any) -> None:
        super().__init__()
        kernel = getattr(config, "conv_kernel_size", 3)
        self.conv_act = getattr(config, "conv_act", "tanh")
        self.conv = nn.Conv1d(config.hidden_size, config.hidden_size, kernel, padding=(kernel - 1) // 2,
                              groups=getattr(config, "conv_groups", 1))
        self.LayerNorm = nn.LayerNorm(config.hidden_size, config.layer_norm_eps)
        self.dropout = nn.Dropout(config.hidden_dropout_prob)

    def forward(self, hidden_states: torch.Tensor, residual_states: torch.Tensor,
                input_mask: torch.Tensor | None) -> torch.Tensor:
        out = self.conv(hidden_states.transpose(1, 2)).transpose(1, 2).contiguous()
        keep = None
        if input_mask is not None:
            keep = input_mask if input_mask.dtype == torch.bool else input_mask != 0
            out = out.masked_fill(~keep.unsqueeze(-1), 0)
        out = _ACTIVATIONS[self.conv_act](self.dropout(out))
        normed = self.LayerNorm(residual_states + out)
        if keep is None:
            return normed
        return normed * keep.unsqueeze(-1).to(normed.dtype)


class Encoder(nn.Module):
    """Module tree of HF ``DebertaV2Encoder`` (layers, rel_embeddings, LayerNorm, conv)."""

    def __init__(self, config: Any) -> None:
        super().__init__()
        self.layer = nn.ModuleList([Layer(config) for _ in range(config.num_hidden_layers)])
        self.relative_attention = getattr(config, "relative_attention", False)
        if self.relative_attention:
            self.max_relative_positions = getattr(config, "max_relative_positions", -1)
            if self.max_relative_positions < 1:
                self.max_relative_positions = config.max_position_embeddings
            self.position_buckets = getattr(config, "position_buckets", -1)
            span = self.position_buckets if self.position_buckets > 0 else self.max_relative_positions
            self.rel_embeddings = nn.Embedding(span * 2, config.hidden_size)
        self.norm_rel_ebd = [x.strip() for x in getattr(config, "norm_rel_ebd", "none").lower().split("|")]
        if "layer_norm" in self.norm_rel_ebd:
            self.LayerNorm = nn.LayerNorm(config.hidden_size, config.layer_norm_eps, elementwise_affine=True)
        self.conv = ConvLayer(config) if getattr(config, "conv_kernel_size", 0) > 0 else None


class Backbone(nn.Module):
    """Smallest object ``enable_deberta_inference`` accepts: ``config`` + ``embeddings`` + ``encoder``.

    ``embeddings`` is a plain token-embedding table followed by LayerNorm
    (DeBERTa-v2/v3 use no absolute position embeddings by default).
    """

    def __init__(self, config: Any, vocab_size: int = 128100) -> None:
        super().__init__()
        self.config = config
        self.embeddings = nn.Sequential()
        self.embeddings.word_embeddings = nn.Embedding(vocab_size, config.hidden_size, padding_idx=0)
        self.embeddings.LayerNorm = nn.LayerNorm(config.hidden_size, config.layer_norm_eps)
        self.encoder = Encoder(config)

    def embed(self, input_ids: torch.Tensor, attention_mask: torch.Tensor) -> torch.Tensor:
        hidden = self.embeddings.LayerNorm(self.embeddings.word_embeddings(input_ids))
        return hidden * attention_mask.unsqueeze(-1).to(hidden.dtype)

    def forward(self, input_ids: torch.Tensor, attention_mask: torch.Tensor) -> torch.Tensor:
        hidden = self.embed(input_ids, attention_mask)
        return self.encoder(hidden, attention_mask, output_hidden_states=False).last_hidden_state


def initialize_parameters(module: nn.Module, seed: int, std: float = 0.02) -> None:
    """Seeded init used by the reference's benchmarks: N(0, std) weights, zero biases, unit LayerNorm."""

    gen = torch.Generator(device="cpu").manual_seed(seed)
    with torch.no_grad():
        for child in module.modules():
            if isinstance(child, (nn.Linear, nn.Conv1d)):
                child.weight.copy_(torch.empty(child.weight.shape).normal_(0.0, std, generator=gen))
                if child.bias is not None:
                    child.bias.zero_()
            elif isinstance(child, nn.Embedding):
                child.weight.copy_(torch.empty(child.weight.shape).normal_(0.0, std, generator=gen))
            elif isinstance(child, nn.LayerNorm):
                if child.weight is not None:
                    child.weight.fill_(1.0)
                if child.bias is not None:
                    child.bias.zero_()


__all__ = ["AttentionParameters", "Backbone", "ConvLayer", "Encoder", "Layer", "initialize_parameters"]
