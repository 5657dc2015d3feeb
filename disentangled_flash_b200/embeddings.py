"""The embedding front-end of a Hugging Face DeBERTa-v2/v3 backbone as one kernel.

``DebertaV2Embeddings.forward`` (Hugging Face ``modeling_deberta_v2.py``) runs, in front of the encoder that
``optimize_deberta`` replaces, an embedding gather, an optional position-embedding add, a LayerNorm and a multiply
by the padding mask - four passes over ``[B, L, hidden]``.  ``fuse_deberta_embeddings`` rebinds that forward to one
launch of ``dfl_embed_layernorm`` (gather, add, LayerNorm and mask in registers) for the calls it covers and keeps
the original forward for the others.  The module, its parameters and its state-dict keys stay as they are.  The
reference leaves ``model.embeddings`` untouched (``deberta.py:322-330``); its benchmark builds the encoder input the
same way (``table[ids]``, ``benchmarks/benchmark_cuda.py:176-183``).
"""

from __future__ import annotations

import types

import torch
from torch import nn

from . import _cabi

_FLOATS = (torch.float16, torch.bfloat16, torch.float32)


def _covered(module: nn.Module, input_ids, token_type_ids, mask, inputs_embeds) -> bool:
    """Whether one call of the embeddings' forward can take the fused kernel."""

    if input_ids is None or inputs_embeds is not None:
        return False
    table = module.word_embeddings.weight
    if table.device.type != "cuda" or table.dtype not in _FLOATS or input_ids.device != table.device:
        return False
    if input_ids.dim() != 2 or input_ids.dtype not in (torch.int32, torch.int64):
        return False
    if getattr(module, "embed_proj", None) is not None or getattr(module, "token_type_embeddings", None) is not None:
        return False
    dropout = getattr(module, "dropout", None)
    if module.training and dropout is not None and getattr(dropout, "p", 0.0) > 0.0:
        return False
    norm = module.LayerNorm
    if norm.weight is None or norm.weight.dtype != table.dtype or not _cabi.add_layernorm_supported(table.dtype, table.shape[1]):
        return False
    if mask is not None and (mask.dim() != 2 or mask.shape != input_ids.shape or mask.device != table.device):
        return False
    return not torch.is_grad_enabled() or not any(p.requires_grad for p in module.parameters())


def _fused_forward(self, input_ids=None, token_type_ids=None, position_ids=None, mask=None, inputs_embeds=None):
    if not _covered(self, input_ids, token_type_ids, mask, inputs_embeds):
        return self._dfl_original_forward(input_ids=input_ids, token_type_ids=token_type_ids, position_ids=position_ids,
                                          mask=mask, inputs_embeds=inputs_embeds)
    table = self.word_embeddings.weight
    ids = input_ids.contiguous()
    pos_ids = pos_table = None
    if getattr(self, "position_biased_input", False) and getattr(self, "position_embeddings", None) is not None:
        if position_ids is None:
            position_ids = self.position_ids[:, : ids.shape[1]]
        pos_ids = position_ids.to(ids.dtype).expand(ids.shape).contiguous()
        pos_table = self.position_embeddings.weight
    keep = None
    if mask is not None:
        keep = (mask != 0) if mask.dtype.is_floating_point else mask
        keep = keep.contiguous()
    status = self.__dict__.get("_dfl_status_word")
    if status is None or status.device != table.device:
        status = _cabi.new_status_word(table.device)
        self.__dict__["_dfl_status_word"] = status
    norm = self.LayerNorm
    eps = float(getattr(norm, "eps", getattr(norm, "variance_epsilon", 1e-7)))
    return _cabi.embed_layernorm(ids, table, norm.weight, norm.bias, eps, row_mask=keep, pos_ids=pos_ids,
                                 pos_table=pos_table, status=status)


def _check_device_status(self) -> None:
    """Raise ``ValueError`` if a token id or position id of an earlier fused call was outside its table."""

    status = self.__dict__.get("_dfl_status_word")
    if status is not None:
        _cabi.check_status(status)


def fuse_deberta_embeddings(model: nn.Module) -> nn.Module:
    """Rebind ``model.embeddings.forward`` (a Hugging Face ``DebertaV2Embeddings``) to the one-kernel front-end.

    Covered per call: token ids given (no ``inputs_embeds``), a CUDA model in FP16/BF16/FP32, no token-type
    embeddings, no embedding projection, no active dropout, a ``[B, L]`` mask or none.  Anything else runs the
    original forward.  Unlike ``nn.Embedding`` an id outside the vocabulary does not raise at once: its row reads as
    zeros and ``model.embeddings.check_device_status()`` reports it.  Returns ``model``.
    """

    embeddings = getattr(model, "embeddings", None)
    if embeddings is None or not hasattr(embeddings, "word_embeddings") or not hasattr(embeddings, "LayerNorm"):
        raise TypeError("expected a backbone whose `embeddings` has `word_embeddings` and `LayerNorm`")
    if "_dfl_original_forward" not in embeddings.__dict__:
        embeddings.__dict__["_dfl_original_forward"] = embeddings.forward
        embeddings.forward = types.MethodType(_fused_forward, embeddings)
        embeddings.check_device_status = types.MethodType(_check_device_status, embeddings)
    return model


__all__ = ["fuse_deberta_embeddings"]
