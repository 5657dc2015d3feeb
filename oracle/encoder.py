"""CPU encoder forward built on the oracle attention.

TEST INFRASTRUCTURE ONLY (see ``oracle/__init__.py``).  The layers around the
attention (output projection, FFN, LayerNorms, layer-0 convolution) are plain
PyTorch modules passed in by the caller; this function replaces only
``layer.attention.self`` by ``oracle.attention_module_forward`` and runs the
same layer loop as the reference's encoder wrapper (reference
``src/disentangled_flash/deberta.py:247-285``).
"""

from __future__ import annotations

import torch

from .attention import attention_module_forward


def _pos_types(value):
    if value is None:
        return ()
    if isinstance(value, str):
        return tuple(p.strip().lower() for p in value.split("|") if p.strip())
    return tuple(str(p).strip().lower() for p in value)


def oracle_encoder_forward(backbone_cpu, config, hidden: torch.Tensor, mask: torch.Tensor) -> torch.Tensor:
    """Run ``backbone_cpu.encoder`` (an un-wrapped hf_modules.Encoder) with oracle attention, fp32 on CPU."""

    enc = backbone_cpu.encoder
    types_ = _pos_types(config.pos_att_type)
    rel = None
    if enc.relative_attention:
        rel = enc.rel_embeddings.weight
        if "layer_norm" in enc.norm_rel_ebd:
            rel = enc.LayerNorm(rel)
    max_rel = config.max_relative_positions if config.max_relative_positions >= 1 else config.max_position_embeddings
    x = hidden
    with torch.no_grad():
        for index, layer in enumerate(enc.layer):
            a = layer.attention.self
            get = lambda name: getattr(a, name, None)  # noqa: E731
            ctx = attention_module_forward(
                x, mask,
                wq=a.query_proj.weight, wk=a.key_proj.weight, wv=a.value_proj.weight,
                bq=a.query_proj.bias, bk=a.key_proj.bias, bv=a.value_proj.bias,
                rel_embeddings=rel, num_heads=config.num_attention_heads,
                position_buckets=config.position_buckets, max_relative_positions=max_rel,
                pos_att_type=types_, relative_attention=config.relative_attention,
                share_att_key=config.share_att_key,
                w_pos_key=get("pos_key_proj").weight if get("pos_key_proj") is not None else None,
                b_pos_key=get("pos_key_proj").bias if get("pos_key_proj") is not None else None,
                w_pos_query=get("pos_query_proj").weight if get("pos_query_proj") is not None else None,
                b_pos_query=get("pos_query_proj").bias if get("pos_query_proj") is not None else None,
            )
            attn_out = layer.attention.output(ctx, x)
            out = layer.output(layer.intermediate(attn_out), attn_out)
            if index == 0 and enc.conv is not None:
                out = enc.conv(hidden, out, mask)
            x = out
    return x
