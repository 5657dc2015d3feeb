"""Generate the golden fixtures in this directory from the real reference.

Run once, in a checkout where the reference sources are available:

    python tests/golden/make_golden.py --reference /path/to/disentangled-flash/src

It imports the reference package (CPU, fp32), runs its own
``make_log_bucket_position`` / ``SharedPositionPlanCache.compact``, its
``original`` and ``torch`` attention backends and its ``DebertaV2Encoder``
(three layers with the layer-0 convolution) on seeded inputs, and stores
inputs and outputs as ``.npz`` files.  The committed ``.npz`` files are what
the test-suite reads; this script is never imported by it.
"""

from __future__ import annotations

import argparse
import sys
from pathlib import Path

import numpy as np
import torch

HERE = Path(__file__).resolve().parent

POSITION_CONFIGS = {
    # name: (position_buckets, max_relative_positions, position_embedding_size)
    "b256_m512": (256, 512, 256),
    "b256_m2048": (256, 2048, 256),
    "b32_m64": (32, 64, 32),
    "nobucket_m512": (-1, 512, 512),
    "nobucket_m64": (0, 64, 64),
}
POSITION_LENGTHS = (1, 2, 3, 16, 31, 32, 33, 63, 64, 65, 127, 128, 129, 255, 256, 257,
                    384, 511, 512, 513, 1024, 2048)

ATTENTION_CASES = {
    # name: dict(config overrides, B, L, mask pattern, seed)
    "both_L33_right": dict(hidden=64, heads=2, d=32, buckets=32, max_pos=64, types=("p2c", "c2p"),
                           share=True, rel=True, B=2, L=33, mask="right", seed=101),
    "c2p_L16_left": dict(hidden=64, heads=2, d=32, buckets=32, max_pos=64, types=("c2p",),
                         share=True, rel=True, B=2, L=16, mask="left", seed=102),
    "p2c_L40_heavy": dict(hidden=64, heads=1, d=64, buckets=32, max_pos=64, types=("p2c",),
                          share=True, rel=True, B=3, L=40, mask="heavy", seed=103),
    "unshared_L70_right": dict(hidden=96, heads=3, d=32, buckets=32, max_pos=64, types=("p2c", "c2p"),
                               share=False, rel=True, B=2, L=70, mask="right", seed=104),
    "log_region_L130_all": dict(hidden=64, heads=2, d=32, buckets=32, max_pos=64, types=("p2c", "c2p"),
                                share=True, rel=True, B=2, L=130, mask="all", seed=105),
    "norel_L20_right": dict(hidden=64, heads=2, d=32, buckets=32, max_pos=64, types=(),
                            share=True, rel=False, B=2, L=20, mask="right", seed=106),
    # relative attention off with both position types still configured: the scale stays 1/sqrt(3d) in the
    # HF-equivalent backends (_reference.py:277-286), where the Triton module would use 1/sqrt(d) (kernel.py:587)
    "norel_c2p_p2c_L20_right": dict(hidden=64, heads=2, d=32, buckets=32, max_pos=64, types=("c2p", "p2c"),
                                    share=True, rel=False, B=2, L=20, mask="right", seed=109),
    "nobucket_L24_none": dict(hidden=64, heads=2, d=32, buckets=-1, max_pos=32, types=("p2c", "c2p"),
                              share=True, rel=True, B=2, L=24, mask="none", seed=107),
    "b256_d64_L160": dict(hidden=128, heads=2, d=64, buckets=256, max_pos=512, types=("p2c", "c2p"),
                          share=True, rel=True, B=2, L=160, mask="right", seed=108, std=0.1),
}


def make_mask(pattern: str, batch: int, length: int, gen: torch.Generator) -> torch.Tensor:
    """Mask patterns follow the reference's validation matrix (validate_cuda.py:42-82)."""

    mask = torch.ones(batch, length, dtype=torch.bool)
    if pattern == "none":
        return mask
    if pattern == "all":
        mask[-1] = False  # last sequence fully padded
        return mask
    lengths = torch.randint(max(1, length // 4), length + 1, (batch,), generator=gen)
    pos = torch.arange(length)[None, :]
    if pattern == "right":
        return pos < lengths[:, None]
    if pattern == "left":
        return pos >= (length - lengths)[:, None]
    if pattern == "heavy":
        keep = torch.rand(batch, length, generator=gen) < 0.3
        keep[:, 0] = True
        return keep
    raise ValueError(pattern)


def generate_positions(ref) -> None:
    out = {}
    deltas = torch.arange(-2047, 2048, dtype=torch.long)
    for name, (buckets, max_pos, span) in POSITION_CONFIGS.items():
        if buckets > 0:
            raw = ref._reference.make_log_bucket_position(deltas, buckets, max_pos)
            out[f"{name}/bucket_f32"] = raw.numpy().astype(np.float32)
        cache = ref.position.SharedPositionPlanCache(
            position_buckets=buckets,
            max_relative_positions=max_pos,
            position_embedding_size=span,
            uses_position_bias=True,
        )
        for length in POSITION_LENGTHS:
            plan = cache.compact(length, torch.device("cpu"))
            out[f"{name}/L{length}/active"] = plan.active_slots.numpy().astype(np.int64)
            out[f"{name}/L{length}/lut"] = plan.delta_to_local.numpy().astype(np.int32)
    np.savez_compressed(HERE / "position_plans.npz", **out)
    print("position_plans.npz:", len(out), "arrays")


def generate_attention(ref, names=None) -> None:
    cfg_cls = ref._reference.DebertaAttentionConfig
    for name, c in ATTENTION_CASES.items():
        if names and name not in names:
            continue
        gen = torch.Generator().manual_seed(c["seed"])
        config = cfg_cls(
            hidden_size=c["hidden"], num_attention_heads=c["heads"], attention_head_size=c["d"],
            attention_probs_dropout_prob=0.0, hidden_dropout_prob=0.0,
            relative_attention=c["rel"], max_relative_positions=-1, max_position_embeddings=c["max_pos"],
            position_buckets=c["buckets"], share_att_key=c["share"], pos_att_type=c["types"],
            norm_rel_ebd="none",
        )
        original = ref._reference.OriginalDisentangledSelfAttention(config).eval()
        std = c.get("std", 0.3)
        with torch.no_grad():
            for p in original.parameters():
                p.normal_(0.0, std, generator=gen)
        # The reference's prepared backend cannot be constructed with
        # relative_attention=False (it reads position_buckets unconditionally),
        # so that case is pinned by the ``original`` backend alone.
        prepared = None
        if c["rel"]:
            prepared = ref._torch.TorchInferenceDisentangledSelfAttention(config).eval()
            prepared.load_state_dict(original.state_dict(), strict=True)

        span = c["buckets"] if c["buckets"] > 0 else c["max_pos"]
        hidden = torch.randn(c["B"], c["L"], c["hidden"], generator=gen)
        rel = torch.randn(2 * span, c["hidden"], generator=gen) * (std / 0.3)
        mask = make_mask(c["mask"], c["B"], c["L"], gen)

        with torch.no_grad():
            ext = ref._reference._prepare_attention_mask(mask, c["L"], c["L"])
            ctx_original, _ = original(hidden, ext, rel_embeddings=rel if c["rel"] else None)
            if prepared is not None:
                prepared.prepare_for_inference(rel)
                plan = prepared.prepare_shape(c["L"], "cpu")
                ctx_torch, _ = prepared.forward_prepared(hidden, mask, plan)
            else:
                ctx_torch = ctx_original

        arrays = {f"param/{k}": v.detach().numpy() for k, v in original.state_dict().items()}
        arrays.update(
            hidden=hidden.numpy(), rel_embeddings=rel.numpy(), mask=mask.numpy(),
            ctx_original=ctx_original.numpy(), ctx_torch=ctx_torch.numpy(),
            meta=np.array([c["hidden"], c["heads"], c["d"], c["buckets"], c["max_pos"],
                           int(c["share"]), int(c["rel"]), int("c2p" in c["types"]),
                           int("p2c" in c["types"])], dtype=np.int64),
        )
        np.savez_compressed(HERE / f"attention_{name}.npz", **arrays)
        diff = (ctx_original - ctx_torch).abs().max().item()
        print(f"attention_{name}.npz: ctx {tuple(ctx_torch.shape)}, original-vs-torch max abs {diff:.2e}")


ENCODER_CASE = dict(hidden=64, heads=2, d=32, layers=3, inter=128, buckets=32, max_pos=64, conv=3,
                    B=2, L=40, mask="right", seed=201, std=0.08)


def generate_encoder(ref) -> None:
    """Three-layer encoder of the reference (``_reference.py:569-698``) with conv and layer-normed rel embeddings."""

    c = ENCODER_CASE
    gen = torch.Generator().manual_seed(c["seed"])
    config = ref._reference.DebertaAttentionConfig(
        hidden_size=c["hidden"], num_attention_heads=c["heads"], attention_head_size=c["d"],
        num_hidden_layers=c["layers"], intermediate_size=c["inter"], attention_probs_dropout_prob=0.0,
        hidden_dropout_prob=0.0, relative_attention=True, max_relative_positions=-1,
        max_position_embeddings=c["max_pos"], position_buckets=c["buckets"], share_att_key=True,
        pos_att_type=("p2c", "c2p"), norm_rel_ebd="layer_norm", conv_kernel_size=c["conv"],
    )
    encoder = ref._reference.DebertaV2Encoder(config).eval()
    with torch.no_grad():
        for name, p in encoder.named_parameters():
            if name.endswith("LayerNorm.weight"):
                p.fill_(1.0).add_(torch.randn(p.shape, generator=gen) * 0.05)
            else:
                p.normal_(0.0, c["std"], generator=gen)
    hidden = torch.randn(c["B"], c["L"], c["hidden"], generator=gen)
    mask = make_mask(c["mask"], c["B"], c["L"], gen)
    with torch.no_grad():
        out = encoder(hidden, mask.long(), output_hidden_states=True)
    arrays = {f"param/{k}": v.detach().numpy() for k, v in encoder.state_dict().items()}
    arrays.update(hidden=hidden.numpy(), mask=mask.numpy(), last_hidden_state=out.last_hidden_state.numpy(),
                  layer1=out.hidden_states[1].numpy(),
                  meta=np.array([c["hidden"], c["heads"], c["d"], c["layers"], c["inter"], c["buckets"],
                                 c["max_pos"], c["conv"]], dtype=np.int64))
    np.savez_compressed(HERE / "encoder_conv_L40.npz", **arrays)
    print("encoder_conv_L40.npz:", tuple(out.last_hidden_state.shape), len(arrays), "arrays")


def main() -> None:
    parser = argparse.ArgumentParser()
    parser.add_argument("--reference", required=True, help="path to the reference's src/ directory")
    parser.add_argument("--only", choices=("positions", "attention", "encoder"), default=None,
                        help="regenerate one family of fixtures only")
    parser.add_argument("--case", action="append", default=None,
                        help="with --only attention: regenerate only the named case(s)")
    args = parser.parse_args()
    sys.path.insert(0, args.reference)
    import disentangled_flash as ref  # noqa: PLC0415
    import disentangled_flash._reference  # noqa: F401,PLC0415
    import disentangled_flash._torch  # noqa: F401,PLC0415
    import disentangled_flash.position  # noqa: F401,PLC0415

    torch.manual_seed(0)
    parser_only = args.only
    if parser_only in (None, "positions"):
        generate_positions(ref)
    if parser_only in (None, "attention"):
        generate_attention(ref, args.case)
    if parser_only in (None, "encoder"):
        generate_encoder(ref)


if __name__ == "__main__":
    main()
