"""``dfl_conv1d`` (1-D convolution as a tensor-core GEMM over the taps, with bias, padding mask and activation in the
epilogue) and the masked ``dfl_add_layernorm``, against plain PyTorch fp32 references of the same ops.

They replace the layer-0 convolution branch of the encoder (reference: ``ConvLayer.forward``,
``_reference.py:534-568``).  Bounds: 2e-3 plus one rounding step of the output type (2^-11 / 2^-8 relative).
"""

import pytest
import torch
from torch.nn import functional as F

pytestmark = pytest.mark.gpu
dev = "cuda"
DTYPES = {"fp16": torch.float16, "bf16": torch.bfloat16}
ULP = {torch.float16: 2.0 ** -11, torch.bfloat16: 2.0 ** -8}
ACTS = {"none": lambda v: v, "tanh": torch.tanh, "gelu": F.gelu}


def _check(got, want, dtype, what):
    err = (got.float().cpu() - want).abs()
    bound = 2e-3 + ULP[dtype] * want.abs()
    assert torch.isfinite(got).all(), what
    assert bool((err <= bound).all()), f"{what}: max abs error {err.max().item():.3e}"


@pytest.mark.parametrize("dtype_name", sorted(DTYPES))
@pytest.mark.parametrize("shape", [(2, 256, 64, 64, 3), (3, 300, 128, 72, 5), (2, 512, 768, 768, 3), (1, 1100, 64, 264, 1)])
@pytest.mark.parametrize("activation", sorted(ACTS))
def test_conv1d_matches_fp32_reference(dtype_name, shape, activation):
    from disentangled_flash_b200 import _cabi as c

    batch, length, c_in, c_out, taps = shape
    dtype = DTYPES[dtype_name]
    code = {"none": c.ACT_NONE, "tanh": c.ACT_TANH, "gelu": c.ACT_GELU}[activation]
    assert c.conv1d_supported(dtype, length, c_in, c_out, taps, code)
    gen = torch.Generator().manual_seed(length + c_in + taps)
    x = torch.randn(batch, length, c_in, generator=gen).to(dtype)
    w = (torch.randn(c_out, c_in, taps, generator=gen) * (1.5 / (c_in * taps) ** 0.5)).to(dtype)   # nn.Conv1d layout
    b = (torch.randn(c_out, generator=gen) * 0.3).to(dtype)
    valid = torch.randint(1, length + 1, (batch,), generator=gen)
    valid[0] = length
    keep = torch.arange(length)[None, :] < valid[:, None]
    conv = F.conv1d(x.float().transpose(1, 2), w.float(), b.float(), padding=(taps - 1) // 2).transpose(1, 2)
    want = ACTS[activation](conv.masked_fill(~keep.unsqueeze(-1), 0.0))
    status = c.new_status_word(dev)
    got = c.conv1d(x.to(dev), w.permute(2, 0, 1).contiguous().to(dev), b.to(dev), keep.to(dev), activation=code,
                   status=status)
    c.check_status(status)
    _check(got, want, dtype, f"conv1d {shape} {dtype_name} {activation}")
    # without a mask and without a bias; an int64 mask gives the same as the bool mask
    got = c.conv1d(x.to(dev), w.permute(2, 0, 1).contiguous().to(dev), None, None, activation=code)
    want_plain = ACTS[activation](F.conv1d(x.float().transpose(1, 2), w.float(), None,
                                           padding=(taps - 1) // 2).transpose(1, 2))
    _check(got, want_plain, dtype, "conv1d without mask and bias")
    got64 = c.conv1d(x.to(dev), w.permute(2, 0, 1).contiguous().to(dev), b.to(dev), keep.long().to(dev), activation=code)
    _check(got64, want, dtype, "conv1d with an int64 mask")


def test_conv1d_refuses_what_it_does_not_cover():
    from disentangled_flash_b200 import _cabi as c

    assert not c.conv1d_supported(torch.float32, 512, 768, 768, 3, c.ACT_TANH)
    assert not c.conv1d_supported(torch.float16, 128, 768, 768, 3, c.ACT_TANH)    # shorter than one pair tile
    assert not c.conv1d_supported(torch.float16, 512, 768, 768, 4, c.ACT_TANH)    # even kernel size
    assert not c.conv1d_supported(torch.float16, 512, 32, 768, 3, c.ACT_TANH)
    x = torch.zeros(1, 128, 64, dtype=torch.float16, device=dev)
    w = torch.zeros(3, 64, 64, dtype=torch.float16, device=dev)
    with pytest.raises((ValueError, RuntimeError)):
        c.conv1d(x, w, None, None)


def test_masked_add_layernorm_zeroes_dropped_rows():
    from disentangled_flash_b200 import _cabi as c

    gen = torch.Generator().manual_seed(8)
    rows, hidden = 77, 768
    x = torch.randn(rows, hidden, generator=gen).to(torch.float16)
    res = torch.randn(rows, hidden, generator=gen).to(torch.float16)
    w = (1 + 0.1 * torch.randn(hidden, generator=gen)).to(torch.float16)
    b = (0.1 * torch.randn(hidden, generator=gen)).to(torch.float16)
    keep = torch.rand(rows, generator=gen) < 0.6
    want = F.layer_norm(x.float() + res.float(), (hidden,), w.float(), b.float(), 1e-7) * keep[:, None]
    for mask in (keep, keep.to(torch.int32), keep.long()):
        got = c.add_layernorm(x.to(dev), res.to(dev), w.to(dev), b.to(dev), 1e-7, row_mask=mask.to(dev))
        _check(got, want, torch.float16, f"masked add + norm ({mask.dtype})")
        assert not got[~keep.to(dev)].any().item()


@pytest.mark.parametrize("dtype_name", sorted(DTYPES))
def test_encoder_convolution_branch_fused_at_long_buckets(dtype_name):
    import hf_modules
    import disentangled_flash_b200 as df
    from helpers import tolerance
    from oracle.encoder import oracle_encoder_forward

    dtype = DTYPES[dtype_name]
    cfg = df.DebertaAttentionConfig(hidden_size=64, num_attention_heads=2, attention_head_size=32, num_hidden_layers=2,
                                    intermediate_size=128, max_position_embeddings=512, position_buckets=64,
                                    norm_rel_ebd="layer_norm", conv_kernel_size=3)
    reference = hf_modules.Backbone(cfg, vocab_size=8).eval()
    hf_modules.initialize_parameters(reference, 12, std=0.08)
    backbone = hf_modules.Backbone(cfg, vocab_size=8).eval()
    backbone.load_state_dict(reference.state_dict())
    backbone = backbone.to(dev, dtype)
    df.optimize_deberta(backbone, sequence_lengths=[64, 256])
    encoder = backbone.encoder
    assert encoder._conv_fused == {64: False, 256: True}
    gen = torch.Generator().manual_seed(4)
    hidden = torch.randn(2, 256, 64, generator=gen).mul_(0.5).to(dtype)
    mask = torch.arange(256)[None, :] < torch.tensor([256, 131])[:, None]
    encoder.activate_shape(256)
    with torch.inference_mode():
        got = encoder(hidden.to(dev), mask.to(dev)).last_hidden_state
        encoder._conv_fused = {}
        unfused = encoder(hidden.to(dev), mask.to(dev)).last_hidden_state
    encoder.check_device_status()
    # against the module path (PyTorch rounds between its kernels) and against the fp32 oracle on the rounded weights
    assert (got.float() - unfused.float()).abs().max().item() < (2e-2 if dtype == torch.float16 else 1.5e-1)
    rounded = hf_modules.Backbone(cfg, vocab_size=8).eval()
    rounded.load_state_dict({k: v.to(dtype).float() for k, v in reference.state_dict().items()})
    want = oracle_encoder_forward(rounded, cfg, hidden.float(), mask)
    err = (got.float().cpu() - want).abs()
    assert err.max().item() < (1.6e-2 if dtype == torch.float16 else 1.2e-1), err.max().item()
    # padded positions leave the convolution branch as zeros and stay finite afterwards
    assert torch.isfinite(got).all()
