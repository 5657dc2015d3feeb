"""``dfl_add_layernorm`` (residual add + LayerNorm in one pass) against a plain PyTorch fp32 reference of the same op.

The kernel replaces the tail of a layer's two output blocks, ``LayerNorm(dense_out + residual)`` (reference:
``_reference.py:108-112`` and ``481-485``).  It is a floating-point kernel, so the reference here is
``torch.nn.functional.layer_norm`` in fp32 on the CPU over the same (rounded) inputs.  Bounds: FP32 1e-5 absolute
plus 1e-5 relative; FP16/BF16 1e-3 plus one rounding step of the output type (2^-11 / 2^-8 relative).
"""

import pytest
import torch
from torch.nn import functional as F

pytestmark = pytest.mark.gpu
dev = "cuda"
DTYPES = {"fp16": torch.float16, "bf16": torch.bfloat16, "fp32": torch.float32}
ULP = {torch.float16: 2.0 ** -11, torch.bfloat16: 2.0 ** -8, torch.float32: 1e-5}


def _reference(x, residual, weight, bias, eps):
    v = x.float() + (residual.float() if residual is not None else 0.0)
    return F.layer_norm(v, (x.shape[-1],), weight.float(), None if bias is None else bias.float(), eps)


def _check(got, want, dtype, what):
    err = (got.float().cpu() - want).abs()
    bound = (1e-5 if dtype == torch.float32 else 1e-3) + ULP[dtype] * want.abs()
    assert torch.isfinite(got).all(), what
    assert bool((err <= bound).all()), f"{what}: max abs error {err.max().item():.3e}"


@pytest.mark.parametrize("dtype_name", sorted(DTYPES))
@pytest.mark.parametrize("rows,hidden", [(1, 64), (7, 768), (33, 776), (300, 1024), (64, 1536), (9, 2048), (5, 8)])
def test_matches_fp32_reference(dtype_name, rows, hidden):
    from disentangled_flash_b200 import _cabi as c

    dtype = DTYPES[dtype_name]
    assert c.add_layernorm_supported(dtype, hidden)
    gen = torch.Generator().manual_seed(rows * 7919 + hidden)
    x = (torch.randn(rows, hidden, generator=gen) * 0.7).to(dtype)
    residual = (torch.randn(rows, hidden, generator=gen) * 1.3 + 0.2).to(dtype)
    weight = (1.0 + 0.1 * torch.randn(hidden, generator=gen)).to(dtype)
    bias = (0.1 * torch.randn(hidden, generator=gen)).to(dtype)
    got = c.add_layernorm(x.to(dev), residual.to(dev), weight.to(dev), bias.to(dev), 1e-7)
    _check(got, _reference(x, residual, weight, bias, 1e-7), dtype, "add + norm")
    # without a residual and without a bias
    got = c.add_layernorm(x.to(dev), None, weight.to(dev), None, 1e-5)
    _check(got, _reference(x, None, weight, None, 1e-5), dtype, "norm only")


def test_output_may_alias_an_input_and_large_batches_use_every_row():
    from disentangled_flash_b200 import _cabi as c

    gen = torch.Generator().manual_seed(3)
    rows, hidden = 16384 + 5, 768     # more rows than one wave of warps: the grid-stride loop is exercised
    x = torch.randn(rows, hidden, generator=gen).to(torch.float16)
    residual = torch.randn(rows, hidden, generator=gen).to(torch.float16)
    weight = (1.0 + 0.1 * torch.randn(hidden, generator=gen)).to(torch.float16)
    bias = (0.1 * torch.randn(hidden, generator=gen)).to(torch.float16)
    want = _reference(x, residual, weight, bias, 1e-7)
    xd = x.to(dev)
    got = c.add_layernorm(xd, residual.to(dev), weight.to(dev), bias.to(dev), 1e-7, out=xd)
    assert got.data_ptr() == xd.data_ptr()
    _check(got, want, torch.float16, "in place")
    again = c.add_layernorm(x.to(dev), residual.to(dev), weight.to(dev), bias.to(dev), 1e-7)
    assert torch.equal(again, got), "not deterministic"


def test_unsupported_sizes_are_refused():
    from disentangled_flash_b200 import _cabi as c

    assert not c.add_layernorm_supported(torch.float16, 12)       # rows of 24 bytes
    assert not c.add_layernorm_supported(torch.float16, 4104)     # beyond 4096
    assert not c.add_layernorm_supported(torch.float32, 2052)
    x = torch.zeros(2, 12, dtype=torch.float16, device=dev)
    w = torch.ones(12, dtype=torch.float16, device=dev)
    with pytest.raises((ValueError, RuntimeError)):
        c.add_layernorm(x, None, w, None, 1e-5)


def test_encoder_uses_the_fused_output_blocks_and_keeps_other_blocks_as_they_are():
    import hf_modules
    import disentangled_flash_b200 as df
    from torch import nn

    cfg = df.DebertaAttentionConfig(hidden_size=64, num_attention_heads=2, attention_head_size=32, num_hidden_layers=2,
                                    intermediate_size=128, max_position_embeddings=64, position_buckets=32,
                                    norm_rel_ebd="layer_norm")
    backbone = hf_modules.Backbone(cfg, vocab_size=8).eval()
    hf_modules.initialize_parameters(backbone, 5)
    backbone = backbone.to(dev, torch.float16)

    class Scaled(nn.Module):   # an output block of another shape: must be called as it is
        def __init__(self, inner):
            super().__init__()
            self.inner = inner

        def forward(self, hidden, residual):
            return self.inner(hidden, residual) * 1.0

    backbone.encoder.layer[1].output = Scaled(backbone.encoder.layer[1].output)
    df.optimize_deberta(backbone, sequence_lengths=[24])
    encoder = backbone.encoder
    assert encoder._fused_output_blocks == [(True, True), (True, False)]
    gen = torch.Generator().manual_seed(1)
    hidden = torch.randn(2, 24, 64, generator=gen).mul_(0.5).to(torch.float16).to(dev)
    mask = (torch.arange(24)[None, :] < torch.tensor([24, 13])[:, None]).to(dev)
    with torch.inference_mode():
        got = encoder(hidden, mask).last_hidden_state
        # the same layers with every output block called as a module
        encoder._fused_output_blocks = [(False, False)] * 2
        want = encoder(hidden, mask).last_hidden_state
    encoder.check_device_status()
    # PyTorch rounds the sum to fp16 before normalising, the fused kernel keeps it in fp32: a few output ulps
    assert (got.float() - want.float()).abs().max().item() < 2e-2
