"""``dfl_dense`` (GEMM with bias and GELU in its epilogue) against a plain PyTorch fp32 reference of the same op.

Replaces the intermediate block of a layer, ``gelu(dense(x))`` (reference: ``_reference.py:461-471``).  The
reference here is ``F.gelu(F.linear(x, w, b))`` in fp32 on the CPU over the same rounded inputs.  Bounds: FP32 1e-5
absolute plus 1e-5 relative; 16-bit 2e-3 plus one rounding step of the output type.
"""

import pytest
import torch
from torch.nn import functional as F

pytestmark = pytest.mark.gpu
dev = "cuda"
DTYPES = {"fp16": torch.float16, "bf16": torch.bfloat16, "fp32": torch.float32}
ULP = {torch.float16: 2.0 ** -11, torch.bfloat16: 2.0 ** -8, torch.float32: 1e-5}


def _check(got, want, dtype, what):
    err = (got.float().cpu() - want).abs()
    bound = (1e-5 if dtype == torch.float32 else 2e-3) + ULP[dtype] * want.abs()
    assert torch.isfinite(got).all(), what
    assert bool((err <= bound).all()), f"{what}: max abs error {err.max().item():.3e}"


@pytest.mark.parametrize("dtype_name", sorted(DTYPES))
@pytest.mark.parametrize("shape", [(40, 96, 64), (300, 256, 128), (1024, 3072, 768), (515, 1000, 264)])
@pytest.mark.parametrize("activation", ("none", "gelu"))
def test_dense_matches_fp32_reference(dtype_name, shape, activation):
    from disentangled_flash_b200 import _cabi as c

    rows, n, k = shape
    dtype = DTYPES[dtype_name]
    gen = torch.Generator().manual_seed(rows + n + k)
    x = torch.randn(rows, k, generator=gen).to(dtype)
    w = (torch.randn(n, k, generator=gen) * (2.0 / k ** 0.5)).to(dtype)
    b = (torch.randn(n, generator=gen) * 0.5).to(dtype)
    want = F.linear(x.float(), w.float(), b.float())
    if activation == "gelu":
        want = F.gelu(want)
    status = c.new_status_word(dev)
    got = c.dense(x.to(dev), w.to(dev), b.to(dev), activation=c.ACT_GELU if activation == "gelu" else c.ACT_NONE,
                  status=status)
    c.check_status(status)
    assert got.shape == (rows, n)
    _check(got, want, dtype, f"dense {shape} {dtype_name} {activation}")
    if dtype != torch.float32:   # the CUDA-core kernels as a second implementation
        simt = c.dense(x.to(dev), w.to(dev), b.to(dev), activation=c.ACT_GELU if activation == "gelu" else c.ACT_NONE,
                       algo=c.ALGO_SIMT)
        _check(simt, want, dtype, f"dense simt {shape} {dtype_name} {activation}")


def test_gelu_epilogue_over_the_whole_input_range():
    """The erf approximation of the 16-bit epilogue, on pre-activations from -12 to 12 (identity weight)."""

    from disentangled_flash_b200 import _cabi as c

    k = 64
    values = torch.linspace(-12.0, 12.0, 256 * k).reshape(256, k).to(torch.float16)
    eye = torch.eye(k).to(torch.float16)
    got = c.dense(values.to(dev), eye.to(dev), None, activation=c.ACT_GELU)
    want = F.gelu(values.float())
    err = (got.float().cpu() - want).abs()
    assert bool((err <= 2.0 ** -11 * want.abs() + 1e-6).all()), f"max abs error {err.max().item():.3e}"


def test_encoder_fuses_the_intermediate_block_only_for_erf_gelu():
    import hf_modules
    import disentangled_flash_b200 as df

    def build(act):
        cfg = df.DebertaAttentionConfig(hidden_size=64, num_attention_heads=2, attention_head_size=32,
                                        num_hidden_layers=2, intermediate_size=128, max_position_embeddings=64,
                                        position_buckets=32, norm_rel_ebd="layer_norm", hidden_act=act)
        backbone = hf_modules.Backbone(cfg, vocab_size=8).eval()
        hf_modules.initialize_parameters(backbone, 5)
        backbone = backbone.to(dev, torch.float16)
        df.optimize_deberta(backbone, sequence_lengths=[24])
        return backbone.encoder

    assert build("gelu")._fused_intermediates == [True, True]
    assert build("gelu_new")._fused_intermediates == [False, False]
    assert build("relu")._fused_intermediates == [False, False]
    encoder = build("gelu")
    gen = torch.Generator().manual_seed(1)
    hidden = torch.randn(2, 24, 64, generator=gen).mul_(0.5).to(torch.float16).to(dev)
    mask = (torch.arange(24)[None, :] < torch.tensor([24, 13])[:, None]).to(dev)
    with torch.inference_mode():
        got = encoder(hidden, mask).last_hidden_state
        encoder._fused_intermediates = [False, False]
        want = encoder(hidden, mask).last_hidden_state
    encoder.check_device_status()
    assert (got.float() - want.float()).abs().max().item() < 1e-2
