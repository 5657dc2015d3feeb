"""Host-side rules of the encoder wrapper that decide which of the caller's blocks run through the fused kernels
(``encoder._output_block_is_fusable``, ``_intermediate_is_fusable``, ``_conv_activation``, ``_is_erf_gelu``) and the
argument checks of ``capture_deberta_buckets`` - everything that can be checked without a GPU."""

import pytest
import torch
from torch import nn
from torch.nn import functional as F

import hf_modules
import disentangled_flash_b200 as df
from disentangled_flash_b200 import encoder as enc


def _config(**overrides):
    base = dict(hidden_size=64, num_attention_heads=2, attention_head_size=32, num_hidden_layers=1,
                intermediate_size=128, max_position_embeddings=64, position_buckets=32, norm_rel_ebd="layer_norm",
                conv_kernel_size=3)
    base.update(overrides)
    return df.DebertaAttentionConfig(**base)


def test_erf_gelu_is_recognised_in_its_usual_forms():
    assert enc._is_erf_gelu(F.gelu)
    assert enc._is_erf_gelu(nn.GELU())
    assert not enc._is_erf_gelu(nn.GELU(approximate="tanh"))
    assert not enc._is_erf_gelu(F.relu)
    assert not enc._is_erf_gelu(lambda x: F.gelu(x, approximate="tanh"))

    class Wrapper(nn.Module):   # the shape of Transformers' GELUActivation
        def __init__(self):
            super().__init__()
            self.act = F.gelu

        def forward(self, x):
            return self.act(x)

    assert enc._is_erf_gelu(Wrapper())


def test_blocks_on_the_cpu_are_never_fused():
    layer = hf_modules.Backbone(_config(), vocab_size=8).encoder.layer[0]
    assert not enc._output_block_is_fusable(layer.attention.output)
    assert not enc._output_block_is_fusable(layer.output)
    assert not enc._intermediate_is_fusable(layer.intermediate)
    assert enc._conv_activation(hf_modules.Backbone(_config(), vocab_size=8).encoder.conv) is None


def test_blocks_of_another_shape_are_left_alone():
    layer = hf_modules.Backbone(_config(), vocab_size=8).encoder.layer[0]

    class Extra(nn.Module):
        def __init__(self, inner):
            super().__init__()
            self.dense, self.LayerNorm, self.dropout = inner.dense, inner.LayerNorm, inner.dropout
            self.gate = nn.Linear(4, 4)     # a child the Hugging Face block does not have

        def forward(self, hidden, residual):
            return self.LayerNorm(self.dropout(self.dense(hidden)) + residual)

    assert not enc._output_block_is_fusable(Extra(layer.output))
    assert not enc._output_block_is_fusable(nn.Identity())
    assert not enc._intermediate_is_fusable(nn.Identity())
    conv = hf_modules.Backbone(_config(), vocab_size=8).encoder.conv
    conv.conv = nn.Conv1d(64, 64, 3, padding=1, groups=2)     # grouped: not a plain GEMM over the taps
    assert enc._conv_activation(conv) is None
    conv.conv = nn.Conv1d(64, 64, 3, padding=0)                # not 'same' padding
    assert enc._conv_activation(conv) is None
    conv.conv = nn.Conv1d(64, 64, 4, padding=1)                # even kernel size
    assert enc._conv_activation(conv) is None


def test_capture_needs_a_cuda_encoder_and_a_positive_batch():
    backbone = hf_modules.Backbone(_config(), vocab_size=8).eval()
    with pytest.raises(ValueError, match="backend"):
        df.enable_deberta_inference(backbone, backend="torch")
    wrapper = enc.DebertaV2InferenceEncoder(backbone.encoder, _config())
    with pytest.raises(ValueError, match="batch_size"):
        df.capture_deberta_buckets(wrapper, 0)
    with pytest.raises(RuntimeError, match="CUDA"):
        df.capture_deberta_buckets(wrapper, 2)


def test_fused_blocks_default_to_the_module_path_until_prepared():
    backbone = hf_modules.Backbone(_config(num_hidden_layers=2), vocab_size=8).eval()
    wrapper = enc.DebertaV2InferenceEncoder(backbone.encoder, _config(num_hidden_layers=2))
    assert wrapper._fused_output_blocks == [(False, False)] * 2
    assert wrapper._fused_intermediates == [False] * 2
    assert wrapper._conv_fused == {} and wrapper._conv_weight is None
