"""Host-side behaviour that needs no GPU: API surface, argument errors, cache invalidation.

Mirrors the reference's tests/test_public_api.py and the rejection rules of
its encoder wrapper (deberta.py:214-245, 327-336).
"""

import re

import pytest
import torch

import disentangled_flash_b200 as df
import hf_modules


def small_config(**kw):
    base = dict(hidden_size=64, num_attention_heads=2, attention_head_size=32, num_hidden_layers=2,
                intermediate_size=128, max_position_embeddings=64, position_buckets=32, norm_rel_ebd="layer_norm",
                conv_kernel_size=3, hidden_dropout_prob=0.0, attention_probs_dropout_prob=0.0)
    base.update(kw)
    return df.DebertaAttentionConfig(**base)


def test_public_api_imports():
    assert callable(df.optimize_deberta)
    assert callable(df.enable_deberta_inference)
    assert callable(df.compile_deberta_buckets)
    assert df.enable_deberta_v2_inference is df.enable_deberta_inference
    assert re.match(r"^\d+\.\d+\.\d+$", df.__version__) is not None


def test_state_dict_keys_are_the_hugging_face_names():
    cfg = small_config(share_att_key=False)
    attention = df.DisentangledFlashAttention(cfg)
    assert set(attention.state_dict()) == {
        "query_proj.weight", "query_proj.bias", "key_proj.weight", "key_proj.bias", "value_proj.weight",
        "value_proj.bias", "pos_key_proj.weight", "pos_key_proj.bias", "pos_query_proj.weight",
        "pos_query_proj.bias",
    }
    backbone = hf_modules.Backbone(small_config(), vocab_size=50).eval()
    before = set(backbone.state_dict())
    df.enable_deberta_inference(backbone)
    assert set(backbone.state_dict()) == before
    assert isinstance(backbone.encoder, df.DebertaV2InferenceEncoder)


def test_backend_and_model_rejections():
    backbone = hf_modules.Backbone(small_config(), vocab_size=50).eval()
    with pytest.raises(ValueError, match="not available"):
        df.enable_deberta_inference(backbone, backend="torch")
    with pytest.raises(ValueError, match="not available"):
        df.enable_deberta_inference(backbone, backend="optimized")
    with pytest.raises(TypeError):
        df.enable_deberta_inference(torch.nn.Linear(2, 2))
    with pytest.raises(ValueError):
        df.DisentangledFlashAttention(small_config(), fp32_precision="sloppy")
    df.enable_deberta_inference(backbone, backend="triton")  # legacy name of the fused backend
    with pytest.raises(TypeError, match="already"):
        df.enable_deberta_inference(backbone)
    training = hf_modules.Backbone(small_config(), vocab_size=50).train()
    with pytest.raises(RuntimeError, match="eval"):
        df.enable_deberta_inference(training, sequence_lengths=[16])


def test_forward_contract_rejections_on_cpu():
    backbone = hf_modules.Backbone(small_config(), vocab_size=50).eval()
    df.enable_deberta_inference(backbone)
    enc = backbone.encoder
    hidden, mask = torch.zeros(1, 8, 64), torch.ones(1, 8, dtype=torch.bool)
    with torch.no_grad():
        with pytest.raises(RuntimeError, match="prepare_for_inference"):
            enc(hidden, mask)
        with pytest.raises(ValueError, match="output_attentions"):
            enc(hidden, mask, output_attentions=True)
        with pytest.raises(ValueError, match=r"\[B, L\]"):
            enc(hidden, mask[:, None, :])
    with pytest.raises(RuntimeError, match="no_grad"):
        enc(hidden, mask)
    with pytest.raises(ValueError, match="positive"):
        enc.prepare_for_inference([])
    attention = enc.layer[0].attention.self
    with torch.no_grad(), pytest.raises(RuntimeError, match="CUDA"):
        attention(hidden, mask)
    with pytest.raises(ValueError, match="was not prepared"):
        enc.activate_shape(8)


def test_caches_are_invalidated_by_load_apply_and_train():
    attention = df.DisentangledFlashAttention(small_config()).eval()
    attention._cached_qkv_weight = torch.zeros(1)
    attention.load_state_dict(attention.state_dict())
    assert attention._cached_qkv_weight is None
    attention._cached_qkv_weight = torch.zeros(1)
    attention.double()
    assert attention._cached_qkv_weight is None
    attention._cached_qkv_weight = torch.zeros(1)
    attention.train(True)
    assert attention._cached_qkv_weight is None
    assert "_cached_qkv_weight" not in attention.state_dict()


def test_head_dim_outside_supported_set_is_rejected():
    cfg = small_config(attention_head_size=48)
    attention = df.DisentangledFlashAttention(cfg).eval()
    with torch.no_grad(), pytest.raises((ValueError, RuntimeError)):
        attention(torch.zeros(1, 4, 64), torch.ones(1, 4, dtype=torch.bool))


def test_position_cache_rejects_cpu_and_bad_length():
    cache = df.SharedPositionPlanCache(position_buckets=256, max_relative_positions=512, position_embedding_size=256)
    with pytest.raises(ValueError, match="positive"):
        cache.compact(0, "cuda")
    with pytest.raises(ValueError, match="CUDA"):
        cache.compact(8, "cpu")


def test_fused_embeddings_fall_back_to_the_original_forward_off_the_gpu():
    """``fuse_deberta_embeddings`` on a CPU model: every call is outside what the kernel covers, so the rebound
    forward must give the original module's output bit for bit, keep the state-dict keys, and be idempotent."""

    import pytest
    import torch
    from torch import nn

    import disentangled_flash_b200 as df

    class Embeddings(nn.Module):
        def __init__(self):
            super().__init__()
            self.word_embeddings = nn.Embedding(50, 32, padding_idx=0)
            self.LayerNorm = nn.LayerNorm(32, 1e-7)
            self.position_embeddings = None
            self.position_biased_input = False

        def forward(self, input_ids=None, token_type_ids=None, position_ids=None, mask=None, inputs_embeds=None):
            hidden = self.LayerNorm(self.word_embeddings(input_ids) if inputs_embeds is None else inputs_embeds)
            return hidden if mask is None else hidden * mask.unsqueeze(-1).to(hidden.dtype)

    class Model(nn.Module):
        def __init__(self):
            super().__init__()
            self.embeddings = Embeddings()

    torch.manual_seed(4)
    model = Model().eval()
    keys = sorted(model.state_dict())
    ids = torch.randint(0, 50, (2, 9))
    mask = torch.ones(2, 9, dtype=torch.bool)
    mask[1, 4:] = False
    want = model.embeddings(input_ids=ids, mask=mask)
    assert df.fuse_deberta_embeddings(model) is model
    df.fuse_deberta_embeddings(model)                      # a second call rebinds nothing
    assert torch.equal(model.embeddings(input_ids=ids, mask=mask), want)
    assert torch.equal(model.embeddings(ids, None, None, mask), want)
    model.embeddings.check_device_status()                 # no fused call was made: nothing to report
    assert sorted(model.state_dict()) == keys
    with pytest.raises(TypeError):
        df.fuse_deberta_embeddings(nn.Linear(2, 2))
