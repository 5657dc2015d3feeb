"""The embedding front-end as one kernel (``dfl_embed_layernorm``, ``fuse_deberta_embeddings``): token-embedding
gather, optional position-embedding add, LayerNorm and padding mask, against PyTorch in fp32 on the same rounded
parameters and against Hugging Face's ``DebertaV2Embeddings.forward``."""

import pytest
import torch
from torch.nn import functional as F

pytestmark = pytest.mark.gpu
dev = "cuda"

TOL = {torch.float32: 2e-6, torch.float16: 2e-3, torch.bfloat16: 1.6e-2}


def _reference(ids, table, gamma, beta, eps, mask, pos_ids=None, pos_table=None):
    rows = table.float()[ids.long()]
    if pos_table is not None:
        rows = rows + pos_table.float()[pos_ids.long()]
    out = F.layer_norm(rows, (table.shape[1],), gamma.float(), None if beta is None else beta.float(), eps)
    return out if mask is None else out * (mask != 0).unsqueeze(-1)


@pytest.mark.parametrize("dtype", (torch.float16, torch.bfloat16, torch.float32))
@pytest.mark.parametrize("hidden,id_dtype,with_pos", ((768, torch.int64, False), (1024, torch.int32, True),
                                                      (96, torch.int64, True), (1536, torch.int64, False)))
def test_embed_layernorm_matches_pytorch(dtype, hidden, id_dtype, with_pos):
    from disentangled_flash_b200 import _cabi as c

    gen = torch.Generator().manual_seed(hidden)
    vocab, positions, batch, length = 1000, 80, 3, 77
    table = torch.randn(vocab, hidden, generator=gen).to(dtype)
    table[0].zero_()
    pos_table = torch.randn(positions, hidden, generator=gen).mul_(0.3).to(dtype)
    gamma = (1.0 + 0.1 * torch.randn(hidden, generator=gen)).to(dtype)
    beta = (0.1 * torch.randn(hidden, generator=gen)).to(dtype)
    ids = torch.randint(0, vocab, (batch, length), generator=gen).to(id_dtype)
    pos_ids = torch.arange(length).expand(batch, length).contiguous().to(id_dtype)
    lengths = torch.tensor([77, 1, 40])
    mask = (torch.arange(length)[None, :] < lengths[:, None])
    status = c.new_status_word(dev)
    got = c.embed_layernorm(ids.to(dev), table.to(dev), gamma.to(dev), beta.to(dev), 1e-7, row_mask=mask.to(dev),
                            pos_ids=pos_ids.to(dev) if with_pos else None,
                            pos_table=pos_table.to(dev) if with_pos else None, status=status)
    c.check_status(status)
    want = _reference(ids, table, gamma, beta, 1e-7, mask, pos_ids if with_pos else None, pos_table if with_pos else None)
    assert got.shape == (batch, length, hidden) and got.dtype == dtype
    err = (got.float().cpu() - want).abs().max().item()
    assert err <= TOL[dtype] * max(1.0, want.abs().max().item()), err
    assert not got[~mask.to(dev)].any().item()          # padded positions are exactly zero
    # no mask, no bias
    got = c.embed_layernorm(ids.to(dev), table.to(dev), gamma.to(dev), None, 1e-7)
    want = _reference(ids, table, gamma, None, 1e-7, None)
    assert (got.float().cpu() - want).abs().max().item() <= TOL[dtype] * max(1.0, want.abs().max().item())


def test_out_of_range_ids_read_as_zero_rows_and_are_reported():
    from disentangled_flash_b200 import _cabi as c

    gen = torch.Generator().manual_seed(3)
    table = torch.randn(50, 64, generator=gen).to(torch.float16).to(dev)
    gamma = torch.ones(64, dtype=torch.float16, device=dev)
    beta = torch.full((64,), 0.25, dtype=torch.float16, device=dev)
    ids = torch.tensor([[1, 50, 7, -1]], device=dev)
    status = c.new_status_word(dev)
    got = c.embed_layernorm(ids, table, gamma, beta, 1e-7, status=status)
    with pytest.raises(ValueError, match="outside its table"):
        c.check_status(status)
    c.check_status(status)      # cleared
    # the layer norm of a row of zeros is its bias
    assert torch.equal(got[0, 1], beta) and torch.equal(got[0, 3], beta)
    good = c.embed_layernorm(torch.tensor([[1, 7]], device=dev), table, gamma, beta, 1e-7, status=status)
    c.check_status(status)
    assert torch.equal(got[0, 0], good[0, 0]) and torch.equal(got[0, 2], good[0, 1])
    with pytest.raises(ValueError):
        c.embed_layernorm(ids, table, gamma, beta, 1e-7, pos_ids=ids)        # position ids without a table
    with pytest.raises(TypeError):
        c.embed_layernorm(ids.float(), table, gamma, beta, 1e-7)


@pytest.mark.parametrize("position_biased", (False, True))
@pytest.mark.parametrize("dtype", (torch.float16, torch.float32))
def test_fused_hugging_face_embeddings(dtype, position_biased):
    transformers = pytest.importorskip("transformers")
    from transformers.models.deberta_v2.modeling_deberta_v2 import DebertaV2Embeddings
    import disentangled_flash_b200 as df

    cfg = transformers.DebertaV2Config(vocab_size=300, hidden_size=128, num_hidden_layers=1, num_attention_heads=2,
                                       intermediate_size=256, max_position_embeddings=96, type_vocab_size=0,
                                       position_biased_input=position_biased, hidden_dropout_prob=0.1)
    torch.manual_seed(11)

    class Holder(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.embeddings = DebertaV2Embeddings(cfg)

    model = Holder().eval().to(dev, dtype)
    keys = sorted(model.state_dict())
    gen = torch.Generator().manual_seed(12)
    ids = torch.randint(1, 300, (4, 64), generator=gen).to(dev)
    mask = (torch.arange(64)[None, :] < torch.tensor([64, 3, 33, 50])[:, None]).to(dev)
    with torch.inference_mode():
        want = model.embeddings(input_ids=ids, mask=mask).float()
        df.fuse_deberta_embeddings(model)
        got = model.embeddings(input_ids=ids, mask=mask)
        assert got.dtype == dtype and got.shape == want.shape
        err = (got.float() - want).abs().max().item()
        assert err <= (4e-3 if dtype == torch.float16 else 2e-6) * max(1.0, want.abs().max().item()), err
        # a long mask [B, L] of 0/1 as tokenizers return it, and no mask at all
        got2 = model.embeddings(input_ids=ids, mask=mask.long())
        assert torch.equal(got, got2)
        plain = model.embeddings(input_ids=ids)
        assert (plain.float() - model.embeddings._dfl_original_forward(input_ids=ids).float()).abs().max().item() <= 4e-3
        # what the kernel does not cover goes through the original forward
        embeds = model.embeddings.word_embeddings(ids)
        assert torch.equal(model.embeddings(inputs_embeds=embeds, mask=mask),
                           model.embeddings._dfl_original_forward(inputs_embeds=embeds, mask=mask))
    model.embeddings.check_device_status()
    assert sorted(model.state_dict()) == keys           # parameters and names untouched
