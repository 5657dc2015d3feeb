"""``DebertaV2InferenceEncoder.forward_packed``: the layers between the attention kernels run on the valid positions
of a right-padded batch only.  Checked at the valid positions against the ordinary forward (same kernels on other
row counts: a few output ulps) and against the fp32 CPU oracle encoder; plus the pieces it is built from
(``dfl_copy_rows``, the packed output of ``dfl_attention_rel_fwd``, the scattered second output of
``dfl_add_layernorm``)."""

import pytest
import torch
from torch.nn import functional as F

pytestmark = pytest.mark.gpu
dev = "cuda"


def test_copy_rows_and_scattered_layernorm():
    from disentangled_flash_b200 import _cabi as c

    gen = torch.Generator().manual_seed(5)
    src = torch.randn(40, 768, generator=gen).to(torch.float16).to(dev)
    rows = torch.tensor([3, 39, -1, 0, 17, 17], dtype=torch.int32, device=dev)
    got = c.copy_rows(src, rows)
    want = src[rows.clamp(min=0).long()].clone()
    want[2] = 0
    assert torch.equal(got, want)

    x = torch.randn(6, 768, generator=gen).to(torch.float16).to(dev)
    res = torch.randn(6, 768, generator=gen).to(torch.float16).to(dev)
    w = torch.ones(768, dtype=torch.float16, device=dev)
    b = torch.zeros(768, dtype=torch.float16, device=dev)
    out2 = torch.zeros(20, 768, dtype=torch.float16, device=dev)
    where = torch.tensor([4, 0, -1, 19, 7, 8], dtype=torch.int32, device=dev)
    out = c.add_layernorm(x, res, w, b, 1e-7, scatter=(out2, where))
    plain = c.add_layernorm(x, res, w, b, 1e-7)
    assert torch.equal(out, plain)
    for r, dst in enumerate(where.tolist()):
        if dst >= 0:
            assert torch.equal(out2[dst], plain[r])
    untouched = [i for i in range(20) if i not in (4, 0, 19, 7, 8)]
    assert not out2[untouched].any().item()


@pytest.mark.parametrize("dtype", (torch.float16, torch.bfloat16))
def test_attention_packed_output_rows(dtype):
    from disentangled_flash_b200 import _cabi as c
    from helpers import make_core_case

    case = make_core_case(4, 3, 384, 64, dtype, seed=77, mask="none")
    lengths = [384, 200, 1, 129]
    case["mask"] = torch.arange(384)[None, :] < torch.tensor(lengths)[:, None]
    to = lambda t: t.to(dev)  # noqa: E731
    lut = to(case["lut"])
    rk, rq = c.expand_rel_tables(to(case["pos_key"]), lut, 384), c.expand_rel_tables(to(case["pos_query"]), lut, 384)
    q, k, v, mask = to(case["q"]), to(case["k"]), to(case["v"]), to(case["mask"])
    full = c.attention_rel_fwd(q, k, v, rk, rq, mask, case["scale"])
    counts = [min(384, -(-n // 32) * 32) for n in lengths]
    bases = [sum(counts[:b]) for b in range(4)]
    packed = c.attention_rel_fwd(q, k, v, rk, rq, mask, case["scale"],
                                 packed_rows=(torch.tensor(bases, dtype=torch.int32, device=dev),
                                              torch.tensor(counts, dtype=torch.int32, device=dev), sum(counts)))
    assert packed.shape == (sum(counts), 3 * 64)
    for b in range(4):
        assert torch.equal(packed[bases[b]:bases[b] + counts[b]], full[b, :counts[b]]), b


@pytest.mark.parametrize("heads,head_dim", ((3, 64), (6, 32), (2, 128)))
def test_projection_of_packed_rows(heads, head_dim):
    """dfl_qkv_proj with row groups: packed input rows land where the unpacked projection puts them (bitwise), and
    rows no group covers keep what the caller's buffers held."""

    from disentangled_flash_b200 import _cabi as c

    gen = torch.Generator().manual_seed(21)
    batch, length, hidden = 5, 256, 192
    width = heads * head_dim
    x = torch.randn(batch, length, hidden, generator=gen).mul_(0.5).to(torch.float16).to(dev)
    w = torch.randn(3 * width, hidden, generator=gen).mul_(0.06).to(torch.float16).to(dev)
    bias = torch.randn(3 * width, generator=gen).to(torch.float16).to(dev)
    counts = [256, 96, 160, 32, 64]
    rows = torch.cat([torch.arange(b * length, b * length + counts[b], dtype=torch.int32) for b in range(batch)]).to(dev)
    groups = rows[::32].contiguous()
    full = c.linear_heads(x, w, bias, n_out=3, heads=heads, head_dim=head_dim, rows_per_seq=length)
    packed_x = c.copy_rows(x.view(batch * length, hidden), rows)
    outs = tuple(torch.full((batch, heads, length, head_dim), 7.0, dtype=torch.float16, device=dev) for _ in range(3))
    got = c.linear_heads(packed_x, w, bias, n_out=3, heads=heads, head_dim=head_dim, rows_per_seq=length,
                         row_groups=groups, outs=outs)
    torch.cuda.synchronize()
    for o in range(3):
        for b in range(batch):
            assert torch.equal(got[o][b, :, :counts[b]], full[o][b, :, :counts[b]]), (o, b)
            assert (got[o][b, :, counts[b]:] == 7.0).all(), (o, b)
    with pytest.raises(c.DflError):   # strict FP32 has no packed projection
        c.linear_heads(packed_x.float(), w.float(), bias.float(), n_out=3, heads=heads, head_dim=head_dim,
                       rows_per_seq=length, row_groups=groups, outs=tuple(o.float() for o in outs))


@pytest.mark.parametrize("length", (256, 250))   # 250: not a multiple of 32, the projection stays on unpacked rows
@pytest.mark.parametrize("dtype_name", ("fp16", "bf16"))
def test_forward_packed_matches_forward_at_valid_positions(dtype_name, length):
    import hf_modules
    import disentangled_flash_b200 as df
    from oracle.encoder import oracle_encoder_forward

    dtype = {"fp16": torch.float16, "bf16": torch.bfloat16}[dtype_name]
    cfg = df.DebertaAttentionConfig(hidden_size=128, num_attention_heads=2, attention_head_size=64, num_hidden_layers=3,
                                    intermediate_size=256, max_position_embeddings=512, position_buckets=64,
                                    norm_rel_ebd="layer_norm", conv_kernel_size=3)
    reference = hf_modules.Backbone(cfg, vocab_size=8).eval()
    hf_modules.initialize_parameters(reference, 14, std=0.08)
    rounded = {k: v.to(dtype).float() for k, v in reference.state_dict().items()}
    backbone = hf_modules.Backbone(cfg, vocab_size=8).eval()
    backbone.load_state_dict(rounded)
    backbone = backbone.to(dev, dtype)
    df.optimize_deberta(backbone, sequence_lengths=[length])
    encoder = backbone.encoder
    lengths = [length, 97, 160, 1, 33]
    gen = torch.Generator().manual_seed(6)
    hidden = torch.randn(5, length, 128, generator=gen).mul_(0.5).to(dtype)
    mask = torch.arange(length)[None, :] < torch.tensor(lengths)[:, None]
    hidden = hidden * mask[..., None]          # embeddings of padding are zero, as Hugging Face's embeddings give them
    with torch.inference_mode():
        want = encoder(hidden.to(dev), mask.to(dev)).last_hidden_state.float().cpu()
        got = encoder.forward_packed(hidden.to(dev), mask.to(dev), lengths).last_hidden_state.float().cpu()
    encoder.check_device_status()
    assert torch.isfinite(got).all()
    ulps = 2.0 ** -10 if dtype == torch.float16 else 2.0 ** -7
    err = (got - want).abs()[mask]
    assert err.max().item() <= 8 * ulps * max(1.0, want[mask].abs().max().item()), err.max().item()
    # beyond a sequence's 32-row block nothing is written
    for b, n in enumerate(lengths):
        block_end = min(length, -(-n // 32) * 32)
        assert not got[b, block_end:].any().item()
    reference.load_state_dict(rounded)
    oracle = oracle_encoder_forward(reference, cfg, hidden.float(), mask)
    err = (got - oracle).abs()[mask]
    assert err.max().item() < (1.6e-2 if dtype == torch.float16 else 1.2e-1), err.max().item()


def test_forward_packed_refuses_what_it_cannot_do():
    import hf_modules
    import disentangled_flash_b200 as df

    cfg = df.DebertaAttentionConfig(hidden_size=64, num_attention_heads=2, attention_head_size=32, num_hidden_layers=1,
                                    intermediate_size=128, max_position_embeddings=64, position_buckets=32,
                                    norm_rel_ebd="layer_norm", hidden_act="relu")
    backbone = hf_modules.Backbone(cfg, vocab_size=8).eval().to(dev, torch.float16)
    df.optimize_deberta(backbone, sequence_lengths=[64])
    hidden = torch.zeros(2, 64, 64, dtype=torch.float16, device=dev)
    mask = torch.ones(2, 64, dtype=torch.bool, device=dev)
    with torch.inference_mode():
        with pytest.raises(NotImplementedError):
            backbone.encoder.forward_packed(hidden, mask, [64, 10])     # relu intermediate: not fused
    cfg = df.DebertaAttentionConfig(hidden_size=64, num_attention_heads=2, attention_head_size=32, num_hidden_layers=1,
                                    intermediate_size=128, max_position_embeddings=64, position_buckets=32,
                                    norm_rel_ebd="layer_norm")
    backbone = hf_modules.Backbone(cfg, vocab_size=8).eval().to(dev, torch.float16)
    df.optimize_deberta(backbone, sequence_lengths=[64])
    with torch.inference_mode():
        with pytest.raises(ValueError):
            backbone.encoder.forward_packed(hidden, mask, [64])          # one length per sequence
        with pytest.raises(ValueError):
            backbone.encoder.forward_packed(hidden, mask, [64, 65])      # longer than the bucket
