"""Robustness of the boundary on a GPU: status word and bounded waits, a refused slot table, torch.compile buckets.

The bounded-wait path is exercised in the only form that leaves the GPU healthy: a diagnostic kernel waits on a
barrier nobody arrives at, with a limit of two milliseconds, gives up, frees its tensor memory and records a code.
Nothing here traps, faults or waits without a limit.
"""

import pytest
import torch

from helpers import assert_close, make_core_case, make_mask, oracle_core

pytestmark = pytest.mark.gpu
dev = "cuda"


def _cabi():
    from disentangled_flash_b200 import _cabi

    return _cabi


def test_bounded_wait_expires_reports_and_leaves_the_device_usable():
    c = _cabi()
    status = c.new_status_word(dev)
    c.check_status(status)                       # nothing happened yet
    c.selftest_bounded_wait(status, 2000)        # a wait that cannot complete: gives up after 2 ms
    with pytest.raises(c.DflError, match="bounded device-side wait expired") as info:
        c.check_status(status)
    assert info.value.status == c.DFL_ERR_DEVICE_TIMEOUT and "99" in str(info.value)
    c.check_status(status)                       # the word was cleared by the failed check
    with pytest.raises(ValueError):
        c.selftest_bounded_wait(status, 0)
    # the diagnostic kernel freed its tensor memory: a tcgen05 kernel that allocates all 512 columns runs after it,
    # with the same status word, and the word stays clean
    case = make_core_case(2, 2, 200, 64, torch.float16, seed=77, mask="right")
    to = lambda t: t.to(dev)  # noqa: E731
    lut = to(case["lut"])
    out = c.attention_rel_fwd(to(case["q"]), to(case["k"]), to(case["v"]), c.expand_rel_tables(to(case["pos_key"]), lut, 200),
                              c.expand_rel_tables(to(case["pos_query"]), lut, 200), to(case["mask"]), case["scale"],
                              status=status)
    c.check_status(status)
    assert_close(out, oracle_core(case), torch.float16, "attention after an expired wait")


def test_every_kernel_call_takes_the_status_word():
    c = _cabi()
    status = c.new_status_word(dev)
    case = make_core_case(2, 2, 130, 64, torch.bfloat16, seed=78, mask="left")
    to = lambda t: t.to(dev)  # noqa: E731
    q, k = to(case["q"]), to(case["k"])
    c2p, p2c, ld = c.pos_scores(q, k, to(case["pos_key"]), to(case["pos_query"]), status=status)
    out = c.attention_fwd(q, k, to(case["v"]), c2p, p2c, to(case["lut"]), to(case["mask"]), case["scale"], ld_slots=ld,
                          status=status)
    x = torch.randn(4, 130, 128, device=dev, dtype=torch.bfloat16)
    w = torch.randn(3 * 2 * 64, 128, device=dev, dtype=torch.bfloat16)
    c.linear_heads(x, w, None, n_out=3, heads=2, head_dim=64, rows_per_seq=130, status=status)
    c.check_status(status)
    assert_close(out, oracle_core(case), torch.bfloat16, "two-call path with a status word")


def test_slot_table_of_the_wrong_shape_is_clamped_not_followed():
    # dfl_attention_fwd documents its slot table as non-decreasing with unit steps and entries below ld_slots.  A table
    # that breaks this (shuffled, with out-of-range entries) must not make the kernel read outside its staged windows:
    # the call completes, the output is finite, and a correct call afterwards is exact again.
    c = _cabi()
    case = make_core_case(2, 2, 200, 64, torch.float16, seed=79, mask="right")
    to = lambda t: t.to(dev)  # noqa: E731
    q, k, v = to(case["q"]), to(case["k"]), to(case["v"])
    c2p, p2c, ld = c.pos_scores(q, k, to(case["pos_key"]), to(case["pos_query"]))
    gen = torch.Generator().manual_seed(5)
    bad = case["lut"][torch.randperm(case["lut"].numel(), generator=gen)].clone()
    bad[::7] = 100000
    bad[3::11] = -5
    status = c.new_status_word(dev)
    out = c.attention_fwd(q, k, v, c2p, p2c, to(bad), to(case["mask"]), case["scale"], ld_slots=ld, status=status)
    c.check_status(status)
    assert torch.isfinite(out.float()).all()
    good = c.attention_fwd(q, k, v, c2p, p2c, to(case["lut"]), to(case["mask"]), case["scale"], ld_slots=ld)
    assert_close(good, oracle_core(case), torch.float16, "correct table after a refused one")


def test_compile_deberta_buckets_traces_through_the_custom_op():
    # the reference compiles one callable per bucket with fullgraph=True and a dynamic batch dimension
    # (deberta.py:349-427); the attention must stay an opaque, traceable custom op
    import disentangled_flash_b200 as df
    import hf_modules

    cfg = df.DebertaAttentionConfig(hidden_size=128, num_attention_heads=2, attention_head_size=64,
                                    num_hidden_layers=2, intermediate_size=256, max_position_embeddings=512,
                                    position_buckets=256, norm_rel_ebd="layer_norm", conv_kernel_size=3,
                                    hidden_dropout_prob=0.0, attention_probs_dropout_prob=0.0)
    model = hf_modules.Backbone(cfg, vocab_size=50).eval()
    hf_modules.initialize_parameters(model, seed=5, std=0.05)
    model = model.to(device=dev, dtype=torch.float16)
    df.optimize_deberta(model, sequence_lengths=[64])
    gen = torch.Generator().manual_seed(9)

    def batch(size):
        return (torch.randn(size, 64, 128, generator=gen).to(dev, torch.float16), make_mask("right", size, 64, gen).to(dev))

    compiled = df.compile_deberta_buckets(model.encoder, [64], mode="default", fullgraph=True, dynamic_batch=True,
                                          examples={64: batch(2)})
    assert set(compiled) == {64} and compiled[64].__name__ == "deberta_bucket_64"
    for size in (2, 5):   # two batch sizes through the one compiled callable
        hidden, mask = batch(size)
        with torch.inference_mode():
            eager = model.encoder(hidden, mask, output_hidden_states=False).last_hidden_state
            traced = compiled[64](hidden, mask)
        assert traced.shape == eager.shape
        # the PyTorch layers around the attention may be fused differently by the compiler: fp16 rounding only
        assert (traced.float() - eager.float()).abs().max().item() <= 2e-2
    model.encoder.check_device_status()
    with pytest.raises(ValueError, match="unprepared bucket lengths"):
        df.compile_deberta_buckets(model.encoder, [32])
    with pytest.raises(ValueError, match="missing compilation example"):
        df.compile_deberta_buckets(model.encoder, [64], examples={})


def test_captured_buckets_replay_the_eager_forward_bitwise():
    """``capture_deberta_buckets``: one CUDA graph per bucket at a fixed batch size; replays equal the eager forward."""

    import hf_modules
    import disentangled_flash_b200 as df

    cfg = df.DebertaAttentionConfig(hidden_size=128, num_attention_heads=2, attention_head_size=64,
                                    num_hidden_layers=2, intermediate_size=256, max_position_embeddings=512,
                                    position_buckets=256, norm_rel_ebd="layer_norm", conv_kernel_size=3)
    backbone = hf_modules.Backbone(cfg, vocab_size=8).eval()
    hf_modules.initialize_parameters(backbone, 9)
    backbone = backbone.to(dev, torch.float16)
    df.optimize_deberta(backbone, sequence_lengths=[64, 160])
    encoder = backbone.encoder
    graphs = df.capture_deberta_buckets(encoder, batch_size=3)
    assert sorted(graphs) == [64, 160]
    gen = torch.Generator().manual_seed(2)
    for round_ in range(2):
        for length in (160, 64):
            hidden = torch.randn(3, length, 128, generator=gen).mul_(0.5).to(torch.float16).to(dev)
            valid = torch.randint(1, length + 1, (3,), generator=gen)
            mask = (torch.arange(length)[None, :] < valid[:, None]).to(dev)
            got = graphs[length](hidden, mask).clone()
            encoder.activate_shape(length)
            with torch.inference_mode():
                want = encoder(hidden, mask, output_hidden_states=False).last_hidden_state
            assert torch.equal(got, want), f"bucket {length}, round {round_}"
    encoder.check_device_status()
    with pytest.raises(ValueError, match="captured for"):
        graphs[64](torch.zeros(2, 64, 128, dtype=torch.float16, device=dev), torch.ones(2, 64, dtype=torch.bool, device=dev))
    # a batch size per bucket (which also selects the buckets)
    sized = df.capture_deberta_buckets(encoder, {160: 2})
    assert sorted(sized) == [160] and sized[160].hidden_states.shape == (2, 160, 128)
    hidden = torch.randn(2, 160, 128, generator=gen).mul_(0.5).to(torch.float16).to(dev)
    mask = torch.ones(2, 160, dtype=torch.bool, device=dev)
    encoder.activate_shape(160)
    with torch.inference_mode():
        want = encoder(hidden, mask, output_hidden_states=False).last_hidden_state
    assert torch.equal(sized[160](hidden, mask), want)
    with pytest.raises(ValueError):
        df.capture_deberta_buckets(encoder, {160: 2}, sequence_lengths=[64])


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs in one process")
def test_second_device_in_one_process_gets_its_own_kernel_configuration():
    """The shared-memory opt-in and the SM count are per-device attributes: every kernel family, called on cuda:0 and
    then on cuda:1 from one process (plain launches, no peer access), gives the same bits on both."""

    c = _cabi()
    case = make_core_case(2, 2, 256, 64, torch.float16, seed=81, mask="right")
    case128 = make_core_case(1, 2, 130, 128, torch.float16, seed=82, mask="right")
    gen = torch.Generator().manual_seed(83)
    x = torch.randn(2, 256, 192, generator=gen).mul_(0.5).to(torch.float16)
    w = torch.randn(3 * 2 * 64, 192, generator=gen).mul_(0.06).to(torch.float16)
    bias = torch.randn(3 * 2 * 64, generator=gen).to(torch.float16)
    results = []
    for index in (0, 1):
        device = torch.device("cuda", index)
        to = lambda t: t.to(device)  # noqa: E731
        status = c.new_status_word(device)
        lut = to(case["lut"])
        rel = c.attention_rel_fwd(to(case["q"]), to(case["k"]), to(case["v"]),
                                  c.expand_rel_tables(to(case["pos_key"]), lut, 256),
                                  c.expand_rel_tables(to(case["pos_query"]), lut, 256), to(case["mask"]), case["scale"],
                                  status=status)
        q, k = to(case128["q"]), to(case128["k"])
        c2p, p2c, ld = c.pos_scores(q, k, to(case128["pos_key"]), to(case128["pos_query"]), status=status)
        two_call = c.attention_fwd(q, k, to(case128["v"]), c2p, p2c, to(case128["lut"]), to(case128["mask"]),
                                   case128["scale"], ld_slots=ld, status=status)
        heads = c.linear_heads(to(x), to(w), to(bias), n_out=3, heads=2, head_dim=64, rows_per_seq=256, status=status)
        dense = c.dense(to(x).view(512, 192), to(w), to(bias), activation=c.ACT_GELU, status=status)
        normed = c.add_layernorm(dense, dense, torch.ones(384, dtype=torch.float16, device=device),
                                 torch.zeros(384, dtype=torch.float16, device=device), 1e-7)
        fp32 = c.linear_heads(to(x).float(), to(w).float(), to(bias).float(), n_out=3, heads=2, head_dim=64,
                              rows_per_seq=256, status=status)
        torch.cuda.synchronize(device)
        c.check_status(status)
        results.append([t.cpu() for t in (rel, two_call, *heads, dense, normed, *fp32)])
    assert_close(results[0][0], oracle_core(case), torch.float16, "single-launch attention on cuda:0")
    for first, second in zip(*results):
        assert torch.equal(first, second)
