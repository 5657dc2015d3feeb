"""GPU parity tests of the relative-table attention path (dfl_expand_rel_tables + dfl_attention_rel_fwd).

The expanded tables are pure row copies and must be bit-exact; the attention
output must satisfy ``helpers.tolerance`` against the fp32 oracle evaluated
on the same rounded inputs, and agree with the two-call path
(dfl_pos_scores + dfl_attention_fwd), which rounds the relative scores the
same way.  The case matrix follows the reference's validation script
(validation/validate_cuda.py): lengths around tile boundaries, mask patterns,
term modes, small bucket tables; plus batches large enough that every CTA of
the persistent kernel walks several (batch, head, query tile) items,
including items without any kept query row.
"""

import pytest
import torch

from helpers import MASK_PATTERNS, assert_close, make_core_case, oracle_core, tolerance

pytestmark = pytest.mark.gpu

DTYPES = {"fp16": torch.float16, "bf16": torch.bfloat16}
dev = "cuda"


def _cabi():
    from disentangled_flash_b200 import _cabi

    return _cabi


def expand(case):
    c = _cabi()
    length = case["q"].shape[2]
    lut = case["lut"].to(dev)
    rel_key = None if case["pos_key"] is None else c.expand_rel_tables(case["pos_key"].to(dev), lut, length)
    rel_query = None if case["pos_query"] is None else c.expand_rel_tables(case["pos_query"].to(dev), lut, length)
    return rel_key, rel_query


def run_rel(case, status=None):
    c = _cabi()
    rel_key, rel_query = expand(case)
    status = torch.zeros(1, dtype=torch.int32, device=dev) if status is None else status
    out = c.attention_rel_fwd(case["q"].to(dev), case["k"].to(dev), case["v"].to(dev), rel_key, rel_query,
                              case["mask"].to(dev), case["scale"], status=status)
    assert status.item() == 0, f"a bounded device-side wait expired (code {status.item()})"
    return out


def run_two_call(case):
    c = _cabi()
    q, k = case["q"].to(dev), case["k"].to(dev)
    pk = None if case["pos_key"] is None else case["pos_key"].to(dev)
    pq = None if case["pos_query"] is None else case["pos_query"].to(dev)
    c2p, p2c, ld = c.pos_scores(q if pk is not None else None, k if pq is not None else None, pk, pq)
    return c.attention_fwd(q, k, case["v"].to(dev), c2p, p2c, case["lut"].to(dev), case["mask"].to(dev), case["scale"],
                           ld_slots=ld)


@pytest.mark.parametrize("dtype_name", sorted(DTYPES))
@pytest.mark.parametrize("d", (32, 64))
def test_expanded_tables_are_row_copies(dtype_name, d):
    dtype = DTYPES[dtype_name]
    for length, buckets, max_pos in ((1, 256, 512), (33, 256, 512), (512, 256, 512), (700, 32, 64), (1024, 256, 512)):
        case = make_core_case(1, 3, length, d, dtype, seed=length, buckets=buckets, max_pos=max_pos)
        rel_key, _ = expand(case)
        lut = case["lut"].long()
        want = case["pos_key"][:, lut.flip(0), :]  # rel[h, e] = pos[h, lut[2L-2-e]]
        assert rel_key.shape == (3, 2 * length - 1, d)
        assert torch.equal(rel_key.cpu(), want), f"L={length} buckets={buckets}"


CORE_LENGTHS = (1, 2, 31, 32, 33, 63, 64, 65, 127, 128, 129, 255, 256, 257, 383, 384, 385, 511, 512, 513, 1024, 1100, 2048)


@pytest.mark.parametrize("dtype_name", sorted(DTYPES))
@pytest.mark.parametrize("d", (32, 64))
def test_rel_kernel_lengths(dtype_name, d):
    dtype = DTYPES[dtype_name]
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    for length in CORE_LENGTHS:
        case = make_core_case(2, 2, length, d, dtype, seed=2000 + length, mask="right")
        assert _cabi().attention_rel_supported(dtype, length, d, True, True)
        got = run_rel(case, status)
        assert_close(got, oracle_core(case), dtype, f"rel kernel L={length} d={d} {dtype_name}")
        # Same arithmetic as the two-call path up to the softmax reference maximum (which changes how P rounds):
        # two results that each meet the bound against the oracle can differ by twice the bound.
        two = run_two_call(case).float().cpu()
        err = (got.float().cpu() - two).abs().double()
        assert (err <= 2 * tolerance(dtype, two)).all(), f"rel vs two-call L={length}: {err.max().item():.3e}"


@pytest.mark.parametrize("dtype_name", sorted(DTYPES))
@pytest.mark.parametrize("mask", MASK_PATTERNS)
@pytest.mark.parametrize("mode", ("both", "c2p", "p2c"))
def test_rel_kernel_masks_and_modes(dtype_name, mask, mode):
    dtype = DTYPES[dtype_name]
    for length, d, buckets, max_pos in ((65, 64, 256, 512), (200, 32, 256, 512), (300, 64, 32, 64), (700, 64, 256, 512)):
        case = make_core_case(2, 2, length, d, dtype, seed=17 + length, mask=mask, mode=mode, buckets=buckets,
                              max_pos=max_pos)
        got = run_rel(case)
        assert_close(got, oracle_core(case), dtype, f"rel kernel mask={mask} mode={mode} L={length}")


@pytest.mark.parametrize("dtype_name", sorted(DTYPES))
@pytest.mark.parametrize("mask", ("none", "right", "left", "heavy"))
def test_rel_kernel_many_items_per_cta(dtype_name, mask):
    # 8 x 12 x 4 = 384 items on at most 148 CTAs: every CTA walks two or three items; with right/left padding some
    # items have short key ranges and some have no kept query row at all (mean-of-V path).
    dtype = DTYPES[dtype_name]
    case = make_core_case(8, 12, 512, 64, dtype, seed=31, mask=mask)
    got = run_rel(case)
    assert_close(got, oracle_core(case), dtype, f"rel kernel many items mask={mask}")
    odd = make_core_case(5, 7, 390, 32, dtype, seed=32, mask=mask)
    assert_close(run_rel(odd), oracle_core(odd), dtype, f"rel kernel ragged items mask={mask}")


def test_rel_kernel_mask_element_types():
    case = make_core_case(2, 2, 200, 64, torch.float16, seed=3, mask="heavy")
    want = oracle_core(case)
    for mask_dtype in (torch.bool, torch.uint8, torch.int32, torch.int64):
        alt = dict(case, mask=case["mask"].to(mask_dtype))
        assert_close(run_rel(alt), want, torch.float16, f"mask dtype {mask_dtype}")


def test_rel_kernel_padded_rows_uniform_deterministic_and_unsupported():
    c = _cabi()
    case = make_core_case(3, 4, 384, 64, torch.float16, seed=5, mask="all")
    a, b = run_rel(case), run_rel(case)
    assert torch.equal(a, b), "two identical launches differ (race)"
    mean_v = case["v"].float().mean(dim=2).reshape(3, 1, -1).expand(3, 384, -1)
    padded = ~case["mask"]
    assert_close(a.cpu()[padded], mean_v[padded], torch.float16, "padded rows = mean(V)")

    big = make_core_case(1, 1, 64, 128, torch.float16, seed=6)
    assert not c.attention_rel_supported(torch.float16, 64, 128, True, True)
    assert not c.attention_rel_supported(torch.float32, 64, 64, True, True)
    assert not c.attention_rel_supported(torch.float16, 384, 64, False, False)
    assert c.attention_rel_supported(torch.float16, 2048, 64, True, True)
    assert not c.attention_rel_supported(torch.float16, 2049, 64, True, True)
    assert c.attention_rel_supported(torch.bfloat16, 1024, 32, False, True)
    with pytest.raises(c.DflError, match="not covered"):
        rel = torch.zeros(1, 127, 128, dtype=torch.float16, device=dev)
        c.attention_rel_fwd(big["q"].to(dev), big["k"].to(dev), big["v"].to(dev), rel, rel, big["mask"].to(dev), 0.1)


def test_module_plan_carries_rel_tables_where_the_kernel_applies():
    import disentangled_flash_b200 as df

    def plan_of(dtype, head_dim, length):
        cfg = df.DebertaAttentionConfig(hidden_size=4 * head_dim, num_attention_heads=4, max_position_embeddings=512,
                                        position_buckets=256, share_att_key=True, pos_att_type=("p2c", "c2p"),
                                        norm_rel_ebd="none")
        module = df.DisentangledFlashAttention(cfg).to(device=dev, dtype=dtype).eval()
        rel = torch.randn(512, 4 * head_dim, device=dev, dtype=dtype)
        with torch.inference_mode():
            module.prepare_for_inference(rel)
            return module, module.prepare_shape(length, dev)

    module, plan = plan_of(torch.float16, 64, 96)
    assert plan.rel_key is not None and plan.rel_key.shape == (4, 2 * 96 - 1, 64)
    assert plan.rel_query is not None and plan.rel_query.dtype == torch.float16
    lut = plan.delta_to_local.long()
    assert torch.equal(plan.rel_key, plan.pos_key[:, lut.flip(0), :])
    # the prepared forward runs through the single-launch kernel and agrees with the two-call path
    hidden = torch.randn(3, 96, 256, device=dev, dtype=torch.float16)
    mask = torch.ones(3, 96, dtype=torch.bool, device=dev)
    mask[1, 70:] = False
    with torch.inference_mode():
        got, _ = module.forward_prepared(hidden, mask, plan)
        bare = plan._replace(rel_key=None, rel_query=None)
        two, _ = module.forward_prepared(hidden, mask, bare)
    err = (got.float() - two.float()).abs().cpu().double()
    assert (err <= 2 * tolerance(torch.float16, two.float().cpu())).all(), err.max().item()

    for dtype, head_dim in ((torch.float32, 64), (torch.float16, 128)):
        _, other = plan_of(dtype, head_dim, 96)
        assert other.rel_key is None and other.rel_query is None
