"""The numpy index-builder oracle must reproduce the reference bit for bit.

Golden data: ``tests/golden/position_plans.npz``, produced by the reference's
own ``make_log_bucket_position`` and ``SharedPositionPlanCache.compact``.
"""

import numpy as np
import pytest

from oracle import compact_position_plan, dense_pair_map, log_bucket_position

CONFIGS = {
    "b256_m512": (256, 512, 256),
    "b256_m2048": (256, 2048, 256),
    "b32_m64": (32, 64, 32),
    "nobucket_m512": (-1, 512, 512),
    "nobucket_m64": (0, 64, 64),
}
LENGTHS = (1, 2, 3, 16, 31, 32, 33, 63, 64, 65, 127, 128, 129, 255, 256, 257, 384, 511, 512, 513, 1024, 2048)


@pytest.mark.parametrize("name", [n for n, c in CONFIGS.items() if c[0] > 0])
def test_log_bucket_bit_exact(position_golden, name):
    buckets, max_pos, _ = CONFIGS[name]
    deltas = np.arange(-2047, 2048)
    got = log_bucket_position(deltas, buckets, max_pos)
    want = position_golden[f"{name}/bucket_f32"]
    assert got.dtype == np.float32
    assert np.array_equal(got, want)


@pytest.mark.parametrize("name", sorted(CONFIGS))
@pytest.mark.parametrize("length", LENGTHS)
def test_compact_plan_bit_exact(position_golden, name, length):
    buckets, max_pos, span = CONFIGS[name]
    plan = compact_position_plan(
        length, position_buckets=buckets, max_relative_positions=max_pos, position_embedding_size=span
    )
    assert np.array_equal(plan.active_slots, position_golden[f"{name}/L{length}/active"])
    assert np.array_equal(plan.delta_to_local, position_golden[f"{name}/L{length}/lut"])
    assert plan.delta_to_local.dtype == np.int32 and plan.delta_to_local.shape == (2 * length - 1,)


def test_reference_shape_pins():
    # reference tests/test_position.py:6-16
    plan = compact_position_plan(65, position_buckets=256, max_relative_positions=512, position_embedding_size=256)
    assert plan.delta_to_local.shape == (129,)
    assert plan.active_slots.ndim == 1 and plan.active_slots.size <= 129


def test_no_position_bias_plan():
    plan = compact_position_plan(
        9, position_buckets=256, max_relative_positions=512, position_embedding_size=256, uses_position_bias=False
    )
    assert plan.active_slots.size == 0 and not plan.delta_to_local.any()


def test_lut_is_monotone_with_unit_steps():
    # Property the CUDA kernels rely on: the local-slot table never decreases
    # and never jumps by more than one, so a tile touches one contiguous window.
    for name, (buckets, max_pos, span) in CONFIGS.items():
        for length in (1, 2, 65, 512, 513, 2048):
            lut = compact_position_plan(
                length, position_buckets=buckets, max_relative_positions=max_pos, position_embedding_size=span
            ).delta_to_local
            steps = np.diff(lut)
            assert steps.min(initial=0) >= 0 and steps.max(initial=0) <= 1, (name, length)


def test_dense_map_matches_definition():
    plan = compact_position_plan(7, position_buckets=4, max_relative_positions=8, position_embedding_size=4)
    dense = dense_pair_map(plan)
    for i in range(7):
        for j in range(7):
            assert dense[i, j] == plan.delta_to_local[i - j + 6]


def test_rejects_nonpositive_length():
    with pytest.raises(ValueError):
        compact_position_plan(0, position_buckets=256, max_relative_positions=512, position_embedding_size=256)
