"""The allocation-free entry point ``dfl_attention_fwd_static`` against the regular two-call path.

Some callers cannot allocate device memory at the point of the call (a server
whose device memory is one arena handed out at start-up, a plug-in inside a
host runtime's callback).  For them the library keeps the C2P/P2C score
tensors in a fixed 32 MiB array of its own.  This test calls that entry point
through the C ABI twice in a row, with different inputs, and requires the
same output as ``dfl_pos_scores`` + ``dfl_attention_fwd`` with
caller-allocated buffers (same kernels, same arithmetic: bitwise equal), and
the standard tolerance against the CPU oracle.  The file name sorts last so
that a run stopping at the first failure has already run every other test.
"""

import pytest
import torch

from helpers import assert_close, make_core_case, oracle_core

pytestmark = pytest.mark.gpu
dev = "cuda"


def _regular(c, case, algo):
    to = lambda t: None if t is None else t.to(dev)  # noqa: E731
    q, k = to(case["q"]), to(case["k"])
    c2p, p2c, ld = c.pos_scores(q if case["pos_key"] is not None else None, k if case["pos_query"] is not None else None,
                                to(case["pos_key"]), to(case["pos_query"]), algo=algo)
    return c.attention_fwd(q, k, to(case["v"]), c2p, p2c, to(case["lut"]), to(case["mask"]), case["scale"],
                           ld_slots=ld, algo=algo)


def _static(c, case, algo):
    to = lambda t: None if t is None else t.to(dev)  # noqa: E731
    q = to(case["q"])
    bsz, heads, length, d = q.shape
    out = torch.full((bsz, length, heads * d), float("nan"), dtype=q.dtype, device=dev)  # caller-owned output
    return c.attention_fwd_static(q, to(case["k"]), to(case["v"]), to(case["pos_key"]), to(case["pos_query"]),
                                  to(case["lut"]), to(case["mask"]), case["scale"], out, algo=algo)


@pytest.mark.parametrize("dtype", (torch.float16, torch.float32))
def test_static_scratch_entry_point_matches_regular_path_twice(dtype):
    from disentangled_flash_b200 import _cabi as c

    assert c.load_library().dfl_static_scratch_bytes() == 32 * 1024 * 1024
    # two calls in a row with different shapes and inputs: the second sees the first one's leftovers
    cases = (make_core_case(2, 2, 200, 64, dtype, seed=41, mask="right"),
             make_core_case(3, 2, 130, 64, dtype, seed=42, mask="left", mode="p2c"))
    for case in cases:
        want = _regular(c, case, c.ALGO_AUTO)
        got = _static(c, case, c.ALGO_AUTO)
        assert torch.equal(got, want), "static-scratch variant differs from the regular path"
        assert_close(got, oracle_core(case), dtype, "static-scratch variant vs oracle")


def test_static_scratch_rejects_requests_beyond_its_size():
    from disentangled_flash_b200 import _cabi as c

    # 2 terms x 8*12*512*512 fp16 scores = 100 MiB > 32 MiB
    case = make_core_case(8, 12, 512, 64, torch.float16, seed=43, mask="none")
    with pytest.raises(ValueError, match="exceeds the built-in"):
        _static(c, case, c.ALGO_AUTO)
