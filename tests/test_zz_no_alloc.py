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
    c2p = p2c = None
    ld = 0
    if case["pos_key"] is not None or case["pos_query"] is not None:
        c2p, p2c, ld = c.pos_scores(q if case["pos_key"] is not None else None,
                                    k if case["pos_query"] is not None else None,
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


def _free_device_bytes():
    torch.cuda.synchronize()
    return torch.cuda.mem_get_info()[0]


def _torch_allocations():
    """Number of allocation requests PyTorch's caching allocator has served so far."""

    return torch.cuda.memory_stats().get("allocation.all.allocated", 0)


@pytest.mark.parametrize("dtype", (torch.float16, torch.bfloat16, torch.float32))
def test_static_scratch_entry_point_matches_regular_path_twice(dtype):
    from disentangled_flash_b200 import _cabi as c

    assert c.load_library().dfl_static_scratch_bytes() == 32 * 1024 * 1024
    # calls in a row with different shapes, term modes and head dims: each sees the previous one's leftovers
    # (inputs of std 0.5 for BF16: with unit-variance inputs one BF16 position score that rounds the other way in
    # the oracle's summation order already moves an output by more than the bound, on any path)
    std = 0.5 if dtype == torch.bfloat16 else 1.0
    cases = (make_core_case(2, 2, 200, 64, dtype, seed=41, mask="right", std=std),
             make_core_case(3, 2, 130, 64, dtype, seed=42, mask="left", mode="p2c", std=std),
             make_core_case(2, 3, 96, 32, dtype, seed=44, mask="heavy", mode="c2p", std=std),
             make_core_case(2, 1, 150, 128, dtype, seed=45, mask="right", std=std),
             make_core_case(2, 2, 70, 64, dtype, seed=46, mask="right", mode="none", std=std))
    for index, case in enumerate(cases):
        want = _regular(c, case, c.ALGO_AUTO)
        to = lambda t: None if t is None else t.to(dev)  # noqa: E731
        tensors = [to(case[k]) for k in ("q", "k", "v", "pos_key", "pos_query", "lut", "mask")]
        q = tensors[0]
        out = torch.full((q.shape[0], q.shape[2], q.shape[1] * q.shape[3]), float("nan"), dtype=q.dtype, device=dev)
        # what the entry point exists for: the call itself takes no device memory - neither from the driver
        # (free bytes on the device) nor from PyTorch's caching allocator
        free_before, torch_before = _free_device_bytes(), _torch_allocations()
        got = c.attention_fwd_static(*tensors, case["scale"], out, algo=c.ALGO_AUTO)
        if index > 0:   # the very first call on a device may load the kernels' code (module loading is lazy)
            assert _free_device_bytes() == free_before, "the allocation-free call changed the free device memory"
        assert _torch_allocations() == torch_before, "the allocation-free call allocated through PyTorch"
        assert got.data_ptr() == out.data_ptr()
        assert torch.equal(got, want), "static-scratch variant differs from the regular path"
        assert_close(got, oracle_core(case), dtype, f"static-scratch variant vs oracle (case {index})")


def test_static_scratch_rejects_requests_beyond_its_size():
    from disentangled_flash_b200 import _cabi as c

    # 2 terms x 8*12*512*512 fp16 scores = 100 MiB > 32 MiB
    case = make_core_case(8, 12, 512, 64, torch.float16, seed=43, mask="none")
    with pytest.raises(ValueError, match="exceeds the built-in"):
        _static(c, case, c.ALGO_AUTO)
