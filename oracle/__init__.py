"""CPU restatement of the reference's disentangled-attention path.

TEST INFRASTRUCTURE ONLY.  Nothing in the shipped package may import this
module: it exists so that the CUDA kernels can be checked against an
independent statement of the reference algorithm, and so that the benchmark
can report a host-CPU baseline next to the GPU number.  The only legitimate
importers are ``tests/``, ``__graft_entry__.smoke()`` and the ``cpu_baseline``
/ ``--impl reference`` legs of ``bench.py``.

Parity status: pinned.  ``tests/golden/make_golden.py`` runs the real
reference (its ``original`` and ``torch`` backends, CPU, fp32) on seeded
inputs and stores inputs and outputs under ``tests/golden/``; the CPU test
suite checks every function here against those files.
"""

from .position import (  # noqa: F401
    PositionPlan,
    compact_position_plan,
    dense_pair_map,
    log_bucket_position,
)
from .attention import (  # noqa: F401
    attention_core,
    attention_module_forward,
    fuse_qkv,
    project_positions,
    split_heads,
)
