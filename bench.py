#!/usr/bin/env python
"""Benchmark of the disentangled-attention inference path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl b200|reference] [--workload NAME]

Workloads (``--workload``; the reference's recipe is benchmarks/benchmark_cuda.py:150-184, 355-595):

``v3-base`` (default)
    One step = one forward of the DeBERTa-v3-base-architecture encoder (12 layers, hidden 768, 12 heads, d=64,
    FFN 3072, conv 3; random-init std 0.02) in FP16 over one synthetic batch of B=32 sequences of L=512 with valid
    lengths uniform in [256, 512] -- per GPU.  With N>1 (one process per GPU, launched by torchrun) every rank runs
    its own batch; there is no collective in the forward, NCCL only gathers per-rank checksums after timing (weak
    scaling).  The JSON line reports encoder sequences/s (`value`, inputs resident in HBM), the same through host
    buffers with the copies overlapped on their own streams (`e2e`), the fused attention kernel's TFLOP/s against
    the measured tensor-core peak (`roofline`, `attention_op`), a host-CPU baseline (`cpu_baseline`), the same step
    replayed as one CUDA graph (`cuda_graph`), the same batches run without their padding (`packed`), and the
    batch-sharded v3-large mixed-bucket throughput of
    `v3-large-mixed` as the extra key `mixed_buckets`.
``attention-sweep``
    The attention operator alone: (H, d) in {(24,32), (12,64), (8,128)}, B=16, L in {16,64,256,512}, BF16 and FP16,
    a quarter of the rows padded; one row per shape with microseconds, TFLOP/s and the fraction of the burst peak.
``v2-xlarge``
    DeBERTa-v2-xlarge-architecture encoder (24 layers, hidden 1536, 24 heads, FFN 6144, conv 3), B=8, buckets
    L in {64,128,256,512} switched with activate_shape(), BF16 and strict FP32; sequences/s per (dtype, L).
``v3-large-mixed``
    DeBERTa-v3-large-architecture encoder (24 layers, hidden 1024, 16 heads, FFN 4096), BF16, a global batch of 512
    sequences in three buckets (171 / 171 / 170 at L = 128 / 256 / 512) sharded over the ranks with
    ``sharding.shard_buckets``; sequences/s = 512 / the slowest rank's time (strong scaling).

Timing: W warm-up steps (at least 3), then regions of exactly K steps between a barrier + synchronize on both sides,
CUDA events on the launching stream, maximum over ranks.  The region is run twice and the faster run is reported
(shared hosts: a stalled launching thread can double a 100 ms region); both times are in ``timed_runs_ms``.

``--impl reference`` times the reference's own PyTorch backend on the host CPU cores (from ``oracle/_ref``, staged by
``oracle/build_ref.py``; the CPU restatement in ``oracle/`` if that copy is absent) on a bounded sample of the
workload; under torchrun only rank 0 runs it.
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import time
from pathlib import Path

import torch

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))
sys.path.insert(1, str(ROOT / "tests"))   # the HF-named module tree the encoders are built from (tests/hf_modules.py)

VOCAB = 128100
GEOMETRY = {
    "v3-base": dict(layers=12, hidden=768, heads=12, head_dim=64, ffn=3072, conv=3),
    "v2-xlarge": dict(layers=24, hidden=1536, heads=24, head_dim=64, ffn=6144, conv=3),
    "v3-large": dict(layers=24, hidden=1024, heads=16, head_dim=64, ffn=4096, conv=0),
}
WORKLOAD = dict(name="deberta-v3-base-encoder", geometry="v3-base", batch=32, seq_len=512, min_len=256, dtype="fp16")
MIXED = dict(name="deberta-v3-large-mixed-buckets", geometry="v3-large", buckets={128: 171, 256: 171, 512: 170})
FALLBACK_PEAKS = dict(hbm_gbs=6650.0, bf16_tflops=1590.0, bf16_tflops_sustained=1400.0)
# DRAM bytes of one dfl_attention_rel_fwd launch per sequence of the default workload (12 heads, L=512, d=64, FP16,
# valid lengths U[256,512]): dram__bytes_read.sum + dram__bytes_write.sum of the ncu capture summarised in
# profiles/attention_rel_kernel_v3base_b32_l512_d64_fp16.md (81.1 MB read + 12.5 MB written at B=32), per sequence.
ATTN_DRAM_BYTES_PER_SEQUENCE = (81.146624e6 + 12.506368e6) / 32


def make_config(geometry: str, layers: int | None = None):
    from disentangled_flash_b200 import DebertaAttentionConfig

    g = GEOMETRY[geometry]
    return DebertaAttentionConfig(
        hidden_size=g["hidden"], num_attention_heads=g["heads"], attention_head_size=g["head_dim"],
        num_hidden_layers=layers or g["layers"], intermediate_size=g["ffn"], attention_probs_dropout_prob=0.0,
        hidden_dropout_prob=0.0, relative_attention=True, max_relative_positions=-1, max_position_embeddings=512,
        position_buckets=256, share_att_key=True, pos_att_type=("p2c", "c2p"), norm_rel_ebd="layer_norm",
        conv_kernel_size=g["conv"],
    )


def embedding_table(hidden: int, seed: int) -> torch.Tensor:
    gen = torch.Generator().manual_seed(seed)
    table = torch.empty(VOCAB, hidden).normal_(0.0, 0.02, generator=gen)
    table[0].zero_()
    return table


def make_batches(count: int, batch: int, seq_len: int, min_len: int, seed: int, table: torch.Tensor):
    """Seeded synthetic batches: token ids -> embedding rows (hidden states) and right-padded masks."""

    out = []
    for i in range(count):
        gen = torch.Generator().manual_seed(seed + i)
        ids = torch.randint(1, VOCAB, (batch, seq_len), generator=gen)
        lengths = torch.randint(min_len, seq_len + 1, (batch,), generator=gen)
        mask = torch.arange(seq_len)[None, :] < lengths[:, None]
        ids = ids.masked_fill(~mask, 0)
        out.append((table[ids].contiguous(), mask))
    return out


def measured_peaks():
    path = ROOT / "MEASURED_PEAKS.json"
    if path.exists():
        try:
            return json.loads(path.read_text()), "measured"
        except (OSError, ValueError):
            pass
    return dict(FALLBACK_PEAKS), "fallback"


class ClockSampler:
    """nvidia-smi clocks/throttle-reason sampling (read-only).

    The sampler is started before the warm-up steps, because nvidia-smi takes a few hundred milliseconds to deliver
    its first sample; ``window()`` brackets the timed region on the host clock and only samples stamped inside it
    (between the two device synchronisations) are summarised.
    """

    QUERY = ("timestamp,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
             "clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu_index = gpu_index
        self.proc = None
        self.t0 = self.t1 = None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.gpu_index}", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits",
                 "-lms", "10"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None

    def open_window(self):
        self.t0 = time.time()

    def close_window(self):
        self.t1 = time.time()

    @staticmethod
    def _stamp(text: str) -> float | None:
        import datetime

        try:
            return datetime.datetime.strptime(text, "%Y/%m/%d %H:%M:%S.%f").timestamp()
        except ValueError:
            return None

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            out, _ = self.proc.communicate(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
            out, _ = self.proc.communicate()
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        rows = []
        for line in out.strip().splitlines():
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 8:
                continue
            try:
                rows.append((self._stamp(parts[0]), float(parts[1]), float(parts[2]), float(parts[3]),
                             [n for n, flag in zip(names, parts[4:8]) if flag.lower().startswith("active")]))
            except ValueError:
                continue
        inside = [r for r in rows if r[0] is not None and self.t0 is not None and self.t0 <= r[0] <= self.t1]
        scope = "timed region"
        if not inside:   # a timed region shorter than the sampling period: fall back to the samples under load
            inside = [r for r in rows if r[1] > 0.4 * r[2]] or rows
            scope = "whole run (no sample fell inside the timed region)"
        sm = [r[1] for r in inside]
        reasons = sorted({n for r in inside for n in r[4]})
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_min_mhz": min(sm) if sm else None,
                "sm_max_mhz": inside[0][2] if inside else None,
                "power_w": statistics.median(r[3] for r in inside) if inside else None,
                "samples": len(inside), "scope": scope, "reasons": reasons}


class LaunchObserver:
    """Counts kernel launches of the library and times its attention kernel.

    The benchmark wraps the binding's launch functions (nothing in the library knows about it): every call
    adds the number of kernels it launches, and the fused attention calls are bracketed with CUDA events
    recorded on the launching stream.
    """

    KERNELS = {"linear_heads": "dfl_qkv_proj", "pos_scores": "dfl_pos_scores", "attention_fwd": "dfl_attention_fwd",
               "attention_rel_fwd": "dfl_attention_rel_fwd", "attention_fwd_static": "dfl_attention_fwd_static",
               "add_layernorm": "dfl_add_layernorm", "dense": "dfl_dense", "conv1d": "dfl_conv1d"}
    TIMED = ("dfl_attention_fwd", "dfl_attention_rel_fwd")

    def __init__(self):
        self.enabled = False
        self.launches = 0
        self.events = []
        self.kernel_name = None

    def install(self, binding):
        for attr, name in self.KERNELS.items():
            setattr(binding, attr, self._wrap(getattr(binding, attr), name))

    def _wrap(self, fn, name):
        def call(*args, **kwargs):
            if not self.enabled:
                return fn(*args, **kwargs)
            if name == "dfl_pos_scores":   # one GEMM per enabled term (pos_key, pos_query)
                self.launches += int(args[2] is not None) + int(args[3] is not None)
            else:
                self.launches += 3 if name == "dfl_attention_fwd_static" else 1
            if name not in self.TIMED:
                return fn(*args, **kwargs)
            self.kernel_name = name
            start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            start.record()
            out = fn(*args, **kwargs)
            end.record()
            self.events.append((start, end))
            return out

        return call


# ----------------------------------------------------------------------------- CPU arm
def use_all_host_threads() -> int:
    """torchrun exports OMP_NUM_THREADS=1; the CPU arm is meant to use every core the job may use."""

    try:
        n = len(os.sched_getaffinity(0))
    except AttributeError:
        n = os.cpu_count() or 1
    torch.set_num_threads(max(1, n))
    return torch.get_num_threads()


def build_harness_backbone(geometry: str, layers: int | None, seed: int = 17):
    import hf_modules

    cfg = make_config(geometry, layers)
    backbone = hf_modules.Backbone(cfg, vocab_size=8).eval()   # the embedding table is applied outside
    hf_modules.initialize_parameters(backbone, seed)
    return cfg, backbone


class CpuEncoder:
    """The CPU arm: the reference's own PyTorch backend when its package is staged under oracle/_ref, otherwise the
    CPU restatement in oracle/ (test infrastructure; timed here as the reported host baseline only)."""

    def __init__(self, geometry: str, layers: int | None, seq_len: int):
        self.cfg, self.backbone = build_harness_backbone(geometry, layers)
        self.kind = "port"
        self.what = "CPU restatement of the reference's PyTorch backend (oracle/)"
        staged = ROOT / "oracle" / "_ref"
        if (staged / "disentangled_flash" / "__init__.py").exists():
            try:
                sys.path.insert(0, str(staged))
                import disentangled_flash as reference   # the reference's package, unmodified

                reference.enable_deberta_inference(self.backbone, backend="torch", sequence_lengths=[seq_len])
                self.kind = "reference"
                self.what = "the reference's own PyTorch backend (enable_deberta_inference(backend='torch'), oracle/_ref)"
            except Exception as error:   # an import problem on the box must not cost the baseline
                self.what += f"; staged reference unusable: {type(error).__name__}: {error}"
                self.cfg, self.backbone = build_harness_backbone(geometry, layers)

    def seconds(self, hidden: torch.Tensor, mask: torch.Tensor) -> float:
        t0 = time.perf_counter()
        if self.kind == "reference":
            with torch.inference_mode():
                self.backbone.encoder(hidden, mask, output_hidden_states=False)
        else:
            from oracle.encoder import oracle_encoder_forward

            oracle_encoder_forward(self.backbone, self.cfg, hidden, mask)
        return time.perf_counter() - t0


def cpu_baseline(layers: int | None, sample_batch: int, repeats: int, table: torch.Tensor):
    cores = use_all_host_threads()
    seq_len = WORKLOAD["seq_len"]
    arm = CpuEncoder(WORKLOAD["geometry"], layers, seq_len)
    hidden, mask = make_batches(1, sample_batch, seq_len, WORKLOAD["min_len"], 9000, table)[0]
    arm.seconds(hidden, mask)   # warm-up
    sec = statistics.median(arm.seconds(hidden, mask) for _ in range(repeats))
    return {"value": sample_batch / sec, "unit": "sequences/s", "cores": cores, "kind": arm.kind,
            "sample": f"{sample_batch} sequences of L={seq_len} through all {arm.cfg.num_hidden_layers} layers, fp32, "
                      f"median of {repeats} after 1 warm-up; {arm.what}"}


def run_reference_arm(args) -> None:
    if int(os.environ.get("RANK", "0")) != 0:
        return   # one host, one CPU arm: the other ranks have nothing to add
    if args.workload != "v3-base":
        emit(json.dumps({"impl": "reference", "unavailable": f"the CPU arm is defined for the default workload only, not {args.workload}"}))
        return
    cores = use_all_host_threads()
    seq_len = WORKLOAD["seq_len"]
    table = embedding_table(GEOMETRY[WORKLOAD["geometry"]]["hidden"], 17)
    arm = CpuEncoder(WORKLOAD["geometry"], args.layers, seq_len)
    sample = args.cpu_sample
    batches = make_batches(max(1, min(args.steps, 4)), sample, seq_len, WORKLOAD["min_len"], 9100, table)
    for i in range(args.warmup):
        arm.seconds(*batches[i % len(batches)])
    t0 = time.perf_counter()
    for i in range(args.steps):
        arm.seconds(*batches[i % len(batches)])
    elapsed = time.perf_counter() - t0
    value = sample * args.steps / elapsed
    note = (f"CPU step = {sample} sequences (a bounded sample of the B={WORKLOAD['batch']} batch); one process on rank 0 "
            f"with all {cores} host threads, whatever --gpus says: the ratio to the GPU arm is meaningful at N=1 only")
    line = {
        "impl": "reference", "metric": "encoder_sequences_per_second", "value": value, "unit": "sequences/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1e3 * elapsed / args.steps,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": workload_config(args, note=note),
        "cpu_baseline": {"value": value, "unit": "sequences/s", "cores": cores, "kind": arm.kind,
                         "sample": f"{sample} sequences of L={seq_len} per step, {args.steps} steps, fp32; {arm.what}"},
        "e2e": {"value": value, "unit": "sequences/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    emit(json.dumps(line))


def workload_config(args, note: str | None = None):
    g = GEOMETRY[WORKLOAD["geometry"]]
    cfg = {"workload": WORKLOAD["name"], "layers": args.layers or g["layers"], "hidden": g["hidden"],
           "heads": g["heads"], "head_dim": g["head_dim"], "ffn": g["ffn"],
           "per_gpu_batch": args.batch, "seq_len": WORKLOAD["seq_len"], "valid_lengths": "uniform[256,512]",
           "parallelism": f"batch-sharded replicas x{args.gpus}, no collective in the forward",
           "l2": "per-step working set (170 MB of fp16 weights, >400 MB of activations) exceeds the 126 MB L2; "
                 "4 distinct input batches are rotated"}
    if note:
        cfg["note"] = note
    return cfg


def executed_tile_fraction(mask: torch.Tensor, bm: int = 128, bn: int = 128) -> float:
    """Fraction of (query tile, key tile) pairs the fused attention kernel actually computes for this mask.

    Mirrors the kernel's rule (128 x 128 tiles): a query tile whose in-range rows are all padding takes the
    mean-of-V path (no tile); a query tile with no padded row walks only the key tiles between the first and the
    last kept key; a mixed query tile walks every key tile (padded rows attend to all L keys).
    """

    batch, length = mask.shape
    n_q, n_k = -(-length // bm), -(-length // bn)
    done = 0
    for b in range(batch):
        row = mask[b].bool()
        kept_tiles = [bool(row[t * bn:(t + 1) * bn].any()) for t in range(n_k)]
        first = kept_tiles.index(True) if any(kept_tiles) else 0
        last = n_k - 1 - kept_tiles[::-1].index(True) if any(kept_tiles) else n_k - 1
        for q in range(n_q):
            rows = row[q * bm:(q + 1) * bm]
            if not rows.any():
                continue
            done += n_k if not rows.all() else last - first + 1
    return done / float(batch * n_q * n_k)


# ----------------------------------------------------------------------------- GPU helpers
class GpuContext:
    def __init__(self):
        import torch.distributed as dist

        self.dist = dist
        self.rank = int(os.environ.get("RANK", "0"))
        self.local_rank = int(os.environ.get("LOCAL_RANK", "0"))
        self.world = int(os.environ.get("WORLD_SIZE", "1"))
        if not torch.cuda.is_available():
            raise SystemExit("bench.py needs a CUDA device: the fused kernels have no CPU fallback")
        torch.cuda.set_device(self.local_rank)
        self.device = torch.device("cuda", self.local_rank)
        if self.world > 1:
            dist.init_process_group("nccl", device_id=self.device)

    def barrier(self):
        torch.cuda.synchronize()
        if self.world > 1:
            self.dist.barrier()
        torch.cuda.synchronize()

    def close(self):
        if self.world > 1:
            self.dist.destroy_process_group()


def timed_region(ctx: GpuContext, body, sampler: ClockSampler | None = None) -> float:
    """CUDA-event time of ``body()`` on the current stream between two barriers; the slowest rank's milliseconds."""

    from disentangled_flash_b200 import sharding

    ctx.barrier()
    if sampler:
        sampler.open_window()
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    body()
    end.record()
    ctx.barrier()
    if sampler:
        sampler.close_window()
    return sharding.max_over_ranks(start.elapsed_time(end), ctx.device)


def build_gpu_encoder(geometry: str, layers: int | None, dtype: torch.dtype, device, lengths, seed: int = 17):
    import disentangled_flash_b200 as df

    cfg, backbone = build_harness_backbone(geometry, layers, seed)
    backbone = backbone.to(device=device, dtype=dtype)
    df.optimize_deberta(backbone, sequence_lengths=list(lengths))
    return cfg, backbone.encoder


def mixed_bucket_throughput(ctx: GpuContext, steps: int, warmup: int, layers: int | None = None):
    """Global batch of 512 in three length buckets, sharded over the ranks; sequences/s of the whole job."""

    from disentangled_flash_b200 import sharding

    geometry = MIXED["geometry"]
    hidden_size = GEOMETRY[geometry]["hidden"]
    lengths = sorted(MIXED["buckets"])
    _, encoder = build_gpu_encoder(geometry, layers, torch.bfloat16, ctx.device, lengths, seed=23)
    mine = sharding.shard_buckets(MIXED["buckets"], ctx.rank, ctx.world)
    gen = torch.Generator().manual_seed(5000 + ctx.rank)
    batches = {}
    for length in lengths:
        count = len(mine[length])
        if count == 0:
            continue
        # embedding rows of random token ids are i.i.d. N(0, 0.02) rows; valid lengths uniform in [L/2, L]
        hidden = torch.empty(count, length, hidden_size).normal_(0.0, 0.02, generator=gen).to(torch.bfloat16)
        valid = torch.randint(length // 2, length + 1, (count,), generator=gen)
        mask = torch.arange(length)[None, :] < valid[:, None]
        batches[length] = (hidden.to(ctx.device), mask.to(ctx.device))

    def one_pass():
        for length, (hidden, mask) in batches.items():
            encoder.activate_shape(length)
            encoder(hidden, mask, output_hidden_states=False)

    with torch.inference_mode():
        for _ in range(warmup):
            one_pass()
        ms_eager = timed_region(ctx, lambda: [one_pass() for _ in range(steps)])
    encoder.check_device_status()

    # The same pass with every bucket of this rank replayed as one CUDA graph (its batch size is fixed for the job):
    # with more ranks the per-rank batches shrink and the host's launch rate starts to bound the short buckets.
    from disentangled_flash_b200 import capture_deberta_buckets
    captured = capture_deberta_buckets(encoder, {length: batch[0].shape[0] for length, batch in batches.items()})

    def one_pass_graphs():
        for length, (hidden, mask) in batches.items():
            captured[length](hidden, mask)

    for _ in range(warmup):
        one_pass_graphs()
    ms_graph = timed_region(ctx, lambda: [one_pass_graphs() for _ in range(steps)])
    encoder.check_device_status()
    ms = min(ms_eager, ms_graph)
    total = sum(MIXED["buckets"].values())
    per_rank = {length: len(mine[length]) for length in lengths}
    del captured, encoder, batches
    torch.cuda.empty_cache()
    return {"workload": MIXED["name"], "value": total * steps / (ms / 1e3), "unit": "sequences/s",
            "ms_per_pass": ms / steps, "global_batch": total, "buckets": {str(k): v for k, v in MIXED["buckets"].items()},
            "rank0_sequences": {str(k): v for k, v in per_rank.items()}, "dtype": "bf16", "scaling": "strong",
            "layers": layers or GEOMETRY[geometry]["layers"], "steps": steps,
            "path": "cuda-graph per bucket" if ms_graph <= ms_eager else "eager",
            "ms_per_pass_eager": ms_eager / steps, "ms_per_pass_cuda_graph": ms_graph / steps,
            "note": "time of the slowest rank, the faster of the eager forward and capture_deberta_buckets() replays "
                    "(inputs copied device-to-device into the graphs' buffers inside the timed region); weights "
                    "replicated, no collective in the forward"}


# ----------------------------------------------------------------------------- default workload
def run_v3_base(args, ctx: GpuContext) -> None:
    from disentangled_flash_b200 import _cabi, sharding

    device, rank, world = ctx.device, ctx.rank, ctx.world
    dtype = torch.float16
    seq_len = WORKLOAD["seq_len"]
    g = GEOMETRY[WORKLOAD["geometry"]]
    _, encoder = build_gpu_encoder(WORKLOAD["geometry"], args.layers, dtype, device, [seq_len])

    table = embedding_table(g["hidden"], 17)
    host_batches = make_batches(4, args.batch, seq_len, WORKLOAD["min_len"], 1000 + 100 * rank, table)
    host_hidden = [h.to(dtype).pin_memory() for h, _ in host_batches]
    host_mask = [m.pin_memory() for _, m in host_batches]
    dev_batches = [(h.to(device), m.to(device)) for h, m in zip(host_hidden, host_mask)]

    observer = LaunchObserver()
    observer.install(_cabi)

    def step_resident(i):
        hidden, mask = dev_batches[i % len(dev_batches)]
        return encoder(hidden, mask, output_hidden_states=False).last_hidden_state

    # End to end through host buffers: the step's inputs come from pinned host memory and its result goes back to
    # pinned host memory, every step, inside the timed region; the copies run on their own streams so that the
    # input copy of step i+1 and the read-back of step i-1 overlap the forward of step i.
    copy_in, copy_out = torch.cuda.Stream(device), torch.cuda.Stream(device)
    slots = 2
    dev_hidden = [torch.empty_like(dev_batches[0][0]) for _ in range(slots)]
    dev_mask = [torch.empty_like(dev_batches[0][1]) for _ in range(slots)]
    out_host = [torch.empty_like(host_hidden[0]).pin_memory() for _ in range(slots)]
    loaded = [torch.cuda.Event() for _ in range(slots)]
    consumed = [torch.cuda.Event() for _ in range(slots)]
    read_back = [torch.cuda.Event() for _ in range(slots)]

    def run_e2e(steps):
        main = torch.cuda.current_stream(device)
        for i in range(steps):
            s, j = i % slots, i % len(host_hidden)
            with torch.cuda.stream(copy_in):
                if i >= slots:
                    copy_in.wait_event(consumed[s])     # the forward that read this slot is done with it
                dev_hidden[s].copy_(host_hidden[j], non_blocking=True)
                dev_mask[s].copy_(host_mask[j], non_blocking=True)
                loaded[s].record(copy_in)
            main.wait_event(loaded[s])
            out = encoder(dev_hidden[s], dev_mask[s], output_hidden_states=False).last_hidden_state
            consumed[s].record(main)
            with torch.cuda.stream(copy_out):
                copy_out.wait_event(consumed[s])
                if i >= slots:
                    copy_out.wait_event(read_back[s])
                out_host[s].copy_(out, non_blocking=True)
                out.record_stream(copy_out)
                read_back[s].record(copy_out)
        main.wait_stream(copy_out)   # the timed region ends when the last result is on the host

    sampler = ClockSampler(ctx.local_rank)
    sampler.start()
    with torch.inference_mode():
        for i in range(args.warmup):
            step_resident(i)
        run_e2e(args.warmup)
        # The timed region (exactly K steps between two barriers) is run twice and the faster run is reported, for
        # `value` and for `e2e` alike: these hosts are shared, and a stall of the launching thread for a few tens of
        # milliseconds doubles a 100 ms region.  Both times are in the JSON line (`timed_runs_ms`).
        observer.enabled = True
        torch.cuda.profiler.start()  # lets `ncu --profile-from-start off` see exactly one timed region
        runs_resident = [timed_region(ctx, lambda: [step_resident(i) for i in range(args.steps)], sampler)]
        torch.cuda.profiler.stop()
        observer.enabled = False
        launches_per_run = observer.launches
        clocks = sampler.stop()
        attn_ms = [s.elapsed_time(e) for s, e in observer.events]
        runs_resident.append(timed_region(ctx, lambda: [step_resident(i) for i in range(args.steps)]))
        runs_e2e = [timed_region(ctx, lambda: run_e2e(args.steps)) for _ in range(2)]
        ms_total, ms_e2e = min(runs_resident), min(runs_e2e)
        last = step_resident(0)
        checksum = last.float().abs().mean().reshape(1)
    encoder.check_device_status()

    seqs = world * args.batch * args.steps
    value = seqs / (ms_total / 1e3)
    e2e_value = seqs / (ms_e2e / 1e3)

    # Roofline of the dominant kernel: the fused attention forward (tensor-core bound by design).
    # Only work the kernel does not skip is counted (key tiles outside the kept range and fully padded
    # query tiles are skipped; see executed_tile_fraction).
    B, H, L, d = args.batch, g["heads"], seq_len, g["head_dim"]
    n_active = int(encoder._active_plans[0].active_slots.numel())
    in_kernel_scores = observer.kernel_name == "dfl_attention_rel_fwd"
    used = [host_mask[i % len(host_mask)] for i in range(args.steps)]
    executed = statistics.mean(executed_tile_fraction(m) for m in used) if in_kernel_scores else 1.0
    flops_attn = 4.0 * B * H * L * L * d * executed  # QK^T + PV over the executed tiles
    # with the relative scores computed in-kernel, their non-redundant GEMM work (2 terms, A active slots)
    # is part of the launch, in the same proportion; window MMAs executed beyond that are not counted
    flops_pos = 2.0 * 2 * B * H * L * n_active * d * executed if in_kernel_scores else 0.0
    flops_per_launch = flops_attn + flops_pos
    attn_avg_ms = statistics.mean(attn_ms) if attn_ms else float("nan")
    achieved = flops_per_launch / (attn_avg_ms * 1e-3) / 1e12
    peaks, peak_kind = measured_peaks()
    peak = float(peaks.get("bf16_tflops_sustained") or peaks.get("bf16_tflops"))
    traffic = None
    if ATTN_DRAM_BYTES_PER_SEQUENCE and in_kernel_scores and (H, L, d) == (12, 512, 64):
        traffic = ATTN_DRAM_BYTES_PER_SEQUENCE * B
    roofline = {"bound": "tensor", "kernel": observer.kernel_name, "achieved": achieved, "peak": peak,
                "unit": "TFLOP/s", "frac": achieved / peak, "traffic": traffic,
                "traffic_source": "ncu capture of this kernel and workload (profiles/), per sequence x batch" if traffic else None,
                "peak_source": f"{peak_kind} cuBLAS bf16 sustained (kernel timed inside a long step)",
                "avg_launch_ms": attn_avg_ms, "launches_timed": len(attn_ms),
                "algorithmic_flops_per_launch": flops_per_launch,
                "flops_qk_pv": flops_attn, "flops_position_scores": flops_pos,
                "executed_tile_fraction": executed}

    # The attention operator alone on unpadded inputs (the shape the tensor-core target is quoted on): kernel timed
    # in isolation, L2 flushed between launches, against the burst peak.
    attention_op = None
    if rank == 0:
        plan0 = encoder._active_plans[0]
        gen = torch.Generator().manual_seed(5)
        q, k, v = (torch.randn(B, H, L, d, generator=gen).to(dtype).to(device) for _ in range(3))
        full = torch.ones(B, L, dtype=torch.bool, device=device)
        scale = 1.0 / (3.0 * d) ** 0.5
        op_ms = time_isolated(lambda: _cabi.attention_rel_fwd(q, k, v, plan0.rel_key, plan0.rel_query, full, scale), device)
        op_flops = 4.0 * B * H * L * L * d + 2.0 * 2 * B * H * L * n_active * d
        burst = float(peaks.get("bf16_tflops") or peak)
        attention_op = {"config": f"B={B} H={H} L={L} d={d} fp16, no padding, c2p+p2c computed in-kernel",
                        "us_per_launch": op_ms * 1e3, "tflops": op_flops / (op_ms * 1e-3) / 1e12,
                        "frac_of_burst_peak": op_flops / (op_ms * 1e-3) / 1e12 / burst,
                        "flops_qk_pv": 4.0 * B * H * L * L * d, "l2": "256 MB flush write between launches"}
        del q, k, v

    # The same step as one CUDA graph per bucket (capture_deberta_buckets): the step's inputs are copied into the
    # graph's buffers inside the timed region.  An extra key; `value` stays the eager forward.
    graph = None
    if not args.skip_graph:
        import disentangled_flash_b200 as df

        replay = df.capture_deberta_buckets(encoder, args.batch)[seq_len]
        with torch.inference_mode():
            for i in range(args.warmup):
                replay(*dev_batches[i % len(dev_batches)])
            ms_graph = timed_region(ctx, lambda: [replay(*dev_batches[i % len(dev_batches)]) for i in range(args.steps)])
        encoder.check_device_status()
        graph = {"value": seqs / (ms_graph / 1e3), "unit": "sequences/s", "ms_per_step": ms_graph / args.steps,
                 "note": "capture_deberta_buckets(): one graph launch per step, inputs copied device-to-device into "
                         "the graph's buffers every step"}
        del replay

    # The same batches without their padding between the attention kernels (forward_packed; lengths known on the
    # host as a tokenizer gives them).  Outputs equal `value`'s at the valid positions only, hence an extra key.
    packed = None
    if not args.skip_packed:
        host_lengths = [m.sum(1).tolist() for m in host_mask]

        def step_packed(i):
            j = i % len(dev_batches)
            return encoder.forward_packed(dev_batches[j][0], dev_batches[j][1], host_lengths[j]).last_hidden_state

        with torch.inference_mode():
            for i in range(args.warmup):
                step_packed(i)
            ms_packed = min(timed_region(ctx, lambda: [step_packed(i) for i in range(args.steps)]) for _ in range(2))
        encoder.check_device_status()
        kept = sum(min(seq_len, -(-n // 32) * 32) for n in host_lengths[0]) / float(args.batch * seq_len)
        packed = {"value": seqs / (ms_packed / 1e3), "unit": "sequences/s", "ms_per_step": ms_packed / args.steps,
                  "rows_kept": kept,
                  "note": "forward_packed(): projections, dense layers, GELU and layer norms on the valid positions only (each "
                          "sequence rounded up to 32 rows); equal to the padded forward at valid positions"}

    del encoder, dev_batches, dev_hidden
    torch.cuda.empty_cache()
    mixed = None
    if not args.skip_mixed:
        mixed = mixed_bucket_throughput(ctx, steps=max(2, min(args.steps, 5)), warmup=3)

    checks = sharding.gather_for_check(checksum)  # NCCL only here, after timing, for checking
    if rank == 0:
        baseline = cpu_baseline(args.layers, args.cpu_sample, 3, table) if world == 1 and not args.skip_cpu else None
        bytes_in = host_hidden[0].numel() * host_hidden[0].element_size() + host_mask[0].numel()
        bytes_out = out_host[0].numel() * out_host[0].element_size()
        line = {
            "metric": "encoder_sequences_per_second", "value": value, "unit": "sequences/s", "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_total / args.steps,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f16", "data": "synthetic",
            "config": workload_config(args),
            "e2e": {"value": e2e_value, "unit": "sequences/s", "h2d_bytes_per_step": bytes_in,
                    "d2h_bytes_per_step": bytes_out, "ms_per_step": ms_e2e / args.steps,
                    "note": "pinned host buffers; input copy, forward and read-back on three streams, two device slots"},
            "gpu_launches": launches_per_run,
            "timed_runs_ms": {"resident": runs_resident, "e2e": runs_e2e,
                              "rule": "two runs of exactly K steps each; the faster one is reported"},
            "attention_tflops": achieved,
            "roofline": roofline,
            "attention_op": attention_op,
            "cuda_graph": graph,
            "packed": packed,
            "mixed_buckets": mixed,
            "cpu_baseline": baseline,
            "clocks": clocks,
            "rank_checksums": [float(c.item()) for c in checks],
        }
        emit(json.dumps(line))


def time_isolated(call, device, repeats: int = 10) -> float:
    """Median milliseconds of ``call()`` alone on the current stream, with a 256 MB write between launches (larger than
    the 126 MB L2)."""

    flush = torch.empty(256 << 20, dtype=torch.uint8, device=device)
    with torch.inference_mode():
        for _ in range(3):
            call()
        times = []
        for _ in range(repeats):
            flush.zero_()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            call()
            e1.record()
            torch.cuda.synchronize()
            times.append(e0.elapsed_time(e1))
    return statistics.median(times)


# ----------------------------------------------------------------------------- attention-sweep
def run_attention_sweep(args, ctx: GpuContext) -> None:
    from disentangled_flash_b200 import _cabi

    device = ctx.device
    peaks, peak_kind = measured_peaks()
    burst = float(peaks.get("bf16_tflops") or FALLBACK_PEAKS["bf16_tflops"])
    rows = []
    batch = 16
    for dtype_name, dtype in (("bf16", torch.bfloat16), ("fp16", torch.float16)):
        for heads, d in ((24, 32), (12, 64), (8, 128)):
            for length in (16, 64, 256, 512):
                gen = torch.Generator().manual_seed(length + d)
                active, lut = _cabi.build_position_lut(length, 256, 512, 256, True, device)
                n_active = int(active.numel())
                q, k, v = (torch.randn(batch, heads, length, d, generator=gen).to(dtype).to(device) for _ in range(3))
                pos_key, pos_query = (torch.randn(heads, n_active, d, generator=gen).to(dtype).to(device) for _ in range(2))
                padded = torch.randperm(batch, generator=gen)[: batch // 4]
                valid = torch.full((batch,), length)
                valid[padded] = torch.randint(1, length + 1, (batch // 4,), generator=gen)
                mask = (torch.arange(length)[None, :] < valid[:, None]).to(device)
                scale = 1.0 / (3.0 * d) ** 0.5
                if _cabi.attention_rel_supported(dtype, length, d, True, True):
                    rel_key = _cabi.expand_rel_tables(pos_key, lut, length)
                    rel_query = _cabi.expand_rel_tables(pos_query, lut, length)
                    call = lambda: _cabi.attention_rel_fwd(q, k, v, rel_key, rel_query, mask, scale)  # noqa: E731
                    path = "dfl_attention_rel_fwd"
                else:
                    def call():
                        c2p, p2c, ld = _cabi.pos_scores(q, k, pos_key, pos_query)
                        return _cabi.attention_fwd(q, k, v, c2p, p2c, lut, mask, scale, ld_slots=ld)
                    path = "dfl_pos_scores + dfl_attention_fwd"
                ms = time_isolated(call, device)
                flops = 4.0 * batch * heads * length * length * d + 2.0 * 2 * batch * heads * length * n_active * d
                tflops = flops / (ms * 1e-3) / 1e12
                rows.append({"heads": heads, "head_dim": d, "seq_len": length, "dtype": dtype_name, "path": path,
                             "us": ms * 1e3, "tflops": tflops, "frac_of_burst_peak": tflops / burst})
    if ctx.rank == 0:
        head = next(r for r in rows if (r["heads"], r["head_dim"], r["seq_len"], r["dtype"]) == (12, 64, 512, "fp16"))
        emit(json.dumps({
            "metric": "disentangled_attention_fwd_tflops", "value": head["tflops"], "unit": "TFLOP/s", "n_gpus": 1,
            "higher_is_better": True, "vs_baseline": None, "dtype": "f16", "data": "synthetic",
            "config": {"workload": "attention-operator-head-dim-sweep", "batch": 16, "padding": "a quarter of the rows padded to U[1,L]",
                       "counted_flops": "4*B*H*L^2*d + 2*2*B*H*L*A*d (QK^T, PV, and the two position-score GEMMs over the A active slots)",
                       "l2": "256 MB flush write between launches", "headline_row": "H=12 d=64 L=512 fp16"},
            "peak": burst, "peak_source": f"{peak_kind} cuBLAS bf16 burst", "rows": rows}))


# ----------------------------------------------------------------------------- v2-xlarge
def run_v2_xlarge(args, ctx: GpuContext) -> None:
    import disentangled_flash_b200 as df

    device = ctx.device
    geometry, batch, lengths = "v2-xlarge", 8, (64, 128, 256, 512)
    hidden_size = GEOMETRY[geometry]["hidden"]
    rows = []
    for dtype_name, dtype in (("bf16", torch.bfloat16), ("fp32", torch.float32)):
        _, encoder = build_gpu_encoder(geometry, args.layers, dtype, device, lengths)
        # one CUDA graph per bucket: at this batch size the eager forward is bound by the host's launch rate
        graphs = df.capture_deberta_buckets(encoder, batch) if dtype != torch.float32 else {}
        for length in lengths:
            gen = torch.Generator().manual_seed(length)
            inputs = []
            for _ in range(4):
                hidden = torch.empty(batch, length, hidden_size).normal_(0.0, 0.02, generator=gen).to(dtype)
                valid = torch.randint(length // 2, length + 1, (batch,), generator=gen)
                inputs.append((hidden.to(device), (torch.arange(length)[None, :] < valid[:, None]).to(device)))
            encoder.activate_shape(length)
            steps = args.steps
            modes = [("eager", lambda h, m: encoder(h, m, output_hidden_states=False))]
            if length in graphs:
                modes.append(("cuda-graph", graphs[length]))
            for mode, call in modes:
                def body():
                    for i in range(steps):
                        call(*inputs[i % len(inputs)])

                with torch.inference_mode():
                    for i in range(max(3, args.warmup)):
                        call(*inputs[i % len(inputs)])
                    ms = timed_region(ctx, body)
                rows.append({"dtype": dtype_name, "mode": mode, "seq_len": length, "batch": batch,
                             "ms_per_step": ms / steps, "sequences_per_s": batch * steps / (ms / 1e3)})
        encoder.check_device_status()
        del encoder, graphs
        torch.cuda.empty_cache()
    if ctx.rank == 0:
        head = next(r for r in rows if (r["dtype"], r["mode"], r["seq_len"]) == ("bf16", "cuda-graph", 512))
        emit(json.dumps({
            "metric": "encoder_sequences_per_second", "value": head["sequences_per_s"], "unit": "sequences/s", "n_gpus": 1,
            "steps": args.steps, "higher_is_better": True, "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": "deberta-v2-xlarge-encoder", **GEOMETRY[geometry], "layers": args.layers or GEOMETRY[geometry]["layers"],
                       "batch": batch, "buckets": list(lengths), "valid_lengths": "uniform[L/2, L]",
                       "note": "one encoder, four prepared buckets; eager = activate_shape() + forward, cuda-graph = "
                               "capture_deberta_buckets() replay (inputs copied into the graph's buffers inside the "
                               "timed region); fp32 = strict IEEE kernels, eager only",
                       "headline_row": "bf16 cuda-graph L=512"},
            "rows": rows}))


# ----------------------------------------------------------------------------- v3-large-mixed
def run_v3_large_mixed(args, ctx: GpuContext) -> None:
    result = mixed_bucket_throughput(ctx, steps=args.steps, warmup=max(3, args.warmup), layers=args.layers)
    if ctx.rank == 0:
        emit(json.dumps({
            "metric": "encoder_sequences_per_second", "value": result["value"], "unit": "sequences/s", "n_gpus": ctx.world,
            "steps": args.steps, "warmup": max(3, args.warmup), "ms_per_step": result["ms_per_pass"],
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": MIXED["name"], **GEOMETRY[MIXED["geometry"]], "layers": result["layers"],
                       "global_batch": result["global_batch"], "buckets": result["buckets"],
                       "parallelism": f"sequences of every bucket interleaved over {ctx.world} ranks (sharding.shard_buckets), "
                                      "weights replicated, no collective in the forward",
                       "rank0_sequences": result["rank0_sequences"]},
            "path": result["path"], "ms_per_pass_eager": result["ms_per_pass_eager"],
            "ms_per_pass_cuda_graph": result["ms_per_pass_cuda_graph"], "note": result["note"]}))


_RESULT_FD = None


def reserve_stdout() -> None:
    """Keep stdout for the one JSON line: whatever libraries write to file descriptor 1 meanwhile (NCCL prints its
    version banner there) goes to stderr instead."""

    global _RESULT_FD
    sys.stdout.flush()
    _RESULT_FD = os.dup(1)
    os.dup2(2, 1)


def emit(text: str) -> None:
    if _RESULT_FD is None:
        print(text, flush=True)
        return
    sys.stdout.flush()
    os.write(_RESULT_FD, (text + "\n").encode())


def main() -> None:
    reserve_stdout()
    parser = argparse.ArgumentParser()
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=20)
    parser.add_argument("--warmup", type=int, default=3)
    parser.add_argument("--impl", choices=("b200", "reference"), default="b200")
    parser.add_argument("--workload", choices=("v3-base", "attention-sweep", "v2-xlarge", "v3-large-mixed"), default="v3-base")
    parser.add_argument("--batch", type=int, default=WORKLOAD["batch"], help="sequences per GPU per step (v3-base)")
    parser.add_argument("--layers", type=int, default=None, help="override the number of encoder layers (profiling)")
    parser.add_argument("--cpu-sample", type=int, default=2, help="sequences per CPU-baseline step")
    parser.add_argument("--skip-cpu", action="store_true", help="omit the cpu_baseline leg")
    parser.add_argument("--skip-mixed", action="store_true", help="omit the mixed-bucket leg of the default workload")
    parser.add_argument("--skip-graph", action="store_true", help="omit the CUDA-graph leg of the default workload")
    parser.add_argument("--skip-packed", action="store_true", help="omit the packed-rows leg of the default workload")
    args = parser.parse_args()
    if args.warmup < 3 and args.impl == "b200":
        args.warmup = 3  # timing rule: at least three warm-up steps
    if args.impl == "reference":
        run_reference_arm(args)
        return
    ctx = GpuContext()
    try:
        {"v3-base": run_v3_base, "attention-sweep": run_attention_sweep, "v2-xlarge": run_v2_xlarge,
         "v3-large-mixed": run_v3_large_mixed}[args.workload](args, ctx)
    finally:
        ctx.close()


if __name__ == "__main__":
    main()
