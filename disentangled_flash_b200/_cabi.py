"""ctypes binding of ``libdfl_b200.so`` (the C ABI in ``include/dfl_b200.h``).

PyTorch is used here only as the owner of device memory and of the current
CUDA stream: every wrapper takes tensors, checks layout, and passes raw
device pointers plus sizes to the C functions.  There is no Python or CPU
implementation behind these calls; if the library is missing the import
fails loudly.
"""

from __future__ import annotations

import ctypes
from ctypes import POINTER, Structure, c_char_p, c_float, c_int, c_int32, c_uint32, c_void_p
from pathlib import Path

import torch

LIB_PATH = Path(__file__).resolve().parent / "libdfl_b200.so"

DFL_F16, DFL_BF16, DFL_F32 = 0, 1, 2
ALGO_AUTO, ALGO_SIMT = 0, 1

DFL_ERR_BAD_ARG = -1
DFL_ERR_UNSUPPORTED = -2
DFL_ERR_ALIGNMENT = -3
DFL_ERR_LAUNCH = -4
DFL_ERR_DRIVER = -5
DFL_ERR_DEVICE_TIMEOUT = -6
DFL_ERR_TOO_LARGE = -7

_DTYPES = {torch.float16: DFL_F16, torch.bfloat16: DFL_BF16, torch.float32: DFL_F32}

EXPORTED_SYMBOLS = (
    "dfl_version",
    "dfl_status_string",
    "dfl_last_error",
    "dfl_check_status",
    "dfl_selftest_bounded_wait",
    "dfl_build_position_lut",
    "dfl_qkv_proj",
    "dfl_gather_slots",
    "dfl_add_layernorm",
    "dfl_embed_layernorm",
    "dfl_dense",
    "dfl_conv1d",
    "dfl_copy_rows",
    "dfl_conv1d_supported",
    "dfl_add_layernorm_supported",
    "dfl_pos_scores",
    "dfl_attention_fwd",
    "dfl_attention_fwd_static",
    "dfl_static_scratch_bytes",
    "dfl_expand_rel_tables",
    "dfl_attention_rel_supported",
    "dfl_attention_rel_fwd",
)


class DflLinearParams(Structure):
    _fields_ = [
        ("x", c_void_p), ("w", c_void_p), ("bias", c_void_p), ("out", c_void_p * 3),
        ("M", c_int32), ("K", c_int32), ("n_out", c_int32), ("heads", c_int32), ("head_dim", c_int32),
        ("rows_per_seq", c_int32), ("dtype", c_int32), ("algo", c_int32), ("status", c_void_p),
        ("row_groups", c_void_p), ("out_seqs", c_int32),
    ]


class DflPosScoreParams(Structure):
    _fields_ = [
        ("q", c_void_p), ("k", c_void_p), ("pos_key", c_void_p), ("pos_query", c_void_p),
        ("c2p", c_void_p), ("p2c", c_void_p),
        ("batch", c_int32), ("heads", c_int32), ("seq_len", c_int32), ("head_dim", c_int32),
        ("n_active", c_int32), ("ld_slots", c_int32), ("dtype", c_int32), ("algo", c_int32), ("status", c_void_p),
    ]


class DflAttnParams(Structure):
    _fields_ = [
        ("q", c_void_p), ("k", c_void_p), ("v", c_void_p), ("c2p", c_void_p), ("p2c", c_void_p),
        ("lut", c_void_p), ("mask", c_void_p), ("out", c_void_p), ("status", c_void_p),
        ("batch", c_int32), ("heads", c_int32), ("seq_len", c_int32), ("head_dim", c_int32),
        ("ld_slots", c_int32), ("mask_elem_size", c_int32), ("scale", c_float),
        ("dtype", c_int32), ("algo", c_int32),
    ]


class DflAttnTablesParams(Structure):
    _fields_ = [
        ("q", c_void_p), ("k", c_void_p), ("v", c_void_p), ("pos_key", c_void_p), ("pos_query", c_void_p),
        ("lut", c_void_p), ("mask", c_void_p), ("out", c_void_p), ("status", c_void_p),
        ("batch", c_int32), ("heads", c_int32), ("seq_len", c_int32), ("head_dim", c_int32),
        ("n_active", c_int32), ("mask_elem_size", c_int32), ("scale", c_float),
        ("dtype", c_int32), ("algo", c_int32),
    ]


class DflAttnRelParams(Structure):
    _fields_ = [
        ("q", c_void_p), ("k", c_void_p), ("v", c_void_p), ("rel_key", c_void_p), ("rel_query", c_void_p),
        ("mask", c_void_p), ("out", c_void_p), ("status", c_void_p),
        ("batch", c_int32), ("heads", c_int32), ("seq_len", c_int32), ("head_dim", c_int32),
        ("mask_elem_size", c_int32), ("scale", c_float), ("dtype", c_int32), ("algo", c_int32),
        ("out_row_base", c_void_p), ("out_row_count", c_void_p),
    ]


class DflDenseParams(Structure):
    _fields_ = [("x", c_void_p), ("w", c_void_p), ("bias", c_void_p), ("out", c_void_p),
                ("M", c_int32), ("N", c_int32), ("K", c_int32), ("activation", c_int32), ("dtype", c_int32),
                ("algo", c_int32), ("status", c_void_p)]


ACT_NONE, ACT_GELU, ACT_TANH = 0, 1, 2


class DflConv1dParams(Structure):
    _fields_ = [("x", c_void_p), ("w", c_void_p), ("bias", c_void_p), ("row_mask", c_void_p), ("out", c_void_p),
                ("batch", c_int32), ("seq_len", c_int32), ("c_in", c_int32), ("c_out", c_int32), ("taps", c_int32),
                ("mask_elem_size", c_int32), ("activation", c_int32), ("dtype", c_int32), ("status", c_void_p)]


class DflAddLayerNormParams(Structure):
    _fields_ = [("x", c_void_p), ("residual", c_void_p), ("gamma", c_void_p), ("beta", c_void_p), ("out", c_void_p),
                ("rows", ctypes.c_int64), ("hidden", c_int), ("eps", ctypes.c_float), ("dtype", c_int),
                ("row_mask", c_void_p), ("mask_elem_size", c_int), ("out2", c_void_p), ("out2_rows", c_void_p)]


class DflEmbedLayerNormParams(Structure):
    _fields_ = [("ids", c_void_p), ("table", c_void_p), ("pos_ids", c_void_p), ("pos_table", c_void_p),
                ("gamma", c_void_p), ("beta", c_void_p), ("row_mask", c_void_p), ("out", c_void_p),
                ("rows", ctypes.c_int64), ("vocab", ctypes.c_int64), ("positions", ctypes.c_int64),
                ("hidden", c_int), ("eps", ctypes.c_float), ("dtype", c_int), ("id_elem_size", c_int),
                ("mask_elem_size", c_int), ("status", c_void_p)]


class DflError(RuntimeError):
    """A C entry point returned a negative status."""

    def __init__(self, status: int, where: str, detail: str):
        super().__init__(f"{where}: {detail} (status {status})")
        self.status = status


_lib = None

def load_library() -> ctypes.CDLL:
    """Load the shared library once; raise if it has not been built."""

    global _lib
    if _lib is not None:
        return _lib
    if not LIB_PATH.exists():
        raise RuntimeError(
            f"{LIB_PATH} is missing: build it with `python -m disentangled_flash_b200.build` "
            "(needs nvcc; there is no CPU or PyTorch fallback for these kernels)"
        )
    lib = ctypes.CDLL(str(LIB_PATH))
    lib.dfl_version.restype = c_int
    lib.dfl_status_string.restype = c_char_p
    lib.dfl_status_string.argtypes = [c_int]
    lib.dfl_last_error.restype = c_char_p
    lib.dfl_check_status.restype = c_int
    lib.dfl_check_status.argtypes = [c_void_p, c_void_p]
    lib.dfl_selftest_bounded_wait.restype = c_int
    lib.dfl_selftest_bounded_wait.argtypes = [c_void_p, c_uint32, c_void_p]
    lib.dfl_build_position_lut.restype = c_int
    lib.dfl_build_position_lut.argtypes = [c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p]
    lib.dfl_qkv_proj.restype = c_int
    lib.dfl_qkv_proj.argtypes = [POINTER(DflLinearParams), c_void_p]
    lib.dfl_conv1d_supported.restype = c_int
    lib.dfl_conv1d_supported.argtypes = [POINTER(DflConv1dParams)]
    lib.dfl_conv1d.restype = c_int
    lib.dfl_conv1d.argtypes = [POINTER(DflConv1dParams), c_void_p]
    lib.dfl_copy_rows.restype = c_int
    lib.dfl_copy_rows.argtypes = [c_void_p, c_void_p, c_void_p, ctypes.c_int64, c_int32, c_void_p]
    lib.dfl_dense.restype = c_int
    lib.dfl_dense.argtypes = [POINTER(DflDenseParams), c_void_p]
    lib.dfl_add_layernorm_supported.restype = c_int
    lib.dfl_add_layernorm_supported.argtypes = [c_int, c_int]
    lib.dfl_add_layernorm.restype = c_int
    lib.dfl_add_layernorm.argtypes = [POINTER(DflAddLayerNormParams), c_void_p]
    lib.dfl_embed_layernorm.restype = c_int
    lib.dfl_embed_layernorm.argtypes = [POINTER(DflEmbedLayerNormParams), c_void_p]
    lib.dfl_gather_slots.restype = c_int
    lib.dfl_gather_slots.argtypes = [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p]
    lib.dfl_pos_scores.restype = c_int
    lib.dfl_pos_scores.argtypes = [POINTER(DflPosScoreParams), c_void_p]
    lib.dfl_attention_fwd.restype = c_int
    lib.dfl_attention_fwd.argtypes = [POINTER(DflAttnParams), c_void_p]
    lib.dfl_attention_fwd_static.restype = c_int
    lib.dfl_attention_fwd_static.argtypes = [POINTER(DflAttnTablesParams), c_void_p]
    lib.dfl_static_scratch_bytes.restype = ctypes.c_size_t
    lib.dfl_expand_rel_tables.restype = c_int
    lib.dfl_expand_rel_tables.argtypes = [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p]
    lib.dfl_attention_rel_supported.restype = c_int
    lib.dfl_attention_rel_supported.argtypes = [POINTER(DflAttnRelParams)]
    lib.dfl_attention_rel_fwd.restype = c_int
    lib.dfl_attention_rel_fwd.argtypes = [POINTER(DflAttnRelParams), c_void_p]
    _lib = lib
    return lib


def _check(status: int, where: str) -> None:
    if status == 0:
        return
    lib = load_library()
    detail = (lib.dfl_last_error() or b"").decode() or lib.dfl_status_string(status).decode()
    if status in (DFL_ERR_BAD_ARG, DFL_ERR_ALIGNMENT, DFL_ERR_TOO_LARGE):
        raise ValueError(f"{where}: {detail} (status {status})")
    raise DflError(status, where, detail)


def new_status_word(device: torch.device | str) -> torch.Tensor:
    """A zeroed device int32 to pass as ``status=`` to the kernel wrappers (see ``check_status``)."""

    return torch.zeros(1, dtype=torch.int32, device=device)


def check_status(status: torch.Tensor) -> None:
    """Read a status word back (synchronises the current stream); raise if a bounded device-side wait expired.

    Mirrors ``dfl_check_status``: the word is cleared when it was non-zero, and the outputs of the calls made
    with it since the previous check are not valid.  Meant for the end of a batch, not for the hot path.
    """

    lib = load_library()
    if status.dtype != torch.int32 or status.numel() != 1 or status.device.type != "cuda":
        raise ValueError("status must be a CUDA int32 tensor with one element")
    with _on_device(status.device):
        _check(lib.dfl_check_status(status.data_ptr(), _stream(status.device)), "dfl_check_status")


def selftest_bounded_wait(status: torch.Tensor, limit_us: int) -> None:
    """Launch the diagnostic kernel whose only wait can never complete (``dfl_selftest_bounded_wait``)."""

    lib = load_library()
    with _on_device(status.device):
        _check(lib.dfl_selftest_bounded_wait(status.data_ptr(), int(limit_us), _stream(status.device)),
               "dfl_selftest_bounded_wait")


def dtype_code(dtype: torch.dtype) -> int:
    try:
        return _DTYPES[dtype]
    except KeyError:
        raise TypeError("the B200 path supports FP16, BF16, and FP32") from None


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def _stream(device: torch.device) -> int:
    """The current stream of ``device`` as an integer handle (the short way round when torch offers it: a forward
    of a small batch is bound by what the host spends per launch)."""

    if _raw_stream is not None and device.index is not None:
        return _raw_stream(device.index)
    return torch.cuda.current_stream(device).cuda_stream


class _on_device:
    """``with _on_device(dev):`` makes ``dev`` the current CUDA device for the call, and costs one query when it
    already is (``torch.cuda.device`` switches and restores unconditionally)."""

    __slots__ = ("index", "previous")

    def __init__(self, device: torch.device | str):
        device = torch.device(device)
        self.index = device.index
        self.previous = -1

    def __enter__(self) -> None:
        if self.index is None:
            return
        current = torch.cuda.current_device()
        if current != self.index:
            self.previous = current
            torch.cuda.set_device(self.index)

    def __exit__(self, *exc) -> None:
        if self.previous >= 0:
            torch.cuda.set_device(self.previous)
            self.previous = -1


def _ptr(t: torch.Tensor | None) -> int | None:
    return None if t is None else t.data_ptr()


def _require_cuda_contiguous(name: str, t: torch.Tensor) -> None:
    if t.device.type != "cuda":
        raise RuntimeError(f"{name} must be a CUDA tensor")
    if not t.is_contiguous():
        raise ValueError(f"{name} must be contiguous")


def build_position_lut(seq_len: int, position_buckets: int, max_relative_positions: int, span: int,
                       uses_position_bias: bool, device: torch.device):
    """Run the index-builder kernel; returns ``(active_slots int64[A], delta_to_local int32[2L-1])``."""

    lib = load_library()
    if seq_len < 1:
        raise ValueError("sequence_length must be positive")
    n = 2 * seq_len - 1
    cap = max(1, min(n, 2 * max(span, 1)))
    with _on_device(device):
        lut = torch.empty(n, dtype=torch.int32, device=device)
        active = torch.empty(cap, dtype=torch.int64, device=device)
        count = torch.zeros(1, dtype=torch.int32, device=device)
        _check(lib.dfl_build_position_lut(seq_len, position_buckets, max_relative_positions, span,
                                          int(uses_position_bias), lut.data_ptr(), active.data_ptr(),
                                          count.data_ptr(), _stream(device)), "dfl_build_position_lut")
        n_active = int(count.item())  # prepare-time only: one 4-byte read-back per bucket length
    return active[:n_active].clone(), lut


def linear_heads(x: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor | None, *, n_out: int, heads: int,
                 head_dim: int, rows_per_seq: int, algo: int = ALGO_AUTO,
                 status: torch.Tensor | None = None, row_groups: torch.Tensor | None = None,
                 outs: tuple[torch.Tensor, ...] | None = None) -> tuple[torch.Tensor, ...]:
    """``x[M,K] @ weight[N,K]^T + bias`` written as ``n_out`` tensors ``[M/rows, heads, rows, head_dim]``.

    With ``row_groups`` (int32 ``[M/32]``) the rows of ``x`` are packed: group ``g`` of 32 rows goes to output rows
    ``row_groups[g] .. +31`` of the caller's ``outs`` (``[B, heads, rows, head_dim]`` each), whose other rows stay
    as they are."""

    lib = load_library()
    _require_cuda_contiguous("x", x)
    _require_cuda_contiguous("weight", weight)
    x2 = x.reshape(-1, x.shape[-1])
    m, k = x2.shape
    if weight.shape != (n_out * heads * head_dim, k):
        raise ValueError(f"weight shape {tuple(weight.shape)} does not match [{n_out * heads * head_dim}, {k}]")
    p = DflLinearParams()
    if row_groups is not None:
        if outs is None or len(outs) != n_out:
            raise ValueError("packed rows need the caller's output tensors")
        if row_groups.dtype != torch.int32 or row_groups.numel() * 32 != m:
            raise ValueError("row_groups must hold one int32 per 32 rows of x")
        _require_cuda_contiguous("row_groups", row_groups)
        for o in outs:
            _require_cuda_contiguous("out", o)
            if o.dtype != x.dtype or o.dim() != 4 or tuple(o.shape[1:]) != (heads, rows_per_seq, head_dim):
                raise ValueError(f"output must be [B, {heads}, {rows_per_seq}, {head_dim}] of {x.dtype}")
        p.row_groups, p.out_seqs = row_groups.data_ptr(), outs[0].shape[0]
    else:
        outs = tuple(torch.empty(m // rows_per_seq, heads, rows_per_seq, head_dim, dtype=x.dtype, device=x.device)
                     for _ in range(n_out))
    p.x, p.w, p.bias = x2.data_ptr(), weight.data_ptr(), _ptr(bias)
    for i, o in enumerate(outs):
        p.out[i] = o.data_ptr()
    p.M, p.K, p.n_out, p.heads, p.head_dim, p.rows_per_seq = m, k, n_out, heads, head_dim, rows_per_seq
    p.dtype, p.algo, p.status = dtype_code(x.dtype), algo, _ptr(status)
    with _on_device(x.device):
        _check(lib.dfl_qkv_proj(ctypes.byref(p), _stream(x.device)), "dfl_qkv_proj")
    return outs


def gather_slots(src: torch.Tensor, active: torch.Tensor) -> torch.Tensor:
    """``src[H, S, d] -> [H, A, d]`` by the active-slot list."""

    lib = load_library()
    _require_cuda_contiguous("src", src)
    heads, n_src, d = src.shape
    n_active = active.numel()
    dst = torch.empty(heads, n_active, d, dtype=src.dtype, device=src.device)
    with _on_device(src.device):
        _check(lib.dfl_gather_slots(src.data_ptr(), active.data_ptr(), dst.data_ptr(), heads, n_src, n_active, d,
                                    dtype_code(src.dtype), _stream(src.device)), "dfl_gather_slots")
    return dst


def dense(x: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor | None, *, activation: int = ACT_NONE,
          algo: int = ALGO_AUTO, status: torch.Tensor | None = None) -> torch.Tensor:
    """``act(x @ weight^T + bias)`` over the last dimension of ``x`` with bias and activation in the GEMM epilogue."""

    lib = load_library()
    for name, t in (("x", x), ("weight", weight), ("bias", bias)):
        if t is None:
            continue
        _require_cuda_contiguous(name, t)
        if t.dtype != x.dtype:
            raise TypeError(f"{name} must have the dtype of x ({x.dtype}), got {t.dtype}")
    n, k = weight.shape
    if x.shape[-1] != k or (bias is not None and bias.numel() != n):
        raise ValueError("shapes of x, weight and bias do not agree")
    out = torch.empty(*x.shape[:-1], n, dtype=x.dtype, device=x.device)
    p = DflDenseParams()
    p.x, p.w, p.bias, p.out = _ptr(x), _ptr(weight), _ptr(bias), _ptr(out)
    p.M, p.N, p.K = x.numel() // k, n, k
    p.activation, p.dtype, p.algo, p.status = activation, dtype_code(x.dtype), algo, _ptr(status)
    with _on_device(x.device):
        _check(lib.dfl_dense(ctypes.byref(p), _stream(x.device)), "dfl_dense")
    return out


def add_layernorm_supported(dtype: torch.dtype, hidden: int) -> bool:
    """Whether ``add_layernorm`` covers rows of ``hidden`` elements of this type."""

    if dtype not in (torch.float16, torch.bfloat16, torch.float32):
        return False
    return bool(load_library().dfl_add_layernorm_supported(dtype_code(dtype), int(hidden)))


def _conv1d_params(x, weight, bias, row_mask, out, activation, status) -> DflConv1dParams:
    p = DflConv1dParams()
    p.x, p.w, p.bias, p.row_mask, p.out = _ptr(x), _ptr(weight), _ptr(bias), _ptr(row_mask), _ptr(out)
    p.batch, p.seq_len, p.c_in = x.shape
    p.taps, p.c_out = weight.shape[0], weight.shape[1]
    p.mask_elem_size = row_mask.element_size() if row_mask is not None else 1
    p.activation, p.dtype, p.status = activation, dtype_code(x.dtype), _ptr(status)
    return p


def conv1d_supported(dtype: torch.dtype, seq_len: int, c_in: int, c_out: int, taps: int, activation: int) -> bool:
    """Whether ``conv1d`` covers this configuration."""

    if dtype not in (torch.float16, torch.bfloat16):
        return False
    p = DflConv1dParams()
    p.batch, p.seq_len, p.c_in, p.c_out, p.taps = 1, seq_len, c_in, c_out, taps
    p.activation, p.dtype, p.mask_elem_size = activation, dtype_code(dtype), 1
    return bool(load_library().dfl_conv1d_supported(ctypes.byref(p)))


def conv1d(x: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor | None, row_mask: torch.Tensor | None, *,
           activation: int = ACT_NONE, status: torch.Tensor | None = None) -> torch.Tensor:
    """``act(keep * (conv1d(x) + bias))`` over the sequence: x [B, L, C_in], weight [taps, C_out, C_in] -> [B, L, C_out]."""

    lib = load_library()
    for name, t in (("x", x), ("weight", weight), ("bias", bias), ("row_mask", row_mask)):
        if t is not None:
            _require_cuda_contiguous(name, t)
    if weight.dtype != x.dtype or (bias is not None and bias.dtype != x.dtype):
        raise TypeError("weight and bias must have the dtype of x")
    if x.dim() != 3 or weight.dim() != 3 or weight.shape[2] != x.shape[2]:
        raise ValueError("x must be [B, L, C_in] and weight [taps, C_out, C_in]")
    if row_mask is not None and tuple(row_mask.shape) != tuple(x.shape[:2]):
        raise ValueError("row_mask must be [B, L]")
    out = torch.empty(x.shape[0], x.shape[1], weight.shape[1], dtype=x.dtype, device=x.device)
    p = _conv1d_params(x, weight, bias, row_mask, out, activation, status)
    with _on_device(x.device):
        _check(lib.dfl_conv1d(ctypes.byref(p), _stream(x.device)), "dfl_conv1d")
    return out


def copy_rows(src: torch.Tensor, rows: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
    """``out[r] = src2d[rows[r]]`` (zeros where ``rows[r] < 0``); ``src`` is read as a matrix of its last dimension."""

    lib = load_library()
    _require_cuda_contiguous("src", src)
    _require_cuda_contiguous("rows", rows)
    if rows.dtype != torch.int32:
        raise TypeError("rows must be int32")
    width = src.shape[-1]
    row_bytes = width * src.element_size()
    if out is None:
        out = torch.empty(rows.numel(), width, dtype=src.dtype, device=src.device)
    with _on_device(src.device):
        _check(lib.dfl_copy_rows(src.data_ptr(), out.data_ptr(), rows.data_ptr(), rows.numel(), row_bytes,
                                 _stream(src.device)), "dfl_copy_rows")
    return out


def embed_layernorm(ids: torch.Tensor, table: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor | None,
                    eps: float, *, row_mask: torch.Tensor | None = None, pos_ids: torch.Tensor | None = None,
                    pos_table: torch.Tensor | None = None, status: torch.Tensor | None = None) -> torch.Tensor:
    """``LayerNorm(table[ids] (+ pos_table[pos_ids])) * weight + bias`` with the rows whose ``row_mask`` element is
    zero written as zeros: ``ids`` of any shape (int32 or int64) -> ``ids.shape + [hidden]``.  An id outside its
    table reads as zeros and is reported by ``check_status(status)``."""

    lib = load_library()
    hidden = table.shape[-1]
    for name, t in (("ids", ids), ("table", table), ("weight", weight), ("bias", bias), ("row_mask", row_mask),
                    ("pos_ids", pos_ids), ("pos_table", pos_table)):
        if t is not None:
            _require_cuda_contiguous(name, t)
    if ids.dtype not in (torch.int32, torch.int64):
        raise TypeError("ids must be int32 or int64")
    for name, t in (("weight", weight), ("bias", bias), ("pos_table", pos_table)):
        if t is not None and t.dtype != table.dtype:
            raise TypeError(f"{name} must have the dtype of the table ({table.dtype}), got {t.dtype}")
    if table.dim() != 2 or weight.numel() != hidden or (bias is not None and bias.numel() != hidden):
        raise ValueError("table must be [vocab, hidden] and weight, bias [hidden]")
    if (pos_ids is None) != (pos_table is None):
        raise ValueError("pos_ids and pos_table go together")
    if pos_ids is not None and (pos_ids.dtype != ids.dtype or pos_ids.shape != ids.shape or pos_table.shape[-1] != hidden):
        raise ValueError("pos_ids must have the type and shape of ids, pos_table the width of table")
    if row_mask is not None and row_mask.numel() != ids.numel():
        raise ValueError("row_mask must have one element per id")
    out = torch.empty(*ids.shape, hidden, dtype=table.dtype, device=table.device)
    p = DflEmbedLayerNormParams()
    p.ids, p.table, p.pos_ids, p.pos_table = _ptr(ids), _ptr(table), _ptr(pos_ids), _ptr(pos_table)
    p.gamma, p.beta, p.row_mask, p.out = _ptr(weight), _ptr(bias), _ptr(row_mask), _ptr(out)
    p.rows, p.vocab, p.positions = ids.numel(), table.shape[0], pos_table.shape[0] if pos_table is not None else 0
    p.hidden, p.eps, p.dtype, p.id_elem_size = hidden, float(eps), dtype_code(table.dtype), ids.element_size()
    p.mask_elem_size = row_mask.element_size() if row_mask is not None else 1
    p.status = _ptr(status)
    with _on_device(table.device):
        _check(lib.dfl_embed_layernorm(ctypes.byref(p), _stream(table.device)), "dfl_embed_layernorm")
    return out


def add_layernorm(x: torch.Tensor, residual: torch.Tensor | None, weight: torch.Tensor, bias: torch.Tensor | None,
                  eps: float, out: torch.Tensor | None = None, row_mask: torch.Tensor | None = None,
                  scatter: tuple[torch.Tensor, torch.Tensor] | None = None) -> torch.Tensor:
    """``LayerNorm(x + residual) * weight + bias`` over the last dimension, sum and statistics in fp32; rows whose
    ``row_mask`` element is zero are written as zeros.  ``scatter = (out2, rows)`` also writes row ``r`` of the
    result to row ``rows[r]`` of ``out2`` (skipped where negative)."""

    lib = load_library()
    hidden = x.shape[-1]
    for name, t in (("x", x), ("residual", residual), ("weight", weight), ("bias", bias)):
        if t is None:
            continue
        _require_cuda_contiguous(name, t)
        if t.dtype != x.dtype:
            raise TypeError(f"{name} must have the dtype of x ({x.dtype}), got {t.dtype}")
    if residual is not None and residual.shape != x.shape:
        raise ValueError("residual must have the shape of x")
    if weight.numel() != hidden or (bias is not None and bias.numel() != hidden):
        raise ValueError("weight and bias must have one element per column of x")
    if out is None:
        out = torch.empty_like(x)
    p = DflAddLayerNormParams()
    p.x, p.residual, p.gamma, p.beta, p.out = _ptr(x), _ptr(residual), _ptr(weight), _ptr(bias), _ptr(out)
    p.rows, p.hidden, p.eps, p.dtype = x.numel() // hidden, hidden, float(eps), dtype_code(x.dtype)
    if row_mask is not None:
        _require_cuda_contiguous("row_mask", row_mask)
        if row_mask.numel() != p.rows:
            raise ValueError("row_mask must have one element per row of x")
        p.row_mask, p.mask_elem_size = _ptr(row_mask), row_mask.element_size()
    if scatter is not None:
        out2, out2_rows = scatter
        _require_cuda_contiguous("out2", out2)
        _require_cuda_contiguous("out2_rows", out2_rows)
        if out2.dtype != x.dtype or out2.shape[-1] != hidden or out2_rows.dtype != torch.int32 or out2_rows.numel() != p.rows:
            raise ValueError("scatter = (out2 [*, hidden] in the dtype of x, rows int32 [rows of x])")
        p.out2, p.out2_rows = _ptr(out2), _ptr(out2_rows)
    with _on_device(x.device):
        _check(lib.dfl_add_layernorm(ctypes.byref(p), _stream(x.device)), "dfl_add_layernorm")
    return out


def padded_slots(n_active: int) -> int:
    """Leading dimension of the position-score tensors: rows stay 16-byte aligned."""

    return max(8, (n_active + 7) // 8 * 8)


def pos_scores(q: torch.Tensor | None, k: torch.Tensor | None, pos_key: torch.Tensor | None,
               pos_query: torch.Tensor | None, *, algo: int = ALGO_AUTO, status: torch.Tensor | None = None):
    """C2P / P2C score GEMMs over the active slots; returns ``(c2p, p2c, ld_slots)``."""

    lib = load_library()
    ref = q if q is not None else k
    bsz, heads, length, d = ref.shape
    n_active = (pos_key if pos_key is not None else pos_query).shape[1]
    ld = padded_slots(n_active)
    c2p = torch.empty(bsz, heads, length, ld, dtype=ref.dtype, device=ref.device) if pos_key is not None else None
    p2c = torch.empty(bsz, heads, length, ld, dtype=ref.dtype, device=ref.device) if pos_query is not None else None
    p = DflPosScoreParams()
    p.q, p.k = _ptr(q) if pos_key is not None else None, _ptr(k) if pos_query is not None else None
    p.pos_key, p.pos_query, p.c2p, p.p2c = _ptr(pos_key), _ptr(pos_query), _ptr(c2p), _ptr(p2c)
    p.batch, p.heads, p.seq_len, p.head_dim = bsz, heads, length, d
    p.n_active, p.ld_slots, p.dtype, p.algo = n_active, ld, dtype_code(ref.dtype), algo
    p.status = _ptr(status)
    with _on_device(ref.device):
        _check(lib.dfl_pos_scores(ctypes.byref(p), _stream(ref.device)), "dfl_pos_scores")
    return c2p, p2c, ld


def attention_fwd(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, c2p: torch.Tensor | None,
                  p2c: torch.Tensor | None, lut: torch.Tensor | None, mask: torch.Tensor, scale: float, *,
                  ld_slots: int = 0, algo: int = ALGO_AUTO, status: torch.Tensor | None = None) -> torch.Tensor:
    """Fused attention; ``q,k,v`` are ``[B,H,L,d]``, result is ``[B,L,H*d]``."""

    lib = load_library()
    for name, t in (("q", q), ("k", k), ("v", v), ("mask", mask)):
        _require_cuda_contiguous(name, t)
    bsz, heads, length, d = q.shape
    if mask.element_size() not in (1, 4, 8) or mask.dtype.is_floating_point:
        raise TypeError("mask must be a bool or integer tensor")
    out = torch.empty(bsz, length, heads * d, dtype=q.dtype, device=q.device)
    p = DflAttnParams()
    p.q, p.k, p.v, p.c2p, p.p2c = q.data_ptr(), k.data_ptr(), v.data_ptr(), _ptr(c2p), _ptr(p2c)
    p.lut, p.mask, p.out, p.status = _ptr(lut), mask.data_ptr(), out.data_ptr(), _ptr(status)
    p.batch, p.heads, p.seq_len, p.head_dim = bsz, heads, length, d
    p.ld_slots, p.mask_elem_size, p.scale = ld_slots, mask.element_size(), scale
    p.dtype, p.algo = dtype_code(q.dtype), algo
    with _on_device(q.device):
        _check(lib.dfl_attention_fwd(ctypes.byref(p), _stream(q.device)), "dfl_attention_fwd")
    return out


def _tables_params(q, k, v, pos_key, pos_query, lut, mask, scale, out, algo, status=None) -> DflAttnTablesParams:
    bsz, heads, length, d = q.shape
    if out.shape != (bsz, length, heads * d) or out.dtype != q.dtype:
        raise ValueError("out must be [B, L, H*d] in the dtype of q")
    if mask.element_size() not in (1, 4, 8) or mask.dtype.is_floating_point:
        raise TypeError("mask must be a bool or integer tensor")
    table = pos_key if pos_key is not None else pos_query
    p = DflAttnTablesParams()
    p.q, p.k, p.v, p.pos_key, p.pos_query = q.data_ptr(), k.data_ptr(), v.data_ptr(), _ptr(pos_key), _ptr(pos_query)
    p.lut, p.mask, p.out, p.status = _ptr(lut), mask.data_ptr(), out.data_ptr(), _ptr(status)
    p.batch, p.heads, p.seq_len, p.head_dim = bsz, heads, length, d
    p.n_active = 0 if table is None else table.shape[1]
    p.mask_elem_size, p.scale, p.dtype, p.algo = mask.element_size(), scale, dtype_code(q.dtype), algo
    return p


def attention_fwd_static(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, pos_key: torch.Tensor | None,
                         pos_query: torch.Tensor | None, lut: torch.Tensor | None, mask: torch.Tensor, scale: float,
                         out: torch.Tensor, *, algo: int = ALGO_AUTO) -> torch.Tensor:
    """Score GEMMs + fused attention without any allocation inside the call.

    For callers that cannot allocate device memory where the call is made (a
    server that owns the device through its own arena, a plug-in inside a
    host runtime's callback): the C2P/P2C scores stay in a fixed 32 MiB array
    inside the library instead of caller-allocated buffers, and ``out`` is
    passed in.  Requests that need more raise ``ValueError``.  Calls share the
    array, so calls that overlap on the GPU race; the first call per device
    does one-time set-up and belongs before any stream capture.
    """

    lib = load_library()
    for name, t in (("q", q), ("k", k), ("v", v), ("mask", mask), ("out", out)):
        _require_cuda_contiguous(name, t)
    p = _tables_params(q, k, v, pos_key, pos_query, lut, mask, scale, out, algo)
    with _on_device(q.device):
        _check(lib.dfl_attention_fwd_static(ctypes.byref(p), _stream(q.device)), "dfl_attention_fwd_static")
    return out


def expand_rel_tables(pos: torch.Tensor, lut: torch.Tensor, seq_len: int) -> torch.Tensor:
    """Pruned table ``pos`` [H, A, d] -> ``rel`` [H, 2L-1, d], rel[h, e] = pos[h, lut[2L-2-e]] (prepare-time)."""

    lib = load_library()
    _require_cuda_contiguous("pos", pos)
    _require_cuda_contiguous("lut", lut)
    if lut.dtype != torch.int32 or lut.numel() != 2 * seq_len - 1:
        raise ValueError("lut must be int32 [2L-1]")
    heads, n_active, d = pos.shape
    rel = torch.empty(heads, 2 * seq_len - 1, d, dtype=pos.dtype, device=pos.device)
    with _on_device(pos.device):
        _check(lib.dfl_expand_rel_tables(pos.data_ptr(), lut.data_ptr(), rel.data_ptr(), heads, n_active, seq_len, d,
                                         dtype_code(pos.dtype), _stream(pos.device)), "dfl_expand_rel_tables")
    return rel


def attention_rel_supported(dtype: torch.dtype, seq_len: int, head_dim: int, has_c2p: bool, has_p2c: bool,
                            algo: int = ALGO_AUTO) -> bool:
    """Whether ``attention_rel_fwd`` covers this configuration."""

    if not (has_c2p or has_p2c) or algo != ALGO_AUTO:
        return False
    p = DflAttnRelParams()
    # only nullness of the table pointers is inspected
    p.rel_key, p.rel_query = (1 if has_c2p else None), (1 if has_p2c else None)
    p.batch, p.heads, p.seq_len, p.head_dim = 1, 1, seq_len, head_dim
    p.dtype, p.algo = dtype_code(dtype), algo
    return bool(load_library().dfl_attention_rel_supported(ctypes.byref(p)))


def attention_rel_fwd(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, rel_key: torch.Tensor | None,
                      rel_query: torch.Tensor | None, mask: torch.Tensor, scale: float, *,
                      status: torch.Tensor | None = None, packed_rows: tuple[torch.Tensor, torch.Tensor, int] | None = None
                      ) -> torch.Tensor:
    """Fused attention over position tables laid out by relative distance ([H, 2L-1, d]).

    ``packed_rows = (row_base int32[B], row_count int32[B], total_rows)`` selects the packed output ``[T, H*d]``:
    sequence ``b`` owns rows ``row_base[b] .. + row_count[b]``."""

    lib = load_library()
    for name, t in (("q", q), ("k", k), ("v", v), ("mask", mask)):
        _require_cuda_contiguous(name, t)
    bsz, heads, length, d = q.shape
    for name, t in (("rel_key", rel_key), ("rel_query", rel_query)):
        if t is not None:
            _require_cuda_contiguous(name, t)
            if t.shape != (heads, 2 * length - 1, d) or t.dtype != q.dtype:
                raise ValueError(f"{name} must be [H, 2L-1, d] in the dtype of q")
    if mask.element_size() not in (1, 4, 8) or mask.dtype.is_floating_point:
        raise TypeError("mask must be a bool or integer tensor")
    p = DflAttnRelParams()
    if packed_rows is None:
        out = torch.empty(bsz, length, heads * d, dtype=q.dtype, device=q.device)
    else:
        row_base, row_count, total_rows = packed_rows
        for name, t in (("row_base", row_base), ("row_count", row_count)):
            _require_cuda_contiguous(name, t)
            if t.dtype != torch.int32 or t.numel() != bsz:
                raise ValueError(f"{name} must be int32 [B]")
        out = torch.empty(total_rows, heads * d, dtype=q.dtype, device=q.device)
        p.out_row_base, p.out_row_count = row_base.data_ptr(), row_count.data_ptr()
    p.q, p.k, p.v, p.rel_key, p.rel_query = q.data_ptr(), k.data_ptr(), v.data_ptr(), _ptr(rel_key), _ptr(rel_query)
    p.mask, p.out, p.status = mask.data_ptr(), out.data_ptr(), _ptr(status)
    p.batch, p.heads, p.seq_len, p.head_dim = bsz, heads, length, d
    p.mask_elem_size, p.scale, p.dtype, p.algo = mask.element_size(), scale, dtype_code(q.dtype), ALGO_AUTO
    with _on_device(q.device):
        _check(lib.dfl_attention_rel_fwd(ctypes.byref(p), _stream(q.device)), "dfl_attention_rel_fwd")
    return out
