"""Python entry points of the CUDA kernels: tensors in, launches on the current stream.

Each function checks shapes, dtypes and devices, then calls the ``extern "C"`` launcher
with raw pointers.  Nothing here has a CPU or library fallback: a tensor that is not on a
CUDA device, or an extension that cannot be built, raises.
"""

from __future__ import annotations

import ctypes
from ctypes import c_float, c_int, c_longlong, c_void_p

import torch

from .build import attention_library, load_library

F32, BF16 = 0, 1

# Launch every kernel of this library as a programmatic dependent of the stream's previous
# kernel: it may then start while that kernel drains, and waits inside for its results.  The
# engine switches it on for its steps; direct callers get ordinary launches.
PDL = False

FAULT_BITS = {
    1: "a token id outside the vocabulary",
    2: "a page id outside the cache pool",
    4: "a position outside the rotary table or block table",
    8: "a slot outside the block table",
    16: "a bounded wait inside a kernel ran out",
}


class KernelError(RuntimeError):
    """A launch was refused (bad size or argument) or failed."""


def dtype_tag(dtype: torch.dtype) -> int:
    if dtype == torch.float32:
        return F32
    if dtype == torch.bfloat16:
        return BF16
    raise KernelError(f"kernels take float32 or bfloat16 tensors, got {dtype}")


def _ptr(tensor: torch.Tensor | None) -> int | None:
    """The address as ctypes takes it for a ``c_void_p`` parameter (a plain integer, ``None`` for null): every
    launcher's signature is declared, so no wrapper object is needed, and a step passes thousands of these."""
    return None if tensor is None else tensor.data_ptr()


# Called before every launch of this module: whoever has queued work that the launch may depend on
# (``ops.gemm`` queues the products of a small step for one persistent kernel) runs it first.
BEFORE_LAUNCH = None


def _stream() -> int:
    """The current stream of the current device as a raw handle (asked of torch's C layer directly: the Stream
    object of ``torch.cuda.current_stream()`` costs several microseconds, and every launch asks)."""
    if BEFORE_LAUNCH is not None:
        BEFORE_LAUNCH()
    return _raw_stream(torch.cuda.current_device())


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None) or (lambda device: torch.cuda.current_stream(device).cuda_stream)


def _need_cuda(*tensors: torch.Tensor | None) -> None:
    for tensor in tensors:
        if tensor is not None and not tensor.is_cuda:
            raise KernelError(
                "kernel arguments must live on a CUDA device; there is no CPU path "
                f"(got a tensor on {tensor.device})"
            )


def _contig(name: str, tensor: torch.Tensor | None) -> None:
    if tensor is not None and not tensor.is_contiguous():
        raise KernelError(f"{name} must be contiguous")


def _expect(name: str, tensor: torch.Tensor | None, dtype: torch.dtype) -> None:
    if tensor is not None and tensor.dtype != dtype:
        raise KernelError(f"{name} must be {dtype}, got {tensor.dtype}")


_CUDA_ERRORS = {1: "invalid value (a size or argument the kernel refuses)"}


class LaunchCounter:
    """Counts launches of this library's kernels (library products are not counted).

    A captured graph's launches are added by whoever replays it (``add``)."""

    def __init__(self) -> None:
        self.count = 0

    def add(self, launches: int) -> None:
        self.count += launches


LAUNCHES = LaunchCounter()


def _check(code: int, what: str) -> None:
    LAUNCHES.count += 1
    if code != 0:
        detail = _CUDA_ERRORS.get(code, f"CUDA error {code}")
        raise KernelError(f"{what}: {detail}")


_SIGNATURES_SET = False


def core() -> ctypes.CDLL:
    """The core kernel library, with argument types declared once."""
    global _SIGNATURES_SET
    lib = load_library("core")
    if not _SIGNATURES_SET:
        lib.rl_embedding.argtypes = [c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_float, c_void_p, c_int, c_void_p]
        lib.rl_add_rmsnorm.argtypes = [c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_float, c_int, c_int, c_void_p, c_void_p, c_int, c_void_p]
        lib.rl_layernorm.argtypes = [c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int,
                                     c_float, c_float, c_int, c_float, c_int, c_void_p]
        lib.rl_row_norm_rope_write.argtypes = [
            c_int, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int,
            c_int, c_int, c_int, c_int, c_int, c_float, c_int, c_int, c_void_p, c_int, c_void_p,
        ]
        lib.rl_sigmoid_gate.argtypes = [c_int, c_void_p, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_void_p]
        lib.rl_silu_mul.argtypes = [c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p]
        lib.rl_clamped_glu.argtypes = [c_int, c_void_p, c_void_p, c_int, c_int, c_float, c_float, c_int, c_void_p]
        lib.rl_rope_unit_write.argtypes = [
            c_int, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p,
            c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_int, c_int, c_void_p, c_int, c_void_p,
        ]
        lib.rl_scatter_rows.argtypes = [c_void_p, c_int, c_int, c_void_p, c_void_p, c_int, c_void_p, c_void_p]
        lib.rl_to_float.argtypes = [c_int, c_void_p, c_void_p, c_longlong, c_int, c_void_p]
        lib.rl_qk_norm_rope_write.argtypes = [
            c_int, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
            c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int,
            c_float, c_int, c_void_p, c_int, c_void_p,
        ]
        lib.rl_attention_generic.argtypes = [
            c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int,
            c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_float, c_void_p, c_int, c_void_p, c_void_p,
        ]
        lib.rl_embedding_sum.argtypes = [
            c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p,
            c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int, c_int, c_longlong, c_longlong, c_int, c_void_p, c_void_p,
        ]
        lib.rl_gemm_f32.argtypes = [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p]
        lib.rl_sample.argtypes = [
            c_int, c_void_p, c_int, c_int, c_longlong, c_void_p, c_void_p, c_void_p, c_void_p,
            c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p,
        ]
        for name in (
            "rl_embedding", "rl_embedding_sum", "rl_scatter_rows", "rl_add_rmsnorm", "rl_silu_mul", "rl_to_float", "rl_clamped_glu",
            "rl_rope_unit_write", "rl_layernorm", "rl_row_norm_rope_write", "rl_sigmoid_gate",
            "rl_qk_norm_rope_write", "rl_attention_generic", "rl_gemm_f32", "rl_sample",
        ):
            getattr(lib, name).restype = c_int
        _SIGNATURES_SET = True
    return lib


# --------------------------------------------------------------------------- ops
def embedding(out: torch.Tensor, table: torch.Tensor, ids: torch.Tensor, fault: torch.Tensor,
              feedback: torch.Tensor | None = None, scale: float = 1.0, stream: torch.Tensor | None = None) -> torch.Tensor:
    """``out[t] = table[ids[t]] * scale``; ``ids`` int32 ``[T]``; bad ids set the fault word.

    With ``feedback`` (int32, on the device) an id ``-(r + 1)`` is replaced by ``feedback[r]``.  ``stream``
    (float32 ``[T, H]``) also receives the rows, as the float32 products before ``out``'s rounding."""
    _need_cuda(out, table, ids, fault, feedback, stream)
    _expect("stream", stream, torch.float32), _contig("stream", stream)
    if stream is not None and stream.shape != out.shape:
        raise KernelError("embedding: stream must have the shape of out")
    _expect("ids", ids, torch.int32), _expect("feedback", feedback, torch.int32)
    _contig("out", out), _contig("table", table), _contig("ids", ids)
    if out.dtype != table.dtype or out.shape != (ids.numel(), table.shape[1]):
        raise KernelError(f"embedding: out {tuple(out.shape)} {out.dtype} does not fit table {tuple(table.shape)} {table.dtype}")
    _check(
        core().rl_embedding(dtype_tag(table.dtype), _ptr(out), _ptr(table), _ptr(ids), _ptr(feedback),
                            0 if feedback is None else feedback.numel(), ids.numel(),
                            table.shape[1], table.shape[0], _ptr(fault), float(scale), _ptr(stream), 0, _stream()),   # first kernel of a step: an ordinary launch
        "embedding",
    )
    return out


def embedding_sum(out: torch.Tensor, stream: torch.Tensor | None, table: torch.Tensor, pair_table: torch.Tensor,
                  position_table: torch.Tensor, batch, last_token: torch.Tensor, *, mul_prev: int, mul_cur: int) -> torch.Tensor:
    """``out[t] = table[id_t] + pair_table[(id_(t-1) * mul_prev + id_t * mul_cur) mod buckets] + position_table[p_t]``
    as a float32 sum (also stored to ``stream`` if given); ``pair_table`` has ``buckets + 1`` rows and a request's first
    token takes the last.  The id before an entry's first row is the one its slot keeps in ``last_token``
    (int32 ``[slots, 1]``), brought up to date here."""
    _need_cuda(out, stream, table, pair_table, position_table, last_token)
    _expect("stream", stream, torch.float32), _expect("last_token", last_token, torch.int32)
    for name, tensor in (("out", out), ("stream", stream), ("table", table), ("pair_table", pair_table),
                         ("position_table", position_table), ("last_token", last_token)):
        _contig(name, tensor)
    rows, hidden = out.shape
    if (table.dtype != out.dtype or pair_table.dtype != out.dtype or position_table.dtype != out.dtype
            or table.shape[1] != hidden or pair_table.shape[1] != hidden or position_table.shape[1] != hidden
            or rows != batch.token_ids.numel() or (stream is not None and stream.shape != out.shape)
            or last_token.numel() != last_token.shape[0] or pair_table.shape[0] < 2):
        raise KernelError("embedding_sum: shapes or dtypes do not agree")
    feedback = batch.feedback
    _check(core().rl_embedding_sum(
        dtype_tag(out.dtype), _ptr(out), _ptr(stream), _ptr(table), _ptr(pair_table), _ptr(position_table),
        _ptr(batch.token_ids), _ptr(feedback), 0 if feedback is None else feedback.numel(), _ptr(batch.positions),
        _ptr(batch.cu_seqlens), _ptr(batch.entry_slot), batch.num_entries, _ptr(last_token), last_token.shape[0], rows,
        hidden, table.shape[0], pair_table.shape[0] - 1, int(mul_prev), int(mul_cur), position_table.shape[0],
        _ptr(batch.fault), _stream()), "embedding_sum")
    return out


def scatter_rows(table: torch.Tensor, slots: torch.Tensor, rows: torch.Tensor, fault: torch.Tensor) -> torch.Tensor:
    """``table[slots[i]] = rows[i]`` for int32 tables; a slot outside the table sets the fault word."""
    _need_cuda(table, slots, rows, fault)
    for name, tensor in (("table", table), ("slots", slots), ("rows", rows)):
        _expect(name, tensor, torch.int32), _contig(name, tensor)
    if table.dim() != 2 or rows.numel() != slots.numel() * table.shape[1]:
        raise KernelError("scatter_rows: rows must hold one table row per slot")
    _check(
        core().rl_scatter_rows(_ptr(table), table.shape[1], table.shape[0], _ptr(slots), _ptr(rows), slots.numel(),
                               _ptr(fault), _stream()),
        "scatter_rows",
    )
    return table


def add_rmsnorm(
    x: torch.Tensor,
    residual: torch.Tensor | None,
    weight: torch.Tensor,
    out: torch.Tensor,
    eps: float,
    *,
    mode: int,
    write_residual: bool,
    row_index: torch.Tensor | None = None,
    extra_rows: torch.Tensor | None = None,
    extra_vector: torch.Tensor | None = None,
) -> torch.Tensor:
    """RMSNorm of ``x`` (mode 0 or 2) or of ``x + residual`` (mode 1), float32 math.

    ``residual`` is the float32 residual stream ``[T, H]``; with ``write_residual`` the
    sum is stored back into it.  ``row_index`` (int32) selects the input rows; ``out`` then
    has one row per index.  ``extra_rows`` (``[T, H]`` of x's dtype) and ``extra_vector``
    (float32 ``[H]``) are added to the sum, in that order, before it is stored or normed.
    """
    _need_cuda(x, residual, weight, out, row_index, extra_rows, extra_vector)
    _contig("extra_rows", extra_rows), _contig("extra_vector", extra_vector)
    _expect("extra_vector", extra_vector, torch.float32)
    if extra_rows is not None and (extra_rows.shape != x.shape or extra_rows.dtype != x.dtype):
        raise KernelError("add_rmsnorm: extra_rows must have the shape and dtype of x")
    if extra_vector is not None and extra_vector.numel() != x.shape[-1]:
        raise KernelError("add_rmsnorm: extra_vector must have one entry per column")
    _expect("weight", weight, torch.float32), _expect("residual", residual, torch.float32)
    _expect("row_index", row_index, torch.int32)
    _contig("x", x), _contig("residual", residual), _contig("out", out)
    hidden = x.shape[-1]
    rows = row_index.numel() if row_index is not None else x.shape[0]
    if weight.numel() != hidden or out.shape != (rows, hidden) or out.dtype != x.dtype:
        raise KernelError("add_rmsnorm: shapes of x, weight and out do not agree")
    if residual is not None and residual.shape != x.shape:
        raise KernelError("add_rmsnorm: residual must have the shape of x")
    _check(
        core().rl_add_rmsnorm(dtype_tag(x.dtype), _ptr(x), _ptr(residual), _ptr(weight), _ptr(out),
                              _ptr(row_index), rows, hidden, float(eps), mode, int(write_residual),
                              _ptr(extra_rows), _ptr(extra_vector), int(PDL), _stream()),
        f"add_rmsnorm(hidden={hidden})",
    )
    return out


def stream_rmsnorm(residual: torch.Tensor, weight: torch.Tensor, out: torch.Tensor, eps: float,
                   row_index: torch.Tensor | None = None) -> torch.Tensor:
    """RMSNorm of the float32 stream itself (rows picked by ``row_index``), into ``out`` of the engine's dtype."""
    _need_cuda(residual, weight, out, row_index)
    _expect("weight", weight, torch.float32), _expect("residual", residual, torch.float32)
    _expect("row_index", row_index, torch.int32), _contig("residual", residual), _contig("out", out)
    hidden = residual.shape[-1]
    rows = row_index.numel() if row_index is not None else residual.shape[0]
    if weight.numel() != hidden or out.shape != (rows, hidden):
        raise KernelError("stream_rmsnorm: shapes of residual, weight and out do not agree")
    _check(core().rl_add_rmsnorm(dtype_tag(out.dtype), None, _ptr(residual), _ptr(weight), _ptr(out), _ptr(row_index),
                                 rows, hidden, float(eps), 3, 0, None, None, int(PDL), _stream()), "stream_rmsnorm")
    return out


def join_rmsnorm(x: torch.Tensor, residual: torch.Tensor, weight: torch.Tensor, out: torch.Tensor, eps: float) -> torch.Tensor:
    """A norm on a sublayer's output: ``residual += x * rsqrt(mean(x^2) + eps) * weight`` (float32, in place) and
    ``out`` = the new residual in the engine's dtype."""
    _need_cuda(x, residual, weight, out)
    _expect("weight", weight, torch.float32), _expect("residual", residual, torch.float32)
    _contig("x", x), _contig("residual", residual), _contig("out", out)
    if residual.shape != x.shape or out.shape != x.shape or out.dtype != x.dtype or weight.numel() != x.shape[-1]:
        raise KernelError("join_rmsnorm: shapes of x, residual, weight and out do not agree")
    _check(core().rl_add_rmsnorm(dtype_tag(x.dtype), _ptr(x), _ptr(residual), _ptr(weight), _ptr(out), None,
                                 x.shape[0], x.shape[1], float(eps), 4, 1, None, None, int(PDL), _stream()), "join_rmsnorm")
    return out


LAYERNORM_KEEP, LAYERNORM_STORE_SUM, LAYERNORM_STORE_NORM = 0, 1, 2


def layernorm(x: torch.Tensor | None, residual: torch.Tensor | None, weight: torch.Tensor, bias: torch.Tensor | None,
              out: torch.Tensor, eps: float, *, residual_scale: float = 1.0, store: int = LAYERNORM_KEEP,
              row_index: torch.Tensor | None = None, gain: float = 1.0) -> torch.Tensor:
    """Layer norm with a mean: with ``r = x + residual_scale * residual`` (either may be ``None``; ``residual`` is the
    float32 stream), ``n = (r - mean r) * rsqrt(var r + eps) * weight + bias``, the variance being the mean of the
    squared deviations, float32 throughout; ``out = n * gain`` in the engine's dtype.  ``store``:
    :data:`LAYERNORM_STORE_SUM` writes ``r`` back into ``residual``, :data:`LAYERNORM_STORE_NORM` writes ``n`` there
    (a norm behind the sum, whose result is the stream's new value).  ``row_index`` (int32) picks the input rows."""
    _need_cuda(x, residual, weight, bias, out, row_index)
    _expect("weight", weight, torch.float32), _expect("bias", bias, torch.float32), _expect("residual", residual, torch.float32)
    _expect("row_index", row_index, torch.int32)
    _contig("x", x), _contig("residual", residual), _contig("out", out), _contig("weight", weight), _contig("bias", bias)
    source = x if x is not None else residual
    if source is None:
        raise KernelError("layernorm: there is nothing to norm")
    hidden = source.shape[-1]
    rows = row_index.numel() if row_index is not None else source.shape[0]
    if (weight.numel() != hidden or (bias is not None and bias.numel() != hidden) or out.shape != (rows, hidden)
            or (x is not None and (x.dtype != out.dtype or (residual is not None and residual.shape != x.shape)))):
        raise KernelError("layernorm: shapes or dtypes of x, residual, weight, bias and out do not agree")
    if store != LAYERNORM_KEEP and (residual is None or row_index is not None):
        raise KernelError("layernorm: storing needs the stream, and every row of it")
    _check(core().rl_layernorm(dtype_tag(out.dtype), _ptr(x), _ptr(residual), _ptr(weight), _ptr(bias), _ptr(out),
                               _ptr(row_index), rows, hidden, float(eps), float(residual_scale), int(store), float(gain),
                               int(PDL), _stream()), f"layernorm(hidden={hidden})")
    return out


def row_norm_rope_write(qkv: torch.Tensor, q_out: torch.Tensor, *, num_heads: int, num_kv_heads: int, head_dim: int,
                        q_weight: torch.Tensor, k_weight: torch.Tensor | None, q_count: int, k_count: int,
                        inv_freq: torch.Tensor | None, positions: torch.Tensor, eps: float, fault: torch.Tensor,
                        kv_dest: torch.Tensor | None = None, cache: torch.Tensor | None = None,
                        page_size: int = 1) -> torch.Tensor:
    """RMS norm of q over ALL its heads at once (and of k likewise), ``q * rsqrt(sum(q^2) / q_count + eps) * q_weight``
    with one weight per laid-out entry, then rotation by halves of the first ``2 len(inv_freq)`` entries of every q and
    k head (angles ``position * inv_freq`` formed in float32), q to ``q_out``, k and v into the pages.  ``qkv`` is
    ``[T, (Hq + 2 Hkv) D]``, or ``[T, Hq D]`` with ``kv_dest`` ``None`` (queries only)."""
    _need_cuda(qkv, q_out, q_weight, k_weight, inv_freq, positions, fault, kv_dest, cache)
    _contig("qkv", qkv), _contig("q_out", q_out), _contig("cache", cache), _contig("inv_freq", inv_freq)
    for name, tensor in (("q_weight", q_weight), ("k_weight", k_weight), ("inv_freq", inv_freq)):
        _expect(name, tensor, torch.float32), _contig(name, tensor)
    _expect("positions", positions, torch.int32), _expect("kv_dest", kv_dest, torch.int32)
    tokens, row_width = qkv.shape
    heads_in = num_heads + 2 * num_kv_heads if kv_dest is not None else num_heads
    if row_width < heads_in * head_dim or q_out.numel() != tokens * num_heads * head_dim or q_out.dtype != qkv.dtype:
        raise KernelError("row_norm_rope_write: qkv or q_out do not fit the heads")      # columns behind the heads are not read
    if q_weight.numel() != num_heads * head_dim or (kv_dest is not None and (k_weight is None or k_weight.numel() != num_kv_heads * head_dim)):
        raise KernelError("row_norm_rope_write: one norm weight per laid-out entry of q (and of k)")
    num_pages = 0
    if kv_dest is not None:
        if cache is None or cache.dtype != qkv.dtype or cache.shape[1:] != (2, num_kv_heads, page_size, head_dim):
            raise KernelError("row_norm_rope_write: cache must be [pages, 2, kv_heads, page_size, head_dim] of qkv's dtype")
        num_pages = cache.shape[0]
    rotary = 0 if inv_freq is None else 2 * inv_freq.numel()
    _check(core().rl_row_norm_rope_write(
        dtype_tag(qkv.dtype), _ptr(qkv), row_width, _ptr(q_weight), _ptr(k_weight), _ptr(inv_freq), _ptr(positions),
        _ptr(kv_dest), _ptr(q_out), _ptr(cache), tokens, num_heads, num_kv_heads, head_dim, rotary, int(q_count),
        int(k_count), float(eps), page_size, num_pages, _ptr(fault), int(PDL), _stream()),
        f"row_norm_rope_write(head_dim={head_dim})")
    return q_out


def sigmoid_gate(rows: torch.Tensor, gate: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """``out = rows * sigmoid(gate)`` entry by entry (float32 arithmetic); ``gate`` may be a view of some columns of
    wider rows."""
    _need_cuda(rows, gate, out)
    _contig("rows", rows), _contig("out", out)
    if gate.shape != rows.shape or out.shape != rows.shape or gate.dtype != rows.dtype or out.dtype != rows.dtype:
        raise KernelError("sigmoid_gate: shapes or dtypes do not agree")
    _check(core().rl_sigmoid_gate(dtype_tag(rows.dtype), _ptr(rows), _ptr(gate), _row_stride("gate", gate), _ptr(out),
                                  rows.shape[0], rows.shape[1], int(PDL), _stream()), "sigmoid_gate")
    return out


def clamped_glu(gate_up: torch.Tensor, out: torch.Tensor, limit: float, alpha: float) -> torch.Tensor:
    """``out = g * sigmoid(alpha g) * (u + 1)`` with ``g = min(gate_up[:, :I], limit)``, ``u = clamp(gate_up[:, I:], +-limit)``."""
    _need_cuda(gate_up, out)
    _contig("gate_up", gate_up), _contig("out", out)
    rows, width = gate_up.shape
    if width % 2 or out.shape != (rows, width // 2) or out.dtype != gate_up.dtype:
        raise KernelError("clamped_glu: out must be [rows, width / 2] of the input's dtype")
    _check(core().rl_clamped_glu(dtype_tag(gate_up.dtype), _ptr(gate_up), _ptr(out), rows, width // 2, float(limit),
                                 float(alpha), int(PDL), _stream()), "clamped_glu")
    return out


def rope_unit_write(rows: torch.Tensor, q_out: torch.Tensor, *, num_heads: int, num_kv_heads: int, head_dim: int,
                    inv_freq: torch.Tensor | None, positions: torch.Tensor, kv_dest: torch.Tensor, cache: torch.Tensor,
                    page_size: int, norm_size: int, unit: bool, eps: float, fault: torch.Tensor,
                    first: torch.Tensor | None = None, first_mode: int = 0, mix: torch.Tensor | None = None) -> torch.Tensor:
    """From float32 ``rows [T, (Hq + 2 Hkv) D]`` (a convolution's results): the first ``2 len(inv_freq)`` entries of
    every q and k head rotate by position, the heads are then divided by their root mean square over the first
    ``norm_size`` entries (``unit``), q goes to ``q_out`` and k, v into the pages.  ``first`` (float32
    ``[T, Hkv D]``): with ``first_mode`` 1 the values are left there, with 2 they are blended with what lies
    there, ``v <- (1 - mix) v + mix first`` (``mix``: one float32 on the device), before they are cached."""
    _need_cuda(rows, q_out, inv_freq, positions, kv_dest, cache, fault, first, mix)
    _expect("rows", rows, torch.float32), _expect("inv_freq", inv_freq, torch.float32), _expect("first", first, torch.float32)
    _expect("mix", mix, torch.float32), _expect("positions", positions, torch.int32), _expect("kv_dest", kv_dest, torch.int32)
    _contig("rows", rows), _contig("q_out", q_out), _contig("cache", cache), _contig("first", first)
    tokens = rows.shape[0]
    if rows.shape[1] != (num_heads + 2 * num_kv_heads) * head_dim or q_out.numel() != tokens * num_heads * head_dim:
        raise KernelError("rope_unit_write: rows or q_out do not fit the heads")
    if cache.dtype != q_out.dtype or cache.shape[1:] != (2, num_kv_heads, page_size, head_dim):
        raise KernelError("rope_unit_write: cache must be [pages, 2, kv_heads, page_size, head_dim] of q_out's dtype")
    if first is not None and first.shape != (tokens, num_kv_heads * head_dim):
        raise KernelError("rope_unit_write: first must be [tokens, kv_heads * head_dim]")
    rotary = 0 if inv_freq is None else 2 * inv_freq.numel()
    _check(core().rl_rope_unit_write(
        dtype_tag(q_out.dtype), _ptr(rows), rows.stride(0), _ptr(inv_freq), _ptr(positions), _ptr(kv_dest), _ptr(mix),
        _ptr(first), int(first_mode), _ptr(q_out), _ptr(cache), tokens, num_heads, num_kv_heads, head_dim, rotary,
        int(norm_size), int(unit), float(eps), page_size, cache.shape[0], _ptr(fault), int(PDL), _stream()),
        f"rope_unit_write(head_dim={head_dim})")
    return q_out


def silu_mul(gate_up: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """``out = silu(gate_up[:, :I]) * gate_up[:, I:]``."""
    _need_cuda(gate_up, out)
    _contig("gate_up", gate_up), _contig("out", out)
    rows, width = gate_up.shape
    if width % 2 or out.shape != (rows, width // 2) or out.dtype != gate_up.dtype:
        raise KernelError("silu_mul: out must be [rows, width / 2] of the input's dtype")
    _check(core().rl_silu_mul(dtype_tag(gate_up.dtype), _ptr(gate_up), _ptr(out), rows, width // 2, int(PDL), _stream()), "silu_mul")
    return out


def to_float(src: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    _need_cuda(src, out)
    _contig("src", src), _contig("out", out)
    _expect("out", out, torch.float32)
    if out.numel() != src.numel():
        raise KernelError("to_float: sizes differ")
    _check(core().rl_to_float(dtype_tag(src.dtype), _ptr(src), _ptr(out), src.numel(), int(PDL), _stream()), "to_float")
    return out


def qk_norm_rope_write(
    qkv: torch.Tensor,
    q_out: torch.Tensor,
    *,
    num_heads: int,
    num_kv_heads: int,
    head_dim: int,
    rotary_dim: int,
    cos: torch.Tensor,
    sin: torch.Tensor,
    positions: torch.Tensor,
    eps: float,
    fault: torch.Tensor,
    q_weight: torch.Tensor | None = None,
    k_weight: torch.Tensor | None = None,
    bias: torch.Tensor | None = None,
    kv_dest: torch.Tensor | None = None,
    cache: torch.Tensor | None = None,
    page_size: int = 1,
    norm_size: int | None = None,
) -> torch.Tensor:
    """Per-head q/k RMSNorm, rotation by position, q to ``q_out``, k and v into the pages.

    ``norm_size``: entries of a head the norm's mean is taken over, when the head's tail is padding.

    ``qkv`` is ``[T, (Hq + 2 Hkv) D]`` (or ``[T, Hq D]`` when ``kv_dest`` is ``None`` and
    only queries are produced).  ``cache`` is one layer's ``[pages, 2, Hkv, page, D]``;
    ``kv_dest[t] = page * page_size + offset``.
    """
    _need_cuda(qkv, q_out, cos, sin, positions, fault, q_weight, k_weight, bias, kv_dest, cache)
    _contig("qkv", qkv), _contig("q_out", q_out), _contig("cache", cache)
    _contig("cos", cos), _contig("sin", sin)
    for name, tensor in (("cos", cos), ("sin", sin), ("q_weight", q_weight), ("k_weight", k_weight), ("bias", bias)):
        _expect(name, tensor, torch.float32)
    _expect("positions", positions, torch.int32), _expect("kv_dest", kv_dest, torch.int32)
    tokens, row_width = qkv.shape
    heads_in = num_heads + 2 * num_kv_heads if kv_dest is not None else num_heads
    if row_width != heads_in * head_dim:
        raise KernelError(f"qk_norm_rope_write: qkv width {row_width} is not {heads_in} heads of {head_dim}")
    if q_out.numel() != tokens * num_heads * head_dim or q_out.dtype != qkv.dtype:
        raise KernelError("qk_norm_rope_write: q_out does not fit")
    if cos.shape != sin.shape or cos.dim() != 2 or cos.shape[1] * 2 != rotary_dim:
        raise KernelError("qk_norm_rope_write: cos/sin must be [positions, rotary_dim / 2]")
    num_pages = 0
    if kv_dest is not None:
        if cache is None or cache.dtype != qkv.dtype or cache.shape[1:] != (2, num_kv_heads, page_size, head_dim):
            raise KernelError("qk_norm_rope_write: cache must be [pages, 2, kv_heads, page_size, head_dim] of qkv's dtype")
        num_pages = cache.shape[0]
    _check(
        core().rl_qk_norm_rope_write(
            dtype_tag(qkv.dtype), _ptr(qkv), row_width, _ptr(bias), _ptr(q_weight), _ptr(k_weight),
            _ptr(cos), _ptr(sin), _ptr(positions), _ptr(kv_dest), _ptr(q_out), _ptr(cache), tokens,
            num_heads, num_kv_heads, head_dim, rotary_dim, cos.shape[0], page_size, num_pages,
            float(eps), int(norm_size or 0), _ptr(fault), int(PDL), _stream(),
        ),
        f"qk_norm_rope_write(head_dim={head_dim})",
    )
    return q_out


def attention_generic(
    q: torch.Tensor,
    cache: torch.Tensor,
    out: torch.Tensor,
    *,
    positions: torch.Tensor,
    token_slot: torch.Tensor,
    block_table: torch.Tensor,
    num_heads: int,
    num_kv_heads: int,
    head_dim: int,
    window: int,
    scale: float,
    fault: torch.Tensor,
    softcap: float = 0.0,
    sink: torch.Tensor | None = None,
) -> torch.Tensor:
    """Causal attention of every token of the step over its request's cached keys.  ``softcap`` > 0 squashes the
    scaled scores to ``softcap * tanh(s / softcap)``; ``sink`` (float32 ``[heads]``) adds ``exp(sink[h])`` to every
    row's denominator."""
    _need_cuda(q, cache, out, positions, token_slot, block_table, fault, sink)
    _expect("sink", sink, torch.float32), _contig("sink", sink)
    if sink is not None and sink.numel() != num_heads:
        raise KernelError("attention: one sink per head")
    _contig("q", q), _contig("cache", cache), _contig("out", out), _contig("block_table", block_table)
    for name, tensor in (("positions", positions), ("token_slot", token_slot), ("block_table", block_table)):
        _expect(name, tensor, torch.int32)
    tokens = positions.numel()
    if q.numel() != tokens * num_heads * head_dim or out.numel() != q.numel():
        raise KernelError("attention: q/out do not hold [tokens, heads, head_dim]")
    if cache.dtype != q.dtype or out.dtype != q.dtype:
        raise KernelError("attention: q, cache and out must share a dtype")
    if cache.dim() != 5 or cache.shape[1] not in (1, 2) or cache.shape[2] != num_kv_heads or cache.shape[4] != head_dim:
        raise KernelError("attention: cache must be [pages, 2 (or 1: values are the keys' rows), kv_heads, page_size, head_dim]")
    if head_dim % 16 or head_dim > 640:
        raise KernelError(f"attention: head_dim {head_dim} must be a multiple of 16 up to 640")
    _check(
        core().rl_attention_generic(
            dtype_tag(q.dtype), _ptr(q), _ptr(cache), _ptr(out), _ptr(positions), _ptr(token_slot),
            _ptr(block_table), tokens, num_heads, num_kv_heads, head_dim, cache.shape[3],
            cache.shape[0], block_table.shape[1], block_table.shape[0], int(window), float(scale),
            float(softcap), _ptr(sink), int(cache.shape[1]), _ptr(fault), _stream(),
        ),
        f"attention_generic(head_dim={head_dim})",
    )
    return out


_ATTENTION_LIBS: dict[int, ctypes.CDLL] = {}

CHUNK_TILE_ROWS = 64       # packed rows (token, head of the group) of a chunk tile of the mma.sync kernel
CHUNK_TILE_ROWS_TC = 256   # ... of the tcgen05 kernel (head size 128, unsplit key ranges)
DECODE_TILE_ROWS = 16      # ... of a decode tile
TC_HEAD_DIM = 128
DECODE_TC_KEYS = 128      # keys per block of the tcgen05 decode kernel


def attention_tc_takes(head_dim: int, page_size: int) -> bool:
    """Whether the tcgen05 attention kernels take this head size and page size."""
    if head_dim != TC_HEAD_DIM or page_size <= 0 or page_size % 8:
        return False
    return 128 % page_size == 0 or page_size % 128 == 0


def attention_lib(head_dim: int) -> ctypes.CDLL:
    """The tensor-core attention library of one head size, built at its first use."""
    lib = _ATTENTION_LIBS.get(head_dim)
    if lib is None:
        lib = load_library(attention_library(head_dim))
        lib.rl_attention_mma.argtypes = [
            c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int,
            c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int,
            c_int, c_int, c_int, c_int, c_float, c_void_p, c_int, c_int, c_int, c_int, c_int, c_float, c_void_p, c_int, c_void_p,
        ]
        lib.rl_attention_mma.restype = c_int
        lib.rl_attention_decode_max_clusters.argtypes = [c_int]
        lib.rl_attention_decode_max_clusters.restype = c_int
        if lib.rl_attention_head_dim() != head_dim:
            raise KernelError(f"the attention library for head size {head_dim} was built for another size")
        if lib.rl_attention_chunk_rows() != CHUNK_TILE_ROWS or lib.rl_attention_decode_rows() != DECODE_TILE_ROWS:
            raise KernelError("the attention library's tile sizes differ from the host's")
        if lib.rl_attention_chunk_rows_tc() != (CHUNK_TILE_ROWS_TC if head_dim == TC_HEAD_DIM else 0):
            raise KernelError("the attention library's tensor-core tile size differs from the host's")
        _ATTENTION_LIBS[head_dim] = lib
    return lib


def attention_decode_clusters(head_dim: int, device: torch.device) -> dict[int, int]:
    """``{cluster size: clusters of the tcgen05 decode kernel the GPU runs at one time}`` for the sizes it can
    launch (a cluster lives inside one GPC, so this is not the number of multiprocessors over the size).
    Empty where that kernel does not exist (other head sizes)."""
    if head_dim != TC_HEAD_DIM:
        return {}
    lib = attention_lib(head_dim)
    table = {}
    with torch.cuda.device(device):
        for size in range(1, 17):
            count = int(lib.rl_attention_decode_max_clusters(size))
            if count > 0:
                table[size] = count
    return table


def attention_mma(
    q: torch.Tensor,
    cache: torch.Tensor,
    out: torch.Tensor,
    *,
    chunk_items: torch.Tensor | None,
    decode_items: torch.Tensor | None,
    splits: int,
    part_out: torch.Tensor | None,
    part_lse: torch.Tensor | None,
    cu_seqlens: torch.Tensor,
    entry_start: torch.Tensor,
    entry_slot: torch.Tensor,
    block_table: torch.Tensor,
    num_heads: int,
    num_kv_heads: int,
    head_dim: int,
    window: int,
    scale: float,
    fault: torch.Tensor,
    decode_kernel: str = "auto",
    decode_rows: int = 0,
    chunk_rows: int = CHUNK_TILE_ROWS,
    decode_splits: int = 0,
    softcap: float = 0.0,
    sink: torch.Tensor | None = None,
) -> torch.Tensor:
    """bfloat16 paged causal attention over work items the host cut the step into.

    Decode tiles run on the tcgen05 kernel where it applies (head size 128, pages of 8 to 64 or
    a multiple of 128 tokens) unless ``decode_kernel`` is ``"mma"``; ``decode_rows`` is the most
    packed rows any decode tile has (0 = not known), which lets that kernel unroll over fewer rows.
    ``chunk_rows`` says how the chunk items were cut: :data:`CHUNK_TILE_ROWS` for the mma.sync
    tiles, :data:`CHUNK_TILE_ROWS_TC` for the tcgen05 kernel (``splits`` must then be 1).

    ``chunk_items`` / ``decode_items`` are int32 ``[n, 4]`` rows ``(entry, first packed row,
    split, 0)`` for tiles of :data:`CHUNK_TILE_ROWS` / :data:`DECODE_TILE_ROWS` packed rows
    (row ``p`` of an entry is token ``p // group``, head ``p % group`` of each kv head).
    With ``splits > 1`` every item exists once per split and ``part_out`` ``[T * Hq * splits,
    D]`` / ``part_lse`` ``[T * Hq * splits]`` (float32) are scratch.  ``decode_splits`` (0 = as ``splits``) gives
    the decode items a split count of their own, merged inside the tcgen05 decode kernel's clusters: only with
    ``splits == 1``, where that kernel applies, up to 16.

    ``softcap`` > 0 squashes the scaled scores to ``softcap * tanh(s / softcap)``; ``sink`` (float32 ``[heads]``)
    adds ``exp(sink[h])`` to every row's denominator, once.  The tcgen05 chunk tiles and the mma.sync tiles take
    both; with either one the decode tiles run on mma.sync (and have no split count of their own).
    """
    _need_cuda(q, cache, out, chunk_items, decode_items, part_out, part_lse, cu_seqlens, entry_start,
               entry_slot, block_table, fault, sink)
    _expect("sink", sink, torch.float32), _contig("sink", sink)
    if sink is not None and sink.numel() != num_heads:
        raise KernelError("attention: one sink per head")
    for name, tensor in (("q", q), ("cache", cache), ("out", out)):
        _expect(name, tensor, torch.bfloat16), _contig(name, tensor)
    for name, tensor in (("chunk_items", chunk_items), ("decode_items", decode_items), ("cu_seqlens", cu_seqlens),
                         ("entry_start", entry_start), ("entry_slot", entry_slot), ("block_table", block_table)):
        _expect(name, tensor, torch.int32), _contig(name, tensor)
    _expect("part_out", part_out, torch.float32), _expect("part_lse", part_lse, torch.float32)
    width = num_heads * head_dim
    if q.dim() != 2 or q.shape[1] != width or out.shape != q.shape:
        raise KernelError("attention: q and out must be [tokens, heads * head_dim]")
    tokens = q.shape[0]
    if cache.dim() != 5 or cache.shape[1] not in (1, 2) or cache.shape[2] != num_kv_heads or cache.shape[4] != head_dim:
        raise KernelError("attention: cache must be [pages, 2 (or 1: values are the keys' rows), kv_heads, page_size, head_dim]")
    if num_heads % num_kv_heads:
        raise KernelError("attention: heads must be a multiple of kv heads")
    n_chunk = 0 if chunk_items is None else chunk_items.shape[0]
    n_decode = 0 if decode_items is None else decode_items.shape[0]
    if splits > 1:
        need = tokens * num_heads * splits
        if part_out is None or part_lse is None or part_out.numel() < need * head_dim or part_lse.numel() < need:
            raise KernelError("attention: scratch for the split key ranges is missing or too small")
    _check(
        attention_lib(head_dim).rl_attention_mma(
            _ptr(q), _ptr(cache), _ptr(out), _ptr(part_out), _ptr(part_lse), _ptr(chunk_items), n_chunk,
            _ptr(decode_items), n_decode, _ptr(cu_seqlens), _ptr(entry_start), _ptr(entry_slot),
            _ptr(block_table), tokens, num_heads, num_kv_heads, head_dim, cache.shape[3], cache.shape[0],
            block_table.shape[1], block_table.shape[0], int(window), int(splits), float(scale),
            _ptr(fault), int(PDL), {"auto": 0, "mma": 1, "deep": 2, "shallow": 3}[decode_kernel], int(decode_rows), int(chunk_rows),
            int(decode_splits), float(softcap), _ptr(sink), int(cache.shape[1]), _stream(),
        ),
        f"attention_mma(head_dim={head_dim})",
    )
    LAUNCHES.count += (1 if n_chunk and n_decode else 0) + (1 if splits > 1 else 0)
    return out


def gemm_f32(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor, bias: torch.Tensor | None = None) -> torch.Tensor:
    """``out[M, N] = a[M, K] @ w[N, K]^T`` in true float32."""
    _need_cuda(a, w, out, bias)
    for name, tensor in (("a", a), ("w", w), ("out", out), ("bias", bias)):
        _expect(name, tensor, torch.float32)
    _contig("w", w)
    if a.dim() != 2 or w.dim() != 2 or a.shape[1] != w.shape[1] or out.shape != (a.shape[0], w.shape[0]):
        raise KernelError(f"gemm_f32: shapes {tuple(a.shape)} x {tuple(w.shape)}^T -> {tuple(out.shape)} do not agree")
    if a.stride(1) != 1 or out.stride(1) != 1:
        raise KernelError("gemm_f32: rows of a and out must be contiguous")
    _check(
        core().rl_gemm_f32(_ptr(a), _ptr(w), _ptr(bias), _ptr(out), a.shape[0], w.shape[0], a.shape[1],
                           a.stride(0), out.stride(0), _stream()),
        "gemm_f32",
    )
    return out


_GEMM_LIB: ctypes.CDLL | None = None


def gemm_lib() -> ctypes.CDLL:
    global _GEMM_LIB
    if _GEMM_LIB is None:
        lib = load_library("gemm")
        lib.rl_gemm_bf16.argtypes = [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int,
                                     c_void_p, c_void_p]
        lib.rl_gemm_bf16.restype = c_int
        lib.rl_gemm_bf16_norm.argtypes = [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int,
                                          c_void_p, c_void_p, c_void_p, c_void_p, c_int, ctypes.c_float, c_int,
                                          c_void_p, c_float, c_float, c_void_p, c_void_p]
        lib.rl_gemm_bf16_norm.restype = c_int
        lib.rl_gemm_bf16_sumsq_count.argtypes = [c_int]
        lib.rl_gemm_bf16_sumsq_count.restype = c_int
        _GEMM_LIB = lib
    return _GEMM_LIB


def gemm_bf16_supports(x: torch.Tensor, w: torch.Tensor) -> bool:
    """Whether the tensor-core product takes these operands (TMA wants 16-byte rows)."""
    return x.shape[1] % 8 == 0 and x.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0


GEMM_NORM_MAX_TOKENS = 64   # most rows of a product that carries a norm's add or a norm's open scale


def gemm_bf16_sumsq_count(n_out: int) -> int:
    """Columns of the table of partial sums of squares that a product of ``n_out`` columns writes."""
    return int(gemm_lib().rl_gemm_bf16_sumsq_count(int(n_out)))


def gemm_bf16(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, fault: torch.Tensor, *, swiglu: bool = False,
              k_split: int = 0, residual: torch.Tensor | None = None, norm_weight: torch.Tensor | None = None,
              sumsq_out: torch.Tensor | None = None, sumsq_in: torch.Tensor | None = None,
              norm_eps: float = 0.0, norm_size: int = 0, bias: torch.Tensor | None = None,
              glu_limit: float = 0.0, glu_alpha: float = 1.0) -> torch.Tensor:
    """``out[T, N] = x[T, K] @ w[N, K]^T`` in bfloat16 on the tcgen05 tensor cores.

    With ``swiglu``, ``w`` is ``[2 N, K]`` (gate rows, then up rows) and
    ``out = silu(x @ gate^T) * (x @ up^T)`` without the ``[T, 2 N]`` intermediate; with ``glu_limit`` > 0 the unit
    is the clamped one instead, ``g * sigmoid(glu_alpha g) * (u + 1)`` with ``g = min(gate, limit)``,
    ``u = clamp(up, -limit, limit)``.
    ``k_split`` forces how many CTAs share a tile's inner range (0 = the kernel chooses).

    A norm between two products rides on them (at most :data:`GEMM_NORM_MAX_TOKENS` rows).
    With ``residual`` (float32 ``[T, N]``), ``norm_weight`` (float32 ``[N]``) and ``sumsq_out``
    (float32 ``[T, gemm_bf16_sumsq_count(N)]``) the product is added to ``residual`` in place,
    ``out = residual * norm_weight`` and ``sumsq_out`` receives partial sums of the new
    residual's squares.  With ``sumsq_in`` (such a table), ``norm_eps`` and ``norm_size``, row
    ``t`` of the product is multiplied by ``rsqrt(sum(sumsq_in[t]) / norm_size + norm_eps)``
    (before the SiLU): the scale that the norm before ``x`` left open.  ``bias`` (float32 ``[N]``, with
    ``swiglu`` ``[2 N]``) is added to every row after that scale.
    """
    _need_cuda(x, w, out, fault, residual, norm_weight, sumsq_out, sumsq_in, bias)
    if bias is not None:
        _expect("bias", bias, torch.float32), _contig("bias", bias)
        if bias.shape != (w.shape[0],):
            raise KernelError(f"gemm_bf16: bias of shape {tuple(bias.shape)} for a weight of {w.shape[0]} rows")
    for name, tensor in (("x", x), ("w", w), ("out", out)):
        _expect(name, tensor, torch.bfloat16), _contig(name, tensor)
    tokens, k = x.shape
    n_out = out.shape[1]
    if w.shape != ((2 if swiglu else 1) * n_out, k) or out.shape[0] != tokens:
        raise KernelError(f"gemm_bf16: shapes {tuple(x.shape)} x {tuple(w.shape)}^T -> {tuple(out.shape)} do not agree")
    if not gemm_bf16_supports(x, w):
        raise KernelError("gemm_bf16: the inner size must be a multiple of 8 and the operands 16-byte aligned")
    norm_follows = residual is not None or norm_weight is not None or sumsq_out is not None
    if norm_follows:
        if residual is None or norm_weight is None or sumsq_out is None or swiglu:
            raise KernelError("gemm_bf16: a following norm needs residual, norm_weight and sumsq_out, and no swiglu")
        for name, tensor in (("residual", residual), ("norm_weight", norm_weight), ("sumsq_out", sumsq_out)):
            _expect(name, tensor, torch.float32), _contig(name, tensor)
        if (residual.shape != (tokens, n_out) or norm_weight.shape != (n_out,)
                or sumsq_out.shape != (tokens, gemm_bf16_sumsq_count(n_out))):
            raise KernelError("gemm_bf16: residual, norm_weight or sumsq_out do not have the product's shape")
    if sumsq_in is not None:
        _expect("sumsq_in", sumsq_in, torch.float32), _contig("sumsq_in", sumsq_in)
        if sumsq_in.dim() != 2 or sumsq_in.shape[0] != tokens or sumsq_in.shape[1] % 4 or norm_size <= 0:
            raise KernelError("gemm_bf16: sumsq_in must be [tokens, a multiple of 4] and norm_size positive")
    if (norm_follows or sumsq_in is not None) and tokens > GEMM_NORM_MAX_TOKENS:
        raise KernelError(f"gemm_bf16: a norm rides on products of at most {GEMM_NORM_MAX_TOKENS} rows, got {tokens}")
    if tokens == 0:
        return out
    _check(
        gemm_lib().rl_gemm_bf16_norm(
            _ptr(x), _ptr(w), _ptr(out), tokens, n_out, k, int(swiglu), int(PDL), int(k_split),
            _ptr(residual), _ptr(norm_weight), _ptr(sumsq_out),
            _ptr(sumsq_in), 0 if sumsq_in is None else sumsq_in.shape[1], float(norm_eps), int(norm_size),
            _ptr(bias), float(glu_limit), float(glu_alpha), _ptr(fault), _stream(),
        ),
        f"gemm_bf16({tokens}x{k} by {n_out})",
    )
    return out


def gemm_bf16_pair(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, fault: torch.Tensor,
                   bias: torch.Tensor | None = None, *, swiglu: bool = False,
                   residual: torch.Tensor | None = None, norm_weight: torch.Tensor | None = None,
                   sumsq_out: torch.Tensor | None = None, sumsq_in: torch.Tensor | None = None,
                   norm_eps: float = 0.0, norm_size: int = 0, glu_limit: float = 0.0, glu_alpha: float = 1.0) -> torch.Tensor:
    """``out[T, N] = x[T, K] @ w[N, K]^T (+ bias)`` in bfloat16 for steps of many tokens: pairs of CTAs on
    256 x 256 tiles (``tcgen05.mma.cta_group::2``), persistent over the tiles, the tokens on the accumulator's lanes.

    The options are those of :func:`gemm_bf16` and mean the same (``swiglu``: ``w`` is ``[2 N, K]``, gate rows
    first; ``residual``, ``norm_weight``, ``sumsq_out``: the norm that follows rides, with a slot of
    ``sumsq_out[T, gemm_bf16_sumsq_count(N)]`` per 32 columns; ``sumsq_in``, ``norm_eps``, ``norm_size``: the scale
    a norm before the product left open), at any number of tokens.  ``N`` must be a multiple of 8."""
    _need_cuda(x, w, out, fault, bias, residual, norm_weight, sumsq_out, sumsq_in)
    for name, tensor in (("x", x), ("w", w), ("out", out)):
        _expect(name, tensor, torch.bfloat16), _contig(name, tensor)
    tokens, k = x.shape
    n_out = out.shape[1]
    if w.shape != ((2 if swiglu else 1) * n_out, k) or out.shape[0] != tokens:
        raise KernelError(f"gemm_bf16_pair: shapes {tuple(x.shape)} x {tuple(w.shape)}^T -> {tuple(out.shape)} do not agree")
    if not gemm_bf16_supports(x, w) or n_out % 8:
        raise KernelError("gemm_bf16_pair: the inner size and the result's width must be multiples of 8 and the operands 16-byte aligned")
    if bias is not None:
        _expect("bias", bias, torch.float32), _contig("bias", bias)
        if bias.shape != (w.shape[0],):
            raise KernelError("gemm_bf16_pair: the bias does not have the weight's rows")
    norm_follows = residual is not None or norm_weight is not None or sumsq_out is not None
    if norm_follows:
        if residual is None or norm_weight is None or sumsq_out is None or swiglu:
            raise KernelError("gemm_bf16_pair: a following norm needs residual, norm_weight and sumsq_out, and no swiglu")
        for name, tensor in (("residual", residual), ("norm_weight", norm_weight), ("sumsq_out", sumsq_out)):
            _expect(name, tensor, torch.float32), _contig(name, tensor)
        if (residual.shape != (tokens, n_out) or norm_weight.shape != (n_out,)
                or sumsq_out.shape != (tokens, gemm_bf16_sumsq_count(n_out))):
            raise KernelError("gemm_bf16_pair: residual, norm_weight or sumsq_out do not have the product's shape")
    if sumsq_in is not None:
        _expect("sumsq_in", sumsq_in, torch.float32), _contig("sumsq_in", sumsq_in)
        if sumsq_in.dim() != 2 or sumsq_in.shape[0] != tokens or sumsq_in.shape[1] % 4 or norm_size <= 0:
            raise KernelError("gemm_bf16_pair: sumsq_in must be [tokens, a multiple of 4] and norm_size positive")
    if tokens == 0:
        return out
    lib = gemm_lib()
    if not getattr(lib, "_pair_declared", False):
        lib.rl_gemm_bf16_pair.argtypes = [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int,
                                          c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int, c_float, c_int, c_void_p,
                                          c_float, c_float, c_void_p, c_void_p, c_void_p, c_void_p]
        lib.rl_gemm_bf16_pair.restype = c_int
        lib.rl_gemm_bf16_pair_scratch_floats.restype = c_longlong
        lib.rl_gemm_bf16_pair_counter_words.restype = c_int
        lib._pair_declared = True
    state = _PAIR_STATE.get(fault.device)
    if state is None:        # partial tiles of the pairs' first segments, and the tiles' counters (the kernel keeps them zero)
        state = (torch.empty(lib.rl_gemm_bf16_pair_scratch_floats(), dtype=torch.float32, device=fault.device),
                 torch.zeros(lib.rl_gemm_bf16_pair_counter_words(), dtype=torch.int32, device=fault.device))
        _PAIR_STATE[fault.device] = state
    _check(lib.rl_gemm_bf16_pair(_ptr(x), _ptr(w), _ptr(out), tokens, n_out, k, int(swiglu), int(PDL),
                                 _ptr(residual), _ptr(norm_weight), _ptr(sumsq_out),
                                 0 if sumsq_out is None else sumsq_out.shape[1],
                                 _ptr(sumsq_in), 0 if sumsq_in is None else sumsq_in.shape[1], float(norm_eps), int(norm_size),
                                 _ptr(bias), float(glu_limit), float(glu_alpha), _ptr(state[0]), _ptr(state[1]), _ptr(fault),
                                 _stream()),
           f"gemm_bf16_pair({tokens}x{k} by {n_out})")
    return out


_PAIR_STATE: dict[torch.device, tuple[torch.Tensor, torch.Tensor]] = {}


def gemm_bf16_pair_takes(tokens: int, n_out: int, swiglu: bool) -> bool:
    """Whether a product of this size is within the pair kernel's table of tiles (256 tokens by 256 columns of the
    result, 128 with ``swiglu``); larger products are the library's."""
    lib = gemm_lib()
    lib.rl_gemm_bf16_pair_counter_words.restype = c_int
    tiles = -(-int(tokens) // 256) * -(-int(n_out) // (128 if swiglu else 256))
    return n_out % 8 == 0 and tiles <= lib.rl_gemm_bf16_pair_counter_words() // 2


class _ChainPhase(ctypes.Structure):
    """``RlChainPhase`` of ``csrc/gemm_chain.cu``."""

    _fields_ = [
        ("x", c_void_p), ("w", c_void_p), ("out", c_void_p), ("n_out", c_int), ("k", c_int), ("swiglu", c_int),
        ("residual", c_void_p), ("norm_weight", c_void_p), ("sumsq_out", c_void_p), ("sumsq_in", c_void_p),
        ("sumsq_count", c_int), ("norm_eps", c_float), ("norm_size", c_int), ("bias", c_void_p),
    ]


GEMM_CHAIN_MAX_PHASES = 4
GEMM_CHAIN_MAX_TOKENS = 64
_CHAIN_STATE: dict[torch.device, dict] = {}


def _chain_lib() -> ctypes.CDLL:
    lib = gemm_lib()
    if not getattr(lib, "_chain_declared", False):
        lib.rl_gemm_chain.argtypes = [c_void_p, c_int, c_int, c_void_p, c_longlong, c_void_p, c_void_p, c_int, c_void_p, c_void_p]
        lib.rl_gemm_chain_scratch_floats.argtypes = [c_void_p, c_int, c_int]
        lib.rl_gemm_chain_scratch_floats.restype = c_longlong
        lib.rl_gemm_chain.restype = c_int
        lib.rl_gemm_chain_counter_words.restype = c_int
        lib._chain_declared = True
    return lib


def gemm_chain_reset(device=None) -> None:
    """Zero the chain kernel's counters (after a fault: the kernel keeps them zero only when it ends well)."""
    for key, state in _CHAIN_STATE.items():
        if device is None or key == torch.device(device):
            state["counters"].zero_()
    for key, state in _PAIR_STATE.items():
        if device is None or key == torch.device(device):
            state[1].zero_()


def gemm_chain(products: list[dict], fault: torch.Tensor, trace: torch.Tensor | None = None) -> None:
    """Two to four bfloat16 products of the same (at most 64) tokens as one persistent kernel, each reading
    what earlier ones wrote.  A product is the keyword arguments of :func:`gemm_bf16` (``x``, ``w``, ``out``,
    ``swiglu``, ``residual``, ``norm_weight``, ``sumsq_out``, ``sumsq_in``, ``norm_eps``, ``norm_size``,
    ``bias``); the results are those of calling it once per product, up to the order of float32 additions.
    Scratch for partial tiles and the kernel's counters are kept per device and grow on demand.  ``trace``
    (int64 ``[multiprocessors, 4, 8]``) receives the kernel's time stamps per CTA, phase and event."""
    count = len(products)
    if not 1 <= count <= GEMM_CHAIN_MAX_PHASES:
        raise KernelError(f"gemm_chain: takes 1 to {GEMM_CHAIN_MAX_PHASES} products, got {count}")
    tokens = products[0]["x"].shape[0]
    if not 0 < tokens <= GEMM_CHAIN_MAX_TOKENS:
        raise KernelError(f"gemm_chain: takes 1 to {GEMM_CHAIN_MAX_TOKENS} tokens, got {tokens}")
    array = (_ChainPhase * count)()
    for slot, product in zip(array, products):
        x, w, out = product["x"], product["w"], product["out"]
        swiglu = bool(product.get("swiglu", False))
        extras = [product.get(name) for name in ("residual", "norm_weight", "sumsq_out", "sumsq_in", "bias")]
        _need_cuda(x, w, out, fault, *extras)
        for name, tensor in (("x", x), ("w", w), ("out", out)):
            _expect(name, tensor, torch.bfloat16), _contig(name, tensor)
        for name, tensor in zip(("residual", "norm_weight", "sumsq_out", "sumsq_in", "bias"), extras):
            _expect(name, tensor, torch.float32), _contig(name, tensor)
        n_out = out.shape[1]
        if x.shape[0] != tokens or out.shape[0] != tokens or w.shape != ((2 if swiglu else 1) * n_out, x.shape[1]):
            raise KernelError(f"gemm_chain: shapes {tuple(x.shape)} x {tuple(w.shape)}^T -> {tuple(out.shape)} do not agree")
        if not gemm_bf16_supports(x, w):
            raise KernelError("gemm_chain: the inner size must be a multiple of 8 and the operands 16-byte aligned")
        residual, norm_weight, sumsq_out, sumsq_in, bias = extras
        if any(t is not None for t in (residual, norm_weight, sumsq_out)):
            if residual is None or norm_weight is None or sumsq_out is None or swiglu:
                raise KernelError("gemm_chain: a following norm needs residual, norm_weight and sumsq_out, and no swiglu")
            if (residual.shape != (tokens, n_out) or norm_weight.shape != (n_out,)
                    or sumsq_out.shape != (tokens, gemm_bf16_sumsq_count(n_out))):
                raise KernelError("gemm_chain: residual, norm_weight or sumsq_out do not have the product's shape")
        if sumsq_in is not None and (sumsq_in.dim() != 2 or sumsq_in.shape[0] != tokens or sumsq_in.shape[1] % 4
                                     or product.get("norm_size", 0) <= 0):
            raise KernelError("gemm_chain: sumsq_in must be [tokens, a multiple of 4] and norm_size positive")
        if bias is not None and bias.shape != (w.shape[0],):
            raise KernelError("gemm_chain: the bias does not have the weight's rows")
        slot.x, slot.w, slot.out = x.data_ptr(), w.data_ptr(), out.data_ptr()
        slot.n_out, slot.k, slot.swiglu = n_out, x.shape[1], int(swiglu)
        slot.residual = None if residual is None else residual.data_ptr()
        slot.norm_weight = None if norm_weight is None else norm_weight.data_ptr()
        slot.sumsq_out = None if sumsq_out is None else sumsq_out.data_ptr()
        slot.sumsq_in = None if sumsq_in is None else sumsq_in.data_ptr()
        slot.sumsq_count = 0 if sumsq_in is None else sumsq_in.shape[1]
        slot.norm_eps, slot.norm_size = float(product.get("norm_eps", 0.0)), int(product.get("norm_size", 0))
        slot.bias = None if bias is None else bias.data_ptr()
    lib = _chain_lib()
    device = fault.device
    state = _CHAIN_STATE.get(device)
    if state is None:
        state = {"counters": torch.zeros(lib.rl_gemm_chain_counter_words(), dtype=torch.int32, device=device),
                 "scratch": torch.empty(1 << 20, dtype=torch.float32, device=device), "retired": []}
        _CHAIN_STATE[device] = state
    need = int(lib.rl_gemm_chain_scratch_floats(ctypes.byref(array), count, tokens))
    if need > state["scratch"].numel():
        state["retired"].append(state["scratch"])          # a captured graph may still hold its address
        state["scratch"] = torch.empty(need, dtype=torch.float32, device=device)
    stream = _stream()
    _check(
        lib.rl_gemm_chain(ctypes.byref(array), count, tokens, _ptr(state["scratch"]), state["scratch"].numel(),
                          _ptr(state["counters"]), _ptr(trace), int(PDL), _ptr(fault), stream),
        f"gemm_chain({count} products of {tokens} tokens)",
    )


def sample(
    logits: torch.Tensor,
    out: torch.Tensor,
    *,
    temperature: torch.Tensor | None = None,
    top_p: torch.Tensor | None = None,
    penalty: torch.Tensor | None = None,
    seeds: torch.Tensor | None = None,
    counters: torch.Tensor | None = None,
    seen_tokens: torch.Tensor | None = None,
    seen_offsets: torch.Tensor | None = None,
) -> torch.Tensor:
    """One token per row of ``logits`` into ``out`` (int32); no ``temperature`` = greedy."""
    _need_cuda(logits, out, temperature, top_p, penalty, seeds, counters, seen_tokens, seen_offsets)
    _expect("out", out, torch.int32)
    for name, tensor in (("temperature", temperature), ("top_p", top_p), ("penalty", penalty)):
        _expect(name, tensor, torch.float32)
    _expect("seeds", seeds, torch.int64), _expect("counters", counters, torch.int32)
    _expect("seen_tokens", seen_tokens, torch.int32), _expect("seen_offsets", seen_offsets, torch.int32)
    if logits.dim() != 2 or logits.stride(1) != 1 or out.numel() != logits.shape[0]:
        raise KernelError("sample: logits must be [rows, vocab] with contiguous rows and out [rows]")
    _check(
        core().rl_sample(
            dtype_tag(logits.dtype), _ptr(logits), logits.shape[0], logits.shape[1], logits.stride(0),
            _ptr(temperature), _ptr(top_p), _ptr(penalty), _ptr(seeds), _ptr(counters),
            _ptr(seen_tokens), _ptr(seen_offsets), _ptr(out), int(PDL), _stream(),
        ),
        f"sample(vocab={logits.shape[1]})",
    )
    return out


# ------------------------------------------------------------- mixers with a state of fixed size
_RECURRENT_SET = False


def recurrent() -> ctypes.CDLL:
    """The library of the recurrent mixers' kernels (``csrc/recurrent.cu``), built at first use."""
    global _RECURRENT_SET
    lib = load_library("recurrent")
    if not _RECURRENT_SET:
        lib.rl_causal_conv_silu.argtypes = [
            c_int, c_void_p, c_int, c_int, c_void_p, c_void_p, c_void_p, c_longlong, c_int, c_void_p, c_void_p,
            c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p, c_int, c_int, c_void_p,
        ]
        lib.rl_activate_rows.argtypes = [c_int, c_void_p, c_int, c_int, c_void_p, c_int, c_int, c_int, c_int, c_void_p]
        lib.rl_decay_gate.argtypes = [c_int, c_void_p, c_int, c_int, c_void_p, c_void_p, c_int, c_void_p, c_void_p,
                                      c_int, c_int, c_int, c_void_p]
        lib.rl_unit_heads.argtypes = [c_int, c_void_p, c_int, c_int, c_int, c_int, c_float, c_int, c_float, c_float,
                                      c_void_p, c_int, c_int, c_int, c_void_p, c_int, c_int, c_void_p]
        lib.rl_rotate_heads.argtypes = [c_int, c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p,
                                        c_int, c_int, c_int, c_int, c_float, c_int, c_int, c_void_p]
        lib.rl_linear_scan.argtypes = [
            c_void_p, c_int, c_void_p, c_int, c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p,
            c_void_p, c_int, c_void_p, c_longlong, c_int, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int,
            c_int, c_int, c_void_p, c_int, c_void_p,
        ]
        lib.rl_exp_decay.argtypes = [c_int, c_void_p, c_int, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p]
        lib.rl_tanh_rows.argtypes = [c_int, c_void_p, c_void_p, c_longlong, c_int, c_void_p]
        lib.rl_shift_mix.argtypes = [c_int, c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p, c_longlong, c_int,
                                     c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_int, c_void_p]
        lib.rl_gated_norm.argtypes = [c_int, c_int, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int, c_int,
                                      c_void_p, c_int, c_float, c_void_p, c_int, c_int, c_int, c_int, c_void_p]
        lib.rl_xielu.argtypes = [c_int, c_void_p, c_void_p, c_void_p, c_longlong, c_int, c_void_p]
        lib.rl_scaled_sum.argtypes = [c_int, c_void_p, c_void_p, c_float, c_float, c_void_p, c_longlong, c_int, c_void_p]
        for name in ("rl_causal_conv_silu", "rl_activate_rows", "rl_decay_gate", "rl_unit_heads", "rl_rotate_heads", "rl_linear_scan",
                     "rl_gated_norm", "rl_xielu", "rl_scaled_sum", "rl_exp_decay", "rl_tanh_rows", "rl_shift_mix"):
            getattr(lib, name).restype = c_int
        _RECURRENT_SET = True
    return lib


def _row_stride(name: str, tensor: torch.Tensor) -> int:
    """Row length of a 2-D tensor whose columns are contiguous (a view of some columns is fine)."""
    if tensor.dim() != 2 or (tensor.shape[1] > 1 and tensor.stride(1) != 1):
        raise KernelError(f"{name} must be rows of contiguous columns")
    return tensor.stride(0)


def _state_row(state: torch.Tensor) -> tuple[int, int]:
    """Slots and row stride of a per-slot float32 state ``[slots, n]`` (a view of some columns is fine)."""
    _expect("state", state, torch.float32)
    return state.shape[0], _row_stride("state", state)


def causal_conv_silu(x: torch.Tensor, taps: torch.Tensor, bias: torch.Tensor | None, tail: torch.Tensor,
                     out: torch.Tensor, batch, act: bool = True) -> torch.Tensor:
    """``out[t, c] = silu(bias[c] + sum_d taps[c, K - 1 - d] * x[t - d, c])`` over each request's own tokens
    (without the SiLU when ``act`` is false).

    ``x`` is ``[T, C]`` (a view of columns of the step's rows), ``taps`` float32 ``[C, K]`` with the current
    token's tap last, ``tail`` float32 ``[slots, (K - 1) * C]``: every slot's last ``K - 1`` inputs, oldest
    first, read for the tokens before this step and brought up to date afterwards.  ``out`` is float32.
    """
    _need_cuda(x, taps, bias, tail, out)
    _expect("taps", taps, torch.float32), _expect("bias", bias, torch.float32), _expect("out", out, torch.float32)
    _contig("taps", taps), _contig("out", out)
    tokens, channels = x.shape
    width = taps.shape[1]
    slots, stride = _state_row(tail)
    if taps.shape[0] != channels or out.shape != (tokens, channels) or tail.shape[1] != (width - 1) * channels:
        raise KernelError("causal_conv_silu: shapes of x, taps, tail and out do not agree")
    if width == 1:
        slots = 1 << 30      # one tap reads no tail: any slot index is fine, whatever rows `tail` has
    _check(
        recurrent().rl_causal_conv_silu(
            dtype_tag(x.dtype), _ptr(x), _row_stride("x", x), 0, _ptr(taps), _ptr(bias), _ptr(tail), stride, 0,
            _ptr(out), _ptr(batch.cu_seqlens), _ptr(batch.entry_slot), _ptr(batch.entry_start), batch.num_entries,
            tokens, channels, width, slots, _ptr(batch.fault), int(bool(act)), int(PDL), _stream()),
        f"causal_conv_silu(width={width})",
    )
    return out


def activate_rows(x: torch.Tensor, out: torch.Tensor, act: bool = True) -> torch.Tensor:
    """``out = silu(x)`` (or ``x`` itself) as float32; ``x [T, C]`` may be a view of columns."""
    _need_cuda(x, out)
    _expect("out", out, torch.float32), _contig("out", out)
    if out.shape != x.shape:
        raise KernelError("activate_rows: out must have the shape of x")
    _check(recurrent().rl_activate_rows(dtype_tag(x.dtype), _ptr(x), _row_stride("x", x), 0, _ptr(out), x.shape[0],
                                        x.shape[1], int(bool(act)), int(PDL), _stream()), "activate_rows")
    return out


def decay_gate(x: torch.Tensor, rate: torch.Tensor, bias: torch.Tensor | None, per: int, decay: torch.Tensor,
               step: torch.Tensor | None = None) -> torch.Tensor:
    """``step = softplus(x + bias)``, ``decay = exp(-rate[c // per] * step)``; float32 results ``[T, C]``.
    ``rate`` is ``exp(A_log)`` (float32), which a mixer takes once when its weights are loaded."""
    a_log = rate
    _need_cuda(x, a_log, bias, decay, step)
    for name, tensor in (("rate", a_log), ("bias", bias), ("decay", decay), ("step", step)):
        _expect(name, tensor, torch.float32), _contig(name, tensor)
    tokens, channels = x.shape
    if decay.shape != (tokens, channels) or (step is not None and step.shape != decay.shape) \
            or a_log.numel() * per != channels or (bias is not None and bias.numel() != channels):
        raise KernelError("decay_gate: shapes do not agree")
    _check(recurrent().rl_decay_gate(dtype_tag(x.dtype), _ptr(x), _row_stride("x", x), 0, _ptr(a_log), _ptr(bias),
                                     int(per), _ptr(decay), _ptr(step), tokens, channels, int(PDL), _stream()), "decay_gate")
    return decay


def unit_heads(rows: torch.Tensor, *, heads: int, dim: int, eps: float, split: int, scale_low: float,
               scale_high: float, gate_in: torch.Tensor | None = None, gate_out: torch.Tensor | None = None) -> None:
    """In place on float32 ``rows [T, heads * dim]`` (a view of columns): every head becomes
    ``x / sqrt(sum(x^2) + eps)`` times ``scale_low`` (heads below ``split``) or ``scale_high``.  With
    ``gate_in [T, n]`` (engine dtype) also ``gate_out = sigmoid(gate_in)`` as float32 ``[T, n]``."""
    _need_cuda(rows, gate_in, gate_out)
    _expect("rows", rows, torch.float32), _expect("gate_out", gate_out, torch.float32), _contig("gate_out", gate_out)
    tokens = rows.shape[0]
    if rows.shape[1] != heads * dim:
        raise KernelError("unit_heads: rows do not hold heads * dim columns")
    gates = 0 if gate_in is None else gate_in.shape[1]
    tag = dtype_tag(gate_in.dtype) if gate_in is not None else F32
    _check(recurrent().rl_unit_heads(tag, _ptr(rows), _row_stride("rows", rows), 0, heads, dim, float(eps), int(split),
                                     float(scale_low), float(scale_high), _ptr(gate_in),
                                     0 if gate_in is None else _row_stride("gate_in", gate_in), 0, gates,
                                     _ptr(gate_out), tokens, int(PDL), _stream()), "unit_heads")


def rotate_heads(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, out: torch.Tensor, positions: torch.Tensor,
                 inv_freq: torch.Tensor, *, heads: int, dim: int, vdim: int, k_scale: float) -> torch.Tensor:
    """``out = [rotated q | rotated k * k_scale | v]`` in float32 from views ``q``, ``k``, ``v`` of columns of
    one buffer of rows; the first ``2 * len(inv_freq)`` entries of each head rotate (entry i with i + half)."""
    _need_cuda(q, k, v, out, positions, inv_freq)
    _expect("out", out, torch.float32), _expect("inv_freq", inv_freq, torch.float32), _expect("positions", positions, torch.int32)
    _contig("out", out)
    tokens = q.shape[0]
    stride = _row_stride("q", q)
    if _row_stride("k", k) != stride or _row_stride("v", v) != stride or q.dtype != k.dtype or q.dtype != v.dtype:
        raise KernelError("rotate_heads: q, k and v must be columns of the same rows")
    if q.shape[1] != heads * dim or k.shape[1] != heads * dim or v.shape[1] != heads * vdim \
            or out.shape != (tokens, 2 * heads * dim + heads * vdim):
        raise KernelError("rotate_heads: shapes do not agree")
    size = q.element_size()
    _check(recurrent().rl_rotate_heads(
        dtype_tag(q.dtype), _ptr(q), stride, 0, (k.data_ptr() - q.data_ptr()) // size, (v.data_ptr() - q.data_ptr()) // size,
        _ptr(out), _ptr(positions), _ptr(inv_freq), heads, dim, vdim, 2 * inv_freq.numel(), float(k_scale), tokens,
        int(PDL), _stream()), "rotate_heads")
    return out


def linear_scan(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, decay: torch.Tensor, out: torch.Tensor,
                state: torch.Tensor, batch, *, heads: int, kv_heads: int, dim: int, vdim: int,
                beta: torch.Tensor | None = None, v_scale: torch.Tensor | None = None,
                skip: torch.Tensor | None = None, bonus: torch.Tensor | None = None) -> torch.Tensor:
    """The recurrence ``S <- decay * S; u = beta * (v - S^T k)`` (or ``v_scale * v`` without ``beta``);
    ``S <- S + k u^T; out = S^T q + skip * v`` per head over every entry's tokens, from and into
    ``state [slots, heads * dim * vdim]`` (float32; a request at position 0 starts from zeros).  With ``bonus``
    (float32 ``[heads, dim]``) the read-out comes first and weighs the token's own pair:
    ``out = (S + diag(bonus) k v^T)^T q``, then ``S <- decay * S + k v^T``.

    All operands float32: ``q``, ``k`` ``[T, kv_heads * dim]`` and ``v`` ``[T, heads * vdim]`` (views of columns
    are fine), ``decay`` ``[heads]`` (fixed), ``[T, heads]`` or ``[T, heads * dim]`` (one per row of ``S``),
    ``beta``/``v_scale`` ``[T, heads]``, ``skip`` ``[heads]``, ``out`` ``[T, heads * vdim]``.
    """
    _need_cuda(q, k, v, decay, out, state, beta, v_scale, skip, bonus)
    for name, tensor in (("q", q), ("k", k), ("v", v), ("decay", decay), ("out", out), ("beta", beta),
                         ("v_scale", v_scale), ("skip", skip), ("bonus", bonus)):
        _expect(name, tensor, torch.float32)
    _contig("decay", decay), _contig("beta", beta), _contig("v_scale", v_scale), _contig("skip", skip), _contig("bonus", bonus)
    if bonus is not None and (bonus.numel() != heads * dim or beta is not None):
        raise KernelError("linear_scan: bonus is [heads, dim] and does not go with beta")
    tokens = q.shape[0]
    if q.shape[1] != kv_heads * dim or k.shape != q.shape or v.shape != (tokens, heads * vdim) or out.shape != v.shape:
        raise KernelError("linear_scan: shapes of q, k, v and out do not agree")
    if decay.dim() == 1 and decay.numel() == heads:
        mode = 0
    elif decay.shape == (tokens, heads):
        mode = 1
    elif decay.shape == (tokens, heads * dim):
        mode = 2
    else:
        raise KernelError("linear_scan: decay must be [heads], [T, heads] or [T, heads * dim]")
    slots, stride = _state_row(state)
    if state.shape[1] != heads * dim * vdim:
        raise KernelError("linear_scan: state must hold heads * dim * vdim floats a slot")
    # A long walk is launched the ordinary way, onto an empty GPU: as a dependent it would be placed while the kernel
    # before it still fills most multiprocessors, several of its few blocks on the same ones (measured: 1.1 ms instead
    # of 0.6 ms for 2,048 tokens).  Steps of single tokens have many short blocks and keep the early start.
    early = PDL and tokens < 8 * batch.num_entries
    _check(
        recurrent().rl_linear_scan(
            _ptr(q), _row_stride("q", q), _ptr(k), _row_stride("k", k), _ptr(v), _row_stride("v", v), _ptr(decay), mode,
            _ptr(beta), _ptr(v_scale), _ptr(skip), _ptr(bonus), _ptr(out), _row_stride("out", out), _ptr(state), stride, 0,
            _ptr(batch.cu_seqlens), _ptr(batch.entry_slot), _ptr(batch.entry_start), batch.num_entries, heads, kv_heads,
            dim, vdim, slots, _ptr(batch.fault), int(early), _stream()),
        f"linear_scan(dim={dim}, vdim={vdim})",
    )
    return out


def exp_decay(x: torch.Tensor, bias: torch.Tensor | None, decay: torch.Tensor) -> torch.Tensor:
    """``decay = exp(-exp(x + bias))`` as float32 ``[T, C]``; ``x`` may be a view of columns."""
    _need_cuda(x, bias, decay)
    _expect("bias", bias, torch.float32), _expect("decay", decay, torch.float32), _contig("bias", bias), _contig("decay", decay)
    tokens, channels = x.shape
    if decay.shape != (tokens, channels) or (bias is not None and bias.numel() != channels):
        raise KernelError("exp_decay: shapes do not agree")
    _check(recurrent().rl_exp_decay(dtype_tag(x.dtype), _ptr(x), _row_stride("x", x), 0, _ptr(bias), _ptr(decay), tokens,
                                    channels, int(PDL), _stream()), "exp_decay")
    return decay


def tanh_rows(x: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """``out = tanh(x)`` (float32 arithmetic, one rounding), both contiguous and of one dtype; may be in place."""
    _need_cuda(x, out)
    _contig("x", x), _contig("out", out)
    if out.shape != x.shape or out.dtype != x.dtype:
        raise KernelError("tanh_rows: out must have the shape and dtype of x")
    _check(recurrent().rl_tanh_rows(dtype_tag(x.dtype), _ptr(x), _ptr(out), x.numel(), int(PDL), _stream()), "tanh_rows")
    return out


def shift_mix(x: torch.Tensor, mu: torch.Tensor, out: torch.Tensor, kept: torch.Tensor, batch) -> torch.Tensor:
    """``out[s, t] = x[t] + (x[t - 1] - x[t]) * mu[s]`` for each of the vectors ``mu [S, C]`` (float32), ``x[t - 1]``
    the row before within the same request: the row before in this step, the request's kept row
    (``kept [slots, C]`` float32, brought up to date here) at the start of a portion, zeros at position 0.
    ``out`` is ``[S * T, C]`` of ``x``'s dtype, plane after plane."""
    _need_cuda(x, mu, out, kept)
    _expect("mu", mu, torch.float32), _contig("mu", mu), _contig("out", out)
    tokens, channels = x.shape
    mixes = mu.shape[0]
    slots, stride = _state_row(kept)
    if mu.shape != (mixes, channels) or out.shape != (mixes * tokens, channels) or out.dtype != x.dtype \
            or kept.shape[1] != channels:
        raise KernelError("shift_mix: shapes do not agree")
    _check(recurrent().rl_shift_mix(dtype_tag(x.dtype), _ptr(x), _row_stride("x", x), _ptr(mu), mixes, _ptr(out),
                                    _ptr(kept), stride, 0, _ptr(batch.cu_seqlens), _ptr(batch.entry_slot),
                                    _ptr(batch.entry_start), batch.num_entries, tokens, channels, slots,
                                    _ptr(batch.fault), int(PDL), _stream()), "shift_mix")
    return out


_LATENT_LIB: ctypes.CDLL | None = None
ROTATE_HALVES, ROTATE_NEIGHBOURS = 0, 1      # entry i with i + R / 2; entry 2i with 2i + 1


def latent_lib() -> ctypes.CDLL:
    global _LATENT_LIB
    if _LATENT_LIB is None:
        lib = load_library("latent")
        lib.rl_latent_norm_write.argtypes = [
            c_int, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_float, c_void_p, c_void_p,
            c_void_p, c_longlong, c_int, c_void_p, c_void_p, c_float, c_int, c_int, c_void_p, c_int, c_void_p]
        lib.rl_latent_rotate_queries.argtypes = [c_int, c_void_p, c_int, c_int, c_int, c_void_p, c_int, c_int, c_void_p,
                                                 c_void_p, c_float, c_int, c_int, c_int, c_void_p]
        lib.rl_sigmoid_scale_heads.argtypes = [c_int, c_void_p, c_int, c_int, c_void_p, c_int, c_int, c_int, c_int, c_void_p]
        lib.rl_heads_linear.argtypes = [c_int, c_void_p, c_int, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int,
                                        c_int, c_void_p]
        for name in ("rl_latent_norm_write", "rl_latent_rotate_queries", "rl_sigmoid_scale_heads", "rl_heads_linear"):
            getattr(lib, name).restype = c_int
        _LATENT_LIB = lib
    return _LATENT_LIB


def latent_norm_write(down: torch.Tensor, *, q_col0: int, q_rank: int, c_col0: int, kv_rank: int, rot: int,
                      q_weight: torch.Tensor, c_weight: torch.Tensor, eps: float, q_out: torch.Tensor, cache: torch.Tensor,
                      kv_dest: torch.Tensor, positions: torch.Tensor, freq: torch.Tensor | None, magnitude: float,
                      layout: int, fault: torch.Tensor) -> None:
    """From a row ``down[t]`` that holds a query latent (``q_rank`` numbers at ``q_col0``) and ``[c | key part]``
    (``kv_rank + rot`` numbers at ``c_col0``): ``q_out[t]`` = RMS norm of the query latent times ``q_weight``; the
    cache row ``kv_dest[t]`` of ``cache [pages, page_size, D]`` = ``[RMS norm of c times c_weight | the key part
    rotated by the position | zeros]``.  float32 arithmetic, one rounding."""
    _need_cuda(down, q_weight, c_weight, q_out, cache, kv_dest, positions, freq, fault)
    _expect("q_weight", q_weight, torch.float32), _expect("c_weight", c_weight, torch.float32), _expect("freq", freq, torch.float32)
    _expect("kv_dest", kv_dest, torch.int32), _expect("positions", positions, torch.int32)
    _contig("q_out", q_out), _contig("cache", cache), _contig("freq", freq)
    tokens, width = down.shape[0], cache.shape[-1]
    if (q_out.shape != (tokens, q_rank) or q_out.dtype != down.dtype or cache.dtype != down.dtype
            or q_weight.numel() != q_rank or c_weight.numel() != kv_rank or (rot and freq.numel() != rot // 2)
            or q_col0 + q_rank > down.shape[1] or c_col0 + kv_rank + rot > down.shape[1] or kv_dest.numel() != tokens):
        raise KernelError("latent_norm_write: shapes or dtypes do not agree")
    _check(latent_lib().rl_latent_norm_write(
        dtype_tag(down.dtype), _ptr(down), _row_stride("down", down), int(q_col0), int(q_rank), int(c_col0), int(kv_rank),
        int(rot), _ptr(q_weight), _ptr(c_weight), float(eps), _ptr(q_out), _ptr(cache), _ptr(kv_dest),
        cache.numel() // width, width, _ptr(positions), _ptr(freq), float(magnitude), int(layout), tokens, _ptr(fault),
        int(PDL), _stream()), "latent_norm_write")


def latent_rotate_queries(q: torch.Tensor, wide: torch.Tensor, *, heads: int, dim: int, rot: int, kv_rank: int,
                          positions: torch.Tensor, freq: torch.Tensor | None, magnitude: float, layout: int) -> torch.Tensor:
    """``q [T, heads * (dim + rot)]``: every head's last ``rot`` numbers, rotated by the position, go to columns
    ``[kv_rank, kv_rank + rot)`` of the head's ``D`` columns of ``wide [T, heads * D]``; the columns behind get zeros."""
    _need_cuda(q, wide, positions, freq)
    _expect("freq", freq, torch.float32), _expect("positions", positions, torch.int32)
    _contig("q", q), _contig("wide", wide), _contig("freq", freq)
    tokens = q.shape[0]
    if (q.shape[1] != heads * (dim + rot) or wide.shape[0] != tokens or wide.shape[1] % heads or wide.dtype != q.dtype
            or (rot and freq.numel() != rot // 2)):
        raise KernelError("latent_rotate_queries: shapes or dtypes do not agree")
    _check(latent_lib().rl_latent_rotate_queries(
        dtype_tag(q.dtype), _ptr(q), int(heads), int(dim), int(rot), _ptr(wide), int(kv_rank), wide.shape[1] // heads,
        _ptr(positions), _ptr(freq), float(magnitude), int(layout), tokens, int(PDL), _stream()), "latent_rotate_queries")
    return wide


def sigmoid_scale_heads(rows: torch.Tensor, gate: torch.Tensor, *, heads: int) -> torch.Tensor:
    """``rows[t, h, :] *= sigmoid(gate[t, h])`` in place; ``rows [T, heads * width]``, ``gate`` ``[T, >= heads]`` (a view
    of columns is fine)."""
    _need_cuda(rows, gate)
    _contig("rows", rows)
    if rows.shape[1] % heads or gate.shape[0] != rows.shape[0] or gate.shape[1] < heads or gate.dtype != rows.dtype:
        raise KernelError("sigmoid_scale_heads: shapes or dtypes do not agree")
    _check(latent_lib().rl_sigmoid_scale_heads(dtype_tag(rows.dtype), _ptr(rows), int(heads), rows.shape[1] // heads,
                                               _ptr(gate), _row_stride("gate", gate), 0, rows.shape[0], int(PDL), _stream()),
           "sigmoid_scale_heads")
    return rows


def heads_linear(x: torch.Tensor, weight: torch.Tensor, out: torch.Tensor, *, x_col0: int = 0) -> torch.Tensor:
    """A product per head: ``out[t, h, :N] = x[t, h, x_col0 : x_col0 + K] @ weight[h]^T`` with ``weight [heads, N, K]``,
    ``x [T, heads * x_width]`` and ``out [T, heads * out_width]``; float32 sums (true 32-bit for float32 operands).
    Columns of ``out`` behind ``N`` in each head are left as they are."""
    _need_cuda(x, weight, out)
    _contig("x", x), _contig("weight", weight), _contig("out", out)
    heads, n_out, k = weight.shape
    if (x.dtype != weight.dtype or out.dtype != x.dtype or x.shape[1] % heads or out.shape[1] % heads
            or out.shape[0] != x.shape[0]):
        raise KernelError("heads_linear: shapes or dtypes do not agree")
    _check(latent_lib().rl_heads_linear(dtype_tag(x.dtype), _ptr(x), x.shape[1] // heads, int(x_col0), _ptr(weight), _ptr(out),
                                        out.shape[1] // heads, x.shape[0], heads, n_out, k, int(PDL), _stream()),
           "heads_linear")
    return out


def join_then_rmsnorm(x: torch.Tensor, residual: torch.Tensor, weight: torch.Tensor, next_weight: torch.Tensor,
                      out: torch.Tensor, eps: float) -> torch.Tensor:
    """A norm on a sublayer's output and the norm in front of the next one in one pass over the row:
    ``residual += x * rsqrt(mean(x^2) + eps) * weight`` (float32, in place), then
    ``out = residual * rsqrt(mean(residual^2) + eps) * next_weight`` in the engine's dtype."""
    _need_cuda(x, residual, weight, next_weight, out)
    for name, tensor in (("weight", weight), ("next_weight", next_weight), ("residual", residual)):
        _expect(name, tensor, torch.float32), _contig(name, tensor)
    _contig("x", x), _contig("out", out)
    if (residual.shape != x.shape or out.shape != x.shape or out.dtype != x.dtype or weight.numel() != x.shape[-1]
            or next_weight.numel() != x.shape[-1]):
        raise KernelError("join_then_rmsnorm: shapes of x, residual, the weights and out do not agree")
    _check(core().rl_add_rmsnorm(dtype_tag(x.dtype), _ptr(x), _ptr(residual), _ptr(weight), _ptr(out), None,
                                 x.shape[0], x.shape[1], float(eps), 5, 1, None, _ptr(next_weight), int(PDL), _stream()),
           "join_then_rmsnorm")
    return out


GATE_NONE, GATE_SIGMOID, GATE_SILU = 0, 1, 2


def gated_norm(y: torch.Tensor, out: torch.Tensor, *, group: int, gate: torch.Tensor | None = None,
               act: int = GATE_NONE, gate_first: bool = False, norm: bool = True, weight: torch.Tensor | None = None,
               eps: float = 0.0) -> torch.Tensor:
    """Norm and gate of a mixer's result: ``y [T, C]`` (float32, or the engine's dtype) in groups of ``group``
    columns, each divided by ``sqrt(mean(z^2) + eps)`` and multiplied by ``weight[c % len(weight)]``; the gate
    ``act(gate[t, c])`` multiplies before (``gate_first``) or after the norm.  ``out`` has the engine's dtype."""
    _need_cuda(y, out, gate, weight)
    _expect("weight", weight, torch.float32), _contig("weight", weight), _contig("out", out)
    tokens, width = y.shape
    if width % group or out.shape != y.shape or (gate is not None and (gate.shape != y.shape or gate.dtype != out.dtype)):
        raise KernelError("gated_norm: shapes do not agree")
    if y.dtype != torch.float32 and y.dtype != out.dtype:
        raise KernelError("gated_norm: y must be float32 or of out's dtype")
    _check(
        recurrent().rl_gated_norm(
            dtype_tag(out.dtype), int(y.dtype == torch.float32), _ptr(y), _row_stride("y", y), _ptr(gate),
            0 if gate is None else _row_stride("gate", gate), 0, int(act), int(gate_first), int(norm), _ptr(weight),
            0 if weight is None else weight.numel(), float(eps), _ptr(out), tokens, group, width // group, int(PDL), _stream()),
        "gated_norm",
    )
    return out


def xielu(x: torch.Tensor, out: torch.Tensor, pq: torch.Tensor) -> torch.Tensor:
    """``z > 0: softplus(p) z^2 + z / 2``; ``z <= 0: (1/2 + softplus(q)) (exp(z) - 1 - z) + z / 2``; ``pq = [p, q]``."""
    _need_cuda(x, out, pq)
    _contig("x", x), _contig("out", out), _expect("pq", pq, torch.float32)
    if out.shape != x.shape or out.dtype != x.dtype or pq.numel() != 2:
        raise KernelError("xielu: shapes do not agree")
    _check(recurrent().rl_xielu(dtype_tag(x.dtype), _ptr(x), _ptr(out), _ptr(pq), x.numel(), int(PDL), _stream()), "xielu")
    return out


def scaled_sum(a: torch.Tensor, b: torch.Tensor, a_scale: float, b_scale: float, out: torch.Tensor) -> torch.Tensor:
    """``out = a_scale * a + b_scale * b`` (float32 arithmetic)."""
    _need_cuda(a, b, out)
    _contig("a", a), _contig("b", b), _contig("out", out)
    if a.shape != b.shape or out.shape != a.shape or a.dtype != b.dtype or out.dtype != a.dtype:
        raise KernelError("scaled_sum: shapes do not agree")
    _check(recurrent().rl_scaled_sum(dtype_tag(a.dtype), _ptr(a), _ptr(b), float(a_scale), float(b_scale), _ptr(out),
                                     a.numel(), int(PDL), _stream()), "scaled_sum")
    return out


# ------------------------------------------------------------- routed feed-forward
_MOE_LIB: ctypes.CDLL | None = None


def moe_lib() -> ctypes.CDLL:
    """The library of the routed feed-forward's kernels (``csrc/moe.cu``), built at first use."""
    global _MOE_LIB
    if _MOE_LIB is None:
        lib = load_library("moe")
        lib.rl_router_topk.argtypes = [c_int, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_void_p,
                                       c_void_p, c_void_p, c_int, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_void_p]
        lib.rl_moe_plan.argtypes = [c_void_p, c_int, c_int, c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p, c_int, c_void_p]
        lib.rl_moe_tile_rows.argtypes = [c_int]
        lib.rl_grouped_linear.argtypes = [c_int, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int,
                                          c_int, c_int, c_int, c_void_p, c_void_p, c_int, c_int, c_float, c_float, c_int,
                                          c_void_p]
        lib.rl_moe_combine.argtypes = [c_int, c_void_p, c_int, c_void_p, c_void_p, c_int, c_void_p, c_int, c_int, c_void_p,
                                       c_void_p, c_int, c_void_p, c_int, c_int, c_void_p]
        lib.rl_moe_combine_layernorm.argtypes = [c_int, c_void_p, c_int, c_void_p, c_void_p, c_int, c_void_p, c_int, c_void_p,
                                                 c_float, c_void_p, c_void_p, c_float, c_void_p, c_int, c_int, c_int, c_void_p]
        for name in ("rl_router_topk", "rl_moe_plan", "rl_grouped_linear", "rl_moe_combine", "rl_moe_tile_rows",
                     "rl_moe_combine_layernorm"):
            getattr(lib, name).restype = c_int
        _MOE_LIB = lib
    return _MOE_LIB


def moe_tile_rows(wide: bool) -> int:
    """Pairs per tile: of the plain tiles, or of the pipelined bfloat16 kernel's (``wide``)."""
    return int(moe_lib().rl_moe_tile_rows(int(bool(wide))))


def moe_wide_takes(dtype: torch.dtype, *inner_sizes: int) -> bool:
    """Whether the pipelined bfloat16 kernel takes products with these inner sizes (16-byte rows)."""
    return dtype == torch.bfloat16 and all(size % 8 == 0 for size in inner_sizes)


def moe_max_tiles(pairs: int, experts: int, wide: bool = False) -> int:
    """Most tiles the (token, expert) pairs of a step can fall into."""
    return -(-int(pairs) // moe_tile_rows(wide)) + int(experts)


def router_topk(x: torch.Tensor, weight: torch.Tensor, *, experts: int, top: int, ids: torch.Tensor,
                weights: torch.Tensor, gates: torch.Tensor | None = None, scores: torch.Tensor | None = None,
                bias: torch.Tensor | None = None, softmax_chosen: bool = False, softmax_all: bool = False,
                correction: torch.Tensor | None = None, groups: int = 1, keep: int = 1) -> None:
    """``z = weight[:experts] @ x[t] (+ bias)`` in float32; ``ids[t]`` the ``top`` largest (ties: the lower index),
    ``weights[t]`` their ``sigmoid(z)``, or with ``softmax_chosen`` the softmax over the chosen ``z`` alone; rows of
    ``weight`` behind the experts' are gates, ``gates[t, g] = sigmoid(.)``.

    With ``softmax_all`` the scores are ``s = softmax(z)`` over all ``experts`` rows; the choice is made on
    ``s + correction`` (one float per row) among the rows of the ``keep`` best of ``groups`` equal groups of
    neighbouring rows (a group ranks by its largest corrected score; rows of the other groups count as minus
    infinity), and the weights are the chosen rows' ``s`` divided by their sum (plus 1e-20).  ``scores`` (float32
    ``[T, experts]``) receives every row's score: the sigmoid of its logit, or its softmax share with ``softmax_all``."""
    _need_cuda(x, weight, ids, weights, gates, scores, bias, correction)
    _expect("bias", bias, torch.float32), _contig("bias", bias)
    _expect("correction", correction, torch.float32), _contig("correction", correction)
    if bias is not None and bias.numel() != experts:
        raise KernelError("router_topk: one bias per expert")
    if softmax_all and (softmax_chosen or bias is not None or groups < 1 or experts % groups or not 1 <= keep <= groups
                        or top > keep * (experts // groups) or (correction is not None and correction.numel() != experts)):
        raise KernelError("router_topk: softmax over all rows takes a correction per row and groups that divide the rows "
                          "and leave at least `top` rows to choose from")
    if not softmax_all and (correction is not None or groups != 1):
        raise KernelError("router_topk: corrections and groups belong to the softmax over all rows")
    _expect("weight", weight, torch.float32), _expect("ids", ids, torch.int32), _expect("weights", weights, torch.float32)
    _expect("gates", gates, torch.float32), _expect("scores", scores, torch.float32)
    _contig("weight", weight), _contig("ids", ids), _contig("weights", weights), _contig("gates", gates), _contig("scores", scores)
    tokens, hidden = x.shape
    extra = weight.shape[0] - experts
    if weight.shape[1] != hidden or extra < 0 or ids.shape != (tokens, top) or weights.shape != (tokens, top) \
            or (extra > 0 and (gates is None or gates.shape != (tokens, extra))):
        raise KernelError("router_topk: shapes do not agree")
    _check(moe_lib().rl_router_topk(dtype_tag(x.dtype), _ptr(x), _row_stride("x", x), _ptr(weight), hidden, experts, extra,
                                    top, _ptr(ids), _ptr(weights), _ptr(gates), _ptr(scores), tokens, _ptr(bias),
                                    2 if softmax_all else int(bool(softmax_chosen)), _ptr(correction), int(groups),
                                    int(keep), int(PDL), _stream()),
           "router_topk")


def moe_plan(ids: torch.Tensor, experts: int, sorted_pairs: torch.Tensor, place_of: torch.Tensor, meta: torch.Tensor,
             fault: torch.Tensor, wide: bool = False) -> int:
    """Groups the pairs ``ids [T, top]`` by expert on the device, in tiles of :func:`moe_tile_rows` pairs; returns the
    most tiles there can be.  The products over the plan must be asked for with the same ``wide``."""
    _need_cuda(ids, sorted_pairs, place_of, meta, fault)
    for name, tensor in (("ids", ids), ("sorted_pairs", sorted_pairs), ("place_of", place_of), ("meta", meta)):
        _expect(name, tensor, torch.int32), _contig(name, tensor)
    pairs = ids.numel()
    max_tiles = moe_max_tiles(pairs, experts, wide)
    if sorted_pairs.numel() < pairs or place_of.numel() < pairs or meta.numel() < 1 + 3 * max_tiles:
        raise KernelError("moe_plan: the tables are too small")
    _check(moe_lib().rl_moe_plan(_ptr(ids), pairs, experts, _ptr(sorted_pairs), _ptr(place_of), _ptr(meta), max_tiles,
                                 moe_tile_rows(wide), _ptr(fault), int(PDL), _stream()), "moe_plan")
    return max_tiles


def grouped_linear(a: torch.Tensor, weight: torch.Tensor, sorted_pairs: torch.Tensor, meta: torch.Tensor, *, top: int,
                   by_token: bool, max_tiles: int, pair_weight: torch.Tensor | None = None,
                   out_act: torch.Tensor | None = None, out_y: torch.Tensor | None = None, wide: bool = False,
                   clamp: tuple[float, float] | None = None) -> None:
    """Products over the pairs grouped by expert: ``weight [E, N or 2 N, K]``.  With ``out_act`` (engine dtype,
    by place) the weight is gate rows then up rows and ``out_act = silu(w g) * (w u)`` with the pair's weight ``w``,
    or with ``clamp = (limit, alpha)`` the clamped unit ``g' sigmoid(alpha g') (u' + 1)``, ``g' = min(g, limit)``,
    ``u' = clamp(u, -limit, limit)``; with ``out_y`` (float32, by pair) the plain product.  ``a`` rows are found by
    token (pair // top) or by place."""
    limit, alpha = (0.0, 0.0) if clamp is None else (float(clamp[0]), float(clamp[1]))
    if clamp is not None and limit <= 0.0:
        raise KernelError("grouped_linear: the clamped unit needs a positive limit")
    _need_cuda(a, weight, sorted_pairs, meta, pair_weight, out_act, out_y)
    _contig("weight", weight), _contig("out_act", out_act), _contig("out_y", out_y)
    _expect("pair_weight", pair_weight, torch.float32), _expect("out_y", out_y, torch.float32)
    gated = out_act is not None
    if (out_y is None) == (out_act is None) or weight.dim() != 3 or weight.dtype != a.dtype or a.shape[1] != weight.shape[2]:
        raise KernelError("grouped_linear: operands do not agree")
    n = (out_act if gated else out_y).shape[1]
    if weight.shape[1] != (2 * n if gated else n) or (gated and out_act.dtype != a.dtype):
        raise KernelError("grouped_linear: the result's width does not fit the weight")
    _check(moe_lib().rl_grouped_linear(dtype_tag(a.dtype), _ptr(a), _row_stride("a", a), _ptr(weight), _ptr(sorted_pairs),
                                       _ptr(meta), _ptr(pair_weight), int(top), int(by_token), n, a.shape[1], int(gated),
                                       _ptr(out_act), _ptr(out_y), int(max_tiles), moe_tile_rows(wide), limit, alpha,
                                       int(PDL), _stream()),
           "grouped_linear")


def moe_combine(y: torch.Tensor, top: int, out: torch.Tensor, shared: torch.Tensor | None = None,
                gate: torch.Tensor | None = None, weights: torch.Tensor | None = None, ids: torch.Tensor | None = None,
                experts: int = 0, x: torch.Tensor | None = None) -> torch.Tensor:
    """``out[t] = sum_j (weights[t, j] *) y[t * top + j] (+ gate[t] * shared[t])``, float32 sums in the order of ``j``.
    With ``ids [T, top]`` and ``x [T, hidden]`` (the experts' input): a choice whose id is ``experts`` or more is an
    identity expert, whose result is the token's own row ``x[t]`` (its row of ``y`` is never read)."""
    _need_cuda(y, out, shared, gate, weights, ids, x)
    _expect("ids", ids, torch.int32), _contig("ids", ids)
    if (ids is None) != (x is None) or (ids is not None and (ids.numel() != y.shape[0] or x.shape != out.shape or x.dtype != out.dtype)):
        raise KernelError("moe_combine: identity experts need the choices' ids and the experts' input rows")
    _expect("weights", weights, torch.float32), _contig("weights", weights)
    if weights is not None and weights.numel() != y.shape[0]:
        raise KernelError("moe_combine: one weight per (token, choice)")
    _expect("y", y, torch.float32), _expect("gate", gate, torch.float32)
    _contig("y", y), _contig("out", out), _contig("shared", shared)
    tokens, hidden = out.shape
    if y.shape != (tokens * top, hidden) or (shared is not None and (shared.shape != out.shape or shared.dtype != out.dtype)):
        raise KernelError("moe_combine: shapes do not agree")
    _check(moe_lib().rl_moe_combine(dtype_tag(out.dtype), _ptr(y), int(top), _ptr(shared), _ptr(gate),
                                    0 if gate is None else _row_stride("gate", gate), _ptr(out), tokens, hidden,
                                    _ptr(weights), _ptr(ids), int(experts), _ptr(x),
                                    0 if x is None else _row_stride("x", x), int(PDL), _stream()), "moe_combine")
    return out


def moe_combine_layernorm(y: torch.Tensor, top: int, stream: torch.Tensor, ln_weight: torch.Tensor,
                          ln_bias: torch.Tensor | None, out: torch.Tensor, eps: float, *, stream_scale: float = 1.0,
                          weights: torch.Tensor | None = None, ids: torch.Tensor | None = None, experts: int = 0,
                          x: torch.Tensor | None = None) -> torch.Tensor:
    """The sum of :func:`moe_combine` (weights, identity experts) and the layer norm that closes it, in one pass:
    ``stream[t] <- LN(stream_scale * stream[t] + sum_j w_j y_j)`` (float32, in place), ``out`` its rounding."""
    _need_cuda(y, stream, ln_weight, ln_bias, out, weights, ids, x)
    for name, tensor in (("y", y), ("stream", stream), ("ln_weight", ln_weight), ("ln_bias", ln_bias), ("weights", weights)):
        _expect(name, tensor, torch.float32), _contig(name, tensor)
    _expect("ids", ids, torch.int32), _contig("ids", ids), _contig("out", out)
    tokens, hidden = out.shape
    if (y.shape != (tokens * top, hidden) or stream.shape != out.shape or ln_weight.numel() != hidden
            or (ln_bias is not None and ln_bias.numel() != hidden) or (weights is not None and weights.numel() != tokens * top)
            or (ids is None) != (x is None) or (ids is not None and (ids.numel() != tokens * top or x.shape != out.shape or x.dtype != out.dtype))):
        raise KernelError("moe_combine_layernorm: shapes or dtypes do not agree")
    _check(moe_lib().rl_moe_combine_layernorm(
        dtype_tag(out.dtype), _ptr(y), int(top), _ptr(weights), _ptr(ids), int(experts), _ptr(x),
        0 if x is None else _row_stride("x", x), _ptr(stream), float(stream_scale), _ptr(ln_weight), _ptr(ln_bias), float(eps),
        _ptr(out), tokens, hidden, int(PDL), _stream()), "moe_combine_layernorm")
    return out


def describe_fault(word: int) -> str:
    parts = [text for bit, text in FAULT_BITS.items() if word & bit]
    return "; ".join(parts) if parts else "no fault"
