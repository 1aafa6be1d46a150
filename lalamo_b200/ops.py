"""Python bindings of the CUDA kernels: tensors in, launches on the current stream.

Every function checks what the kernel cannot check for itself (device, dtype, contiguity,
size limits) and raises :class:`KernelError` with a clear message instead of launching with
arguments the kernel does not support.  Matrix products of the 32-bit path go to the library
(cuBLAS through ``torch.matmul``, with TF32 and reduced-precision reductions switched off), as
the reference's go to XLA (``lalamo/weight_matrix.py:418-432``).
"""

from __future__ import annotations

from dataclasses import dataclass

import ctypes
import os
from ctypes import c_float, c_int, c_longlong, c_void_p

import torch

from . import native

__all__ = ["KernelError", "SlicedSum", "dtype_code", "launch_count", "reset_launch_count"]


class KernelError(RuntimeError):
    pass


@dataclass
class SlicedSum:
    """A product ``x @ weight.T`` left as the partial sums of its K slices, ``partials[slice, token, row]``
    in float32.  Whoever consumes it adds the slices in order and rounds the sum to ``dtype``, as the
    product's own epilogue would have: :func:`rmsnorm` and :func:`residual_add` take it as their
    ``delta``, :meth:`sum` gives the plain tensor."""

    partials: torch.Tensor
    dtype: torch.dtype

    @property
    def shape(self) -> torch.Size:
        return self.partials.shape[1:]

    def sum(self) -> torch.Tensor:
        slices, tokens, rows = self.partials.shape
        out = torch.empty(tokens, rows, dtype=self.dtype, device=self.partials.device)
        _sum_slices(self.partials, out, "store")
        return out


_ACTIVATIONS = {"silu": 0, "gelu": 1, "identity": 2}
_launches = 0


def launch_count() -> int:
    """Kernels of this library launched since the last reset."""
    return _launches


def add_launches(count: int) -> None:
    """Counts launches that did not go through these bindings (replays of a recorded graph)."""
    global _launches
    _launches += count


def reset_launch_count() -> None:
    global _launches
    _launches = 0


def dtype_code(dtype: torch.dtype) -> int:
    if dtype == torch.float32:
        return 0
    if dtype == torch.bfloat16:
        return 1
    raise KernelError(f"kernels exist for float32 and bfloat16, not {dtype}")


# The current stream's handle straight from torch's bindings where they exist: the public
# torch.cuda.current_stream() builds a Stream object and costs 3 us a call, which a step of a
# hundred-odd launches feels.
_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)
_raw_device = getattr(torch._C, "_cuda_getDevice", None)


def _stream() -> c_void_p:
    if _raw_stream is not None and _raw_device is not None:
        return c_void_p(_raw_stream(_raw_device()))
    return c_void_p(torch.cuda.current_stream().cuda_stream)


def _ptr(tensor: torch.Tensor | None) -> c_void_p:
    if tensor is None:
        return c_void_p(0)
    return c_void_p(tensor.data_ptr())


def _check(tensor: torch.Tensor, name: str, dtype: torch.dtype | None = None) -> None:
    if not tensor.is_cuda:
        raise KernelError(f"{name} must live on a CUDA device (there is no CPU path)")
    if not tensor.is_contiguous():
        raise KernelError(f"{name} must be contiguous")
    if dtype is not None and tensor.dtype != dtype:
        raise KernelError(f"{name} must be {dtype}, got {tensor.dtype}")


def _done(code: int, what: str, launches: int = 1) -> None:
    global _launches
    if code != 0:
        if code == -1:
            raise KernelError(f"{what}: unsupported element type")
        if code == -2:
            raise KernelError(f"{what}: a size is outside what the kernel supports")
        raise KernelError(f"{what}: CUDA error {code} at launch")
    _launches += launches


def _lib() -> ctypes.CDLL:
    return native.library()


# --------------------------------------------------------------------------- elementwise
def embed(table: torch.Tensor, ids: torch.Tensor, out: torch.Tensor, scale: float, status: torch.Tensor) -> None:
    """``out[t] = float(table[ids[t]]) * scale`` into the 32-bit residual stream."""
    _check(table, "table")
    _check(ids, "ids", torch.int32)
    _check(out, "out", torch.float32)
    tokens, dim = out.shape
    vocab = table.shape[0]
    if table.shape[1] != dim or ids.numel() < tokens:
        raise KernelError("embed: shapes of table, ids and out do not agree")
    code = _lib().lb_embed(_ptr(table), _ptr(ids), _ptr(out), c_int(tokens), c_int(dim), c_int(vocab), c_float(scale),
                           c_int(dtype_code(table.dtype)), _ptr(status), _stream())
    _done(code, "embed")


def rmsnorm(
    x: torch.Tensor,
    weight: torch.Tensor,
    out: torch.Tensor,
    eps: float,
    *,
    delta: torch.Tensor | SlicedSum | None = None,
    rows: torch.Tensor | None = None,
    scale_offset: float = 0.0,
    write_back: bool = False,
) -> None:
    """``out[r] = rms_norm(x[src] + delta[src]) * (weight + offset)``, ``src = rows[r]`` or ``r``.

    ``x`` is the 32-bit residual stream or has ``out``'s type.  With ``write_back`` the sum is
    stored back into ``x``.  ``delta`` may be a :class:`SlicedSum`: its slices are added here.
    """
    _check(x, "x")
    _check(weight, "weight", torch.float32)
    _check(out, "out")
    dim = x.shape[-1]
    out_rows = out.numel() // dim if dim else 0
    if out.shape[-1] != dim or weight.numel() != dim:
        raise KernelError("rmsnorm: the last dimensions of x, weight and out differ")
    if x.dtype != torch.float32 and x.dtype != out.dtype:
        raise KernelError("rmsnorm: x must be float32 or of out's type")
    partials, slices, slice_stride = None, 0, 0
    if isinstance(delta, SlicedSum):
        _check(delta.partials, "delta.partials", torch.float32)
        if delta.shape != x.shape or delta.dtype != out.dtype:
            raise KernelError("rmsnorm: the sliced delta and x differ in shape, or its type is not out's")
        partials, slices, slice_stride = delta.partials, delta.partials.shape[0], delta.partials.shape[1] * delta.partials.shape[2]
        delta = None
    elif delta is not None:
        _check(delta, "delta", out.dtype)
        if delta.shape != x.shape:
            raise KernelError("rmsnorm: delta and x differ in shape")
    if rows is not None:
        _check(rows, "rows", torch.int32)
        if rows.numel() < out_rows:
            raise KernelError("rmsnorm: fewer row indices than output rows")
    elif out_rows != x.numel() // dim:
        raise KernelError("rmsnorm: x and out differ in rows")
    if dim > 50000:
        raise KernelError(f"rmsnorm: rows of {dim} elements exceed the supported 50000")
    code = _lib().lb_rmsnorm(_ptr(x), c_int(1 if x.dtype == torch.float32 else 0),
                             _ptr(delta), _ptr(partials), c_int(slices), c_longlong(slice_stride), _ptr(weight), _ptr(rows), _ptr(out), c_int(out_rows), c_int(dim), c_float(eps),
                             c_float(scale_offset), c_int(1 if write_back else 0), c_int(dtype_code(out.dtype)), _stream())
    _done(code, "rmsnorm")


def _sum_slices(partials: torch.Tensor, out: torch.Tensor, epilogue: str) -> None:
    _check(partials, "partials", torch.float32)
    slices, tokens, rows = partials.shape
    if out.shape != (tokens, rows):
        raise KernelError("sum_slices: out must be [tokens, rows]")
    code = _lib().lb_sum_slices(_ptr(partials), _ptr(out), c_int(tokens), c_int(rows), c_int(slices), c_int(_TC_EPILOGUES[epilogue]), _stream())
    _done(code, "sum_slices")


def residual_add(x: torch.Tensor, delta: torch.Tensor | SlicedSum) -> None:
    """``x += delta`` on the 32-bit residual stream (a :class:`SlicedSum` is summed and rounded first)."""
    _check(x, "x", torch.float32)
    if isinstance(delta, SlicedSum):
        if delta.dtype != torch.bfloat16:
            raise KernelError("residual_add: a sliced sum is rounded to bfloat16")
        _sum_slices(delta.partials, x, "residual_add")
        return
    _check(delta, "delta")
    if x.shape != delta.shape:
        raise KernelError("residual_add: shapes differ")
    code = _lib().lb_residual_add(_ptr(x), _ptr(delta), c_longlong(x.numel()), c_int(dtype_code(delta.dtype)), _stream())
    _done(code, "residual_add")


def gather_rows(src: torch.Tensor, rows: torch.Tensor, out: torch.Tensor) -> None:
    _check(src, "src")
    _check(rows, "rows", torch.int32)
    _check(out, "out", src.dtype)
    dim = src.shape[-1]
    if out.shape[-1] != dim or rows.numel() < out.shape[0]:
        raise KernelError("gather_rows: shapes do not agree")
    code = _lib().lb_gather_rows(_ptr(src), _ptr(rows), _ptr(out), c_int(out.shape[0]), c_int(dim), c_int(src.element_size()), _stream())
    _done(code, "gather_rows")


def fill_slots(table: torch.Tensor, largest_bytes: int, slot: int, pattern: int = 0) -> None:
    """Fills slot ``slot`` of every per-request state tensor with the 32-bit ``pattern`` in one launch.
    ``table`` is int64 ``[states, 2]`` on the device: each state's base address and bytes per slot."""
    _check(table, "table", torch.int64)
    if table.dim() != 2 or table.shape[1] != 2:
        raise KernelError("fill_slots: table must be [states, 2]")
    if slot < 0:
        raise KernelError("fill_slots: negative slot")
    code = _lib().lb_fill_slots(_ptr(table), c_int(table.shape[0]), c_longlong(largest_bytes), c_int(slot), ctypes.c_uint(pattern & 0xFFFFFFFF), _stream())
    _done(code, "fill_slots")


def feed_tokens(token_ids: torch.Tensor, segment_start: torch.Tensor, segment_length: torch.Tensor, source: torch.Tensor,
                sampled: torch.Tensor, status: torch.Tensor | None = None) -> None:
    """Writes token ids that the step before sampled on the device into this step's ``token_ids``: the last
    token of segment ``s`` becomes ``sampled[source[s]]`` wherever ``source[s] >= 0``."""
    for name, tensor in (("token_ids", token_ids), ("segment_start", segment_start), ("segment_length", segment_length), ("source", source), ("sampled", sampled)):
        _check(tensor, name, torch.int32)
    segments = source.numel()
    if segment_start.numel() != segments or segment_length.numel() != segments:
        raise KernelError("feed_tokens: one start, length and source per segment")
    if status is not None:
        _check(status, "status", torch.int32)
    code = _lib().lb_feed_tokens(_ptr(token_ids), _ptr(segment_start), _ptr(segment_length), _ptr(source), _ptr(sampled), c_int(sampled.numel()),
                                 c_int(segments), _ptr(status), _stream())
    _done(code, "feed_tokens")


def gated_activation(fused: torch.Tensor, out: torch.Tensor, activation: str) -> None:
    """``out = up * act(gate)`` for ``fused = [up ; gate]`` along the last dimension."""
    _check(fused, "fused")
    _check(out, "out", fused.dtype)
    if activation not in _ACTIVATIONS:
        raise KernelError(f"unknown activation {activation!r}; known: {sorted(_ACTIVATIONS)}")
    tokens, hidden = out.shape
    if fused.shape != (tokens, 2 * hidden):
        raise KernelError("gated_activation: fused must be [tokens, 2 * hidden]")
    code = _lib().lb_gated_activation(_ptr(fused), _ptr(out), c_int(tokens), c_int(hidden), c_int(_ACTIVATIONS[activation]),
                                      c_int(dtype_code(out.dtype)), _stream())
    _done(code, "gated_activation")


# ----------------------------------------------------------------------------- attention
def _check_paged(k_pages: torch.Tensor, v_pages: torch.Tensor, block_table: torch.Tensor, num_groups: int, head_dim: int) -> tuple[int, int, int]:
    _check(k_pages, "k_pages")
    _check(v_pages, "v_pages", k_pages.dtype)
    _check(block_table, "block_table", torch.int32)
    if k_pages.dim() != 4 or k_pages.shape[2:] != (num_groups, head_dim):
        raise KernelError("the key cache must be [pages, page_size, groups, head_dim]")
    if v_pages.shape != (k_pages.shape[0], num_groups, head_dim, k_pages.shape[1]):
        raise KernelError("the value cache must be [pages, groups, head_dim, page_size] (values are stored transposed)")
    if block_table.dim() != 2:
        raise KernelError("block_table must be [segments, max_blocks]")
    return k_pages.shape[1], k_pages.shape[0], block_table.shape[1]


def qk_norm_rope_write(
    qkv: torch.Tensor,
    q_out: torch.Tensor,
    k_pages: torch.Tensor,
    v_pages: torch.Tensor,
    *,
    q_weight: torch.Tensor | None,
    k_weight: torch.Tensor | None,
    eps: float,
    scale_offset: float,
    inv_freq: torch.Tensor | None,
    rotary_dim: int,
    positions: torch.Tensor,
    token_segment: torch.Tensor,
    block_table: torch.Tensor,
    num_heads: int,
    num_groups: int,
    head_dim: int,
    write_kv: bool,
    status: torch.Tensor,
) -> None:
    """Splits ``qkv`` rows into heads, applies per-head norm and rotary embedding to queries and
    keys, writes queries to ``q_out`` and keys/values into their pages."""
    _check(qkv, "qkv")
    _check(q_out, "q_out", qkv.dtype)
    tokens = qkv.shape[0]
    if qkv.shape[1] != (num_heads + 2 * num_groups) * head_dim or q_out.numel() != tokens * num_heads * head_dim:
        raise KernelError("qk_norm_rope_write: qkv / q_out widths do not match the head counts")
    page_size, num_pages, max_blocks = _check_paged(k_pages, v_pages, block_table, num_groups, head_dim)
    if k_pages.dtype != qkv.dtype:
        raise KernelError("qk_norm_rope_write: cache and activations differ in type")
    if (q_weight is None) != (k_weight is None):
        raise KernelError("qk_norm_rope_write: give both norm weights or neither")
    for name, weight in (("q_weight", q_weight), ("k_weight", k_weight)):
        if weight is not None:
            _check(weight, name, torch.float32)
            if weight.numel() != head_dim:
                raise KernelError(f"{name} must have head_dim elements")
    if rotary_dim:
        if inv_freq is None:
            raise KernelError("qk_norm_rope_write: rotary_dim > 0 needs inv_freq")
        _check(inv_freq, "inv_freq", torch.float32)
        if inv_freq.numel() != rotary_dim // 2 or rotary_dim % 2 or rotary_dim > head_dim:
            raise KernelError("qk_norm_rope_write: inv_freq must have rotary_dim / 2 elements, rotary_dim even and <= head_dim")
    _check(positions, "positions", torch.int32)
    _check(token_segment, "token_segment", torch.int32)
    code = _lib().lb_qk_norm_rope_write(
        _ptr(qkv), _ptr(q_out), _ptr(k_pages), _ptr(v_pages), _ptr(q_weight), _ptr(k_weight), c_float(eps), c_float(scale_offset),
        _ptr(inv_freq), c_int(rotary_dim), _ptr(positions), _ptr(token_segment), _ptr(block_table), c_int(tokens), c_int(num_heads),
        c_int(num_groups), c_int(head_dim), c_int(page_size), c_int(num_pages), c_int(max_blocks), c_int(1 if write_kv else 0),
        c_int(dtype_code(qkv.dtype)), _ptr(status), _stream())
    _done(code, "qk_norm_rope_write")


def paged_attention_plain(
    q: torch.Tensor,
    k_pages: torch.Tensor,
    v_pages: torch.Tensor,
    out: torch.Tensor,
    *,
    positions: torch.Tensor,
    token_segment: torch.Tensor,
    block_table: torch.Tensor,
    num_heads: int,
    num_groups: int,
    head_dim: int,
    scale: float,
    window: int | None,
    status: torch.Tensor,
) -> None:
    """Causal (optionally windowed) attention of every token over its request's pages."""
    _check(q, "q")
    _check(out, "out", q.dtype)
    tokens = q.shape[0]
    if q.numel() != tokens * num_heads * head_dim or out.numel() != q.numel():
        raise KernelError("paged_attention: q / out sizes do not match the head counts")
    page_size, num_pages, max_blocks = _check_paged(k_pages, v_pages, block_table, num_groups, head_dim)
    if k_pages.dtype != q.dtype:
        raise KernelError("paged_attention: cache and queries differ in type")
    if head_dim > 512:
        raise KernelError(f"paged_attention: head_dim {head_dim} exceeds the supported 512")
    if num_heads % num_groups:
        raise KernelError("paged_attention: num_heads must be a multiple of num_groups")
    code = _lib().lb_paged_attention_plain(
        _ptr(q), _ptr(k_pages), _ptr(v_pages), _ptr(out), _ptr(positions), _ptr(token_segment), _ptr(block_table), c_int(tokens),
        c_int(num_heads), c_int(num_groups), c_int(head_dim), c_int(page_size), c_int(num_pages), c_int(max_blocks), c_float(scale),
        c_int(window if window else 0), c_int(dtype_code(q.dtype)), _ptr(status), _stream())
    _done(code, "paged_attention_plain")


DECODE_HEAD_DIMS = (16, 32, 48, 64, 80, 96, 112, 128)
_sm_counts: dict[int, int] = {}
_decode_ctas_per_sm: dict[tuple[int, int], int] = {}


def sm_count() -> int:
    """Multiprocessors of the current device (asked once per device)."""
    device = torch.cuda.current_device()
    if device not in _sm_counts:
        _sm_counts[device] = torch.cuda.get_device_properties(device).multi_processor_count
    return _sm_counts[device]


def decode_ctas_per_sm(head_dim: int) -> int:
    """CTAs of the split-key attention kernel an SM of the current device holds at this head size
    (the library asks the runtime; registers and the ring's shared memory decide)."""
    key = (torch.cuda.current_device(), head_dim)
    if key not in _decode_ctas_per_sm:
        _decode_ctas_per_sm[key] = max(1, int(_lib().lb_attention_decode_ctas_per_sm(c_int(head_dim))))
    return _decode_ctas_per_sm[key]


def decode_attention_supported(dtype: torch.dtype, head_dim: int, page_size: int) -> bool:
    return dtype == torch.bfloat16 and head_dim in DECODE_HEAD_DIMS and page_size % 16 == 0


def decode_attention_plan(tokens: int, num_heads: int, num_groups: int, max_context: int, window: int | None, head_dim: int = 64,
                          resident_ctas: int | None = None) -> tuple[int, int]:
    """``(splits, blocks_per_split)`` in 16-key blocks.  Depends on the batch's size and longest
    context only.  The grid has ``splits * pairs`` CTAs of four warps, of which the device holds
    ``resident_ctas`` to a round (default: its multiprocessors times three quarters of the CTAs each
    holds at this head size, rounded: measured, plans made for every resident CTA at once run 3 to
    9 % longer at batch 64, since the CTAs of a round do not start and end together); a CTA costs
    about six blocks' time beside the blocks each of its warps walks.  The number of splits that
    makes the fewest rounds' worth of that is taken, with at least eight blocks to a split."""
    span = min(max_context, window + 15) if window else max_context
    blocks_total = span // 16 + 1
    pairs = max(1, tokens * num_groups * -(-(num_heads // num_groups) // 16))
    slots = resident_ctas if resident_ctas is not None else sm_count() * ((3 * decode_ctas_per_sm(head_dim) + 2) // 4)
    best, best_cost = 1, None
    for splits in range(1, max(1, blocks_total // 8) + 1):
        per_warp = -(-(-(-blocks_total // splits)) // 4)
        cost = -(-pairs * splits // slots) * (per_warp + 6)
        if best_cost is None or cost < best_cost:
            best, best_cost = splits, cost
    blocks_per_split = -(-blocks_total // best)
    return -(-blocks_total // blocks_per_split), blocks_per_split


def attention_decode(
    q: torch.Tensor,
    k_pages: torch.Tensor,
    v_pages: torch.Tensor,
    out: torch.Tensor,
    *,
    positions: torch.Tensor,
    token_segment: torch.Tensor,
    block_table: torch.Tensor,
    num_heads: int,
    num_groups: int,
    head_dim: int,
    scale: float,
    window: int | None,
    max_context: int,
    status: torch.Tensor,
    scratch: torch.Tensor | None = None,
    token_list: torch.Tensor | None = None,
    num_listed: int | None = None,
    fresh_keys: int | None = None,
) -> None:
    """Split-key tensor-core attention for tokens that attend alone (bfloat16 only).  ``max_context``
    is the largest position + 1 in the batch; it sizes the grid.  ``token_list`` (its first
    ``num_listed`` entries) restricts the call to some tokens of the batch.  ``fresh_keys``: the kernel
    launched just before on this stream is :func:`qk_norm_rope_write` (which lets its successor start
    early) and writes at most that many of the newest positions each token sees; the attention then
    starts early and reads the older keys while that kernel runs.  ``None``: an ordinary launch."""
    _check(q, "q", torch.bfloat16)
    _check(out, "out", torch.bfloat16)
    if q.numel() != q.shape[0] * num_heads * head_dim or out.numel() != q.numel():
        raise KernelError("attention_decode: q / out sizes do not match the head counts")
    tokens = q.shape[0]
    if token_list is not None:
        _check(token_list, "token_list", torch.int32)
        tokens = token_list.numel() if num_listed is None else num_listed
        if tokens > token_list.numel():
            raise KernelError("attention_decode: token_list is shorter than num_listed")
    page_size, num_pages, max_blocks = _check_paged(k_pages, v_pages, block_table, num_groups, head_dim)
    if k_pages.dtype != torch.bfloat16:
        raise KernelError("attention_decode: the cache must be bfloat16")
    if not decode_attention_supported(q.dtype, head_dim, page_size):
        raise KernelError(f"attention_decode: head_dim {head_dim} (supported: {DECODE_HEAD_DIMS}) or page_size {page_size} (a multiple of 16) is not supported")
    if num_heads % num_groups:
        raise KernelError("attention_decode: num_heads must be a multiple of num_groups")
    splits, blocks_per_split = decode_attention_plan(tokens, num_heads, num_groups, max_context, window, head_dim)
    needed = tokens * num_heads * splits * (head_dim + 2)
    if scratch is None:
        scratch = torch.empty(needed, dtype=torch.float32, device=q.device)
    else:
        _check(scratch, "scratch", torch.float32)
        if scratch.numel() < needed:
            raise KernelError(f"attention_decode: scratch holds {scratch.numel()} floats, {needed} are needed")
    code = _lib().lb_attention_decode(
        _ptr(q), _ptr(k_pages), _ptr(v_pages), _ptr(out), _ptr(scratch), _ptr(positions), _ptr(token_segment), _ptr(block_table),
        _ptr(token_list), c_int(tokens), c_int(num_heads), c_int(num_groups), c_int(head_dim), c_int(page_size), c_int(num_pages), c_int(max_blocks),
        c_float(scale), c_int(window if window else 0), c_int(splits), c_int(blocks_per_split), c_int(-1 if fresh_keys is None else fresh_keys),
        _ptr(status), _stream())
    _done(code, "attention_decode", 2 if splits > 1 else 1)   # the kernel and the merge of its splits


PREFILL_TILE = 32
PREFILL_MAX_HEADS_PER_CTA = 8


def prefill_attention_supported(dtype: torch.dtype, num_heads: int, num_groups: int, head_dim: int, page_size: int) -> bool:
    heads_per_group = num_heads // max(num_groups, 1)
    chunks = -(-heads_per_group // PREFILL_MAX_HEADS_PER_CTA)
    return decode_attention_supported(dtype, head_dim, page_size) and heads_per_group % chunks == 0


def attention_prefill(
    q: torch.Tensor,
    k_pages: torch.Tensor,
    v_pages: torch.Tensor,
    out: torch.Tensor,
    *,
    tiles: torch.Tensor,
    num_tiles: int,
    positions: torch.Tensor,
    token_segment: torch.Tensor,
    block_table: torch.Tensor,
    num_heads: int,
    num_groups: int,
    head_dim: int,
    scale: float,
    window: int | None,
    status: torch.Tensor,
    kernel: str | None = None,
    split_tiles: int = 0,
) -> None:
    """Tensor-core attention for portions of prompts (bfloat16 only).  ``tiles`` is ``[num_tiles, 2]``:
    first token and count (at most 32) of runs of consecutive tokens of one request.  Head size 64 runs
    on the tcgen05 kernel (scores and output in tensor memory), the other sizes on the ``mma.sync``
    one; ``kernel="mma"`` or ``"tcgen05"`` forces one of them.  ``split_tiles`` > 1 (tcgen05 kernel only):
    a tile that sees at least that many tiles of 64 keys is worked on by two CTAs, half of the keys each,
    for launches of few tiles that the longest tile's chain of keys would bound."""
    _check(q, "q", torch.bfloat16)
    _check(out, "out", torch.bfloat16)
    _check(tiles, "tiles", torch.int32)
    if q.numel() != q.shape[0] * num_heads * head_dim or out.numel() != q.numel():
        raise KernelError("attention_prefill: q / out sizes do not match the head counts")
    if tiles.numel() < 2 * num_tiles:
        raise KernelError("attention_prefill: fewer tile records than num_tiles")
    page_size, num_pages, max_blocks = _check_paged(k_pages, v_pages, block_table, num_groups, head_dim)
    if not prefill_attention_supported(k_pages.dtype, num_heads, num_groups, head_dim, page_size):
        raise KernelError(f"attention_prefill: head_dim {head_dim} (supported: {DECODE_HEAD_DIMS}), page_size {page_size} (a multiple of 16) "
                          f"or {num_heads} heads over {num_groups} groups is not supported")
    if kernel not in (None, "mma", "tcgen05"):
        raise KernelError(f"attention_prefill: unknown kernel {kernel!r}")
    takes_tcgen05 = head_dim == 64 and num_heads // num_groups <= 128
    if kernel == "tcgen05" and not takes_tcgen05:
        raise KernelError(f"attention_prefill: the tcgen05 kernel takes head size 64 and up to 128 query heads per K/V head, not {head_dim} and {num_heads // num_groups}")
    if kernel == "tcgen05" or (kernel is None and takes_tcgen05 and USE_TCGEN05_ATTENTION):
        code = _lib().lb_attention_prefill_tcgen05(
            _ptr(q), _ptr(k_pages), _ptr(v_pages), _ptr(out), _ptr(tiles), c_int(num_tiles), c_int(q.shape[0]), _ptr(positions), _ptr(token_segment),
            _ptr(block_table), c_int(num_heads), c_int(num_groups), c_int(head_dim), c_int(page_size), c_int(num_pages), c_int(max_blocks),
            c_float(scale), c_int(window if window else 0), c_int(split_tiles), _ptr(status), _stream())
        if code == -5:
            raise KernelError("attention_prefill: the driver made no tensor map for these tensors")
        _done(code, "attention_prefill (tcgen05)")
        return
    code = _lib().lb_attention_prefill(
        _ptr(q), _ptr(k_pages), _ptr(v_pages), _ptr(out), _ptr(tiles), c_int(num_tiles), _ptr(positions), _ptr(token_segment), _ptr(block_table),
        c_int(num_heads), c_int(num_groups), c_int(head_dim), c_int(page_size), c_int(num_pages), c_int(max_blocks), c_float(scale),
        c_int(window if window else 0), _ptr(status), _stream())
    _done(code, "attention_prefill")


# ---------------------------------------------------------------------------- short conv
def short_conv(
    proj: torch.Tensor | SlicedSum,
    state: torch.Tensor,
    weight: torch.Tensor,
    bias: torch.Tensor | None,
    out: torch.Tensor,
    *,
    token_segment: torch.Tensor,
    segment_start: torch.Tensor,
    segment_length: torch.Tensor,
    segment_slot: torch.Tensor,
    segments: int,
    status: torch.Tensor,
) -> None:
    """Gated depthwise causal convolution of every portion, reading and updating each request's
    state slot (``state`` is ``[slots, kernel_size - 1, dim]``).  ``proj`` may be a :class:`SlicedSum`
    (the in-projection left in its K slices): a step of single tokens adds them in the convolution's own
    kernel, any other step sums them first."""
    _check(out, "out")
    _check(weight, "weight", torch.float32)
    tokens, dim = out.shape
    kernel_size = weight.shape[1]
    single_tokens = segments == tokens and out.dtype == torch.bfloat16 and dim % 8 == 0 and dim >= 8
    if isinstance(proj, SlicedSum):
        if proj.dtype != out.dtype:
            raise KernelError("short_conv: the sliced in-projection is rounded to another type than out's")
        if not single_tokens:
            proj = proj.sum()
    sliced = isinstance(proj, SlicedSum)
    if sliced:
        _check(proj.partials, "proj.partials", torch.float32)
    else:
        _check(proj, "proj", out.dtype)
    if tuple(proj.shape) != (tokens, 3 * dim) or weight.shape[0] != dim:
        raise KernelError("short_conv: proj must be [tokens, 3 * dim] and weight [dim, kernel_size]")
    if kernel_size > 1:
        _check(state, "state", out.dtype)
        if state.dim() != 3 or state.shape[1:] != (kernel_size - 1, dim):
            raise KernelError("short_conv: state must be [slots, kernel_size - 1, dim]")
    if bias is not None:
        _check(bias, "bias", torch.float32)
        if bias.numel() != dim:
            raise KernelError("short_conv: bias must have dim elements")
    if single_tokens:
        # every portion is one token: one kernel for the slices' sum, the convolution and the state
        code = _lib().lb_short_conv_single(
            _ptr(proj.partials if sliced else None), c_int(proj.partials.shape[0] if sliced else 0), _ptr(None if sliced else proj), _ptr(state), _ptr(weight),
            _ptr(bias), _ptr(out), _ptr(token_segment), _ptr(segment_slot), c_int(tokens), c_int(dim), c_int(kernel_size), c_int(state.shape[0]), _ptr(status),
            _stream())
        _done(code, "short_conv_single")
        return
    code = _lib().lb_short_conv(
        _ptr(proj), _ptr(state), _ptr(weight), _ptr(bias), _ptr(out), _ptr(token_segment), _ptr(segment_start), _ptr(segment_length),
        _ptr(segment_slot), c_int(tokens), c_int(segments), c_int(dim), c_int(kernel_size), c_int(state.shape[0]),
        c_int(dtype_code(proj.dtype)), _ptr(status), _stream())
    _done(code, "short_conv", 2 if kernel_size > 1 else 1)


# ------------------------------------------------------------------------------ sampling
SAMPLE_PARAM_WORDS = 27


def sample(logits: torch.Tensor, work: torch.Tensor, counts: torch.Tensor | None, params: torch.Tensor, out_tokens: torch.Tensor) -> None:
    _check(logits, "logits", torch.float32)
    _check(work, "work", torch.float32)
    _check(params, "params", torch.int32)
    _check(out_tokens, "out_tokens", torch.int32)
    rows, vocab = logits.shape
    if work.numel() < rows * vocab or params.shape != (rows, SAMPLE_PARAM_WORDS) or out_tokens.numel() < rows:
        raise KernelError("sample: work, params or out_tokens are too small for the logits")
    if counts is not None:
        _check(counts, "counts", torch.int32)
        if counts.shape[1] != vocab:
            raise KernelError("sample: counts must be [slots, vocab]")
    lib = _lib()
    if lib.lb_sample_params_size() != 4 * SAMPLE_PARAM_WORDS:
        raise KernelError("sample: parameter record sizes of the library and the bindings differ")
    code = lib.lb_sample(_ptr(logits), _ptr(work), _ptr(counts), _ptr(params), _ptr(out_tokens), c_int(rows), c_int(vocab), _stream())
    _done(code, "sample")


def argmax(logits: torch.Tensor, out_tokens: torch.Tensor) -> None:
    _check(logits, "logits", torch.float32)
    _check(out_tokens, "out_tokens", torch.int32)
    rows, vocab = logits.shape
    if out_tokens.numel() < rows:
        raise KernelError("argmax: out_tokens is too small")
    if vocab >= 8192 and rows <= 256:
        # Few long rows: spread each over many blocks.
        chunks = max(2, min(64, vocab // 2048))
        scratch = torch.empty(2 * rows * chunks, dtype=torch.float32, device=logits.device)
        code = _lib().lb_argmax_chunked(_ptr(logits), _ptr(scratch), _ptr(out_tokens), c_int(rows), c_int(vocab), c_int(chunks), _stream())
        _done(code, "argmax", 2)
        return
    code = _lib().lb_argmax(_ptr(logits), _ptr(out_tokens), c_int(rows), c_int(vocab), _stream())
    _done(code, "argmax")


def update_counts(counts: torch.Tensor, slots: torch.Tensor, add: torch.Tensor, remove: torch.Tensor) -> None:
    _check(counts, "counts", torch.int32)
    for name, tensor in (("slots", slots), ("add", add), ("remove", remove)):
        _check(tensor, name, torch.int32)
    rows = slots.numel()
    if add.numel() != rows or remove.numel() != rows:
        raise KernelError("update_counts: slots, add and remove differ in length")
    code = _lib().lb_update_counts(_ptr(counts), _ptr(slots), _ptr(add), _ptr(remove), c_int(rows), c_int(counts.shape[1]), _stream())
    _done(code, "update_counts")


# --------------------------------------------------------------------------------- linear
def configure_matmul_precision() -> None:
    """Makes library float32 products true 32-bit (no TF32, no reduced-precision reductions)."""
    torch.backends.cuda.matmul.allow_tf32 = False
    torch.backends.cudnn.allow_tf32 = False
    torch.backends.cuda.matmul.allow_bf16_reduced_precision_reduction = False
    torch.set_float32_matmul_precision("highest")


_SKINNY_EPILOGUES = {"store": 0, "store_float": 1, "residual_add": 2, "gated": 3, "short_conv": 4}
SKINNY_MAX_TOKENS = 16


def skinny_supported(x: torch.Tensor, rows: int) -> bool:
    """Whether the weight-streaming kernel takes this product: bfloat16, 1..16 tokens, an input width
    that is a multiple of 32 and a multiple of 8 output rows."""
    return (
        x.dtype == torch.bfloat16
        and x.dim() == 2
        and 1 <= x.shape[0] <= SKINNY_MAX_TOKENS
        and x.shape[1] % 32 == 0
        and x.shape[1] >= 32
        and rows % 8 == 0
        and rows > 0
    )


def _skinny(x: torch.Tensor, weight: torch.Tensor, out: torch.Tensor, n: int, epilogue: str, activation: str = "identity", conv: dict | None = None,
            prefetch: bool = True) -> None:
    """``prefetch``: the kernel asks for its weights towards L2 before it waits for the kernel before it; off where
    that kernel does not let it start early (see :func:`successor_starts_early`)."""
    conv = conv or {}
    code = _lib().lb_gemm_skinny(
        _ptr(x), _ptr(weight), _ptr(out), c_int(x.shape[0]), c_int(x.shape[1]), c_int(n), c_int(_SKINNY_EPILOGUES[epilogue]),
        c_int(_ACTIVATIONS[activation]), _ptr(conv.get("state")), _ptr(conv.get("weight")), _ptr(conv.get("bias")), _ptr(conv.get("token_segment")),
        _ptr(conv.get("segment_start")), _ptr(conv.get("segment_length")), _ptr(conv.get("segment_slot")), c_int(conv.get("segments", 0)),
        c_int(conv.get("taps", 0)), c_int(conv.get("num_slots", 0)), c_int(1 if prefetch else 0), _ptr(conv.get("status")), _stream())
    _done(code, f"gemm_skinny[{epilogue}]")


# Products of more than 16 tokens run on the tcgen05 kernel when this is on (LALAMO_B200_TCGEN05=0
# sends them to the library instead).
USE_TCGEN05 = os.environ.get("LALAMO_B200_TCGEN05", "1") != "0"
# Prefill attention with head size 64 runs on the tcgen05 kernel when this is on
# (LALAMO_B200_TCGEN05_ATTENTION=0 keeps it on the mma.sync kernel).
USE_TCGEN05_ATTENTION = os.environ.get("LALAMO_B200_TCGEN05_ATTENTION", "1") != "0"
# With at most 16 tokens, products of at least this many rows of W fill the GPU with 128-row tiles and
# stream faster through the TMA pipeline than through the register-direct kernel.
TCGEN05_MIN_ROWS_FEW_TOKENS = 16384
_TC_EPILOGUES = {"store": 0, "store_float": 1, "residual_add": 2, "gated": 4}
_tc_scratch: dict[int, torch.Tensor] = {}
_tc_retired: list[torch.Tensor] = []  # outgrown scratch buffers, kept: a recorded graph may hold their address
# Products cut into K slices hand their partial sums to the next norm instead of summing them in a launch of their own
# (LALAMO_B200_DEFER_SLICE_SUMS=0 sums at once).
DEFER_SLICE_SUMS = os.environ.get("LALAMO_B200_DEFER_SLICE_SUMS", "1") != "0"


def tcgen05_supported(x: torch.Tensor, rows: int) -> bool:
    """Whether the tcgen05 kernel takes this product: bfloat16, rows of 16-byte multiples."""
    return x.dtype == torch.bfloat16 and x.dim() == 2 and x.shape[0] >= 1 and x.shape[1] % 8 == 0 and x.shape[1] >= 8 and rows >= 1


def tcgen05_slices(tokens: int, rows: int, width: int, sms: int | None = None) -> int:
    """K slices for a product whose tiles alone would leave most of the multiprocessors idle."""
    blocks = -(-width // 64)
    sms = sms or sm_count()
    if tokens > 128:
        # The walking kernel with tiles of 128 rows x 256 tokens: slices until the tiles fill the SMs, of at least 16
        # blocks each.  Measured against one slice: 1024 x 4608 at 2,048 tokens 22.6 against 28.5 us, at 512 tokens 14.0
        # against 25.5; 2048 x 8192 at 512 tokens 21.5 against 43.2, at 1,024 tokens 33.6 against 46.7; 1024 x 1024 at
        # 2,048 tokens (16 blocks in all) 12.5 against 9.8, hence the floor.
        tiles = -(-rows // 128) * -(-tokens // 256)
        return max(1, min(sms // tiles, blocks // 16, 12))
    tile = 32 if tokens <= 32 else 64 if tokens <= 64 else 128
    ctas = -(-rows // 128) * -(-tokens // tile)
    if ctas >= 96 or blocks < 8:
        return 1
    # more than a dozen slices cost more in partial sums than they gain in CTAs (1024 x 4608 at 64 tokens: 8.7 us with 12,
    # 9.4 with 18)
    return max(1, min(-(-sms // ctas), blocks // 4, 12))


def _settled_slices(slices: int, width: int) -> int:
    """The number of K slices the kernel makes of ``slices`` asked for (whole blocks of 64 columns each)."""
    blocks = -(-width // 64)
    slices = max(1, min(slices, blocks))
    per_slice = -(-blocks // slices)
    return -(-blocks // per_slice)


def linear_tcgen05(x: torch.Tensor, weight: torch.Tensor, epilogue: str = "store", residual: torch.Tensor | None = None,
                   slices: int | None = None, activation: str = "identity", status: torch.Tensor | None = None,
                   defer_sum: bool = False) -> torch.Tensor | SlicedSum:
    """``x @ weight.T`` on the tcgen05 tensor cores.  ``epilogue``: ``"store"`` (bfloat16),
    ``"store_float"``, ``"residual_add"`` (into ``residual``, float32, which is returned) or ``"gated"``
    (``weight`` is ``[up ; gate]``, the result ``up * activation(gate)`` of half as many columns).
    ``status``: the int32 word in which the kernel reports a wait that gave up.  ``defer_sum``: if the
    product is cut into K slices, return them as a :class:`SlicedSum` (nothing is stored or added) for a
    consumer that adds them itself."""
    if status is not None:
        _check(status, "status", torch.int32)
    _check(x, "x", torch.bfloat16)
    _check(weight, "weight", torch.bfloat16)
    tokens, width = x.shape
    rows = weight.shape[0]
    if weight.shape[1] != width or not tcgen05_supported(x, rows):
        raise KernelError(f"linear_tcgen05: a [{tokens}, {width}] x [{rows}, {weight.shape[1]}] product is not supported (widths must agree and be multiples of 8)")
    if epilogue == "residual_add":
        if residual is None:
            raise KernelError("linear_tcgen05: residual_add needs the residual stream")
        _check(residual, "residual", torch.float32)
        if residual.shape != (tokens, rows):
            raise KernelError("linear_tcgen05: residual must be [tokens, rows]")
        out = residual
    elif epilogue == "gated":
        if rows % 2 or activation not in _ACTIVATIONS:
            raise KernelError("linear_tcgen05: gated needs an even number of rows and a known activation")
        out = torch.empty(tokens, rows // 2, dtype=torch.bfloat16, device=x.device)
        slices = 1
    else:
        out = torch.empty(tokens, rows, dtype=torch.float32 if epilogue == "store_float" else torch.bfloat16, device=x.device)
    slices = tcgen05_slices(tokens, rows, width) if slices is None else slices
    slices = 1 if epilogue == "gated" else _settled_slices(slices, width)
    deferred = defer_sum and slices > 1 and epilogue in ("store", "residual_add")
    scratch = None
    if deferred:
        scratch = torch.empty(slices, tokens, rows, dtype=torch.float32, device=x.device)
    elif slices > 1:
        needed = slices * tokens * rows
        index = x.device.index if x.device.index is not None else torch.cuda.current_device()
        if index not in _tc_scratch or _tc_scratch[index].numel() < needed:
            if index in _tc_scratch:
                _tc_retired.append(_tc_scratch[index])  # recorded graphs may still write there
            _tc_scratch[index] = torch.empty(max(needed, 1 << 22), dtype=torch.float32, device=x.device)
        scratch = _tc_scratch[index]
    code = _lib().lb_gemm_tcgen05(_ptr(x), _ptr(weight), _ptr(out), _ptr(scratch), c_longlong(scratch.numel() if scratch is not None else 0),
                                  c_int(tokens), c_int(width), c_int(rows), c_int(_TC_EPILOGUES[epilogue]), c_int(_ACTIVATIONS[activation]), c_int(slices),
                                  c_int(1 if deferred else 0), _ptr(status), _stream())
    if code == -5:
        raise KernelError("linear_tcgen05: the driver gave no tensor map (cuTensorMapEncodeTiled)")
    _done(code, "gemm_tcgen05", 2 if slices > 1 and not deferred else 1)
    if deferred:
        return SlicedSum(scratch, torch.bfloat16)
    return out


def tcgen05_wait_probe(status: torch.Tensor, nanoseconds: int = 1_000_000) -> None:
    """Lets the tcgen05 kernels' bounded barrier wait run out on a barrier that nothing completes
    (after ``nanoseconds``, at most 0.1 s) and report it in ``status``, as a product would whose
    copy or arrival got lost."""
    _check(status, "status", torch.int32)
    _done(_lib().lb_tcgen05_wait_probe(_ptr(status), c_longlong(nanoseconds), _stream()), "tcgen05_wait_probe")


def linear(x: torch.Tensor, weight: torch.Tensor, out_dtype: torch.dtype | None = None, status: torch.Tensor | None = None) -> torch.Tensor:
    """``x @ weight.T`` with 32-bit accumulation; ``out_dtype`` float32 gives 32-bit results from
    bfloat16 operands (the LM head's logits).  Steps of up to 16 tokens go to the weight-streaming
    kernel, everything else to the library."""
    _check(x, "x")
    _check(weight, "weight", x.dtype)
    if x.shape[-1] != weight.shape[1]:
        raise KernelError(f"linear: input width {x.shape[-1]} does not match the weight's {weight.shape[1]}")
    wants_float = out_dtype is not None and out_dtype != x.dtype
    if USE_TCGEN05 and x.shape[0] <= SKINNY_MAX_TOKENS and weight.shape[0] >= TCGEN05_MIN_ROWS_FEW_TOKENS and tcgen05_supported(x, weight.shape[0]):
        return linear_tcgen05(x, weight, "store_float" if wants_float else "store", slices=1, status=status)
    if skinny_supported(x, weight.shape[0]):
        out = torch.empty(x.shape[0], weight.shape[0], dtype=torch.float32 if wants_float else x.dtype, device=x.device)
        _skinny(x, weight, out, weight.shape[0], "store_float" if wants_float else "store")
        return out
    if USE_TCGEN05 and tcgen05_supported(x, weight.shape[0]):
        return linear_tcgen05(x, weight, "store_float" if wants_float else "store", status=status)
    if wants_float:
        return torch.mm(x, weight.t(), out_dtype=out_dtype)
    return torch.mm(x, weight.t())


def gated_linear_starts_successor_early(tokens: int, rows: int, width: int) -> bool:
    """Whether the kernel :func:`gated_linear` runs for these sizes lets the kernel after it start before it has
    finished (the weight-streaming kernel does; the TMA kernel only with more than 16 tokens): a successor that
    cannot start early has nothing to gain from asking for its weights before it waits."""
    on_tcgen05 = USE_TCGEN05 and tokens <= SKINNY_MAX_TOKENS and rows >= TCGEN05_MIN_ROWS_FEW_TOKENS and width % 8 == 0
    return not on_tcgen05


def linear_accumulate(x: torch.Tensor, weight: torch.Tensor, residual: torch.Tensor, status: torch.Tensor | None = None,
                      started_early: bool = True) -> torch.Tensor | SlicedSum | None:
    """``residual += x @ weight.T`` (the product rounded to the activation type first) when the fused
    kernel takes the product: returns ``None``.  Otherwise returns the product, not yet added: a tensor,
    or a :class:`SlicedSum` when the product was cut into K slices (the norm that follows adds them).
    ``started_early=False``: the kernel before this one does not let its successor start early."""
    _check(x, "x")
    _check(weight, "weight", x.dtype)
    _check(residual, "residual", torch.float32)
    if x.shape[-1] != weight.shape[1] or residual.shape != (x.shape[0], weight.shape[0]):
        raise KernelError("linear_accumulate: shapes of x, weight and residual do not agree")
    if skinny_supported(x, weight.shape[0]):
        _skinny(x, weight, residual, weight.shape[0], "residual_add", prefetch=started_early)
        return None
    if USE_TCGEN05 and tcgen05_supported(x, weight.shape[0]):
        result = linear_tcgen05(x, weight, "residual_add", residual, status=status, defer_sum=DEFER_SLICE_SUMS)
        return result if isinstance(result, SlicedSum) else None
    return torch.mm(x, weight.t())


def gated_linear(x: torch.Tensor, up_gate: torch.Tensor, activation: str, status: torch.Tensor | None = None) -> torch.Tensor:
    """``up * act(gate)`` for ``[up ; gate] = x @ up_gate.T`` (``up_gate``: ``[2 * hidden, width]``)."""
    _check(x, "x")
    _check(up_gate, "up_gate", x.dtype)
    if activation not in _ACTIVATIONS:
        raise KernelError(f"unknown activation {activation!r}; known: {sorted(_ACTIVATIONS)}")
    hidden = up_gate.shape[0] // 2
    if x.shape[-1] != up_gate.shape[1] or up_gate.shape[0] != 2 * hidden:
        raise KernelError("gated_linear: shapes of x and up_gate do not agree")
    if USE_TCGEN05 and x.shape[0] <= SKINNY_MAX_TOKENS and up_gate.shape[0] >= TCGEN05_MIN_ROWS_FEW_TOKENS and tcgen05_supported(x, up_gate.shape[0]):
        return linear_tcgen05(x, up_gate, "gated", activation=activation, status=status)
    out = torch.empty(x.shape[0], hidden, dtype=x.dtype, device=x.device)
    if skinny_supported(x, hidden):
        _skinny(x, up_gate, out, hidden, "gated", activation)
        return out
    if USE_TCGEN05 and tcgen05_supported(x, up_gate.shape[0]):
        return linear_tcgen05(x, up_gate, "gated", activation=activation, status=status)
    gated_activation(linear(x, up_gate, status=status), out, activation)
    return out


def short_conv_linear(
    x: torch.Tensor,
    in_proj: torch.Tensor,
    state: torch.Tensor,
    weight: torch.Tensor,
    bias: torch.Tensor | None,
    *,
    token_segment: torch.Tensor,
    segment_start: torch.Tensor,
    segment_length: torch.Tensor,
    segment_slot: torch.Tensor,
    segments: int,
    status: torch.Tensor,
) -> torch.Tensor:
    """The in-projection and the gated short convolution (with its state update) in one:
    ``in_proj`` is ``[3 * dim, width]`` with row blocks (B, C, x)."""
    _check(x, "x")
    _check(in_proj, "in_proj", x.dtype)
    dim = in_proj.shape[0] // 3
    if x.shape[-1] != in_proj.shape[1] or in_proj.shape[0] != 3 * dim:
        raise KernelError("short_conv_linear: shapes of x and in_proj do not agree")
    out = torch.empty(x.shape[0], dim, dtype=x.dtype, device=x.device)
    taps = weight.shape[1]
    if skinny_supported(x, dim) and segments <= x.shape[0]:
        _check(weight, "weight", torch.float32)
        if weight.shape[0] != dim:
            raise KernelError("short_conv_linear: weight must be [dim, taps]")
        if taps > 1:
            _check(state, "state", x.dtype)
            if state.dim() != 3 or state.shape[1:] != (taps - 1, dim):
                raise KernelError("short_conv_linear: state must be [slots, taps - 1, dim]")
        if bias is not None:
            _check(bias, "bias", torch.float32)
        _skinny(x, in_proj, out, dim, "short_conv", conv=dict(
            state=state, weight=weight, bias=bias, token_segment=token_segment, segment_start=segment_start, segment_length=segment_length,
            segment_slot=segment_slot, segments=segments, taps=taps, num_slots=state.shape[0], status=status))
        return out
    if segments == x.shape[0] and x.dtype == torch.bfloat16 and dim % 8 == 0 and USE_TCGEN05 and not skinny_supported(x, dim) and tcgen05_supported(x, in_proj.shape[0]):
        # a step of single tokens: the product's K slices, if it has any, are added by the convolution's kernel
        proj = linear_tcgen05(x, in_proj, "store", status=status, defer_sum=DEFER_SLICE_SUMS)
    else:
        proj = linear(x, in_proj, status=status)
    short_conv(proj, state, weight, bias, out, token_segment=token_segment, segment_start=segment_start,
               segment_length=segment_length, segment_slot=segment_slot, segments=segments, status=status)
    return out
