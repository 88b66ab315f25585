"""Tensor-level wrappers of the kernel entry points.

Each function checks what the kernel cannot check itself (device, dtype, contiguity, shapes),
launches on torch's current CUDA stream and raises :class:`KernelError` on a refusal.  There
is no CPU path: a tensor that is not on a CUDA device is an error.
"""
from __future__ import annotations

from typing import Optional

import torch

from .library import KernelError, check, kernel

F32, BF16 = 0, 1
_DTYPE_CODE = {torch.float32: F32, torch.bfloat16: BF16}

MASK_FULL, MASK_CHUNK, MASK_WINDOW = 0, 1, 2
ROPE_NONE, ROPE_INTERLEAVED, ROPE_HALVES = 0, 1, 2


def dtype_code(dtype: torch.dtype) -> int:
    try:
        return _DTYPE_CODE[dtype]
    except KeyError:
        raise KernelError(f"dtype {dtype} is not supported by the kernels (float32 and bfloat16 are)") from None


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def _ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    return None if t is None else t.data_ptr()


def _need(t: torch.Tensor, name: str, dtype=None) -> None:
    if not t.is_cuda:
        raise KernelError(f"{name} must be a CUDA tensor (the engine has no CPU path); found device {t.device}")
    if not t.is_contiguous():
        raise KernelError(f"{name} must be contiguous")
    if dtype is not None and t.dtype != dtype:
        raise KernelError(f"{name} must have dtype {dtype}, found {t.dtype}")


# ---------------------------------------------------------------------------------------
def embed_gather(ids: torch.Tensor, table: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``out[t] = table[ids[t]]`` as fp32.  ``ids`` int32 [T], ``table`` [V, H] fp32 or bf16."""
    _need(ids, "ids", torch.int32)
    _need(table, "table")
    T, (V, H) = ids.numel(), table.shape
    if out is None:
        out = torch.empty((T, H), dtype=torch.float32, device=table.device)
    _need(out, "out", torch.float32)
    check(kernel("sharpi_embed_gather")(ids.data_ptr(), table.data_ptr(), dtype_code(table.dtype), out.data_ptr(),
                                        T, H, V, _stream()), "sharpi_embed_gather")
    return out


def add_rmsnorm(x: torch.Tensor, delta: Optional[torch.Tensor], weight: torch.Tensor, eps: float,
                out_dtype: torch.dtype, *, rows: Optional[torch.Tensor] = None, want_fp32: bool = False,
                out: Optional[torch.Tensor] = None, out32: Optional[torch.Tensor] = None):
    """Residual add fused with RMSNorm.

    Without ``rows``: ``x += delta`` in place (when ``delta`` is given) and the norm of every
    row is returned.  With ``rows`` (int32 indices): the norm of ``x[rows] + delta[rows]``, and
    ``x`` stays as it is.  Returns ``(out, out32)``; ``out32`` is the unrounded fp32 copy when
    ``want_fp32`` (or ``out32``) is given, else ``None``.
    """
    _need(x, "x", torch.float32)
    if weight is not None:                  # None: the weightless norm
        _need(weight, "weight", torch.float32)
    H = x.shape[-1]
    if delta is not None:
        _need(delta, "delta", torch.float32)
        if delta.shape != x.shape:
            raise KernelError(f"delta shape {tuple(delta.shape)} differs from x shape {tuple(x.shape)}")
    if rows is not None:
        _need(rows, "rows", torch.int32)
        T = rows.numel()
    else:
        T = x.numel() // H
    if out is None:
        out = torch.empty((T, H), dtype=out_dtype, device=x.device)
    if want_fp32 and out32 is None:
        out32 = out if out_dtype == torch.float32 else torch.empty((T, H), dtype=torch.float32, device=x.device)
    alias = out32 is not None and out32.data_ptr() == out.data_ptr()
    check(kernel("sharpi_add_rmsnorm")(x.data_ptr(), _ptr(delta), _ptr(weight), float(eps), _ptr(rows), T, H,
                                       out.data_ptr(), dtype_code(out.dtype), None if alias else _ptr(out32),
                                       _stream()), "sharpi_add_rmsnorm")
    return out, out32


def swiglu(gate_up: torch.Tensor, out_dtype: torch.dtype, *, row_scale: Optional[torch.Tensor] = None,
           scale_rows: Optional[torch.Tensor] = None, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``silu(s g) * (s u)`` over a fused ``[M, 2I]`` gate|up product (fp32 in)."""
    _need(gate_up, "gate_up", torch.float32)
    M, I2 = gate_up.shape
    I = I2 // 2
    if out is None:
        out = torch.empty((M, I), dtype=out_dtype, device=gate_up.device)
    check(kernel("sharpi_swiglu")(gate_up.data_ptr(), _ptr(row_scale), _ptr(scale_rows), out.data_ptr(),
                                  dtype_code(out.dtype), M, I, _stream()), "sharpi_swiglu")
    return out


def timestamp(slots: torch.Tensor, index: int) -> None:
    """Write the GPU's nanosecond clock into ``slots[index]`` (int64) at this point of the current stream."""
    _need(slots, "slots", torch.int64)
    if not 0 <= index < slots.numel():
        raise KernelError(f"timestamp slot {index} outside 0 .. {slots.numel() - 1}")
    check(kernel("sharpi_timestamp")(slots.data_ptr(), index, _stream()), "sharpi_timestamp")


def add_bias(y: torch.Tensor, bias: torch.Tensor) -> torch.Tensor:
    """``y[m, :] += bias`` in place (float32)."""
    _need(y, "y", torch.float32)
    _need(bias, "bias", torch.float32)
    M, N = y.shape
    if bias.numel() != N:
        raise KernelError(f"bias has {bias.numel()} entries, the rows have {N}")
    check(kernel("sharpi_add_bias")(y.data_ptr(), bias.data_ptr(), M, N, _stream()), "sharpi_add_bias")
    return y


def add(a: torch.Tensor, b: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    _need(a, "a", torch.float32)
    _need(b, "b", torch.float32)
    if out is None:
        out = torch.empty_like(a)
    check(kernel("sharpi_add")(a.data_ptr(), b.data_ptr(), out.data_ptr(), a.numel(), _stream()), "sharpi_add")
    return out


def qkv_post(qkv: torch.Tensor, positions: torch.Tensor, row_req: torch.Tensor, block_table: torch.Tensor,
             inv_freq: Optional[torch.Tensor], q_out: torch.Tensor, kv_layer: torch.Tensor, *, nq: int, nkv: int,
             d: int, page_size: int, pairing: int, l2_eps: float, temp_attn_scale: float, temp_floor_scale: float,
             write_kv: bool) -> None:
    """RoPE, per-head L2 norm, temperature factor, q store and K/V scatter into pages.

    ``qkv`` fp32 [T, (nq + 2 nkv) d]; ``kv_layer`` is one layer's pages
    ``[pages, 2, nkv, page_size, d]`` in the dtype of ``q_out``; ``l2_eps < 0`` and
    ``temp_floor_scale <= 0`` switch the norm and the temperature factor off.
    """
    _need(qkv, "qkv", torch.float32)
    _need(positions, "positions", torch.int32)
    _need(row_req, "row_req", torch.int32)
    _need(block_table, "block_table", torch.int32)
    _need(q_out, "q_out")
    _need(kv_layer, "kv_layer", q_out.dtype)
    T = positions.numel()
    if qkv.shape != (T, (nq + 2 * nkv) * d):
        raise KernelError(f"qkv shape {tuple(qkv.shape)} is not [T={T}, (nq + 2 nkv) d = {(nq + 2 * nkv) * d}]")
    if tuple(kv_layer.shape[1:]) != (2, nkv, page_size, d):
        raise KernelError(f"kv_layer shape {tuple(kv_layer.shape)} is not [pages, 2, {nkv}, {page_size}, {d}]")
    if inv_freq is not None:
        _need(inv_freq, "inv_freq", torch.float32)
        if inv_freq.numel() != d // 2:
            raise KernelError(f"inv_freq has {inv_freq.numel()} entries, head size {d} needs {d // 2}")
    check(kernel("sharpi_qkv_post")(qkv.data_ptr(), positions.data_ptr(), row_req.data_ptr(),
                                    block_table.data_ptr(), _ptr(inv_freq), q_out.data_ptr(), kv_layer.data_ptr(),
                                    dtype_code(q_out.dtype), T, nq, nkv, d, block_table.shape[-1], page_size,
                                    pairing, float(l2_eps), float(temp_attn_scale), float(temp_floor_scale),
                                    int(write_kv), _stream()), "sharpi_qkv_post")


def paged_attention_generic(q: torch.Tensor, kv_layer: torch.Tensor, block_table: torch.Tensor,
                            row_req: torch.Tensor, positions: torch.Tensor, *, nq: int, nkv: int, d: int,
                            page_size: int, mask_kind: int, mask_span: int, scale: float,
                            out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Attention of every row over the keys it may see in its request's pages; [T, nq d]."""
    _need(q, "q")
    _need(kv_layer, "kv_layer", q.dtype)
    _need(block_table, "block_table", torch.int32)
    _need(row_req, "row_req", torch.int32)
    _need(positions, "positions", torch.int32)
    T = positions.numel()
    if out is None:
        out = torch.empty((T, nq * d), dtype=q.dtype, device=q.device)
    check(kernel("sharpi_paged_attention_generic")(q.data_ptr(), kv_layer.data_ptr(), block_table.data_ptr(),
                                                   row_req.data_ptr(), positions.data_ptr(), out.data_ptr(),
                                                   dtype_code(q.dtype), T, nq, nkv, d, block_table.shape[-1],
                                                   page_size, mask_kind, mask_span, float(scale), _stream()),
          "sharpi_paged_attention_generic")
    return out


FAST_ATTENTION_HEAD_SIZES = (16, 32, 48, 64, 80, 96, 112, 128)
DECODE_SPLIT = 256


_ticket_buffers = {}


def zeroed_tickets(device, count: int) -> torch.Tensor:
    """``count`` int32 zeros for kernels whose last CTA finishes a piece of work (it counts arrivals there and
    leaves the counters at zero).  One buffer per device and stream, so that launches that may overlap on two
    streams never share counters; it grows when a launch needs more."""
    key = (torch.device(device), torch.cuda.current_stream(device).cuda_stream)
    buf = _ticket_buffers.get(key)
    if buf is None or buf.numel() < count:
        buf = torch.zeros(max(count, 4096), dtype=torch.int32, device=device)
        _ticket_buffers[key] = buf
    return buf


def decode_splits(max_context: int, mask_kind: int, mask_span: int) -> int:
    """An upper bound on the 256-key splits a decode row needs (the kernel skips the empty ones)."""
    full = (max_context + DECODE_SPLIT - 1) // DECODE_SPLIT
    if mask_kind == MASK_FULL:
        return max(full, 1)
    return max(1, min(full, (mask_span + DECODE_SPLIT - 1) // DECODE_SPLIT + 1))


def attention_decode(q: torch.Tensor, kv_layer: torch.Tensor, block_table: torch.Tensor, row_req: torch.Tensor,
                     positions: torch.Tensor, out: torch.Tensor, *, rows: Optional[torch.Tensor], num_rows: int,
                     nq: int, nkv: int, d: int, page_size: int, mask_kind: int, mask_span: int, scale: float,
                     max_context: int, max_keys: Optional[int] = None) -> None:
    """Split-KV paged attention for rows that bring one query each (bfloat16).  ``rows`` (int32) names
    the rows to serve, or None for rows ``0 .. num_rows - 1``; results go to ``out[row]``.  ``max_context`` bounds
    the longest row (position + 1), ``max_keys`` the sum of position + 1 over the served rows: with it the launch
    holds about as many CTAs as the rows have splits together, not rows times the longest row's splits."""
    _need(q, "q", torch.bfloat16)
    _need(kv_layer, "kv_layer", torch.bfloat16)
    _need(out, "out", torch.bfloat16)
    _need(block_table, "block_table", torch.int32)
    if d not in FAST_ATTENTION_HEAD_SIZES:
        raise KernelError(f"head size {d} is not served by the tensor-core attention kernels "
                          f"({FAST_ATTENTION_HEAD_SIZES}); use the generic kernel")
    splits = decode_splits(max_context, mask_kind, mask_span)
    # a row at position p has at most p // 256 + 1 splits, so the rows together at most max_keys // 256 + rows
    items = num_rows * splits if max_keys is None else min(num_rows * splits, max_keys // DECODE_SPLIT + num_rows)
    part_o = torch.empty((num_rows, nq, splits, d), dtype=torch.float32, device=q.device)
    part_ml = torch.empty((num_rows, nq, splits, 2), dtype=torch.float32, device=q.device)
    check(kernel("sharpi_attention_decode")(q.data_ptr(), kv_layer.data_ptr(), block_table.data_ptr(),
                                            row_req.data_ptr(), positions.data_ptr(), _ptr(rows), part_o.data_ptr(),
                                            part_ml.data_ptr(), out.data_ptr(), status_word(q.device).data_ptr(),
                                            kv_layer.shape[0], num_rows, nq, nkv, d,
                                            block_table.shape[-1], page_size, mask_kind, mask_span, splits, items,
                                            float(scale), _stream()), "sharpi_attention_decode")


def attention_prefill(q: torch.Tensor, kv_layer: torch.Tensor, block_table: torch.Tensor, tiles: torch.Tensor,
                      out: torch.Tensor, *, nq: int, nkv: int, d: int, page_size: int, mask_kind: int,
                      mask_span: int, scale: float) -> None:
    """Paged attention for tiles of up to 64 consecutive rows of one request (bfloat16).  ``tiles`` is
    int32 [n, 4]: first row, number of rows, position of the first row, request index."""
    _need(q, "q", torch.bfloat16)
    _need(kv_layer, "kv_layer", torch.bfloat16)
    _need(out, "out", torch.bfloat16)
    _need(tiles, "tiles", torch.int32)
    if d not in FAST_ATTENTION_HEAD_SIZES:
        raise KernelError(f"head size {d} is not served by the tensor-core attention kernels "
                          f"({FAST_ATTENTION_HEAD_SIZES}); use the generic kernel")
    check(kernel("sharpi_attention_prefill")(q.data_ptr(), kv_layer.data_ptr(), block_table.data_ptr(),
                                             tiles.data_ptr(), out.data_ptr(), tiles.shape[0], nq, nkv, d,
                                             block_table.shape[-1], page_size, mask_kind, mask_span, float(scale),
                                             _stream()), "sharpi_attention_prefill")


TC_PREFILL_TILE = 128


def tc_prefill_supported(dtype: torch.dtype, d: int, page_size: int) -> bool:
    """Whether the tcgen05 prefill attention kernel takes this layer: bfloat16, head size 64 or 128,
    pages of a power of two >= 64 positions."""
    return dtype == torch.bfloat16 and d in (64, 128) and page_size >= 64 and (page_size & (page_size - 1)) == 0


def attention_prefill_tc(q: torch.Tensor, kv_layer: torch.Tensor, block_table: torch.Tensor, tiles: torch.Tensor,
                         out: torch.Tensor, *, nq: int, nkv: int, d: int, page_size: int, mask_kind: int,
                         mask_span: int, scale: float) -> None:
    """Paged attention for tiles of up to 128 consecutive rows of one request on tcgen05 / TMEM / TMA."""
    _need(q, "q", torch.bfloat16)
    _need(kv_layer, "kv_layer", torch.bfloat16)
    _need(out, "out", torch.bfloat16)
    _need(tiles, "tiles", torch.int32)
    if not tc_prefill_supported(q.dtype, d, page_size):
        raise KernelError(f"the tcgen05 attention kernel takes head sizes 64 and 128 and pages of 64 * 2^k positions, "
                          f"found head size {d}, page size {page_size}")
    check(kernel("sharpi_attention_prefill_tc")(q.data_ptr(), kv_layer.data_ptr(), block_table.data_ptr(),
                                                tiles.data_ptr(), out.data_ptr(), status_word(q.device).data_ptr(),
                                                q.shape[0], kv_layer.shape[0], tiles.shape[0], nq, nkv, d,
                                                block_table.shape[-1], page_size, mask_kind, mask_span, float(scale),
                                                _stream()), "sharpi_attention_prefill_tc")


def gemm_nt(a: torch.Tensor, w: torch.Tensor, *, out: Optional[torch.Tensor] = None,
            group_offsets: Optional[torch.Tensor] = None, a_rows: Optional[torch.Tensor] = None,
            out_rows: Optional[torch.Tensor] = None, rows: Optional[int] = None, accumulate: bool = False,
            bias: Optional[torch.Tensor] = None, row_scale: Optional[torch.Tensor] = None,
            scale_rows: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``C = A . W^T`` with fp32 accumulation on the CUDA cores.

    Dense: ``w`` is [N, K].  Grouped: ``w`` is [E, N, K] and ``group_offsets`` (int32 [E+1])
    gives the first sorted row of every expert.  ``a_rows`` / ``out_rows`` (int32 [rows]) make
    sorted row r read ``A[a_rows[r]]`` and write ``C[out_rows[r]]``.  ``row_scale`` (float32)
    multiplies row r of the product by ``row_scale[scale_rows[r] or r]``, ``bias`` (float32 [N]) is
    added to it, before the row is stored or added in.
    """
    _need(a, "a")
    _need(w, "w")
    K = a.shape[-1]
    if w.shape[-1] != K:
        raise KernelError(f"inner sizes differ: a [..., {K}] against w [..., {w.shape[-1]}]")
    if group_offsets is not None:
        _need(group_offsets, "group_offsets", torch.int32)
        if w.dim() != 3 or group_offsets.numel() != w.shape[0] + 1:
            raise KernelError("a grouped product needs w [E, N, K] and group_offsets [E + 1]")
        E, N = w.shape[0], w.shape[1]
    else:
        if w.dim() != 2:
            raise KernelError("a dense product needs w [N, K]")
        E, N = 1, w.shape[0]
    M = rows if rows is not None else (a_rows.numel() if a_rows is not None else a.shape[0])
    if out is None:
        if accumulate:
            raise KernelError("accumulate=True needs an output tensor to add to")
        out = torch.empty((M, N), dtype=torch.float32, device=a.device)
    _need(out, "out", torch.float32)
    if a_rows is not None:
        _need(a_rows, "a_rows", torch.int32)
    if out_rows is not None:
        _need(out_rows, "out_rows", torch.int32)
    if bias is not None:
        _need(bias, "bias", torch.float32)
        if bias.numel() != N:
            raise KernelError(f"bias has {bias.numel()} entries, the product has {N} columns")
    if row_scale is not None:
        _need(row_scale, "row_scale", torch.float32)
    if scale_rows is not None:
        _need(scale_rows, "scale_rows", torch.int32)
    check(kernel("sharpi_gemm_nt")(a.data_ptr(), dtype_code(a.dtype), w.data_ptr(), dtype_code(w.dtype),
                                   out.data_ptr(), _ptr(group_offsets), _ptr(a_rows), _ptr(out_rows), M, N, K, E,
                                   int(accumulate), _ptr(bias), _ptr(row_scale), _ptr(scale_rows), _stream()),
          "sharpi_gemm_nt")
    return out


# ---------------------------------------------------------------------------------------
# tensor-core kernels (tcgen05 / TMEM / TMA)
# ---------------------------------------------------------------------------------------
_status_words = {}


def status_word(device) -> torch.Tensor:
    """The device word in which a tensor-core kernel records a wait that gave up (0 = none)."""
    device = torch.device(device)
    w = _status_words.get(device)
    if w is None:
        w = torch.zeros(1, dtype=torch.int32, device=device)
        _status_words[device] = w
    return w


def check_status(device) -> None:
    """Raise if a tensor-core kernel gave up on a wait since the last check (synchronises)."""
    w = _status_words.get(torch.device(device))
    if w is not None:
        code = int(w.item())
        if code != 0:
            w.zero_()
            for buf in list(_ticket_buffers.values()) + list(_argmax_scratches.values()) + list(_sliced_work.values()):
                buf.zero_()               # a kernel that gave up may have left counters behind
            raise KernelError(f"a tensor-core kernel gave up (code {code}: 1 = wait for a free stage, 2 = for a loaded "
                              f"stage, 3 = for the accumulator, 4 = for a key/value copy, 5 = misaligned staging "
                              f"buffer, 6 = misaligned shared memory, 7 = for drained tensor memory, 11-18 = "
                              f"attention: queries, keys, values, scores, probabilities, outputs, free stage, "
                              f"misaligned shared memory); its output is incomplete")


TC_MODE_STORE, TC_MODE_SWIGLU = 0, 1


TC_PERSISTENT = 0            # row_tile value that selects the persistent kernel
TC_PERSISTENT_MAX_GROUPS = 256


def tc_row_tile(rows: int, mode: Optional[int] = None, groups: int = 1) -> int:
    """Activation rows per CTA for a grouped product over `rows` rows in all; TC_PERSISTENT for the kernel
    that walks work items (gate|up products of 1024 rows and more: measured 406 vs 455 us at 1024 rows,
    490 vs 563 us at 2048 unevenly spread rows, 634 vs 753 us at 4096; the down product has too few items
    per SM to gain and stays on the tiled kernel)."""
    if mode == TC_MODE_SWIGLU and rows >= 1024 and groups <= TC_PERSISTENT_MAX_GROUPS:
        return TC_PERSISTENT
    if rows <= 128:
        return 16
    if rows <= 256:
        return 32
    if rows <= 512:
        return 64
    return 128


_sm_counts = {}


def sm_count(device=None) -> int:
    """Streaming multiprocessors of the device (asked once)."""
    device = torch.device(device) if device is not None else torch.device("cuda", torch.cuda.current_device())
    n = _sm_counts.get(device)
    if n is None:
        n = _sm_counts[device] = torch.cuda.get_device_properties(device).multi_processor_count
    return n


def tc_k_split(rows: int, n_out: int, sms: int = 148) -> int:
    """Into how many CTAs a tile's K range is cut.  With few rows few experts are active (at most one
    per row), so 128-row weight tiles alone cannot fill the GPU; cutting K makes up to four times as many
    CTAs.  The CTA of a tile that finishes last adds the parts in a fixed order."""
    if rows > 16:
        return 1
    ctas = rows * ((n_out + 127) // 128)
    if ctas >= sms:
        return 1
    return max(1, min(4, (2 * sms + ctas - 1) // ctas))


def gather_rows_bf16(x: torch.Tensor, rows: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``out[r] = x[rows[r]]`` for bfloat16 rows whose width is a multiple of 8."""
    _need(x, "x", torch.bfloat16)
    _need(rows, "rows", torch.int32)
    R, K = rows.numel(), x.shape[-1]
    if out is None:
        out = torch.empty((R, K), dtype=torch.bfloat16, device=x.device)
    check(kernel("sharpi_gather_rows_bf16")(x.data_ptr(), rows.data_ptr(), out.data_ptr(), R, K, _stream()),
          "sharpi_gather_rows_bf16")
    return out


def tc_grouped_gemm(a: torch.Tensor, w: torch.Tensor, group_offsets: torch.Tensor, *, mode: int,
                    out: Optional[torch.Tensor] = None, out_rows: Optional[torch.Tensor] = None,
                    row_scale: Optional[torch.Tensor] = None, scale_rows: Optional[torch.Tensor] = None,
                    accumulate: bool = False, row_tile: Optional[int] = None,
                    k_split: Optional[int] = None, max_ctas: int = 0) -> torch.Tensor:
    """Per-expert products on the tensor cores.  ``a`` bfloat16 [rows, K] sorted by expert,
    ``w`` bfloat16 [E, N, K], ``group_offsets`` int32 [E + 1].

    ``mode=TC_MODE_STORE``: float32 ``out[out_rows[r] or r] (+)= s * a[r] . w[e(r)]^T``, shape [*, N], with
    ``s = row_scale[scale_rows[r] or r]`` when ``row_scale`` is given (a router that weights outputs), else 1.
    ``mode=TC_MODE_SWIGLU``: ``w`` holds gate rows then up rows (N = 2 I); bfloat16
    ``out[r] = silu(s g) * (s u)``, shape [rows, I], ``s = row_scale[scale_rows[r]]``.
    ``max_ctas`` > 0 (persistent kernel only) keeps the launch to that many SMs, for running beside another kernel.
    """
    _need(a, "a", torch.bfloat16)
    _need(w, "w", torch.bfloat16)
    _need(group_offsets, "group_offsets", torch.int32)
    rows, K = a.shape
    E, N, Kw = w.shape
    if Kw != K or group_offsets.numel() != E + 1:
        raise KernelError(f"shapes disagree: a {tuple(a.shape)}, w {tuple(w.shape)}, offsets {group_offsets.numel()}")
    if K % 8 != 0:
        raise KernelError(f"the tensor-core product needs an inner size that is a multiple of 8, found {K}")
    if out is None:
        if accumulate:
            raise KernelError("accumulate=True needs an output tensor to add to")
        out = (torch.empty((rows, N // 2), dtype=torch.bfloat16, device=a.device) if mode == TC_MODE_SWIGLU
               else torch.empty((rows, N), dtype=torch.float32, device=a.device))
    _need(out, "out", torch.bfloat16 if mode == TC_MODE_SWIGLU else torch.float32)
    status = status_word(a.device)
    if k_split is None:
        k_split = tc_k_split(rows, (N // 2 if mode == TC_MODE_SWIGLU else N), sm_count(a.device))
    partial = torch.empty((k_split, rows, N), dtype=torch.float32, device=a.device) if k_split > 1 else None
    if row_tile is None:
        row_tile = tc_row_tile(rows, mode, E)
    tickets = None
    if k_split > 1:           # one counter per (weight tile, row tile) of the launch grid
        tickets = zeroed_tickets(a.device, ((N + 127) // 128) * (rows // max(row_tile, 1) + min(rows, E)))
    check(kernel("sharpi_tc_grouped_gemm")(a.data_ptr(), w.data_ptr(), group_offsets.data_ptr(), out.data_ptr(),
                                           _ptr(out_rows), _ptr(row_scale), _ptr(scale_rows), status.data_ptr(),
                                           _ptr(partial), _ptr(tickets), rows, N, K, E, mode, row_tile,
                                           int(accumulate), k_split, int(max_ctas) if row_tile == TC_PERSISTENT else 0,
                                           _stream()), "sharpi_tc_grouped_gemm")
    return out


def tc_set_wait_test(limit: int, drop_from: int) -> None:
    """Test hook: the next ``tc_grouped_gemm`` launch (tiled kernel) polls each wait at most ``limit`` times and
    loads nothing from K block ``drop_from`` on, so a wait runs out, the kernel records its code in the status
    word and returns; ``check_status`` then raises.  Consumed by that one launch."""
    import ctypes
    from .library import load_library
    fn = load_library("tc_gemm").sharpi_tc_set_wait_test
    fn.argtypes, fn.restype = [ctypes.c_uint, ctypes.c_int], None
    fn(int(limit), int(drop_from))


_dense_offsets = {}


def tc_dense(a: torch.Tensor, w: torch.Tensor, *, out: Optional[torch.Tensor] = None,
             accumulate: bool = False) -> torch.Tensor:
    """A dense product ``a . w^T`` for a few rows on the grouped tensor-core kernel with one group: the
    weights stream once through 128-row tiles, K cut over CTAs when the tiles alone would not fill the GPU.
    float32 ``[M, N]``, added into ``out`` with reductions when ``accumulate`` (so that another launch may add
    into the same rows meanwhile).  Alone it is slower than :func:`dense_rows` and the library; its small CTAs
    run well beside the routed experts' kernels, which is where the mixture part uses it."""
    M = a.shape[0]
    key = (a.device, M)
    offsets = _dense_offsets.get(key)
    if offsets is None:
        offsets = torch.tensor([0, M], dtype=torch.int32, device=a.device)
        _dense_offsets[key] = offsets
    N = w.shape[0]
    n_tiles = (N + 127) // 128
    sms = sm_count(a.device)
    k_split = 1 if n_tiles >= sms else max(1, min(4, (2 * sms + n_tiles - 1) // n_tiles))
    row_tile = 16 if M <= 16 else 32 if M <= 32 else 64 if M <= 64 else 128
    return tc_grouped_gemm(a, w.unsqueeze(0), offsets, mode=TC_MODE_STORE, out=out, row_tile=row_tile,
                           k_split=k_split, accumulate=accumulate)


DENSE_ROWS_MAX = 16           # rows the weight-streaming dense kernel takes


def dense_rows(a: torch.Tensor, w: torch.Tensor, *, swiglu: bool = False, out: Optional[torch.Tensor] = None,
               accumulate: bool = False, bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``a . w^T`` for up to 16 bfloat16 rows against a bfloat16 weight ``[N, K]`` that streams in once
    (``dense_rows.cu``): float32 ``[M, N]`` (plus ``bias``), added into ``out`` with reductions when
    ``accumulate``, or with ``swiglu`` (``w`` = gate rows then up rows) ``silu(g) * u`` in bfloat16 ``[M, N / 2]``."""
    _need(a, "a", torch.bfloat16)
    _need(w, "w", torch.bfloat16)
    M, K = a.shape
    N = w.shape[0]
    if w.shape[1] != K:
        raise KernelError(f"weight is {tuple(w.shape)}, activations have width {K}")
    if M > DENSE_ROWS_MAX:
        raise KernelError(f"dense_rows takes up to {DENSE_ROWS_MAX} rows, found {M}")
    if swiglu and (accumulate or bias is not None):
        raise KernelError("the SwiGLU epilogue neither accumulates nor takes a bias")
    if accumulate and out is None:
        raise KernelError("accumulate needs an output to add to")
    if bias is not None:
        _need(bias, "bias", torch.float32)
    if out is None:
        out = torch.empty((M, N // 2), dtype=torch.bfloat16, device=a.device) if swiglu else \
            torch.empty((M, N), dtype=torch.float32, device=a.device)
    else:
        _need(out, "out", torch.bfloat16 if swiglu else torch.float32)
        if tuple(out.shape) != ((M, N // 2) if swiglu else (M, N)):
            raise KernelError(f"out is {tuple(out.shape)} for a product of {M} rows and a weight of {N} rows")
    mode = 2 if swiglu else 1 if accumulate else 0
    check(kernel("sharpi_dense_rows")(a.data_ptr(), w.data_ptr(), _ptr(bias), out.data_ptr(), M, N, K, mode,
                                      _stream()), "sharpi_dense_rows")
    return out


def router_top1(h32: torch.Tensor, router_weight: torch.Tensor, *, want_logits: bool = False, sort: bool = False):
    """Top-1 sigmoid routing.  Returns ``(expert_id int32 [T], weight fp32 [T], logits or None)``; with
    ``sort`` also ``offsets`` and ``sorted_rows`` as :func:`moe_sort` gives them (from the same launch for
    steps of up to 32 tokens)."""
    _need(h32, "h32", torch.float32)
    _need(router_weight, "router_weight", torch.float32)
    T, H = h32.shape
    E = router_weight.shape[0]
    if router_weight.shape[1] != H:
        raise KernelError(f"router weight is {tuple(router_weight.shape)}, activations have width {H}")
    expert = torch.empty((T,), dtype=torch.int32, device=h32.device)
    weight = torch.empty((T,), dtype=torch.float32, device=h32.device)
    logits = torch.empty((T, E), dtype=torch.float32, device=h32.device) if want_logits else None
    scratch = _router_scratch(h32.device, E) if T <= 32 else None
    offsets = sorted_rows = None
    if sort:
        offsets = torch.empty((E + 1,), dtype=torch.int32, device=h32.device)
        sorted_rows = torch.empty((T,), dtype=torch.int32, device=h32.device)
    check(kernel("sharpi_router_top1")(h32.data_ptr(), router_weight.data_ptr(), T, H, E, 0, expert.data_ptr(),
                                       weight.data_ptr(), _ptr(logits), _ptr(scratch), _ptr(offsets), _ptr(sorted_rows),
                                       _stream()), "sharpi_router_top1")
    if sort:
        return expert, weight, logits, offsets, sorted_rows
    return expert, weight, logits


_router_scratches = {}


def _router_scratch(device, num_experts: int) -> torch.Tensor:
    """Scratch of the few-token router kernel: 32 x E logits, then 32 ticket counters that start at zero
    and are left at zero by every launch.  One per device and expert count, shared by all layers (launches
    on one stream run one after the other)."""
    key = (torch.device(device), num_experts)
    buf = _router_scratches.get(key)
    if buf is None:
        buf = torch.zeros(32 * num_experts + 33, dtype=torch.float32, device=device)
        _router_scratches[key] = buf
    return buf


def moe_sort(expert_id: torch.Tensor, num_experts: int):
    """Stable sort of rows by expert: ``(offsets int32 [E+1], sorted_rows int32 [T])``."""
    _need(expert_id, "expert_id", torch.int32)
    T = expert_id.numel()
    offsets = torch.empty((num_experts + 1,), dtype=torch.int32, device=expert_id.device)
    sorted_rows = torch.empty((T,), dtype=torch.int32, device=expert_id.device)
    check(kernel("sharpi_moe_sort")(expert_id.data_ptr(), T, num_experts, offsets.data_ptr(),
                                    sorted_rows.data_ptr(), _stream()), "sharpi_moe_sort")
    return offsets, sorted_rows


_argmax_scratches = {}


def argmax_rows(logits: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Index of the largest entry of every row (the lowest index among equals), int32 [R]."""
    _need(logits, "logits", torch.float32)
    R, V = logits.shape
    if out is None:
        out = torch.empty((R,), dtype=torch.int32, device=logits.device)
    scratch = None
    if R <= 64:       # few rows: every row is cut over 32 blocks; 64 counters (kept at zero), then the slices' candidates
        key = (logits.device, torch.cuda.current_stream(logits.device).cuda_stream)
        scratch = _argmax_scratches.get(key)
        if scratch is None:
            scratch = _argmax_scratches[key] = torch.zeros(64 + 64 * 32 * 2, dtype=torch.int32, device=logits.device)
    check(kernel("sharpi_argmax_rows")(logits.data_ptr(), R, V, out.data_ptr(), _ptr(scratch), _stream()),
          "sharpi_argmax_rows")
    return out


def apply_penalties(logits: torch.Tensor, entry_row: torch.Tensor, entry_token: torch.Tensor,
                    entry_count: torch.Tensor, rep: torch.Tensor, freq: torch.Tensor, pres: torch.Tensor) -> None:
    _need(logits, "logits", torch.float32)
    for name, t in (("entry_row", entry_row), ("entry_token", entry_token), ("entry_count", entry_count)):
        _need(t, name, torch.int32)
    for name, t in (("rep", rep), ("freq", freq), ("pres", pres)):
        _need(t, name, torch.float32)
    check(kernel("sharpi_apply_penalties")(logits.data_ptr(), logits.shape[1], entry_row.data_ptr(),
                                           entry_token.data_ptr(), entry_count.data_ptr(), rep.data_ptr(),
                                           freq.data_ptr(), pres.data_ptr(), entry_row.numel(), _stream()),
          "sharpi_apply_penalties")


def add_logit_bias(logits: torch.Tensor, entry_row: torch.Tensor, entry_token: torch.Tensor,
                   entry_bias: torch.Tensor) -> None:
    _need(logits, "logits", torch.float32)
    _need(entry_row, "entry_row", torch.int32)
    _need(entry_token, "entry_token", torch.int32)
    _need(entry_bias, "entry_bias", torch.float32)
    check(kernel("sharpi_add_logit_bias")(logits.data_ptr(), logits.shape[1], entry_row.data_ptr(),
                                          entry_token.data_ptr(), entry_bias.data_ptr(), entry_row.numel(),
                                          _stream()), "sharpi_add_logit_bias")


_sliced_work = {}
SLICED_SAMPLER_FROM = 4096        # vocabularies from this size on take the sampler that cuts rows over 32 blocks
_SLICED_ROW_BYTES = 56 + 32 * 16 + 2048 * 12


def sample_rows(logits: torch.Tensor, temperature: torch.Tensor, top_k: torch.Tensor, top_p: torch.Tensor,
                min_p: torch.Tensor, uniform: torch.Tensor, *, probs: Optional[torch.Tensor] = None,
                out: Optional[torch.Tensor] = None, any_top_k: bool = True, any_top_p: bool = True,
                sliced: Optional[bool] = None) -> torch.Tensor:
    """One token per row: greedy where ``temperature <= 0``, else filtered temperature sampling.

    Large vocabularies take the sampler that cuts every row over 32 blocks and finds the thresholds by
    radix selection (``sliced``; ``any_top_k`` / ``any_top_p`` = False skip the passes of a filter that no
    row uses); small ones the one-block-per-row sampler with its ``probs`` work area."""
    _need(logits, "logits", torch.float32)
    R, V = logits.shape
    _need(temperature, "temperature", torch.float32)
    _need(top_k, "top_k", torch.int32)
    _need(top_p, "top_p", torch.float32)
    _need(min_p, "min_p", torch.float32)
    _need(uniform, "uniform", torch.float32)
    if out is None:
        out = torch.empty((R,), dtype=torch.int32, device=logits.device)
    if sliced is None:
        sliced = V >= SLICED_SAMPLER_FROM and probs is None
    if sliced:
        key = (logits.device, torch.cuda.current_stream(logits.device).cuda_stream)
        work = _sliced_work.get(key)
        need = R * _SLICED_ROW_BYTES + 256
        if work is None or work.numel() < need:        # all zero before the first call; every call leaves it so
            work = _sliced_work[key] = torch.zeros(max(need, 64 * _SLICED_ROW_BYTES), dtype=torch.uint8,
                                                   device=logits.device)
        check(kernel("sharpi_sample_rows_sliced")(logits.data_ptr(), R, V, temperature.data_ptr(), top_k.data_ptr(),
                                                  top_p.data_ptr(), min_p.data_ptr(), uniform.data_ptr(),
                                                  work.data_ptr(), int(any_top_k), int(any_top_p), out.data_ptr(),
                                                  _stream()), "sharpi_sample_rows_sliced")
        return out
    if probs is None:
        probs = torch.empty((R, V), dtype=torch.float32, device=logits.device)
    check(kernel("sharpi_sample_rows")(logits.data_ptr(), R, V, temperature.data_ptr(), top_k.data_ptr(),
                                       top_p.data_ptr(), min_p.data_ptr(), uniform.data_ptr(), probs.data_ptr(),
                                       out.data_ptr(), _stream()), "sharpi_sample_rows")
    return out
