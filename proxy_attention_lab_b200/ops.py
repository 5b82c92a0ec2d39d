"""Proxy Attention Lab's operator API on PyTorch CUDA tensors, backed by libpal_b200.so.

Same names, argument order and cache layouts as the reference's Python layer
(``src/proxy_attention_lab/ops.py:33-171``, bound in ``src/pal_core/bindings.cpp:44-222``),
with ``torch.Tensor`` where the reference takes ``mx.array`` and eager launches on the current
CUDA stream where the reference builds lazy MLX graph nodes.  Every operator launches
hand-written sm_100a kernels through the C ABI; nothing here computes on the host and there is
no fallback path.
"""

from __future__ import annotations

import functools
import math

import torch

from . import _lib
from ._lib import lib

_DTYPES = {torch.float16: _lib.PAL_DTYPE_F16, torch.bfloat16: _lib.PAL_DTYPE_BF16}


def _dtype_code(dtype: torch.dtype) -> int:
    try:
        return _DTYPES[dtype]
    except KeyError:
        raise ValueError(f"dtype {dtype} is not supported (float16 and bfloat16 are)") from None


def _stream_ptr(stream, device) -> int:
    if stream is None:
        return torch.cuda.current_stream(device).cuda_stream
    if isinstance(stream, torch.cuda.Stream):
        return stream.cuda_stream
    if isinstance(stream, int):
        return stream
    raise TypeError("stream must be None, a torch.cuda.Stream or a raw cudaStream_t integer")


def _need_cuda(name: str, t: torch.Tensor) -> None:
    if not isinstance(t, torch.Tensor):
        raise TypeError(f"{name} must be a torch.Tensor")
    if not t.is_cuda:
        raise RuntimeError(f"{name} must live on a CUDA device; this library has no CPU path")


def _contig(t: torch.Tensor) -> torch.Tensor:
    return t if t.is_contiguous() else t.contiguous()


def _index32(name: str, t: torch.Tensor) -> torch.Tensor:
    """Page tables / positions as 32-bit words (uint32 and int32 share their bits for valid ids)."""
    if t.dtype in (torch.int32, torch.uint32):
        return _contig(t)
    if t.dtype in (torch.int64, torch.int16, torch.uint8, torch.uint16):
        return _contig(t.to(torch.int32))
    raise TypeError(f"{name} must be an integer tensor, got {t.dtype}")


def _ptr(t) -> int:
    return 0 if t is None or t.numel() == 0 else t.data_ptr()


_WORKSPACES: dict = {}


def _workspace(nbytes: int, device, stream_ptr: int) -> torch.Tensor:
    """Scratch for one call.  Calls on one stream run in order, so they share one buffer per (device, stream);
    it only ever grows, which also keeps its address stable for a caller that captures the call in a CUDA graph."""
    need = max(int(nbytes), 256)
    key = (device.index, stream_ptr)
    ws = _WORKSPACES.get(key)
    if ws is None or ws.numel() < need:
        ws = torch.empty(max(need, 4096), dtype=torch.uint8, device=device)
        _WORKSPACES[key] = ws
    return ws


class _NoGuard:
    def __enter__(self):
        return None

    def __exit__(self, *exc):
        return False


_NO_GUARD = _NoGuard()


def _on(device):
    """Device guard that costs nothing when `device` is already current."""
    return _NO_GUARD if torch.cuda.current_device() == device.index else torch.cuda.device(device)


@functools.lru_cache(maxsize=256)
def _decode_ws_bytes(S, hq, hkv, d, tpp, mp, pp) -> int:
    return lib.pal_decode_workspace_bytes(S, hq, hkv, d, tpp, mp, pp)


# ---------------------------------------------------------------------------------------------
# layout helpers (src/pal_core/bindings.cpp:44-72)
# ---------------------------------------------------------------------------------------------
def get_k_cache_stripe_size(dtype: torch.dtype) -> int:
    rc = lib.pal_get_k_cache_stripe_size(_dtype_code(dtype))
    if rc < 0:
        _lib.check(rc)
    return rc


def get_optimal_page_size() -> int:
    return lib.pal_get_optimal_page_size()


def get_k_cache_shape(num_total_pages: int, num_kv_heads: int, head_dim: int, tokens_per_page: int, dtype):
    out = (_lib.c_int64 * 5)()
    _lib.check(lib.pal_get_k_cache_shape(num_total_pages, num_kv_heads, head_dim, tokens_per_page, _dtype_code(dtype), out))
    return tuple(int(v) for v in out)


def get_v_cache_shape(num_total_pages: int, num_kv_heads: int, head_dim: int, tokens_per_page: int, dtype):
    out = (_lib.c_int64 * 4)()
    _lib.check(lib.pal_get_v_cache_shape(num_total_pages, num_kv_heads, head_dim, tokens_per_page, _dtype_code(dtype), out))
    return tuple(int(v) for v in out)


# ---------------------------------------------------------------------------------------------
# fill_kv_pages (src/proxy_attention_lab/ops.py:133-171, src/pal_core/src/ops.cpp:188-239)
# ---------------------------------------------------------------------------------------------
def fill_kv_pages(
    new_keys,
    new_values,
    global_key_pool,
    global_value_pool,
    page_table=None,
    current_token_write_positions=None,
    query_to_seq_map=None,
    *,
    slot_mapping=None,
    inplace: bool = True,
    stream=None,
):
    """Scatter ``new_keys`` / ``new_values`` ``[T, Hkv, D]`` into the page pools.

    Reference form: ``fill_kv_pages(new_keys, new_values, k_pool, v_pool, page_table,
    current_token_write_positions, query_to_seq_map)``.  Slot-mapping form:
    ``fill_kv_pages(new_keys, new_values, k_pool, v_pool, slot_mapping)`` (a single index tensor in
    the fifth position, or ``slot_mapping=``), with ``slot = page * tokens_per_page + slot_in_page``.

    Returns ``(k_pool, v_pool)``.  The pools are updated in place and returned (the reference
    returns fresh copies; pass ``inplace=False`` to clone first and leave the inputs untouched).
    """
    if slot_mapping is None and page_table is not None and current_token_write_positions is None and query_to_seq_map is None:
        slot_mapping, page_table = page_table, None
    for name, t in (("new_keys", new_keys), ("new_values", new_values), ("global_key_pool", global_key_pool),
                    ("global_value_pool", global_value_pool)):
        _need_cuda(name, t)
    # src/pal_core/src/ops.cpp:204-211
    if global_key_pool.dim() != 5:
        raise ValueError("global_key_pool must be 5-D [pages, kv_heads, head_dim/x, tokens_per_page, x]")
    if global_value_pool.dim() != 4:
        raise ValueError("global_value_pool must be 4-D [pages, kv_heads, head_dim, tokens_per_page]")
    dt = _dtype_code(global_value_pool.dtype)
    if not (new_keys.dtype == new_values.dtype == global_key_pool.dtype == global_value_pool.dtype):
        raise ValueError("new_keys, new_values and both pools must share one dtype")
    num_pages, hkv, d, tpp = global_value_pool.shape
    if new_keys.dim() != 3 or new_keys.shape != new_values.shape or new_keys.shape[1:] != (hkv, d):
        raise ValueError(f"new_keys / new_values must be [T, {hkv}, {d}], got {tuple(new_keys.shape)} / {tuple(new_values.shape)}")
    if tuple(global_key_pool.shape) != (num_pages, hkv, d // 8, tpp, 8):
        raise ValueError("global_key_pool shape does not match global_value_pool")
    if not inplace:
        global_key_pool = global_key_pool.clone()
        global_value_pool = global_value_pool.clone()
    if not (global_key_pool.is_contiguous() and global_value_pool.is_contiguous()):
        raise ValueError("the page pools must be contiguous")
    T = new_keys.shape[0]
    if T == 0:
        return global_key_pool, global_value_pool
    new_keys, new_values = _contig(new_keys), _contig(new_values)
    dev = global_value_pool.device
    with _on(dev):
        sp = _stream_ptr(stream, dev)
        if slot_mapping is not None:
            _need_cuda("slot_mapping", slot_mapping)
            slots = _contig(slot_mapping.to(torch.int64))
            if slots.numel() != T:
                raise ValueError("slot_mapping must have one entry per new token")
            rc = lib.pal_fill_kv_pages_slots(new_keys.data_ptr(), new_values.data_ptr(), global_key_pool.data_ptr(),
                                             global_value_pool.data_ptr(), slots.data_ptr(), T, hkv, d, tpp, num_pages, dt, sp)
        else:
            if page_table is None or current_token_write_positions is None or query_to_seq_map is None:
                raise ValueError("page_table, current_token_write_positions and query_to_seq_map are required")
            for name, t in (("page_table", page_table), ("current_token_write_positions", current_token_write_positions),
                            ("query_to_seq_map", query_to_seq_map)):
                _need_cuda(name, t)
            if page_table.dim() != 2:
                raise ValueError("page_table must be 2-D [num_sequences, max_logical_pages]")
            pt = _index32("page_table", page_table)
            pos = _index32("current_token_write_positions", current_token_write_positions)
            seqmap = _index32("query_to_seq_map", query_to_seq_map)
            if pos.numel() != T or seqmap.numel() != T:
                raise ValueError("write positions and query_to_seq_map must have one entry per new token")
            rc = lib.pal_fill_kv_pages(new_keys.data_ptr(), new_values.data_ptr(), global_key_pool.data_ptr(),
                                       global_value_pool.data_ptr(), pt.data_ptr(), pos.data_ptr(), seqmap.data_ptr(), T,
                                       pt.shape[0], hkv, d, tpp, num_pages, pt.shape[1], dt, sp)
        _lib.check(rc)
    return global_key_pool, global_value_pool


# ---------------------------------------------------------------------------------------------
# paged_attention_decode (src/proxy_attention_lab/ops.py:42-84, src/pal_core/src/ops.cpp:36-108)
# ---------------------------------------------------------------------------------------------
def _decode_shapes(queries, k_cache_pool, v_cache_pool, page_table, sequence_lengths):
    for name, t in (("queries", queries), ("k_cache_pool", k_cache_pool), ("v_cache_pool", v_cache_pool),
                    ("page_table", page_table), ("sequence_lengths", sequence_lengths)):
        _need_cuda(name, t)
    if v_cache_pool.dim() != 4 or k_cache_pool.dim() != 5:
        raise ValueError("k_cache_pool must be 5-D and v_cache_pool 4-D")
    num_pages, hkv, d, tpp = v_cache_pool.shape  # ops.cpp:50-60
    if tuple(k_cache_pool.shape) != (num_pages, hkv, d // 8, tpp, 8):
        raise ValueError("k_cache_pool shape does not match v_cache_pool")
    if not (k_cache_pool.is_contiguous() and v_cache_pool.is_contiguous()):
        raise ValueError("the page pools must be contiguous")
    if not (queries.dtype == k_cache_pool.dtype == v_cache_pool.dtype):
        raise ValueError("queries and both pools must share one dtype")
    if page_table.dim() != 2:
        raise ValueError("page_table must be 2-D [num_sequences, max_logical_pages]")
    hq = queries.shape[1] if queries.dim() == 3 else 1  # ops.cpp:62-66
    if queries.shape[-1] != d and queries.dim() >= 2:
        raise ValueError(f"queries head_dim {queries.shape[-1]} does not match the cache head_dim {d}")
    S = page_table.shape[0]
    if queries.dim() >= 2 and queries.shape[0] < S:
        raise ValueError("queries has fewer rows than page_table has sequences")
    if sequence_lengths.numel() < S:
        raise ValueError("sequence_lengths has fewer entries than page_table has sequences")
    if hq % hkv != 0:
        raise ValueError(f"num_q_heads ({hq}) must be a multiple of num_kv_heads ({hkv})")
    return S, hq, hkv, d, tpp, num_pages


def paged_attention_decode(queries, k_cache_pool, v_cache_pool, page_table, sequence_lengths, *, stream=None,
                           partition_pages=None, scale=None):
    """One query token per sequence attending to its paged KV history.

    ``queries [>=S, Hq, D]`` (2-D means one query head), pools in the reference layouts,
    ``page_table [S, max_pages]``, ``sequence_lengths [S]``.  Returns ``[S, Hq, D]`` in the query
    dtype.  ``partition_pages``: None = let the library choose, 0 = fused single pass,
    n > 0 = two-pass split-KV with n-page partitions and a log-sum-exp combine.
    """
    S, hq, hkv, d, tpp, num_pages = _decode_shapes(queries, k_cache_pool, v_cache_pool, page_table, sequence_lengths)
    dev = queries.device
    out = torch.empty((S, hq, d), dtype=queries.dtype, device=dev)
    if S == 0:
        return out
    q = _contig(queries)
    pt = _index32("page_table", page_table)
    lens = _index32("sequence_lengths", sequence_lengths)
    pp = _lib.PAL_DECODE_AUTO if partition_pages is None else int(partition_pages)
    with _on(dev):
        sp = _stream_ptr(stream, dev)
        ws = _workspace(_decode_ws_bytes(S, hq, hkv, d, tpp, pt.shape[1], pp), dev, sp)
        rc = lib.pal_paged_attention_decode(q.data_ptr(), _ptr(k_cache_pool), _ptr(v_cache_pool), _ptr(pt), lens.data_ptr(),
                                            out.data_ptr(), S, hq, hkv, d, tpp, num_pages, pt.shape[1],
                                            0.0 if scale is None else float(scale), _dtype_code(q.dtype), pp,
                                            ws.data_ptr(), ws.numel(), sp)
        _lib.check(rc)
    return out


def paged_attention_decode_append(new_keys, new_values, queries, k_cache_pool, v_cache_pool, page_table, sequence_lengths, *,
                                  stream=None, partition_pages=None, scale=None):
    """``fill_kv_pages`` of each sequence's newest token and ``paged_attention_decode`` in one launch.

    ``new_keys / new_values [S, Hkv, D]`` belong to position ``sequence_lengths[s] - 1`` (the lengths already
    count the new token).  The pools are updated in place exactly as ``fill_kv_pages`` would; returns the
    attention output ``[S, Hq, D]``.
    """
    S, hq, hkv, d, tpp, num_pages = _decode_shapes(queries, k_cache_pool, v_cache_pool, page_table, sequence_lengths)
    for name, t in (("new_keys", new_keys), ("new_values", new_values)):
        _need_cuda(name, t)
        if tuple(t.shape) != (S, hkv, d) or t.dtype != queries.dtype:
            raise ValueError(f"{name} must be [{S}, {hkv}, {d}] of {queries.dtype}")
    dev = queries.device
    out = torch.empty((S, hq, d), dtype=queries.dtype, device=dev)
    if S == 0:
        return out
    q = _contig(queries)
    nk, nv = _contig(new_keys), _contig(new_values)
    pt = _index32("page_table", page_table)
    lens = _index32("sequence_lengths", sequence_lengths)
    pp = _lib.PAL_DECODE_AUTO if partition_pages is None else int(partition_pages)
    with _on(dev):
        sp = _stream_ptr(stream, dev)
        ws = _workspace(_decode_ws_bytes(S, hq, hkv, d, tpp, pt.shape[1], pp), dev, sp)
        rc = lib.pal_paged_attention_decode_append(nk.data_ptr(), nv.data_ptr(), q.data_ptr(), _ptr(k_cache_pool),
                                                   _ptr(v_cache_pool), _ptr(pt), lens.data_ptr(), out.data_ptr(), S, hq, hkv, d,
                                                   tpp, num_pages, pt.shape[1], 0.0 if scale is None else float(scale),
                                                   _dtype_code(q.dtype), pp, ws.data_ptr(), ws.numel(), sp)
        _lib.check(rc)
    return out


def paged_attention_decode_partials(queries, k_cache_pool, v_cache_pool, page_table, sequence_lengths, *,
                                    partition_pages: int = 256, scale=None, stream=None):
    """Split-KV pass without the final normalisation: returns fp32 ``(m [S,Hq], l [S,Hq], acc [S,Hq,D])``.

    For callers that merge partial results themselves, e.g. GPUs that each hold a slice of every
    sequence's context; merge with :func:`lse_combine`.
    """
    S, hq, hkv, d, tpp, num_pages = _decode_shapes(queries, k_cache_pool, v_cache_pool, page_table, sequence_lengths)
    dev = queries.device
    m = torch.empty((S, hq), dtype=torch.float32, device=dev)
    l = torch.empty((S, hq), dtype=torch.float32, device=dev)
    acc = torch.empty((S, hq, d), dtype=torch.float32, device=dev)
    if S == 0:
        return m, l, acc
    q = _contig(queries)
    pt = _index32("page_table", page_table)
    lens = _index32("sequence_lengths", sequence_lengths)
    with _on(dev):
        sp = _stream_ptr(stream, dev)
        ws = _workspace(_decode_ws_bytes(S, hq, hkv, d, tpp, pt.shape[1], int(partition_pages)), dev, sp)
        rc = lib.pal_paged_attention_decode_partials(q.data_ptr(), _ptr(k_cache_pool), _ptr(v_cache_pool), _ptr(pt),
                                                     lens.data_ptr(), m.data_ptr(), l.data_ptr(), acc.data_ptr(), S, hq, hkv, d,
                                                     tpp, num_pages, pt.shape[1], 0.0 if scale is None else float(scale),
                                                     _dtype_code(q.dtype), int(partition_pages), ws.data_ptr(), ws.numel(),
                                                     sp)
        _lib.check(rc)
    return m, l, acc


def lse_combine(m, l, acc, out_dtype=torch.bfloat16, *, stream=None):
    """Merge partial triples along their leading axis: ``m, l [parts, ...]``, ``acc [parts, ..., D]`` -> ``[..., D]``."""
    for name, t in (("m", m), ("l", l), ("acc", acc)):
        _need_cuda(name, t)
        if t.dtype != torch.float32:
            raise ValueError(f"{name} must be float32")
    parts = m.shape[0]
    d = acc.shape[-1]
    if m.shape != l.shape or acc.shape[:-1] != m.shape:
        raise ValueError("m, l and acc shapes do not agree")
    rows = m[0].numel()
    out = torch.empty(tuple(acc.shape[1:]), dtype=out_dtype, device=m.device)
    if rows == 0:
        return out
    m, l, acc = _contig(m), _contig(l), _contig(acc)
    with torch.cuda.device(m.device):
        _lib.check(lib.pal_lse_combine(m.data_ptr(), l.data_ptr(), acc.data_ptr(), out.data_ptr(), parts, rows, d,
                                       _dtype_code(out_dtype), _stream_ptr(stream, m.device)))
    return out


# ---------------------------------------------------------------------------------------------
# paged_attention_prefill (src/proxy_attention_lab/ops.py:87-130, src/pal_core/src/ops.cpp:110-185)
# ---------------------------------------------------------------------------------------------
PREFILL_IMPL = {"auto": 0, "mma": 1, "tcgen05": 2}


def paged_attention_prefill(q_prompt, k_prompt, v_prompt, k_cache_paged, v_cache_paged, page_table, context_len_arr, *,
                            stream=None, impl="auto", scale=None):
    """Causal attention of N new tokens per sequence over their paged history plus themselves.

    ``q_prompt [S*N, Hq, D]``, ``k_prompt / v_prompt [S*N, Hkv, D]`` (sequence-major), history in
    the pools through ``page_table [S, max_pages]`` with ``context_len_arr [S]`` history lengths.
    Returns ``[S*N*Hq, D]`` (row ``(s*N + i)*Hq + h``), as the reference does
    (``src/pal_core/src/paged_attention_prefill_primitive.cpp:188-192``).
    """
    for name, t in (("q_prompt", q_prompt), ("k_prompt", k_prompt), ("v_prompt", v_prompt),
                    ("k_cache_paged", k_cache_paged), ("v_cache_paged", v_cache_paged), ("page_table", page_table),
                    ("context_len_arr", context_len_arr)):
        _need_cuda(name, t)
    if v_cache_paged.dim() != 4 or k_cache_paged.dim() != 5:
        raise ValueError("k_cache_paged must be 5-D and v_cache_paged 4-D")
    num_pages, hkv, d, tpp = v_cache_paged.shape
    if q_prompt.dim() != 3 or k_prompt.dim() != 3 or v_prompt.dim() != 3:
        raise ValueError("q_prompt, k_prompt and v_prompt must be 3-D [tokens, heads, head_dim]")
    if not (q_prompt.dtype == k_prompt.dtype == v_prompt.dtype == k_cache_paged.dtype == v_cache_paged.dtype):
        raise ValueError("all data tensors must share one dtype")
    total, hq, dq = q_prompt.shape
    if dq != d or tuple(k_prompt.shape) != (total, hkv, d) or tuple(v_prompt.shape) != (total, hkv, d):
        raise ValueError("prompt tensor shapes do not match the cache (expected k/v [tokens, kv_heads, head_dim])")
    if page_table.dim() != 2:
        raise ValueError("page_table must be 2-D [num_sequences, max_logical_pages]")
    S = context_len_arr.numel()
    if S == 0 or total % S != 0:
        # every sequence carries the same number of new tokens (paged_attention_prefill_primitive.cpp:115-116)
        raise ValueError("the number of prompt tokens must be a multiple of the number of sequences")
    if page_table.shape[0] < S:
        raise ValueError("page_table has fewer rows than there are sequences")
    if hq % hkv != 0:
        raise ValueError(f"num_q_heads ({hq}) must be a multiple of num_kv_heads ({hkv})")
    n = total // S
    dev = q_prompt.device
    out = torch.empty((total * hq, d), dtype=q_prompt.dtype, device=dev)
    if total == 0:
        return out
    q, k, v = _contig(q_prompt), _contig(k_prompt), _contig(v_prompt)
    if not (k_cache_paged.is_contiguous() and v_cache_paged.is_contiguous()):
        raise ValueError("the page pools must be contiguous")
    pt = _index32("page_table", page_table)
    ctx = _index32("context_len_arr", context_len_arr)
    with _on(dev):
        sp = _stream_ptr(stream, dev)
        ws = _workspace(lib.pal_prefill_workspace_bytes(S, n, hq, hkv, d), dev, sp)
        rc = lib.pal_paged_attention_prefill(q.data_ptr(), k.data_ptr(), v.data_ptr(), _ptr(k_cache_paged), _ptr(v_cache_paged),
                                             _ptr(pt), ctx.data_ptr(), out.data_ptr(), S, n, hq, hkv, d, tpp, num_pages,
                                             pt.shape[1], 0.0 if scale is None else float(scale), _dtype_code(q.dtype),
                                             PREFILL_IMPL[impl] if isinstance(impl, str) else int(impl), ws.data_ptr(),
                                             ws.numel(), sp)
        _lib.check(rc)
    return out


def paged_attention_prefill_ragged(q_prompt, k_prompt, v_prompt, k_cache_paged, v_cache_paged, page_table, context_len_arr,
                                   cu_seqlens, *, max_new_tokens=None, stream=None, impl="auto", scale=None):
    """``paged_attention_prefill`` for batches whose sequences bring different numbers of new tokens.

    ``cu_seqlens [S + 1]`` (int32, starting at 0) gives each sequence's first row in ``q_prompt [T, Hq, D]`` and
    ``k_prompt / v_prompt [T, Hkv, D]``; sequence ``s`` owns rows ``cu_seqlens[s] .. cu_seqlens[s+1] - 1``.  A count of 1
    is a decode step, so prefill chunks and decode steps can share one call.  ``max_new_tokens`` (the largest count)
    is read back from ``cu_seqlens`` when not given, which synchronises with the device.  Returns ``[T*Hq, D]``.
    """
    for name, t in (("q_prompt", q_prompt), ("k_prompt", k_prompt), ("v_prompt", v_prompt),
                    ("k_cache_paged", k_cache_paged), ("v_cache_paged", v_cache_paged), ("page_table", page_table),
                    ("context_len_arr", context_len_arr), ("cu_seqlens", cu_seqlens)):
        _need_cuda(name, t)
    if v_cache_paged.dim() != 4 or k_cache_paged.dim() != 5:
        raise ValueError("k_cache_paged must be 5-D and v_cache_paged 4-D")
    num_pages, hkv, d, tpp = v_cache_paged.shape
    if q_prompt.dim() != 3 or k_prompt.dim() != 3 or v_prompt.dim() != 3:
        raise ValueError("q_prompt, k_prompt and v_prompt must be 3-D [tokens, heads, head_dim]")
    if not (q_prompt.dtype == k_prompt.dtype == v_prompt.dtype == k_cache_paged.dtype == v_cache_paged.dtype):
        raise ValueError("all data tensors must share one dtype")
    total, hq, dq = q_prompt.shape
    if dq != d or tuple(k_prompt.shape) != (total, hkv, d) or tuple(v_prompt.shape) != (total, hkv, d):
        raise ValueError("prompt tensor shapes do not match the cache (expected k/v [tokens, kv_heads, head_dim])")
    if page_table.dim() != 2:
        raise ValueError("page_table must be 2-D [num_sequences, max_logical_pages]")
    S = context_len_arr.numel()
    if cu_seqlens.dim() != 1 or cu_seqlens.numel() != S + 1:
        raise ValueError("cu_seqlens must hold num_sequences + 1 row offsets")
    if page_table.shape[0] < S:
        raise ValueError("page_table has fewer rows than there are sequences")
    if hq % hkv != 0:
        raise ValueError(f"num_q_heads ({hq}) must be a multiple of num_kv_heads ({hkv})")
    dev = q_prompt.device
    out = torch.empty((total * hq, d), dtype=q_prompt.dtype, device=dev)
    if total == 0 or S == 0:
        return out
    cu = _index32("cu_seqlens", cu_seqlens)
    if max_new_tokens is None:
        max_new_tokens = int((cu[1:] - cu[:-1]).max().item())
    q, k, v = _contig(q_prompt), _contig(k_prompt), _contig(v_prompt)
    if not (k_cache_paged.is_contiguous() and v_cache_paged.is_contiguous()):
        raise ValueError("the page pools must be contiguous")
    pt = _index32("page_table", page_table)
    ctx = _index32("context_len_arr", context_len_arr)
    with _on(dev):
        sp = _stream_ptr(stream, dev)
        ws = _workspace(lib.pal_prefill_workspace_bytes(S, int(max_new_tokens), hq, hkv, d), dev, sp)
        rc = lib.pal_paged_attention_prefill_ragged(q.data_ptr(), k.data_ptr(), v.data_ptr(), _ptr(k_cache_paged),
                                                    _ptr(v_cache_paged), _ptr(pt), ctx.data_ptr(), cu.data_ptr(), out.data_ptr(),
                                                    S, total, int(max_new_tokens), hq, hkv, d, tpp, num_pages, pt.shape[1],
                                                    0.0 if scale is None else float(scale), _dtype_code(q.dtype),
                                                    PREFILL_IMPL[impl] if isinstance(impl, str) else int(impl), ws.data_ptr(),
                                                    ws.numel(), sp)
        _lib.check(rc)
    return out


def paged_attention(queries, k_cache_pool, v_cache_pool, page_table, sequence_lengths, *, k_prompt=None, v_prompt=None,
                    stream=None, **kw):
    """Single entry point: decode when no prompt K/V are given, prefill otherwise."""
    if k_prompt is None and v_prompt is None:
        return paged_attention_decode(queries, k_cache_pool, v_cache_pool, page_table, sequence_lengths, stream=stream, **kw)
    return paged_attention_prefill(queries, k_prompt, v_prompt, k_cache_pool, v_cache_pool, page_table, sequence_lengths,
                                   stream=stream, **kw)
