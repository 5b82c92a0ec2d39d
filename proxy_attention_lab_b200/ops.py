"""Proxy Attention Lab's operator API on PyTorch CUDA tensors, backed by libpal_b200.so.

Same names, argument order and cache layouts as the reference's Python layer
(``src/proxy_attention_lab/ops.py:33-171``, bound in ``src/pal_core/bindings.cpp:44-222``),
with ``torch.Tensor`` where the reference takes ``mx.array`` and eager launches on a CUDA stream
where the reference builds lazy MLX graph nodes.  Every operator launches hand-written sm_100a
kernels through the C ABI; nothing here computes on the host and there is no fallback path.

Streams: ``stream=None`` means torch's current stream.  When a stream is named (a
``torch.cuda.Stream`` or a raw ``cudaStream_t`` integer) the whole operator - index conversions,
contiguity copies, output and workspace allocation, and the launch - runs with that stream current,
so everything the kernel reads is ordered before it and the outputs belong to that stream.
"""

from __future__ import annotations

import functools

import torch

from . import _lib
from ._lib import lib

try:  # C++ front of the hot operators (csrc/torch_fastpath.cpp): same C-ABI calls, without ctypes and Python-side checks
    from . import _pal_fast as _fast
except ImportError:  # not built: every call takes the ctypes path below
    _fast = None

_DTYPES = {torch.float16: _lib.PAL_DTYPE_F16, torch.bfloat16: _lib.PAL_DTYPE_BF16}


def _dtype_code(dtype: torch.dtype) -> int:
    try:
        return _DTYPES[dtype]
    except KeyError:
        raise ValueError(f"dtype {dtype} is not supported (float16 and bfloat16 are)") from None


def _out_code(in_dtype: torch.dtype, out_dtype) -> tuple:
    """(dtype argument of the C call, torch dtype of the output): the input type, or float32 on request."""
    code = _dtype_code(in_dtype)
    if out_dtype is None or out_dtype == in_dtype:
        return code, in_dtype
    if out_dtype == torch.float32:
        return code | _lib.PAL_OUT_F32, torch.float32
    raise ValueError(f"out_dtype must be None, the input dtype ({in_dtype}) or torch.float32, got {out_dtype}")


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


class _Scope:
    """Makes ``device`` current and, when the caller named a stream, makes that stream torch's current one for the
    duration of an operator; yields the raw ``cudaStream_t``.  Costs two cheap queries when nothing has to change."""

    __slots__ = ("device", "stream", "_guards")

    def __init__(self, device, stream):
        if stream is not None and not isinstance(stream, (torch.cuda.Stream, int)):
            raise TypeError("stream must be None, a torch.cuda.Stream or a raw cudaStream_t integer")
        self.device, self.stream, self._guards = device, stream, None

    def __enter__(self) -> int:
        dev, stream = self.device, self.stream
        guards = []
        if torch.cuda.current_device() != dev.index:
            g = torch.cuda.device(dev)
            g.__enter__()
            guards.append(g)
        if stream is not None:
            if isinstance(stream, int):
                stream = torch.cuda.ExternalStream(stream, device=dev)
            if stream.cuda_stream != torch.cuda.current_stream(dev).cuda_stream:
                g = torch.cuda.stream(stream)
                g.__enter__()
                guards.append(g)
        self._guards = guards
        return torch.cuda.current_stream(dev).cuda_stream

    def __exit__(self, *exc):
        for g in reversed(self._guards):
            g.__exit__(*exc)
        return False


# (device index, stream) -> every scratch buffer ever handed out for that pair, newest (largest) last
_WORKSPACES: dict = {}


def _workspace(nbytes: int, device, stream_ptr: int) -> torch.Tensor:
    """Scratch for one call, allocated (zeroed, as the C ABI asks for the header) on the stream that will use it.

    Calls on one stream run in order, so they share one buffer per (device, stream).  When a call needs more than the
    newest buffer holds, a larger one (at least twice the size) is added; the earlier buffers are kept for the life of
    the process, because a CUDA graph captured from an earlier call still writes to the address it recorded.
    """
    need = max(int(nbytes), 256)
    key = (device.index, stream_ptr)
    held = _WORKSPACES.get(key)
    if held is None:
        held = _WORKSPACES[key] = []
    if not held or held[-1].numel() < need:
        held.append(torch.zeros(max(need, 2 * held[-1].numel() if held else 4096), dtype=torch.uint8, device=device))
    return held[-1]


@functools.lru_cache(maxsize=256)
def _decode_ws_bytes(S, hq, hkv, d, tpp, mp, pp) -> int:
    return lib.pal_decode_workspace_bytes(S, hq, hkv, d, tpp, mp, pp)


@functools.lru_cache(maxsize=256)
def _prefill_ws_bytes(S, n, hq, hkv, d) -> int:
    return lib.pal_prefill_workspace_bytes(S, n, hq, hkv, d)


def resolve_partition_pages(partition_pages, S, hq, hkv, d, tpp, max_pages) -> int:
    """Partition size of a split-KV pass that always splits (the partials forms): a positive request is taken as it is,
    ``None`` / ``PAL_DECODE_AUTO`` asks the library, and where the library would run a single pass the whole page table
    is one partition."""
    if partition_pages is not None and int(partition_pages) > 0:
        return int(partition_pages)
    pp = lib.pal_decode_auto_partition_pages(S, hq, hkv, d, tpp, max_pages) if (S > 0 and max_pages > 0) else 0
    return pp if pp > 0 else max(int(max_pages), 1)


def check_status(stream=None, device=None) -> None:
    """Raise ``RuntimeError`` if a kernel of the last call on this (device, stream) gave up a bounded wait.

    Synchronises with the stream; meant for tests and debugging."""
    device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    with _Scope(device, stream) as sp:
        held = _WORKSPACES.get((device.index, sp))
        if held:
            _lib.check(lib.pal_check_status(held[-1].data_ptr(), sp))


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
    if _fast is not None and stream is None and inplace:
        try:
            if slot_mapping is not None:
                done = page_table is None and _fast.fill(new_keys, new_values, global_key_pool, global_value_pool, slot_mapping, None, None)
            else:
                done = _fast.fill(new_keys, new_values, global_key_pool, global_value_pool, page_table, current_token_write_positions,
                                  query_to_seq_map)
        except TypeError:
            done = False
        if done:
            return global_key_pool, global_value_pool
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
    T = new_keys.shape[0]
    if slot_mapping is not None:
        _need_cuda("slot_mapping", slot_mapping)
        if slot_mapping.numel() != T:
            raise ValueError("slot_mapping must have one entry per new token")
    else:
        if page_table is None or current_token_write_positions is None or query_to_seq_map is None:
            raise ValueError("page_table, current_token_write_positions and query_to_seq_map are required")
        for name, t in (("page_table", page_table), ("current_token_write_positions", current_token_write_positions),
                        ("query_to_seq_map", query_to_seq_map)):
            _need_cuda(name, t)
        if page_table.dim() != 2:
            raise ValueError("page_table must be 2-D [num_sequences, max_logical_pages]")
        if current_token_write_positions.numel() != T or query_to_seq_map.numel() != T:
            raise ValueError("write positions and query_to_seq_map must have one entry per new token")
    dev = global_value_pool.device
    with _Scope(dev, stream) as sp:
        if not inplace:
            global_key_pool = global_key_pool.clone()
            global_value_pool = global_value_pool.clone()
        if not (global_key_pool.is_contiguous() and global_value_pool.is_contiguous()):
            raise ValueError("the page pools must be contiguous")
        if T == 0:
            return global_key_pool, global_value_pool
        new_keys, new_values = _contig(new_keys), _contig(new_values)
        if slot_mapping is not None:
            slots = _contig(slot_mapping.to(torch.int64))
            rc = lib.pal_fill_kv_pages_slots(new_keys.data_ptr(), new_values.data_ptr(), global_key_pool.data_ptr(),
                                             global_value_pool.data_ptr(), slots.data_ptr(), T, hkv, d, tpp, num_pages, dt, sp)
        else:
            pt = _index32("page_table", page_table)
            pos = _index32("current_token_write_positions", current_token_write_positions)
            seqmap = _index32("query_to_seq_map", query_to_seq_map)
            rc = lib.pal_fill_kv_pages(new_keys.data_ptr(), new_values.data_ptr(), global_key_pool.data_ptr(),
                                       global_value_pool.data_ptr(), pt.data_ptr(), pos.data_ptr(), seqmap.data_ptr(), T,
                                       pt.shape[0], hkv, d, tpp, num_pages, pt.shape[1], dt, sp)
        _lib.check(rc)
    return global_key_pool, global_value_pool


# ---------------------------------------------------------------------------------------------
# paged_attention_decode (src/proxy_attention_lab/ops.py:42-84, src/pal_core/src/ops.cpp:36-108)
# ---------------------------------------------------------------------------------------------
def _decode_shapes(queries, k_cache_pool, v_cache_pool, page_table, sequence_lengths):
    # (this runs on every call: each tensor attribute is read once)
    try:
        on_gpu = queries.is_cuda and k_cache_pool.is_cuda and v_cache_pool.is_cuda and page_table.is_cuda and sequence_lengths.is_cuda
    except AttributeError:
        on_gpu = False
    if not on_gpu:
        for name, t in (("queries", queries), ("k_cache_pool", k_cache_pool), ("v_cache_pool", v_cache_pool),
                        ("page_table", page_table), ("sequence_lengths", sequence_lengths)):
            _need_cuda(name, t)
    vs, ks, qs, ps = v_cache_pool.shape, k_cache_pool.shape, queries.shape, page_table.shape
    if len(vs) != 4 or len(ks) != 5:
        raise ValueError("k_cache_pool must be 5-D and v_cache_pool 4-D")
    num_pages, hkv, d, tpp = vs  # ops.cpp:50-60
    if ks != (num_pages, hkv, d // 8, tpp, 8):
        raise ValueError("k_cache_pool shape does not match v_cache_pool")
    if not (k_cache_pool.is_contiguous() and v_cache_pool.is_contiguous()):
        raise ValueError("the page pools must be contiguous")
    if not (queries.dtype == k_cache_pool.dtype == v_cache_pool.dtype):
        raise ValueError("queries and both pools must share one dtype")
    if len(ps) != 2:
        raise ValueError("page_table must be 2-D [num_sequences, max_logical_pages]")
    S = ps[0]
    # ops.cpp:62-66: the head count comes from a 3-D query only; the kernel then reads row s of the flat buffer as
    # Hq * D elements (paged_attention_decode.h.metal:106-108), whatever the number of dimensions.
    qdim = len(qs)
    hq = qs[1] if qdim == 3 else 1
    if qdim == 2 or qdim == 3:
        if qs[-1] != d:
            raise ValueError(f"queries head_dim {qs[-1]} does not match the cache head_dim {d}")
        if qs[0] < S:
            raise ValueError("queries has fewer rows than page_table has sequences")
    elif qdim == 1:
        # a flat buffer of S rows of head_dim elements, one query head
        if queries.numel() < S * d or queries.numel() % d != 0:
            raise ValueError(f"1-D queries must hold a whole number (>= {S}) of rows of head_dim = {d} elements, got {queries.numel()} elements")
    else:
        raise ValueError("queries must be 1-D, 2-D [S, D] or 3-D [S, Hq, D]")
    if sequence_lengths.numel() < S:
        raise ValueError("sequence_lengths has fewer entries than page_table has sequences")
    if hq % hkv != 0:
        raise ValueError(f"num_q_heads ({hq}) must be a multiple of num_kv_heads ({hkv})")
    return S, hq, hkv, d, tpp, num_pages


def paged_attention_decode(queries, k_cache_pool, v_cache_pool, page_table, sequence_lengths, *, stream=None,
                           partition_pages=None, scale=None, out_dtype=None):
    """One query token per sequence attending to its paged KV history.

    ``queries [>=S, Hq, D]`` (2-D ``[>=S, D]`` or a flat 1-D buffer of such rows means one query head), pools in the
    reference layouts, ``page_table [S, max_pages]``, ``sequence_lengths [S]``.  Returns ``[S, Hq, D]`` in the query
    dtype, or in float32 with ``out_dtype=torch.float32`` (same arithmetic, the final rounding to 16 bits left out).
    ``partition_pages``: None = let the library choose, 0 = fused single pass, n > 0 = two-pass split-KV with n-page
    partitions and a log-sum-exp combine.
    """
    if _fast is not None and stream is None and (out_dtype is None or out_dtype is torch.float32):
        # the common case (3-D queries, contiguous tensors, 32-bit indices, a workspace from an earlier call) from C++;
        # None means "not the common case": the checks and conversions below then run as usual
        try:
            out = _fast.decode(queries, k_cache_pool, v_cache_pool, page_table, sequence_lengths,
                               _lib.PAL_DECODE_AUTO if partition_pages is None else int(partition_pages),
                               0.0 if scale is None else float(scale), out_dtype is torch.float32, _WORKSPACES, None, None)
        except TypeError:
            out = None
        if out is not None:
            return out
    S, hq, hkv, d, tpp, num_pages = _decode_shapes(queries, k_cache_pool, v_cache_pool, page_table, sequence_lengths)
    dev = queries.device
    code, odt = _out_code(queries.dtype, out_dtype)
    pp = _lib.PAL_DECODE_AUTO if partition_pages is None else int(partition_pages)
    with _Scope(dev, stream) as sp:
        out = torch.empty((S, hq, d), dtype=odt, device=dev)
        if S == 0:
            return out
        q = _contig(queries)
        pt = _index32("page_table", page_table)
        lens = _index32("sequence_lengths", sequence_lengths)
        mp = pt.shape[1]
        ws = _workspace(_decode_ws_bytes(S, hq, hkv, d, tpp, mp, pp), dev, sp)
        rc = lib.pal_paged_attention_decode(q.data_ptr(), k_cache_pool.data_ptr() if num_pages else 0,
                                            v_cache_pool.data_ptr() if num_pages else 0, pt.data_ptr() if mp else 0, lens.data_ptr(),
                                            out.data_ptr(), S, hq, hkv, d, tpp, num_pages, mp,
                                            0.0 if scale is None else float(scale), code, pp, ws.data_ptr(), ws.numel(), sp)
        if rc:
            _lib.check(rc)
    return out


def paged_attention_decode_append(new_keys, new_values, queries, k_cache_pool, v_cache_pool, page_table, sequence_lengths, *,
                                  stream=None, partition_pages=None, scale=None, out_dtype=None):
    """``fill_kv_pages`` of each sequence's newest token and ``paged_attention_decode`` in one launch.

    ``new_keys / new_values [S, Hkv, D]`` belong to position ``sequence_lengths[s] - 1`` (the lengths already
    count the new token).  The pools are updated in place exactly as ``fill_kv_pages`` would; returns the
    attention output ``[S, Hq, D]``.
    """
    if _fast is not None and stream is None and (out_dtype is None or out_dtype is torch.float32):
        try:
            out = _fast.decode(queries, k_cache_pool, v_cache_pool, page_table, sequence_lengths,
                               _lib.PAL_DECODE_AUTO if partition_pages is None else int(partition_pages),
                               0.0 if scale is None else float(scale), out_dtype is torch.float32, _WORKSPACES, new_keys, new_values)
        except TypeError:
            out = None
        if out is not None:
            return out
    S, hq, hkv, d, tpp, num_pages = _decode_shapes(queries, k_cache_pool, v_cache_pool, page_table, sequence_lengths)
    for name, t in (("new_keys", new_keys), ("new_values", new_values)):
        _need_cuda(name, t)
        if tuple(t.shape) != (S, hkv, d) or t.dtype != queries.dtype:
            raise ValueError(f"{name} must be [{S}, {hkv}, {d}] of {queries.dtype}")
    dev = queries.device
    code, odt = _out_code(queries.dtype, out_dtype)
    pp = _lib.PAL_DECODE_AUTO if partition_pages is None else int(partition_pages)
    with _Scope(dev, stream) as sp:
        out = torch.empty((S, hq, d), dtype=odt, device=dev)
        if S == 0:
            return out
        q = _contig(queries)
        nk, nv = _contig(new_keys), _contig(new_values)
        pt = _index32("page_table", page_table)
        lens = _index32("sequence_lengths", sequence_lengths)
        ws = _workspace(_decode_ws_bytes(S, hq, hkv, d, tpp, pt.shape[1], pp), dev, sp)
        rc = lib.pal_paged_attention_decode_append(nk.data_ptr(), nv.data_ptr(), q.data_ptr(), _ptr(k_cache_pool),
                                                   _ptr(v_cache_pool), _ptr(pt), lens.data_ptr(), out.data_ptr(), S, hq, hkv, d,
                                                   tpp, num_pages, pt.shape[1], 0.0 if scale is None else float(scale),
                                                   code, pp, ws.data_ptr(), ws.numel(), sp)
        _lib.check(rc)
    return out


def paged_attention_decode_partials(queries, k_cache_pool, v_cache_pool, page_table, sequence_lengths, *,
                                    partition_pages=256, scale=None, stream=None, packed: bool = False, out=None):
    """Split-KV pass without the final normalisation: returns fp32 ``(m [S,Hq], l [S,Hq], acc [S,Hq,D])``.

    For callers that merge partial results themselves, e.g. GPUs that each hold a slice of every
    sequence's context; merge with :func:`lse_combine`.  ``packed=True`` returns the same triple as one
    ``[S*Hq, D + 2]`` buffer (``acc``, then ``m``, then ``l`` in every row; written into ``out`` when given) - the
    form a single collective moves; merge gathered buffers with :func:`lse_combine_packed`.
    """
    S, hq, hkv, d, tpp, num_pages = _decode_shapes(queries, k_cache_pool, v_cache_pool, page_table, sequence_lengths)
    dev = queries.device
    partition_pages = resolve_partition_pages(partition_pages, S, hq, hkv, d, tpp, page_table.shape[1])
    with _Scope(dev, stream) as sp:
        if packed:
            if out is None:
                out = torch.empty((S * hq, d + 2), dtype=torch.float32, device=dev)
            elif out.dtype != torch.float32 or tuple(out.shape) != (S * hq, d + 2) or not out.is_contiguous() or out.device != dev:
                raise ValueError(f"out must be a contiguous float32 [{S * hq}, {d + 2}] tensor on {dev}")
            result = out
        else:
            m = torch.empty((S, hq), dtype=torch.float32, device=dev)
            l = torch.empty((S, hq), dtype=torch.float32, device=dev)
            acc = torch.empty((S, hq, d), dtype=torch.float32, device=dev)
            result = (m, l, acc)
        if S == 0:
            return result
        q = _contig(queries)
        pt = _index32("page_table", page_table)
        lens = _index32("sequence_lengths", sequence_lengths)
        ws = _workspace(_decode_ws_bytes(S, hq, hkv, d, tpp, pt.shape[1], int(partition_pages)), dev, sp)
        common = (S, hq, hkv, d, tpp, num_pages, pt.shape[1], 0.0 if scale is None else float(scale), _dtype_code(q.dtype),
                  int(partition_pages), ws.data_ptr(), ws.numel(), sp)
        if packed:
            rc = lib.pal_paged_attention_decode_partials_packed(q.data_ptr(), _ptr(k_cache_pool), _ptr(v_cache_pool), _ptr(pt),
                                                                lens.data_ptr(), out.data_ptr(), *common)
        else:
            rc = lib.pal_paged_attention_decode_partials(q.data_ptr(), _ptr(k_cache_pool), _ptr(v_cache_pool), _ptr(pt),
                                                         lens.data_ptr(), m.data_ptr(), l.data_ptr(), acc.data_ptr(), *common)
        _lib.check(rc)
    return result


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
    code = _lib.PAL_OUT_F32 if out_dtype == torch.float32 else _dtype_code(out_dtype)
    with _Scope(m.device, stream) as sp:
        out = torch.empty(tuple(acc.shape[1:]), dtype=out_dtype, device=m.device)
        if rows == 0:
            return out
        m, l, acc = _contig(m), _contig(l), _contig(acc)
        _lib.check(lib.pal_lse_combine(m.data_ptr(), l.data_ptr(), acc.data_ptr(), out.data_ptr(), parts, rows, d, code, sp))
    return out


def lse_combine_packed(packed, out_dtype=torch.bfloat16, *, out_shape=None, stream=None):
    """Merge packed partial triples ``[parts, rows, D + 2]`` (see :func:`paged_attention_decode_partials`) -> ``[rows, D]``
    (or ``out_shape``, e.g. ``(S, Hq, D)``), reading the gathered buffer in place."""
    _need_cuda("packed", packed)
    if packed.dtype != torch.float32 or packed.dim() != 3 or packed.shape[-1] < 3 or not packed.is_contiguous():
        raise ValueError("packed must be a contiguous float32 [parts, rows, D + 2] tensor")
    parts, rows, d = packed.shape[0], packed.shape[1], packed.shape[2] - 2
    code = _lib.PAL_OUT_F32 if out_dtype == torch.float32 else _dtype_code(out_dtype)
    with _Scope(packed.device, stream) as sp:
        out = torch.empty((rows, d) if out_shape is None else tuple(out_shape), dtype=out_dtype, device=packed.device)
        if out.numel() != rows * d:
            raise ValueError("out_shape does not hold rows * D elements")
        if rows == 0 or parts == 0:
            return out.zero_()
        _lib.check(lib.pal_lse_combine_packed(packed.data_ptr(), out.data_ptr(), parts, rows, d, code, sp))
    return out


# ---------------------------------------------------------------------------------------------
# paged_attention_prefill (src/proxy_attention_lab/ops.py:87-130, src/pal_core/src/ops.cpp:110-185)
# ---------------------------------------------------------------------------------------------
PREFILL_IMPL = {"auto": 0, "mma": 1, "tcgen05": 2, "tcgen05_single": 3, "tcgen05_pair": 4}


def _prefill_shapes(q_prompt, k_prompt, v_prompt, k_cache_paged, v_cache_paged, page_table, context_len_arr):
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
    if page_table.shape[0] < S:
        raise ValueError("page_table has fewer rows than there are sequences")
    if hq % hkv != 0:
        raise ValueError(f"num_q_heads ({hq}) must be a multiple of num_kv_heads ({hkv})")
    if not (k_cache_paged.is_contiguous() and v_cache_paged.is_contiguous()):
        raise ValueError("the page pools must be contiguous")
    return S, total, hq, hkv, d, tpp, num_pages


def paged_attention_prefill(q_prompt, k_prompt, v_prompt, k_cache_paged, v_cache_paged, page_table, context_len_arr, *,
                            stream=None, impl="auto", scale=None, out_dtype=None):
    """Causal attention of N new tokens per sequence over their paged history plus themselves.

    ``q_prompt [S*N, Hq, D]``, ``k_prompt / v_prompt [S*N, Hkv, D]`` (sequence-major), history in
    the pools through ``page_table [S, max_pages]`` with ``context_len_arr [S]`` history lengths.
    Returns ``[S*N*Hq, D]`` (row ``(s*N + i)*Hq + h``), as the reference does
    (``src/pal_core/src/paged_attention_prefill_primitive.cpp:188-192``), in the query dtype or, with
    ``out_dtype=torch.float32``, in float32.
    """
    if _fast is not None and stream is None and (out_dtype is None or out_dtype is torch.float32) and (impl in PREFILL_IMPL or type(impl) is int):
        try:
            out = _fast.prefill(q_prompt, k_prompt, v_prompt, k_cache_paged, v_cache_paged, page_table, context_len_arr,
                                PREFILL_IMPL[impl] if type(impl) is str else impl, 0.0 if scale is None else float(scale),
                                out_dtype is torch.float32, _WORKSPACES, None, 0)
        except TypeError:
            out = None
        if out is not None:
            return out
    S, total, hq, hkv, d, tpp, num_pages = _prefill_shapes(q_prompt, k_prompt, v_prompt, k_cache_paged, v_cache_paged,
                                                           page_table, context_len_arr)
    if S == 0 or total % S != 0:
        # every sequence carries the same number of new tokens (paged_attention_prefill_primitive.cpp:115-116)
        raise ValueError("the number of prompt tokens must be a multiple of the number of sequences")
    n = total // S
    dev = q_prompt.device
    code, odt = _out_code(q_prompt.dtype, out_dtype)
    with _Scope(dev, stream) as sp:
        out = torch.empty((total * hq, d), dtype=odt, device=dev)
        if total == 0:
            return out
        q, k, v = _contig(q_prompt), _contig(k_prompt), _contig(v_prompt)
        pt = _index32("page_table", page_table)
        ctx = _index32("context_len_arr", context_len_arr)
        ws = _workspace(_prefill_ws_bytes(S, n, hq, hkv, d), dev, sp)
        rc = lib.pal_paged_attention_prefill(q.data_ptr(), k.data_ptr(), v.data_ptr(), _ptr(k_cache_paged), _ptr(v_cache_paged),
                                             _ptr(pt), ctx.data_ptr(), out.data_ptr(), S, n, hq, hkv, d, tpp, num_pages,
                                             pt.shape[1], 0.0 if scale is None else float(scale), code,
                                             PREFILL_IMPL[impl] if isinstance(impl, str) else int(impl), ws.data_ptr(),
                                             ws.numel(), sp)
        _lib.check(rc)
    return out


def paged_attention_prefill_ragged(q_prompt, k_prompt, v_prompt, k_cache_paged, v_cache_paged, page_table, context_len_arr,
                                   cu_seqlens, *, max_new_tokens=None, stream=None, impl="auto", scale=None, out_dtype=None):
    """``paged_attention_prefill`` for batches whose sequences bring different numbers of new tokens.

    ``cu_seqlens [S + 1]`` (int32, starting at 0) gives each sequence's first row in ``q_prompt [T, Hq, D]`` and
    ``k_prompt / v_prompt [T, Hkv, D]``; sequence ``s`` owns rows ``cu_seqlens[s] .. cu_seqlens[s+1] - 1``.  A count of 1
    is a decode step, so prefill chunks and decode steps can share one call.  ``max_new_tokens`` (the largest count)
    is read back from ``cu_seqlens`` when not given, which synchronises with the device.  Returns ``[T*Hq, D]``.
    """
    if (_fast is not None and stream is None and max_new_tokens is not None and (out_dtype is None or out_dtype is torch.float32)
            and (impl in PREFILL_IMPL or type(impl) is int)):
        try:
            out = _fast.prefill(q_prompt, k_prompt, v_prompt, k_cache_paged, v_cache_paged, page_table, context_len_arr,
                                PREFILL_IMPL[impl] if type(impl) is str else impl, 0.0 if scale is None else float(scale),
                                out_dtype is torch.float32, _WORKSPACES, cu_seqlens, int(max_new_tokens))
        except TypeError:
            out = None
        if out is not None:
            return out
    _need_cuda("cu_seqlens", cu_seqlens)
    S, total, hq, hkv, d, tpp, num_pages = _prefill_shapes(q_prompt, k_prompt, v_prompt, k_cache_paged, v_cache_paged,
                                                           page_table, context_len_arr)
    if cu_seqlens.dim() != 1 or cu_seqlens.numel() != S + 1:
        raise ValueError("cu_seqlens must hold num_sequences + 1 row offsets")
    dev = q_prompt.device
    code, odt = _out_code(q_prompt.dtype, out_dtype)
    with _Scope(dev, stream) as sp:
        out = torch.empty((total * hq, d), dtype=odt, device=dev)
        if total == 0 or S == 0:
            return out
        cu = _index32("cu_seqlens", cu_seqlens)
        if max_new_tokens is None:
            max_new_tokens = int((cu[1:] - cu[:-1]).max().item())
        q, k, v = _contig(q_prompt), _contig(k_prompt), _contig(v_prompt)
        pt = _index32("page_table", page_table)
        ctx = _index32("context_len_arr", context_len_arr)
        ws = _workspace(_prefill_ws_bytes(S, int(max_new_tokens), hq, hkv, d), dev, sp)
        rc = lib.pal_paged_attention_prefill_ragged(q.data_ptr(), k.data_ptr(), v.data_ptr(), _ptr(k_cache_paged),
                                                    _ptr(v_cache_paged), _ptr(pt), ctx.data_ptr(), cu.data_ptr(), out.data_ptr(),
                                                    S, total, int(max_new_tokens), hq, hkv, d, tpp, num_pages, pt.shape[1],
                                                    0.0 if scale is None else float(scale), code,
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
