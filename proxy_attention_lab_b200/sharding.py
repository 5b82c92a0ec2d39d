"""Host-side plumbing for running the operators on several GPUs of one node.

The attention output of (sequence s, query head h) depends only on that sequence's pages of kv head
``h // group``, so a batch shards by sequence and by kv head with no communication at all.  The one
exchange step is the long-context layout in which every GPU holds a slice of each sequence's
context: each rank produces un-normalised ``(m, l, acc)`` partials over its slice, the partials are
all-gathered (NCCL over NVLink on GPUs) and merged by the log-sum-exp combine kernel.

The reference has no multi-device code (it is a single-GPU MLX extension); this module has no
counterpart there.
"""

from __future__ import annotations

from typing import Callable, List, Sequence

import torch
import torch.distributed as dist


def partition_sequences(lengths: Sequence[int], world_size: int) -> List[List[int]]:
    """Greedy longest-first assignment of sequences to ranks, balancing the tokens each rank streams."""
    order = sorted(range(len(lengths)), key=lambda i: (-int(lengths[i]), i))
    loads = [0] * world_size
    parts: List[List[int]] = [[] for _ in range(world_size)]
    for i in order:
        r = min(range(world_size), key=lambda j: (loads[j], j))
        parts[r].append(i)
        loads[r] += int(lengths[i])
    for p in parts:
        p.sort()
    return parts


def kv_head_range(num_kv_heads: int, world_size: int, rank: int) -> range:
    """Contiguous kv heads owned by ``rank`` (the query heads ``h*group .. (h+1)*group-1`` go with them)."""
    if num_kv_heads % world_size != 0:
        raise ValueError(f"num_kv_heads ({num_kv_heads}) must be a multiple of the world size ({world_size})")
    per = num_kv_heads // world_size
    return range(rank * per, (rank + 1) * per)


def context_slice(num_pages: int, world_size: int, rank: int) -> range:
    """Logical pages of a sequence owned by ``rank`` when its context is cut into contiguous slices."""
    per = (num_pages + world_size - 1) // world_size
    lo = min(rank * per, num_pages)
    return range(lo, min(lo + per, num_pages))


def all_gather_partials(m: torch.Tensor, l: torch.Tensor, acc: torch.Tensor, group=None):
    """All-gather one ``(m [R], l [R], acc [R, D])`` triple per rank into ``[world, ...]`` stacks.

    Convenience form for callers that hold the three tensors separately; it packs, gathers and unpacks with
    several small copies.  The hot path is :func:`all_gather_packed`, which moves the buffer the kernel wrote.
    """
    world = dist.get_world_size(group)
    rows, d = acc.shape[:-1], acc.shape[-1]
    packed = torch.cat([acc.reshape(-1, d), m.reshape(-1, 1), l.reshape(-1, 1)], dim=1).contiguous()
    out = all_gather_packed(packed, group=group)
    acc_all = out[:, :, :d].reshape((world,) + tuple(rows) + (d,))
    m_all = out[:, :, d].reshape((world,) + tuple(rows))
    l_all = out[:, :, d + 1].reshape((world,) + tuple(rows))
    return m_all.contiguous(), l_all.contiguous(), acc_all.contiguous()


def all_gather_packed(packed: torch.Tensor, out: torch.Tensor = None, group=None) -> torch.Tensor:
    """One collective for the whole exchange: every rank contributes its packed ``[rows, D + 2]`` partials (``acc``, then
    ``m``, then ``l`` per row, as ``paged_attention_decode_partials(..., packed=True)`` writes them) and receives
    ``[world, rows, D + 2]``, which ``lse_combine_packed`` reads in place.  The payload is small (266 KB per GPU for batch
    8 x 64 heads x D = 128), so the step is latency-bound: nothing is copied before or after the collective."""
    world = dist.get_world_size(group)
    if out is None:
        out = torch.empty((world,) + tuple(packed.shape), dtype=packed.dtype, device=packed.device)
    dist.all_gather_into_tensor(out.view(world * packed.shape[0], packed.shape[1]), packed, group=group)
    return out


def decode_context_parallel(partials_fn: Callable[[], tuple], combine_fn: Callable, group=None):
    """Long-context decode with the context of every sequence sliced across the ranks of ``group``.

    ``partials_fn()`` returns this rank's partials over its slice: either the packed ``[rows, D + 2]`` buffer of
    ``paged_attention_decode_partials(..., packed=True)`` - then ``combine_fn(gathered)`` gets the ``[world, rows, D + 2]``
    stack (on GPUs: ``lse_combine_packed``) - or a ``(m, l, acc)`` triple, then ``combine_fn(m_all, l_all, acc_all)`` gets the
    three stacks (``lse_combine``).  Every rank ends up with the full result.
    """
    part = partials_fn()
    if isinstance(part, torch.Tensor):
        return combine_fn(all_gather_packed(part, group=group))
    m_all, l_all, acc_all = all_gather_partials(*part, group=group)
    return combine_fn(m_all, l_all, acc_all)


class ContextExchange:
    """Peer-memory exchange for context-sharded decode: the fused alternative to ``all_gather_packed`` + ``lse_combine_packed``.

    Every rank allocates one exchange buffer in symmetric memory (``torch.distributed._symmetric_memory``, which maps each
    rank's buffer into every process of the group over NVLink), zeroes it, and from then on one call of :meth:`decode` per
    step runs the split-KV pass over the rank's slice of the context plus ONE kernel that publishes the rank's merged
    partials to all peers with plain stores, waits (bounded) for theirs and writes the full attention output.  No
    collective is issued and nothing is copied on the host side of a step.

    ``rows`` is the largest ``num_sequences * num_q_heads`` a step will carry.  All ranks of ``group`` construct the object
    together and call :meth:`decode` once per step in the same order.  Multicast (NVLS) is not used and is switched off
    for the allocation.
    """

    def __init__(self, rows: int, head_dim: int, device, group=None):
        import ctypes
        import os

        import torch.distributed._symmetric_memory as symm_mem

        from . import _lib

        self._lib = _lib
        group = dist.group.WORLD if group is None else group
        self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)
        self.rows, self.head_dim, self.device = int(rows), int(head_dim), torch.device(device)
        nbytes = _lib.lib.pal_exchange_bytes(self.world, self.rows, self.head_dim)
        os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")  # plain peer stores only: nothing binds to a multicast object
        self.buffer = symm_mem.empty(nbytes, dtype=torch.uint8, device=self.device)
        self.buffer.zero_()
        self.handle = symm_mem.rendezvous(self.buffer, group.group_name)
        ptrs = [int(p) for p in self.handle.buffer_ptrs]
        if len(ptrs) != self.world or any(p == 0 for p in ptrs):
            raise RuntimeError("symmetric memory did not return a peer mapping for every rank")
        self._peer_bases = (ctypes.c_void_p * self.world)(*ptrs)
        torch.cuda.synchronize(self.device)
        dist.barrier(group)  # every rank's buffer is zero before anyone's first step

    def decode(self, queries, k_cache_pool, v_cache_pool, page_table, sequence_lengths, *, partition_pages=256,
               scale=None, out_dtype=None, stream=None):
        """``paged_attention_decode`` over a context that is sliced across the ranks: ``page_table`` / ``sequence_lengths``
        describe this rank's slice (length 0 where the rank holds nothing of a sequence), ``queries`` are the same on every
        rank.  ``partition_pages=None`` lets the library size the partitions of the local split-KV pass.  Returns the full
        ``[S, Hq, D]`` result on every rank."""
        from . import ops

        _lib, lib = self._lib, self._lib.lib
        S, hq, hkv, d, tpp, num_pages = ops._decode_shapes(queries, k_cache_pool, v_cache_pool, page_table, sequence_lengths)
        if S * hq > self.rows or d != self.head_dim:
            raise ValueError(f"this exchange was sized for {self.rows} rows of head_dim {self.head_dim}, got {S * hq} x {d}")
        if S == 0 or page_table.shape[1] == 0:
            raise ValueError("every rank takes part in every step: the batch and the page table must not be empty")
        code, odt = ops._out_code(queries.dtype, out_dtype)
        partition_pages = ops.resolve_partition_pages(partition_pages, S, hq, hkv, d, tpp, page_table.shape[1])
        with ops._Scope(self.device, stream) as sp:
            out = torch.empty((S, hq, d), dtype=odt, device=self.device)
            q = ops._contig(queries)
            pt = ops._index32("page_table", page_table)
            lens = ops._index32("sequence_lengths", sequence_lengths)
            ws = ops._workspace(ops._decode_ws_bytes(S, hq, hkv, d, tpp, pt.shape[1], int(partition_pages)), self.device, sp)
            rc = lib.pal_paged_attention_decode_ctx_exchange(
                q.data_ptr(), ops._ptr(k_cache_pool), ops._ptr(v_cache_pool), pt.data_ptr(), lens.data_ptr(), out.data_ptr(), S, hq,
                hkv, d, tpp, num_pages, pt.shape[1], 0.0 if scale is None else float(scale), code, int(partition_pages),
                ws.data_ptr(), ws.numel(), self._peer_bases, self.world, self.rank, self.rows, sp)
            _lib.check(rc)
        return out
