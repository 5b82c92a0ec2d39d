"""Cache layouts of the paged KV pools, restated on CPU (test infrastructure).

K pool ``[pages, kv_heads, head_dim/x, tokens_per_page, x]`` with ``x = 16 / sizeof(dtype)``
and V pool ``[pages, kv_heads, head_dim, tokens_per_page]`` follow
``src/pal_core/src/paged_attention_decode_primitive.cpp:373-397``.  Element addressing
follows ``src/pal_core/kernels/paged_attention/decode/paged_attention_decode.h.metal:142-190``
(K) and ``:248-295`` (V); the dense->paged packing recipe follows
``tests/paged_attention/decode/test_sdpa_equivalency.py:141-173``.
"""

from __future__ import annotations

import torch

MEMORY_ALIGNMENT_BYTES = 16  # src/pal_core/include/kernels/paged_attention_types.h:36


def k_cache_stripe_size(dtype: torch.dtype) -> int:
    """Elements per 16-byte stripe (``src/pal_core/bindings.cpp:44-46``)."""
    return MEMORY_ALIGNMENT_BYTES // torch.empty((), dtype=dtype).element_size()


def k_cache_shape(num_pages: int, num_kv_heads: int, head_dim: int, tokens_per_page: int, dtype: torch.dtype):
    x = k_cache_stripe_size(dtype)
    return (num_pages, num_kv_heads, head_dim // x, tokens_per_page, x)


def v_cache_shape(num_pages: int, num_kv_heads: int, head_dim: int, tokens_per_page: int, dtype: torch.dtype):
    return (num_pages, num_kv_heads, head_dim, tokens_per_page)


def pack_sequences_into_pages(k_seqs, v_seqs, page_lists, k_pool, v_pool):
    """Write dense per-sequence K/V ``[L_s, Hkv, D]`` into the pools, in place.

    ``page_lists[s]`` gives the physical page of each logical block of sequence s.
    Slots past L_s in the last page are left as they were.
    """
    tpp = v_pool.shape[3]
    x = k_pool.shape[4]
    for k, v, pages in zip(k_seqs, v_seqs, page_lists):
        L, hkv, d = k.shape
        for blk in range((L + tpp - 1) // tpp):
            t0 = blk * tpp
            n = min(tpp, L - t0)
            p = int(pages[blk])
            # [n, Hkv, D] -> [Hkv, D/x, n, x]
            k_pool[p, :, :, :n, :] = k[t0:t0 + n].reshape(n, hkv, d // x, x).permute(1, 2, 0, 3)
            # [n, Hkv, D] -> [Hkv, D, n]
            v_pool[p, :, :, :n] = v[t0:t0 + n].permute(1, 2, 0)


def gather_sequence_kv(k_pool, v_pool, pages, length: int):
    """Gather one sequence's first ``length`` tokens into dense ``[L, Hkv, D]`` K and V.

    Only the first ceil(length / tokens_per_page) entries of ``pages`` are read
    (``paged_attention_decode.h.metal:125-128``).
    """
    tpp = v_pool.shape[3]
    hkv, d = v_pool.shape[1], v_pool.shape[2]
    nblk = (length + tpp - 1) // tpp
    if nblk == 0:
        empty = torch.zeros((0, hkv, d), dtype=k_pool.dtype)
        return empty, empty.clone()
    idx = torch.as_tensor([int(p) for p in pages[:nblk]], dtype=torch.long)
    kb = k_pool[idx]  # [nblk, Hkv, D/x, tpp, x]
    vb = v_pool[idx]  # [nblk, Hkv, D, tpp]
    k = kb.permute(0, 3, 1, 2, 4).reshape(nblk * tpp, hkv, d)[:length]
    v = vb.permute(0, 3, 1, 2).reshape(nblk * tpp, hkv, d)[:length]
    return k, v
