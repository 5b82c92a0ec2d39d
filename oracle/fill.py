"""fill_kv_pages restated on CPU as indexed assignment (test infrastructure).

Follows ``src/pal_core/kernels/paged_attention/fill_kv_pages.h.metal:56-119``: token t goes to
physical page ``page_table[seq_t, pos_t // TPP]``, slot ``pos_t % TPP`` (``:64-72``);
``K[page, h, d // x, slot, d % x] = new_keys[t, h, d]`` (``:94-101``) and
``V[page, h, d, slot] = new_values[t, h, d]`` (``:106-114``).  Every reference fill test builds
its expectation with exactly this assignment
(e.g. ``tests/paged_attention/fill_kv_pages/test_fill_multiple_tokens_single_sequence.py:287-303``).
The copy is exact, so the comparison is bit-for-bit.
"""

from __future__ import annotations

import torch


def slots_from_page_table(page_table, write_positions, query_to_seq_map, tokens_per_page: int):
    """Flat slot ``page * TPP + pos % TPP`` of each new token (int64)."""
    pos = write_positions.to(torch.int64)
    seq = query_to_seq_map.to(torch.int64)
    page = page_table.to(torch.int64)[seq, pos // tokens_per_page]
    return page * tokens_per_page + pos % tokens_per_page


def fill_kv_pages_oracle(new_keys, new_values, k_pool, v_pool, slots):
    """Return updated clones of the pools; ``slots`` are flat slot ids (page*TPP + slot_in_page)."""
    k_out = k_pool.clone()
    v_out = v_pool.clone()
    T = new_keys.shape[0]
    if T == 0:
        return k_out, v_out
    tpp = v_pool.shape[3]
    x = k_pool.shape[4]
    hkv, d = new_keys.shape[1], new_keys.shape[2]
    slots = slots.to(torch.int64)
    page = slots // tpp
    slot = slots % tpp
    # K[page, :, :, slot, :] <- [T, Hkv, D/x, x]
    k_out[page, :, :, slot, :] = new_keys.reshape(T, hkv, d // x, x)
    v_out[page, :, :, slot] = new_values
    return k_out, v_out
