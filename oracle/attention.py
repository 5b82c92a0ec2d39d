"""Decode / prefill attention over a paged KV cache, restated on CPU (test infrastructure).

Semantics follow the reference kernels:

* decode  - ``src/pal_core/kernels/paged_attention/decode/paged_attention_decode.h.metal:29-412``:
  one query row per sequence, keys = tokens ``0 .. L_s-1`` found through the page table,
  score = (q . k) / sqrt(D), GQA map ``kv_head = q_head // (Hq / Hkv)`` (``:64-65``).
* split-KV combine - ``.../decode/paged_reduce_decode.h.metal:27-129``.
* prefill - ``.../prefill/paged_attention_prefill.h.metal:28-389``: query row i of sequence s
  sees all ``H_s`` history tokens from the pages plus new tokens ``0 .. i`` (``:136-165,243-266``);
  output row ``(s*N + i)*Hq + h`` (``:379-381``).

The comparator the reference's tests use is scaled-dot-product attention over gathered
pages (``tests/paged_attention/decode/test_sdpa_equivalency.py:87-246``,
``tests/paged_attention/prefill/test_sdpa_equivalency.py:48-182``); that is what is
computed here, in fp32, from the same 16-bit-rounded inputs the kernels read.  The
reference kernels' ``exp`` clamp at -88 and ``+1e-6`` in the denominator are artefacts
far below the comparison tolerance and are not reproduced.
"""

from __future__ import annotations

import math

import torch

from .layouts import gather_sequence_kv


def _scale(head_dim: int, scale):
    return (1.0 / math.sqrt(head_dim)) if scale is None else float(scale)


def decode_oracle(queries, k_pool, v_pool, page_table, sequence_lengths, scale=None):
    """fp32 ``[S, Hq, D]``; a sequence of length 0 yields zeros."""
    S = page_table.shape[0]
    hkv, d = v_pool.shape[1], v_pool.shape[2]
    q = queries.reshape(queries.shape[0], -1, d) if queries.dim() != 3 else queries
    hq = q.shape[1]
    g = hq // hkv
    sc = _scale(d, scale)
    out = torch.zeros((S, hq, d), dtype=torch.float32)
    for s in range(S):
        L = int(sequence_lengths[s])
        if L <= 0:
            continue
        k, v = gather_sequence_kv(k_pool, v_pool, page_table[s], L)
        kf = k.float().permute(1, 0, 2)  # [Hkv, L, D]
        vf = v.float().permute(1, 0, 2)
        qf = q[s].float().reshape(hkv, g, d)
        scores = torch.einsum("hgd,hld->hgl", qf, kf) * sc
        p = torch.softmax(scores, dim=-1)
        out[s] = torch.einsum("hgl,hld->hgd", p, vf).reshape(hq, d)
    return out


def decode_partials_oracle(queries, k_pool, v_pool, page_table, sequence_lengths, partition_tokens, scale=None):
    """Un-normalised split-KV partials.

    Partition j of a sequence covers tokens ``[j*partition_tokens, (j+1)*partition_tokens)``.
    Returns ``m [S,Hq,parts]`` (max scaled score, -inf when the partition is empty),
    ``l [S,Hq,parts]`` (sum of exp(score - m)) and ``acc [S,Hq,parts,D]``
    (sum of exp(score - m) * v), all fp32.
    """
    S = page_table.shape[0]
    hkv, d = v_pool.shape[1], v_pool.shape[2]
    q = queries
    hq = q.shape[1]
    g = hq // hkv
    sc = _scale(d, scale)
    max_len = int(max([int(x) for x in sequence_lengths] + [0]))
    parts = max(1, (max_len + partition_tokens - 1) // partition_tokens)
    m = torch.full((S, hq, parts), float("-inf"), dtype=torch.float32)
    l = torch.zeros((S, hq, parts), dtype=torch.float32)
    acc = torch.zeros((S, hq, parts, d), dtype=torch.float32)
    for s in range(S):
        L = int(sequence_lengths[s])
        if L <= 0:
            continue
        k, v = gather_sequence_kv(k_pool, v_pool, page_table[s], L)
        kf = k.float().permute(1, 0, 2)
        vf = v.float().permute(1, 0, 2)
        qf = q[s].float().reshape(hkv, g, d)
        scores = torch.einsum("hgd,hld->hgl", qf, kf) * sc
        for j in range(parts):
            a, b = j * partition_tokens, min(L, (j + 1) * partition_tokens)
            if a >= b:
                continue
            sj = scores[:, :, a:b]
            mj = sj.max(dim=-1).values
            pj = torch.exp(sj - mj[..., None])
            m[s, :, j] = mj.reshape(hq)
            l[s, :, j] = pj.sum(-1).reshape(hq)
            acc[s, :, j] = torch.einsum("hgl,hld->hgd", pj, vf[:, a:b]).reshape(hq, d)
    return m, l, acc


def lse_combine_oracle(m, l, acc):
    """Merge partials along the partition axis: ``[..., parts]`` / ``[..., parts, D]`` -> ``[..., D]``."""
    M = m.max(dim=-1, keepdim=True).values
    w = torch.where(torch.isinf(m) & (m < 0), torch.zeros_like(m), torch.exp(m - torch.where(torch.isinf(M), torch.zeros_like(M), M)))
    den = (w * l).sum(-1)
    num = (w[..., None] * acc).sum(-2)
    out = torch.where(den[..., None] > 0, num / den.clamp_min(1e-38)[..., None], torch.zeros_like(num))
    return out


def prefill_oracle(q_prompt, k_prompt, v_prompt, k_pool, v_pool, page_table, context_lens, scale=None):
    """fp32 ``[S*N*Hq, D]``: causal over the N new tokens, full over H_s paged history tokens."""
    S = context_lens.shape[0]
    hkv, d = k_prompt.shape[1], k_prompt.shape[2]
    hq = q_prompt.shape[1]
    g = hq // hkv
    n = q_prompt.shape[0] // S
    sc = _scale(d, scale)
    out = torch.zeros((S, n, hq, d), dtype=torch.float32)
    for s in range(S):
        H = int(context_lens[s])
        if H > 0:
            kh, vh = gather_sequence_kv(k_pool, v_pool, page_table[s], H)
        else:
            kh = torch.zeros((0, hkv, d), dtype=k_prompt.dtype)
            vh = torch.zeros((0, hkv, d), dtype=v_prompt.dtype)
        k = torch.cat([kh.to(k_prompt.dtype), k_prompt[s * n:(s + 1) * n]], dim=0).float()  # [H+N, Hkv, D]
        v = torch.cat([vh.to(v_prompt.dtype), v_prompt[s * n:(s + 1) * n]], dim=0).float()
        q = q_prompt[s * n:(s + 1) * n].float()  # [N, Hq, D]
        key_pos = torch.arange(H + n)
        visible = key_pos[None, :] <= (H + torch.arange(n))[:, None]  # [N, H+N]
        for h in range(hkv):
            qh = q[:, h * g:(h + 1) * g, :].permute(1, 0, 2)  # [G, N, D]
            scores = torch.matmul(qh, k[:, h, :].t()) * sc  # [G, N, H+N]
            scores = scores.masked_fill(~visible[None], float("-inf"))
            p = torch.softmax(scores, dim=-1)
            out[s, :, h * g:(h + 1) * g, :] = torch.matmul(p, v[:, h, :]).permute(1, 0, 2)
    return out.reshape(S * n * hq, d)


def prefill_ragged_oracle(q_prompt, k_prompt, v_prompt, k_pool, v_pool, page_table, context_lens, cu_seqlens, scale=None):
    """fp32 ``[T*Hq, D]`` for sequences with different numbers of new tokens: sequence ``s`` owns rows
    ``cu_seqlens[s] .. cu_seqlens[s+1] - 1`` and is computed exactly as a one-sequence uniform batch
    (the per-row semantics of ``paged_attention_prefill.h.metal:136-165,243-266`` do not depend on the other sequences)."""
    hq, d = q_prompt.shape[1], q_prompt.shape[2]
    out = torch.zeros((q_prompt.shape[0], hq, d), dtype=torch.float32)
    for s in range(context_lens.shape[0]):
        a, b = int(cu_seqlens[s]), int(cu_seqlens[s + 1])
        if b <= a:
            continue
        out[a:b] = prefill_oracle(q_prompt[a:b], k_prompt[a:b], v_prompt[a:b], k_pool, v_pool, page_table[s:s + 1],
                                  context_lens[s:s + 1], scale=scale).reshape(b - a, hq, d)
    return out.reshape(-1, d)

