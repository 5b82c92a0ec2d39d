"""The oracle against dense scaled-dot-product attention that never sees the page layout (CPU).

Structure of the reference's own equivalence tests (tests/paged_attention/decode/test_sdpa_equivalency.py:87-246,
tests/paged_attention/prefill/test_sdpa_equivalency.py:48-182): draw dense Q / K / V, compute
``softmax(scale * Q K^T + mask) V`` on the dense tensors, pack K / V into pages, run the paged operator, compare.
Here the paged operator under test is the CPU oracle, the comparator is ``torch.nn.functional.scaled_dot_product_attention``
in fp32 (GQA by repeating kv heads, the causal mask of prefill offset by the history length), and the pages are packed
by this file's own packer - flat element addresses written out from the Metal kernels' index arithmetic
(paged_attention_decode.h.metal:142-144,170-190 for K, :248-250,294 for V) - so the GQA head map, the order of pages
within a sequence and the causal offset are pinned by code that shares nothing with ``oracle/layouts.py``.
"""

import numpy as np
import pytest
import torch
import torch.nn.functional as F

from oracle import decode_oracle, prefill_oracle, prefill_ragged_oracle

DECODE_SHAPES = [  # tests/paged_attention/decode/test_sdpa_equivalency.py:43-59 (the 4096 / 8192 cases are left to the GPU tests)
    (1, 16, (1, 1), 32), (1, 32, (1, 1), 32), (1, 16, (4, 1), 32), (1, 16, (4, 2), 32), (1, 16, (1, 1), 64),
    (1, 64, (2, 2), 32), (1, 64, (4, 2), 128), (1, 64, (32, 16), 128), (2, 32, (4, 4), 32), (2, 64, (32, 16), 128),
    (3, 128, (32, 16), 128), (16, 64, (4, 4), 32), (1, 1024, (32, 16), 128),
]
PREFILL_SHAPES = [  # tests/paged_attention/prefill/test_sdpa_equivalency.py:21-27
    (1, 0, 16, (4, 4), 64), (1, 128, 16, (4, 4), 64), (2, 64, 32, (8, 2), 128), (1, 256, 1, (32, 8), 128), (1, 0, 128, (32, 8), 128),
]


def pack_pages_flat(k_dense, v_dense, page_ids, num_pages, tpp, dtype):
    """Pack dense per-sequence K / V ``[L, Hkv, D]`` into flat pools by element address.

    K element (page p, head h, slot t, dim d) lives at ``((p*Hkv + h)*(D/x) + d//x)*TPP*x + t*x + d%x`` with x = 8,
    V element at ``((p*Hkv + h)*D + d)*TPP + t``; token j of a sequence sits in page ``page_ids[j // TPP]``, slot ``j % TPP``.
    """
    hkv, d = k_dense[0].shape[1], k_dense[0].shape[2]
    x = 8
    k_flat = np.zeros(num_pages * hkv * d * tpp, dtype=np.float32)
    v_flat = np.zeros(num_pages * hkv * d * tpp, dtype=np.float32)
    for k, v, pages in zip(k_dense, v_dense, page_ids):
        L = k.shape[0]
        if L == 0:
            continue
        j = np.arange(L)[:, None, None]
        h = np.arange(hkv)[None, :, None]
        e = np.arange(d)[None, None, :]
        p = np.asarray(pages, dtype=np.int64)[j // tpp]
        t = j % tpp
        k_addr = ((p * hkv + h) * (d // x) + e // x) * tpp * x + t * x + e % x
        v_addr = ((p * hkv + h) * d + e) * tpp + t
        k_flat[k_addr.reshape(-1)] = k.float().numpy().reshape(-1)
        v_flat[v_addr.reshape(-1)] = v.float().numpy().reshape(-1)
    k_pool = torch.from_numpy(k_flat).to(dtype).reshape(num_pages, hkv, d // x, tpp, x)
    v_pool = torch.from_numpy(v_flat).to(dtype).reshape(num_pages, hkv, d, tpp)
    return k_pool, v_pool


def dense_sdpa(q, k, v, history=None):
    """fp32 SDPA on dense tensors: q ``[N, Hq, D]``, k / v ``[L, Hkv, D]``; with ``history`` = H the mask lets query i see
    keys 0 .. H + i (the reference's ``triu(-inf, k=1)`` mask shifted by the history length)."""
    hq, hkv = q.shape[1], k.shape[1]
    qf = q.float().permute(1, 0, 2)[None]                                   # [1, Hq, N, D]
    kf = k.float().permute(1, 0, 2).repeat_interleave(hq // hkv, dim=0)[None]  # q head h reads kv head h // group
    vf = v.float().permute(1, 0, 2).repeat_interleave(hq // hkv, dim=0)[None]
    mask = None
    if history is not None:
        n, L = q.shape[0], k.shape[0]
        mask = torch.arange(L)[None, :] <= (history + torch.arange(n))[:, None]
    out = F.scaled_dot_product_attention(qf, kf, vf, attn_mask=mask, scale=1.0 / (q.shape[-1] ** 0.5))
    return out[0].permute(1, 0, 2)                                           # [N, Hq, D]


def _page_ids(rng, counts, shuffled):
    total = sum(counts)
    perm = rng.permutation(total) if shuffled else np.arange(total)
    out, off = [], 0
    for c in counts:
        out.append(perm[off:off + c].tolist())
        off += c
    return out, total


@pytest.mark.parametrize("shuffled", [False, True])
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("batch,hist,heads,d", DECODE_SHAPES)
def test_decode_oracle_matches_dense_sdpa(batch, hist, heads, d, dtype, shuffled):
    hq, hkv = heads
    tpp = 16
    g = torch.Generator().manual_seed(hash((batch, hist, hq, d)) & 0xFFFF)
    rng = np.random.default_rng(5)
    q = torch.randn((batch, hq, d), generator=g).to(dtype)
    ks = [torch.randn((hist, hkv, d), generator=g).to(dtype) for _ in range(batch)]
    vs = [torch.randn((hist, hkv, d), generator=g).to(dtype) for _ in range(batch)]
    npg = (hist + tpp - 1) // tpp
    pages, total = _page_ids(rng, [npg] * batch, shuffled)
    k_pool, v_pool = pack_pages_flat(ks, vs, pages, total, tpp, dtype)
    table = torch.tensor(pages, dtype=torch.int32)
    got = decode_oracle(q, k_pool, v_pool, table, torch.full((batch,), hist, dtype=torch.int32))
    want = torch.stack([dense_sdpa(q[b:b + 1], ks[b], vs[b])[0] for b in range(batch)])
    assert got.shape == want.shape
    assert torch.allclose(got, want, atol=2e-5, rtol=1e-5), (got - want).abs().max().item()


@pytest.mark.parametrize("tpp", [16, 32])
def test_decode_oracle_ragged_lengths_gqa_and_shuffled_pages(tpp):
    """Lengths that end inside a page, several pages per sequence in shuffled order, 4 query heads per kv head."""
    lens, hq, hkv, d, dtype = [1, 15, 16, 17, 100, 333], 8, 2, 64, torch.bfloat16
    g = torch.Generator().manual_seed(99)
    rng = np.random.default_rng(7)
    q = torch.randn((len(lens), hq, d), generator=g).to(dtype)
    ks = [torch.randn((L, hkv, d), generator=g).to(dtype) for L in lens]
    vs = [torch.randn((L, hkv, d), generator=g).to(dtype) for L in lens]
    counts = [(L + tpp - 1) // tpp for L in lens]
    pages, total = _page_ids(rng, counts, True)
    k_pool, v_pool = pack_pages_flat(ks, vs, pages, total, tpp, dtype)
    table = torch.zeros((len(lens), max(counts)), dtype=torch.int32)
    for s, p in enumerate(pages):
        table[s, :len(p)] = torch.tensor(p, dtype=torch.int32)
    got = decode_oracle(q, k_pool, v_pool, table, torch.tensor(lens, dtype=torch.int32))
    for s in range(len(lens)):
        want = dense_sdpa(q[s:s + 1], ks[s], vs[s])[0]
        assert torch.allclose(got[s], want, atol=2e-5, rtol=1e-5), (s, (got[s] - want).abs().max().item())


@pytest.mark.parametrize("shuffled", [False, True])
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("batch,hist,n,heads,d", PREFILL_SHAPES)
def test_prefill_oracle_matches_dense_sdpa(batch, hist, n, heads, d, dtype, shuffled):
    hq, hkv = heads
    tpp = 16
    g = torch.Generator().manual_seed(hash((batch, hist, n, hq, d)) & 0xFFFF)
    rng = np.random.default_rng(11)
    q = torch.randn((batch * n, hq, d), generator=g).to(dtype)
    k_new = torch.randn((batch * n, hkv, d), generator=g).to(dtype)
    v_new = torch.randn((batch * n, hkv, d), generator=g).to(dtype)
    kh = [torch.randn((hist, hkv, d), generator=g).to(dtype) for _ in range(batch)]
    vh = [torch.randn((hist, hkv, d), generator=g).to(dtype) for _ in range(batch)]
    npg = (hist + tpp - 1) // tpp
    pages, total = _page_ids(rng, [npg] * batch, shuffled)
    k_pool, v_pool = pack_pages_flat(kh, vh, pages, max(total, 1), tpp, dtype)
    if total == 0:
        k_pool, v_pool = k_pool[:0], v_pool[:0]
    table = torch.tensor(pages, dtype=torch.int32).reshape(batch, npg)
    got = prefill_oracle(q, k_new, v_new, k_pool, v_pool, table, torch.full((batch,), hist, dtype=torch.int32))
    got = got.reshape(batch, n, hq, d)
    for b in range(batch):
        k_all = torch.cat([kh[b], k_new[b * n:(b + 1) * n]])
        v_all = torch.cat([vh[b], v_new[b * n:(b + 1) * n]])
        want = dense_sdpa(q[b * n:(b + 1) * n], k_all, v_all, history=hist)
        assert torch.allclose(got[b], want, atol=2e-5, rtol=1e-5), (b, (got[b] - want).abs().max().item())


def test_prefill_ragged_oracle_matches_dense_sdpa():
    """Different history lengths and different numbers of new tokens per sequence, GQA 4:1, shuffled pages."""
    hist, counts, hq, hkv, d, tpp, dtype = [0, 37, 200], [5, 70, 1], 8, 2, 64, 16, torch.bfloat16
    g = torch.Generator().manual_seed(3)
    rng = np.random.default_rng(13)
    T = sum(counts)
    q = torch.randn((T, hq, d), generator=g).to(dtype)
    k_new = torch.randn((T, hkv, d), generator=g).to(dtype)
    v_new = torch.randn((T, hkv, d), generator=g).to(dtype)
    kh = [torch.randn((H, hkv, d), generator=g).to(dtype) for H in hist]
    vh = [torch.randn((H, hkv, d), generator=g).to(dtype) for H in hist]
    npg = [(H + tpp - 1) // tpp for H in hist]
    pages, total = _page_ids(rng, npg, True)
    k_pool, v_pool = pack_pages_flat(kh, vh, pages, total, tpp, dtype)
    table = torch.zeros((len(hist), max(npg)), dtype=torch.int32)
    for s, p in enumerate(pages):
        table[s, :len(p)] = torch.tensor(p, dtype=torch.int32)
    cu = torch.tensor([0] + np.cumsum(counts).tolist(), dtype=torch.int32)
    got = prefill_ragged_oracle(q, k_new, v_new, k_pool, v_pool, table, torch.tensor(hist, dtype=torch.int32), cu).reshape(T, hq, d)
    for s in range(len(hist)):
        a, b = int(cu[s]), int(cu[s + 1])
        want = dense_sdpa(q[a:b], torch.cat([kh[s], k_new[a:b]]), torch.cat([vh[s], v_new[a:b]]), history=hist[s])
        assert torch.allclose(got[a:b], want, atol=2e-5, rtol=1e-5), (s, (got[a:b] - want).abs().max().item())
