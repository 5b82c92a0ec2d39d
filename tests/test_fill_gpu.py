"""GPU parity of fill_kv_pages against the CPU oracle: bit-exact, through the C ABI."""

import pytest
import torch

from oracle import fill_kv_pages_oracle, k_cache_shape, slots_from_page_table, v_cache_shape

pytestmark = pytest.mark.gpu


def _pools(P, hkv, d, tpp, dtype, sentinel=None, seed=0):
    k = torch.zeros(k_cache_shape(P, hkv, d, tpp, dtype), dtype=dtype)
    v = torch.zeros(v_cache_shape(P, hkv, d, tpp, dtype), dtype=dtype)
    if sentinel is not None:
        k.view(torch.int16).fill_(sentinel)
        v.view(torch.int16).fill_(sentinel ^ 0x0101)
    return k, v


def _bit_equal(a, b):
    return torch.equal(a.view(torch.int16), b.view(torch.int16))


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize(
    "T,hkv,d,tpp,P,table,start",
    [
        (1, 1, 64, 2, 1, [[0]], 0),            # test_fill_kv_pages_data.py: one token
        (3, 2, 32, 4, 2, [[1]], 0),            # three tokens inside page 1
        (3, 2, 32, 2, 12, [[5, 10]], 1),       # crossing pages 5 -> 10 from position 1
        (17, 8, 128, 16, 3, [[1, 2]], 0),      # a full page plus one token
    ],
)
def test_reference_single_sequence_cases(pal, cuda, dtype, T, hkv, d, tpp, P, table, start):
    """Placement cases of tests/paged_attention/fill_kv_pages/test_fill_multiple_tokens_single_sequence.py."""
    keys = torch.tensor([[[t * 1000 + h * 100 + x for x in range(d)] for h in range(hkv)] for t in range(T)]).to(dtype)
    vals = (keys.float() + 5000).to(dtype)
    k, v = _pools(P, hkv, d, tpp, dtype)
    pt = torch.tensor(table, dtype=torch.int32)
    pos = torch.arange(start, start + T, dtype=torch.int32)
    seqmap = torch.zeros(T, dtype=torch.int32)
    ek, ev = fill_kv_pages_oracle(keys, vals, k, v, slots_from_page_table(pt, pos, seqmap, tpp))
    # the expectation the reference test spells out, element by element
    for t in range(T):
        page = table[0][(start + t) // tpp]
        slot = (start + t) % tpp
        assert torch.equal(ek[page, :, :, slot, :].reshape(hkv, d), keys[t])
        assert torch.equal(ev[page, :, :, slot], vals[t])
    gk, gv = pal.fill_kv_pages(keys.to(cuda), vals.to(cuda), k.to(cuda), v.to(cuda), pt.to(cuda), pos.to(cuda), seqmap.to(cuda))
    assert _bit_equal(gk.cpu(), ek) and _bit_equal(gv.cpu(), ev)


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_two_sequences_distinct_and_shared_pages(pal, cuda, dtype):
    """tests/paged_attention/fill_kv_pages/test_fill_single_token_multiple_sequences.py:32-207."""
    g = torch.Generator().manual_seed(1)
    for table, pos in (([[2], [2]], [1, 3]), ([[0], [3]], [0, 2])):
        keys = torch.randn((2, 2, 32), generator=g).to(dtype)
        vals = torch.randn((2, 2, 32), generator=g).to(dtype)
        k, v = _pools(4, 2, 32, 4, dtype)
        pt = torch.tensor(table, dtype=torch.int32)
        p = torch.tensor(pos, dtype=torch.int32)
        sm = torch.tensor([0, 1], dtype=torch.int32)
        ek, ev = fill_kv_pages_oracle(keys, vals, k, v, slots_from_page_table(pt, p, sm, 4))
        gk, gv = pal.fill_kv_pages(keys.to(cuda), vals.to(cuda), k.to(cuda), v.to(cuda), pt.to(cuda), p.to(cuda), sm.to(cuda))
        assert _bit_equal(gk.cpu(), ek) and _bit_equal(gv.cpu(), ev)


@pytest.mark.parametrize("tokens_per_seq", [1, 512])
def test_scatter_config_random_slots(pal, cuda, tokens_per_seq):
    """64 sequences x {1, 512} tokens, Hkv=8, D=128, bf16, TPP=16, 65536-page pool, random free slots."""
    P, hkv, d, tpp, dtype = 65536, 8, 128, 16, torch.bfloat16
    T = 64 * tokens_per_seq
    g = torch.Generator().manual_seed(0)
    keys = torch.randn((T, hkv, d), generator=g).to(dtype)
    vals = torch.randn((T, hkv, d), generator=g).to(dtype)
    slots = torch.randperm(P * tpp, generator=g)[:T]
    k, v = _pools(P, hkv, d, tpp, dtype, sentinel=0x7A5C)
    gk, gv = pal.fill_kv_pages(keys.to(cuda), vals.to(cuda), k.to(cuda), v.to(cuda), slots.to(cuda))
    ek, ev = fill_kv_pages_oracle(keys, vals, k, v, slots)
    assert _bit_equal(gk.cpu(), ek) and _bit_equal(gv.cpu(), ev)


def test_scatter_config_reference_triple(pal, cuda):
    """Same scatter expressed as (page_table, positions, seq map): 64 sequences appending 512 tokens."""
    P, hkv, d, tpp, dtype = 4096, 8, 128, 16, torch.bfloat16
    S, n = 64, 512
    g = torch.Generator().manual_seed(0)
    keys = torch.randn((S * n, hkv, d), generator=g).to(dtype)
    vals = torch.randn((S * n, hkv, d), generator=g).to(dtype)
    start = torch.randint(0, 100, (S,), generator=g)
    width = (100 + n + tpp - 1) // tpp + 1
    pt = torch.randperm(P, generator=g)[: S * width].reshape(S, width).to(torch.int32)
    pos = (start[:, None] + torch.arange(n)[None]).reshape(-1).to(torch.int32)
    seqmap = torch.arange(S).repeat_interleave(n).to(torch.int32)
    k, v = _pools(P, hkv, d, tpp, dtype, sentinel=0x1234)
    ek, ev = fill_kv_pages_oracle(keys, vals, k, v, slots_from_page_table(pt, pos, seqmap, tpp))
    gk, gv = pal.fill_kv_pages(keys.to(cuda), vals.to(cuda), k.to(cuda), v.to(cuda), pt.to(cuda), pos.to(cuda), seqmap.to(cuda))
    assert _bit_equal(gk.cpu(), ek) and _bit_equal(gv.cpu(), ev)


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("hkv,d,tpp", [(8, 128, 16), (2, 64, 32), (1, 32, 8), (3, 80, 16), (8, 256, 16), (4, 128, 4), (32, 256, 16)])
def test_runs_mixed_with_scattered_and_skipped_tokens(pal, cuda, dtype, hkv, d, tpp):
    """Token lists that mix appended runs (aligned and not), isolated tokens and slots that must be skipped, with a
    length that is not a multiple of the kernel's token group: both store paths and their edges, bit for bit."""
    P = 512
    g = torch.Generator().manual_seed(hkv * 1000 + d + tpp)
    pages = torch.randperm(P, generator=g).tolist()
    slots = []
    for rep in range(4):  # enough tokens for the grouped kernel to be the one that runs
        for start, n in ((0, 40), (5, 23), (tpp - 1, 3), (3, 1), (8 % tpp, 8), (0, tpp), (1, 2 * tpp + 7 + rep)):
            pgs = [pages.pop() for _ in range((start + n) // tpp + 1)]
            slots += [pgs[(start + i) // tpp] * tpp + (start + i) % tpp for i in range(n)]
            slots += [-1, P * tpp + 3]  # skipped entries between the runs
            slots += [pages.pop() * tpp + int(torch.randint(0, tpp, (1,), generator=g))]  # an isolated token
    slots = torch.tensor(slots, dtype=torch.int64)
    T = slots.numel()
    assert T >= 256 and T % 16 != 0
    keys = torch.randn((T, hkv, d), generator=g).to(dtype)
    vals = torch.randn((T, hkv, d), generator=g).to(dtype)
    k, v = _pools(P, hkv, d, tpp, dtype, sentinel=0x3C3C)
    valid = (slots >= 0) & (slots < P * tpp)  # the library skips the others; the oracle is given only the valid ones
    ek, ev = fill_kv_pages_oracle(keys[valid], vals[valid], k, v, slots[valid])
    gk, gv = pal.fill_kv_pages(keys.to(cuda), vals.to(cuda), k.to(cuda), v.to(cuda), slots.to(cuda))
    assert _bit_equal(gk.cpu(), ek) and _bit_equal(gv.cpu(), ev)
    # a reversed list has the same destinations but no ascending runs
    rk, rv = pal.fill_kv_pages(keys.flip(0).to(cuda), vals.flip(0).to(cuda), k.to(cuda), v.to(cuda), slots.flip(0).to(cuda))
    assert _bit_equal(rk.cpu(), ek) and _bit_equal(rv.cpu(), ev)


def test_empty_and_functional_forms(pal, cuda):
    dtype = torch.float16
    k, v = _pools(2, 2, 32, 4, dtype, sentinel=0x0F0F)
    kd, vd = k.to(cuda), v.to(cuda)
    e = torch.zeros((0, 2, 32), dtype=dtype, device=cuda)
    i = torch.zeros((0,), dtype=torch.int32, device=cuda)
    gk, gv = pal.fill_kv_pages(e, e, kd, vd, torch.zeros((1, 1), dtype=torch.int32, device=cuda), i, i)
    assert _bit_equal(gk.cpu(), k) and _bit_equal(gv.cpu(), v)
    # inplace=False leaves the inputs untouched, as the reference does
    keys = torch.ones((1, 2, 32), dtype=dtype, device=cuda)
    gk, gv = pal.fill_kv_pages(keys, keys, kd, vd, torch.tensor([5], device=cuda), inplace=False)
    assert _bit_equal(kd.cpu(), k) and not _bit_equal(gk.cpu(), k)
    # out-of-range slots are skipped, not written
    gk, gv = pal.fill_kv_pages(keys, keys, kd, vd, torch.tensor([2 * 4 + 3], device=cuda))
    assert _bit_equal(gk.cpu(), k) and _bit_equal(gv.cpu(), v)


def test_fill_then_decode_round_trip(pal, cuda):
    """Tokens written by fill_kv_pages are what decode reads back."""
    from cases import make_decode_case, max_abs
    from oracle import decode_oracle

    case = make_decode_case(3, [75, 200], 8, 2, 128, dtype=torch.bfloat16)
    ks, vs = case.meta["k_seqs"], case.meta["v_seqs"]
    kd = torch.zeros_like(case.k_pool).to(cuda)
    vd = torch.zeros_like(case.v_pool).to(cuda)
    keys = torch.cat(ks).to(cuda)
    vals = torch.cat(vs).to(cuda)
    pos = torch.cat([torch.arange(len(x)) for x in ks]).to(torch.int32).to(cuda)
    seqmap = torch.cat([torch.full((len(x),), i) for i, x in enumerate(ks)]).to(torch.int32).to(cuda)
    pal.fill_kv_pages(keys, vals, kd, vd, case.page_table.to(cuda), pos, seqmap)
    assert _bit_equal(kd.cpu(), case.k_pool) and _bit_equal(vd.cpu(), case.v_pool)
    out = pal.paged_attention_decode(case.q.to(cuda), kd, vd, case.page_table.to(cuda), case.lens.to(cuda))
    assert max_abs(out.cpu(), decode_oracle(case.q, case.k_pool, case.v_pool, case.page_table, case.lens)) <= 2e-3
