"""Seeded random configurations of every operator against the CPU oracle: shapes, head groupings, page sizes,
lengths around page / tile / partition boundaries and launch modes are drawn together, so that index arithmetic is
exercised off the beaten path of the fixed-shape tests."""

import random

import pytest
import torch

from cases import make_decode_case, parity_report
from oracle import decode_oracle, fill_kv_pages_oracle, prefill_ragged_oracle, slots_from_page_table
from oracle import k_cache_shape, v_cache_shape

pytestmark = pytest.mark.gpu

TOL = 2e-3
HEAD_DIMS = [32, 64, 80, 96, 128, 256]


def _within(out, ref):
    return parity_report(out, ref)


def _interesting_length(rng, tpp, hi):
    """Lengths biased towards page, 64-, 128-token and partition boundaries."""
    base = rng.choice([1, tpp, 2 * tpp, 64, 128, 256, 4 * tpp * rng.randint(1, 8), rng.randint(1, hi)])
    return max(0, min(hi, base + rng.choice([-1, 0, 0, 1])))


@pytest.mark.parametrize("seed", range(24))
def test_decode_random(pal, cuda, seed):
    rng = random.Random(1000 + seed)
    d, tpp = rng.choice(HEAD_DIMS), rng.choice([16, 32])
    hkv = rng.choice([1, 2, 3, 4, 8])
    group = rng.choice([1, 2, 3, 4, 7, 8, 9, 16])
    S = rng.randint(1, 9)
    dtype = rng.choice([torch.float16, torch.bfloat16])
    lens = [_interesting_length(rng, tpp, 700) for _ in range(S)]
    if rng.random() < 0.3:
        lens[rng.randrange(S)] = 0
    case = make_decode_case(seed, lens, hkv * group, hkv, d, tpp=tpp, dtype=dtype, extra_pages=rng.randint(0, 5),
                            poison_unused=rng.random() < 0.5, pad_entry=rng.choice([0, 0xFFFFFFFF]),
                            table_width=max((max(lens) + tpp - 1) // tpp, 1) + rng.randint(0, 3))
    ref = decode_oracle(case.q, case.k_pool, case.v_pool, case.page_table, case.lens)
    q, k, v = case.q.to(cuda), case.k_pool.to(cuda), case.v_pool.to(cuda)
    table, ln = case.page_table.to(cuda), case.lens.to(cuda)
    for pp in (0, None, rng.choice([1, 2, 3, 5, 8])):
        out = pal.paged_attention_decode(q, k, v, table, ln, partition_pages=pp).cpu()
        assert torch.isfinite(out.float()).all()
        ok, msg = _within(out, ref)
        assert ok, f"partition_pages={pp}: {msg}"
    # the fused append step: the newest token's slot is poisoned and supplied separately
    ks, vs = case.meta["k_seqs"], case.meta["v_seqs"]
    new_k = torch.zeros((S, hkv, d), dtype=dtype)
    new_v = torch.zeros((S, hkv, d), dtype=dtype)
    kb, vb = case.k_pool.clone(), case.v_pool.clone()
    for s, L in enumerate(lens):
        if L > 0:
            new_k[s], new_v[s] = ks[s][L - 1], vs[s][L - 1]
            page, slot = int(case.page_table[s, (L - 1) // tpp]), (L - 1) % tpp
            kb[page, :, :, slot, :] = float("nan")
            vb[page, :, :, slot] = float("nan")
    kd, vd = kb.to(cuda), vb.to(cuda)
    out = pal.paged_attention_decode_append(new_k.to(cuda), new_v.to(cuda), q, kd, vd, table, ln,
                                            partition_pages=rng.choice([0, None, 2])).cpu()
    ok, msg = _within(out, ref)
    assert ok, f"append: {msg}"
    if not case.k_pool.isnan().any():  # NaN-poisoned unused slots cannot be compared bit for bit through ==
        assert torch.equal(kd.cpu().view(torch.int16), case.k_pool.view(torch.int16))
        assert torch.equal(vd.cpu().view(torch.int16), case.v_pool.view(torch.int16))


@pytest.mark.parametrize("seed", range(16))
def test_prefill_random(pal, cuda, seed):
    rng = random.Random(2000 + seed)
    tc_shape = rng.random() < 0.6
    d, tpp = (128, 16) if tc_shape else (rng.choice(HEAD_DIMS), rng.choice([16, 32]))
    hkv = rng.choice([1, 2, 4])
    group = rng.choice([1, 2, 3, 4, 6, 8])
    S = rng.randint(1, 5)
    dtype = rng.choice([torch.float16, torch.bfloat16])
    hist = [_interesting_length(rng, tpp, 600) for _ in range(S)]
    counts = [max(0, _interesting_length(rng, tpp, 300)) for _ in range(S)]
    if sum(counts) == 0:
        counts[0] = 5
    base = make_decode_case(seed, hist, hkv * group, hkv, d, tpp=tpp, dtype=dtype, poison_unused=rng.random() < 0.5)
    g = torch.Generator().manual_seed(seed)
    T = sum(counts)
    q = torch.randn((T, hkv * group, d), generator=g).to(dtype)
    k = torch.randn((T, hkv, d), generator=g).to(dtype)
    v = torch.randn((T, hkv, d), generator=g).to(dtype)
    cu = torch.tensor([0] + torch.tensor(counts).cumsum(0).tolist(), dtype=torch.int32)
    hist_t = torch.tensor(hist, dtype=torch.int32)
    ref = prefill_ragged_oracle(q, k, v, base.k_pool, base.v_pool, base.page_table, hist_t, cu)
    impls = ["mma", "tcgen05", "auto"] if tc_shape else ["mma", "auto"]
    for impl in impls:
        out = pal.paged_attention_prefill_ragged(q.to(cuda), k.to(cuda), v.to(cuda), base.k_pool.to(cuda), base.v_pool.to(cuda),
                                                 base.page_table.to(cuda), hist_t.to(cuda), cu.to(cuda), impl=impl).cpu()
        assert torch.isfinite(out.float()).all()
        ok, msg = _within(out, ref)
        assert ok, f"impl={impl}: {msg}"
    if len(set(counts)) == 1:  # equal counts: the uniform entry point must agree bit for bit
        out_u = pal.paged_attention_prefill(q.to(cuda), k.to(cuda), v.to(cuda), base.k_pool.to(cuda), base.v_pool.to(cuda),
                                            base.page_table.to(cuda), hist_t.to(cuda), impl="mma").cpu()
        out_r = pal.paged_attention_prefill_ragged(q.to(cuda), k.to(cuda), v.to(cuda), base.k_pool.to(cuda), base.v_pool.to(cuda),
                                                   base.page_table.to(cuda), hist_t.to(cuda), cu.to(cuda), impl="mma").cpu()
        assert torch.equal(out_u.view(torch.int16), out_r.view(torch.int16))


@pytest.mark.parametrize("seed", range(16))
def test_fill_random(pal, cuda, seed):
    rng = random.Random(3000 + seed)
    d, tpp = rng.choice(HEAD_DIMS), rng.choice([2, 4, 8, 16, 32])
    hkv = rng.choice([1, 2, 3, 8])
    dtype = rng.choice([torch.float16, torch.bfloat16])
    S = rng.randint(1, 6)
    g = torch.Generator().manual_seed(seed)
    # every sequence appends a run of tokens at consecutive positions after its own start
    starts = [rng.randint(0, 3 * tpp) for _ in range(S)]
    counts = [rng.choice([1, 2, tpp, tpp + 1, rng.randint(1, 200)]) for _ in range(S)]
    width = max((s + c + tpp - 1) // tpp for s, c in zip(starts, counts)) + 1
    P = S * width + rng.randint(0, 4)
    pt = torch.randperm(P, generator=g)[: S * width].reshape(S, width).to(torch.int32)
    pos = torch.cat([torch.arange(s, s + c) for s, c in zip(starts, counts)]).to(torch.int32)
    seqmap = torch.cat([torch.full((c,), i) for i, c in enumerate(counts)]).to(torch.int32)
    if rng.random() < 0.5:  # interleave the sequences' tokens instead of keeping runs together
        perm = torch.randperm(pos.numel(), generator=g)
        pos, seqmap = pos[perm], seqmap[perm]
    T = pos.numel()
    keys = torch.randn((T, hkv, d), generator=g).to(dtype)
    vals = torch.randn((T, hkv, d), generator=g).to(dtype)
    k = torch.zeros(k_cache_shape(P, hkv, d, tpp, dtype), dtype=dtype)
    v = torch.zeros(v_cache_shape(P, hkv, d, tpp, dtype), dtype=dtype)
    k.view(torch.int16).fill_(0x5A5A)
    v.view(torch.int16).fill_(0x2B2B)
    slots = slots_from_page_table(pt, pos, seqmap, tpp)
    ek, ev = fill_kv_pages_oracle(keys, vals, k, v, slots)
    gk, gv = pal.fill_kv_pages(keys.to(cuda), vals.to(cuda), k.to(cuda), v.to(cuda), pt.to(cuda), pos.to(cuda), seqmap.to(cuda))
    assert torch.equal(gk.cpu().view(torch.int16), ek.view(torch.int16)) and torch.equal(gv.cpu().view(torch.int16), ev.view(torch.int16))
    sk, sv = pal.fill_kv_pages(keys.to(cuda), vals.to(cuda), k.to(cuda), v.to(cuda), slots.to(cuda))
    assert torch.equal(sk.cpu().view(torch.int16), ek.view(torch.int16)) and torch.equal(sv.cpu().view(torch.int16), ev.view(torch.int16))


@pytest.mark.parametrize("seed", range(40))
def test_prefill_kernels_agree_random(pal, cuda, seed):
    """The prefill kernels against each other on random problems (head_dim 128 / 256, both page sizes, groups of 1-8, 1-5
    sequences of 1-1024 new tokens over histories around every boundary): the two-CTA kernel equals the one-CTA kernel bit for
    bit wherever both do the same arithmetic (heads paired or float16, and no history split for that shape), and every
    tcgen05 form stays within two output roundings of the mma.sync kernel; no bounded wait expires."""
    from cases import make_prefill_case
    from proxy_attention_lab_b200._lib import lib

    rng = random.Random(5000 + seed)
    d = rng.choice([128, 256, 256])
    tpp = rng.choice([16, 32])
    hkv = rng.choice([1, 2, 4])
    group = rng.choice([2, 4, 8] if d == 128 else [1, 2, 3, 4])
    S = rng.choice([1, 2, 3, 5])
    n = rng.choice([1, 17, 64, 128, 129, 300, 700, 1024])
    hist = [rng.choice([0, 1, 15, 63, 64, 65, 127, 128, 500, 1000, 2049, rng.randint(0, 3000)]) for _ in range(S)]
    dtype = rng.choice([torch.float16, torch.bfloat16])
    case = make_prefill_case(seed, hist, n, hkv * group, hkv, d, tpp=tpp, dtype=dtype)
    t = {k: getattr(case, k).to(cuda) for k in ("q", "k_new", "v_new", "k_pool", "v_pool", "page_table", "hist")}
    run = lambda impl: pal.paged_attention_prefill(t["q"], t["k_new"], t["v_new"], t["k_pool"], t["v_pool"], t["page_table"], t["hist"], impl=impl)
    pair, single, auto, mma = run("tcgen05_pair"), run("tcgen05_single"), run("tcgen05"), run("mma")
    torch.cuda.synchronize()
    pal.check_status()
    split = lib.pal_prefill_workspace_bytes(S, n, hkv * group, hkv, d) > 256
    scale = mma.float().abs().max().item()
    if (group % 2 == 0 or dtype == torch.float16) and not split:
        assert torch.equal(pair, single)
    for other in (pair, single, auto):
        assert torch.isfinite(other.float()).all()
        assert (other.float() - mma.float()).abs().max().item() <= 2 * TOL + 2.0 ** -7 * scale
