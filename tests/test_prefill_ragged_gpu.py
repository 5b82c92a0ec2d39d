"""GPU parity of paged_attention_prefill_ragged (different numbers of new tokens per sequence) against the CPU oracle."""

import pytest
import torch

from cases import assert_parity, make_decode_case
from oracle import prefill_ragged_oracle

pytestmark = pytest.mark.gpu

TOL = 2e-3
IMPLS = ["mma", "tcgen05", "tcgen05_single"]


def make_ragged_case(seed, hist_lens, new_counts, hq, hkv, d, tpp=16, dtype=torch.bfloat16, poison_unused=False):
    base = make_decode_case(seed, hist_lens, hq, hkv, d, tpp=tpp, dtype=dtype, poison_unused=poison_unused)
    g = torch.Generator().manual_seed(seed + 2000)
    total = sum(new_counts)
    q = torch.randn((total, hq, d), generator=g).to(dtype)
    k = torch.randn((total, hkv, d), generator=g).to(dtype)
    v = torch.randn((total, hkv, d), generator=g).to(dtype)
    cu = torch.tensor([0] + torch.tensor(new_counts).cumsum(0).tolist(), dtype=torch.int32)
    return dict(q=q, k=k, v=v, k_pool=base.k_pool, v_pool=base.v_pool, table=base.page_table,
                hist=torch.tensor(hist_lens, dtype=torch.int32), cu=cu)


def run(pal, cuda, c, **kw):
    out = pal.paged_attention_prefill_ragged(c["q"].to(cuda), c["k"].to(cuda), c["v"].to(cuda), c["k_pool"].to(cuda),
                                             c["v_pool"].to(cuda), c["table"].to(cuda), c["hist"].to(cuda), c["cu"].to(cuda), **kw)
    torch.cuda.synchronize()
    return out.cpu()


def check(pal, cuda, c, impl):
    ref = prefill_ragged_oracle(c["q"], c["k"], c["v"], c["k_pool"], c["v_pool"], c["table"], c["hist"], c["cu"])
    assert_parity(run(pal, cuda, c, impl=impl, out_dtype=torch.float32), ref, f"{impl}, float32 output")
    out = run(pal, cuda, c, impl=impl)
    assert out.shape == ref.shape and out.dtype == c["q"].dtype
    assert_parity(out, ref, f"{impl}, 16-bit output")


@pytest.mark.parametrize("impl", IMPLS)
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_mixed_counts_around_tile_edges(pal, cuda, impl, dtype):
    """Counts on both sides of the 64- and 128-row tiles, single tokens (decode steps) and an empty sequence in one batch."""
    counts = [1, 300, 0, 64, 127, 128, 129, 5, 1, 200]
    hist = [100, 0, 50, 129, 16, 0, 1000, 77, 2048, 255]
    check(pal, cuda, make_ragged_case(11, hist, counts, 8, 2, 128, dtype=dtype), impl)


@pytest.mark.parametrize("impl", ["tcgen05", "tcgen05_single"])
@pytest.mark.parametrize("d,tpp", [(32, 16), (32, 32), (64, 16), (64, 32), (80, 16), (80, 32), (96, 16), (96, 32), (128, 32), (256, 16), (256, 32)])
def test_ragged_batches_on_the_other_tcgen05_shapes(pal, cuda, impl, d, tpp):
    counts = [1, 140, 0, 64, 129, 5]
    hist = [100, 0, 50, 129, 16, 300]
    check(pal, cuda, make_ragged_case(21, hist, counts, 4, 2, d, tpp=tpp, poison_unused=True), impl)


def test_neighbours_values_cannot_leak_into_a_short_sequence(pal, cuda):
    """The dense V tile of a short sequence also brings in rows of the next sequence; their keys are masked, and their
    values - here NaN for every sequence but the one under test - must not reach the accumulator either."""
    counts = [5, 130, 7]
    c = make_ragged_case(22, [40, 0, 10], counts, 4, 2, 128)
    ref = prefill_ragged_oracle(c["q"], c["k"], c["v"], c["k_pool"], c["v_pool"], c["table"], c["hist"], c["cu"])
    cu = c["cu"].tolist()
    for victim in range(3):
        poisoned = dict(c)
        v = c["v"].clone()
        for s in range(3):
            if s != victim:
                v[cu[s]:cu[s + 1]] = float("nan")
        poisoned["v"] = v
        for impl in ("mma", "tcgen05", "tcgen05_single", "tcgen05_pair"):
            out = run(pal, cuda, poisoned, impl=impl).reshape(-1, 4, 128)
            got = out[cu[victim]:cu[victim + 1]]
            assert torch.isfinite(got.float()).all(), (victim, impl)
            assert_parity(got, ref.reshape(-1, 4, 128)[cu[victim]:cu[victim + 1]], f"{impl}, sequence {victim}")


@pytest.mark.parametrize("impl", IMPLS)
def test_poisoned_unused_slots_and_foreign_rows(pal, cuda, impl):
    """Unused page slots hold NaN; a tile of a short sequence also covers rows of its neighbours, which must stay masked."""
    counts = [3, 130, 2, 61]
    hist = [5, 200, 0, 33]
    check(pal, cuda, make_ragged_case(12, hist, counts, 4, 2, 128, poison_unused=True), impl)


@pytest.mark.parametrize("d,tpp", [(64, 16), (80, 16), (96, 32), (256, 16), (32, 32)])
def test_other_shapes_mma(pal, cuda, d, tpp):
    counts = [70, 1, 33, 128]
    hist = [40, 300, 0, 65]
    check(pal, cuda, make_ragged_case(13, hist, counts, 6, 3, d, tpp=tpp), "mma")


@pytest.mark.parametrize("impl", ["tcgen05", "tcgen05_single"])
@pytest.mark.parametrize("num_seqs", [5, 32, 35])
def test_ragged_batches_ordered_by_work(pal, cuda, impl, num_seqs):
    """The tcgen05 kernel takes the sequences of a batch in order of decreasing history + new tokens (up to 32 sequences);
    counts and histories with ties, a count of 1 and the longest sequence in the middle."""
    counts = [1 + (53 * i) % 140 for i in range(num_seqs)]
    hist = [(29 * i) % 90 for i in range(num_seqs)]
    counts[num_seqs // 2], hist[num_seqs // 2] = 200, 260
    counts[-1], hist[-1] = counts[0], hist[0]
    counts[1] = 1
    c = make_ragged_case(600 + num_seqs, hist, counts, 4, 2, 128, poison_unused=True)
    check(pal, cuda, c, impl)


@pytest.mark.parametrize("d,tpp", [(128, 16), (128, 32), (256, 16), (256, 32)])
def test_ragged_batches_on_the_two_cta_kernel(pal, cuda, d, tpp):
    """Counts around the tile edges, single tokens, an empty sequence, foreign rows after a short sequence's last tile
    (their V rows are zero-filled by each CTA for its half of the head dimension)."""
    counts = [1, 140, 0, 64, 129, 5, 128, 300]
    hist = [100, 0, 50, 129, 16, 300, 63, 1000]
    check(pal, cuda, make_ragged_case(31, hist, counts, 4, 2, d, tpp=tpp, poison_unused=True), "tcgen05_pair")
    if d == 256:  # odd group: query tiles paired
        check(pal, cuda, make_ragged_case(32, hist, counts, 3, 3, d, tpp=tpp, poison_unused=True), "tcgen05_pair")


@pytest.mark.parametrize("impl", ["tcgen05", "tcgen05_single"])
@pytest.mark.parametrize("d", [128, 64])
def test_small_ragged_batches_are_cut_along_the_history(pal, cuda, impl, d):
    """Decode steps and short chunks in one ragged call, too few CTAs to fill the GPU: the launch is cut along the history."""
    counts = [1, 20, 5, 0, 1]
    hist = [2000, 0, 700, 300, 4000]
    check(pal, cuda, make_ragged_case(41, hist, counts, 8, 2, d, poison_unused=True), impl)


@pytest.mark.parametrize("impl", IMPLS)
def test_equal_counts_match_the_uniform_call_bit_for_bit(pal, cuda, impl):
    counts = [192] * 3
    c = make_ragged_case(14, [0, 500, 129], counts, 8, 4, 128)
    ragged = run(pal, cuda, c, impl=impl)
    uniform = pal.paged_attention_prefill(c["q"].to(cuda), c["k"].to(cuda), c["v"].to(cuda), c["k_pool"].to(cuda),
                                          c["v_pool"].to(cuda), c["table"].to(cuda), c["hist"].to(cuda), impl=impl).cpu()
    assert torch.equal(ragged.view(torch.int16), uniform.view(torch.int16))


def test_auto_choice_and_explicit_maximum(pal, cuda):
    counts = [256, 17, 1]
    c = make_ragged_case(15, [64, 0, 700], counts, 32, 8, 128)
    ref = prefill_ragged_oracle(c["q"], c["k"], c["v"], c["k_pool"], c["v_pool"], c["table"], c["hist"], c["cu"])
    for kw in (dict(), dict(max_new_tokens=256), dict(max_new_tokens=300)):
        assert_parity(run(pal, cuda, c, **kw), ref, str(kw))


def test_empty_batch(pal, cuda):
    c = make_ragged_case(16, [10, 20], [0, 0], 4, 2, 128)
    assert run(pal, cuda, c).shape == (0, 128)
