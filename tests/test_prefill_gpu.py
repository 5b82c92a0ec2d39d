"""GPU parity of paged_attention_prefill against the CPU oracle (through the C ABI)."""

import pytest
import torch

from cases import assert_parity, make_prefill_case, max_abs, to_dev
from oracle import prefill_oracle

pytestmark = pytest.mark.gpu

TOL = 2e-3


def run_prefill(pal, case, device, **kw):
    t = to_dev(case, device)
    out = pal.paged_attention_prefill(t["q"], t["k_new"], t["v_new"], t["k_pool"], t["v_pool"], t["page_table"], t["hist"], **kw)
    torch.cuda.synchronize()
    return out.cpu()


def supported(impl, d, tpp=16):
    """Both kernels cover the reference's whole grid: head_dim 32 / 64 / 80 / 96 / 128 / 256 with 16- or 32-token pages (the
    tcgen05 kernel lays 32, 80 and 96 out in tiles padded to whole 64-element swizzle blocks)."""
    return d in (32, 64, 80, 96, 128, 256) and tpp in (16, 32)


def check(pal, cuda, case, impl):
    """float32 output: plain max-abs <= 2e-3 on every element.  16-bit output: early causal rows attend to one or two
    keys, so |out| reaches a few units and the rounding of the output alone exceeds 2e-3; those elements must sit
    within one unit in the last place of the oracle rounded to the output type (cases.parity_report)."""
    ref = prefill_oracle(case.q, case.k_new, case.v_new, case.k_pool, case.v_pool, case.page_table, case.hist)
    out32 = run_prefill(pal, case, cuda, impl=impl, out_dtype=torch.float32)
    assert out32.shape == ref.shape and out32.dtype == torch.float32
    assert_parity(out32, ref, f"{impl}, float32 output")
    out = run_prefill(pal, case, cuda, impl=impl)
    assert out.shape == ref.shape and out.dtype == case.q.dtype
    assert_parity(out, ref, f"{impl}, 16-bit output")


IMPLS = ["mma", "tcgen05", "tcgen05_single"]  # tcgen05_single: one accumulator tile per CTA, S double-buffered


@pytest.mark.parametrize("impl", IMPLS)
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize(
    "batch,hist,n,heads,d",
    [(1, 0, 16, (4, 4), 64), (1, 128, 16, (4, 4), 64), (2, 64, 32, (8, 2), 128), (1, 256, 1, (32, 8), 128), (1, 0, 128, (32, 8), 128)],
)
def test_reference_shape_list(pal, cuda, impl, dtype, batch, hist, n, heads, d):
    """Shape list of tests/paged_attention/prefill/test_sdpa_equivalency.py:21-27."""
    if not supported(impl, d):
        pytest.skip("shape outside the tcgen05 kernel")
    case = make_prefill_case(5, [hist] * batch, n, heads[0], heads[1], d, dtype=dtype)
    check(pal, cuda, case, impl)


@pytest.mark.parametrize("impl", IMPLS)
@pytest.mark.parametrize("d", [32, 64, 80, 96, 128, 256])
@pytest.mark.parametrize("tpp", [16, 32])
def test_head_dims_and_page_sizes(pal, cuda, impl, d, tpp):
    if not supported(impl, d, tpp):
        pytest.skip("shape outside the tcgen05 kernel")
    case = make_prefill_case(9, [0, 70, 129], 77, 4, 2, d, tpp=tpp, dtype=torch.bfloat16)
    check(pal, cuda, case, impl)


@pytest.mark.parametrize("impl", ["tcgen05", "tcgen05_single"])
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("d", [32, 64, 80, 96, 128, 256])
@pytest.mark.parametrize("tpp", [16, 32])
def test_tcgen05_shapes_with_long_history_and_several_tiles(pal, cuda, impl, dtype, d, tpp):
    """Every tcgen05 instantiation over several history tiles (a partial last page, a partial last tile), several query
    tiles and a poisoned pool; heads paired per kv head (group 2), a lone head per kv head (query tiles paired) and the
    single-tile form."""
    for hq, hkv in ((4, 2), (3, 3)):
        case = make_prefill_case(17 + d + tpp, [700, 0, 131], 300, hq, hkv, d, tpp=tpp, dtype=dtype, poison_unused=True)
        check(pal, cuda, case, impl)


@pytest.mark.parametrize("impl", IMPLS)
def test_ragged_history_with_poisoned_padding(pal, cuda, impl):
    case = make_prefill_case(13, [0, 1, 15, 16, 17, 300], 130, 8, 2, 128, dtype=torch.bfloat16, poison_unused=True)
    check(pal, cuda, case, impl)


@pytest.mark.parametrize("impl", IMPLS)
def test_llama8b_shape_reduced(pal, cuda, impl):
    """Llama-3-8B head shape, 2 sequences x 512 new tokens over ragged history."""
    case = make_prefill_case(0, [1000, 37], 512, 32, 8, 128, dtype=torch.bfloat16)
    check(pal, cuda, case, impl)


@pytest.mark.parametrize("impl", IMPLS)
def test_no_history_empty_pool(pal, cuda, impl):
    """tests/paged_attention/prefill/test_softmax_and_value.py:72-78: zero-page pools and an (S, 0) page table."""
    dtype, d = torch.float16, (64 if impl == "mma" else 128)
    q = torch.ones((1, 1, d), dtype=dtype, device=cuda)
    k = torch.ones((1, 1, d), dtype=dtype, device=cuda)
    v = torch.zeros((1, 1, d), dtype=dtype, device=cuda)
    v[0, 0, :4] = torch.tensor([10.0, 20.0, 30.0, 40.0], dtype=dtype)
    kp = torch.zeros(pal.get_k_cache_shape(0, 1, d, 16, dtype), dtype=dtype, device=cuda)
    vp = torch.zeros(pal.get_v_cache_shape(0, 1, d, 16, dtype), dtype=dtype, device=cuda)
    pt = torch.zeros((1, 0), dtype=torch.int32, device=cuda)
    out = pal.paged_attention_prefill(q, k, v, kp, vp, pt, torch.zeros(1, dtype=torch.int32, device=cuda), impl=impl)
    assert out.shape == (1, d)
    assert torch.equal(out[0].cpu(), v[0, 0].cpu())


@pytest.mark.parametrize("impl", IMPLS)
@pytest.mark.parametrize("n,hist", [(64, 64), (256, 1024), (1024, 64)])
def test_determinism(pal, cuda, impl, n, hist):
    """tests/paged_attention/prefill/test_determinism.py:16-127."""
    case = make_prefill_case(21, [hist], n, 8, 2, 128, dtype=torch.bfloat16)
    a = run_prefill(pal, case, cuda, impl=impl)
    b = run_prefill(pal, case, cuda, impl=impl)
    assert torch.equal(a, b)


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_tcgen05_matches_mma(pal, cuda, dtype):
    """The two implementations agree with each other (odd group size -> one head per CTA, ragged N)."""
    case = make_prefill_case(33, [0, 500, 129], 200, 6, 2, 128, dtype=dtype)
    a = run_prefill(pal, case, cuda, impl="mma")
    b = run_prefill(pal, case, cuda, impl="tcgen05")
    assert max_abs(a, b) <= 2 * TOL + 2.0 ** -7 * a.float().abs().max().item()
    check(pal, cuda, case, "tcgen05")


def test_unsupported_head_dim_raises(pal, cuda):
    """A head_dim outside the reference's grid is refused by either kernel (nothing is launched)."""
    case = make_prefill_case(35, [10], 16, 4, 2, 48, dtype=torch.float16)
    t = to_dev(case, cuda)
    for impl in ("tcgen05", "mma", "auto"):
        with pytest.raises(RuntimeError):
            pal.paged_attention_prefill(t["q"], t["k_new"], t["v_new"], t["k_pool"], t["v_pool"], t["page_table"], t["hist"], impl=impl)


def test_chunked_prefill_config_reduced(pal, cuda):
    """Llama-3-8B chunked causal prefill shape, 3 sequences x 2048 new tokens over ragged history (auto impl)."""
    case = make_prefill_case(0, [0, 4096, 1111], 2048, 32, 8, 128, dtype=torch.bfloat16)
    check(pal, cuda, case, "auto")


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize(
    "hist,n,hq,hkv",
    [([0, 300], 256, 4, 4), ([129], 384, 2, 2), ([1000, 0, 64], 300, 3, 3), ([50], 129, 6, 2), ([0], 640, 1, 1), ([17], 128, 5, 5)],
)
def test_odd_head_groups_pair_query_tiles(pal, cuda, dtype, hist, n, hq, hkv):
    """One or three query heads per kv head: the tcgen05 kernel pairs two query tiles of a head in a CTA (odd and even tile
    counts, a sequence of exactly one tile, with and without history)."""
    check(pal, cuda, make_prefill_case(7, hist, n, hq, hkv, 128, dtype=dtype), "tcgen05")



@pytest.mark.parametrize("impl", ["tcgen05", "tcgen05_single"])
@pytest.mark.parametrize("num_seqs", [2, 31, 32, 33, 40])
def test_sequences_are_processed_in_order_of_work(pal, cuda, impl, num_seqs):
    """The tcgen05 kernel hands its grid's z index to the sequences in order of decreasing history (batches of up to 32
    sequences; larger ones keep the caller's order).  Every sequence must still be computed exactly once: histories
    with ties, zeros and a maximum in the middle, on both sides of the 32-sequence limit."""
    hist = [(37 * i) % 150 for i in range(num_seqs)]
    hist[num_seqs // 2] = 300
    hist[-1] = hist[0]
    case = make_prefill_case(400 + num_seqs, hist, 64, 4, 2, 128, dtype=torch.bfloat16, poison_unused=True)
    check(pal, cuda, case, impl)


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("d", [128, 256])
@pytest.mark.parametrize("tpp", [16, 32])
def test_two_cta_kernel(pal, cuda, dtype, d, tpp):
    """The cta_group::2 form (two CTAs per MMA, each loading half of every K / V tile): histories that end inside a page and
    inside a tile, none, shorter than the 64 keys of CTA 0's half, just past them; several query tiles; groups of 2 and 4
    query heads per kv head; unused pool slots poisoned."""
    for hq, hkv, hist, n in ((4, 2, [700, 0, 131], 300), (8, 2, [40, 64, 65, 2000], 130)):
        case = make_prefill_case(50 + d + tpp, hist, n, hq, hkv, d, tpp=tpp, dtype=dtype, poison_unused=True)
        check(pal, cuda, case, "tcgen05_pair")


def test_two_cta_kernel_serves_head_dim_256_by_default(pal, cuda):
    """With head_dim 256 and an even group the launcher's choice is the two-CTA form (bit-equal to asking for it); an odd
    group, or impl="tcgen05_single", runs the one-CTA kernel; the two agree within the tolerance of either."""
    case = make_prefill_case(61, [300, 17], 200, 4, 2, 256, dtype=torch.bfloat16)
    auto = run_prefill(pal, case, cuda, impl="tcgen05")
    assert torch.equal(auto, run_prefill(pal, case, cuda, impl="tcgen05_pair"))
    assert torch.equal(auto, run_prefill(pal, case, cuda))
    single = run_prefill(pal, case, cuda, impl="tcgen05_single")
    assert max_abs(auto, single) <= 2 * TOL + 2.0 ** -7 * single.float().abs().max().item()
    # an odd group pairs two query tiles of one head instead (the second tile of the last pair lies past the sequence's end)
    odd = make_prefill_case(62, [300, 17], 300, 3, 3, 256, dtype=torch.bfloat16)
    check(pal, cuda, odd, "tcgen05")
    check(pal, cuda, odd, "tcgen05_pair")
    # with head_dim 128 an odd group is left to the one-CTA kernel, which pairs query tiles itself
    odd128 = make_prefill_case(62, [300, 17], 200, 3, 3, 128, dtype=torch.bfloat16)
    t = to_dev(odd128, cuda)
    with pytest.raises(RuntimeError):
        pal.paged_attention_prefill(t["q"], t["k_new"], t["v_new"], t["k_pool"], t["v_pool"], t["page_table"], t["hist"], impl="tcgen05_pair")


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("tpp", [16, 32])
def test_two_cta_kernel_with_query_tiles_paired(pal, cuda, dtype, tpp):
    """head_dim 256 with an odd number of query heads per kv head: the pair is query tiles 2t and 2t + 1 of one head.  Odd and
    even numbers of query tiles, a last tile that is partial, histories ending inside a page, a tile and CTA 0's half."""
    for hq, hkv, hist, n in ((3, 3, [700, 0, 131], 300), (2, 2, [40, 65], 512), (5, 1, [2000], 130), (1, 1, [100], 129)):
        case = make_prefill_case(80 + tpp + n, hist, n, hq, hkv, 256, tpp=tpp, dtype=dtype, poison_unused=True)
        check(pal, cuda, case, "tcgen05_pair")
        if dtype == torch.float16:
            # (bfloat16 differs in the last bit here and there: whether the rounding residual of P is fed is decided for the pair
            # as a whole, so a later tile may get it where the one-CTA kernel, deciding per tile, leaves it out)
            assert torch.equal(run_prefill(pal, case, cuda, impl="tcgen05_pair"), run_prefill(pal, case, cuda, impl="tcgen05_single"))


@pytest.mark.parametrize("d", [128, 256])
def test_two_cta_kernel_determinism_and_status(pal, cuda, d):
    case = make_prefill_case(63, [1024, 0], 384, 8, 2, d, dtype=torch.bfloat16)
    a = run_prefill(pal, case, cuda, impl="tcgen05_pair")
    b = run_prefill(pal, case, cuda, impl="tcgen05_pair")
    assert torch.equal(a, b)
    pal.check_status()


@pytest.mark.parametrize("d,dtype", [(256, torch.bfloat16), (256, torch.float16), (128, torch.bfloat16)])
def test_two_cta_kernel_equals_the_one_cta_kernel_bit_for_bit(pal, cuda, d, dtype):
    """Both kernels multiply the same tiles in the same order (M = 256 across two CTAs against M = 128 in one) and share the
    softmax code, so on a problem of several waves - long and short histories, 16 query tiles - every output bit agrees."""
    case = make_prefill_case(71, [3000, 0, 517, 2048], 2048, 8, 4, d, dtype=dtype)
    pair = run_prefill(pal, case, cuda, impl="tcgen05_pair")
    single = run_prefill(pal, case, cuda, impl="tcgen05_single")
    assert torch.equal(pair, single)
    pal.check_status()


@pytest.mark.parametrize("impl", ["tcgen05", "tcgen05_single"])
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("d,tpp", [(128, 16), (64, 32), (96, 16), (32, 16)])
def test_small_batches_are_cut_along_the_history(pal, cuda, impl, dtype, d, tpp):
    """A batch that gives the GPU less than one CTA per SM is cut along the history (parts of the history tiles per CTA, fp32
    partial triples, one combine launch): one token over a long history, a few tokens over histories of very different
    lengths (the short one leaves most parts empty), more than one query tile, even and odd groups, no history at all."""
    for hq, hkv, hist, n in ((8, 2, [4096], 1), (4, 2, [3000, 50], 16), (3, 3, [1000], 130), (8, 2, [0, 0], 5), (2, 1, [129, 2047, 128], 64)):
        case = make_prefill_case(90 + d + n, hist, n, hq, hkv, d, tpp=tpp, dtype=dtype, poison_unused=True)
        check(pal, cuda, case, impl)
    from proxy_attention_lab_b200._lib import lib

    assert lib.pal_prefill_workspace_bytes(1, 1, 8, 2, d) > 256
    assert lib.pal_prefill_workspace_bytes(8, 2048, 32, 8, d) == 256
    pal.check_status()
