"""GPU parity of paged_attention_decode against the CPU oracle (through the C ABI)."""

import pytest
import torch

from cases import assert_parity, make_decode_case, max_abs, to_dev, uniform_lengths
from oracle import decode_oracle

pytestmark = pytest.mark.gpu

TOL = 2e-3  # max-abs, fp16/bf16 outputs with fp32 accumulation


def run_decode(pal, case, device, **kw):
    t = to_dev(case, device)
    out = pal.paged_attention_decode(t["q"], t["k_pool"], t["v_pool"], t["page_table"], t["lens"], **kw)
    torch.cuda.synchronize()
    return out.cpu()


def check(pal, cuda, case, **kw):
    """float32 output: plain max-abs <= 2e-3.  16-bit output: 2e-3, or one unit in the last place of the oracle
    rounded to the output type (cases.parity_report)."""
    ref = decode_oracle(case.q, case.k_pool, case.v_pool, case.page_table, case.lens)
    out32 = run_decode(pal, case, cuda, out_dtype=torch.float32, **kw)
    assert out32.shape == ref.shape and out32.dtype == torch.float32
    assert_parity(out32, ref, "float32 output")
    out = run_decode(pal, case, cuda, **kw)
    assert out.shape == ref.shape and out.dtype == case.q.dtype
    assert_parity(out, ref, "16-bit output")


def test_cpu_equivalence_config(pal, cuda):
    """Seed 0, 4 sequences U[64,512], Hq=8 / Hkv=2, D=128, TPP=16, fp16, 256-page pool."""
    lens = uniform_lengths(0, 4, 64, 512)
    used = sum((L + 15) // 16 for L in lens)
    case = make_decode_case(0, lens, 8, 2, 128, dtype=torch.float16, extra_pages=256 - used, table_width=32)
    for pp in (0, None, 4):
        check(pal, cuda, case, partition_pages=pp)


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize(
    "batch,hist,heads,d",
    [
        (1, 16, (1, 1), 32), (1, 32, (1, 1), 32), (1, 16, (4, 1), 32), (1, 16, (4, 2), 32), (1, 16, (1, 1), 64),
        (1, 64, (2, 2), 32), (1, 64, (4, 2), 128), (1, 64, (32, 16), 128), (2, 32, (4, 4), 32), (2, 64, (32, 16), 128),
        (3, 128, (32, 16), 128), (16, 64, (4, 4), 32), (1, 1024, (32, 16), 128),
        (1, 4096, (32, 16), 128), (1, 8192, (32, 16), 128),  # the long-context cases the reference leaves disabled
    ],
)
def test_reference_shape_list(pal, cuda, batch, hist, heads, d, dtype):
    """Shape list of tests/paged_attention/decode/test_sdpa_equivalency.py:43-59."""
    case = make_decode_case(7, [hist] * batch, heads[0], heads[1], d, dtype=dtype, shuffle=False)
    check(pal, cuda, case)


@pytest.mark.parametrize("d", [32, 64, 80, 96, 128, 256])
@pytest.mark.parametrize("tpp", [16, 32])
def test_head_dims_and_page_sizes(pal, cuda, d, tpp):
    lens = [1, 15, 16, 17, 33, 250, 511]
    case = make_decode_case(3, lens, 8, 2, d, tpp=tpp, dtype=torch.bfloat16)
    check(pal, cuda, case, partition_pages=0)
    check(pal, cuda, case, partition_pages=3)


@pytest.mark.parametrize("hq,hkv", [(8, 8), (8, 1), (32, 8), (64, 8), (24, 2), (32, 1)])
def test_gqa_group_sizes(pal, cuda, hq, hkv):
    case = make_decode_case(5, [100, 37, 260], hq, hkv, 128, dtype=torch.bfloat16)
    check(pal, cuda, case, partition_pages=0)
    check(pal, cuda, case, partition_pages=5)


def test_ragged_and_empty_sequences(pal, cuda):
    lens = [0, 1, 300, 0, 16, 31]
    case = make_decode_case(11, lens, 8, 2, 128, dtype=torch.float16)
    for pp in (0, 2):
        out = run_decode(pal, case, cuda, partition_pages=pp)
        ref = decode_oracle(case.q, case.k_pool, case.v_pool, case.page_table, case.lens)
        assert max_abs(out, ref) <= TOL
        assert (out[0] == 0).all() and (out[3] == 0).all()


def test_unused_table_entries_and_slots_are_never_read(pal, cuda):
    """Entries past the used length hold 0xFFFFFFFF and unused slots / pages hold NaN."""
    lens = [70, 129, 5]
    case = make_decode_case(13, lens, 8, 2, 128, dtype=torch.float16, pad_entry=0xFFFFFFFF, poison_unused=True,
                            extra_pages=7, table_width=12)
    check(pal, cuda, case, partition_pages=0)
    check(pal, cuda, case, partition_pages=2)


def test_two_pass_agrees_with_single_pass(pal, cuda):
    case = make_decode_case(17, [5000, 777, 4096, 3], 32, 8, 128, dtype=torch.bfloat16)
    a = run_decode(pal, case, cuda, partition_pages=0)
    for pp in (16, 64, 256):
        b = run_decode(pal, case, cuda, partition_pages=pp)
        assert max_abs(a, b) <= TOL


def test_extra_query_rows_are_ignored(pal, cuda):
    """tests/paged_attention/decode/test_decode_smoke.py:43-45,103: 4 query rows, 1 sequence."""
    case = make_decode_case(19, [40], 4, 2, 64, dtype=torch.float16)
    t = to_dev(case, cuda)
    q4 = torch.cat([t["q"], torch.randn(3, 4, 64, device=cuda).to(torch.float16)])
    out = pal.paged_attention_decode(q4, t["k_pool"], t["v_pool"], t["page_table"], t["lens"])
    assert out.shape == (1, 4, 64)
    ref = decode_oracle(case.q, case.k_pool, case.v_pool, case.page_table, case.lens)
    assert max_abs(out.cpu(), ref) <= TOL


def test_two_dim_queries_mean_one_head(pal, cuda):
    case = make_decode_case(23, [33, 20], 1, 1, 64, dtype=torch.float16)
    t = to_dev(case, cuda)
    out = pal.paged_attention_decode(t["q"].reshape(2, 64), t["k_pool"], t["v_pool"], t["page_table"], t["lens"])
    assert out.shape == (2, 1, 64)
    ref = decode_oracle(case.q, case.k_pool, case.v_pool, case.page_table, case.lens)
    assert max_abs(out.cpu(), ref) <= TOL


@pytest.mark.parametrize("hist", [16, 128, 1024, 4096])
@pytest.mark.parametrize("d", [32, 64, 128, 256])
def test_determinism(pal, cuda, hist, d):
    """tests/paged_attention/decode/test_determinism.py:35-117, here also with several sequences."""
    case = make_decode_case(29, [hist, hist // 2 + 1, hist], 8, 2, d, dtype=torch.bfloat16)
    a = run_decode(pal, case, cuda)
    b = run_decode(pal, case, cuda)
    assert torch.equal(a, b)


def test_caches_are_not_modified(pal, cuda):
    case = make_decode_case(31, [50, 60], 4, 2, 64, dtype=torch.float16)
    t = to_dev(case, cuda)
    k0, v0 = t["k_pool"].clone(), t["v_pool"].clone()
    pal.paged_attention_decode(t["q"], t["k_pool"], t["v_pool"], t["page_table"], t["lens"])
    torch.cuda.synchronize()
    assert torch.equal(k0, t["k_pool"]) and torch.equal(v0, t["v_pool"])


def test_llama8b_shape_small_batch(pal, cuda):
    """Llama-3-8B head shape with ragged 1k-8k contexts (8 sequences to keep the oracle quick)."""
    lens = uniform_lengths(0, 8, 1024, 8192)
    case = make_decode_case(0, lens, 32, 8, 128, dtype=torch.bfloat16, table_width=512)
    check(pal, cuda, case, partition_pages=0)


def test_partials_and_combine_match_oracle(pal, cuda):
    from oracle import decode_partials_oracle, lse_combine_oracle

    case = make_decode_case(37, [900, 100, 0], 16, 2, 128, dtype=torch.bfloat16)
    t = to_dev(case, cuda)
    m, l, acc = pal.paged_attention_decode_partials(t["q"], t["k_pool"], t["v_pool"], t["page_table"], t["lens"],
                                                    partition_pages=8)
    ref = decode_oracle(case.q, case.k_pool, case.v_pool, case.page_table, case.lens)
    mo, lo, ao = decode_partials_oracle(case.q, case.k_pool, case.v_pool, case.page_table, case.lens, 1 << 20)
    assert torch.isinf(m[2]).all() and (l[2] == 0).all()
    got = (acc / l.clamp_min(1e-30)[..., None]).cpu()
    assert max_abs(got[:2], ref[:2]) <= TOL
    assert max_abs(m[:2].cpu(), mo[:2, :, 0]) <= 1e-3
    # merge two artificial "ranks": the same triple twice must give the same answer
    out = pal.lse_combine(torch.stack([m, m]), torch.stack([l, l]), torch.stack([acc, acc]), out_dtype=torch.bfloat16)
    assert max_abs(out.cpu(), ref) <= TOL


def test_bad_arguments_raise(pal, cuda):
    case = make_decode_case(41, [20], 3, 2, 64, dtype=torch.float16)
    t = to_dev(case, cuda)
    with pytest.raises(ValueError):
        pal.paged_attention_decode(t["q"], t["k_pool"], t["v_pool"], t["page_table"], t["lens"])  # 3 % 2 != 0
    case = make_decode_case(41, [20], 2, 2, 48, dtype=torch.float16)
    t = to_dev(case, cuda)
    with pytest.raises(RuntimeError):
        pal.paged_attention_decode(t["q"], t["k_pool"], t["v_pool"], t["page_table"], t["lens"])  # D=48: no kernel
    with pytest.raises(RuntimeError):
        pal.paged_attention_decode(case.q, case.k_pool, case.v_pool, case.page_table, case.lens)  # CPU tensors
