"""GPU parity of the fused append + attend decode step against fill_kv_pages followed by decode on the oracle.

The expectation is built exactly as a serving loop would produce it without the fusion: the newest token of every
sequence is written with the fill oracle, then the decode oracle attends over the full length.  Before the fused
call the newest token's slot holds NaN, so an output that read the pool instead of the new rows is not finite.
"""

import pytest
import torch

from cases import assert_parity, make_decode_case, uniform_lengths
from oracle import decode_oracle

pytestmark = pytest.mark.gpu

TOL = 2e-3


def _bit_equal(a, b):
    return torch.equal(a.view(torch.int16), b.view(torch.int16))


def _run(pal, cuda, case, partition_pages):
    """Returns (out, k_pool_after, v_pool_after, k_pool_expected, v_pool_expected)."""
    tpp = case.meta["tpp"]
    lens = case.lens.tolist()
    ks, vs = case.meta["k_seqs"], case.meta["v_seqs"]
    hkv, d, dtype = case.meta["hkv"], case.meta["d"], case.meta["dtype"]
    new_k = torch.zeros((len(lens), hkv, d), dtype=dtype)
    new_v = torch.zeros((len(lens), hkv, d), dtype=dtype)
    k_before, v_before = case.k_pool.clone(), case.v_pool.clone()
    for s, L in enumerate(lens):
        if L <= 0:
            continue
        new_k[s], new_v[s] = ks[s][L - 1], vs[s][L - 1]
        page, slot = int(case.page_table[s, (L - 1) // tpp]), (L - 1) % tpp
        k_before[page, :, :, slot, :] = float("nan")
        v_before[page, :, :, slot] = float("nan")
    kd, vd = k_before.to(cuda), v_before.to(cuda)
    out = pal.paged_attention_decode_append(new_k.to(cuda), new_v.to(cuda), case.q.to(cuda), kd, vd, case.page_table.to(cuda),
                                            case.lens.to(cuda), partition_pages=partition_pages)
    torch.cuda.synchronize()
    return out.cpu(), kd.cpu(), vd.cpu()


def _check(pal, cuda, case, partition_pages):
    ref = decode_oracle(case.q, case.k_pool, case.v_pool, case.page_table, case.lens)
    out, k_after, v_after = _run(pal, cuda, case, partition_pages)
    # the pools end up exactly as fill_kv_pages leaves them (case.k_pool / v_pool were packed with every token)
    assert _bit_equal(k_after, case.k_pool) and _bit_equal(v_after, case.v_pool)
    assert_parity(out, ref, "fused append + decode")


@pytest.mark.parametrize("partition_pages", [0, None, 4])
def test_cpu_equivalence_config(pal, cuda, partition_pages):
    """Seed 0, 4 sequences U[64,512], Hq=8 / Hkv=2, D=128, TPP=16, fp16: the reference's own CPU-runnable shape."""
    lens = uniform_lengths(0, 4, 64, 512)
    case = make_decode_case(0, lens, 8, 2, 128, dtype=torch.float16, table_width=32)
    _check(pal, cuda, case, partition_pages)


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("partition_pages", [0, 2])
def test_page_boundaries_and_empty_sequences(pal, cuda, dtype, partition_pages):
    """Newest token in the first slot of a fresh page, in the last slot of a page, alone in the cache; empty sequences."""
    lens = [1, 16, 17, 32, 33, 0, 100, 15, 0, 64, 65]
    case = make_decode_case(3, lens, 8, 2, 128, dtype=dtype)
    _check(pal, cuda, case, partition_pages)


@pytest.mark.parametrize("hq,hkv,d,tpp", [(32, 2, 128, 16), (4, 4, 64, 32), (6, 3, 80, 16), (16, 2, 256, 16), (8, 8, 32, 32), (12, 4, 96, 16)])
def test_shapes_and_head_groups(pal, cuda, hq, hkv, d, tpp):
    """Every head_dim / page size of the decode grid; Hq/Hkv = 16 makes two work items share a (sequence, kv head)."""
    lens = uniform_lengths(hq + d, 5, 1, 300)
    case = make_decode_case(7, lens, hq, hkv, d, tpp=tpp, dtype=torch.bfloat16)
    for pp in (0, 3):
        _check(pal, cuda, case, pp)


def test_matches_unfused_pair_bit_for_bit(pal, cuda):
    """Same output bits as fill_kv_pages + paged_attention_decode on the GPU (the pages hold the same data either way)."""
    lens = uniform_lengths(5, 16, 200, 2000)
    case = make_decode_case(5, lens, 32, 8, 128, dtype=torch.bfloat16)
    out, k_after, v_after = _run(pal, cuda, case, 0)
    plain = pal.paged_attention_decode(case.q.to(cuda), case.k_pool.to(cuda), case.v_pool.to(cuda), case.page_table.to(cuda),
                                       case.lens.to(cuda), partition_pages=0).cpu()
    assert _bit_equal(out, plain)
    assert _bit_equal(k_after, case.k_pool) and _bit_equal(v_after, case.v_pool)


def test_full_size_llama8b_batch(pal, cuda):
    """Batch 64, context U[1024,8192], 32q/8kv heads, D=128, bf16: pools bit-exact, output equal to the plain decode."""
    lens = uniform_lengths(0, 64, 1024, 8192)
    case = make_decode_case(0, lens, 32, 8, 128, dtype=torch.bfloat16)
    out, k_after, v_after = _run(pal, cuda, case, 0)
    plain = pal.paged_attention_decode(case.q.to(cuda), case.k_pool.to(cuda), case.v_pool.to(cuda), case.page_table.to(cuda),
                                       case.lens.to(cuda), partition_pages=0).cpu()
    assert _bit_equal(out, plain)
    assert _bit_equal(k_after, case.k_pool) and _bit_equal(v_after, case.v_pool)
