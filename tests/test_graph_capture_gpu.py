"""The operators can be captured into a CUDA graph and replayed (what a serving loop does with its decode step)."""

import pytest
import torch

from cases import make_decode_case, make_prefill_case, uniform_lengths

pytestmark = pytest.mark.gpu


def _bit_equal(a, b):
    return torch.equal(a.view(torch.int16), b.view(torch.int16))


@pytest.mark.parametrize("partition_pages", [0, 8])
def test_decode_step_replays_with_new_inputs(pal, cuda, partition_pages):
    lens = uniform_lengths(3, 8, 100, 1500)
    case = make_decode_case(3, lens, 32, 8, 128, dtype=torch.bfloat16)
    q, k, v = case.q.to(cuda), case.k_pool.to(cuda), case.v_pool.to(cuda)
    table, ln = case.page_table.to(cuda), case.lens.to(cuda)
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):  # warm-up outside the capture: kernel attributes are set on first use
        pal.paged_attention_decode(q, k, v, table, ln, partition_pages=partition_pages)
    torch.cuda.current_stream().wait_stream(side)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        out = pal.paged_attention_decode(q, k, v, table, ln, partition_pages=partition_pages)
    for seed in (1, 2):
        g = torch.Generator().manual_seed(seed)
        q.copy_(torch.randn(case.q.shape, generator=g).to(torch.bfloat16))
        ln.copy_(torch.tensor([max(1, L - seed * 7) for L in lens], dtype=torch.int32))
        graph.replay()
        torch.cuda.synchronize()
        eager = pal.paged_attention_decode(q, k, v, table, ln, partition_pages=partition_pages)
        assert _bit_equal(out.cpu(), eager.cpu())


def test_append_and_prefill_replay(pal, cuda):
    lens = uniform_lengths(4, 6, 50, 700)
    case = make_decode_case(4, lens, 16, 4, 128, dtype=torch.bfloat16)
    q, k, v = case.q.to(cuda), case.k_pool.to(cuda), case.v_pool.to(cuda)
    table, ln = case.page_table.to(cuda), case.lens.to(cuda)
    nk = torch.randn((6, 4, 128), device=cuda).to(torch.bfloat16)
    nv = torch.randn((6, 4, 128), device=cuda).to(torch.bfloat16)
    pc = make_prefill_case(5, [0, 300], 192, 8, 2, 128)
    pq, pk, pv = pc.q.to(cuda), pc.k_new.to(cuda), pc.v_new.to(cuda)
    pkp, pvp, ptab, phist = pc.k_pool.to(cuda), pc.v_pool.to(cuda), pc.page_table.to(cuda), pc.hist.to(cuda)
    pal.paged_attention_decode_append(nk, nv, q, k, v, table, ln)  # warm-up
    pal.paged_attention_prefill(pq, pk, pv, pkp, pvp, ptab, phist)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        out_a = pal.paged_attention_decode_append(nk, nv, q, k, v, table, ln)
        out_p = pal.paged_attention_prefill(pq, pk, pv, pkp, pvp, ptab, phist)
    nk.copy_(torch.randn_like(nk))
    pq.copy_(torch.randn_like(pq))
    graph.replay()
    torch.cuda.synchronize()
    assert _bit_equal(out_a.cpu(), pal.paged_attention_decode_append(nk, nv, q, k, v, table, ln).cpu())
    assert _bit_equal(out_p.cpu(), pal.paged_attention_prefill(pq, pk, pv, pkp, pvp, ptab, phist).cpu())


def test_two_cta_prefill_replays_from_a_graph(pal, cuda):
    """The head_dim 256 prefill kernel is launched with a cluster-dimension attribute; a captured launch replays with new
    inputs like any other."""
    pc = make_prefill_case(7, [0, 300, 77], 192, 8, 2, 256)
    pq, pk, pv = pc.q.to(cuda), pc.k_new.to(cuda), pc.v_new.to(cuda)
    pkp, pvp, ptab, phist = pc.k_pool.to(cuda), pc.v_pool.to(cuda), pc.page_table.to(cuda), pc.hist.to(cuda)
    pal.paged_attention_prefill(pq, pk, pv, pkp, pvp, ptab, phist)  # warm-up
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        out_p = pal.paged_attention_prefill(pq, pk, pv, pkp, pvp, ptab, phist)
    pq.copy_(torch.randn_like(pq))
    phist.copy_(torch.tensor([16, 120, 300], dtype=phist.dtype, device=cuda))
    graph.replay()
    torch.cuda.synchronize()
    assert _bit_equal(out_p.cpu(), pal.paged_attention_prefill(pq, pk, pv, pkp, pvp, ptab, phist).cpu())
    pal.check_status()
