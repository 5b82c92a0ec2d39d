"""Behaviour at the operator boundary on a GPU: streams, workspaces, the status word of the bounded waits, query forms."""

import pytest
import torch

from cases import assert_parity, make_decode_case, make_prefill_case, to_dev
from oracle import decode_oracle, prefill_oracle

pytestmark = pytest.mark.gpu


def test_status_is_ok_after_normal_calls(pal, cuda):
    from proxy_attention_lab_b200 import _lib

    case = make_decode_case(61, [300, 40], 8, 2, 128, dtype=torch.bfloat16)
    t = to_dev(case, cuda)
    for pp in (0, 4):
        pal.paged_attention_decode(t["q"], t["k_pool"], t["v_pool"], t["page_table"], t["lens"], partition_pages=pp)
        pal.check_status()  # raises on PAL_ERR_TIMEOUT
    pc = make_prefill_case(62, [50, 0], 200, 8, 2, 128, dtype=torch.bfloat16)
    p = to_dev(pc, cuda)
    for impl in ("mma", "tcgen05"):
        pal.paged_attention_prefill(p["q"], p["k_new"], p["v_new"], p["k_pool"], p["v_pool"], p["page_table"], p["hist"], impl=impl)
        pal.check_status()
    # through the C ABI, on a workspace of the test's own
    lib = _lib.lib
    ws = torch.zeros(4096, dtype=torch.uint8, device=cuda)
    stream = torch.cuda.current_stream().cuda_stream
    assert lib.pal_workspace_init(ws.data_ptr(), ws.numel(), stream) == _lib.PAL_OK
    assert lib.pal_check_status(ws.data_ptr(), stream) == _lib.PAL_OK


def test_an_expired_wait_is_reported_and_the_workspace_recovers(pal, cuda):
    """A wait that nothing ends runs into its limit (a few thousand cycles here): the kernel returns normally, the
    status word says PAL_ERR_TIMEOUT, and the next call on the same workspace works."""
    from proxy_attention_lab_b200 import _lib

    lib = _lib.lib
    case = make_decode_case(63, [500, 77, 129], 8, 2, 128, dtype=torch.float16)
    t = to_dev(case, cuda)
    S, hq, hkv, d = 3, 8, 2, 128
    nbytes = lib.pal_decode_workspace_bytes(S, hq, hkv, d, 16, t["page_table"].shape[1], 4)
    ws = torch.empty(nbytes, dtype=torch.uint8, device=cuda)
    stream = torch.cuda.current_stream().cuda_stream
    assert lib.pal_workspace_init(ws.data_ptr(), ws.numel(), stream) == _lib.PAL_OK
    assert lib.pal_selftest_bounded_wait(ws.data_ptr(), 5000, stream) == _lib.PAL_OK
    assert lib.pal_check_status(ws.data_ptr(), stream) == _lib.PAL_ERR_TIMEOUT
    assert "timed out" in _lib.last_error()
    with pytest.raises(RuntimeError, match="timed out"):
        _lib.check(_lib.PAL_ERR_TIMEOUT)
    # reading the timeout cleared it; the workspace serves a normal call again
    assert lib.pal_check_status(ws.data_ptr(), stream) == _lib.PAL_OK
    out = torch.empty((S, hq, d), dtype=torch.float16, device=cuda)
    rc = lib.pal_paged_attention_decode(t["q"].data_ptr(), t["k_pool"].data_ptr(), t["v_pool"].data_ptr(), t["page_table"].data_ptr(),
                                        t["lens"].data_ptr(), out.data_ptr(), S, hq, hkv, d, 16, t["k_pool"].shape[0],
                                        t["page_table"].shape[1], 0.0, 0, 4, ws.data_ptr(), ws.numel(), stream)
    assert rc == _lib.PAL_OK, _lib.last_error()
    assert lib.pal_check_status(ws.data_ptr(), stream) == _lib.PAL_OK
    assert_parity(out, decode_oracle(case.q, case.k_pool, case.v_pool, case.page_table, case.lens))
    # the limit of the library's own waits can be changed and restored
    old = lib.pal_set_wait_limit_cycles(123456789)
    assert lib.pal_set_wait_limit_cycles(old) == 123456789
    assert lib.pal_selftest_bounded_wait(ws.data_ptr(), 0, stream) == _lib.PAL_ERR_BAD_ARG


def test_calls_on_a_side_stream_with_inputs_that_need_conversion(pal, cuda):
    """int64 page table and lengths, a non-contiguous query: the conversions, the allocations and the launch all happen
    on the stream that was named, with nothing ordering it against the current stream."""
    case = make_decode_case(64, [1000, 333, 2047, 64], 32, 8, 128, dtype=torch.bfloat16)
    ref = decode_oracle(case.q, case.k_pool, case.v_pool, case.page_table, case.lens)
    t = to_dev(case, cuda)
    q_nc = torch.empty((4, 32, 256), dtype=torch.bfloat16, device=cuda)[:, :, ::2]
    q_nc.copy_(t["q"])
    table64, lens64 = t["page_table"].to(torch.int64), t["lens"].to(torch.int64)
    torch.cuda.synchronize()
    side = torch.cuda.Stream()
    for stream in (side, side.cuda_stream):
        for _ in range(20):  # many short calls: a launch that overtook its conversions would show here
            out = pal.paged_attention_decode(q_nc, t["k_pool"], t["v_pool"], table64, lens64, stream=stream, partition_pages=0)
        side.synchronize()
        assert_parity(out, ref, "side stream")
    pc = make_prefill_case(65, [100, 0], 150, 8, 2, 128, dtype=torch.bfloat16)
    p = to_dev(pc, cuda)
    pref = prefill_oracle(pc.q, pc.k_new, pc.v_new, pc.k_pool, pc.v_pool, pc.page_table, pc.hist)
    torch.cuda.synchronize()
    out = pal.paged_attention_prefill(p["q"], p["k_new"], p["v_new"], p["k_pool"], p["v_pool"], p["page_table"].to(torch.int64),
                                      p["hist"].to(torch.int64), stream=side)
    side.synchronize()
    assert_parity(out, pref, "prefill on a side stream")


def test_workspace_growth_keeps_earlier_buffers(pal, cuda):
    """A larger problem gets a larger workspace; the earlier one stays alive (a captured graph may still use it)."""
    from proxy_attention_lab_b200 import ops

    small = make_decode_case(66, [200, 100], 8, 2, 64, dtype=torch.float16)
    big = make_decode_case(67, [3000] * 6, 32, 8, 128, dtype=torch.float16)
    side = torch.cuda.Stream()
    ts, tb = to_dev(small, cuda), to_dev(big, cuda)
    torch.cuda.synchronize()
    pal.paged_attention_decode(ts["q"], ts["k_pool"], ts["v_pool"], ts["page_table"], ts["lens"], partition_pages=2, stream=side)
    held = ops._WORKSPACES[(cuda.index, side.cuda_stream)]
    first, first_ptr = held[-1], held[-1].data_ptr()
    out = pal.paged_attention_decode(tb["q"], tb["k_pool"], tb["v_pool"], tb["page_table"], tb["lens"], partition_pages=1, stream=side)
    side.synchronize()
    assert len(held) >= 2 and held[0] is first and held[0].data_ptr() == first_ptr and held[-1].numel() > first.numel()
    assert_parity(out, decode_oracle(big.q, big.k_pool, big.v_pool, big.page_table, big.lens))


def test_one_dimensional_queries(pal, cuda):
    """A flat query buffer is read as rows of head_dim elements with one query head (what the reference's kernel does
    with it); anything that is not a whole number of rows is refused."""
    case = make_decode_case(68, [33, 20, 64], 1, 1, 64, dtype=torch.float16)
    t = to_dev(case, cuda)
    ref = decode_oracle(case.q, case.k_pool, case.v_pool, case.page_table, case.lens)
    out = pal.paged_attention_decode(t["q"].reshape(-1), t["k_pool"], t["v_pool"], t["page_table"], t["lens"])
    assert out.shape == (3, 1, 64)
    assert_parity(out, ref)
    with pytest.raises(ValueError):
        pal.paged_attention_decode(t["q"].reshape(-1)[:3], t["k_pool"], t["v_pool"], t["page_table"], t["lens"])
    with pytest.raises(ValueError):
        pal.paged_attention_decode(t["q"].reshape(-1)[: 2 * 64 + 5], t["k_pool"], t["v_pool"], t["page_table"], t["lens"])
    with pytest.raises(ValueError):
        pal.paged_attention_decode(t["q"][:, :, None, :], t["k_pool"], t["v_pool"], t["page_table"], t["lens"])


def test_out_dtype_is_checked(pal, cuda):
    case = make_decode_case(69, [20], 2, 2, 64, dtype=torch.float16)
    t = to_dev(case, cuda)
    with pytest.raises(ValueError):
        pal.paged_attention_decode(t["q"], t["k_pool"], t["v_pool"], t["page_table"], t["lens"], out_dtype=torch.bfloat16)
    out = pal.paged_attention_decode(t["q"], t["k_pool"], t["v_pool"], t["page_table"], t["lens"], out_dtype=torch.float16)
    assert out.dtype == torch.float16


def test_cpp_front_and_ctypes_path_agree(pal, cuda, monkeypatch):
    """The operators' C++ front (the common case) and the ctypes path behind it make the same C-ABI calls: identical
    outputs for decode, append + decode, prefill and fill; and what the front declines (int64 page table, 2-D queries,
    a side stream) still works."""
    from proxy_attention_lab_b200 import ops

    assert ops._fast is not None, "the C++ front was not built (proxy_attention_lab_b200/build.py builds it)"
    g = torch.Generator(device=cuda).manual_seed(3)
    S, hq, hkv, d, tpp, P = 3, 8, 2, 128, 16, 24
    mk = lambda *shape: torch.randn(shape, device=cuda, dtype=torch.bfloat16, generator=g)
    q, kp, vp = mk(S, hq, d), mk(P, hkv, d // 8, tpp, 8), mk(P, hkv, d, tpp)
    table = torch.randperm(P, device=cuda).reshape(S, P // S).to(torch.int32)
    lens = torch.tensor([100, 17, 128], dtype=torch.int32, device=cuda)
    qp, kn, vn = mk(S * 70, hq, d), mk(S * 70, hkv, d), mk(S * 70, hkv, d)
    nk, nv = mk(S, hkv, d), mk(S, hkv, d)
    slots = torch.tensor([5, 77, 300], dtype=torch.int64, device=cuda)
    cu = torch.tensor([0, 130, 131, 210], dtype=torch.int32, device=cuda)  # ragged view of the same 210 prompt rows

    def run_all():
        k2, v2 = kp.clone(), vp.clone()
        outs = [pal.paged_attention_decode(q, kp, vp, table, lens), pal.paged_attention_decode(q, kp, vp, table, lens, partition_pages=2),
                pal.paged_attention_decode(q, kp, vp, table, lens, out_dtype=torch.float32),
                pal.paged_attention_prefill(qp, kn, vn, kp, vp, table, lens),
                pal.paged_attention_prefill_ragged(qp, kn, vn, kp, vp, table, lens, cu, max_new_tokens=130),
                pal.paged_attention_decode_append(nk, nv, q, k2, v2, table, lens)]
        pal.fill_kv_pages(nk, nv, k2, v2, slots)
        pal.fill_kv_pages(nk, nv, k2, v2, table, lens - 1, torch.arange(S, dtype=torch.int32, device=cuda))
        torch.cuda.synchronize()
        return [o.cpu() for o in outs] + [k2.cpu(), v2.cpu()]

    fast = run_all()
    monkeypatch.setattr(ops, "_fast", None)
    slow = run_all()
    for a, b in zip(fast, slow):
        assert a.dtype == b.dtype and torch.equal(a.view(torch.int16) if a.dtype != torch.float32 else a, b.view(torch.int16) if b.dtype != torch.float32 else b)
    monkeypatch.undo()
    # declined by the front, served by the path behind it
    ref = pal.paged_attention_decode(q, kp, vp, table, lens).cpu()
    assert torch.equal(pal.paged_attention_decode(q, kp, vp, table.to(torch.int64), lens).cpu().view(torch.int16), ref.view(torch.int16))
    side = torch.cuda.Stream(device=cuda)
    side.wait_stream(torch.cuda.current_stream(cuda))
    out_side = pal.paged_attention_decode(q, kp, vp, table, lens, stream=side)
    side.synchronize()
    assert torch.equal(out_side.cpu().view(torch.int16), ref.view(torch.int16))
    pal.check_status()
