"""pal_paged_attention_decode_static: the decode entry point that brings its own scratch memory.

It exists for hosts that cannot give the library a workspace (all device memory committed to the page
pools, or a plugin interface without temporaries).  Checked here through the C ABI against the regular
entry point, on calls in a row that leave different contents in the shared scratch array, and for the
claim in its name: device memory in use does not change across a call.
"""

import ctypes

import pytest
import torch

from cases import make_decode_case

pytestmark = pytest.mark.gpu


def _call(lib, fn_name, t, S, hq, hkv, d, tpp, partition_pages, workspace=None):
    out = torch.empty((S, hq, d), dtype=t["q"].dtype, device=t["q"].device)
    stream = torch.cuda.current_stream(out.device).cuda_stream
    args = [t["q"].data_ptr(), t["k_pool"].data_ptr(), t["v_pool"].data_ptr(), t["page_table"].data_ptr(), t["lens"].data_ptr(),
            out.data_ptr(), S, hq, hkv, d, tpp, t["k_pool"].shape[0], t["page_table"].shape[1], 0.0,
            1 if out.dtype == torch.bfloat16 else 0, partition_pages]
    if workspace is not None:
        args += [workspace.data_ptr(), workspace.numel()]
    args.append(stream)
    rc = getattr(lib, fn_name)(*args)
    torch.cuda.synchronize()
    return rc, out


def test_static_scratch_decode_matches_regular_entry_point(pal, cuda):
    from proxy_attention_lab_b200 import _lib

    lib = _lib.lib
    # two different problems back to back: the second finds the first one's partials in the scratch array
    problems = [
        (make_decode_case(51, [3000, 500, 1777], 32, 8, 128, dtype=torch.bfloat16), 32, 8, 128, 16),
        (make_decode_case(52, [90, 1200], 8, 2, 64, dtype=torch.float16), 8, 2, 64, 8),
    ]
    for case, hq, hkv, d, pp in problems:
        t = {k: v.to(cuda) for k, v in vars(case).items() if isinstance(v, torch.Tensor)}
        S = len(case.lens)
        for partition_pages in (pp, 0, -1):
            nbytes = lib.pal_decode_workspace_bytes(S, hq, hkv, d, 16, t["page_table"].shape[1], partition_pages)
            ws = torch.zeros(nbytes, dtype=torch.uint8, device=cuda)  # the header starts at zero
            rc_ref, ref = _call(lib, "pal_paged_attention_decode", t, S, hq, hkv, d, 16, partition_pages, workspace=ws)
            rc, out = _call(lib, "pal_paged_attention_decode_static", t, S, hq, hkv, d, 16, partition_pages)
            assert rc_ref == _lib.PAL_OK and rc == _lib.PAL_OK, _lib.last_error()
            # the same deterministic kernels on the same inputs: every bit agrees
            assert torch.equal(out.view(torch.int16), ref.view(torch.int16))
            assert torch.isfinite(out.float()).all()
            assert lib.pal_check_status_static(torch.cuda.current_stream(cuda).cuda_stream) == _lib.PAL_OK


def test_static_scratch_call_allocates_nothing(pal, cuda):
    """Free device memory, as the driver reports it, is the same before and after a call (taken after one warm-up call:
    the first call on a device loads the array's module, which is when its 16 MiB are set aside)."""
    from proxy_attention_lab_b200 import _lib

    lib = _lib.lib
    assert lib.pal_static_scratch_init() == _lib.PAL_OK
    case = make_decode_case(53, [2000, 300, 41], 16, 4, 128, dtype=torch.bfloat16)
    t = {k: v.to(cuda) for k, v in vars(case).items() if isinstance(v, torch.Tensor)}
    out = torch.empty((3, 16, 128), dtype=torch.bfloat16, device=cuda)
    stream = torch.cuda.current_stream(cuda).cuda_stream
    args = [t["q"].data_ptr(), t["k_pool"].data_ptr(), t["v_pool"].data_ptr(), t["page_table"].data_ptr(), t["lens"].data_ptr(),
            out.data_ptr(), 3, 16, 4, 128, 16, t["k_pool"].shape[0], t["page_table"].shape[1], 0.0, 1]
    for partition_pages in (8, 0):
        assert lib.pal_paged_attention_decode_static(*args, partition_pages, stream) == _lib.PAL_OK  # warm-up: kernels loaded
        torch.cuda.synchronize()
        free_before, _ = torch.cuda.mem_get_info(cuda)
        assert lib.pal_paged_attention_decode_static(*args, partition_pages, stream) == _lib.PAL_OK
        torch.cuda.synchronize()
        free_after, _ = torch.cuda.mem_get_info(cuda)
        assert free_after == free_before


def test_static_scratch_rejects_oversized_problems(pal, cuda):
    from proxy_attention_lab_b200 import _lib

    lib = _lib.lib
    # 64 sequences x 64 heads x 128 partitions of one page: far more partial rows than 16 MiB holds
    need = lib.pal_decode_workspace_bytes(64, 64, 8, 128, 16, 128, 1)
    assert need > 16 * 1024 * 1024
    dummy = torch.zeros(16, dtype=torch.int32, device=cuda)
    p = dummy.data_ptr()
    rc = lib.pal_paged_attention_decode_static(p, p, p, p, p, p, 64, 64, 8, 128, 16, 1, 128, 0.0, 1, 1, None)
    assert rc == _lib.PAL_ERR_WORKSPACE
    assert "built-in scratch" in _lib.last_error()
