"""pal_paged_attention_decode_static: the decode entry point that brings its own scratch memory.

It exists for hosts that cannot give the library a workspace (all device memory committed to the page
pools, or a plugin interface without temporaries).  Checked here through the C ABI against the regular
entry point, on two calls in a row that leave different contents in the shared scratch array.
This file sorts last on purpose, so a run that stops at the first failure has covered everything else.
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
        for partition_pages in (pp, 0):
            nbytes = lib.pal_decode_workspace_bytes(S, hq, hkv, d, 16, t["page_table"].shape[1], partition_pages)
            ws = torch.empty(nbytes, dtype=torch.uint8, device=cuda)
            rc_ref, ref = _call(lib, "pal_paged_attention_decode", t, S, hq, hkv, d, 16, partition_pages, workspace=ws)
            rc, out = _call(lib, "pal_paged_attention_decode_static", t, S, hq, hkv, d, 16, partition_pages)
            assert rc_ref == _lib.PAL_OK and rc == _lib.PAL_OK, _lib.last_error()
            # same kernels, same inputs: the results agree far inside the 2e-3 tolerance of the parity tests
            assert (out.float() - ref.float()).abs().max().item() <= 2e-3
            assert torch.isfinite(out.float()).all()


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
