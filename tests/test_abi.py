"""The C-ABI library loads, exports every symbol the header declares, and validates arguments
before it touches a device (no GPU needed: none of these calls reaches a kernel launch)."""

import ctypes
import re
from pathlib import Path

import pytest
import torch

ROOT = Path(__file__).resolve().parent.parent


def declared_symbols():
    text = (ROOT / "include" / "pal_b200.h").read_text()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(pal_[a-z0-9_]+)\s*\(", text)))


def test_header_symbols_are_exported_and_bound():
    from proxy_attention_lab_b200 import _lib

    names = declared_symbols()
    assert len(names) >= 14
    for name in names:
        assert hasattr(_lib.lib, name), f"{name} is declared in the header but not exported"
        assert name in _lib.SIGNATURES, f"{name} has no ctypes signature"
    assert sorted(_lib.SIGNATURES) == names


def test_layout_helpers():
    import proxy_attention_lab_b200 as pal
    from oracle import k_cache_shape, k_cache_stripe_size, v_cache_shape

    for dtype in (torch.float16, torch.bfloat16):
        assert pal.get_k_cache_stripe_size(dtype) == k_cache_stripe_size(dtype) == 8
        assert pal.get_k_cache_shape(7, 2, 128, 16, dtype) == k_cache_shape(7, 2, 128, 16, dtype) == (7, 2, 16, 16, 8)
        assert pal.get_v_cache_shape(7, 2, 128, 16, dtype) == v_cache_shape(7, 2, 128, 16, dtype) == (7, 2, 128, 16)
    assert pal.get_optimal_page_size() == 16
    assert pal.pal_core.get_optimal_page_size() == 16
    with pytest.raises(ValueError):
        pal.get_k_cache_stripe_size(torch.float32)


def test_reference_names_are_exported():
    import proxy_attention_lab_b200 as pal

    for name in ("fill_kv_pages", "paged_attention_decode", "paged_attention_prefill", "get_k_cache_shape",
                 "get_v_cache_shape", "get_k_cache_stripe_size", "get_optimal_page_size"):
        assert callable(getattr(pal, name)) and callable(getattr(pal.pal_core, name))


def test_validation_errors_come_back_as_codes():
    from proxy_attention_lab_b200 import _lib

    lib = _lib.lib
    # dtype 7 does not exist
    rc = lib.pal_get_k_cache_stripe_size(7)
    assert rc == _lib.PAL_ERR_UNSUPPORTED and "dtype" in _lib.last_error()
    rc = lib.pal_fill_kv_pages_slots(None, None, None, None, None, 1, 1, 64, 16, 1, 0, None)
    assert rc == _lib.PAL_ERR_BAD_ARG and "slot_mapping" in _lib.last_error()
    # Hq not a multiple of Hkv
    dummy = ctypes.create_string_buffer(64)  # only has to be non-null: validation fails before any use
    rc = lib.pal_paged_attention_decode(None, None, None, None, None, ctypes.addressof(dummy), 1, 3, 2, 64, 16, 1, 1, 0.0, 0, 0,
                                        None, 0, None)
    assert rc == _lib.PAL_ERR_BAD_ARG and "multiple" in _lib.last_error()
    # null pointers
    rc = lib.pal_paged_attention_decode(None, None, None, None, None, None, 1, 2, 2, 64, 16, 1, 1, 0.0, 0, 0, None, 0, None)
    assert rc == _lib.PAL_ERR_BAD_ARG
    # zero work is fine and launches nothing
    assert lib.pal_fill_kv_pages_slots(None, None, None, None, None, 0, 1, 64, 16, 1, 0, None) == _lib.PAL_OK
    assert lib.pal_paged_attention_decode(None, None, None, None, None, None, 0, 2, 2, 64, 16, 1, 1, 0.0, 0, 0, None, 0, None) == _lib.PAL_OK
    # workspace sizing: header only for the single pass, partials for the two-pass form
    assert lib.pal_decode_workspace_bytes(8, 64, 8, 128, 16, 8192, 0) == 256
    two_pass = lib.pal_decode_workspace_bytes(8, 64, 8, 128, 16, 8192, 256)
    rows = 8 * 64 * 32
    assert two_pass >= 256 + rows * (128 + 2) * 4
    with pytest.raises(RuntimeError):
        _lib.check(_lib.PAL_ERR_UNSUPPORTED)
    with pytest.raises(ValueError):
        _lib.check(_lib.PAL_ERR_BAD_ARG)


def test_cpu_tensors_are_rejected():
    import proxy_attention_lab_b200 as pal

    q = torch.zeros((1, 2, 64), dtype=torch.float16)
    k = torch.zeros((1, 2, 8, 16, 8), dtype=torch.float16)
    v = torch.zeros((1, 2, 64, 16), dtype=torch.float16)
    with pytest.raises(RuntimeError, match="no CPU path"):
        pal.paged_attention_decode(q, k, v, torch.zeros((1, 1), dtype=torch.int32), torch.ones(1, dtype=torch.int32))
    with pytest.raises(RuntimeError, match="no CPU path"):
        pal.fill_kv_pages(q, q, k, v, torch.zeros(1, dtype=torch.int64))


def test_validators_are_reentrant_from_several_threads():
    """Argument validation, error strings and the one-time set-up guards can be used from many host threads at once:
    every thread sees its own error message (thread-local), and no call reaches a device."""
    import threading

    from proxy_attention_lab_b200 import _lib

    lib = _lib.lib
    errors = []

    def worker(i):
        try:
            dummy = ctypes.create_string_buffer(64)
            for k in range(300):
                if (i + k) % 2:
                    rc = lib.pal_paged_attention_decode(None, None, None, None, None, ctypes.addressof(dummy), 1, 3, 2, 64, 16, 1, 1,
                                                        0.0, 0, 0, None, 0, None)
                    assert rc == _lib.PAL_ERR_BAD_ARG and "multiple" in _lib.last_error(), _lib.last_error()
                else:
                    rc = lib.pal_get_k_cache_stripe_size(7 + i)
                    assert rc == _lib.PAL_ERR_UNSUPPORTED and f"dtype {7 + i}" in _lib.last_error(), _lib.last_error()
                assert lib.pal_decode_workspace_bytes(8, 64, 8, 128, 16, 8192, 0) == 256
                assert lib.pal_set_wait_limit_cycles(0) > 0
        except Exception as e:  # noqa: BLE001
            errors.append(repr(e))

    threads = [threading.Thread(target=worker, args=(i,)) for i in range(8)]
    for t in threads:
        t.start()
    for t in threads:
        t.join()
    assert not errors, errors


def test_out_f32_flag_and_new_entry_points_validate():
    from proxy_attention_lab_b200 import _lib

    lib = _lib.lib
    # the flag is accepted together with a valid element type and refused with an invalid one
    assert lib.pal_paged_attention_decode(None, None, None, None, None, None, 0, 2, 2, 64, 16, 1, 1, 0.0, _lib.PAL_OUT_F32 | 1, 0,
                                          None, 0, None) == _lib.PAL_OK
    assert lib.pal_paged_attention_decode(None, None, None, None, None, None, 0, 2, 2, 64, 16, 1, 1, 0.0, _lib.PAL_OUT_F32 | 5, 0,
                                          None, 0, None) == _lib.PAL_ERR_UNSUPPORTED
    assert lib.pal_lse_combine_packed(None, None, 2, 4, 64, 1, None) == _lib.PAL_ERR_BAD_ARG
    assert lib.pal_lse_combine_packed(None, None, 2, 0, 64, 1, None) == _lib.PAL_OK
    assert lib.pal_workspace_init(None, 0, None) == _lib.PAL_ERR_WORKSPACE
    assert lib.pal_check_status(None, None) == _lib.PAL_ERR_BAD_ARG
    rc = lib.pal_paged_attention_decode_partials_packed(None, None, None, None, None, None, 1, 2, 2, 64, 16, 1, 1, 0.0, 0, 0, None, 0, None)
    assert rc == _lib.PAL_ERR_BAD_ARG and "partition_pages" in _lib.last_error()


def test_auto_partition_size_gives_the_memory_system_enough_ctas():
    """PAL_DECODE_AUTO: single pass when the batch alone fills the GPU; otherwise as few partitions as still put a work
    item on most of the resident CTAs (two per SM; 148 SMs assumed when no device is present) in a single wave."""
    from proxy_attention_lab_b200 import _lib, ops

    f = _lib.lib.pal_decode_auto_partition_pages
    assert f(64, 32, 8, 128, 16, 512) == 0            # Llama-3-8B batch: 512 work items, single pass
    assert f(4, 8, 2, 128, 16, 32) == 0               # short contexts are never split
    for seqs, hq, hkv, mp in ((8, 8, 1, 8192), (8, 64, 8, 8192), (8, 64, 8, 1024), (8, 32, 4, 8192)):
        pp = f(seqs, hq, hkv, 128, 16, mp)            # the 70B long-context shape, whole and sharded 8 ways
        items = seqs * hkv * -(-mp // pp)
        assert 16 <= pp < mp and 200 <= items <= 296, (seqs, hkv, mp, pp, items)
    assert f(0, 8, 1, 128, 16, 8192) == 0 and f(8, 8, 1, 128, 16, 0) == 0
    # the forms that always split fall back to one partition where the launcher would not split at all
    assert ops.resolve_partition_pages(None, 64, 32, 8, 128, 16, 512) == 512
    assert ops.resolve_partition_pages(37, 64, 32, 8, 128, 16, 512) == 37
    assert ops.resolve_partition_pages(-1, 8, 8, 1, 128, 16, 8192) == f(8, 8, 1, 128, 16, 8192)


def test_prefill_impl_argument_is_validated_before_anything_runs():
    """impl 0..4 exist; 4 (two CTAs per MMA) needs head_dim 128 / 256 and an even number of query heads per kv head.
    The buffers are host memory that is never touched: every call fails in validation."""
    from proxy_attention_lab_b200 import _lib

    lib = _lib.lib
    raw = ctypes.create_string_buffer(4096)
    base = (ctypes.addressof(raw) + 255) & ~255  # 256-byte aligned, as the workspace must be
    buf = ctypes.c_void_p(base)

    def call(hq, hkv, d, impl):
        return lib.pal_paged_attention_prefill(buf, buf, buf, buf, buf, buf, ctypes.cast(buf, ctypes.POINTER(ctypes.c_int32)), buf, 1, 64,
                                               hq, hkv, d, 16, 1, 1, 0.0, 1, impl, buf, 256, None)

    assert call(4, 2, 128, 5) == _lib.PAL_ERR_BAD_ARG and "impl" in _lib.last_error()
    assert call(4, 2, 128, -1) == _lib.PAL_ERR_BAD_ARG
    assert call(4, 2, 64, 4) == _lib.PAL_ERR_UNSUPPORTED and "two-CTA" in _lib.last_error()
    assert call(3, 3, 128, 4) == _lib.PAL_ERR_UNSUPPORTED
    assert call(4, 2, 48, 2) == _lib.PAL_ERR_UNSUPPORTED


def test_cpp_front_is_built_and_declines_what_it_does_not_handle():
    """The operators' C++ front end (csrc/torch_fastpath.cpp) loads beside the library, and answers None / False for calls
    that are not its common case - here CPU tensors - so that the Python path behind it raises the usual errors."""
    import torch

    from proxy_attention_lab_b200 import ops

    assert ops._fast is not None
    x = torch.zeros((2, 4, 64), dtype=torch.float16)
    assert ops._fast.decode(x, x, x, x, x, 0, 0.0, False, {}, None, None) is None
    assert ops._fast.prefill(x, x, x, x, x, x, x, 0, 0.0, False, {}, None, 0) is None
    assert ops._fast.fill(x, x, x, x, x, None, None) is False
    with pytest.raises(RuntimeError):
        ops.paged_attention_decode(x, x, x, x, x)


def test_prefill_workspace_plans_the_history_split_from_the_shape():
    """pal_prefill_workspace_bytes: the header alone for batches that fill the GPU (and for head_dim 256, which runs the
    two-CTA kernel), header + fp32 partial triples - rows x parts x (D + 2) floats, at most 32 MB - for the few-CTA batches
    that the tcgen05 kernel cuts along the history."""
    from proxy_attention_lab_b200 import _lib

    f = _lib.lib.pal_prefill_workspace_bytes
    assert f(8, 2048, 32, 8, 128) == 256 and f(64, 16, 32, 8, 128) == 256 and f(1, 1, 8, 2, 256) == 256
    one = f(1, 1, 8, 2, 128)  # 4 CTAs: 16 parts at most
    assert one == 256 + 1 * 1 * 8 * 16 * 130 * 4
    big = f(1, 128, 32, 8, 128)  # 16 CTAs -> 9 parts
    assert big == 256 + 128 * 32 * 9 * 130 * 4
    assert f(4, 128, 32, 8, 128) - 256 <= 32 << 20
    assert f(0, 16, 8, 2, 128) == 256
