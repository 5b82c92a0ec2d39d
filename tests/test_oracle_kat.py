"""Pins the CPU oracle against the reference's hand-computed known-answer cases (no GPU needed)."""

import pytest
import torch

import kat
from oracle import decode_oracle, fill_kv_pages_oracle, k_cache_shape, prefill_oracle, slots_from_page_table, v_cache_shape

DTYPES = [torch.float16, torch.bfloat16]


def close(out, expected, atol=kat.ATOL):
    return torch.allclose(out.float(), expected.float(), atol=atol, rtol=1e-2)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("head_dim", [32, 64, 128, 256])
@pytest.mark.parametrize("whole", [False, True])
def test_decode_first_token(head_dim, dtype, whole):
    args, expected = kat.decode_first_token(head_dim, dtype, whole)
    out = decode_oracle(*args)
    assert out.shape == (2, 1, head_dim) and close(out, expected)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("head_dim", [32, 64, 128, 256])
def test_decode_single_token_value(head_dim, dtype):
    args, expected = kat.decode_single_token_value(head_dim, dtype)
    assert close(decode_oracle(*args), expected)


@pytest.mark.parametrize("dtype", DTYPES)
def test_decode_three_equal_scores(dtype):
    args, expected = kat.decode_three_equal_scores(dtype)
    assert close(decode_oracle(*args), expected)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("head_dim", [32, 64, 128, 256])
def test_decode_full_attention_one_block(head_dim, dtype):
    args, expected = kat.decode_full_attention_one_block(head_dim, dtype)
    out = decode_oracle(*args)  # 2-D queries: one query head, output still [S, 1, D]
    assert out.shape == (1, 1, head_dim) and close(out, expected)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("head_dim", [32, 64, 128])
def test_prefill_single_query_no_history(head_dim, dtype):
    args, expected = kat.prefill_single_query_no_history(head_dim, dtype)
    out = prefill_oracle(*args)
    assert out.shape == (1, head_dim) and close(out, expected)


@pytest.mark.parametrize("dtype", DTYPES)
def test_prefill_causal_two_tokens(dtype):
    args, expected = kat.prefill_causal_two_tokens(dtype)
    assert close(prefill_oracle(*args), expected)


@pytest.mark.parametrize("dtype", DTYPES)
def test_prefill_with_history(dtype):
    args, expected = kat.prefill_with_history(dtype)
    assert close(prefill_oracle(*args), expected)


@pytest.mark.parametrize("dtype", DTYPES)
def test_fill_full_page_plus_one(dtype):
    """tests/paged_attention/fill_kv_pages/test_fill_multiple_tokens_single_sequence.py:208-324, incl. the
    checks that page 2 holds only slot 0."""
    T, hkv, d, tpp = 17, 8, 128, 16
    keys = torch.tensor([[[t * 10000 + h * 1000 + x for x in range(d)] for h in range(hkv)] for t in range(T)]).to(dtype)
    vals = torch.tensor([[[t * 10000 + h * 1000 + x + 50000 for x in range(d)] for h in range(hkv)] for t in range(T)]).to(dtype)
    k = torch.zeros(k_cache_shape(3, hkv, d, tpp, dtype), dtype=dtype)
    v = torch.zeros(v_cache_shape(3, hkv, d, tpp, dtype), dtype=dtype)
    pt = torch.tensor([[1, 2]], dtype=torch.int32)
    slots = slots_from_page_table(pt, torch.arange(T, dtype=torch.int32), torch.zeros(T, dtype=torch.int32), tpp)
    ek, ev = fill_kv_pages_oracle(keys, vals, k, v, slots)
    for t in range(T):
        page, slot = (1, t) if t < 16 else (2, 0)
        for h in range(hkv):
            for x in range(0, d, 17):
                assert ev[page, h, x, slot] == vals[t, h, x]
                assert ek[page, h, x // 8, slot, x % 8] == keys[t, h, x]
    assert (ek[2, :, :, 1:, :] == 0).all() and (ev[2, :, :, 1:] == 0).all()
    assert (ek[0] == 0).all() and (ev[0] == 0).all()
