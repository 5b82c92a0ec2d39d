"""The reference's known-answer cases run through the CUDA kernels (via the C ABI)."""

import pytest
import torch

import kat

pytestmark = pytest.mark.gpu
DTYPES = [torch.float16, torch.bfloat16]


def close(out, expected, atol=kat.ATOL):
    return torch.allclose(out.float().cpu(), expected.float(), atol=atol, rtol=1e-2)


def dev(args, cuda):
    return [a.to(cuda) for a in args]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("head_dim", [32, 64, 128, 256])
@pytest.mark.parametrize("whole", [False, True])
def test_decode_first_token(pal, cuda, head_dim, dtype, whole):
    args, expected = kat.decode_first_token(head_dim, dtype, whole)
    out = pal.paged_attention_decode(*dev(args, cuda))
    assert out.shape == (2, 1, head_dim) and out.dtype == dtype and close(out, expected)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("head_dim", [32, 64, 128, 256])
def test_decode_single_token_value(pal, cuda, head_dim, dtype):
    args, expected = kat.decode_single_token_value(head_dim, dtype)
    assert close(pal.paged_attention_decode(*dev(args, cuda)), expected)


@pytest.mark.parametrize("dtype", DTYPES)
def test_decode_three_equal_scores(pal, cuda, dtype):
    args, expected = kat.decode_three_equal_scores(dtype)
    assert close(pal.paged_attention_decode(*dev(args, cuda)), expected)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("head_dim", [32, 64, 128, 256])
def test_decode_full_attention_one_block(pal, cuda, head_dim, dtype):
    args, expected = kat.decode_full_attention_one_block(head_dim, dtype)
    out = pal.paged_attention_decode(*dev(args, cuda))
    assert out.shape == (1, 1, head_dim) and close(out, expected)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("head_dim", [32, 64, 128])
def test_prefill_single_query_no_history(pal, cuda, head_dim, dtype):
    args, expected = kat.prefill_single_query_no_history(head_dim, dtype)
    out = pal.paged_attention_prefill(*dev(args, cuda))
    assert out.shape == (1, head_dim) and out.dtype == dtype and close(out, expected)


@pytest.mark.parametrize("dtype", DTYPES)
def test_prefill_causal_two_tokens(pal, cuda, dtype):
    args, expected = kat.prefill_causal_two_tokens(dtype)
    assert close(pal.paged_attention_prefill(*dev(args, cuda)), expected)


@pytest.mark.parametrize("dtype", DTYPES)
def test_prefill_with_history(pal, cuda, dtype):
    args, expected = kat.prefill_with_history(dtype)
    assert close(pal.paged_attention_prefill(*dev(args, cuda)), expected)
