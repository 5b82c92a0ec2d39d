"""The reference's hand-computed known-answer cases, restated on torch CPU tensors.

Each builder returns the operator inputs and the expected output the reference test asserts, so the
same case can be run through the CPU oracle (pinning it) and through the CUDA kernels.
Sources: tests/paged_attention/decode/test_core_functionality.py:38-316,
tests/paged_attention/decode/test_softmax_and_value.py:38-241,
tests/paged_attention/decode/test_full_attention.py:38-204,
tests/paged_attention/prefill/test_softmax_and_value.py:38-284.
"""

from __future__ import annotations

import math

import torch

from oracle import k_cache_shape, v_cache_shape

ATOL = 1e-2  # the tolerance those reference tests use


def _set_k(k_pool, page, head, token, vec):
    """Write a K vector the way the reference tests do: stripe d // 8, offset d % 8."""
    d = vec.numel()
    for i in range(d):
        k_pool[page, head, i // 8, token, i % 8] = vec[i]


def decode_first_token(head_dim, dtype, whole_vector):
    """test_fetch_k_vector_element_for_first_token_of_sequence / test_fetch_entire_k_vector_for_specific_token_slot."""
    q = torch.zeros((2, 1, head_dim), dtype=dtype)
    k = torch.zeros(k_cache_shape(2, 1, head_dim, 16, dtype), dtype=dtype)
    v = torch.zeros(v_cache_shape(2, 1, head_dim, 16, dtype), dtype=dtype)
    if whole_vector:
        q[0, 0, :] = 100.0
        q[1, 0, :] = 200.0
        k0 = torch.zeros(head_dim)
        k0[:4] = torch.tensor([1.0, 2.0, 3.0, 4.0])
        k1 = torch.zeros(head_dim)
        k1[:4] = torch.tensor([5.0, 6.0, 7.0, 8.0])
        v[0, 0, :, 0] = (torch.arange(head_dim) * 10.0 + 10.0).to(dtype)
        v[1, 0, :, 0] = (torch.arange(head_dim) * 10.0 + 50.0).to(dtype)
    else:
        q[0, 0, 0] = 100.0
        q[1, 0, 0] = 200.0
        k0 = torch.zeros(head_dim)
        k0[0] = 11.0
        k1 = torch.zeros(head_dim)
        k1[0] = 22.0
        v[0, 0, :, 0] = (torch.arange(head_dim) * 10.0 + 10.0).to(dtype)
        v[1, 0, :, 0] = (torch.arange(head_dim) * 100.0 + 100.0).to(dtype)
    _set_k(k, 0, 0, 0, k0.to(dtype))
    _set_k(k, 1, 0, 0, k1.to(dtype))
    # unused second entries hold page ids far outside the pool (99 / 88 in the reference)
    table = torch.tensor([[0, 99], [1, 88]], dtype=torch.int32)
    lens = torch.tensor([1, 1], dtype=torch.int32)
    expected = torch.stack([v[0, 0, :, 0], v[1, 0, :, 0]]).reshape(2, 1, head_dim)
    return (q, k, v, table, lens), expected


def decode_single_token_value(head_dim, dtype):
    """test_v_aggregation_decode_single_sequence: one cached token, output == its V."""
    q = torch.ones((1, 1, head_dim), dtype=dtype)
    k = torch.zeros(k_cache_shape(1, 1, head_dim, 16, dtype), dtype=dtype)
    v = torch.zeros(v_cache_shape(1, 1, head_dim, 16, dtype), dtype=dtype)
    kv = torch.zeros(head_dim, dtype=dtype)
    kv[:4] = 1.0
    _set_k(k, 0, 0, 0, kv)
    v[0, 0, :4, 0] = torch.tensor([10.0, 20.0, 30.0, 40.0], dtype=dtype)
    expected = torch.zeros((1, 1, head_dim), dtype=dtype)
    expected[0, 0, :4] = torch.tensor([10.0, 20.0, 30.0, 40.0], dtype=dtype)
    return (q, k, v, torch.tensor([[0]], dtype=torch.int32), torch.tensor([1], dtype=torch.int32)), expected


def decode_three_equal_scores(dtype):
    """test_decode_multi_token_context: three keys with equal scores -> probabilities 1/3 each."""
    d = 32
    q = torch.ones((1, 1, d), dtype=dtype)
    k = torch.zeros(k_cache_shape(1, 1, d, 16, dtype), dtype=dtype)
    v = torch.zeros(v_cache_shape(1, 1, d, 16, dtype), dtype=dtype)
    for tok, sl in enumerate((slice(0, 2), slice(1, 3), slice(2, 4))):
        kv = torch.zeros(d, dtype=dtype)
        kv[sl] = 1.0
        _set_k(k, 0, 0, tok, kv)
        v[0, 0, tok, tok] = 1.0
    expected = torch.zeros((1, 1, d), dtype=torch.float32)
    expected[0, 0, :3] = 1.0 / 3.0
    return (q, k, v, torch.tensor([[0]], dtype=torch.int32), torch.tensor([3], dtype=torch.int32)), expected


def decode_full_attention_one_block(head_dim, dtype):
    """test_full_attention_in_one_block: K = ones * {1, 2, 0.5}, V rows arange(base, base + D)."""
    q = (torch.arange(1, head_dim + 1, dtype=torch.float32) / 10.0).to(dtype).reshape(1, head_dim)
    k = torch.zeros(k_cache_shape(1, 1, head_dim, 16, dtype), dtype=dtype)
    v = torch.zeros(v_cache_shape(1, 1, head_dim, 16, dtype), dtype=dtype)
    mult = [1.0, 2.0, 0.5]
    for tok, mval in enumerate(mult):
        _set_k(k, 0, 0, tok, (torch.ones(head_dim) * mval).to(dtype))
    for pos, base in enumerate([10.0, 20.0, 30.0]):
        v[0, 0, :, pos] = torch.arange(base, base + head_dim, dtype=torch.float32).to(dtype)
    # expectation computed as the reference test does, from first principles
    scale = 1.0 / math.sqrt(head_dim)
    qf = q[0].float()
    scores = torch.tensor([float((qf * mval).sum()) * scale for mval in mult])
    probs = torch.softmax(scores, dim=0)
    expected = sum(v[0, 0, :, i].float() * probs[i] for i in range(3)).reshape(1, 1, head_dim)
    return (q, k, v, torch.tensor([[0]], dtype=torch.int32), torch.tensor([3], dtype=torch.int32)), expected


def _empty_pools(d, dtype):
    return (torch.zeros(k_cache_shape(0, 1, d, 16, dtype), dtype=dtype), torch.zeros(v_cache_shape(0, 1, d, 16, dtype), dtype=dtype),
            torch.zeros((1, 0), dtype=torch.int32), torch.tensor([0], dtype=torch.int32))


def prefill_single_query_no_history(head_dim, dtype):
    """test_v_aggregation_prefill_single_query_no_history: output == V."""
    q = torch.ones((1, 1, head_dim), dtype=dtype)
    k = torch.ones((1, 1, head_dim), dtype=dtype)
    k[0, 0, :4] = torch.tensor([1.0, 1.0, 0.0, 0.0], dtype=dtype)
    v = torch.zeros((1, 1, head_dim), dtype=dtype)
    v[0, 0, :4] = torch.tensor([10.0, 20.0, 30.0, 40.0], dtype=dtype)
    kp, vp, pt, ctx = _empty_pools(head_dim, dtype)
    expected = torch.zeros((1, head_dim), dtype=torch.float32)
    expected[0, :4] = torch.tensor([10.0, 20.0, 30.0, 40.0])
    return (q, k, v, kp, vp, pt, ctx), expected


def prefill_causal_two_tokens(dtype):
    """test_prefill_causal_mask_two_tokens: rows [1,0,..] and [.5,.5,..]."""
    d = 32
    q = torch.ones((2, 1, d), dtype=dtype)
    k = torch.zeros((2, 1, d), dtype=dtype)
    k[0, 0, :2] = 1.0
    k[1, 0, 1:3] = 1.0
    v = torch.zeros((2, 1, d), dtype=dtype)
    v[0, 0, 0] = 1.0
    v[1, 0, 1] = 1.0
    kp, vp, pt, ctx = _empty_pools(d, dtype)
    expected = torch.zeros((2, d), dtype=torch.float32)
    expected[0, 0] = 1.0
    expected[1, :2] = 0.5
    return (q, k, v, kp, vp, pt, ctx), expected


def prefill_with_history(dtype):
    """test_prefill_with_history: 2 cached + 2 new tokens -> rows [1/3,1/3,1/3,0], [1/4]*4."""
    d = 32
    q = torch.ones((2, 1, d), dtype=dtype)
    k = torch.zeros((2, 1, d), dtype=dtype)
    k[0, 0, 2:4] = 1.0
    k[1, 0, 3:5] = 1.0
    v = torch.zeros((2, 1, d), dtype=dtype)
    v[0, 0, 2] = 1.0
    v[1, 0, 3] = 1.0
    kp = torch.zeros(k_cache_shape(1, 1, d, 16, dtype), dtype=dtype)
    vp = torch.zeros(v_cache_shape(1, 1, d, 16, dtype), dtype=dtype)
    h0 = torch.zeros(d, dtype=dtype)
    h0[:2] = 1.0
    h1 = torch.zeros(d, dtype=dtype)
    h1[1:3] = 1.0
    _set_k(kp, 0, 0, 0, h0)
    _set_k(kp, 0, 0, 1, h1)
    vp[0, 0, 0, 0] = 1.0
    vp[0, 0, 1, 1] = 1.0
    expected = torch.zeros((2, d), dtype=torch.float32)
    expected[0, :3] = 1.0 / 3.0
    expected[1, :4] = 0.25
    return (q, k, v, kp, vp, torch.tensor([[0]], dtype=torch.int32), torch.tensor([2], dtype=torch.int32)), expected
