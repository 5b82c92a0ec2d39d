"""B200 (sm_100a) paged-attention operators behind Proxy Attention Lab's Python API.

Exports the names of ``src/proxy_attention_lab/__init__.py:17-37`` plus the split-KV building
blocks used for multi-GPU long-context decode.
"""

from . import pal_core, sharding  # noqa: F401
from .ops import (  # noqa: F401
    fill_kv_pages,
    get_k_cache_shape,
    get_k_cache_stripe_size,
    get_optimal_page_size,
    get_v_cache_shape,
    check_status,
    lse_combine,
    lse_combine_packed,
    paged_attention,
    paged_attention_decode,
    paged_attention_decode_append,
    paged_attention_decode_partials,
    paged_attention_prefill,
    paged_attention_prefill_ragged,
)

__all__ = [
    "fill_kv_pages",
    "get_k_cache_shape",
    "get_k_cache_stripe_size",
    "get_optimal_page_size",
    "get_v_cache_shape",
    "check_status",
    "lse_combine",
    "lse_combine_packed",
    "paged_attention",
    "paged_attention_decode",
    "paged_attention_decode_append",
    "paged_attention_decode_partials",
    "paged_attention_prefill",
    "paged_attention_prefill_ragged",
]
