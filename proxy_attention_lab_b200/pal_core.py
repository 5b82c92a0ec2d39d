"""Stand-in for the reference's compiled ``proxy_attention_lab.pal_core`` module: the same seven
names (``src/pal_core/bindings.cpp:44-222``) so that code importing them from there keeps working."""

from .ops import (  # noqa: F401
    fill_kv_pages,
    get_k_cache_shape,
    get_k_cache_stripe_size,
    get_optimal_page_size,
    get_v_cache_shape,
    paged_attention_decode,
    paged_attention_prefill,
)

__version__ = "2025.06.4+b200"
