"""CPU oracle for the paged-attention hot path.  TEST INFRASTRUCTURE ONLY.

This package is a CPU restatement (torch-CPU / numpy, fp32 arithmetic) of what
Proxy Attention Lab's three Metal kernels compute.  It exists so that the CUDA
kernels can be checked against something that does not share their code.

Only the test-suite, the smoke check and the benchmark's CPU-baseline leg may
import it.  The product package never does: it fails loudly when its CUDA
library is missing instead of falling back to this code.

How the oracle itself is pinned: the reference has no CPU implementation
(``eval_cpu`` throws in all three primitives,
``src/pal_core/src/paged_attention_decode_primitive.cpp:63-69``) and cannot be
built or imported off Apple hardware, so the oracle is checked against the
hand-computed known-answer cases in the reference's own tests (ported in
``tests/test_oracle_kat.py``) and against the exact-placement expectations of all
its ``fill_kv_pages`` tests.  The reference's randomized SDPA-equivalence tests
draw unseeded inputs, so they pin semantics (softmax(QK^T/sqrt(D)+mask)V with GQA
broadcast), not vectors.
"""

from .layouts import (  # noqa: F401
    MEMORY_ALIGNMENT_BYTES,
    gather_sequence_kv,
    k_cache_shape,
    k_cache_stripe_size,
    pack_sequences_into_pages,
    v_cache_shape,
)
from .attention import (  # noqa: F401
    decode_oracle,
    decode_partials_oracle,
    lse_combine_oracle,
    prefill_oracle,
    prefill_ragged_oracle,
)
from .fill import fill_kv_pages_oracle, slots_from_page_table  # noqa: F401
