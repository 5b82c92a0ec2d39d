"""Regenerates the golden input/output vectors in this directory.

The reference (Proxy Attention Lab) cannot be built or imported off Apple hardware and has no CPU
path, so these vectors come from the CPU oracle after it has been pinned against the reference's
hand-computed known-answer tests (tests/test_oracle_kat.py).  Inputs are seeded; outputs are fp32.
Run from the repository root:  python tests/golden/make_golden.py
"""

import os
import sys

import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))

from cases import make_decode_case, make_prefill_case  # noqa: E402
from oracle import decode_oracle, fill_kv_pages_oracle, prefill_oracle  # noqa: E402


def main():
    out = {}
    for name, dtype in (("f16", torch.float16), ("bf16", torch.bfloat16)):
        c = make_decode_case(101, [37, 100, 16, 1], 4, 2, 64, dtype=dtype, extra_pages=3, table_width=8)
        out[f"decode_{name}"] = dict(q=c.q, k_pool=c.k_pool, v_pool=c.v_pool, page_table=c.page_table, lens=c.lens,
                                     expected=decode_oracle(c.q, c.k_pool, c.v_pool, c.page_table, c.lens))
        p = make_prefill_case(202, [21, 0], 24, 4, 2, 64, dtype=dtype)
        out[f"prefill_{name}"] = dict(q=p.q, k_new=p.k_new, v_new=p.v_new, k_pool=p.k_pool, v_pool=p.v_pool, page_table=p.page_table,
                                      hist=p.hist, expected=prefill_oracle(p.q, p.k_new, p.v_new, p.k_pool, p.v_pool, p.page_table, p.hist))
        g = torch.Generator().manual_seed(303)
        keys = torch.randn((9, 2, 64), generator=g).to(dtype)
        vals = torch.randn((9, 2, 64), generator=g).to(dtype)
        slots = torch.randperm(c.k_pool.shape[0] * 16, generator=g)[:9]
        ek, ev = fill_kv_pages_oracle(keys, vals, c.k_pool, c.v_pool, slots)
        out[f"fill_{name}"] = dict(keys=keys, vals=vals, slots=slots, k_pool=c.k_pool, v_pool=c.v_pool, expected_k=ek, expected_v=ev)
    torch.save(out, os.path.join(HERE, "vectors.pt"))
    print("wrote", os.path.join(HERE, "vectors.pt"), os.path.getsize(os.path.join(HERE, "vectors.pt")), "bytes")


if __name__ == "__main__":
    main()
