"""Golden vectors: the oracle must keep reproducing them (CPU), and the kernels must match them (GPU)."""

import os

import pytest
import torch

from cases import assert_parity
from oracle import decode_oracle, fill_kv_pages_oracle, prefill_oracle

VECTORS = torch.load(os.path.join(os.path.dirname(__file__), "golden", "vectors.pt"))
NAMES = ["f16", "bf16"]


def bit_equal(a, b):
    return torch.equal(a.view(torch.int16), b.view(torch.int16))


@pytest.mark.parametrize("name", NAMES)
def test_oracle_reproduces_golden(name):
    d = VECTORS[f"decode_{name}"]
    assert torch.allclose(decode_oracle(d["q"], d["k_pool"], d["v_pool"], d["page_table"], d["lens"]), d["expected"], atol=1e-6)
    p = VECTORS[f"prefill_{name}"]
    assert torch.allclose(prefill_oracle(p["q"], p["k_new"], p["v_new"], p["k_pool"], p["v_pool"], p["page_table"], p["hist"]),
                          p["expected"], atol=1e-6)
    f = VECTORS[f"fill_{name}"]
    ek, ev = fill_kv_pages_oracle(f["keys"], f["vals"], f["k_pool"], f["v_pool"], f["slots"])
    assert bit_equal(ek, f["expected_k"]) and bit_equal(ev, f["expected_v"])


@pytest.mark.gpu
@pytest.mark.parametrize("name", NAMES)
def test_kernels_match_golden(pal, cuda, name):
    d = {k: v.to(cuda) for k, v in VECTORS[f"decode_{name}"].items()}
    for pp in (0, 2):
        out = pal.paged_attention_decode(d["q"], d["k_pool"], d["v_pool"], d["page_table"], d["lens"], partition_pages=pp)
        assert_parity(out, d["expected"], f"decode_{name}, partition_pages={pp}")
    p = {k: v.to(cuda) for k, v in VECTORS[f"prefill_{name}"].items()}
    out = pal.paged_attention_prefill(p["q"], p["k_new"], p["v_new"], p["k_pool"], p["v_pool"], p["page_table"], p["hist"])
    assert_parity(out, p["expected"], f"prefill_{name}")
    out32 = pal.paged_attention_prefill(p["q"], p["k_new"], p["v_new"], p["k_pool"], p["v_pool"], p["page_table"], p["hist"],
                                        out_dtype=torch.float32)
    assert_parity(out32, p["expected"], f"prefill_{name}, float32 output")
    f = {k: v.to(cuda) for k, v in VECTORS[f"fill_{name}"].items()}
    gk, gv = pal.fill_kv_pages(f["keys"], f["vals"], f["k_pool"].clone(), f["v_pool"].clone(), f["slots"])
    assert bit_equal(gk, f["expected_k"]) and bit_equal(gv, f["expected_v"])
