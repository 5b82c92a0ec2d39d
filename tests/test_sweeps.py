"""The sweep tool writes the reference's results.json layout (benchmarks/benchmarks.md:198-236)."""

import json

import pytest
import torch

from proxy_attention_lab_b200 import sweeps


def test_refuses_to_run_without_a_gpu(tmp_path):
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    assert sweeps.main(["--out", str(tmp_path / "r.json"), "--quick"]) == 2
    assert not (tmp_path / "r.json").exists()


@pytest.mark.gpu
def test_quick_sweep_schema(tmp_path):
    out = tmp_path / "results.json"
    assert sweeps.main(["--out", str(out), "--quick", "--warmup", "1", "--iters", "2", "--reps", "2"]) == 0
    r = json.loads(out.read_text())
    assert set(r) == {"latency_vs_seq_len", "batch_decode_latency", "fill_kv_pages"}
    fill = r["fill_kv_pages"]
    assert set(fill) == {"latency_vs_num_new_tokens", "latency_vs_num_sequences", "latency_vs_dimensions"}
    for series in list(fill["latency_vs_num_new_tokens"].values()) + list(fill["latency_vs_num_sequences"].values()) + list(fill["latency_vs_dimensions"].values()):
        assert series and all(v > 0 for v in series.values())
    for kind in ("prefill", "decode"):
        series = r["latency_vs_seq_len"][kind][sweeps.GROUP]
        assert series and all(float(k) > 0 and v > 0 for k, v in series.items())
    lat = r["batch_decode_latency"]["latency_vs_num_sequences"]
    thr = r["batch_decode_latency"]["throughput_vs_num_sequences"]
    assert set(lat) == set(thr) and all(k.startswith("H=") for k in lat)
    for h in lat:
        for n, ms in lat[h].items():
            assert thr[h][n] == pytest.approx(int(n) / (ms * 1e-3))
