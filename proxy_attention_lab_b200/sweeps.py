"""Latency sweeps in the shapes Proxy Attention Lab benchmarks, written in its ``results.json`` layout.

Mirrors what the reference's benchmark suite measures so that its analyzer can plot B200 numbers next to
its Metal ones: Hq=32 / Hkv=16, D=128, bf16, TPP=16 (``benchmarks/paged_attention/cpp/seq_len_vs_latency.cpp:47-55``);
decode latency against history length at batch 1 (``:210-223``), prefill latency against sequence length with no
history (``:292,382-388``), batch decode latency and throughput against the number of sequences
(``benchmarks/paged_attention/cpp/batch_latency_vs_num_sequences.cpp:258-268``).  The output nests
``benchmark -> sub-category -> group -> {parameter: value}`` as ``benchmarks/benchmarks.md:198-236`` describes;
throughput is ``num_sequences / latency`` (``benchmarks/analyzer/plotters/batch_decode_latency.py:151``).
``fill_kv_pages`` is swept as the reference's pytest-benchmark file does
(``benchmarks/fill_kv_pages/python/test_fill_kv_pages_python.py:13,73,136-137``): new tokens of one sequence, one token each
of many sequences (sequences sharing pages), and head_dim x kv heads at 32 tokens; 8 kv heads, D = 128, TPP = 16 otherwise.
The group name is ``cuda_pal_b200`` where the reference writes ``cpp_pal``.

    python -m proxy_attention_lab_b200.sweeps --out results.json [--quick]

Every point is timed with CUDA events over ``--iters`` calls after ``--warmup`` calls; the median of ``--reps``
repetitions is reported, as the reference does (10 iterations x 10 repetitions, median aggregate,
``seq_len_vs_latency.cpp:207-208``).
"""

from __future__ import annotations

import argparse
import json
import statistics
import sys

import torch

HQ, HKV, D, TPP = 32, 16, 128, 16
GROUP = "cuda_pal_b200"


def _time_ms(fn, warmup: int, iters: int, reps: int) -> float:
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    samples = []
    for _ in range(reps):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(iters):
            fn()
        e1.record()
        torch.cuda.synchronize()
        samples.append(e0.elapsed_time(e1) / iters)
    return statistics.median(samples)


def _pools(num_pages: int, device, gen):
    k = torch.randn((num_pages, HKV, D // 8, TPP, 8), device=device, dtype=torch.bfloat16, generator=gen)
    v = torch.randn((num_pages, HKV, D, TPP), device=device, dtype=torch.bfloat16, generator=gen)
    return k, v


def decode_point(pal, device, num_seqs: int, history: int, timing) -> float:
    """Latency of one decode step for `num_seqs` sequences of `history` tokens each (shuffled pages)."""
    gen = torch.Generator(device=device).manual_seed(history * 131 + num_seqs)
    pages_per_seq = (history + TPP - 1) // TPP
    k, v = _pools(num_seqs * pages_per_seq, device, gen)
    table = torch.randperm(num_seqs * pages_per_seq, device=device).reshape(num_seqs, pages_per_seq).to(torch.int32)
    lens = torch.full((num_seqs,), history, dtype=torch.int32, device=device)
    q = torch.randn((num_seqs, HQ, D), device=device, dtype=torch.bfloat16, generator=gen)
    return _time_ms(lambda: pal.paged_attention_decode(q, k, v, table, lens), *timing)


def prefill_point(pal, device, seq_len: int, timing) -> float:
    """Latency of a causal prefill of one sequence of `seq_len` new tokens with no history."""
    gen = torch.Generator(device=device).manual_seed(seq_len)
    k_pool, v_pool = _pools(1, device, gen)
    table = torch.zeros((1, 1), dtype=torch.int32, device=device)
    hist = torch.zeros((1,), dtype=torch.int32, device=device)
    q = torch.randn((seq_len, HQ, D), device=device, dtype=torch.bfloat16, generator=gen)
    k = torch.randn((seq_len, HKV, D), device=device, dtype=torch.bfloat16, generator=gen)
    v = torch.randn((seq_len, HKV, D), device=device, dtype=torch.bfloat16, generator=gen)
    return _time_ms(lambda: pal.paged_attention_prefill(q, k, v, k_pool, v_pool, table, hist), *timing)


def fill_point(pal, device, timing, *, tokens: int = 0, sequences: int = 0, hkv: int = 8, d: int = 128, dtype=torch.bfloat16) -> float:
    """Latency of one fill_kv_pages call: `tokens` consecutive tokens of one sequence, or one token each of `sequences`
    sequences whose pages are shared two to a page (the reference's two set-ups)."""
    gen = torch.Generator(device=device).manual_seed(tokens * 7 + sequences)
    n = tokens or sequences
    if tokens:
        pages = max(4, tokens // TPP + 2)
        table = torch.arange((tokens + TPP - 1) // TPP, dtype=torch.int32, device=device).reshape(1, -1)
        pos = torch.arange(tokens, dtype=torch.int32, device=device)
        seq = torch.zeros(tokens, dtype=torch.int32, device=device)
    else:
        pages = max(4, sequences // 2)
        table = (torch.arange(sequences, dtype=torch.int32, device=device) % pages).reshape(sequences, 1)
        pos = torch.arange(sequences, dtype=torch.int32, device=device) % TPP
        seq = torch.arange(sequences, dtype=torch.int32, device=device)
    keys = torch.randn((n, hkv, d), device=device, dtype=dtype, generator=gen)
    vals = torch.randn((n, hkv, d), device=device, dtype=dtype, generator=gen)
    k_pool = torch.zeros((pages, hkv, d // 8, TPP, 8), device=device, dtype=dtype)
    v_pool = torch.zeros((pages, hkv, d, TPP), device=device, dtype=dtype)
    return _time_ms(lambda: pal.fill_kv_pages(keys, vals, k_pool, v_pool, table, pos, seq), *timing)


def run(pal, device, quick: bool, timing) -> dict:
    decode_hist = [64, 256, 1024, 4096] if quick else [64 << i for i in range(14)]           # 64 .. 524288
    prefill_len = [64, 256, 1024] if quick else [64, 128, 256, 512, 1024, 2048, 4096]
    batch_sizes = [1, 4, 16] if quick else [1, 2, 4, 8, 16, 32, 64]
    batch_hist = [256, 4096] if quick else [64, 256, 1024, 4096]
    out = {"latency_vs_seq_len": {"prefill": {GROUP: {}}, "decode": {GROUP: {}}},
           "batch_decode_latency": {"latency_vs_num_sequences": {}, "throughput_vs_num_sequences": {}}}
    for n in prefill_len:
        out["latency_vs_seq_len"]["prefill"][GROUP][f"{float(n)}"] = prefill_point(pal, device, n, timing)
    for h in decode_hist:
        out["latency_vs_seq_len"]["decode"][GROUP][f"{float(h)}"] = decode_point(pal, device, 1, h, timing)
    for h in batch_hist:
        lat, thr = {}, {}
        for s in batch_sizes:
            ms = decode_point(pal, device, s, h, timing)
            lat[str(s)] = ms
            thr[str(s)] = s / (ms * 1e-3)
        out["batch_decode_latency"]["latency_vs_num_sequences"][f"H={h}"] = lat
        out["batch_decode_latency"]["throughput_vs_num_sequences"][f"H={h}"] = thr
    fill = {"latency_vs_num_new_tokens": {}, "latency_vs_num_sequences": {}, "latency_vs_dimensions": {GROUP: {}}}
    for name, dtype in (("float16", torch.float16), ("bfloat16", torch.bfloat16)):
        fill["latency_vs_num_new_tokens"][f"{GROUP}_{name}"] = {
            str(t): fill_point(pal, device, timing, tokens=t, dtype=dtype) for t in ([1, 16, 128] if quick else [1, 4, 8, 16, 32, 64, 128])}
        fill["latency_vs_num_sequences"][f"{GROUP}_{name}"] = {
            str(n): fill_point(pal, device, timing, sequences=n, dtype=dtype) for n in ([1, 8, 64] if quick else [1, 2, 4, 8, 16, 32, 64])}
    for d in ([128] if quick else [64, 128, 256]):
        for hkv in ([8] if quick else [1, 4, 8, 16]):
            fill["latency_vs_dimensions"][GROUP][f"D={d},Hkv={hkv}"] = fill_point(pal, device, timing, tokens=32, hkv=hkv, d=d, dtype=torch.float16)
    out["fill_kv_pages"] = fill
    return out


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("--out", default="results.json")
    ap.add_argument("--quick", action="store_true", help="a few points per sweep")
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--reps", type=int, default=10)
    ap.add_argument("--device", type=int, default=0)
    args = ap.parse_args(argv)
    if not torch.cuda.is_available():
        print("sweeps need a CUDA device; there is no CPU path", file=sys.stderr)
        return 2
    import proxy_attention_lab_b200 as pal

    device = torch.device("cuda", args.device)
    torch.cuda.set_device(device)
    results = run(pal, device, args.quick, (args.warmup, args.iters, args.reps))
    with open(args.out, "w") as f:
        json.dump(results, f, indent=2)
    print(json.dumps(results["latency_vs_seq_len"]["decode"][GROUP]))
    return 0


if __name__ == "__main__":
    sys.exit(main())
