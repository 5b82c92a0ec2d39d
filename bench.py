#!/usr/bin/env python
"""Benchmark of the paged-attention hot path on B200.

``python bench.py --gpus N --steps K --warmup W`` prints ONE JSON line (rank 0).  A step is one pass
of the operator over one batch of synthetic input already resident in HBM.  The headline workload is
the Llama-3-8B-shaped decode batch the metric (paged decode KV GB/s) is quoted on; the same line carries,
under ``workloads``, one record each for the other parts of the metric - chunked prefill (TFLOP/s), the
Llama-3-70B long-context two-pass decode, fill_kv_pages - and, under torchrun, the multi-GPU forms of the long
decode (kv-head sharded; context sharded with the NCCL all-gather + combine; context sharded with the fused
peer-store exchange).  ``--workload NAME`` makes another workload the headline; ``--workloads none`` leaves the
extra records out (profiler captures use that).

Every figure is the median over ``--blocks`` (default 20) timed blocks of K steps each (barrier + synchronize around every
block, CUDA events on the launching stream, max over ranks); the fastest block is reported beside it.

``--impl reference`` times the reference side of the comparison instead.  Proxy Attention Lab has no
CPU implementation and its Metal kernels cannot run here, so that arm is the CPU oracle (the
restatement of the reference test-suite's gather-pages + SDPA comparator) on all host threads.
"""

from __future__ import annotations

import argparse
import json
import math
import os
import sys
import threading
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

WORKLOADS = {
    # name: (kind, params)
    "decode_8b": dict(kind="decode", S=64, lo=1024, hi=8192, hq=32, hkv=8, d=128, tpp=16, partition_pages=0,
                      desc="Llama-3-8B decode: batch 64, context U[1024,8192], 32q/8kv heads, D=128, bf16, TPP=16, fused single pass"),
    "decode_8b_append": dict(kind="decode", S=64, lo=1024, hi=8192, hq=32, hkv=8, d=128, tpp=16, partition_pages=0, append="fused",
                             desc="Llama-3-8B decode step with the newest token appended in the same launch (paged_attention_decode_append): "
                                  "batch 64, context U[1024,8192], 32q/8kv heads, D=128, bf16, TPP=16"),
    "decode_8b_append_pair": dict(kind="decode", S=64, lo=1024, hi=8192, hq=32, hkv=8, d=128, tpp=16, partition_pages=0, append="pair",
                                  desc="the same decode step as two calls, fill_kv_pages then paged_attention_decode: "
                                       "batch 64, context U[1024,8192], 32q/8kv heads, D=128, bf16, TPP=16"),
    "decode_small_append": dict(kind="decode", S=4, lo=64, hi=512, hq=8, hkv=2, d=128, tpp=16, partition_pages=0, append="fused",
                                desc="latency case, newest token appended in the same launch: batch 4, context U[64,512], 8q/2kv heads, D=128, bf16, TPP=16"),
    "decode_small_append_pair": dict(kind="decode", S=4, lo=64, hi=512, hq=8, hkv=2, d=128, tpp=16, partition_pages=0, append="pair",
                                     desc="latency case as two calls, fill_kv_pages then paged_attention_decode: batch 4, context U[64,512], 8q/2kv heads, D=128, bf16, TPP=16"),
    "decode_70b_small": dict(kind="decode", S=2, lo=131072, hi=131072, hq=64, hkv=8, d=128, tpp=16, partition_pages=256,
                             desc="reduced long decode for profiler captures: batch 2, context 131072, 64q/8kv heads, D=128, bf16, TPP=16, "
                                  "two-pass 256-page partitions"),
    "decode_70b": dict(kind="decode", S=8, lo=131072, hi=131072, hq=64, hkv=8, d=128, tpp=16, partition_pages=256,
                       desc="Llama-3-70B long decode: batch 8, context 131072, 64q/8kv heads, D=128, bf16, TPP=16, two-pass 256-page partitions"),
    "decode_70b_auto": dict(kind="decode", S=8, lo=131072, hi=131072, hq=64, hkv=8, d=128, tpp=16, partition_pages=-1,
                            desc="Llama-3-70B long decode: batch 8, context 131072, 64q/8kv heads, D=128, bf16, TPP=16, two-pass with the partition size "
                                 "chosen by the launcher from the work items per SM"),
    "decode_70b_ctx": dict(kind="decode", S=8, lo=131072, hi=131072, hq=64, hkv=8, d=128, tpp=16, partition_pages=256, ctx="nccl",
                           desc="Llama-3-70B long decode, context sharded: batch 8, context 131072 cut into N contiguous slices (one per GPU), "
                                "64q/8kv heads, D=128, bf16, TPP=16, 256-page partitions, per-GPU (m,l,acc) all-gathered over NCCL and merged"),
    "decode_70b_ctx_fused": dict(kind="decode", S=8, lo=131072, hi=131072, hq=64, hkv=8, d=128, tpp=16, partition_pages=256, ctx="fused",
                                 desc="Llama-3-70B long decode, context sharded: batch 8, context 131072 cut into N contiguous slices (one per GPU), "
                                      "64q/8kv heads, D=128, bf16, TPP=16, 256-page partitions, per-GPU (m,l,acc) exchanged by peer stores inside the combine kernel"),
    "decode_70b_ctx_fused_auto": dict(kind="decode", S=8, lo=131072, hi=131072, hq=64, hkv=8, d=128, tpp=16, partition_pages=-1, ctx="fused",
                                      desc="Llama-3-70B long decode, context sharded: batch 8, context 131072 cut into N contiguous slices (one per GPU), "
                                           "64q/8kv heads, D=128, bf16, TPP=16, partition size chosen by the launcher, per-GPU (m,l,acc) exchanged by peer stores "
                                           "inside the combine kernel"),
    "prefill_8b": dict(kind="prefill", S=8, n=2048, hlo=0, hhi=4096, hq=32, hkv=8, d=128, tpp=16,
                       desc="Llama-3-8B chunked causal prefill: 8 x 2048 new tokens, history U[0,4096], 32q/8kv heads, D=128, bf16, TPP=16"),
    "prefill_small": dict(kind="prefill", S=2, n=1024, hlo=0, hhi=2048, hq=32, hkv=8, d=128, tpp=16,
                          desc="reduced chunked prefill for profiler captures: 2 x 1024 new tokens, history U[0,2048], 32q/8kv heads, D=128, bf16, TPP=16"),
    "prefill_wave": dict(kind="prefill", S=4, n=2048, hlo=2048, hhi=2048, hq=32, hkv=8, d=128, tpp=16,
                         desc="one full wave of prefill CTAs for profiler captures: 4 x 2048 new tokens, history 2048, 32q/8kv heads, D=128, bf16, TPP=16"),
    "prefill_d256": dict(kind="prefill", S=8, n=2048, hlo=0, hhi=4096, hq=32, hkv=8, d=256, tpp=16,
                         desc="chunked causal prefill at head_dim 256 (the two-CTA tcgen05 kernel): 8 x 2048 new tokens, history U[0,4096], "
                              "32q/8kv heads, D=256, bf16, TPP=16"),
    "prefill_d256_wave": dict(kind="prefill", S=2, n=2048, hlo=2048, hhi=2048, hq=32, hkv=8, d=256, tpp=16,
                              desc="full waves of two-CTA prefill clusters for profiler captures: 2 x 2048 new tokens, history 2048, 32q/8kv heads, "
                                   "D=256, bf16, TPP=16"),
    "prefill_ragged": dict(kind="prefill", S=8, n=2048, nlo=128, hlo=0, hhi=4096, hq=32, hkv=8, d=128, tpp=16,
                           desc="ragged chunked causal prefill (paged_attention_prefill_ragged): 8 sequences with U[128,2048] new tokens each, "
                                "history U[0,4096], 32q/8kv heads, D=128, bf16, TPP=16"),
    "fill": dict(kind="fill", S=64, n=512, hkv=8, d=128, tpp=16, pages=65536,
                 desc="fill_kv_pages: 64 x 512 tokens, 8 kv heads, D=128, bf16, TPP=16, 65536-page pool, random free slots"),
    "fill_append_small": dict(kind="fill", S=48, n=1024, hkv=8, d=128, tpp=16, pages=16384, append=True, hhi=4096,
                              desc="reduced prefill append for profiler captures: 48 sequences x 1024 consecutive positions after a history U[0,4096], "
                                   "8 kv heads, D=128, bf16, TPP=16, 16384-page pool"),
    "fill_append": dict(kind="fill", S=64, n=512, hkv=8, d=128, tpp=16, pages=65536, append=True, hhi=4096,
                        desc="fill_kv_pages: prefill append, 64 sequences x 512 consecutive positions after a history U[0,4096], random pages, "
                             "8 kv heads, D=128, bf16, TPP=16, 65536-page pool"),
}


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            p = json.load(f)
        return dict(hbm=float(p["hbm_gbs"]), tensor=float(p["bf16_tflops"]), tensor_sustained=float(p.get("bf16_tflops_sustained", p["bf16_tflops"])), source="measured")
    except Exception:
        return dict(hbm=6650.0, tensor=1590.0, tensor_sustained=1400.0, source="fallback")


class ClockSampler:
    """Samples SM clock and throttle reasons through NVML (read-only) while a region runs."""

    def __init__(self, index: int, period_s: float = 0.002):
        self.index, self.period = index, period_s
        self.samples, self.reasons = [], set()
        self.max_mhz = None
        self._stop = threading.Event()
        self._thread = None
        try:
            import pynvml

            pynvml.nvmlInit()
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
        except Exception:
            self.nv = None

    def _reason_names(self, mask):
        nv = self.nv
        table = [("hw_slowdown", "nvmlClocksThrottleReasonHwSlowdown"), ("hw_thermal_slowdown", "nvmlClocksThrottleReasonHwThermalSlowdown"),
                 ("sw_thermal_slowdown", "nvmlClocksThrottleReasonSwThermalSlowdown"), ("sw_power_cap", "nvmlClocksThrottleReasonSwPowerCap"),
                 ("hw_power_brake", "nvmlClocksThrottleReasonHwPowerBrakeSlowdown")]
        out = []
        for name, attr in table:
            bit = getattr(nv, attr, None)
            if bit is not None and mask & bit:
                out.append(name)
        return out

    def _once(self):
        try:
            self.samples.append(self.nv.nvmlDeviceGetClockInfo(self.h, self.nv.NVML_CLOCK_SM))
            self.reasons.update(self._reason_names(self.nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h)))
        except Exception:
            pass

    def _run(self):
        while not self._stop.is_set():
            self._once()
            self._stop.wait(self.period)

    def __enter__(self):
        if self.nv is not None:
            self._thread = threading.Thread(target=self._run, daemon=True)
            self._thread.start()
        return self

    def __exit__(self, *a):
        if self._thread is not None:
            self._once()
            self._stop.set()
            self._thread.join()

    def summary(self):
        if not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": self.max_mhz, "reasons": ["unavailable"]}
        s = sorted(self.samples)
        return {"sm_mhz": s[len(s) // 2], "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons), "samples": len(s)}


# ------------------------------------------------------------------------------------------------
# synthetic workloads
# ------------------------------------------------------------------------------------------------
def make_lengths(seed, count, lo, hi):
    g = torch.Generator().manual_seed(seed)
    return torch.randint(lo, hi + 1, (count,), generator=g)


def build_decode(cfg, device, seed, hkv_local=None):
    """Device-resident decode batch: shuffled page pool sized to the total tokens."""
    tpp, d, hq = cfg["tpp"], cfg["d"], cfg["hq"]
    hkv = hkv_local or cfg["hkv"]
    hq_local = hq * hkv // cfg["hkv"]
    # The same context lengths on every rank (weak scaling = the same work per GPU as N grows); pages and data differ.
    lens = make_lengths(0, cfg["S"], cfg["lo"], cfg["hi"])
    npg = (lens + tpp - 1) // tpp
    P, MP = int(npg.sum()), int(npg.max())
    g = torch.Generator().manual_seed(seed + 1)
    perm = torch.randperm(P, generator=g)
    table = torch.zeros((cfg["S"], MP), dtype=torch.int32)
    off = 0
    for s in range(cfg["S"]):
        n = int(npg[s])
        table[s, :n] = perm[off:off + n].to(torch.int32)
        off += n
    gen = torch.Generator(device=device).manual_seed(seed + 2)
    k_pool = torch.randn((P, hkv, d // 8, tpp, 8), device=device, dtype=torch.bfloat16, generator=gen)
    v_pool = torch.randn((P, hkv, d, tpp), device=device, dtype=torch.bfloat16, generator=gen)
    q_host = torch.randn((cfg["S"], hq_local, d), generator=g).to(torch.bfloat16).pin_memory()
    table_host = table.pin_memory()
    lens_host = lens.to(torch.int32).pin_memory()
    total_tokens = int(lens.sum())
    kv_bytes = total_tokens * hkv * d * 2 * 2
    alg_bytes = kv_bytes + 2 * cfg["S"] * hq_local * d * 2 + 4 * int(npg.sum()) + 4 * cfg["S"]
    pp = cfg["partition_pages"]
    if pp < 0:  # the launcher's own choice, asked from the library
        from proxy_attention_lab_b200 import _lib

        pp = _lib.lib.pal_decode_auto_partition_pages(cfg["S"], hq_local, hkv, d, tpp, MP)
    if pp:
        parts = (MP + pp - 1) // pp
        alg_bytes += 2 * cfg["S"] * hq_local * parts * (d + 2) * 4
    return dict(k_pool=k_pool, v_pool=v_pool, q_host=q_host, table_host=table_host, lens_host=lens_host,
                q=q_host.to(device), table=table_host.to(device), lens=lens_host.to(device), kv_bytes=kv_bytes,
                alg_bytes=alg_bytes, tokens=cfg["S"], hq=hq_local, hkv=hkv, lens_cpu=lens, partition_pages=pp)


def build_prefill(cfg, device, seed, seqs=None, hkv_local=None):
    tpp, d, n = cfg["tpp"], cfg["d"], cfg["n"]
    hkv = hkv_local or cfg["hkv"]            # kv-head sharded: this GPU's kv heads and their query heads, every sequence
    hq = cfg["hq"] * hkv // cfg["hkv"]
    hist_all = make_lengths(seed, cfg["S"], cfg["hlo"], cfg["hhi"])
    idx = list(range(cfg["S"])) if seqs is None else seqs
    hist = hist_all[idx]
    S = len(idx)
    npg = (hist + tpp - 1) // tpp
    P, MP = max(int(npg.sum()), 1), max(int(npg.max()), 1)
    g = torch.Generator().manual_seed(seed + 1)
    perm = torch.randperm(P, generator=g)
    table = torch.zeros((S, MP), dtype=torch.int32)
    off = 0
    for s in range(S):
        m = int(npg[s])
        table[s, :m] = perm[off:off + m].to(torch.int32)
        off += m
    gen = torch.Generator(device=device).manual_seed(seed + 2)
    mk = lambda *shape: torch.randn(shape, device=device, dtype=torch.bfloat16, generator=gen)
    # ragged workloads draw every sequence's number of new tokens from U[nlo, n]
    counts = make_lengths(seed + 5, cfg["S"], cfg["nlo"], n)[idx] if "nlo" in cfg else torch.full((S,), n, dtype=torch.int64)
    T = int(counts.sum())
    data = dict(k_pool=mk(P, hkv, d // 8, tpp, 8), v_pool=mk(P, hkv, d, tpp), q=mk(T, hq, d), k=mk(T, hkv, d), v=mk(T, hkv, d),
                table=table.to(device), hist=hist.to(torch.int32).to(device))
    if "nlo" in cfg:
        data["cu"] = torch.cat([torch.zeros(1, dtype=torch.int64), counts.cumsum(0)]).to(torch.int32).to(device)
        data["max_new"] = int(counts.max())
    data["flops"] = 4 * hq * d * sum(int(c) * int(h) + int(c) * (int(c) + 1) // 2 for c, h in zip(counts, hist))
    data["tokens"] = T
    data["hist_cpu"] = hist
    data["hq"] = hq
    return data


def build_fill(cfg, device, seed):
    tpp, d, hkv = cfg["tpp"], cfg["d"], cfg["hkv"]
    T, P = cfg["S"] * cfg["n"], cfg["pages"]
    gen = torch.Generator(device=device).manual_seed(seed)
    keys = torch.randn((T, hkv, d), device=device, dtype=torch.bfloat16, generator=gen)
    vals = torch.randn((T, hkv, d), device=device, dtype=torch.bfloat16, generator=gen)
    g = torch.Generator().manual_seed(seed + 1)
    if cfg.get("append"):
        # every sequence appends n consecutive positions after its history; its blocks sit on random distinct pages
        hist = torch.randint(0, cfg["hhi"], (cfg["S"],), generator=g)
        pos = hist[:, None] + torch.arange(cfg["n"])[None, :]
        blocks_per_seq = (cfg["hhi"] + cfg["n"]) // tpp + 1
        pages = torch.randperm(P, generator=g)[: cfg["S"] * blocks_per_seq].reshape(cfg["S"], blocks_per_seq)
        slots = (torch.gather(pages, 1, pos // tpp) * tpp + pos % tpp).reshape(-1)
    else:
        slots = torch.randperm(P * tpp, generator=g)[:T]
    k_pool = torch.zeros((P, hkv, d // 8, tpp, 8), device=device, dtype=torch.bfloat16)
    v_pool = torch.zeros((P, hkv, d, tpp), device=device, dtype=torch.bfloat16)
    return dict(keys=keys, vals=vals, slots=slots.to(device), k_pool=k_pool, v_pool=v_pool, alg_bytes=4 * T * hkv * d * 2 + 8 * T, tokens=T,
                keys_host=keys.cpu().pin_memory(), vals_host=vals.cpu().pin_memory(), slots_host=slots.pin_memory())


# ------------------------------------------------------------------------------------------------
# CPU side (oracle) - the reference arm and the cpu_baseline leg
# ------------------------------------------------------------------------------------------------
def cpu_decode_sample(cfg, budget_s, seed=0, data=None):
    """Times the oracle on the first sequences of the workload until `budget_s` is spent. Returns (bytes, seconds, n_seqs).
    With `data` (the GPU arm's batch) the sequences' own pages and queries are copied to the host; otherwise data of the
    same shapes is drawn from a seeded generator."""
    from oracle import decode_oracle

    tpp, d, hq, hkv = cfg["tpp"], cfg["d"], cfg["hq"], cfg["hkv"]
    lens = make_lengths(seed, cfg["S"], cfg["lo"], cfg["hi"])
    g = torch.Generator().manual_seed(seed + 7)
    done_bytes, spent, nseq = 0, 0.0, 0
    for s in range(cfg["S"]):
        L = int(lens[s])
        if L * hkv * d * 4 > 8e9:  # keep one sequence's fp32 copy within host memory
            L = int(8e9 // (hkv * d * 4))
        npg = (L + tpp - 1) // tpp
        if data is not None:
            pages = data["table"][s, :npg].long()
            k_pool, v_pool = data["k_pool"][pages].cpu(), data["v_pool"][pages].cpu()
            q = data["q"][s:s + 1].cpu()
            table = torch.arange(npg, dtype=torch.int32).reshape(1, npg)
        else:
            k_pool = torch.randn((npg, hkv, d // 8, tpp, 8), generator=g).to(torch.bfloat16)
            v_pool = torch.randn((npg, hkv, d, tpp), generator=g).to(torch.bfloat16)
            q = torch.randn((1, hq, d), generator=g).to(torch.bfloat16)
            table = torch.randperm(npg, generator=g).reshape(1, npg).to(torch.int32)
        t0 = time.perf_counter()
        decode_oracle(q, k_pool, v_pool, table, torch.tensor([L], dtype=torch.int32))
        spent += time.perf_counter() - t0
        done_bytes += L * hkv * d * 2 * 2
        nseq += 1
        if spent >= budget_s:
            break
    return done_bytes, spent, nseq


def cpu_prefill_sample(cfg, budget_s, seed=0, data=None):
    from oracle import prefill_oracle

    tpp, d, hq, hkv = cfg["tpp"], cfg["d"], cfg["hq"], cfg["hkv"]
    n = min(cfg["n"], 512)  # a 512-token slice of one sequence keeps the score matrix small
    hist = int(make_lengths(seed, cfg["S"], cfg["hlo"], cfg["hhi"])[0])
    g = torch.Generator().manual_seed(seed + 7)
    npg = max((hist + tpp - 1) // tpp, 1)
    if data is not None and "cu" not in data:
        # the first sequence of the GPU arm's batch: its history pages and the first n of its new tokens
        pages = data["table"][0, :npg].long()
        k_pool, v_pool = data["k_pool"][pages].cpu(), data["v_pool"][pages].cpu()
        q, k, v = data["q"][:n].cpu(), data["k"][:n].cpu(), data["v"][:n].cpu()
        table = torch.arange(npg, dtype=torch.int32).reshape(1, npg)
    else:
        k_pool = torch.randn((npg, hkv, d // 8, tpp, 8), generator=g).to(torch.bfloat16)
        v_pool = torch.randn((npg, hkv, d, tpp), generator=g).to(torch.bfloat16)
        q = torch.randn((n, hq, d), generator=g).to(torch.bfloat16)
        k = torch.randn((n, hkv, d), generator=g).to(torch.bfloat16)
        v = torch.randn((n, hkv, d), generator=g).to(torch.bfloat16)
        table = torch.randperm(npg, generator=g).reshape(1, npg).to(torch.int32)
    flops, spent, reps = 0, 0.0, 0
    while spent < budget_s:
        t0 = time.perf_counter()
        prefill_oracle(q, k, v, k_pool, v_pool, table, torch.tensor([hist], dtype=torch.int32))
        spent += time.perf_counter() - t0
        flops += 4 * hq * d * (n * hist + n * (n + 1) // 2)
        reps += 1
    return flops, spent, f"{reps} x (1 sequence, {n} new tokens, history {hist})"


def cpu_fill_sample(cfg, budget_s, seed=0):
    from oracle import fill_kv_pages_oracle

    tpp, d, hkv = cfg["tpp"], cfg["d"], cfg["hkv"]
    T, P = 4096, 4096
    g = torch.Generator().manual_seed(seed)
    keys = torch.randn((T, hkv, d), generator=g).to(torch.bfloat16)
    vals = torch.randn((T, hkv, d), generator=g).to(torch.bfloat16)
    slots = torch.randperm(P * tpp, generator=g)[:T]
    k_pool = torch.zeros((P, hkv, d // 8, tpp, 8), dtype=torch.bfloat16)
    v_pool = torch.zeros((P, hkv, d, tpp), dtype=torch.bfloat16)
    nbytes, spent, reps = 0, 0.0, 0
    while spent < budget_s:
        t0 = time.perf_counter()
        fill_kv_pages_oracle(keys, vals, k_pool, v_pool, slots)
        spent += time.perf_counter() - t0
        nbytes += 4 * T * hkv * d * 2 + 8 * T
        reps += 1
    return nbytes, spent, f"{reps} x ({T} tokens into a {P}-page pool, pool clone included as in the reference)"


class HostPipeline:
    """End-to-end stepping as a serving loop does it: the inputs of a step come from pinned host memory and its result goes
    back to the host, on copy streams of their own and with two sets of device buffers, so that the copies of one step
    overlap the kernels of its neighbours.  Every step still copies all of its inputs in and its whole result out."""

    def __init__(self, host, call, out_host, device):
        self.host, self.call, self.out_host = host, call, out_host
        self.bufs = [{k: torch.empty(v.shape, dtype=v.dtype, device=device) for k, v in host.items()} for _ in range(2)]
        self.s_in, self.s_out = torch.cuda.Stream(device), torch.cuda.Stream(device)
        self.ready = [torch.cuda.Event() for _ in range(2)]  # the inputs of slot b are on the device
        self.free = [torch.cuda.Event() for _ in range(2)]   # the kernels that read slot b have finished
        self.copied = [torch.cuda.Event() for _ in range(2)]  # the result of slot b has reached the host
        self.keep = [None, None]
        self.i = 0
        for e in self.free:
            e.record()

    def step(self):
        b = self.i & 1
        self.i += 1
        cur = torch.cuda.current_stream()
        with torch.cuda.stream(self.s_in):
            self.s_in.wait_event(self.free[b])
            for k, v in self.host.items():
                self.bufs[b][k].copy_(v, non_blocking=True)
            self.ready[b].record(self.s_in)
        cur.wait_event(self.ready[b])
        out = self.call(self.bufs[b])
        self.free[b].record(cur)
        if self.out_host is not None:
            # the result tensor is kept alive until its copy has finished (two steps later it surely has), so the
            # caching allocator never has to track it across streams
            if self.keep[b] is not None:
                self.copied[b].synchronize()
            with torch.cuda.stream(self.s_out):
                self.s_out.wait_event(self.free[b])
                self.out_host.copy_(out, non_blocking=True)
                self.copied[b].record(self.s_out)
            self.keep[b] = out

    def drain(self):
        cur = torch.cuda.current_stream()
        cur.wait_stream(self.s_in)
        cur.wait_stream(self.s_out)


def metric_of(kind):
    return {"decode": ("paged decode KV GB/s", "GB/s"), "prefill": ("prefill TFLOPS", "TFLOP/s"), "fill": ("fill_kv_pages payload GB/s", "GB/s")}[kind]


def cpu_measure(cfg, budget_s, data=None):
    """The oracle on a bounded sample of the workload.  `data` = the GPU arm's tensors (the sample is then cut from the very
    inputs the kernels ran on); without it the sample is seeded N(0,1) data of the same shapes."""
    kind = cfg["kind"]
    src = "the GPU arm's own tensors" if data is not None else "seeded N(0,1) data of the same shapes (not the GPU arm's tensors)"
    if kind == "decode":
        nbytes, spent, nseq = cpu_decode_sample(cfg, budget_s, data=data)
        return nbytes / spent / 1e9, f"first {nseq} sequences of the batch ({nbytes / 1e9:.3f} GB of KV), {src}"
    if kind == "prefill":
        flops, spent, what = cpu_prefill_sample(cfg, budget_s, data=data)
        return flops / spent / 1e12, f"{what}, {src}"
    nbytes, spent, what = cpu_fill_sample(cfg, budget_s)
    return nbytes / spent / 1e9, f"{what}, seeded N(0,1) data of the same shapes"


def run_reference(args, cfg, rank):
    """The reference arm: the CPU oracle on all host threads, rank 0 only."""
    if rank != 0:
        return
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    metric, unit = metric_of(cfg["kind"])
    per_step_budget = max(0.2, min(3.0, 150.0 / max(args.steps + args.warmup, 1)))
    for _ in range(args.warmup):
        cpu_measure(cfg, per_step_budget / 4)
    vals, what, t0 = [], "", time.perf_counter()
    for _ in range(args.steps):
        v, what = cpu_measure(cfg, per_step_budget)
        vals.append(v)
    wall = time.perf_counter() - t0
    value = sum(vals) / len(vals)
    line = {"impl": "reference", "metric": metric, "value": value, "unit": unit, "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": wall / args.steps * 1e3, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16 storage, f32 arithmetic",
            "data": "synthetic", "config": {"workload": cfg["desc"]}, "blocks": 1,
            "cpu_baseline": {"value": value, "unit": unit, "cores": torch.get_num_threads(), "kind": "port", "sample": f"each step: {what}"},
            "e2e": {"value": value, "unit": unit, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}, "gpu_launches": 0}
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------------------------------------------
# GPU side
# ------------------------------------------------------------------------------------------------
class Env:
    """Rank / device / process group of this run, and the barrier every timed block is bracketed with."""

    def __init__(self):
        self.rank = int(os.environ.get("RANK", "0"))
        self.world = int(os.environ.get("WORLD_SIZE", "1"))
        self.local_rank = int(os.environ.get("LOCAL_RANK", "0"))
        self.device = torch.device("cuda", self.local_rank)
        self.dist = None

    def init(self):
        torch.cuda.set_device(self.device)
        if self.world > 1:
            import torch.distributed as dist

            dist.init_process_group("nccl", device_id=self.device)
            self.dist = dist

    def barrier(self):
        if self.dist is not None:
            self.dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(self, x: float) -> float:
        if self.dist is None:
            return x
        t = torch.tensor([x], device=self.device, dtype=torch.float64)
        self.dist.all_reduce(t, op=self.dist.ReduceOp.MAX)
        return float(t.item())

    def sum_over_ranks(self, x: float) -> float:
        if self.dist is None:
            return x
        t = torch.tensor([x], device=self.device, dtype=torch.float64)
        self.dist.all_reduce(t, op=self.dist.ReduceOp.SUM)
        return float(t.item())


class Prepared:
    """One workload made ready on this rank: the step to time, its end-to-end pipeline and what a step amounts to."""

    def __init__(self, **kw):
        self.extra_cfg, self.pipe, self.scaling, self.notes = {}, None, "weak", []
        self.units_are_global = False  # True: every rank reports the whole job's units (strong scaling of one problem)
        self.__dict__.update(kw)


def prepare(name, env, pal, peaks, args, force_single=False):
    """Build the synthetic inputs of workload `name` on this rank.  `force_single` builds the one-GPU form of the problem on
    every rank (the N = 1 baseline a strong-scaling record is compared with)."""
    cfg = WORKLOADS[name]
    kind, device, rank = cfg["kind"], env.device, env.rank
    world = 1 if force_single else env.world
    metric, unit = metric_of(kind)
    w = Prepared(name=name, cfg=cfg, kind=kind, metric=metric, unit=unit)
    if kind == "decode":
        hkv_local = None
        ctx = cfg.get("ctx")  # None | "nccl" | "fused"
        base = cfg
        if ctx:
            w.scaling, w.units_are_global = "strong", False
            how = ("partials + one NCCL all-gather of the packed (acc, m, l) buffer + LSE combine" if ctx == "nccl"
                   else "split-KV pass + one kernel that stores the merged (acc, m, l) into every peer's buffer over NVLink, waits on flags and combines")
            w.extra_cfg["parallelism"] = f"context sharded x{world}: {how}"
            cfg = dict(cfg, lo=cfg["lo"] // world, hi=cfg["hi"] // world)  # this rank's slice of every sequence
        if name.startswith("decode_70b") and not ctx and world > 1:
            # total work fixed: each GPU owns Hkv/N kv heads (and their query heads) of every sequence
            hkv_local, w.scaling = cfg["hkv"] // world, "strong"
            w.extra_cfg["parallelism"] = f"kv-head sharded x{world}, no collective"
        elif world > 1 and not ctx:
            w.extra_cfg["parallelism"] = f"sequence sharded x{world} (each GPU its own batch of {cfg['S']}), no collective"
        data = build_decode(cfg, device, seed=rank if (hkv_local is None and not ctx) else 0, hkv_local=hkv_local)
        pp = cfg["partition_pages"] if cfg["partition_pages"] > 0 or not ctx else None  # ctx forms: None = the library's choice
        if ctx and env.dist is not None and world > 1:
            env.dist.broadcast(data["q"], src=0)  # every rank must hold the same queries
        append = cfg.get("append")
        if append:
            gen = torch.Generator(device=device).manual_seed(1234 + rank)
            new_k = torch.randn((cfg["S"], data["k_pool"].shape[1], cfg["d"]), device=device, dtype=torch.bfloat16, generator=gen)
            new_v = torch.randn_like(new_k)
            new_k_host, new_v_host = new_k.cpu().pin_memory(), new_v.cpu().pin_memory()
            last_pos = (data["lens"] - 1).to(torch.int32)
            seq_ids = torch.arange(cfg["S"], device=device, dtype=torch.int32)
        xchg = gathered = None
        rows = cfg["S"] * data["hq"]
        if ctx == "fused":
            from proxy_attention_lab_b200.sharding import ContextExchange

            if env.dist is None:
                import torch.distributed as dist

                # a single process still needs a (one-rank) group for the symmetric-memory rendezvous
                os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
                os.environ.setdefault("MASTER_PORT", "29533")
                dist.init_process_group("nccl", rank=0, world_size=1, device_id=device)
                env.own_group = dist
            xchg = ContextExchange(rows=rows, head_dim=cfg["d"], device=device)
        elif ctx == "nccl" and world > 1:
            from proxy_attention_lab_b200.sharding import all_gather_packed

            gathered = torch.empty((world, rows, cfg["d"] + 2), dtype=torch.float32, device=device)
            packed = torch.empty((rows, cfg["d"] + 2), dtype=torch.float32, device=device)

        def decode_call(q, table, lens, nk=None, nv=None):
            nk, nv = (new_k, new_v) if nk is None and append else (nk, nv)
            if append == "fused":
                return pal.paged_attention_decode_append(nk, nv, q, data["k_pool"], data["v_pool"], table, lens, partition_pages=pp)
            if append == "pair":
                pal.fill_kv_pages(nk, nv, data["k_pool"], data["v_pool"], table, last_pos, seq_ids)
            if not ctx:
                return pal.paged_attention_decode(q, data["k_pool"], data["v_pool"], table, lens, partition_pages=pp)
            if ctx == "fused":
                return xchg.decode(q, data["k_pool"], data["v_pool"], table, lens, partition_pages=pp)
            if world == 1:
                part = pal.paged_attention_decode_partials(q, data["k_pool"], data["v_pool"], table, lens, partition_pages=pp, packed=True)
                return pal.lse_combine_packed(part[None], out_dtype=torch.bfloat16, out_shape=(cfg["S"], data["hq"], cfg["d"]))
            pal.paged_attention_decode_partials(q, data["k_pool"], data["v_pool"], table, lens, partition_pages=pp, packed=True, out=packed)
            all_gather_packed(packed, out=gathered)
            return pal.lse_combine_packed(gathered, out_dtype=torch.bfloat16, out_shape=(cfg["S"], data["hq"], cfg["d"]))

        w.step = lambda: decode_call(data["q"], data["table"], data["lens"])
        out_host = torch.empty((cfg["S"], data["hq"], cfg["d"]), dtype=torch.bfloat16).pin_memory()
        e2e_inputs = {"q": data["q_host"], "table": data["table_host"], "lens": data["lens_host"]}
        if append:
            e2e_inputs.update(new_k=new_k_host, new_v=new_v_host)
        w.pipe = HostPipeline(e2e_inputs, lambda d: decode_call(d["q"], d["table"], d["lens"], d.get("new_k"), d.get("new_v")), out_host, device)
        w.h2d = data["q_host"].numel() * 2 + data["table_host"].numel() * 4 + data["lens_host"].numel() * 4 + (2 * new_k_host.numel() * 2 if append else 0)
        w.d2h = out_host.numel() * 2
        w.units_per_step, w.alg_per_step = data["kv_bytes"], data["alg_bytes"]
        w.scale = 1e9
        w.launches_per_step = (2 if data["partition_pages"] else 1) + (1 if append == "pair" else 0)
        if cfg["partition_pages"] < 0:
            w.extra_cfg["partition_pages_chosen"] = data["partition_pages"]
        w.collectives_per_step = 1 if (ctx == "nccl" and world > 1) else 0
        w.bound, w.peak, w.roof_unit = "hbm", peaks["hbm"], "GB/s"
        w.l2_note = "KV pool per GPU is larger than L2 (126 MB); every step streams it from HBM"
        w.tokens = cfg["S"]
        w.tokens_are_global = w.scaling == "strong"
        w.data = data
        w.graph = bool(ctx) and not args.no_cuda_graph
    elif kind == "prefill":
        seqs, hkv_local = None, None
        if world > 1 and cfg["hkv"] % world == 0:
            # every GPU does the same work (its share of the heads of every sequence), so no GPU waits for the one that
            # drew the long sequences
            hkv_local = cfg["hkv"] // world
            w.scaling = "strong"
            w.extra_cfg["parallelism"] = f"kv-head sharded x{world}, no collective"
        elif world > 1:
            from proxy_attention_lab_b200.sharding import partition_sequences

            hist_all = make_lengths(0, cfg["S"], cfg["hlo"], cfg["hhi"])
            n_all = make_lengths(5, cfg["S"], cfg["nlo"], cfg["n"]).tolist() if "nlo" in cfg else [cfg["n"]] * cfg["S"]
            work = [n * int(h) + n * (n + 1) // 2 for n, h in zip(n_all, hist_all)]
            seqs = partition_sequences(work, world)[rank] or [rank % cfg["S"]]
            w.scaling = "strong"
            w.extra_cfg["parallelism"] = f"sequence sharded x{world} (balanced by attention work), no collective"
        data = build_prefill(cfg, device, seed=0, seqs=seqs, hkv_local=hkv_local)

        def prefill_call(q, k, v, table, hist, cu=None):
            if cu is None:
                return pal.paged_attention_prefill(q, k, v, data["k_pool"], data["v_pool"], table, hist, impl=args.prefill_impl)
            return pal.paged_attention_prefill_ragged(q, k, v, data["k_pool"], data["v_pool"], table, hist, cu,
                                                      max_new_tokens=data["max_new"], impl=args.prefill_impl)

        w.step = lambda: prefill_call(data["q"], data["k"], data["v"], data["table"], data["hist"], data.get("cu"))
        host = {k: data[k].cpu().pin_memory() for k in ("q", "k", "v", "table", "hist") + (("cu",) if "cu" in data else ())}
        out_host = torch.empty((data["tokens"] * data["hq"], cfg["d"]), dtype=torch.bfloat16).pin_memory()
        w.pipe = HostPipeline(host, lambda d: prefill_call(d["q"], d["k"], d["v"], d["table"], d["hist"], d.get("cu")), out_host, device)
        w.h2d = sum(t.numel() * t.element_size() for t in host.values())
        w.d2h = out_host.numel() * 2
        w.units_per_step = w.alg_per_step = data["flops"]
        w.scale = 1e12
        w.launches_per_step, w.collectives_per_step = 1, 0
        w.bound, w.roof_unit = "tensor", "TFLOP/s"
        w.peak = None  # chosen by the length of the timed block (burst or sustained figure)
        w.l2_note = "Q/K/V/out of a step total ~0.4 GB (> 126 MB L2)"
        w.tokens = data["tokens"]
        w.tokens_are_global = hkv_local is not None  # every GPU sees all tokens, for its own heads
        w.data = data
        w.graph = False
    else:
        data = build_fill(cfg, device, seed=rank)
        w.step = lambda: pal.fill_kv_pages(data["keys"], data["vals"], data["k_pool"], data["v_pool"], data["slots"])
        w.pipe = HostPipeline({"keys": data["keys_host"], "vals": data["vals_host"], "slots": data["slots_host"]},
                              lambda d: pal.fill_kv_pages(d["keys"], d["vals"], data["k_pool"], data["v_pool"], d["slots"]) and None, None, device)
        w.h2d = data["keys_host"].numel() * 4 + data["slots_host"].numel() * 8
        w.d2h = 0
        w.units_per_step = w.alg_per_step = data["alg_bytes"]
        w.scale = 1e9
        w.launches_per_step, w.collectives_per_step = 1, 0
        w.bound, w.peak, w.roof_unit = "hbm", peaks["hbm"], "GB/s"
        w.l2_note = "source tokens plus touched sectors exceed L2 (126 MB)"
        w.tokens = data["tokens"]
        w.tokens_are_global = False
        w.data = data
        w.graph = False
        if world > 1:
            w.extra_cfg["parallelism"] = f"token sharded x{world} (each GPU its own tokens and pool), no collective"
    return w


def timed_blocks(env, fn, steps, warmup, blocks, drain=None, sampler=None, gap_s=0.0):
    """`blocks` timed blocks of exactly `steps` calls each, every block bracketed by barrier + synchronize and timed with
    CUDA events on the launching stream; per block the slowest rank's time.  Returns seconds per block.
    `gap_s`: idle time before every block (tensor-bound work: each block then starts from boost clocks, which is how the
    burst peak it is compared with was measured)."""
    for _ in range(warmup):
        fn()
    if drain:
        drain()
    env.barrier()
    if sampler:
        sampler.__enter__()
    out = []
    for _ in range(blocks):
        if gap_s:
            time.sleep(gap_s)
        env.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            fn()
        if drain:
            drain()  # the end event waits for the copy streams as well
        e1.record()
        env.barrier()
        out.append(env.max_over_ranks(e0.elapsed_time(e1)) / 1e3)
    if sampler:
        sampler.__exit__()
    return out


def median(xs):
    s = sorted(xs)
    return s[len(s) // 2] if len(s) % 2 else 0.5 * (s[len(s) // 2 - 1] + s[len(s) // 2])


def measure(w, env, peaks, steps, warmup, blocks, e2e=True):
    """Time a prepared workload; returns the record that goes into the JSON line (identical on every rank)."""
    step = w.step
    graph_note = None
    keep = None
    if w.graph:
        # The context-sharded step is a handful of small launches (and a collective) around tens of microseconds of
        # attention per GPU: it is replayed from a CUDA graph, as a serving loop would do.  If the capture is refused the
        # step stays eager and the record says so.
        try:
            for _ in range(3):
                step()
            env.barrier()
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g):
                keep = step()  # kept alive: the graph writes into it
            step, graph_note = g.replay, True
            w.held_graph = (g, keep)
        except Exception as exc:  # noqa: BLE001
            graph_note = f"capture failed ({type(exc).__name__}: {str(exc)[:80]}); eager"
    sampler = ClockSampler(env.local_rank)
    burst = w.bound == "tensor" and steps * blocks < 2000
    secs = timed_blocks(env, step, steps, warmup, blocks, sampler=sampler, gap_s=0.1 if burst else 0.0)
    sec_med, sec_min = median(secs), min(secs)
    units = w.units_per_step if w.units_are_global else env.sum_over_ranks(float(w.units_per_step))
    tokens = w.tokens if (w.tokens_are_global or env.world == 1) else env.sum_over_ranks(float(w.tokens))
    per_step = sec_med / steps
    rec = {
        "metric": w.metric, "unit": w.unit, "workload": w.cfg["desc"], "scaling": w.scaling,
        "value": units * steps / sec_med / w.scale, "value_best_block": units * steps / sec_min / w.scale,
        "ms_per_step": per_step * 1e3, "blocks": blocks, "steps_per_block": steps, "tokens_per_s": tokens / per_step,
        "gpu_launches_per_step": w.launches_per_step, "collectives_per_step": w.collectives_per_step,
    }
    rec.update(w.extra_cfg)
    if graph_note is not None:
        rec["cuda_graph"] = graph_note
    peak = w.peak
    if peak is None:
        # tensor-bound: short blocks separated by idle gaps run at burst clocks and are compared with the burst peak (itself
        # the best of ten short GEMMs); one block of about a second, under the power cap, is compared with the sustained peak
        peak, rec["peak_kind"] = (peaks["tensor"], "burst: 0.1 s idle before every block") if burst else (peaks["tensor_sustained"], "sustained")
        if burst and not getattr(w, "no_sustained", False):
            long_steps = max(steps, int(1.0 / max(sec_med / steps, 1e-6)))
            sec_long = timed_blocks(env, step, long_steps, 0, 1)[0]
            sustained = units * long_steps / sec_long / w.scale
            rec["sustained"] = {"value": sustained, "steps": long_steps, "peak": peaks["tensor_sustained"],
                                "frac": (w.alg_per_step * long_steps / sec_long / w.scale) / peaks["tensor_sustained"]}
    achieved = w.alg_per_step / per_step / w.scale  # this rank's algorithmic bytes / flops over the step time
    rec["roofline"] = {"bound": w.bound, "achieved": achieved, "peak": peak, "unit": w.roof_unit, "frac": achieved / peak,
                       "peak_source": peaks["source"], "per": "GPU (rank 0's algorithmic work / step time of the slowest rank)"}
    rec["clocks"] = sampler.summary()
    rec["l2"] = w.l2_note
    if e2e and w.pipe is not None:
        e2e_steps = max(3, min(steps, 200))
        e2e_blocks = max(3, min(blocks, 5))
        secs_e = timed_blocks(env, w.pipe.step, e2e_steps, 3, e2e_blocks, drain=w.pipe.drain)
        rec["e2e"] = {"value": units * e2e_steps / median(secs_e) / w.scale, "unit": w.unit, "h2d_bytes_per_step": int(w.h2d),
                      "d2h_bytes_per_step": int(w.d2h), "steps": e2e_steps, "blocks": e2e_blocks,
                      "overlap": "copies on their own streams, two sets of device buffers"}
    return rec


# DRAM bytes per launch from `ncu --set full` captures of the same workloads, not measured in this run; fill_append is
# 0.904 x its algorithmic bytes (captured on the reduced case; the traffic grows with the tokens).
PROFILED_TRAFFIC = {"decode_8b": 1.3866e9, "decode_8b_append": 1.3889e9, "fill": 2.49e9}


def profiled_traffic(name, alg_bytes):
    """DRAM bytes per launch of workload `name` from the committed ncu summaries (None where there is no capture)."""
    if name == "fill_append":
        return 0.904 * alg_bytes
    if name in ("decode_70b", "decode_70b_auto", "decode_70b_small"):
        return 1.0065 * alg_bytes  # captured on the batch-2 case; one read of every page plus the partial triples
    return PROFILED_TRAFFIC.get(name)

EXTRA_SINGLE = ["prefill_8b", "prefill_ragged", "prefill_d256", "decode_8b_append", "decode_70b", "decode_70b_auto", "fill", "fill_append"]
EXTRA_MULTI = ["decode_70b", "decode_70b_auto", "decode_70b_ctx", "decode_70b_ctx_fused", "decode_70b_ctx_fused_auto", "prefill_8b"]


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=500)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--blocks", type=int, default=20, help="timed blocks of --steps steps each; the median block is reported")
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="decode_8b", choices=sorted(WORKLOADS), help="the headline workload")
    ap.add_argument("--workloads", default="all", help="extra records in the same line: all | none | comma-separated names")
    ap.add_argument("--prefill-impl", default="auto")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-cuda-graph", action="store_true", help="context-sharded workloads: enqueue every step from the host")
    ap.add_argument("--no-sustained", action="store_true", help="tensor-bound workloads: skip the one-second block (profiler captures)")
    args = ap.parse_args()
    cfg = WORKLOADS[args.workload]
    env = Env()
    if args.impl == "reference":
        run_reference(args, cfg, env.rank)
        return
    args.warmup = max(args.warmup, 3)
    args.blocks = max(args.blocks, 1)

    import proxy_attention_lab_b200 as pal  # raises if the CUDA library is missing: no fallback

    if not torch.cuda.is_available():
        raise RuntimeError("bench.py needs a CUDA device; there is no CPU path")
    env.init()
    peaks = measured_peaks()

    head = prepare(args.workload, env, pal, peaks, args)
    head.no_sustained = args.no_sustained
    rec = measure(head, env, peaks, args.steps, args.warmup, args.blocks)
    line = {
        "metric": rec["metric"], "value": rec["value"], "unit": rec["unit"], "n_gpus": env.world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": rec["ms_per_step"], "higher_is_better": True, "scaling": rec["scaling"], "vs_baseline": None,
        "dtype": "bf16 (f32 accumulate)", "data": "synthetic",
        "config": {"workload": cfg["desc"]},
        "blocks": args.blocks, "value_best_block": rec["value_best_block"], "timing": "median of the timed blocks; each block is exactly `steps` steps",
        "l2": rec["l2"], "tokens_per_s": rec["tokens_per_s"], "e2e": rec.get("e2e"),
        "gpu_launches": head.launches_per_step * args.steps * args.blocks,
        "clocks": rec["clocks"], "roofline": dict(rec["roofline"]),
    }
    line.update(head.extra_cfg)  # how the workload is spread over the GPUs, beside `config` (which both arms share)
    if "cuda_graph" in rec:
        line["cuda_graph"] = rec["cuda_graph"]
    traffic = profiled_traffic(args.workload, head.alg_per_step) if env.world == 1 else None
    line["roofline"]["traffic"] = traffic
    line["roofline"]["traffic_source"] = "ncu capture of this workload (summary committed with the sources), not measured in this run" if traffic else None
    if env.world == 1 and not args.no_cpu_baseline and env.rank == 0:
        cores = os.cpu_count() or 1
        torch.set_num_threads(cores)
        v, what = cpu_measure(cfg, 12.0, data=head.data if head.kind in ("decode", "prefill") else None)
        line["cpu_baseline"] = {"value": v, "unit": rec["unit"], "cores": torch.get_num_threads(), "kind": "port", "sample": what}
    head_data_kept = head  # noqa: F841  (its tensors stay resident; the extra workloads are sized to fit beside them)

    # ---- the other parts of the metric, one record each ----
    names = []
    if args.workloads == "all":
        names = [n for n in (EXTRA_SINGLE if env.world == 1 else EXTRA_MULTI) if n != args.workload]
    elif args.workloads != "none":
        names = [n for n in args.workloads.split(",") if n]
    records = {}
    # shorter blocks for the extras: they only have to carry two digits
    x_steps, x_blocks = max(5, min(args.steps, 50)), max(3, min(args.blocks, 10))
    for name in names:
        if name not in WORKLOADS:
            records[name] = {"unavailable": "unknown workload"}
            continue
        wcfg = WORKLOADS[name]
        steps_n = x_steps if wcfg["kind"] != "prefill" else max(5, min(args.steps, 20))
        w = None
        try:
            if wcfg.get("ctx") == "nccl" and env.world == 1:
                continue  # on one GPU this is decode_70b
            if wcfg["kind"] == "decode" and env.world > 1 and wcfg["hkv"] % env.world and not wcfg.get("ctx"):
                records[name] = {"unavailable": f"{wcfg['hkv']} kv heads do not divide over {env.world} GPUs"}
                continue
            w = prepare(name, env, pal, peaks, args)
            w.no_sustained = args.no_sustained
            r = measure(w, env, peaks, steps_n, max(3, min(args.warmup, 5)), x_blocks)
            t = profiled_traffic(name, w.alg_per_step) if env.world == 1 else None
            r["roofline"]["traffic"] = t
            r["roofline"]["traffic_source"] = "ncu capture of this workload or of its reduced case, scaled (summary committed with the sources), not measured in this run" if t else None
            if env.world > 1 and w.scaling == "strong":
                # the same problem on ONE GPU, run by every rank at the same time: the N = 1 figure of this very run
                base_name = "decode_70b" if wcfg["kind"] == "decode" else name
                solo = Env.__new__(Env)
                solo.__dict__.update(rank=0, world=1, local_rank=env.local_rank, device=env.device, dist=None)
                del w
                w = None
                torch.cuda.empty_cache()
                w1 = prepare(base_name, solo, pal, peaks, args, force_single=True)
                gap = 0.1 if (w1.bound == "tensor" and steps_n * x_blocks < 2000) else 0.0  # timed as the N-GPU record was
                secs = timed_blocks(env, w1.step, steps_n, 3, x_blocks, gap_s=gap)  # env: barriers keep the ranks in step, max over ranks
                n1 = w1.units_per_step * steps_n / median(secs) / w1.scale
                r["n1_value_same_run"] = n1
                r["speedup_vs_n1"] = r["value"] / n1
                r["efficiency_vs_n1"] = r["value"] / n1 / env.world
                del w1
            records[name] = r
        except Exception as exc:  # noqa: BLE001  (one record failing must not take the headline with it)
            records[name] = {"unavailable": f"{type(exc).__name__}: {str(exc)[:200]}"}
        finally:
            w = None
            torch.cuda.empty_cache()
    if names:
        line["workloads"] = records
    if env.rank == 0:
        print(json.dumps(line), flush=True)
    if env.dist is not None or getattr(env, "own_group", None) is not None:
        d = env.dist or env.own_group
        if env.dist is not None:
            env.dist.barrier()
        # captured graphs hold the collective's communicator: release them before the process group goes away
        head = head_data_kept = None  # noqa: F841
        torch.cuda.synchronize()
        d.destroy_process_group()


if __name__ == "__main__":
    main()
