#!/usr/bin/env python
"""Benchmark of the paged-attention hot path on B200.

``python bench.py --gpus N --steps K --warmup W`` prints ONE JSON line (rank 0).  A step is one pass
of the operator over one batch of synthetic input already resident in HBM.  The default workload is
the Llama-3-8B-shaped decode batch the headline metric (paged decode KV GB/s) is quoted on; other
workloads (``--workload decode_70b | prefill_8b | fill | fill_append``) cover the remaining configurations.

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
    "decode_70b": dict(kind="decode", S=8, lo=131072, hi=131072, hq=64, hkv=8, d=128, tpp=16, partition_pages=256,
                       desc="Llama-3-70B long decode: batch 8, context 131072, 64q/8kv heads, D=128, bf16, TPP=16, two-pass 256-page partitions"),
    "decode_70b_ctx": dict(kind="decode", S=8, lo=131072, hi=131072, hq=64, hkv=8, d=128, tpp=16, partition_pages=256, ctx_sharded=True,
                           desc="Llama-3-70B long decode, context sharded: batch 8, context 131072 cut into N contiguous slices (one per GPU), "
                                "64q/8kv heads, D=128, bf16, TPP=16, 256-page partitions, per-GPU (m,l,acc) all-gathered over NCCL and merged"),
    "prefill_8b": dict(kind="prefill", S=8, n=2048, hlo=0, hhi=4096, hq=32, hkv=8, d=128, tpp=16,
                       desc="Llama-3-8B chunked causal prefill: 8 x 2048 new tokens, history U[0,4096], 32q/8kv heads, D=128, bf16, TPP=16"),
    "prefill_small": dict(kind="prefill", S=2, n=1024, hlo=0, hhi=2048, hq=32, hkv=8, d=128, tpp=16,
                          desc="reduced chunked prefill for profiler captures: 2 x 1024 new tokens, history U[0,2048], 32q/8kv heads, D=128, bf16, TPP=16"),
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

    def __init__(self, index: int, period_s: float = 0.01):
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
    if cfg["partition_pages"]:
        parts = (MP + cfg["partition_pages"] - 1) // cfg["partition_pages"]
        alg_bytes += 2 * cfg["S"] * hq_local * parts * (d + 2) * 4
    return dict(k_pool=k_pool, v_pool=v_pool, q_host=q_host, table_host=table_host, lens_host=lens_host,
                q=q_host.to(device), table=table_host.to(device), lens=lens_host.to(device), kv_bytes=kv_bytes,
                alg_bytes=alg_bytes, tokens=cfg["S"], hq=hq_local, hkv=hkv, lens_cpu=lens)


def build_prefill(cfg, device, seed, seqs=None):
    tpp, d, hq, hkv, n = cfg["tpp"], cfg["d"], cfg["hq"], cfg["hkv"], cfg["n"]
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
def cpu_decode_sample(cfg, budget_s, seed=0):
    """Times the oracle on the first sequences of the workload until `budget_s` is spent. Returns (bytes, seconds, n_seqs)."""
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


def cpu_prefill_sample(cfg, budget_s, seed=0):
    from oracle import prefill_oracle

    tpp, d, hq, hkv = cfg["tpp"], cfg["d"], cfg["hq"], cfg["hkv"]
    n = min(cfg["n"], 512)  # a 512-token slice of one sequence keeps the score matrix small
    hist = int(make_lengths(seed, cfg["S"], cfg["hlo"], cfg["hhi"])[0])
    g = torch.Generator().manual_seed(seed + 7)
    npg = max((hist + tpp - 1) // tpp, 1)
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


def cpu_measure(cfg, budget_s):
    kind = cfg["kind"]
    if kind == "decode":
        nbytes, spent, nseq = cpu_decode_sample(cfg, budget_s)
        return nbytes / spent / 1e9, f"first {nseq} sequences of the batch ({nbytes / 1e9:.3f} GB of KV)"
    if kind == "prefill":
        flops, spent, what = cpu_prefill_sample(cfg, budget_s)
        return flops / spent / 1e12, what
    nbytes, spent, what = cpu_fill_sample(cfg, budget_s)
    return nbytes / spent / 1e9, what


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
            "data": "synthetic", "config": {"workload": cfg["desc"]},
            "cpu_baseline": {"value": value, "unit": unit, "cores": torch.get_num_threads(), "kind": "port", "sample": f"each step: {what}"},
            "e2e": {"value": value, "unit": unit, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}, "gpu_launches": 0}
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------------------------------------------
# GPU side
# ------------------------------------------------------------------------------------------------
def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=2000)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="decode_8b", choices=sorted(WORKLOADS))
    ap.add_argument("--prefill-impl", default="auto")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-cuda-graph", action="store_true", help="context-sharded workload: enqueue every step from the host")
    args = ap.parse_args()
    cfg = WORKLOADS[args.workload]
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        run_reference(args, cfg, rank)
        return

    import torch.distributed as dist

    import proxy_attention_lab_b200 as pal  # raises if the CUDA library is missing: no fallback

    if not torch.cuda.is_available():
        raise RuntimeError("bench.py needs a CUDA device; there is no CPU path")
    device = torch.device("cuda", local_rank)
    torch.cuda.set_device(device)
    if world > 1:
        dist.init_process_group("nccl", device_id=device)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    kind = cfg["kind"]
    metric, unit = metric_of(kind)
    peaks = measured_peaks()
    scaling = "weak"
    extra_cfg = {}
    if kind == "decode":
        hkv_local = None
        ctx = bool(cfg.get("ctx_sharded"))
        if ctx:
            scaling = "strong"
            extra_cfg["parallelism"] = f"context sharded x{world}: partials + one NCCL all-gather + LSE combine per step"
            cfg = dict(cfg, lo=cfg["lo"] // world, hi=cfg["hi"] // world)  # this rank's slice of every sequence
        if args.workload == "decode_70b" and world > 1:
            # total work fixed: each GPU owns Hkv/N kv heads (and their query heads) of every sequence
            hkv_local, scaling = cfg["hkv"] // world, "strong"
            extra_cfg["parallelism"] = f"kv-head sharded x{world}, no collective"
        elif world > 1 and not ctx:
            extra_cfg["parallelism"] = f"sequence sharded x{world} (each GPU its own batch of {cfg['S']}), no collective"
        data = build_decode(cfg, device, seed=rank if hkv_local is None else 0, hkv_local=hkv_local)
        pp = cfg["partition_pages"]
        if ctx:
            from proxy_attention_lab_b200.sharding import all_gather_partials

            if world > 1:  # every rank must hold the same queries
                dist.broadcast(data["q"], src=0)

        append = cfg.get("append")
        if append:
            gen = torch.Generator(device=device).manual_seed(1234 + rank)
            new_k = torch.randn((cfg["S"], data["k_pool"].shape[1], cfg["d"]), device=device, dtype=torch.bfloat16, generator=gen)
            new_v = torch.randn_like(new_k)
            new_k_host, new_v_host = new_k.cpu().pin_memory(), new_v.cpu().pin_memory()
            last_pos = (data["lens"] - 1).to(torch.int32)
            seq_ids = torch.arange(cfg["S"], device=device, dtype=torch.int32)

        def decode_call(q, table, lens, nk=None, nv=None):
            nk, nv = (new_k, new_v) if nk is None and append else (nk, nv)
            if append == "fused":
                return pal.paged_attention_decode_append(nk, nv, q, data["k_pool"], data["v_pool"], table, lens, partition_pages=pp)
            if append == "pair":
                pal.fill_kv_pages(nk, nv, data["k_pool"], data["v_pool"], table, last_pos, seq_ids)
            if not ctx:
                return pal.paged_attention_decode(q, data["k_pool"], data["v_pool"], table, lens, partition_pages=pp)
            m, l, acc = pal.paged_attention_decode_partials(q, data["k_pool"], data["v_pool"], table, lens, partition_pages=pp)
            if world > 1:
                m, l, acc = all_gather_partials(m, l, acc)
            else:
                m, l, acc = m[None], l[None], acc[None]
            return pal.lse_combine(m, l, acc, out_dtype=torch.bfloat16)

        def step():
            return decode_call(data["q"], data["table"], data["lens"])

        out_host = torch.empty((cfg["S"], data["hq"], cfg["d"]), dtype=torch.bfloat16).pin_memory()
        e2e_inputs = {"q": data["q_host"], "table": data["table_host"], "lens": data["lens_host"]}
        if append:
            e2e_inputs.update(new_k=new_k_host, new_v=new_v_host)
        pipe = HostPipeline(e2e_inputs, lambda d: decode_call(d["q"], d["table"], d["lens"], d.get("new_k"), d.get("new_v")), out_host, device)

        h2d = data["q_host"].numel() * 2 + data["table_host"].numel() * 4 + data["lens_host"].numel() * 4
        d2h = out_host.numel() * 2
        if append:
            h2d += 2 * new_k_host.numel() * 2
        units_per_step, alg_per_step = data["kv_bytes"], data["alg_bytes"]
        to_value = lambda units, sec: units / sec / 1e9
        launches_per_step = (3 if ctx else 2) if pp else 1
        if append == "pair":
            launches_per_step += 1
        bound, peak = "hbm", peaks["hbm"]
        achieved_of = lambda sec: alg_per_step / sec / 1e9
        roof_unit = "GB/s"
        l2_note = "KV pool per GPU is larger than L2 (126 MB); every step streams it from HBM"
    elif kind == "prefill":
        seqs = None
        if world > 1:
            from proxy_attention_lab_b200.sharding import partition_sequences

            hist_all = make_lengths(0, cfg["S"], cfg["hlo"], cfg["hhi"])
            n_all = make_lengths(5, cfg["S"], cfg["nlo"], cfg["n"]).tolist() if "nlo" in cfg else [cfg["n"]] * cfg["S"]
            work = [n * int(h) + n * (n + 1) // 2 for n, h in zip(n_all, hist_all)]
            seqs = partition_sequences(work, world)[rank] or [rank % cfg["S"]]
            scaling = "strong"
            extra_cfg["parallelism"] = f"sequence sharded x{world}, no collective"
        data = build_prefill(cfg, device, seed=0, seqs=seqs)

        def prefill_call(q, k, v, table, hist, cu=None):
            if cu is None:
                return pal.paged_attention_prefill(q, k, v, data["k_pool"], data["v_pool"], table, hist, impl=args.prefill_impl)
            return pal.paged_attention_prefill_ragged(q, k, v, data["k_pool"], data["v_pool"], table, hist, cu,
                                                      max_new_tokens=data["max_new"], impl=args.prefill_impl)

        def step():
            return prefill_call(data["q"], data["k"], data["v"], data["table"], data["hist"], data.get("cu"))

        host = {k: data[k].cpu().pin_memory() for k in ("q", "k", "v", "table", "hist") + (("cu",) if "cu" in data else ())}
        out_host = torch.empty((data["tokens"] * cfg["hq"], cfg["d"]), dtype=torch.bfloat16).pin_memory()
        pipe = HostPipeline(host, lambda d: prefill_call(d["q"], d["k"], d["v"], d["table"], d["hist"], d.get("cu")), out_host, device)

        h2d = sum(t.numel() * t.element_size() for t in host.values())
        d2h = out_host.numel() * 2
        units_per_step = alg_per_step = data["flops"]
        to_value = lambda units, sec: units / sec / 1e12
        launches_per_step = 1
        bound, peak = "tensor", peaks["tensor_sustained"] if args.steps >= 200 else peaks["tensor"]
        achieved_of = lambda sec: alg_per_step / sec / 1e12
        roof_unit = "TFLOP/s"
        l2_note = "L2 flushed by design of the workload: Q/K/V/out of a step total ~0.4 GB (> 126 MB L2)"
    else:
        data = build_fill(cfg, device, seed=rank)

        def step():
            return pal.fill_kv_pages(data["keys"], data["vals"], data["k_pool"], data["v_pool"], data["slots"])

        pipe = HostPipeline({"keys": data["keys_host"], "vals": data["vals_host"], "slots": data["slots_host"]},
                            lambda d: pal.fill_kv_pages(d["keys"], d["vals"], data["k_pool"], data["v_pool"], d["slots"]) and None, None, device)

        h2d = data["keys_host"].numel() * 4 + data["slots_host"].numel() * 8
        d2h = 0
        units_per_step = alg_per_step = data["alg_bytes"]
        to_value = lambda units, sec: units / sec / 1e9
        launches_per_step = 1
        bound, peak = "hbm", peaks["hbm"]
        achieved_of = lambda sec: alg_per_step / sec / 1e9
        roof_unit = "GB/s"
        l2_note = "source tokens plus touched sectors exceed L2 (126 MB)"

    def timed(fn, steps, warmup, sample_clocks, drain=None):
        for _ in range(warmup):
            fn()
        if drain:
            drain()
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        sampler = ClockSampler(local_rank) if sample_clocks else None
        if sampler:
            sampler.__enter__()
        e0.record()
        for _ in range(steps):
            fn()
        if drain:
            drain()  # the end event waits for the copy streams as well
        e1.record()
        barrier()
        if sampler:
            sampler.__exit__()
        ms = e0.elapsed_time(e1)
        if world > 1:
            t = torch.tensor([ms], device=device, dtype=torch.float64)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        return ms / 1e3, sampler

    # The context-sharded step is nine small launches and an NCCL call around 85 us of attention per GPU at 8 GPUs: the
    # host cannot enqueue it as fast as the GPU runs it.  It is replayed from a CUDA graph, as a serving loop would do
    # (every rank captures the same sequence; if the capture is refused the step stays eager and the line says so).
    graph = graph_out = None
    if cfg.get("ctx_sharded") and not args.no_cuda_graph:
        try:
            for _ in range(3):
                step()
            barrier()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                graph_out = step()  # noqa: F841  (kept alive: the graph writes into it)
            step = graph.replay
            extra_cfg["cuda_graph"] = True
        except Exception as exc:  # capture of the collective refused: fall back, visibly
            extra_cfg["cuda_graph"] = f"capture failed ({type(exc).__name__}); eager"
    sec, sampler = timed(step, args.steps, args.warmup, True)
    e2e_steps = max(3, min(args.steps, 200))
    sec_e2e, _ = timed(pipe.step, e2e_steps, 3, False, drain=pipe.drain)

    total_units, total_tokens = units_per_step, data["tokens"]
    if world > 1:
        kv_head_sharded = args.workload in ("decode_70b", "decode_70b_ctx")
        t = torch.tensor([float(units_per_step), 0.0 if kv_head_sharded else float(data["tokens"])], device=device, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.SUM)
        total_units = float(t[0].item())
        total_tokens = data["tokens"] if kv_head_sharded else float(t[1].item())
    per_step = sec / args.steps
    value = to_value(total_units * args.steps, sec)
    e2e_value = to_value(total_units * e2e_steps, sec_e2e)

    if rank == 0:
        achieved = achieved_of(per_step)
        # DRAM bytes per launch from one `ncu --set full` capture of the same workload (see profiles/)
        # fill_append: 0.904 x the algorithmic bytes, from the capture of the reduced case (traffic grows with the tokens)
        traffic = {"decode_8b": 1.3866e9, "decode_8b_append": 1.3889e9,
                   "fill_append": 0.904 * alg_per_step}.get(args.workload) if world == 1 else None
        line = {
            "metric": metric, "value": value, "unit": unit, "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": per_step * 1e3, "higher_is_better": True, "scaling": scaling, "vs_baseline": None,
            "dtype": "bf16 (f32 accumulate)", "data": "synthetic",
            "config": {"workload": cfg["desc"], "l2": l2_note, **extra_cfg},
            "tokens_per_s": total_tokens / per_step,
            "e2e": {"value": e2e_value, "unit": unit, "h2d_bytes_per_step": int(h2d), "d2h_bytes_per_step": int(d2h), "steps": e2e_steps,
                    "overlap": "copies on their own streams, two sets of device buffers"},
            "gpu_launches": launches_per_step * args.steps,
            "clocks": sampler.summary() if sampler else None,
            "roofline": {"bound": bound, "achieved": achieved, "peak": peak, "unit": roof_unit, "frac": achieved / peak, "traffic": traffic,
                         "peak_source": peaks["source"], "kernel": "rank 0 per-step time over the timed region (CUDA events)"},
        }
        if world == 1 and not args.no_cpu_baseline:
            cores = os.cpu_count() or 1
            torch.set_num_threads(cores)
            v, what = cpu_measure(cfg, 12.0)
            line["cpu_baseline"] = {"value": v, "unit": unit, "cores": torch.get_num_threads(), "kind": "port", "sample": what}
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        # a captured graph holds the collective's communicator: release it before the process group goes away
        step = pipe = graph = graph_out = None  # noqa: F841
        torch.cuda.synchronize()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
