"""Seeded builders of paged-attention test cases, shared by the CPU (oracle) and GPU (kernel) tests.

Everything is generated on the CPU with a seeded generator so that the oracle and the kernels see
identical bits; GPU tests copy the tensors over.
"""

from __future__ import annotations

import math
from dataclasses import dataclass, field

import torch

from oracle import k_cache_shape, pack_sequences_into_pages, v_cache_shape


@dataclass
class DecodeCase:
    q: torch.Tensor
    k_pool: torch.Tensor
    v_pool: torch.Tensor
    page_table: torch.Tensor
    lens: torch.Tensor
    meta: dict = field(default_factory=dict)


def make_decode_case(seed, lens, hq, hkv, d, tpp=16, dtype=torch.float16, extra_pages=0, shuffle=True,
                     pad_entry=0, poison_unused=False, table_width=None, q_scale=1.0) -> DecodeCase:
    g = torch.Generator().manual_seed(seed)
    S = len(lens)
    pages_per_seq = [(L + tpp - 1) // tpp for L in lens]
    total = sum(pages_per_seq) + extra_pages
    total = max(total, 1)
    perm = torch.randperm(total, generator=g) if shuffle else torch.arange(total)
    width = table_width or max(max(pages_per_seq), 1)
    table = torch.full((S, width), pad_entry, dtype=torch.int64)
    page_lists, off = [], 0
    for s, n in enumerate(pages_per_seq):
        ids = perm[off:off + n]
        off += n
        table[s, :n] = ids
        page_lists.append(ids.tolist())
    k_pool = torch.zeros(k_cache_shape(total, hkv, d, tpp, dtype), dtype=dtype)
    v_pool = torch.zeros(v_cache_shape(total, hkv, d, tpp, dtype), dtype=dtype)
    if poison_unused:
        k_pool.fill_(float("nan"))
        v_pool.fill_(float("nan"))
    ks = [torch.randn((L, hkv, d), generator=g).to(dtype) for L in lens]
    vs = [torch.randn((L, hkv, d), generator=g).to(dtype) for L in lens]
    pack_sequences_into_pages(ks, vs, page_lists, k_pool, v_pool)
    q = (torch.randn((S, hq, d), generator=g) * q_scale).to(dtype)
    # int32 carries the same bits as the reference's uint32 for every valid id; 0xFFFFFFFF pads show as -1
    table = table.to(torch.int64)
    table = torch.where(table > 0x7FFFFFFF, table - (1 << 32), table).to(torch.int32)
    return DecodeCase(q, k_pool, v_pool, table, torch.tensor(lens, dtype=torch.int32),
                      dict(hq=hq, hkv=hkv, d=d, tpp=tpp, dtype=dtype, k_seqs=ks, v_seqs=vs))


@dataclass
class PrefillCase:
    q: torch.Tensor
    k_new: torch.Tensor
    v_new: torch.Tensor
    k_pool: torch.Tensor
    v_pool: torch.Tensor
    page_table: torch.Tensor
    hist: torch.Tensor


def make_prefill_case(seed, hist_lens, n_new, hq, hkv, d, tpp=16, dtype=torch.bfloat16, poison_unused=False) -> PrefillCase:
    base = make_decode_case(seed, hist_lens, hq, hkv, d, tpp=tpp, dtype=dtype, poison_unused=poison_unused)
    g = torch.Generator().manual_seed(seed + 1000)
    S = len(hist_lens)
    q = torch.randn((S * n_new, hq, d), generator=g).to(dtype)
    k = torch.randn((S * n_new, hkv, d), generator=g).to(dtype)
    v = torch.randn((S * n_new, hkv, d), generator=g).to(dtype)
    return PrefillCase(q, k, v, base.k_pool, base.v_pool, base.page_table, torch.tensor(hist_lens, dtype=torch.int32))


def uniform_lengths(seed, count, lo, hi):
    g = torch.Generator().manual_seed(seed)
    return torch.randint(lo, hi + 1, (count,), generator=g).tolist()


def to_dev(case, device):
    out = {}
    for k, v in vars(case).items():
        if isinstance(v, torch.Tensor):
            out[k] = v.to(device)
    return out


def max_abs(a, b):
    return (a.float() - b.float()).abs().max().item() if a.numel() else 0.0


# ------------------------------------------------------------------------------------------------
# the parity rule
# ------------------------------------------------------------------------------------------------
TOL = 2e-3  # max-abs against the fp32 oracle, for 16-bit inputs with fp32 accumulation


def ulp_distance(a16: torch.Tensor, b16: torch.Tensor) -> torch.Tensor:
    """Distance in units in the last place between two tensors of one 16-bit float type (same-sign values:
    the difference of their bit patterns; across zero: the sum of both magnitudes' patterns)."""
    ia = a16.contiguous().view(torch.int16).to(torch.int32)
    ib = b16.contiguous().view(torch.int16).to(torch.int32)
    # map sign-magnitude patterns onto a monotone integer line
    ka = torch.where(ia < 0, -(ia & 0x7FFF), ia)
    kb = torch.where(ib < 0, -(ib & 0x7FFF), ib)
    return (ka - kb).abs()


def parity_report(out: torch.Tensor, ref32: torch.Tensor):
    """Compare a kernel output with the fp32 oracle.

    float32 outputs: every element must be within TOL (plain max-abs).
    16-bit outputs: an element passes when it is within TOL of the fp32 oracle, or within one unit in the last
    place (by bit pattern) of the oracle rounded to the output type - rounding a result of magnitude >= 0.5 to
    bf16 alone moves it by more than TOL.
    Returns (ok, message); the message carries both max-abs figures and lists the elements that needed the
    second clause.
    """
    out = out.detach().cpu()
    ref32 = ref32.detach().cpu().float().reshape(out.shape)
    if out.numel() == 0:
        return True, "empty"
    if not torch.isfinite(out.float()).all():
        return False, "non-finite values in the output"
    diff = (out.float() - ref32).abs()
    max_abs_fp32 = diff.max().item()
    if out.dtype == torch.float32:
        return max_abs_fp32 <= TOL, f"max-abs vs fp32 oracle {max_abs_fp32:.3e} (float32 output, limit {TOL})"
    ref16 = ref32.to(out.dtype)
    max_abs_rounded = (out.float() - ref16.float()).abs().max().item()
    over = diff > TOL
    n_over = int(over.sum())
    msg = f"max-abs vs fp32 oracle {max_abs_fp32:.3e}, vs oracle rounded to {out.dtype} {max_abs_rounded:.3e}"
    if n_over == 0:
        return True, msg
    dist = ulp_distance(out[over], ref16[over])
    bad = int((dist > 1).sum())
    mags = ref32[over].abs()
    msg += (f"; {n_over} elements beyond {TOL} pass by the 1-ulp clause only if their distance <= 1 "
            f"(|ref| from {mags.min().item():.3f} to {mags.max().item():.3f}, largest distance {int(dist.max())} ulp, {bad} fail)")
    return bad == 0, msg


def assert_parity(out, ref32, what=""):
    ok, msg = parity_report(out, ref32)
    assert ok, f"{what}: {msg}" if what else msg
    return msg
