"""The BASELINE configurations at full size.  The oracle is run on slices small enough for the CPU; the
rest of each batch is covered by size-independent properties (two-pass == single pass, batch-order
invariance, linearity of the log-sum-exp combine, agreement of the two prefill kernels)."""

import pytest
import torch

from cases import parity_report
from oracle import decode_oracle, prefill_oracle

pytestmark = pytest.mark.gpu
TOL = 2e-3


def within(out, ref):
    """Against the fp32 oracle (cases.parity_report): float32 outputs by plain max-abs <= 2e-3, 16-bit outputs with the
    one-unit-in-the-last-place clause for elements whose rounding alone exceeds that."""
    return parity_report(out, ref)


def close(a, b):
    """Two kernel results of one output type that must agree: each is within tolerance of the oracle, so their distance is
    bounded by twice that plus one rounding step of the larger magnitude."""
    a, b = a.float().cpu(), b.float().cpu()
    diff = (a - b).abs()
    return bool((diff <= 2 * TOL + b.abs() * 2.0 ** -7).all()), diff.max().item()


def build_decode(cuda, S, lo, hi, hq, hkv, seed=0, d=128, tpp=16):
    g = torch.Generator().manual_seed(seed)
    lens = torch.randint(lo, hi + 1, (S,), generator=g)
    npg = (lens + tpp - 1) // tpp
    P, MP = int(npg.sum()), int(npg.max())
    perm = torch.randperm(P, generator=g)
    table = torch.zeros((S, MP), dtype=torch.int32)
    off = 0
    for s in range(S):
        n = int(npg[s])
        table[s, :n] = perm[off:off + n].to(torch.int32)
        off += n
    gen = torch.Generator(device=cuda).manual_seed(seed + 1)
    k_pool = torch.randn((P, hkv, d // 8, tpp, 8), device=cuda, dtype=torch.bfloat16, generator=gen)
    v_pool = torch.randn((P, hkv, d, tpp), device=cuda, dtype=torch.bfloat16, generator=gen)
    q = torch.randn((S, hq, d), device=cuda, dtype=torch.bfloat16, generator=gen)
    return q, k_pool, v_pool, table.to(cuda), lens.to(torch.int32).to(cuda)


def oracle_decode_slice(q, k_pool, v_pool, table, lens, seqs, kv_heads, group):
    """Oracle for the given sequences and kv heads only (their pages are copied to the CPU)."""
    outs = []
    for s in seqs:
        L = int(lens[s])
        n = (L + 15) // 16
        pages = table[s, :n].long()
        kp = k_pool[pages][:, kv_heads].cpu()
        vp = v_pool[pages][:, kv_heads].cpu()
        qh = torch.cat([q[s:s + 1, h * group:(h + 1) * group] for h in kv_heads], dim=1).cpu()
        outs.append(decode_oracle(qh, kp, vp, torch.arange(n, dtype=torch.int32).reshape(1, n), torch.tensor([L], dtype=torch.int32)))
    return torch.cat(outs)


def test_llama8b_decode_batch_full(pal, cuda):
    """Batch 64, contexts U[1024,8192], 32 q / 8 kv heads, D=128, bf16, TPP=16, fused single pass."""
    q, kp, vp, table, lens = build_decode(cuda, 64, 1024, 8192, 32, 8)
    out = pal.paged_attention_decode(q, kp, vp, table, lens, partition_pages=0)
    seqs = [0, 17, int(lens.argmax()), int(lens.argmin())]
    ref = oracle_decode_slice(q, kp, vp, table, lens, seqs, list(range(8)), 4)
    ok, err = within(out[seqs], ref)
    assert ok, err
    out32 = pal.paged_attention_decode(q, kp, vp, table, lens, partition_pages=0, out_dtype=torch.float32)
    ok, err = within(out32[seqs], ref)
    assert ok, err
    # two-pass gives the same answer on the whole batch
    ok, err = close(pal.paged_attention_decode(q, kp, vp, table, lens, partition_pages=64), out)
    assert ok, err
    ok, err = close(pal.paged_attention_decode(q, kp, vp, table, lens, partition_pages=64, out_dtype=torch.float32), out32)
    assert ok, err
    # the order of the sequences in the batch does not change any sequence's result (bit for bit)
    perm = torch.randperm(64, generator=torch.Generator().manual_seed(3)).to(cuda)
    out_p = pal.paged_attention_decode(q[perm].contiguous(), kp, vp, table[perm].contiguous(), lens[perm].contiguous(), partition_pages=0)
    assert torch.equal(out_p, out[perm])


def test_llama70b_long_decode_full(pal, cuda):
    """Batch 8, context 131072, 64 q / 8 kv heads, two-pass with 256-page partitions."""
    q, kp, vp, table, lens = build_decode(cuda, 8, 131072, 131072, 64, 8, seed=5)
    out = pal.paged_attention_decode(q, kp, vp, table, lens, partition_pages=256)
    ref = oracle_decode_slice(q, kp, vp, table, lens, [3], [0, 5], 8)
    got = torch.cat([out[3:4, 0:8], out[3:4, 40:48]], dim=1)
    ok, err = within(got, ref)
    assert ok, err
    out32 = pal.paged_attention_decode(q, kp, vp, table, lens, partition_pages=256, out_dtype=torch.float32)
    ok, err = within(torch.cat([out32[3:4, 0:8], out32[3:4, 40:48]], dim=1), ref)
    assert ok, err
    # single pass, a different partition size and the launcher's own choice agree with it
    for pp in (0, 1024, None):
        ok, err = close(pal.paged_attention_decode(q, kp, vp, table, lens, partition_pages=pp), out)
        assert ok, err
    # linearity of the combine: partials over the two halves of every context merge to the full result
    half = table.shape[1] // 2
    zeros = torch.zeros_like(lens)
    m1, l1, a1 = pal.paged_attention_decode_partials(q, kp, vp, table[:, :half].contiguous(), torch.minimum(lens, zeros + half * 16), partition_pages=256)
    m2, l2, a2 = pal.paged_attention_decode_partials(q, kp, vp, table[:, half:].contiguous(), torch.clamp(lens - half * 16, min=0), partition_pages=256)
    merged = pal.lse_combine(torch.stack([m1, m2]), torch.stack([l1, l2]), torch.stack([a1, a2]), out_dtype=torch.bfloat16)
    ok, err = close(merged, out)
    assert ok, err
    # the packed form of the same exchange: one [rows, D + 2] buffer per half, merged in place
    p1 = pal.paged_attention_decode_partials(q, kp, vp, table[:, :half].contiguous(), torch.minimum(lens, zeros + half * 16), partition_pages=256, packed=True)
    p2 = pal.paged_attention_decode_partials(q, kp, vp, table[:, half:].contiguous(), torch.clamp(lens - half * 16, min=0), partition_pages=256, packed=True)
    merged_p = pal.lse_combine_packed(torch.stack([p1, p2]), out_dtype=torch.bfloat16, out_shape=out.shape)
    assert torch.equal(merged_p, merged)


def test_chunked_prefill_full(pal, cuda):
    """8 sequences x 2048 new tokens, history U[0,4096], 32 q / 8 kv heads: tcgen05 kernel."""
    S, N, hq, hkv, d, tpp = 8, 2048, 32, 8, 128, 16
    g = torch.Generator().manual_seed(0)
    hist = torch.randint(0, 4097, (S,), generator=g)
    hist[1] = 0      # one sequence without history, one with a partial last page
    hist[2] = 1003
    npg = (hist + tpp - 1) // tpp
    P, MP = int(npg.sum()), int(npg.max())
    perm = torch.randperm(P, generator=g)
    table = torch.zeros((S, MP), dtype=torch.int32)
    off = 0
    for s in range(S):
        n = int(npg[s])
        table[s, :n] = perm[off:off + n].to(torch.int32)
        off += n
    gen = torch.Generator(device=cuda).manual_seed(1)
    mk = lambda *shape: torch.randn(shape, device=cuda, dtype=torch.bfloat16, generator=gen)
    kp, vp = mk(P, hkv, d // 8, tpp, 8), mk(P, hkv, d, tpp)
    q, k, v = mk(S * N, hq, d), mk(S * N, hkv, d), mk(S * N, hkv, d)
    table, hist_d = table.to(cuda), hist.to(torch.int32).to(cuda)
    out = pal.paged_attention_prefill(q, k, v, kp, vp, table, hist_d, impl="tcgen05").reshape(S, N, hq, d)
    out32 = pal.paged_attention_prefill(q, k, v, kp, vp, table, hist_d, impl="tcgen05", out_dtype=torch.float32).reshape(S, N, hq, d)
    # oracle on two whole sequences, one kv head (4 query heads) each
    for s, kvh in ((1, 0), (2, 7)):
        n = int(npg[s])
        pages = table[s, :n].long()
        ref = prefill_oracle(q[s * N:(s + 1) * N, kvh * 4:(kvh + 1) * 4].cpu(), k[s * N:(s + 1) * N, kvh:kvh + 1].cpu(),
                             v[s * N:(s + 1) * N, kvh:kvh + 1].cpu(), kp[pages][:, kvh:kvh + 1].cpu(), vp[pages][:, kvh:kvh + 1].cpu(),
                             torch.arange(max(n, 1), dtype=torch.int32).reshape(1, -1)[:, :n], hist[s:s + 1].to(torch.int32))
        ok, err = within(out[s, :, kvh * 4:(kvh + 1) * 4].reshape(N * 4, d), ref)
        assert ok, (s, err)
        ok, err = within(out32[s, :, kvh * 4:(kvh + 1) * 4].reshape(N * 4, d), ref)
        assert ok, (s, err)
    # the mma.sync kernel agrees with it on the whole batch (each is within tolerance of the oracle,
    # so their distance is bounded by twice that)
    out2 = pal.paged_attention_prefill(q, k, v, kp, vp, table, hist_d, impl="mma").reshape(S, N, hq, d)
    diff = (out.float() - out2.float()).abs()
    allowed = 2 * TOL + out2.float().abs() * 2.0 ** -6
    assert bool((diff <= allowed).all()), diff.max().item()
    assert torch.isfinite(out.float()).all()
