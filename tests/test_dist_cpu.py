"""Multi-rank host logic on CPU: gloo, world_size 2.  The compute inside each rank is the CPU oracle;
what is under test is the sharding arithmetic and the gather-then-combine protocol."""

import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from cases import make_decode_case
from oracle import decode_oracle, decode_partials_oracle, lse_combine_oracle
from proxy_attention_lab_b200.sharding import (
    all_gather_partials,
    context_slice,
    decode_context_parallel,
    kv_head_range,
    partition_sequences,
)


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, fn, ret):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        ret[rank] = fn(rank, world)
    finally:
        dist.destroy_process_group()


def _run(fn, world=2):
    ctx = mp.get_context("spawn")
    ret = ctx.Manager().dict()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, fn, ret)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(120)
        assert p.exitcode == 0
    return dict(ret)


def test_partition_sequences_balances_tokens():
    lens = [8192, 1024, 4000, 4100, 7000, 1500, 3000, 2500]
    parts = partition_sequences(lens, 2)
    assert sorted(i for p in parts for i in p) == list(range(len(lens)))
    loads = [sum(lens[i] for i in p) for p in parts]
    assert abs(loads[0] - loads[1]) <= min(lens)
    assert [list(kv_head_range(8, 4, r)) for r in range(4)] == [[0, 1], [2, 3], [4, 5], [6, 7]]
    with pytest.raises(ValueError):
        kv_head_range(8, 3, 0)
    assert [list(context_slice(10, 4, r)) for r in range(4)] == [[0, 1, 2], [3, 4, 5], [6, 7, 8], [9]]


def _case():
    return make_decode_case(5, [300, 77, 1000, 16], 8, 2, 64, dtype=torch.bfloat16)


def _sequence_sharded(rank, world):
    c = _case()
    mine = partition_sequences(c.lens.tolist(), world)[rank]
    out = decode_oracle(c.q[mine], c.k_pool, c.v_pool, c.page_table[mine], c.lens[mine])
    gathered = [None] * world
    dist.all_gather_object(gathered, (mine, out))
    full = torch.zeros((len(c.lens),) + tuple(out.shape[1:]))
    for idx, o in gathered:
        full[idx] = o
    return full


def test_sequence_sharding_needs_no_collective_on_the_data_path():
    c = _case()
    ref = decode_oracle(c.q, c.k_pool, c.v_pool, c.page_table, c.lens)
    res = _run(_sequence_sharded)
    for r in range(2):
        assert torch.allclose(res[r], ref, atol=1e-6)


def _kv_head_sharded(rank, world):
    c = _case()
    hk = kv_head_range(2, world, rank)
    g = 8 // 2
    qh = slice(hk.start * g, hk.stop * g)
    out = decode_oracle(c.q[:, qh], c.k_pool[:, hk.start:hk.stop], c.v_pool[:, hk.start:hk.stop], c.page_table, c.lens)
    gathered = [None] * world
    dist.all_gather_object(gathered, out)
    return torch.cat(gathered, dim=1)


def test_kv_head_sharding():
    c = _case()
    ref = decode_oracle(c.q, c.k_pool, c.v_pool, c.page_table, c.lens)
    res = _run(_kv_head_sharded)
    assert torch.allclose(res[0], ref, atol=1e-6) and torch.allclose(res[1], ref, atol=1e-6)


def _context_sharded(rank, world):
    """Each rank owns a contiguous slice of every sequence's pages; partials -> all-gather -> combine."""
    c = _case()
    tpp = 16

    def partials():
        ms, ls, accs = [], [], []
        for s in range(len(c.lens)):
            L = int(c.lens[s])
            npg = (L + tpp - 1) // tpp
            sl = context_slice(npg, world, rank)
            local_len = max(0, min(L, sl.stop * tpp) - sl.start * tpp) if len(sl) else 0
            table = c.page_table[s:s + 1, sl.start:sl.stop] if len(sl) else torch.zeros((1, 1), dtype=torch.int32)
            m, l, acc = decode_partials_oracle(c.q[s:s + 1], c.k_pool, c.v_pool, table, torch.tensor([local_len]), 1 << 30)
            ms.append(m[:, :, 0]); ls.append(l[:, :, 0]); accs.append(acc[:, :, 0])
        return torch.cat(ms), torch.cat(ls), torch.cat(accs)

    return decode_context_parallel(partials, lse_combine_oracle_stack)


def lse_combine_oracle_stack(m_all, l_all, acc_all):
    # gathered stacks are [world, S, Hq(, D)]; the oracle merges along the last partition axis
    return lse_combine_oracle(m_all.permute(1, 2, 0), l_all.permute(1, 2, 0), acc_all.permute(1, 2, 0, 3))


def test_context_sharding_gather_and_combine():
    c = _case()
    ref = decode_oracle(c.q, c.k_pool, c.v_pool, c.page_table, c.lens)
    res = _run(_context_sharded)
    for r in range(2):
        assert torch.allclose(res[r], ref, atol=1e-5), (res[r] - ref).abs().max()


def _gather_shapes(rank, world):
    m = torch.full((3, 4), float(rank))
    l = torch.full((3, 4), 10.0 + rank)
    acc = torch.full((3, 4, 8), 100.0 + rank)
    m_all, l_all, acc_all = all_gather_partials(m, l, acc)
    return tuple(m_all.shape), tuple(acc_all.shape), m_all[:, 0, 0].tolist(), l_all[:, 0, 0].tolist(), acc_all[:, 0, 0, 0].tolist()


def test_all_gather_partials_layout():
    res = _run(_gather_shapes)
    assert res[0] == ((2, 3, 4), (2, 3, 4, 8), [0.0, 1.0], [10.0, 11.0], [100.0, 101.0])
    assert res[1] == res[0]


def _packed_partials(c, rank, world, q=None, tpp=16):
    """This rank's packed [rows, D + 2] partials (acc, m, l per row) over its slice of every sequence, from the oracle."""
    q = c.q if q is None else q
    rows = []
    for s in range(len(c.lens)):
        L = int(c.lens[s])
        npg = (L + tpp - 1) // tpp
        sl = context_slice(npg, world, rank)
        local_len = max(0, min(L, sl.stop * tpp) - sl.start * tpp) if len(sl) else 0
        table = c.page_table[s:s + 1, sl.start:sl.stop] if len(sl) else torch.zeros((1, 1), dtype=torch.int32)
        m, l, acc = decode_partials_oracle(q[s:s + 1], c.k_pool, c.v_pool, table, torch.tensor([local_len]), 1 << 30)
        rows.append(torch.cat([acc[0, :, 0], m[0, :, 0, None], l[0, :, 0, None]], dim=1))
    return torch.cat(rows).contiguous()


def _merge_packed(gathered, shape):
    d = gathered.shape[-1] - 2
    m, l, acc = gathered[:, :, d], gathered[:, :, d + 1], gathered[:, :, :d]
    return lse_combine_oracle(m.permute(1, 0), l.permute(1, 0), acc.permute(1, 0, 2)).reshape(shape)


def _context_sharded_packed(rank, world):
    from proxy_attention_lab_b200.sharding import all_gather_packed

    c = _case()
    out = decode_context_parallel(lambda: _packed_partials(c, rank, world), lambda g: _merge_packed(g, (len(c.lens), 8, 64)))
    # the collective writes into a caller-owned buffer when one is given
    buf = torch.empty((world, out.shape[0] * out.shape[1], 66))
    assert all_gather_packed(_packed_partials(c, rank, world), out=buf) is buf
    return out, _merge_packed(buf, (len(c.lens), 8, 64))


def test_context_sharding_packed_buffer_goes_through_one_collective():
    c = _case()
    ref = decode_oracle(c.q, c.k_pool, c.v_pool, c.page_table, c.lens)
    res = _run(_context_sharded_packed)
    for r in range(2):
        assert torch.allclose(res[r][0], ref, atol=1e-5) and torch.allclose(res[r][1], ref, atol=1e-5)


def _exchange_protocol(rank, world):
    """The fused exchange's protocol with host ranks: every rank stores its packed rows into slot
    [step & 1][rank] of EVERY rank's gather buffer (point-to-point sends stand for the peer stores), the receiver's
    flag for that source takes the step number once the rows have landed, and a rank merges a step only when all
    its flags show it.  Buffers and flags persist across steps; nothing is cleared in between."""
    c = _case()
    rows, d = len(c.lens) * 8, 64
    gather = torch.zeros((2, world, rows, d + 2))
    flags = [0] * world
    epoch = 0
    outs = []
    for it in range(4):
        g = torch.Generator().manual_seed(200 + it)
        q = torch.randn(c.q.shape, generator=g).to(torch.bfloat16)
        step = epoch + 1
        slot = step & 1
        mine = _packed_partials(c, rank, world, q=q)
        sends = [dist.isend(mine, dst=r) for r in range(world) if r != rank]
        gather[slot, rank] = mine
        flags[rank] = step
        for r in range(world):
            if r != rank:
                dist.recv(gather[slot, r], src=r)
                flags[r] = step
        for s in sends:
            s.wait()
        assert all(f - step >= 0 for f in flags)
        outs.append((q, _merge_packed(gather[slot], (len(c.lens), 8, d))))
        epoch = step
    return outs


def test_fused_exchange_protocol_on_host_ranks():
    c = _case()
    res = _run(_exchange_protocol)
    for r in range(2):
        for q, out in res[r]:
            ref = decode_oracle(q, c.k_pool, c.v_pool, c.page_table, c.lens)
            assert torch.allclose(out, ref, atol=1e-5), (out - ref).abs().max()
