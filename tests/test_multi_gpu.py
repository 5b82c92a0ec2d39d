"""Two ranks on two GPUs (NCCL): context-sharded long decode with the all-gather + LSE combine, and
kv-head sharding without any collective.  Skipped when fewer than two GPUs are visible."""

import os
import socket

import pytest
import torch

pytestmark = pytest.mark.gpu


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, ret):
    import torch.distributed as dist

    import proxy_attention_lab_b200 as pal
    from cases import make_decode_case
    from oracle import decode_oracle
    from proxy_attention_lab_b200.sharding import context_slice, decode_context_parallel, kv_head_range

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dev = torch.device("cuda", rank)
    torch.cuda.set_device(dev)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        tpp = 16
        c = make_decode_case(77, [5000, 1234, 16, 4097], 16, 4, 128, dtype=torch.bfloat16)
        ref = decode_oracle(c.q, c.k_pool, c.v_pool, c.page_table, c.lens)
        # --- context sharding: this rank sees only its slice of every sequence's pages ---
        S = len(c.lens)
        slices = [context_slice((int(L) + tpp - 1) // tpp, world, rank) for L in c.lens]
        width = max(max(len(s) for s in slices), 1)
        table = torch.zeros((S, width), dtype=torch.int32)
        local_len = torch.zeros(S, dtype=torch.int32)
        for s, sl in enumerate(slices):
            if len(sl):
                table[s, :len(sl)] = c.page_table[s, sl.start:sl.stop]
                local_len[s] = min(int(c.lens[s]), sl.stop * tpp) - sl.start * tpp
        q, kp, vp = c.q.to(dev), c.k_pool.to(dev), c.v_pool.to(dev)
        out = decode_context_parallel(
            lambda: pal.paged_attention_decode_partials(q, kp, vp, table.to(dev), local_len.to(dev), partition_pages=64),
            lambda m, l, a: pal.lse_combine(m, l, a, out_dtype=torch.bfloat16))
        def excess(o, r):
            # worst violation of "within 2e-3 or within one bf16 unit in the last place"
            diff = (o.float().cpu() - r).abs()
            return (diff - torch.maximum(torch.tensor(2e-3), r.abs() * 2.0 ** -7)).max().item()

        err_ctx = excess(out, ref)
        # --- kv-head sharding: no collective on the data path ---
        hk = kv_head_range(4, world, rank)
        g = 16 // 4
        o = pal.paged_attention_decode(q[:, hk.start * g:hk.stop * g].contiguous(), kp[:, hk.start:hk.stop].contiguous(),
                                       vp[:, hk.start:hk.stop].contiguous(), c.page_table.to(dev), c.lens.to(dev))
        err_head = excess(o, ref[:, hk.start * g:hk.stop * g])
        torch.cuda.synchronize()
        ret[rank] = (err_ctx, err_head)
    finally:
        dist.destroy_process_group()


def test_context_and_head_sharding_two_gpus():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp

    ctx = mp.get_context("spawn")
    ret = ctx.Manager().dict()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, ret)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(300)
        assert p.exitcode == 0
    for r in range(2):
        err_ctx, err_head = ret[r]
        assert err_ctx <= 0 and err_head <= 0, ret[r]
