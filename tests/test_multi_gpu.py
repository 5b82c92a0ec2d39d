"""Context-sharded long decode across GPUs - all-gather (NCCL) + LSE combine in its two forms, and the fused
peer-store exchange - and kv-head sharding without any collective.  The two-rank test is skipped when fewer than two
GPUs are visible; the self-exchange test (one rank that publishes to itself) runs the fused kernel on one GPU."""

import os
import socket

import pytest
import torch

pytestmark = pytest.mark.gpu


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _local_slice(c, world, rank, tpp=16):
    """This rank's slice of every sequence's pages: (page table, local lengths)."""
    from proxy_attention_lab_b200.sharding import context_slice

    S = len(c.lens)
    slices = [context_slice((int(L) + tpp - 1) // tpp, world, rank) for L in c.lens]
    width = max(max(len(s) for s in slices), 1)
    table = torch.zeros((S, width), dtype=torch.int32)
    local_len = torch.zeros(S, dtype=torch.int32)
    for s, sl in enumerate(slices):
        if len(sl):
            table[s, :len(sl)] = c.page_table[s, sl.start:sl.stop]
            local_len[s] = min(int(c.lens[s]), sl.stop * tpp) - sl.start * tpp
    return table, local_len


def _worker(rank, world, port, ret):
    import torch.distributed as dist

    import proxy_attention_lab_b200 as pal
    from cases import make_decode_case, parity_report
    from oracle import decode_oracle
    from proxy_attention_lab_b200.sharding import ContextExchange, decode_context_parallel, kv_head_range

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    dev = torch.device("cuda", rank)
    torch.cuda.set_device(dev)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        c = make_decode_case(77, [5000, 1234, 16, 4097], 16, 4, 128, dtype=torch.bfloat16)
        ref = decode_oracle(c.q, c.k_pool, c.v_pool, c.page_table, c.lens)
        table, local_len = _local_slice(c, world, rank)
        q, kp, vp = c.q.to(dev), c.k_pool.to(dev), c.v_pool.to(dev)
        table_d, len_d = table.to(dev), local_len.to(dev)
        results = {}
        # --- context sharding, triple form: three tensors packed, gathered and unpacked on the host side ---
        out = decode_context_parallel(
            lambda: pal.paged_attention_decode_partials(q, kp, vp, table_d, len_d, partition_pages=64),
            lambda m, l, a: pal.lse_combine(m, l, a, out_dtype=torch.bfloat16))
        results["nccl_triple"] = parity_report(out, ref)
        # --- packed form: the kernel's buffer goes through one collective and is merged in place ---
        out_p = decode_context_parallel(
            lambda: pal.paged_attention_decode_partials(q, kp, vp, table_d, len_d, partition_pages=64, packed=True),
            lambda g: pal.lse_combine_packed(g, out_dtype=torch.bfloat16, out_shape=ref.shape))
        results["nccl_packed"] = parity_report(out_p, ref)
        results["packed_equals_triple"] = (bool(torch.equal(out_p, out)), "bitwise")
        # --- fused exchange: peer stores + flags inside the combine kernel, several steps with changing queries ---
        xchg = ContextExchange(rows=len(c.lens) * 16, head_dim=128, device=dev)
        for step in range(5):
            g = torch.Generator().manual_seed(100 + step)
            q_step = torch.randn(c.q.shape, generator=g).to(torch.bfloat16)
            ref_step = decode_oracle(q_step, c.k_pool, c.v_pool, c.page_table, c.lens)
            odt = torch.float32 if step % 2 else None
            out_x = xchg.decode(q_step.to(dev), kp, vp, table_d, len_d, partition_pages=64, out_dtype=odt)
            torch.cuda.synchronize()
            results[f"fused_step{step}"] = parity_report(out_x, ref_step)
        pal.check_status()
        out_x = xchg.decode(q, kp, vp, table_d, len_d, partition_pages=64)
        results["fused_equals_packed"] = (bool(torch.equal(out_x, out_p)), "bitwise")
        # --- kv-head sharding: no collective on the data path ---
        hk = kv_head_range(4, world, rank)
        g = 16 // 4
        o = pal.paged_attention_decode(q[:, hk.start * g:hk.stop * g].contiguous(), kp[:, hk.start:hk.stop].contiguous(),
                                       vp[:, hk.start:hk.stop].contiguous(), c.page_table.to(dev), c.lens.to(dev))
        results["kv_head"] = parity_report(o, ref[:, hk.start * g:hk.stop * g])
        torch.cuda.synchronize()
        dist.barrier()
        ret[rank] = results
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
        for name, (ok, msg) in ret[r].items():
            assert ok, (r, name, msg)


def _self_exchange_worker(port, ret):
    import torch.distributed as dist

    import proxy_attention_lab_b200 as pal
    from cases import make_decode_case, parity_report
    from oracle import decode_oracle
    from proxy_attention_lab_b200.sharding import ContextExchange

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    dist.init_process_group("nccl", rank=0, world_size=1, device_id=dev)
    try:
        results = {}
        xchg = ContextExchange(rows=3 * 64, head_dim=128, device=dev)
        for step, (lens, hq, hkv) in enumerate([([3000, 0, 77], 64, 8), ([129, 500], 16, 2), ([4096, 4096, 1], 32, 8)]):
            c = make_decode_case(80 + step, lens, hq, hkv, 128, dtype=torch.bfloat16 if step != 1 else torch.float16)
            ref = decode_oracle(c.q, c.k_pool, c.v_pool, c.page_table, c.lens)
            out = xchg.decode(c.q.to(dev), c.k_pool.to(dev), c.v_pool.to(dev), c.page_table.to(dev), c.lens.to(dev), partition_pages=32)
            two_pass = pal.paged_attention_decode(c.q.to(dev), c.k_pool.to(dev), c.v_pool.to(dev), c.page_table.to(dev), c.lens.to(dev),
                                                  partition_pages=32)
            torch.cuda.synchronize()
            results[f"step{step}"] = parity_report(out, ref)
            results[f"step{step}_vs_two_pass"] = (float((out.float() - two_pass.float()).abs().max()) <= 2e-3, "against the two-pass call")
        pal.check_status()
        ret[0] = results
    finally:
        dist.destroy_process_group()


def test_fused_exchange_with_a_single_rank():
    """world_size 1: the kernel publishes to its own buffer, raises and observes its own flag, advances the step number."""
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    import torch.multiprocessing as mp

    ctx = mp.get_context("spawn")
    ret = ctx.Manager().dict()
    p = ctx.Process(target=_self_exchange_worker, args=(_free_port(), ret))
    p.start()
    p.join(300)
    assert p.exitcode == 0
    for name, (ok, msg) in ret[0].items():
        assert ok, (name, msg)
