"""Key-split decode attention across 2 GPUs (NCCL all-gather + LSE combine, and the peer-memory
exchange fused into the attention kernels) against the oracle.  Needs two CUDA devices; skipped otherwise."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, ret):
    import torch.distributed as dist
    from nanochat_b200 import ops
    from nanochat_b200.dist import KVSplitAttention
    from oracle import kv_oracle as O
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        B, Hq, Hkv, T = 4, 16, 4, 4096
        g = torch.Generator().manual_seed(11)  # identical data on every rank
        q = torch.randn(B, Hq, 128, generator=g).to(torch.bfloat16)
        kc = torch.randn(B, T, Hkv, 128, generator=g).to(torch.bfloat16)
        vc = torch.randn(B, T, Hkv, 128, generator=g).to(torch.bfloat16)
        lens = torch.tensor([4095, 2047, 100, 3000], dtype=torch.int32)
        # (1) contiguous ranges in a full-capacity cache
        att = KVSplitAttention(T, block=0)
        kd, vd = kc.to(dev), vc.to(dev)
        kd[:, :att.kv_begin] = float("nan")  # keys of other ranks must never be read here
        kd[:, att.kv_end:] = float("nan")
        out = att.attend(q.to(dev), kd, vd, lens.to(dev))
        torch.cuda.synchronize()
        full, _ = O.attention_kvcache(q.float().numpy()[:, None], kc.float().numpy(), vc.float().numpy(), lens.numpy())
        err = float(np.abs(out.float().cpu().numpy() - full[:, 0]).max() / np.abs(full).max())
        # (2) block-cyclic ownership in compact caches, including the owner-only append of the new token
        from oracle import torch_ref as R
        block = 256
        att2 = KVSplitAttention(T, block=block)
        owner = (torch.arange(T) // block) % world
        mine = (owner == rank).nonzero()[:, 0]
        kl = torch.full((B, att2.local_capacity, Hkv, 128), float("nan"), dtype=torch.bfloat16)
        vl = kl.clone()
        for b_, L_ in enumerate(lens.tolist()):  # rows hold their first L keys; the rest stays NaN
            keep = mine[mine < L_]
            kl[b_, :keep.numel()] = kc[b_, keep]
            vl[b_, :keep.numel()] = vc[b_, keep]
        cos, sin = R.rotary_tables(T, 128, "cpu", torch.bfloat16)
        q_raw = torch.randn(B, 1, Hq, 128, generator=g).to(torch.bfloat16)
        k_raw = torch.randn(B, 1, Hkv, 128, generator=g).to(torch.bfloat16)
        v_raw = torch.randn(B, 1, Hkv, 128, generator=g).to(torch.bfloat16)
        out2 = att2.append_and_attend(q_raw.to(dev), k_raw.to(dev), v_raw.to(dev), kl.to(dev), vl.to(dev), lens.to(dev),
                                      cos.to(dev), sin.to(dev))
        torch.cuda.synchronize()
        kc2, vc2 = kc.clone(), vc.clone()  # single-device reference: same append, full attention
        q2 = R.rope_norm_scale_rows(q_raw, cos, sin, lens)
        k2 = R.rope_norm_scale_rows(k_raw, cos, sin, lens)
        for b_, L_ in enumerate(lens.tolist()):
            kc2[b_, L_] = k2[b_, 0]
            vc2[b_, L_] = v_raw[b_, 0]
        full2, _ = O.attention_kvcache(q2.float().numpy(), kc2.float().numpy(), vc2.float().numpy(), lens.numpy())
        err2 = float(np.abs(out2.float().cpu().numpy() - full2[:, 0]).max() / np.abs(full2).max())
        err = max(err, err2)
        # (3) the same with the exchange over peer memory instead of NCCL, several steps in a row
        att3 = KVSplitAttention(T, block=block, exchange="p2p")
        for step in range(3):
            lens3 = (lens - step * 7).clamp(min=0)
            kl3 = torch.full((B, att3.local_capacity, Hkv, 128), float("nan"), dtype=torch.bfloat16)
            vl3 = kl3.clone()
            for b_, L_ in enumerate((lens3 + 1).tolist()):
                keep = mine[mine < L_]
                kl3[b_, :keep.numel()] = kc[b_, keep]
                vl3[b_, :keep.numel()] = vc[b_, keep]
            out3 = att3.attend(q.to(dev), kl3.to(dev), vl3.to(dev), lens3.to(dev))
            torch.cuda.synchronize()
            full3, _ = O.attention_kvcache(q.float().numpy()[:, None], kc.float().numpy(), vc.float().numpy(), lens3.numpy())
            err = max(err, float(np.abs(out3.float().cpu().numpy() - full3[:, 0]).max() / np.abs(full3).max()))
        # (3b) the whole fused step over peer memory: owner-only append inside the append kernel, local
        # lengths inside the attention kernel, push inside the merge kernel, then wait + combine
        out4 = att3.append_and_attend(q_raw.to(dev), k_raw.to(dev), v_raw.to(dev), kl.to(dev), vl.to(dev), lens.to(dev),
                                      cos.to(dev), sin.to(dev))
        torch.cuda.synchronize()
        err = max(err, float(np.abs(out4.float().cpu().numpy() - full2[:, 0]).max() / np.abs(full2).max()))
        assert torch.equal(out4.view(torch.int16), out2.view(torch.int16)) or err <= 1e-2
        # (4) prefill broadcast with the sample rows sharded over the ranks: the prompt cache of rank 0
        # is broadcast once, every rank fills its own rows from its local copy (kernel (c))
        from nanochat_b200.dist import shard_rows, sharded_prefill
        from nanochat_b200.engine import KVCache
        Lyr, Hh, pp, cap, rows_total = 3, 4, 777, 1024, 9
        gp = torch.Generator().manual_seed(5)
        src_k = torch.randn(Lyr, 1, pp, Hh, 128, generator=gp).to(torch.bfloat16)
        src_v = torch.randn(Lyr, 1, pp, Hh, 128, generator=gp).to(torch.bfloat16)
        emb = torch.randn(1, 1, 64, generator=gp).to(torch.bfloat16)
        prompt = None
        if rank == 0:
            prompt = KVCache(batch_size=1, num_heads=Hh, seq_len=pp, head_dim=128, num_layers=Lyr, device=dev, dtype=torch.bfloat16)
            prompt.k_cache.copy_(src_k)
            prompt.v_cache.copy_(src_v)
            prompt.cache_seqlens.fill_(pp)
            prompt.prev_embedding = emb.to(dev)
        lo, hi = shard_rows(rows_total, rank, world)
        local = KVCache(batch_size=hi - lo, num_heads=Hh, seq_len=cap, head_dim=128, num_layers=Lyr, device=dev, dtype=torch.bfloat16)
        got_p = sharded_prefill(prompt, local, src=0)
        torch.cuda.synchronize()
        same = (got_p == pp and local.cache_seqlens.tolist() == [pp] * (hi - lo)
                and torch.equal(local.k_cache[:, :, :pp].cpu().view(torch.int16), src_k.expand(Lyr, hi - lo, pp, Hh, 128).contiguous().view(torch.int16))
                and torch.equal(local.v_cache[:, :, :pp].cpu().view(torch.int16), src_v.expand(Lyr, hi - lo, pp, Hh, 128).contiguous().view(torch.int16))
                and torch.equal(local.prev_embedding.cpu(), emb.expand(hi - lo, -1, -1)))
        if not same:
            err = float("inf")
        status = ops.read_status(dev)
        res = [None] * world
        dist.all_gather_object(res, (err, status))
        if rank == 0:
            ret.put(res)
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_kv_split_attention_two_gpus():
    ctx = mp.get_context("spawn")
    ret = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, ret)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(300)
        assert p.exitcode == 0
    res = ret.get(timeout=10)
    assert all(st == 0 for _, st in res), res
    assert max(e for e, _ in res) <= 1e-2, res
