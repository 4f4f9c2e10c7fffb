"""N > 1 host logic on CPU: world_size-2, 3 and 8 gloo groups exercise the row sharding and the
key-split exchange (all-gather + log-sum-exp combine) with the oracle standing in for the kernels."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from nanochat_b200.dist import KVSplitAttention, kv_shard_range, owned_below, shard_rows, sharded_prefill
from oracle import kv_oracle as O


def test_shard_rows_and_kv_ranges():
    assert [shard_rows(64, r, 8) for r in range(8)] == [(8 * r, 8 * r + 8) for r in range(8)]
    assert [shard_rows(10, r, 4) for r in range(4)] == [(0, 3), (3, 6), (6, 8), (8, 10)]
    with pytest.raises(ValueError):
        shard_rows(3, 0, 4)  # fewer rows than ranks
    with pytest.raises(ValueError):
        shard_rows(8, 4, 4)
    rng = [kv_shard_range(65536, r, 8) for r in range(8)]
    assert rng[0] == (0, 8192) and rng[-1] == (57344, 65536)
    assert all(a[1] == b[0] for a, b in zip(rng, rng[1:]))
    odd = [kv_shard_range(100, r, 3) for r in range(3)]
    assert odd == [(0, 64), (64, 100), (100, 100)]  # tile-aligned cuts; the last rank is empty
    assert all(b % 32 == 0 for b, _ in odd[:2])


def test_block_cyclic_ownership_counts():
    world, block = 4, 64
    for n in [0, 1, 63, 64, 65, 255, 256, 257, 1000, 4096]:
        counts = [owned_below(n, world, r, block) for r in range(world)]
        assert sum(counts) == n
        brute = [sum(1 for p in range(n) if (p // block) % world == r) for r in range(world)]
        assert counts == brute


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, B, Hq, Hkv, D, T, seqlens, window, ret):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        g = torch.Generator().manual_seed(7)  # identical data on every rank
        q = torch.randn(B, Hq, D, generator=g)
        kc = torch.randn(B, T, Hkv, D, generator=g)
        vc = torch.randn(B, T, Hkv, D, generator=g)
        lens = torch.tensor(seqlens, dtype=torch.int32)

        class OracleSplit(KVSplitAttention):
            """The exchange logic on CPU: the two kernel calls are replaced by the numpy oracle."""

            def _partial(self, q_, kc_, vc_, lens_, out_buf, lse_buf, push):
                o, l = O.attention_kvcache(q_.numpy()[:, None], kc_.numpy(), vc_.numpy(), lens_.numpy(),
                                           window_left=window, kv_begin=self.kv_begin, kv_end=self.kv_end)
                if self.kv_end <= self.kv_begin:
                    o[:], l[:] = 0.0, -np.inf
                out_buf.copy_(torch.from_numpy(o[:, 0]))
                lse_buf.copy_(torch.from_numpy(l[:, 0]))

            def _combine(self, po, pl):
                o, l = O.lse_combine(po.numpy(), pl.numpy())
                return torch.from_numpy(o), torch.from_numpy(l)

        att = OracleSplit(T, window_left=window, block=0)
        # poison the keys this rank does not own: the result must not depend on them
        kc_local, vc_local = kc.clone(), vc.clone()
        kc_local[:, :att.kv_begin] = 1e4
        kc_local[:, att.kv_end:] = -1e4
        out = att.attend(q, kc_local, vc_local, lens)
        full, _ = O.attention_kvcache(q.numpy()[:, None], kc.numpy(), vc.numpy(), lens.numpy(), window_left=window)
        err = float(np.abs(out.numpy() - full[:, 0]).max())
        gathered = [None] * world
        dist.all_gather_object(gathered, err)
        if rank == 0:
            ret.put(gathered)
    finally:
        dist.destroy_process_group()


def _cyclic_worker(rank, world, port, block, seqlens, ret):
    """Block-cyclic ownership: every rank attends over the keys it owns (stored compactly), partials are
    exchanged and combined; the kernels are replaced by the numpy oracle."""
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        B, Hq, Hkv, D, T = len(seqlens), 4, 2, 16, 160
        g = torch.Generator().manual_seed(3)
        q = torch.randn(B, Hq, D, generator=g)
        kc = torch.randn(B, T, Hkv, D, generator=g)
        vc = torch.randn(B, T, Hkv, D, generator=g)
        lens = torch.tensor(seqlens, dtype=torch.int32)
        mine = torch.tensor([p for p in range(T) if (p // block) % world == rank], dtype=torch.long)

        class OracleSplit(KVSplitAttention):
            def _partial(self, q_, kc_, vc_, lens_, out_buf, lse_buf, push):
                assert self.split == (world, rank, block) and not push
                local = torch.tensor([owned_below(int(L) + 1, world, rank, block) for L in lens_], dtype=torch.int32)
                # the oracle takes lengths before the new token; the local caches already hold it
                o, l = O.attention_kvcache(q_.numpy()[:, None], kc_.numpy(), vc_.numpy(), (local - 1).clamp(min=-1).numpy())
                empty = (local == 0).numpy()
                o[empty], l[empty] = 0.0, -np.inf
                out_buf.copy_(torch.from_numpy(o[:, 0]))
                lse_buf.copy_(torch.from_numpy(l[:, 0]))

            def _combine(self, po, pl):
                o, l = O.lse_combine(po.numpy(), pl.numpy())
                return torch.from_numpy(o), torch.from_numpy(l)

        att = OracleSplit(T, block=block)
        assert att.local_capacity == owned_below(T, world, rank, block) == mine.numel()
        out = att.attend(q, kc[:, mine].contiguous(), vc[:, mine].contiguous(), lens)
        full, _ = O.attention_kvcache(q.numpy()[:, None], kc.numpy(), vc.numpy(), lens.numpy())
        err = float(np.abs(out.numpy() - full[:, 0]).max())
        gathered = [None] * world
        dist.all_gather_object(gathered, err)
        if rank == 0:
            ret.put(gathered)
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world,block", [(2, 16), (3, 32), (8, 16)])
def test_block_cyclic_split_matches_unsplit_attention(world, block):
    ctx = mp.get_context("spawn")
    ret = ctx.Queue()
    port = _free_port()
    seqlens = [159, 3, 40, 95]  # row 1 lives on the first rank only
    procs = [ctx.Process(target=_cyclic_worker, args=(r, world, port, block, seqlens, ret)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(120)
        assert p.exitcode == 0
    errs = ret.get(timeout=10)
    assert len(errs) == world and max(errs) < 1e-5, errs


@pytest.mark.parametrize("world,window", [(2, -1), (2, 40), (3, -1)])
def test_kv_split_exchange_matches_unsplit_attention(world, window):
    ctx = mp.get_context("spawn")
    ret = ctx.Queue()
    port = _free_port()
    B, Hq, Hkv, D, T = 3, 4, 2, 16, 100
    seqlens = [99, 10, 63]  # row 1 leaves the later ranks without keys
    procs = [ctx.Process(target=_worker, args=(r, world, port, B, Hq, Hkv, D, T,
                                               seqlens, window, ret)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(120)
        assert p.exitcode == 0
    errs = ret.get(timeout=10)
    assert len(errs) == world and max(errs) < 1e-5, errs



def _prefill_worker(rank, world, port, ret):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from nanochat_b200.engine import KVCache
        from tests.cpu_backend import oracle_backend
        L, H, D, p, cap, rows_total = 3, 2, 16, 11, 20, 5
        lo, hi = shard_rows(rows_total, rank, world)
        g = torch.Generator().manual_seed(3)  # the same reference data on every rank (only rank 0 uses it as source)
        src_k = torch.randn(L, 1, p, H, D, generator=g)
        src_v = torch.randn(L, 1, p, H, D, generator=g)
        emb = torch.randn(1, 1, 8, generator=g)
        prompt = None
        if rank == 0:
            prompt = KVCache(batch_size=1, num_heads=H, seq_len=p, head_dim=D, num_layers=L, device="cpu", dtype=torch.float32)
            prompt.k_cache.copy_(src_k)
            prompt.v_cache.copy_(src_v)
            prompt.cache_seqlens.fill_(p)
            prompt.prev_embedding = emb.clone()
        local = KVCache(batch_size=hi - lo, num_heads=H, seq_len=cap, head_dim=D, num_layers=L, device="cpu", dtype=torch.float32)
        with oracle_backend():
            got_p = sharded_prefill(prompt, local, src=0)
        ok = got_p == p and local.cache_seqlens.tolist() == [p] * (hi - lo)
        ok = ok and torch.equal(local.k_cache[:, :, :p], src_k.expand(L, hi - lo, p, H, D))
        ok = ok and torch.equal(local.v_cache[:, :, :p], src_v.expand(L, hi - lo, p, H, D))
        ok = ok and float(local.k_cache[:, :, p:].abs().sum()) == 0.0
        ok = ok and torch.equal(local.prev_embedding, emb.expand(hi - lo, -1, -1))
        ret.put(bool(ok))
    finally:
        dist.destroy_process_group()


def test_sharded_prefill_fills_every_ranks_rows_from_one_broadcast():
    ctx = mp.get_context("spawn")
    ret = ctx.Queue()
    port = _free_port()
    world = 2
    procs = [ctx.Process(target=_prefill_worker, args=(r, world, port, ret)) for r in range(world)]
    for pr in procs:
        pr.start()
    for pr in procs:
        pr.join(120)
        assert pr.exitcode == 0
    assert all(ret.get(timeout=10) for _ in range(world))
