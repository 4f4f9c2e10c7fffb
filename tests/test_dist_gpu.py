"""Key-split decode attention across 2 GPUs (NCCL all-gather + LSE combine) against the oracle.
Needs two CUDA devices; skipped otherwise."""
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
        att = KVSplitAttention(T)
        kd, vd = kc.to(dev), vc.to(dev)
        kd[:, :att.kv_begin] = float("nan")  # keys of other ranks must never be read here
        kd[:, att.kv_end:] = float("nan")
        out = att.attend(q.to(dev), kd, vd, lens.to(dev))
        torch.cuda.synchronize()
        status = ops.read_status(dev)
        full, _ = O.attention_kvcache(q.float().numpy()[:, None], kc.float().numpy(), vc.float().numpy(), lens.numpy())
        err = float(np.abs(out.float().cpu().numpy() - full[:, 0]).max() / np.abs(full).max())
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
