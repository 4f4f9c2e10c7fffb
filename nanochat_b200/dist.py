"""Multi-GPU forms of the decode path (one process per GPU, torch.distributed for the plumbing).

Two partitionings, both from BASELINE.json's north star:

* by sequence (``shard_rows``): rows are independent, every rank owns a contiguous block of rows
  with its own KVCache and nothing crosses GPUs on the data path.  This is the replica-per-GPU
  form the reference itself serves with (scripts/chat_web.py:94-141).
* by key range for long context (``KVSplitAttention``): rank r attends over keys
  [r*T/N, (r+1)*T/N) of every row and the partial results (normalised fp32 output + log-sum-exp per
  (row, q head), 66 KB per rank at B=8 x 16 heads) are exchanged with ONE all-gather and merged by
  the log-sum-exp combine kernel.  The reference has no counterpart (it never splits keys); the
  result equals a single softmax over all keys.

Each rank keeps a cache of full capacity but only reads (and needs valid data in) its own key
range; the append kernel writes the new token on every rank, which is harmless outside the owner's
range and keeps positions and windows in global token indices.
"""
import torch

from . import ops


def shard_rows(n_rows, rank, world_size):
    """Contiguous block [lo, hi) of rows for ``rank``; the first ``n_rows % world_size`` ranks get
    one extra row.  Raises if a rank would be left without rows."""
    if not 0 <= rank < world_size:
        raise ValueError(f"rank {rank} outside world of {world_size}")
    if n_rows < world_size:
        raise ValueError(f"{n_rows} rows cannot be sharded over {world_size} ranks")
    q, r = divmod(n_rows, world_size)
    lo = rank * q + min(rank, r)
    return lo, lo + q + (1 if rank < r else 0)


def kv_shard_range(capacity, rank, world_size, align=32):
    """Key range [begin, end) of ``rank``: equal contiguous ranges, boundaries rounded up to a
    multiple of ``align`` tokens (the decode kernel's tile) so no tile straddles two ranks."""
    if not 0 <= rank < world_size:
        raise ValueError(f"rank {rank} outside world of {world_size}")
    per = -(-capacity // world_size)
    per = -(-per // align) * align
    begin = min(capacity, rank * per)
    return begin, min(capacity, begin + per)


class KVSplitAttention:
    """Decode attention with the keys split across the ranks of ``group``.

    ``attend(q, k_cache, v_cache, cache_seqlens)`` — q (B, Hq, D) replicated on every rank,
    caches (B, T_max, Hkv, D) holding at least this rank's key range, cache_seqlens the global
    lengths BEFORE the new token — returns the full attention output (B, Hq, D) bf16 on every rank.
    """

    def __init__(self, capacity, group=None, window_left=-1, partial_fn=None, combine_fn=None):
        import torch.distributed as dist
        self.dist = dist
        self.group = group
        self.rank = dist.get_rank(group)
        self.world = dist.get_world_size(group)
        self.capacity = capacity
        self.window_left = window_left
        self.kv_begin, self.kv_end = kv_shard_range(capacity, self.rank, self.world)
        # injectable for CPU tests of the exchange logic; the product path is the CUDA ops
        self._partial = partial_fn or self._partial_cuda
        self._combine = combine_fn or ops.lse_combine
        self._gather = None

    def _partial_cuda(self, q, k_cache, v_cache, cache_seqlens):
        if self.kv_end <= self.kv_begin:  # more ranks than tiles: this rank has nothing
            B, Hq, D = q.shape
            return (torch.zeros(B, Hq, D, dtype=torch.float32, device=q.device),
                    torch.full((B, Hq), float("-inf"), dtype=torch.float32, device=q.device))
        _, o32, lse = ops.decode_attention(q, k_cache, v_cache, cache_seqlens, seqlen_offset=1,
                                           window_left=self.window_left, kv_begin=self.kv_begin, kv_end=self.kv_end,
                                           partial=True)
        return o32, lse

    def attend(self, q, k_cache, v_cache, cache_seqlens):
        B, Hq, D = q.shape
        rows = B * Hq
        o32, lse = self._partial(q, k_cache, v_cache, cache_seqlens)
        if o32.shape != (B, Hq, D) or lse.shape != (B, Hq):
            raise RuntimeError(f"partial result has shape {tuple(o32.shape)} / {tuple(lse.shape)}, expected "
                               f"{(B, Hq, D)} / {(B, Hq)}")
        if self.world == 1:
            return self._combine(o32.view(1, rows, D), lse.view(1, rows))[0].view(B, Hq, D)
        # one packed message per rank: [rows*D output | rows lse], padded to a multiple of 4 floats
        per = rows * D + -(-rows // 4) * 4
        if self._gather is None or self._gather.numel() != self.world * per or self._gather.device != q.device:
            self._gather = torch.empty(self.world, per, dtype=torch.float32, device=q.device)
            self._send = torch.empty(per, dtype=torch.float32, device=q.device)
        self._send[:rows * D].copy_(o32.reshape(-1))
        self._send[rows * D:rows * D + rows].copy_(lse.reshape(-1))
        self.dist.all_gather_into_tensor(self._gather.view(-1), self._send, group=self.group)
        parts_o = self._gather[:, :rows * D].unflatten(1, (rows, D))
        parts_lse = self._gather[:, rows * D:rows * D + rows]
        out, _ = self._combine(parts_o, parts_lse)
        return out.view(B, Hq, D)
