"""Multi-GPU forms of the decode path (one process per GPU, torch.distributed for the plumbing).

Two partitionings:

* by sequence (``shard_rows``): rows are independent, every rank owns a contiguous block of rows
  with its own KVCache and nothing crosses GPUs on the data path.  This is the replica-per-GPU
  form the reference itself serves with (scripts/chat_web.py:94-141).
* by key position for long context (``KVSplitAttention``): every rank holds a slice of the keys of
  every row, attends over it, and the partial results (normalised fp32 output + log-sum-exp per
  (row, q head); 66 KB per rank at B=8 x 16 heads) are exchanged with ONE all-gather and merged by
  the log-sum-exp combine kernel.  The reference has no counterpart (it never splits keys); the
  result equals a single softmax over all keys.

Two ownership layouts:
  ``block > 0``  block-cyclic (the default for full-causal attention): position p belongs to rank
                 (p / block) % N and is stored at local index (p / (block*N)) * block + p % block
                 of that rank's compact cache (capacity about T/N).  Ragged and growing rows stay
                 balanced across ranks; the new token is appended by its owner only.
  ``block == 0`` contiguous ranges [r*T/N, (r+1)*T/N) in a cache of full capacity (global token
                 indices, so sliding windows work); ranks are balanced only for rows of similar,
                 full length.
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


def sharded_prefill(prompt_cache, local_cache, group=None, src=0):
    """``KVCache.prefill`` (engine.py:123-137) when the sample rows are spread over ranks.

    Rank ``src`` holds the batch-1 cache of the prompt (``prompt_cache``; the others pass None).
    Its keys and values (and the smear state) are sent ONCE to every rank with a broadcast, land in
    that rank's own memory, and each rank then fills its own rows from the local copy with the
    broadcast-copy kernel -- no rank reads another GPU's memory inside a kernel.  ``local_cache``
    is this rank's (empty) KVCache for its share of the rows (``shard_rows``).  Returns the prompt
    length."""
    import torch.distributed as dist
    from .engine import KVCache
    rank = dist.get_rank(group)
    dev = local_cache.k_cache.device
    meta = torch.zeros(2, dtype=torch.int64, device=dev)
    if rank == src:
        assert prompt_cache is not None and prompt_cache.batch_size == 1, "the source is a batch-1 prompt cache"
        meta[0] = prompt_cache.get_pos()
        meta[1] = 0 if prompt_cache.prev_embedding is None else prompt_cache.prev_embedding.size(-1)
    dist.broadcast(meta, src=src, group=group)
    p, emb = int(meta[0]), int(meta[1])
    if rank == src:
        staged = prompt_cache
    else:
        staged = KVCache(batch_size=1, num_heads=local_cache.n_heads, seq_len=max(p, 1), head_dim=local_cache.head_dim,
                         num_layers=local_cache.n_layers, device=dev, dtype=local_cache.k_cache.dtype)
        staged.cache_seqlens.fill_(p)
        if emb:
            staged.prev_embedding = torch.empty(1, 1, emb, device=dev, dtype=local_cache.k_cache.dtype)
    if p > 0:
        # only the filled part of the source travels: (L, 1, p, H, D) for K and for V
        k_part = staged.k_cache[:, :, :p].contiguous()
        v_part = staged.v_cache[:, :, :p].contiguous()
        dist.broadcast(k_part, src=src, group=group)
        dist.broadcast(v_part, src=src, group=group)
        if rank != src:
            staged.k_cache[:, :, :p] = k_part
            staged.v_cache[:, :, :p] = v_part
    if emb:
        dist.broadcast(staged.prev_embedding, src=src, group=group)
    local_cache.prefill(staged)
    return p


def kv_shard_range(capacity, rank, world_size, align=32):
    """Key range [begin, end) of ``rank`` in the contiguous layout: equal ranges, boundaries rounded
    up to a multiple of ``align`` tokens.  (Any boundary is correct: a shard's tiles start at its own
    first key.  The rounding only keeps the ranges tidy.)"""
    if not 0 <= rank < world_size:
        raise ValueError(f"rank {rank} outside world of {world_size}")
    per = -(-capacity // world_size)
    per = -(-per // align) * align
    begin = min(capacity, rank * per)
    return begin, min(capacity, begin + per)


def owned_below(n, world_size, rank, block):
    """Positions p < n owned by ``rank`` in the block-cyclic layout (host-side twin of the kernel)."""
    cycle = block * world_size
    full, rem = divmod(n, cycle)
    return full * block + min(max(rem - rank * block, 0), block)


class KVSplitAttention:
    """Decode attention with the keys split across the ranks of ``group``.

    ``attend(q, k_cache, v_cache, cache_seqlens)`` — q (B, Hq, D) replicated on every rank, caches
    in this rank's layout (see module docstring), cache_seqlens the GLOBAL lengths before the new
    token — returns the full attention output (B, Hq, D) bf16 on every rank.
    ``append_and_attend`` first runs the fused RoPE/norm/append for the rows this rank owns.

    Kernels per step in the block-cyclic layout with ``exchange="p2p"``: append (works out the owner
    and the local slot itself), streaming attention over the local part (works out the local
    lengths itself), merge of the split partials (stores every finished row into all peers'
    exchange buffers and releases the step's flags), wait + combine.  With ``exchange="nccl"`` the
    third kernel only fills the local send buffer and an all-gather plus the combine kernel follow.
    """

    def __init__(self, capacity, group=None, window_left=-1, block=1024, exchange="nccl"):
        import torch.distributed as dist
        self.dist = dist
        self.group = group
        # without a process group this is the single-rank case (same kernels, no exchange)
        alone = not (dist.is_available() and dist.is_initialized())
        self.rank = 0 if alone else dist.get_rank(group)
        self.world = 1 if alone else dist.get_world_size(group)
        self.capacity = capacity
        self.window_left = window_left
        if block and window_left >= 0:
            raise ValueError("the block-cyclic layout stores keys compactly and cannot express a sliding window; "
                             "use block=0 (contiguous ranges) for windowed layers")
        if block < 0:
            raise ValueError("block must be positive (block-cyclic) or 0 (contiguous ranges)")
        self.block = block
        if block:
            self.kv_begin = self.kv_end = 0
            self.local_capacity = owned_below(capacity, self.world, self.rank, block)
        else:
            self.kv_begin, self.kv_end = kv_shard_range(capacity, self.rank, self.world)
            self.local_capacity = capacity
        self._gather = self._send = None
        if exchange not in ("nccl", "p2p"):
            raise ValueError("exchange must be 'nccl' (all-gather + combine kernel) or 'p2p' (peer-memory push + "
                             "wait/combine kernel)")
        self.exchange = exchange if self.world > 1 else "nccl"
        self._symm = self._peer_ptrs = None
        self.wait_limit_ns = 0  # 0 = the library default (2 s)

    @property
    def split(self):
        """(world, rank, block) as the *_split kernels take it."""
        return self.world, self.rank, self.block

    # ---- buffers: [rows*D output | rows lse] per rank, padded to a multiple of 4 floats ----------
    def _buffers(self, rows, D, device):
        per = rows * D + -(-rows // 4) * 4
        if self._gather is None or self._gather.numel() != self.world * per or self._gather.device != device:
            self._gather = torch.empty(self.world, per, dtype=torch.float32, device=device)
            self._send = torch.empty(per, dtype=torch.float32, device=device)
        return self._send[:rows * D], self._send[rows * D:rows * D + rows]

    def _partial(self, q, k_cache, v_cache, cache_seqlens, out_f32, lse, push):
        """This rank's normalised partial output and log-sum-exp into out_f32 / lse; with ``push`` the
        same kernels also deliver them to every peer (block-cyclic layout only)."""
        if self.block:
            ops.decode_attention_split(q, k_cache, v_cache, cache_seqlens, self.split, out_f32, lse, seqlen_offset=1,
                                       peer_ptrs=self._peer_ptrs if push else None,
                                       step_counter=self._step_ctr if push else None)
        elif self.kv_end <= self.kv_begin:  # more ranks than tiles: this rank has nothing
            out_f32.zero_()
            lse.fill_(float("-inf"))
        else:
            ops.decode_attention(q, k_cache, v_cache, cache_seqlens, seqlen_offset=1, window_left=self.window_left,
                                 kv_begin=self.kv_begin, kv_end=self.kv_end, partial=True, out_f32=out_f32, lse=lse)

    def _combine(self, parts_o, parts_lse):
        return ops.lse_combine(parts_o, parts_lse)

    def append_and_attend(self, q, k, v, k_cache, v_cache, cache_seqlens, cos, sin):
        """q, k, v: (B, 1, H, D) raw projections.  RoPE/QK-norm/scale on q and k (positions are the
        global lengths), the owner of position L_b stores k/v, then ``attend``."""
        if self.block:
            q2 = ops.append_rope_norm(q, k, v, k_cache, v_cache, cache_seqlens, cos, sin, split=self.split)
        else:  # global indices: every rank may write, only the owner's range is ever read
            q2 = ops.append_rope_norm(q, k, v, k_cache, v_cache, cache_seqlens, cos, sin)
        return self.attend(q2[:, 0], k_cache, v_cache, cache_seqlens)

    def attend(self, q, k_cache, v_cache, cache_seqlens):
        B, Hq, D = q.shape
        rows = B * Hq
        out_f32, lse = self._buffers(rows, D, q.device)
        p2p = self.exchange == "p2p"
        if p2p and (self._symm is None or self._p2p_rows != rows):
            self._setup_p2p(rows, D, q.device)
        fused_push = p2p and bool(self.block)
        self._partial(q, k_cache, v_cache, cache_seqlens, out_f32.view(B, Hq, D), lse.view(B, Hq), fused_push)
        if self.world == 1:
            return self._combine(out_f32.view(1, rows, D), lse.view(1, rows))[0].view(B, Hq, D)
        if p2p:
            return self._exchange_p2p(rows, D, q.device, pushed=fused_push).view(B, Hq, D)
        self.dist.all_gather_into_tensor(self._gather.view(-1), self._send, group=self.group)
        parts_o = self._gather[:, :rows * D].unflatten(1, (rows, D))
        parts_lse = self._gather[:, rows * D:rows * D + rows]
        out, _ = self._combine(parts_o, parts_lse)
        return out.view(B, Hq, D)

    # ---- exchange over NVLink peer memory (no collective library on the data path) ---------------
    def _setup_p2p(self, rows, D, device):
        import ctypes
        import torch.distributed._symmetric_memory as symm_mem
        from . import _lib
        nbytes = _lib.lib.nckv_p2p_buffer_bytes(self.world, rows, D)
        if nbytes == 0:
            raise RuntimeError(f"p2p exchange: unsupported shape (world={self.world}, rows={rows}, D={D})")
        buf = symm_mem.empty((nbytes + 3) // 4, dtype=torch.float32, device=device)
        buf.zero_()
        hdl = symm_mem.rendezvous(buf, self.group if self.group is not None else self.dist.group.WORLD)
        ptrs = (ctypes.c_void_p * self.world)(*[int(p) for p in hdl.buffer_ptrs])
        torch.cuda.synchronize(device)
        self.dist.barrier(group=self.group)  # every buffer is zeroed before anyone pushes
        self._symm, self._symm_hdl, self._peer_ptrs, self._p2p_rows = buf, hdl, ptrs, rows
        self._p2p_out = torch.empty(rows, D, dtype=torch.bfloat16, device=device)
        self._step_ctr = torch.zeros(2, dtype=torch.int32, device=device)  # [step, finished blocks]

    def _exchange_p2p(self, rows, D, device, pushed):
        from . import _lib
        idx = device.index if device.index is not None else torch.cuda.current_device()
        stream = torch.cuda.current_stream(idx).cuda_stream
        ws = ops.workspace(device, 1, 1, 1)
        if not pushed:
            _lib.call("nckv_p2p_push", self._send.data_ptr(), rows, D, self._peer_ptrs, self.world, self.rank,
                      self._step_ctr.data_ptr(), stream)
        _lib.call("nckv_p2p_wait_combine", self._symm.data_ptr(), self.world, rows, D, self._step_ctr.data_ptr(),
                  self._p2p_out.data_ptr(), None, ws.data_ptr(), self.wait_limit_ns, stream)
        return self._p2p_out
