"""KV cache with the reference's interface (nanochat/engine.py:82-137), storage on the GPU.

``KVCache`` keeps the reference's constructor, attributes (``k_cache`` / ``v_cache`` of shape
(n_layers, B, T_max, Hkv, D), int32 ``cache_seqlens``, ``prev_embedding``) and methods
(``reset / get_pos / get_layer_cache / advance / prefill``).  Bookkeeping is integer tensor
arithmetic and works on any device; ``prefill`` — the batch-1 -> num_samples broadcast — is the
CUDA copy kernel of libnckv and raises for non-CUDA caches (there is no CPU path).
"""
import signal
import warnings
from collections import deque

import torch
import torch.nn.functional as F

from . import ops


class KVCache:
    """Pre-allocated per-layer K/V storage plus per-row lengths (engine.py:82-104)."""

    def __init__(self, batch_size, num_heads, seq_len, head_dim, num_layers, device, dtype):
        self.batch_size = batch_size
        self.max_seq_len = seq_len
        self.n_layers = num_layers
        self.n_heads = num_heads
        self.head_dim = head_dim
        shape = (num_layers, batch_size, seq_len, num_heads, head_dim)
        # zero-filled like the reference: rows past cache_seqlens are never attended, but a
        # zeroed cache keeps byte-for-byte comparisons against the reference meaningful
        self.k_cache = torch.zeros(shape, device=device, dtype=dtype)
        self.v_cache = torch.zeros(shape, device=device, dtype=dtype)
        self.cache_seqlens = torch.zeros(batch_size, dtype=torch.int32, device=device)
        self.prev_embedding = None  # smear state owned by the model's forward pass

    def reset(self):
        """Empty the cache (engine.py:106-109); storage is kept."""
        self.cache_seqlens.zero_()
        self.prev_embedding = None

    def get_pos(self):
        """Length of row 0 as a Python int (engine.py:111-113). This synchronises with the device;
        the kernels never call it — they read ``cache_seqlens`` on the device, per row."""
        return int(self.cache_seqlens[0].item())

    def get_layer_cache(self, layer_idx):
        """(k_cache, v_cache) views of one layer, each (B, T_max, Hkv, D) (engine.py:115-117)."""
        return self.k_cache[layer_idx], self.v_cache[layer_idx]

    def advance(self, num_tokens):
        """cache_seqlens += num_tokens for every row (engine.py:119-121)."""
        self.cache_seqlens += num_tokens

    def prefill(self, other):
        """Broadcast a batch-1 prompt cache into every row of this (empty) cache (engine.py:123-137).

        Same preconditions as the reference: this cache is empty, layer/head/dim counts agree and
        it is at least as long as ``other``.  One kernel launch copies K and V of all layers and
        sets ``cache_seqlens`` to the prompt length; ``prev_embedding`` is expanded to B rows.
        """
        assert self.get_pos() == 0, "Cannot prefill a non-empty KV cache"
        assert self.n_layers == other.n_layers and self.n_heads == other.n_heads and self.head_dim == other.head_dim
        assert self.max_seq_len >= other.max_seq_len
        assert other.batch_size == 1, "prefill broadcasts a batch-1 cache"
        other_pos = other.get_pos()
        ops.prefill_broadcast(other.k_cache, other.v_cache, self.k_cache, self.v_cache, self.cache_seqlens, other_pos)
        if other.prev_embedding is not None:
            self.prev_embedding = other.prev_embedding.expand(self.batch_size, -1, -1).clone()


class PagedKVCache:
    """KV storage in pages with a per-row block table: the compact successor of the dense
    (n_layers, B, T_max, Hkv, D) tensors of engine.py:98-100, behind the same methods.

    ``k_cache`` / ``v_cache`` are pools of shape (n_layers, n_pages, page_tokens, Hkv, D);
    ``block_table`` is int32 (B, max_pages): token t of row b lives in page ``block_table[b, t //
    page_tokens]``.  Pages are handed out from a free list on the host, ahead of need: ``reserve(n)``
    makes every row able to hold n tokens (the caller knows an upper bound of every row's length; the
    device-side ``cache_seqlens`` is never read back for this).  What the format buys:
      * rows take pages as they grow, so ``n_pages`` can be sized for the tokens a batch really holds
        instead of B x T_max;
      * ``prefill`` shares the prompt: the pages that hold a whole page of prompt tokens are written
        once and referenced by every row's table; only the page with the prompt's tail is copied per
        row (rows append there).  Shared pages are never written again, so no copy-on-write is needed.
    CUDA only: the kernels that read and write through the table have no CPU implementation."""

    paged = True

    def __init__(self, batch_size, num_heads, seq_len, head_dim, num_layers, device, dtype, page_tokens=192,
                 n_pages=None):
        if page_tokens % ops.PAGE_TILE:
            raise ValueError(f"page_tokens must be a multiple of {ops.PAGE_TILE}")
        self.batch_size = batch_size
        self.max_seq_len = seq_len
        self.n_layers = num_layers
        self.n_heads = num_heads
        self.head_dim = head_dim
        self.page_tokens = page_tokens
        self.max_pages = -(-seq_len // page_tokens)
        self.n_pages = n_pages if n_pages is not None else batch_size * self.max_pages
        shape = (num_layers, self.n_pages, page_tokens, num_heads, head_dim)
        # not zero-filled: nothing beyond cache_seqlens is ever attended
        self.k_cache = torch.empty(shape, device=device, dtype=dtype)
        self.v_cache = torch.empty(shape, device=device, dtype=dtype)
        self.cache_seqlens = torch.zeros(batch_size, dtype=torch.int32, device=device)
        self.block_table = torch.full((batch_size, self.max_pages), -1, dtype=torch.int32, device=device)
        self._table_host = torch.full((batch_size, self.max_pages), -1, dtype=torch.int32)
        if torch.device(device).type == "cuda":
            self._table_host = self._table_host.pin_memory()
        self._free = list(range(self.n_pages - 1, -1, -1))
        self._count = [0] * batch_size   # pages in each row's table, shared ones included
        self._shared = 0                 # leading pages of every row that all rows share
        self.prev_embedding = None

    # ---- the reference's KVCache methods -------------------------------------------------------
    def reset(self):
        self._free = list(range(self.n_pages - 1, -1, -1))
        self._count = [0] * self.batch_size
        self._shared = 0
        self._table_host.fill_(-1)
        self.block_table.fill_(-1)
        self.cache_seqlens.zero_()
        self.prev_embedding = None

    def get_pos(self):
        return int(self.cache_seqlens[0].item())

    def get_layer_cache(self, layer_idx):
        """(k_pool, v_pool) of one layer, each (n_pages, page_tokens, Hkv, D)."""
        return self.k_cache[layer_idx], self.v_cache[layer_idx]

    def advance(self, num_tokens):
        self.cache_seqlens += num_tokens

    # ---- page bookkeeping (host) ---------------------------------------------------------------
    def pages_in_use(self):
        return self.n_pages - len(self._free)

    def _take(self, n):
        if n > len(self._free):
            raise RuntimeError(f"PagedKVCache: page pool of {self.n_pages} pages exhausted ({n} more pages needed, "
                               f"{len(self._free)} free)")
        taken = self._free[len(self._free) - n:]
        del self._free[len(self._free) - n:]
        taken.reverse()
        return taken

    def reserve(self, n_tokens):
        """Give every row the pages for positions < n_tokens.  Cheap when nothing has to be added."""
        need = -(-min(n_tokens, self.max_pages * self.page_tokens) // self.page_tokens)
        lo = min(self._count)
        if lo >= need:
            return
        if lo == max(self._count):  # the usual case: rows grow in lock step, one block of table columns
            fresh = self._take(self.batch_size * (need - lo))
            self._table_host[:, lo:need] = torch.tensor(fresh, dtype=torch.int32).view(self.batch_size, need - lo)
            self._count = [need] * self.batch_size
        else:
            for b, have in enumerate(self._count):
                if have < need:
                    self._table_host[b, have:need] = torch.tensor(self._take(need - have), dtype=torch.int32)
                    self._count[b] = need
        self.block_table.copy_(self._table_host, non_blocking=True)

    def prefill(self, other):
        """KVCache.prefill (engine.py:123-137) from a dense batch-1 prompt cache, sharing the prompt's
        full pages between the rows."""
        assert self.pages_in_use() == 0 and max(self._count) == 0, "Cannot prefill a non-empty KV cache"
        assert self.n_layers == other.n_layers and self.n_heads == other.n_heads and self.head_dim == other.head_dim
        assert self.max_seq_len >= other.max_seq_len
        assert other.batch_size == 1 and not getattr(other, "paged", False), "prefill takes a dense batch-1 cache"
        p = other.get_pos()
        pt = self.page_tokens
        n_full, tail = divmod(p, pt)
        B = self.batch_size
        pages = torch.tensor(self._take(n_full + (B if tail else 0)), dtype=torch.int32)
        shared, private = pages[:n_full], pages[n_full:]
        jobs = torch.empty(pages.numel(), 3, dtype=torch.int32)
        jobs[:, 0] = pages
        jobs[:n_full, 1] = torch.arange(n_full, dtype=torch.int32) * pt
        jobs[:n_full, 2] = pt
        jobs[n_full:, 1] = n_full * pt
        jobs[n_full:, 2] = tail
        self._table_host[:, :n_full] = shared
        if tail:
            self._table_host[:, n_full] = private
        self._shared = n_full
        self._count = [n_full + (1 if tail else 0)] * B
        self.block_table.copy_(self._table_host, non_blocking=True)
        if pages.numel():
            ops.paged_fill(other.k_cache, other.v_cache, self.k_cache, self.v_cache, jobs.to(self.block_table.device))
        self.cache_seqlens.fill_(p)
        if other.prev_embedding is not None:
            self.prev_embedding = other.prev_embedding.expand(B, -1, -1).clone()


# ------------------------------------------------------------------------------------------------
# The caller of the hot path: token-level generation (nanochat/engine.py:141-304)
# ------------------------------------------------------------------------------------------------
def _eval_with_deadline(expr, seconds=3):
    """Evaluate a vetted arithmetic/string expression with an alarm-based deadline; None on failure."""
    def on_alarm(signum, frame):
        raise TimeoutError(expr)

    try:
        signal.signal(signal.SIGALRM, on_alarm)
        signal.alarm(seconds)
        try:
            with warnings.catch_warnings():
                warnings.simplefilter("ignore", SyntaxWarning)
                return eval(expr, {"__builtins__": {}}, {})
        finally:
            signal.alarm(0)
    except Exception:
        return None


_MATH_CHARS = set("0123456789*+-/.() ")
_TEXT_CHARS = set("abcdefghijklmnopqrstuvwxyzABCDEFGHIJKLMNOPQRSTUVWXYZ0123456789'\"()._ ")
_BANNED = ("__", "import", "exec", "eval", "compile", "open", "file", "input", "raw_input", "globals", "locals",
           "vars", "dir", "getattr", "setattr", "delattr", "hasattr")


def use_calculator(expr):
    """The calculator tool of the reference (engine.py:47-79): plain arithmetic without ``**``, or a
    ``.count()`` call on a string literal; anything else yields None."""
    expr = expr.replace(",", "")
    if all(ch in _MATH_CHARS for ch in expr):
        return None if "**" in expr else _eval_with_deadline(expr)
    if not all(ch in _TEXT_CHARS for ch in expr):
        return None
    lowered = expr.lower()
    if any(word in lowered for word in _BANNED) or ".count(" not in expr:
        return None
    return _eval_with_deadline(expr)


@torch.inference_mode()
def sample_next_token(logits, rng, temperature=1.0, top_k=None):
    """One token per row from (B, vocab) logits -> (B, 1); argmax at temperature 0, otherwise
    (top-k) softmax sampling with ``rng`` (engine.py:141-156)."""
    assert temperature >= 0.0, "temperature must be non-negative"
    if temperature == 0.0:
        return torch.argmax(logits, dim=-1, keepdim=True)
    if top_k is not None and top_k > 0:
        vals, idx = torch.topk(logits, min(top_k, logits.size(-1)), dim=-1)
        choice = torch.multinomial(F.softmax(vals / temperature, dim=-1), num_samples=1, generator=rng)
        return idx.gather(1, choice)
    return torch.multinomial(F.softmax(logits / temperature, dim=-1), num_samples=1, generator=rng)


class RowState:
    """Per-row bookkeeping of the generation loop (engine.py:160-167)."""

    def __init__(self, current_tokens=None):
        self.current_tokens = current_tokens or []
        self.forced_tokens = deque()    # tool output waiting to be injected
        self.in_python_block = False
        self.python_expr_tokens = []
        self.completed = False


class Engine:
    """Batch-1 prefill, broadcast of the prompt cache to ``num_samples`` rows, then one forward per
    generated token (engine.py:169-304).  The model only has to offer ``config``, ``get_device()``
    and ``forward(ids, kv_cache=...)``; the tokenizer only the special-token lookups, ``encode``
    and ``decode``."""

    def __init__(self, model, tokenizer, cuda_graph=True, page_tokens=None):
        self.model = model
        self.tokenizer = tokenizer
        # page_tokens: keep the decode cache in pages of that many tokens (PagedKVCache; the prompt's
        # pages are shared between the samples) instead of dense rows.  CUDA only.
        self.page_tokens = page_tokens
        # On a CUDA device the decode step is replayed from a CUDA graph once a generation is long
        # enough to pay for the capture (same tokens, cache lengths and cache bytes as eager steps).
        self.cuda_graph = cuda_graph

    @torch.inference_mode()
    def generate(self, tokens, num_samples=1, max_tokens=None, temperature=1.0, top_k=None, seed=42):
        assert isinstance(tokens, list) and isinstance(tokens[0], int), "expecting list of ints"
        device = self.model.get_device()
        dtype = torch.bfloat16 if device.type == "cuda" else torch.float32
        rng = torch.Generator(device=device)
        rng.manual_seed(seed)
        special = self.tokenizer.encode_special
        python_start, python_end = special("<|python_start|>"), special("<|python_end|>")
        output_start, output_end = special("<|output_start|>"), special("<|output_end|>")
        assistant_end = special("<|assistant_end|>")
        bos = self.tokenizer.get_bos_token_id()

        cfg = self.model.config
        geometry = dict(num_heads=cfg.n_kv_head, head_dim=cfg.n_embd // cfg.n_head, num_layers=cfg.n_layer)
        prompt_cache = KVCache(batch_size=1, seq_len=len(tokens), device=device, dtype=dtype, **geometry)
        ids = torch.tensor([tokens], dtype=torch.long, device=device)
        logits = self.model.forward(ids, kv_cache=prompt_cache)[:, -1, :].expand(num_samples, -1)

        capacity = (len(tokens) + max_tokens) if max_tokens is not None else cfg.sequence_len
        if self.page_tokens:
            # shared prompt pages + per row the pages its own continuation can need
            pt = self.page_tokens
            own = -(-capacity // pt) - len(tokens) // pt
            cache = PagedKVCache(batch_size=num_samples, seq_len=capacity, device=device, dtype=dtype, page_tokens=pt,
                                 n_pages=len(tokens) // pt + num_samples * own, **geometry)
        else:
            cache = KVCache(batch_size=num_samples, seq_len=capacity, device=device, dtype=dtype, **geometry)
        cache.prefill(prompt_cache)
        del prompt_cache

        rows = [RowState(tokens.copy()) for _ in range(num_samples)]
        produced = 0
        graphed = None
        on_gpu = device.type == "cuda"
        staged = torch.empty(num_samples, dtype=torch.long, pin_memory=True) if on_gpu else None
        arrived = torch.cuda.Event() if on_gpu else None

        def run_step(ids, n_done):
            """One forward of the new tokens ids (B, 1) on the device, the n_done-th generated column;
            returns the logits (B, vocab)."""
            nonlocal graphed
            if self.page_tokens:  # pages for this step's token (and the throw-away steps of a capture)
                cache.reserve(min(capacity, len(tokens) + n_done + 4))
            if graphed is None and self.cuda_graph and on_gpu and n_done >= 2:
                # capture runs three throw-away steps behind the current position: needs that room,
                # and only pays off if enough steps are still to come
                room = capacity - (len(tokens) + n_done)
                left = (max_tokens - n_done) if max_tokens is not None else room
                if room >= 4 and left >= 16 and cache.prev_embedding is not None:
                    graphed = GraphedDecodeStep(self.model, cache, ids)
            if graphed is not None:
                return graphed.step(ids)
            return self.model.forward(ids, kv_cache=cache)[:, -1, :]

        while (max_tokens is None or produced < max_tokens) and not all(r.completed for r in rows):
            drawn_dev = sample_next_token(logits, rng, temperature, top_k)  # (B, 1), stays on the device
            # Unless a row has tool output waiting to be injected, the tokens the model sees next are
            # exactly the ones just drawn: the next forward is enqueued straight from the device tensor,
            # before the host has looked at them, and the host-side bookkeeping below (token lists, the
            # tool-use state machine, the caller's work between yields) overlaps with it.  The reference
            # reads the tokens first (engine.py:240) and only then launches; the tokens are the same.
            ahead = not any(r.forced_tokens for r in rows)
            if on_gpu:
                staged.copy_(drawn_dev[:, 0], non_blocking=True)
                arrived.record()
            if ahead:
                logits = run_step(drawn_dev, produced + 1)
            if on_gpu:
                arrived.synchronize()
                sampled = staged.tolist()
            else:
                sampled = drawn_dev[:, 0].tolist()
            column, masks = [], []
            for row, drawn in zip(rows, sampled):
                forced = len(row.forced_tokens) > 0
                tok = row.forced_tokens.popleft() if forced else drawn
                masks.append(0 if forced else 1)
                column.append(tok)
                row.current_tokens.append(tok)
                if tok == assistant_end or tok == bos:
                    row.completed = True
                if tok == python_start:
                    row.in_python_block, row.python_expr_tokens = True, []
                elif tok == python_end and row.in_python_block:
                    row.in_python_block = False
                    if row.python_expr_tokens:
                        result = use_calculator(self.tokenizer.decode(row.python_expr_tokens))
                        if result is not None:
                            row.forced_tokens.append(output_start)
                            row.forced_tokens.extend(self.tokenizer.encode(str(result)))
                            row.forced_tokens.append(output_end)
                    row.python_expr_tokens = []
                elif row.in_python_block:
                    row.python_expr_tokens.append(tok)
            yield column, masks
            produced += 1
            if not ahead:
                logits = run_step(torch.tensor(column, dtype=torch.long, device=device).unsqueeze(1), produced)
            if on_gpu and produced % 64 == 0:
                ops.check_status(device)  # capacity / RoPE-range overflow raises like the reference's slice-assign
        if on_gpu:
            ops.check_status(device)

    def generate_batch(self, tokens, num_samples=1, **kwargs):
        """Run ``generate`` to the end; returns (token lists, sampled/forced masks) without the
        terminal tokens (engine.py:282-304)."""
        assistant_end = self.tokenizer.encode_special("<|assistant_end|>")
        bos = self.tokenizer.get_bos_token_id()
        results = [tokens.copy() for _ in range(num_samples)]
        masks = [[0] * len(tokens) for _ in range(num_samples)]
        done = [False] * num_samples
        for column, column_masks in self.generate(tokens, num_samples, **kwargs):
            for i, (tok, m) in enumerate(zip(column, column_masks)):
                if done[i]:
                    continue
                if tok == assistant_end or tok == bos:
                    done[i] = True
                else:
                    results[i].append(tok)
                    masks[i].append(m)
            if all(done):
                break
        return results, masks


class GraphedDecodeStep:
    """One decode step (``model.forward(ids (B, 1), kv_cache)``) captured in a CUDA graph.

    Possible because nothing on the cached path synchronises with the host: positions are read
    from ``cache_seqlens`` on the device, the append and attention kernels take no host-known
    lengths, and ``KVCache.advance`` is an in-place device add.  The reference's step cannot be
    captured (``get_pos()`` / ``.item()`` per forward and per layer, gpt.py:424, flash_attention.py:157).

    ``step(ids)`` copies the token ids into the graph's input buffer, replays, and returns the
    logits buffer (B, vocab) — overwritten by the next call.  The smear state
    (``kv_cache.prev_embedding``) is kept in a persistent buffer that the graph reads and updates.
    """

    def __init__(self, model, kv_cache, warmup_ids):
        assert warmup_ids.dim() == 2 and warmup_ids.size(1) == 1
        self.model, self.cache = model, kv_cache
        dev = warmup_ids.device
        self.ids = warmup_ids.clone()
        if kv_cache.prev_embedding is None:
            raise RuntimeError("capture after the prefill forward: the cache has no smear state yet")
        self._prev = kv_cache.prev_embedding.clone()
        kv_cache.prev_embedding = self._prev
        # capture must not move the real cache forward: remember lengths, restore after warm-up/capture
        saved_lens = kv_cache.cache_seqlens.clone()
        side = torch.cuda.Stream(dev)
        side.wait_stream(torch.cuda.current_stream(dev))
        with torch.cuda.stream(side):
            for _ in range(2):  # warm-up on the capture stream (allocates workspaces, autotunes GEMMs)
                self._body()
            side.synchronize()
            self.graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(self.graph, stream=side):
                self.logits = self._body()
        torch.cuda.current_stream(dev).wait_stream(side)
        kv_cache.cache_seqlens.copy_(saved_lens)
        self._prev.copy_(self._prev_saved)

    def _body(self):
        if not hasattr(self, "_prev_saved"):
            self._prev_saved = self._prev.clone()
        self.cache.prev_embedding = self._prev
        logits = self.model.forward(self.ids, kv_cache=self.cache)[:, -1, :]
        self._prev.copy_(self.cache.prev_embedding)
        self.cache.prev_embedding = self._prev
        return logits

    def step(self, ids):
        self.ids.copy_(ids, non_blocking=True)
        self.graph.replay()
        return self.logits
