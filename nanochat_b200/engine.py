"""KV cache with the reference's interface (nanochat/engine.py:82-137), storage on the GPU.

``KVCache`` keeps the reference's constructor, attributes (``k_cache`` / ``v_cache`` of shape
(n_layers, B, T_max, Hkv, D), int32 ``cache_seqlens``, ``prev_embedding``) and methods
(``reset / get_pos / get_layer_cache / advance / prefill``).  Bookkeeping is integer tensor
arithmetic and works on any device; ``prefill`` — the batch-1 -> num_samples broadcast — is the
CUDA copy kernel of libnckv and raises for non-CUDA caches (there is no CPU path).
"""
import torch

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
