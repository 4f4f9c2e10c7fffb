"""The attention KV branch of nanochat's GPT (gpt.py:97-121) on the fused kernels, plus the two
pure-host helpers it depends on (rotary tables, per-layer windows)."""
import torch

from . import ops


def precompute_rotary_embeddings(seq_len, head_dim, base=100000, device=None, dtype=torch.bfloat16):
    """cos/sin tables of shape (1, seq_len, 1, head_dim/2): the op sequence of
    GPT._precompute_rotary_embeddings (gpt.py:268-283), so the tables are bit-identical to the
    reference's when made on the same device with the same dtype."""
    channel_range = torch.arange(0, head_dim, 2, dtype=torch.float32, device=device)
    inv_freq = 1.0 / (base ** (channel_range / head_dim))
    t = torch.arange(seq_len, dtype=torch.float32, device=device)
    freqs = torch.outer(t, inv_freq)
    cos, sin = freqs.cos().to(dtype), freqs.sin().to(dtype)
    return cos[None, :, None, :], sin[None, :, None, :]


def compute_window_sizes(sequence_len, n_layer, window_pattern="SSSL"):
    """Per-layer (left, right) windows as GPT._compute_window_sizes (gpt.py:285-312): 'L' is
    sequence_len, 'S' is ceil(sequence_len / 4 / 128) * 128, the pattern is tiled over the
    layers and the last layer is always 'L'."""
    pattern = window_pattern.upper()
    assert pattern and all(c in "SL" for c in pattern), f"Invalid window_pattern: {pattern}. Use only S and L."
    long_window = sequence_len
    short_window = -(-long_window // 4 // 128) * 128
    sizes = [(long_window if pattern[i % len(pattern)] == "L" else short_window, 0) for i in range(n_layer)]
    sizes[-1] = (long_window, 0)
    return sizes


def kv_attention(q, k, v, cos_sin_tables, window_size, kv_cache, layer_idx):
    """The KV-cache branch of CausalSelfAttention.forward (gpt.py:97-121) in two launches.

    q: (B, T, Hq, D), k, v: (B, T, Hkv, D) straight from the projections (v already carries the
    value-embedding gate).  ``cos_sin_tables`` are the FULL tables (1, rope_len, 1, D/2): each row
    is rotated at its own position ``kv_cache.cache_seqlens[b] + t`` on the device, so no
    ``get_pos()`` synchronisation and no table slicing is needed.  Launch 1 applies RoPE, QK-norm
    and the 1.2 scale to q and k and appends k/v to the layer's cache; launch 2 attends.
    As in the reference the cache position is advanced once, after the last layer.
    Returns y of shape (B, T, Hq, D).
    """
    cos, sin = cos_sin_tables
    k_cache, v_cache = kv_cache.get_layer_cache(layer_idx)
    seqlens = kv_cache.cache_seqlens
    T = q.size(1)
    q2 = ops.append_rope_norm(q, k, v, k_cache, v_cache, seqlens, cos, sin)
    left = int(window_size[0])
    left = left if left >= 0 else -1
    if T == 1:
        y = ops.decode_attention(q2[:, 0], k_cache, v_cache, seqlens, seqlen_offset=1, window_left=left).unsqueeze(1)
    else:
        y = ops.prefill_attention(q2, k_cache, v_cache, seqlens, left)
    if layer_idx == kv_cache.n_layers - 1:
        kv_cache.advance(T)
    return y
