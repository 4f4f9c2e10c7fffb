"""Torch-eager port of the reference's op sequence for the KV-cache decode path.  TEST
INFRASTRUCTURE ONLY: imported by tests/ (as "the reference bf16 GPU path" when run on CUDA
tensors) and by the cpu_baseline / reference legs of bench.py (as the reference's CPU path, fp32
on the host cores).  Nothing in the nanochat_b200 package imports it.

The functions issue the same ATen ops in the same order as the reference does:
  rotary_tables      gpt.py:268-283      rope / rope_norm_scale   gpt.py:57-63, 42-43, 101-102
  sdpa_window        flash_attention.py:69-102
  kvcache_attention_row / kvcache_attention   flash_attention.py:155-177 (one row at a time for
                     ragged lengths: the fallback itself assumes row 0's length for every row)
  prefill_broadcast  engine.py:123-137
Pinned against the fixtures of tests/golden/ (made by the reference itself) in
tests/test_oracle_golden.py.
"""
import torch
import torch.nn.functional as F


def rotary_tables(seq_len, head_dim, device, dtype, base=100000):
    """cos/sin of shape (1, seq_len, 1, head_dim/2), the op sequence of gpt.py:268-283."""
    channel_range = torch.arange(0, head_dim, 2, dtype=torch.float32, device=device)
    inv_freq = 1.0 / (base ** (channel_range / head_dim))
    t = torch.arange(seq_len, dtype=torch.float32, device=device)
    freqs = torch.outer(t, inv_freq)
    cos, sin = freqs.cos().to(dtype), freqs.sin().to(dtype)
    return cos[None, :, None, :], sin[None, :, None, :]


def rope(x, cos, sin):
    d = x.shape[3] // 2
    x1, x2 = x[..., :d], x[..., d:]
    y1 = x1 * cos + x2 * sin
    y2 = x1 * (-sin) + x2 * cos
    return torch.cat([y1, y2], 3)


def rope_norm_scale(x, cos, sin):
    y = rope(x, cos, sin)
    y = F.rms_norm(y, (y.size(-1),))
    return y * 1.2


def rope_norm_scale_rows(x, cos_table, sin_table, cache_seqlens):
    """Per-row positions: row b, token t uses table row cache_seqlens[b] + t (the reference slices
    one range for all rows, gpt.py:424-425; with equal lengths this is the same thing)."""
    B, T = x.shape[:2]
    pos = cache_seqlens.long()[:, None] + torch.arange(T, device=x.device)[None, :]
    cos = cos_table[0, :, 0][pos][:, :, None, :]
    sin = sin_table[0, :, 0][pos][:, :, None, :]
    return rope_norm_scale(x, cos, sin)


def sdpa_window(q, k, v, window, enable_gqa):
    """q, k, v in (B, H, T, D); the three regimes of flash_attention.py:69-102."""
    Tq, Tk = q.size(2), k.size(2)
    if (window < 0 or window >= Tq) and Tq == Tk:
        return F.scaled_dot_product_attention(q, k, v, is_causal=True, enable_gqa=enable_gqa)
    if Tq == 1:
        if 0 <= window < Tk:
            start = max(0, Tk - (window + 1))
            k, v = k[:, :, start:], v[:, :, start:]
        return F.scaled_dot_product_attention(q, k, v, is_causal=False, enable_gqa=enable_gqa)
    row = (Tk - Tq) + torch.arange(Tq, device=q.device).unsqueeze(1)
    col = torch.arange(Tk, device=q.device).unsqueeze(0)
    mask = col <= row
    if 0 <= window < Tk:
        mask = mask & ((row - col) <= window)
    return F.scaled_dot_product_attention(q, k, v, attn_mask=mask, enable_gqa=enable_gqa)


def kvcache_attention_row(q, k_cache, v_cache, k, v, pos, window):
    """One row (batch 1 slices): append at pos, attend over [0, pos + T_new). Mutates the caches."""
    T_new = q.size(1)
    if k is not None:
        k_cache[:, pos:pos + T_new] = k
        v_cache[:, pos:pos + T_new] = v
    end = pos + T_new
    y = sdpa_window(q.transpose(1, 2), k_cache[:, :end].transpose(1, 2), v_cache[:, :end].transpose(1, 2), window,
                    q.size(2) != k_cache.size(2))
    return y.transpose(1, 2)


def kvcache_attention(q, k_cache, v_cache, k, v, cache_seqlens, window):
    """Ragged rows = the reference run one row at a time and stacked."""
    outs = []
    lens = cache_seqlens.tolist()
    for b in range(q.size(0)):
        kb = k[b:b + 1] if k is not None else None
        vb = v[b:b + 1] if v is not None else None
        outs.append(kvcache_attention_row(q[b:b + 1], k_cache[b:b + 1], v_cache[b:b + 1], kb, vb, lens[b], window))
    return torch.cat(outs, 0)


def prefill_broadcast(src_k, src_v, dst_k, dst_v, dst_seqlens, p):
    """KVCache.prefill's two slice-assigns and the fill of cache_seqlens."""
    dst_k[:, :, :p, :, :] = src_k[:, :, :p, :, :]
    dst_v[:, :, :p, :, :] = src_v[:, :, :p, :, :]
    dst_seqlens.fill_(p)
