"""CPU restatement (numpy) of nanochat's KV-cache decode path.  TEST INFRASTRUCTURE ONLY.

This module is the checker for the CUDA kernels: only tests/, __graft_entry__.smoke() and the
cpu_baseline / reference legs of bench.py import it.  Nothing in the nanochat_b200 package does.

Each function restates one piece of the reference (paths are relative to the nanochat tree):

  bf16 helpers            torch's float32 -> bfloat16 cast (round to nearest even)
  rotary_tables           GPT._precompute_rotary_embeddings              gpt.py:268-283
  window_sizes            GPT._compute_window_sizes                      gpt.py:285-312
  rope                    apply_rotary_emb                               gpt.py:57-63
  rms_norm                norm = F.rms_norm(x, (D,))                     gpt.py:42-43
  rope_norm_scale         the q/k pipeline of CausalSelfAttention        gpt.py:99-102
  append                  cache slice-assign                             flash_attention.py:160-162
  visible_range           key range of the Tq==1 / masked branches       flash_attention.py:83-100
  attention_kvcache       flash_attn_with_kvcache (SDPA fallback)        flash_attention.py:155-177
  attention_nocache       flash_attn_func (SDPA fallback)                flash_attention.py:122-128
  prefill_broadcast       KVCache.prefill                                engine.py:123-137
  lse_combine             (no reference counterpart) merge of softmax partials over disjoint keys

Pinned by tests/test_oracle_golden.py against tests/golden/*.npz, which
tests/golden/make_golden.py produced by importing and running the reference itself on CPU.

bf16 mode reproduces the eager bf16 tensor path: every reference op computes in fp32 and rounds
its result to bf16.  The fp32 sum of squares inside rms_norm is order-sensitive in its last bit;
``order="lanes4"`` is the order of torch's CUDA row kernel for a 128-wide row (32 lanes x 4
consecutive elements, sequential in a lane, then a halving tree over lanes with offsets
16, 8, 4, 2, 1) which the CUDA append kernel follows; ``order="sequential"`` is a plain left-to-right sum.
"""
import numpy as np

FP32_EPS = np.float32(1.1920928955078125e-07)


# ---------------------------------------------------------------------------------------------
# bf16 helpers
# ---------------------------------------------------------------------------------------------
def f32_to_bf16_bits(x):
    """Round-to-nearest-even float32 -> bfloat16 bit patterns (uint16). NaN stays NaN."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    u = x.view(np.uint32)
    rounding = ((u >> 16) & 1) + np.uint32(0x7FFF)
    r = ((u + rounding) >> 16).astype(np.uint16)
    nan = np.isnan(x)
    if nan.any():
        r = np.where(nan, ((u >> 16) | 0x0040).astype(np.uint16), r)
    return r


def bf16_bits_to_f32(b):
    return (np.ascontiguousarray(b, dtype=np.uint16).astype(np.uint32) << 16).view(np.float32)


def bf16_round(x):
    """float32 values rounded to the nearest bfloat16, returned as float32."""
    return bf16_bits_to_f32(f32_to_bf16_bits(x))


# ---------------------------------------------------------------------------------------------
# tables and integer bookkeeping
# ---------------------------------------------------------------------------------------------
def rotary_tables(seq_len, head_dim, base=100000.0, bf16=False):
    """cos/sin of shape (seq_len, head_dim/2): fp32 outer(t, base^(-2i/D)), optionally cast to bf16."""
    channel = np.arange(0, head_dim, 2, dtype=np.float32)
    inv_freq = (np.float32(1.0) / np.power(np.float32(base), channel / np.float32(head_dim))).astype(np.float32)
    t = np.arange(seq_len, dtype=np.float32)
    freqs = np.outer(t, inv_freq).astype(np.float32)
    cos, sin = np.cos(freqs).astype(np.float32), np.sin(freqs).astype(np.float32)
    if bf16:
        cos, sin = bf16_round(cos), bf16_round(sin)
    return cos, sin


def window_sizes(sequence_len, n_layer, pattern="SSSL"):
    """Per-layer (left, right) windows: L = sequence_len, S = ceil(sequence_len/4/128)*128, the
    pattern tiled over layers, last layer always L."""
    pattern = pattern.upper()
    if not pattern or any(c not in "SL" for c in pattern):
        raise ValueError(f"invalid window pattern {pattern!r}")
    long_w = sequence_len
    short_w = -(-long_w // 4 // 128) * 128
    out = [((long_w if pattern[i % len(pattern)] == "L" else short_w), 0) for i in range(n_layer)]
    out[-1] = (long_w, 0)
    return out


def visible_range(length_before, t, T_new, window_left):
    """Half-open key range [lo, hi) seen by new token t (0-based) of a row that held
    ``length_before`` keys before T_new tokens were appended."""
    p = length_before + t            # absolute position of the query (row_idx = (Tk - Tq) + t)
    Tk = length_before + T_new
    lo = 0
    if 0 <= window_left < Tk:
        lo = max(0, p - window_left)
    return lo, p + 1


# ---------------------------------------------------------------------------------------------
# RoPE / rms-norm / scale
# ---------------------------------------------------------------------------------------------
def rope(x, cos, sin, bf16=False):
    """x: (..., D); cos/sin broadcastable to (..., D/2). Half-split rotation with the reference's signs."""
    x = np.asarray(x, dtype=np.float32)
    d = x.shape[-1] // 2
    x1, x2 = x[..., :d], x[..., d:]
    cos = np.asarray(cos, dtype=np.float32)
    sin = np.asarray(sin, dtype=np.float32)
    if bf16:
        y1 = bf16_round(bf16_round(x1 * cos) + bf16_round(x2 * sin))
        y2 = bf16_round(bf16_round(x1 * (-sin)) + bf16_round(x2 * cos))
    else:
        y1 = x1 * cos + x2 * sin
        y2 = x1 * (-sin) + x2 * cos
    return np.concatenate([y1, y2], axis=-1).astype(np.float32)


def _sumsq(y, order):
    sq = (y * y).astype(np.float32)
    D = y.shape[-1]
    if order == "sequential":
        acc = np.zeros(y.shape[:-1], dtype=np.float32)
        for i in range(D):
            acc = (acc + sq[..., i]).astype(np.float32)
        return acc
    if order == "lanes4":
        assert D % 4 == 0 and (D // 4) & (D // 4 - 1) == 0, "lanes4 order needs D/4 a power of two"
        lanes = sq.reshape(*y.shape[:-1], D // 4, 4)
        acc = lanes[..., 0]
        for i in range(1, 4):
            acc = (acc + lanes[..., i]).astype(np.float32)
        n = D // 4
        while n > 1:
            n //= 2
            acc = (acc[..., :n] + acc[..., n:2 * n]).astype(np.float32)
        return acc[..., 0]
    if order == "numpy":
        return sq.sum(axis=-1, dtype=np.float32)
    raise ValueError(order)


def rms_norm(y, eps=FP32_EPS, bf16=False, order="lanes4"):
    """y * rsqrt(mean(y^2) + eps) over the last dim, fp32 statistics; bf16 mode rounds the result."""
    y = np.asarray(y, dtype=np.float32)
    D = y.shape[-1]
    mean = (_sumsq(y, order) / np.float32(D)).astype(np.float32)
    rstd = (np.float32(1.0) / np.sqrt((mean + np.float32(eps)).astype(np.float32))).astype(np.float32)
    z = (y * rstd[..., None]).astype(np.float32)
    return bf16_round(z) if bf16 else z


def rope_norm_scale(x, cos, sin, scale=1.2, eps=FP32_EPS, bf16=False, order="lanes4"):
    """rope -> rms_norm -> * scale, with a bf16 rounding after every op in bf16 mode."""
    z = rms_norm(rope(x, cos, sin, bf16=bf16), eps=eps, bf16=bf16, order=order)
    out = (z * np.float32(scale)).astype(np.float32)
    return bf16_round(out) if bf16 else out


def rope_norm_scale_rows(x, cos_table, sin_table, cache_seqlens, scale=1.2, eps=FP32_EPS, bf16=False,
                         order="lanes4"):
    """x: (B, T, H, D); token t of row b uses table row cache_seqlens[b] + t."""
    B, T = x.shape[:2]
    pos = np.asarray(cache_seqlens, dtype=np.int64)[:, None] + np.arange(T)[None, :]
    cos = cos_table[pos][:, :, None, :]
    sin = sin_table[pos][:, :, None, :]
    return rope_norm_scale(x, cos, sin, scale=scale, eps=eps, bf16=bf16, order=order)


# ---------------------------------------------------------------------------------------------
# cache update and attention
# ---------------------------------------------------------------------------------------------
def append(k_cache, v_cache, k, v, cache_seqlens):
    """In place: cache[b, L_b + t] = new[b, t].  Raises on capacity overflow like the slice-assign."""
    B, T_new = k.shape[:2]
    T_max = k_cache.shape[1]
    for b in range(B):
        L = int(cache_seqlens[b])
        if L < 0 or L + T_new > T_max:
            raise ValueError(f"row {b}: appending {T_new} tokens at {L} overflows capacity {T_max}")
        k_cache[b, L:L + T_new] = k[b]
        v_cache[b, L:L + T_new] = v[b]


def _softmax_av(q, K, V, scale):
    """q: (Hq, D), K/V: (n, Hkv, D) fp32 -> (out (Hq, D), lse (Hq,)) with GQA head h -> h // G."""
    Hq, D = q.shape
    Hkv = K.shape[1]
    G = Hq // Hkv
    out = np.zeros((Hq, D), dtype=np.float64)
    lse = np.full((Hq,), -np.inf, dtype=np.float64)
    if K.shape[0] == 0:
        return out.astype(np.float32), lse.astype(np.float32)
    for h in range(Hq):
        kh = K[:, h // G, :].astype(np.float64)
        vh = V[:, h // G, :].astype(np.float64)
        s = kh @ q[h].astype(np.float64) * scale
        m = s.max()
        p = np.exp(s - m)
        l = p.sum()
        out[h] = (p @ vh) / l
        lse[h] = m + np.log(l)
    return out.astype(np.float32), lse.astype(np.float32)


def attention_kvcache(q, k_cache, v_cache, cache_seqlens, window_left=-1, kv_begin=0, kv_end=0):
    """Attention of T_new new tokens per row against caches that already contain them.

    q: (B, T_new, Hq, D); caches: (B, T_max, Hkv, D); cache_seqlens: lengths BEFORE the append.
    Returns (out (B, T_new, Hq, D) fp32, lse (B, T_new, Hq) fp32).  A non-empty [kv_begin, kv_end)
    restricts the keys to that shard (rows with no key left give out = 0, lse = -inf).
    """
    q = np.asarray(q, dtype=np.float32)
    B, T_new, Hq, D = q.shape
    scale = 1.0 / np.sqrt(D)
    out = np.zeros((B, T_new, Hq, D), dtype=np.float32)
    lse = np.zeros((B, T_new, Hq), dtype=np.float32)
    for b in range(B):
        L = int(cache_seqlens[b])
        for t in range(T_new):
            lo, hi = visible_range(L, t, T_new, window_left)
            if kv_end > kv_begin:
                lo, hi = max(lo, kv_begin), min(hi, kv_end)
                hi = max(hi, lo)
            K = np.asarray(k_cache[b, lo:hi], dtype=np.float32)
            V = np.asarray(v_cache[b, lo:hi], dtype=np.float32)
            out[b, t], lse[b, t] = _softmax_av(q[b, t], K, V, scale)
    return out, lse


def attention_nocache(q, k, v, window_left=-1):
    """flash_attn_func: causal (+ left window) attention, q/k/v (B, T, H, D) of equal length."""
    B, T = q.shape[:2]
    zeros = np.zeros((B,), dtype=np.int32)
    return attention_kvcache(q, k, v, zeros, window_left=window_left)[0]


def lse_combine(parts_o, parts_lse):
    """parts_o: (n, ..., D) normalised partial outputs, parts_lse: (n, ...).  Returns (out, lse)."""
    parts_o = np.asarray(parts_o, dtype=np.float64)
    parts_lse = np.asarray(parts_lse, dtype=np.float64)
    M = parts_lse.max(axis=0)
    safe_M = np.where(np.isfinite(M), M, 0.0)
    w = np.exp(parts_lse - safe_M)
    w = np.where(np.isfinite(parts_lse), w, 0.0)
    L = w.sum(axis=0)
    with np.errstate(invalid="ignore", divide="ignore"):
        out = (w[..., None] * parts_o).sum(axis=0) / L[..., None]
        lse = safe_M + np.log(L)
    out = np.where((L > 0)[..., None], out, 0.0)
    lse = np.where(L > 0, lse, -np.inf)
    return out.astype(np.float32), lse.astype(np.float32)


# ---------------------------------------------------------------------------------------------
# prefill broadcast
# ---------------------------------------------------------------------------------------------
def prefill_broadcast(src_k, src_v, dst_k, dst_v, dst_seqlens, p):
    """dst[:, b, :p] = src[:, 0, :p] for every row b; dst_seqlens[:] = p.  In place."""
    if dst_k.shape[0] != src_k.shape[0] or dst_k.shape[3:] != src_k.shape[3:]:
        raise ValueError("layer/head/dim mismatch")
    if p > src_k.shape[2] or p > dst_k.shape[2]:
        raise ValueError("p exceeds a cache capacity")
    dst_k[:, :, :p] = src_k[:, :1, :p]
    dst_v[:, :, :p] = src_v[:, :1, :p]
    if dst_seqlens is not None:
        dst_seqlens[...] = p
