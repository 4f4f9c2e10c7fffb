"""Test-only stand-ins that let the host logic (KVCache, GPT glue, Engine) run on CPU tensors.

The product has no CPU path: ``nanochat_b200.ops`` raises for non-CUDA tensors.  These helpers
swap the three op entry points the host logic calls for the torch port of the reference under
oracle/ (which is the checker, never the product), so that bookkeeping, glue arithmetic and the
generation loop can be pinned against the reference's fixtures without a GPU.
"""
import contextlib
from types import SimpleNamespace

import torch

from oracle import torch_ref as R


def _kv_attention(q, k, v, cos_sin_tables, window_size, kv_cache, layer_idx):
    cos, sin = cos_sin_tables
    lens = kv_cache.cache_seqlens
    q2 = R.rope_norm_scale_rows(q, cos, sin, lens)
    k2 = R.rope_norm_scale_rows(k, cos, sin, lens)
    k_cache, v_cache = kv_cache.get_layer_cache(layer_idx)
    y = R.kvcache_attention(q2, k_cache, v_cache, k2, v, lens, int(window_size[0]))
    if layer_idx == kv_cache.n_layers - 1:
        kv_cache.advance(q.size(1))
    return y


def _flash_attn_func(q, k, v, causal=False, window_size=(-1, -1)):
    y = R.sdpa_window(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2), int(window_size[0]),
                      q.size(2) != k.size(2))
    return y.transpose(1, 2)


def _prefill_broadcast(src_k, src_v, dst_k, dst_v, dst_seqlens, p):
    R.prefill_broadcast(src_k, src_v, dst_k, dst_v, dst_seqlens, p)


@contextlib.contextmanager
def oracle_backend():
    import nanochat_b200.gpt as gpt
    import nanochat_b200.ops as ops
    saved = (gpt.kv_attention, gpt.flash_attn, ops.prefill_broadcast)
    gpt.kv_attention = _kv_attention
    gpt.flash_attn = SimpleNamespace(flash_attn_func=_flash_attn_func)
    ops.prefill_broadcast = _prefill_broadcast
    try:
        yield
    finally:
        gpt.kv_attention, gpt.flash_attn, ops.prefill_broadcast = saved


class SpecialsTokenizer:
    """The six special ids Engine asks for, placed above the vocabulary so argmax never hits them."""
    names = ["<|bos|>", "<|python_start|>", "<|python_end|>", "<|output_start|>", "<|output_end|>",
             "<|assistant_end|>"]

    def __init__(self, base=32768 + 100):
        self.base = base

    def encode_special(self, s):
        return self.base + self.names.index(s)

    def get_bos_token_id(self):
        return self.encode_special("<|bos|>")

    def encode(self, s, prepend=None):
        return list(s.encode())

    def decode(self, ids):
        return bytes(i for i in ids if i < 256).decode("utf-8", "replace")
