"""Attention entry points with the reference's names and signatures, backed by libnckv.

Mirror of nanochat/flash_attention.py: ``flash_attn.flash_attn_func`` (flash_attention.py:107-128)
and ``flash_attn.flash_attn_with_kvcache`` (flash_attention.py:131-177) keep their Python
signatures, layouts ((B, T, H, D) activations, (B, T_max, Hkv, D) caches, int32 cache_seqlens) and
in-place cache update, but run hand-written sm_100a kernels through the ``nckv`` custom ops.
What differs from the SDPA fallback they replace on Blackwell:

* positions are per row: row b appends at ``cache_seqlens[b]`` and attends over its own length
  (the per-row contract of flash_attention.py:142, which the fallback narrows to row 0's length
  at flash_attention.py:157); with lock-step rows, as ``Engine`` keeps them, results coincide;
* no host synchronisation: ``cache_seqlens`` is only read on the device;
* bf16 CUDA tensors with head_dim 128 only.  Anything else raises; there is no CPU or eager path.

``HAS_FA3`` / ``USE_FA3`` / ``_override_impl`` / ``_resolve_use_fa3`` stay importable because the
reference's scripts and tests read them (scripts/base_train.py:35,103,
tests/test_attention_fallback.py:23-26); FA3 itself is a Hopper-only binary and is never used here.
"""
from types import SimpleNamespace

import torch

from . import ops

HAS_FA3 = False
_override_impl = None  # 'fa3', 'sdpa' or None, as in the reference; selects nothing here


def _resolve_use_fa3():
    """Same decision table as flash_attention.py:48-63 with FA3 absent."""
    if _override_impl == "fa3":
        assert HAS_FA3, "Cannot override to FA3: not available on this hardware"
        return True
    return False


USE_FA3 = _resolve_use_fa3()


def _window_left(window_size):
    left = int(window_size[0])
    return left if left >= 0 else -1


def flash_attn_func(q, k, v, causal=False, window_size=(-1, -1)):
    """Attention without a cache. q, k, v: (B, T, H, D); returns (B, T, H, D).

    As in the fallback it replaces (flash_attention.py:122-128), masking is always causal with the
    left window ``window_size[0]``; ``causal`` and ``window_size[1]`` are accepted and not consulted.
    When an input requires grad (training, gpt.py:108) the call goes through an autograd function whose
    backward runs the library's own dq/dk/dv kernels; the forward is the same kernel either way.
    """
    if torch.is_grad_enabled() and (q.requires_grad or k.requires_grad or v.requires_grad):
        return ops.FlashAttnTrainFunction.apply(q, k, v, _window_left(window_size))
    return ops.prefill_attention(q, k, v, None, _window_left(window_size))


def flash_attn_with_kvcache(q, k_cache, v_cache, k=None, v=None, cache_seqlens=None,
                            causal=False, window_size=(-1, -1)):
    """Append k/v to the cache in place, then attend. Returns (B, T_new, H, D).

    q: (B, T_new, H, D); k_cache, v_cache: (B, T_max, Hkv, D) views updated in place;
    k, v: (B, T_new, Hkv, D) or None; cache_seqlens: (B,) int32, NOT advanced by this call
    (the caller advances it after the last layer, gpt.py:120-121).  Query t of row b sits at
    position ``cache_seqlens[b] + t`` and sees keys ``j <= position`` with
    ``position - j <= window_size[0]`` (flash_attention.py:83-88, 92-100).  As in the fallback, the
    keys ``[0, cache_seqlens + T_new)`` are attended whether or not k/v were given.
    """
    if cache_seqlens is None:
        raise ValueError("flash_attn_with_kvcache needs cache_seqlens")
    if (k is None) != (v is None):
        raise ValueError("k and v must be given together")
    T_new = q.size(1)
    if k is not None:
        ops.append_kv(k, v, k_cache, v_cache, cache_seqlens)
    left = _window_left(window_size)
    if T_new == 1:
        out = ops.decode_attention(q[:, 0], k_cache, v_cache, cache_seqlens, seqlen_offset=1, window_left=left)
        return out.unsqueeze(1)
    return ops.prefill_attention(q, k_cache, v_cache, cache_seqlens, left)


flash_attn = SimpleNamespace(
    flash_attn_func=flash_attn_func,
    flash_attn_with_kvcache=flash_attn_with_kvcache,
)
