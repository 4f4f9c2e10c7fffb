"""PyTorch custom ops (namespace ``nckv``) over the C ABI of libnckv.so.

Each op validates shapes/dtypes on the host, hands raw device pointers, element strides and the
current CUDA stream of the tensors' device to the library, and returns torch tensors it
allocated with ``torch.empty``.  Tensors must live on a CUDA device: there is no CPU
implementation and no eager fallback, a non-CUDA tensor raises.
"""
import ctypes

import torch

from . import _lib

HEAD_DIM = 128
# F.rms_norm(x, (D,)) with eps=None on bf16 inputs (gpt.py:42-43) resolves to the fp32 machine epsilon.
RMS_EPS = 1.1920928955078125e-07
QK_SCALE = 1.2  # gpt.py:101-102

_NS = torch.library.Library("nckv", "DEF")
_F_APPEND_ROPE = _lib.lib.nckv_append_rope_norm
_F_APPEND = _lib.lib.nckv_append
_F_DECODE = _lib.lib.nckv_decode_attn
_F_PREFILL = _lib.lib.nckv_prefill_attn
_workspaces = {}  # (device index, stream id) -> uint8 tensor
# Workspaces that a larger one has replaced.  They are kept alive for the life of the process: a CUDA
# graph captured while one of them was current still launches kernels that point at it.  A (device,
# stream) pair only ever grows its workspace a handful of times (the size depends on Hq / Hkv alone).
_retired_workspaces = []
_bwd_status = {}  # device index -> int32 view of the status word of the latest flash_attn_bwd call's scratch


def _ptr(t):
    return ctypes.c_void_p(t.data_ptr()) if t is not None else ctypes.c_void_p(0)


def _stream(device):
    return ctypes.c_void_p(torch.cuda.current_stream(device).cuda_stream)


def _require_cuda(name, *tensors):
    for t in tensors:
        if t is None:
            continue
        if not t.is_cuda:
            raise RuntimeError(
                f"nckv::{name} needs CUDA tensors (got device {t.device}); the KV-cache decode path "
                "has no CPU implementation")


def _require_bf16(name, *tensors):
    for t in tensors:
        if t is not None and t.dtype != torch.bfloat16:
            raise RuntimeError(f"nckv::{name} needs bfloat16 tensors, got {t.dtype}")


def _cache_strides(name, cache):
    """(batch_stride, token_stride) in elements of a (B, T, Hkv, D) cache view."""
    if cache.dim() != 4 or cache.size(3) != HEAD_DIM:
        raise RuntimeError(f"nckv::{name}: cache must be (B, T_max, Hkv, {HEAD_DIM}), got {tuple(cache.shape)}")
    sb, st, sh, sd = cache.stride()
    if sd != 1 or sh != HEAD_DIM:
        raise RuntimeError(f"nckv::{name}: cache heads must be packed (strides {cache.stride()})")
    return sb, st


class _device_guard:
    """Make `idx` the current CUDA device for the duration of a call; free when it already is."""
    __slots__ = ("idx", "prev")

    def __init__(self, idx):
        self.idx = idx
        self.prev = -1

    def __enter__(self):
        cur = torch.cuda.current_device()
        if cur != self.idx:
            self.prev = cur
            torch.cuda.set_device(self.idx)

    def __exit__(self, *exc):
        if self.prev >= 0:
            torch.cuda.set_device(self.prev)
        return False


_ws_need = {}  # (B, Hq, Hkv) -> bytes


def _launch_ctx(t, B, Hq, Hkv):
    """(device index, raw stream handle, workspace tensor) for a launch on t's device."""
    idx = t.device.index
    stream = torch.cuda.current_stream(idx).cuda_stream
    ws = _workspaces.get((idx, stream))
    need = _ws_need.get((B, Hq, Hkv))
    if ws is None or need is None or ws.numel() < need:
        ws = workspace(t.device, B, Hq, Hkv)
        _ws_need[(B, Hq, Hkv)] = _lib.lib.nckv_workspace_bytes(B, Hq, Hkv, HEAD_DIM)
    return idx, stream, ws


def workspace(device, B, Hq, Hkv):
    """Zero-initialised scratch for the split-KV kernels, cached per (device, stream)."""
    device = torch.device(device)
    idx = device.index if device.index is not None else torch.cuda.current_device()
    with torch.cuda.device(idx):
        need = _lib.lib.nckv_workspace_bytes(B, Hq, Hkv, HEAD_DIM)
    if need == 0:
        raise RuntimeError(f"nckv: unsupported shape B={B} Hq={Hq} Hkv={Hkv}")
    key = (idx, torch.cuda.current_stream(idx).cuda_stream)
    ws = _workspaces.get(key)
    if ws is None or ws.numel() < need:
        if ws is not None:
            _retired_workspaces.append(ws)
        ws = torch.zeros(max(need, 1 << 20), dtype=torch.uint8, device=torch.device("cuda", idx))
        _workspaces[key] = ws
    return ws


def read_status(device, clear=True):
    """Synchronously read (and by default clear) the device status word of the current stream's
    workspace (and of the device's latest attention backward); 0 means no guard fired.  Bits: 1 overflow, 2 timeout, 4 bad cache_seqlens, 8 bad page."""
    device = torch.device(device)
    idx = device.index if device.index is not None else torch.cuda.current_device()
    key = (idx, torch.cuda.current_stream(idx).cuda_stream)
    ws = _workspaces.get(key)
    with torch.cuda.device(idx):
        st = _lib.call("nckv_read_status", _ptr(ws), int(bool(clear)), _stream(idx)) if ws is not None else 0
        for old in _retired_workspaces:  # graphs captured earlier report into the workspace they were captured with
            if old.device.index == idx:
                st |= _lib.call("nckv_read_status", _ptr(old), int(bool(clear)), _stream(idx))
        last_bwd = _bwd_status.get(idx)  # the latest attention backward on this device reports into its own scratch
        if last_bwd is not None:
            st |= int(last_bwd.item())
            if clear:
                del _bwd_status[idx]
    return st


def check_status(device):
    st = read_status(device, clear=True)
    if st:
        names = [n for bit, n in ((1, "capacity overflow"), (2, "barrier timeout"), (4, "negative cache_seqlens"),
                                  (8, "block-table entry outside the page pool")) if st & bit]
        raise RuntimeError("nckv device status: " + ", ".join(names))


# ------------------------------------------------------------------------------------------------
# append (+ RoPE, QK-norm, scale)
# ------------------------------------------------------------------------------------------------
_NS.define("append_rope_norm(Tensor q, Tensor k, Tensor v, Tensor(a!) k_cache, Tensor(b!) v_cache, "
           "Tensor cache_seqlens, Tensor cos, Tensor sin, float qk_scale, float eps) -> Tensor")


def _append_rope_norm(q, k, v, k_cache, v_cache, cache_seqlens, cos, sin, qk_scale, eps, write_slots=None, split=None):
    name = "append_rope_norm"
    _require_cuda(name, q, k, v, k_cache, v_cache, cache_seqlens, cos, sin)
    _require_bf16(name, q, k, v, k_cache, v_cache, cos, sin)
    if cache_seqlens.dtype != torch.int32:
        raise RuntimeError("nckv::append_rope_norm: cache_seqlens must be int32")
    B, T_new, Hq, D = q.shape
    Hkv = k.size(2)
    if k.shape != (B, T_new, Hkv, D) or v.shape != k.shape:
        raise RuntimeError(f"nckv::{name}: k/v shapes {tuple(k.shape)}/{tuple(v.shape)} do not match q {tuple(q.shape)}")
    if k_cache.shape != v_cache.shape or k_cache.stride() != v_cache.stride():
        raise RuntimeError(f"nckv::{name}: k_cache and v_cache must share shape and strides")
    if k_cache.size(0) != B or k_cache.size(2) != Hkv:
        raise RuntimeError(f"nckv::{name}: cache {tuple(k_cache.shape)} does not match B={B}, Hkv={Hkv}")
    sb, st = _cache_strides(name, k_cache)
    cos2 = cos.reshape(-1, D // 2)
    sin2 = sin.reshape(-1, D // 2)
    if not (cos2.is_contiguous() and sin2.is_contiguous()):
        cos2, sin2 = cos2.contiguous(), sin2.contiguous()
    # q, k, v may be column slices of one projection output: packed heads, a common token stride per tensor
    strided = None
    if split is None and write_slots is None and not (q.is_contiguous() and k.is_contiguous() and v.is_contiguous()):
        def token_stride(t, H):
            ok = t.stride(3) == 1 and t.stride(2) == D and (T_new == 1 or t.stride(0) == T_new * t.stride(1)) and \
                t.stride(1 if T_new > 1 else 0) % 8 == 0 and t.data_ptr() % 16 == 0
            return t.stride(1 if T_new > 1 else 0) if ok else None
        strided = (token_stride(q, Hq), token_stride(k, Hkv), token_stride(v, Hkv))
        if None in strided:
            strided = None
    if strided is None:
        q, k, v = q.contiguous(), k.contiguous(), v.contiguous()
    q_out = torch.empty((B, T_new, Hq, D), dtype=q.dtype, device=q.device)
    idx, stream, ws = _launch_ctx(q, B, Hq, Hkv)
    with _device_guard(idx):
        if strided is not None:
            rc = _lib.lib.nckv_append_rope_norm_strided(q.data_ptr(), k.data_ptr(), v.data_ptr(), strided[0], strided[1],
                                                        strided[2], q_out.data_ptr(), k_cache.data_ptr(),
                                                        v_cache.data_ptr(), cache_seqlens.data_ptr(), cos2.data_ptr(),
                                                        sin2.data_ptr(), B, T_new, Hq, Hkv, D, k_cache.size(1), sb, st,
                                                        cos2.size(0), qk_scale, eps, ws.data_ptr(), stream)
        elif split is not None:
            world, rank, block = split
            rc = _lib.lib.nckv_append_rope_norm_split(q.data_ptr(), k.data_ptr(), v.data_ptr(), q_out.data_ptr(),
                                                      k_cache.data_ptr(), v_cache.data_ptr(), cache_seqlens.data_ptr(),
                                                      cos2.data_ptr(), sin2.data_ptr(), B, T_new, Hq, Hkv, D,
                                                      k_cache.size(1), sb, st, cos2.size(0), qk_scale, eps, world, rank,
                                                      block, ws.data_ptr(), stream)
        elif write_slots is None:
            rc = _F_APPEND_ROPE(q.data_ptr(), k.data_ptr(), v.data_ptr(), q_out.data_ptr(), k_cache.data_ptr(),
                                v_cache.data_ptr(), cache_seqlens.data_ptr(), cos2.data_ptr(), sin2.data_ptr(), B, T_new,
                                Hq, Hkv, D, k_cache.size(1), sb, st, cos2.size(0), qk_scale, eps, ws.data_ptr(), stream)
        else:
            if write_slots.dtype != torch.int32 or not write_slots.is_cuda or write_slots.numel() != B:
                raise RuntimeError(f"nckv::{name}: write_slots must be a CUDA int32 tensor of {B} rows")
            rc = _lib.lib.nckv_append_rope_norm_at(q.data_ptr(), k.data_ptr(), v.data_ptr(), q_out.data_ptr(),
                                                   k_cache.data_ptr(), v_cache.data_ptr(), cache_seqlens.data_ptr(),
                                                   write_slots.data_ptr(), cos2.data_ptr(), sin2.data_ptr(), B, T_new, Hq,
                                                   Hkv, D, k_cache.size(1), sb, st, cos2.size(0), qk_scale, eps,
                                                   ws.data_ptr(), stream)
    if rc < 0:
        _lib.check("nckv_append_rope_norm", rc)
    return q_out


_NS.impl("append_rope_norm", _append_rope_norm, "CUDA")
_NS.impl("append_rope_norm", _append_rope_norm, "CPU")  # raises: no CPU implementation

_NS.define("append_kv(Tensor k, Tensor v, Tensor(a!) k_cache, Tensor(b!) v_cache, Tensor cache_seqlens) -> ()")


def _append_kv(k, v, k_cache, v_cache, cache_seqlens):
    name = "append_kv"
    _require_cuda(name, k, v, k_cache, v_cache, cache_seqlens)
    _require_bf16(name, k, v, k_cache, v_cache)
    if cache_seqlens.dtype != torch.int32:
        raise RuntimeError("nckv::append_kv: cache_seqlens must be int32")
    B, T_new, Hkv, D = k.shape
    if v.shape != k.shape:
        raise RuntimeError(f"nckv::{name}: k/v shapes differ")
    if k_cache.shape != v_cache.shape or k_cache.stride() != v_cache.stride():
        raise RuntimeError(f"nckv::{name}: k_cache and v_cache must share shape and strides")
    if k_cache.size(0) != B or k_cache.size(2) != Hkv:
        raise RuntimeError(f"nckv::{name}: cache {tuple(k_cache.shape)} does not match B={B}, Hkv={Hkv}")
    sb, st = _cache_strides(name, k_cache)
    k, v = k.contiguous(), v.contiguous()
    idx, stream, ws = _launch_ctx(k, B, Hkv, Hkv)
    with _device_guard(idx):
        rc = _F_APPEND(k.data_ptr(), v.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(), cache_seqlens.data_ptr(), B,
                       T_new, Hkv, D, k_cache.size(1), sb, st, ws.data_ptr(), stream)
    if rc < 0:
        _lib.check("nckv_append", rc)


_NS.impl("append_kv", _append_kv, "CUDA")
_NS.impl("append_kv", _append_kv, "CPU")

# ------------------------------------------------------------------------------------------------
# decode attention (T_new == 1)
# ------------------------------------------------------------------------------------------------
_NS.define("decode_attn(Tensor q, Tensor k_cache, Tensor v_cache, Tensor cache_seqlens, int seqlen_offset, "
           "int window_left, int kv_begin, int kv_end, bool partial) -> (Tensor, Tensor, Tensor)")


def _decode_attn_core(q, k_cache, v_cache, cache_seqlens, seqlen_offset, window_left, kv_begin, kv_end, partial,
                      out_f32=None, lse=None):
    name = "decode_attn"
    _require_cuda(name, q, k_cache, v_cache, cache_seqlens)
    _require_bf16(name, q, k_cache, v_cache)
    if cache_seqlens.dtype != torch.int32:
        raise RuntimeError("nckv::decode_attn: cache_seqlens must be int32")
    if q.dim() != 3 or q.size(2) != HEAD_DIM:
        raise RuntimeError(f"nckv::{name}: q must be (B, Hq, {HEAD_DIM}), got {tuple(q.shape)}")
    B, Hq, D = q.shape
    if k_cache.shape != v_cache.shape or k_cache.stride() != v_cache.stride():
        raise RuntimeError(f"nckv::{name}: k_cache and v_cache must share shape and strides")
    Hkv = k_cache.size(2)
    if k_cache.size(0) != B or Hq % Hkv:
        raise RuntimeError(f"nckv::{name}: cache {tuple(k_cache.shape)} does not match q {tuple(q.shape)}")
    sb, st = _cache_strides(name, k_cache)
    q = q.contiguous()
    out = torch.empty_like(q)
    if partial:
        if out_f32 is None:
            out_f32 = torch.empty(B, Hq, D, dtype=torch.float32, device=q.device)
            lse = torch.empty(B, Hq, dtype=torch.float32, device=q.device)
        elif (out_f32.dtype != torch.float32 or lse.dtype != torch.float32 or out_f32.numel() != B * Hq * D or
              lse.numel() != B * Hq or not out_f32.is_contiguous() or not lse.is_contiguous() or out_f32.data_ptr() % 16):
            raise RuntimeError(f"nckv::{name}: out_f32 / lse buffers do not fit (B={B}, Hq={Hq})")
    else:
        out_f32 = lse = None
    idx, stream, ws = _launch_ctx(q, B, Hq, Hkv)
    with _device_guard(idx):
        rc = _F_DECODE(q.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(), cache_seqlens.data_ptr(), out.data_ptr(),
                       out_f32.data_ptr() if partial else None, lse.data_ptr() if partial else None, B, Hq, Hkv, D,
                       k_cache.size(1), sb, st, seqlen_offset, window_left, kv_begin, kv_end, ws.data_ptr(), ws.numel(),
                       stream)
    if rc < 0:
        _lib.check("nckv_decode_attn", rc)
    return out, out_f32, lse


def _decode_attn_op(q, k_cache, v_cache, cache_seqlens, seqlen_offset, window_left, kv_begin, kv_end, partial):
    out, out_f32, lse = _decode_attn_core(q, k_cache, v_cache, cache_seqlens, seqlen_offset, window_left, kv_begin,
                                          kv_end, partial)
    if not partial:  # the op schema returns three tensors
        out_f32, lse = out.new_empty(0, dtype=torch.float32), out.new_empty(0, dtype=torch.float32)
    return out, out_f32, lse


_NS.impl("decode_attn", _decode_attn_op, "CUDA")
_NS.impl("decode_attn", _decode_attn_op, "CPU")

# ------------------------------------------------------------------------------------------------
# dense prefill attention (T_new >= 1)
# ------------------------------------------------------------------------------------------------
_NS.define("prefill_attn(Tensor q, Tensor k, Tensor v, Tensor? cache_seqlens, int window_left) -> Tensor")


def _prefill_attn(q, k, v, cache_seqlens, window_left):
    name = "prefill_attn"
    _require_cuda(name, q, k, v, cache_seqlens)
    _require_bf16(name, q, k, v)
    if cache_seqlens is not None and cache_seqlens.dtype != torch.int32:
        raise RuntimeError("nckv::prefill_attn: cache_seqlens must be int32")
    if q.dim() != 4 or q.size(3) != HEAD_DIM:
        raise RuntimeError(f"nckv::{name}: q must be (B, T, Hq, {HEAD_DIM}), got {tuple(q.shape)}")
    B, T_new, Hq, D = q.shape
    if k.shape != v.shape or k.stride() != v.stride():
        raise RuntimeError(f"nckv::{name}: k and v must share shape and strides")
    Hkv = k.size(2)
    if k.size(0) != B or Hq % Hkv:
        raise RuntimeError(f"nckv::{name}: k {tuple(k.shape)} does not match q {tuple(q.shape)}")
    sb, st = _cache_strides(name, k)
    q = q.contiguous()
    out = torch.empty_like(q)
    idx, stream, ws = _launch_ctx(q, B, Hq, Hkv)
    with _device_guard(idx):
        rc = _F_PREFILL(q.data_ptr(), k.data_ptr(), v.data_ptr(), cache_seqlens.data_ptr() if cache_seqlens is not None else None,
                        out.data_ptr(), B, T_new, Hq, Hkv, D, k.size(1), sb, st, window_left, ws.data_ptr(), stream)
    if rc < 0:
        _lib.check("nckv_prefill_attn", rc)
    return out


_NS.impl("prefill_attn", _prefill_attn, "CUDA")
_NS.impl("prefill_attn", _prefill_attn, "CPU")

# ------------------------------------------------------------------------------------------------
# flash_attn_func for training: forward that keeps the log-sum-exp, and backward
# ------------------------------------------------------------------------------------------------
def _check_train_qkv(name, q, k, v):
    _require_cuda(name, q, k, v)
    _require_bf16(name, q, k, v)
    if q.dim() != 4 or q.size(3) != HEAD_DIM:
        raise RuntimeError(f"nckv::{name}: q must be (B, T, Hq, {HEAD_DIM}), got {tuple(q.shape)}")
    B, T, Hq, _ = q.shape
    if k.shape != v.shape or k.dim() != 4 or k.size(0) != B or k.size(1) != T or k.size(3) != HEAD_DIM or Hq % k.size(2):
        raise RuntimeError(f"nckv::{name}: k/v {tuple(k.shape)} / {tuple(v.shape)} do not match q {tuple(q.shape)}")
    return B, T, Hq, k.size(2)


def flash_attn_fwd(q, k, v, window_left=-1):
    """Causal attention (left window) over plain (B, T, H, D) tensors; returns (out, lse (B, Hq, T) fp32)."""
    name = "flash_attn_fwd"
    B, T, Hq, Hkv = _check_train_qkv(name, q, k, v)
    q, k, v = q.contiguous(), k.contiguous(), v.contiguous()
    out = torch.empty_like(q)
    lse = torch.empty(B, Hq, T, dtype=torch.float32, device=q.device)
    idx, stream, ws = _launch_ctx(q, B, Hq, Hkv)
    with _device_guard(idx):
        rc = _lib.call("nckv_flash_attn_fwd", _ptr(q), _ptr(k), _ptr(v), _ptr(out), _ptr(lse), B, T, Hq, Hkv, HEAD_DIM,
                       int(window_left), _ptr(ws), stream)
    if rc < 0:
        _lib.check("nckv_flash_attn_fwd", rc)
    return out, lse


def flash_attn_bwd(q, k, v, out, dout, lse, window_left=-1):
    """Gradients (dq, dk, dv) of flash_attn_fwd's output with respect to q, k, v."""
    name = "flash_attn_bwd"
    B, T, Hq, Hkv = _check_train_qkv(name, q, k, v)
    _require_cuda(name, out, dout, lse)
    _require_bf16(name, out, dout)
    if out.shape != q.shape or dout.shape != q.shape or tuple(lse.shape) != (B, Hq, T) or lse.dtype != torch.float32:
        raise RuntimeError(f"nckv::{name}: out/dout must have q's shape and lse must be fp32 (B, Hq, T)")
    q, k, v, out, dout, lse = (t.contiguous() for t in (q, k, v, out, dout, lse))
    dq, dk, dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
    scratch = torch.empty(_lib.call("nckv_flash_attn_bwd_workspace_bytes", B, T, Hq), dtype=torch.uint8, device=q.device)
    idx = q.device.index if q.device.index is not None else torch.cuda.current_device()
    with _device_guard(idx):
        rc = _lib.call("nckv_flash_attn_bwd", _ptr(q), _ptr(k), _ptr(v), _ptr(out), _ptr(dout), _ptr(lse), _ptr(dq), _ptr(dk),
                       _ptr(dv), _ptr(scratch), B, T, Hq, Hkv, HEAD_DIM, int(window_left), _stream(idx))
    if rc < 0:
        _lib.check("nckv_flash_attn_bwd", rc)
    _bwd_status[idx] = scratch[-256:-252].view(torch.int32)  # the call's device status word; read_status() looks at it
    return dq, dk, dv


class FlashAttnTrainFunction(torch.autograd.Function):
    """flash_attn_func with a backward pass: both directions run libnckv kernels."""

    @staticmethod
    def forward(ctx, q, k, v, window_left):
        out, lse = flash_attn_fwd(q, k, v, window_left)
        ctx.save_for_backward(q, k, v, out, lse)
        ctx.window_left = window_left
        return out

    @staticmethod
    def backward(ctx, dout):
        q, k, v, out, lse = ctx.saved_tensors
        dq, dk, dv = flash_attn_bwd(q, k, v, out, dout.to(torch.bfloat16), lse, ctx.window_left)
        return dq, dk, dv, None


# ------------------------------------------------------------------------------------------------
# prefill broadcast and LSE combine
# ------------------------------------------------------------------------------------------------
_NS.define("prefill_broadcast(Tensor src_k, Tensor src_v, Tensor(a!) dst_k, Tensor(b!) dst_v, "
           "Tensor(c!)? dst_seqlens, int p) -> ()")


def _prefill_broadcast(src_k, src_v, dst_k, dst_v, dst_seqlens, p):
    name = "prefill_broadcast"
    _require_cuda(name, src_k, src_v, dst_k, dst_v, dst_seqlens)
    for t in (src_k, src_v, dst_k, dst_v):
        if t.dim() != 5 or not t.is_contiguous():
            raise RuntimeError(f"nckv::{name}: caches must be contiguous (L, B, T, Hkv, D) tensors")
        if t.dtype != dst_k.dtype or t.element_size() != 2:
            raise RuntimeError(f"nckv::{name}: caches must share a 16-bit dtype")
    L, B, T_dst, Hkv, D = dst_k.shape
    if src_k.shape != src_v.shape or dst_k.shape != dst_v.shape:
        raise RuntimeError(f"nckv::{name}: K and V shapes differ")
    if src_k.size(0) != L or src_k.size(1) != 1 or src_k.size(3) != Hkv or src_k.size(4) != D:
        raise RuntimeError(f"nckv::{name}: source {tuple(src_k.shape)} does not match destination {tuple(dst_k.shape)}")
    if dst_seqlens is not None and (dst_seqlens.dtype != torch.int32 or dst_seqlens.numel() != B):
        raise RuntimeError(f"nckv::{name}: dst_seqlens must be int32 of {B} rows")
    with torch.cuda.device(dst_k.device):
        _lib.call("nckv_prefill_broadcast", _ptr(src_k), _ptr(src_v), _ptr(dst_k), _ptr(dst_v), _ptr(dst_seqlens), L, B,
                  int(p), Hkv, D, src_k.size(2), T_dst, _stream(dst_k.device))


_NS.impl("prefill_broadcast", _prefill_broadcast, "CUDA")
_NS.impl("prefill_broadcast", _prefill_broadcast, "CPU")

_NS.define("lse_combine(Tensor parts_o, Tensor parts_lse) -> (Tensor, Tensor)")


def _lse_combine(parts_o, parts_lse):
    name = "lse_combine"
    _require_cuda(name, parts_o, parts_lse)
    if parts_o.dtype != torch.float32 or parts_lse.dtype != torch.float32:
        raise RuntimeError("nckv::lse_combine: partials must be float32")
    n_parts = parts_o.size(0)
    D = parts_o.size(-1)
    rows = parts_lse[0].numel()
    if parts_o[0].numel() != rows * D or parts_lse.size(0) != n_parts:
        raise RuntimeError(f"nckv::{name}: shapes {tuple(parts_o.shape)} / {tuple(parts_lse.shape)} do not match")
    # each part must be dense; the parts themselves may be strided (views of one gathered buffer)
    if not parts_o[0].is_contiguous() or parts_o.stride(0) % 4 or parts_o.data_ptr() % 16:
        parts_o = parts_o.contiguous()
    if not parts_lse[0].is_contiguous():
        parts_lse = parts_lse.contiguous()
    out = torch.empty(parts_o.shape[1:], dtype=torch.bfloat16, device=parts_o.device)
    lse = torch.empty(parts_lse.shape[1:], dtype=torch.float32, device=parts_o.device)
    with torch.cuda.device(parts_o.device):
        _lib.call("nckv_lse_combine", _ptr(parts_o), _ptr(parts_lse), n_parts, rows, D,
                  parts_o.stride(0) if n_parts > 1 else rows * D, parts_lse.stride(0) if n_parts > 1 else rows,
                  _ptr(out), _ptr(lse), _stream(parts_o.device))
    return out, lse


_NS.impl("lse_combine", _lse_combine, "CUDA")
_NS.impl("lse_combine", _lse_combine, "CPU")

# ------------------------------------------------------------------------------------------------
# thin Python entry points.  They call the op implementations directly (the dispatcher round trip of
# a Python-defined op costs more than the kernels at decode sizes); the same functions are what
# ``torch.ops.nckv.*`` dispatches to.
# ------------------------------------------------------------------------------------------------


def append_rope_norm(q, k, v, k_cache, v_cache, cache_seqlens, cos, sin, qk_scale=QK_SCALE, eps=RMS_EPS,
                     write_slots=None, split=None):
    """RoPE + QK-norm + scale on q and k, append k/v at ``cache_seqlens`` (per row); returns q'.
    With ``write_slots`` (int32 per row; sequence-split caches) the position still comes from
    ``cache_seqlens`` but k/v are written at ``write_slots[b]``, or not at all where it is -1.
    With ``split=(world, rank, block)`` the kernel works those slots out itself from the global
    ``cache_seqlens`` (block-cyclic ownership; only the owner of the position stores k/v)."""
    return _append_rope_norm(q, k, v, k_cache, v_cache, cache_seqlens, cos, sin, qk_scale, eps, write_slots, split)


def decode_attention_split(q, k_cache, v_cache, cache_seqlens, split, part_out, part_lse, seqlen_offset=1,
                           peer_ptrs=None, step_counter=None):
    """One-token attention over this rank's block-cyclic part of the keys (``split = (world, rank,
    block)``; ``cache_seqlens`` are the global lengths).  Fills ``part_out`` (B, Hq, D) fp32 and
    ``part_lse`` (B, Hq) fp32.  With ``peer_ptrs`` (a ctypes array of every rank's exchange buffer)
    the merge kernel also pushes the packed partial to all peers and releases the step's flags."""
    name = "decode_attn_split"
    _require_cuda(name, q, k_cache, v_cache, cache_seqlens, part_out, part_lse)
    _require_bf16(name, q, k_cache, v_cache)
    if cache_seqlens.dtype != torch.int32:
        raise RuntimeError(f"nckv::{name}: cache_seqlens must be int32")
    if q.dim() != 3 or q.size(2) != HEAD_DIM:
        raise RuntimeError(f"nckv::{name}: q must be (B, Hq, {HEAD_DIM}), got {tuple(q.shape)}")
    B, Hq, D = q.shape
    if k_cache.shape != v_cache.shape or k_cache.stride() != v_cache.stride():
        raise RuntimeError(f"nckv::{name}: k_cache and v_cache must share shape and strides")
    Hkv = k_cache.size(2)
    if k_cache.size(0) != B or Hq % Hkv:
        raise RuntimeError(f"nckv::{name}: cache {tuple(k_cache.shape)} does not match q {tuple(q.shape)}")
    if (part_out.dtype != torch.float32 or part_lse.dtype != torch.float32 or part_out.numel() != B * Hq * D or
            part_lse.numel() != B * Hq or not part_out.is_contiguous() or not part_lse.is_contiguous()):
        raise RuntimeError(f"nckv::{name}: part_out / part_lse buffers do not fit (B={B}, Hq={Hq})")
    sb, st = _cache_strides(name, k_cache)
    q = q.contiguous()
    world, rank, block = split
    idx, stream, ws = _launch_ctx(q, B, Hq, Hkv)
    with _device_guard(idx):
        rc = _lib.lib.nckv_decode_attn_split(q.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(), cache_seqlens.data_ptr(),
                                             part_out.data_ptr(), part_lse.data_ptr(), B, Hq, Hkv, D, k_cache.size(1), sb, st,
                                             seqlen_offset, world, rank, block, peer_ptrs,
                                             step_counter.data_ptr() if step_counter is not None else None,
                                             ws.data_ptr(), ws.numel(), stream)
    if rc < 0:
        _lib.check("nckv_decode_attn_split", rc)


def append_kv(k, v, k_cache, v_cache, cache_seqlens):
    """Write already-transformed k/v at ``cache_seqlens`` (per row)."""
    _append_kv(k, v, k_cache, v_cache, cache_seqlens)


def decode_attention(q, k_cache, v_cache, cache_seqlens, seqlen_offset=1, window_left=-1, kv_begin=0, kv_end=0,
                     partial=False, out_f32=None, lse=None):
    """One-token attention over the cache. q: (B, Hq, D). With ``partial`` also returns the fp32
    normalised output and the natural-log sum-exp (for a cross-GPU combine)."""
    out, out_f32, lse = _decode_attn_core(q, k_cache, v_cache, cache_seqlens, seqlen_offset, window_left, kv_begin,
                                          kv_end, partial, out_f32, lse)
    return (out, out_f32, lse) if partial else out


def kv_split_plan(cache_seqlens, world, rank, block, T_new=1):
    """Block-cyclic sequence split: (keys of each row this shard holds after the append, local
    write index of the new token or -1) as two int32 tensors."""
    _require_cuda("kv_split_plan", cache_seqlens)
    B = cache_seqlens.numel()
    local_len = torch.empty_like(cache_seqlens)
    slot = torch.empty_like(cache_seqlens)
    idx = cache_seqlens.device.index
    with _device_guard(idx):
        _lib.call("nckv_kv_split_plan", cache_seqlens.data_ptr(), B, T_new, world, rank, block, local_len.data_ptr(),
                  slot.data_ptr(), torch.cuda.current_stream(idx).cuda_stream)
    return local_len, slot


def decode_key_ranges(cache_seqlens, T_max, seqlen_offset=1, window_left=-1, kv_begin=0, kv_end=0, split=(0, 0, 0)):
    """Key positions [begin, end) per row that decode_attention reads for these arguments, as two
    int32 tensors (computed on the device by the routine the attention kernels use).  With
    ``split = (world, rank, block)`` the ranges are local indices of that block-cyclic shard."""
    _require_cuda("decode_key_ranges", cache_seqlens)
    B = cache_seqlens.numel()
    begin = torch.empty_like(cache_seqlens)
    end = torch.empty_like(cache_seqlens)
    idx = cache_seqlens.device.index
    ws = workspace(cache_seqlens.device, 1, 1, 1)
    with _device_guard(idx):
        _lib.call("nckv_decode_key_ranges", cache_seqlens.data_ptr(), B, T_max, seqlen_offset, window_left, kv_begin,
                  kv_end, int(split[0]), int(split[1]), int(split[2]), begin.data_ptr(), end.data_ptr(), ws.data_ptr(), torch.cuda.current_stream(idx).cuda_stream)
    return begin, end


def prefill_attention(q, k, v, cache_seqlens=None, window_left=-1):
    """Dense causal attention of T_new query tokens per row against a cache view or plain k/v."""
    return _prefill_attn(q, k, v, cache_seqlens, window_left)


def prefill_broadcast(src_k, src_v, dst_k, dst_v, dst_seqlens, p):
    """Copy the first p tokens of a batch-1 (L,1,T,H,D) cache into all rows of (L,B,T',H,D)."""
    _prefill_broadcast(src_k, src_v, dst_k, dst_v, dst_seqlens, p)


def lse_combine(parts_o, parts_lse):
    """Merge partial attention results over disjoint key ranges; returns (bf16 out, fp32 lse)."""
    return _lse_combine(parts_o, parts_lse)


# ------------------------------------------------------------------------------------------------
# paged KV storage: pools (n_pages, page_tokens, Hkv, D) + an int32 block table (B, max_pages)
# ------------------------------------------------------------------------------------------------
PAGE_TILE = _lib.lib.nckv_paged_tile_tokens()  # page_tokens must be a multiple of this


def _pool_strides(name, pool, table, B):
    if pool.dim() != 4 or pool.size(3) != HEAD_DIM or pool.stride(3) != 1 or pool.stride(2) != HEAD_DIM:
        raise RuntimeError(f"nckv::{name}: pool must be (n_pages, page_tokens, Hkv, {HEAD_DIM}) with packed heads, got "
                           f"{tuple(pool.shape)} / {pool.stride()}")
    if table.dtype != torch.int32 or table.dim() != 2 or table.size(0) != B or not table.is_contiguous() or not table.is_cuda:
        raise RuntimeError(f"nckv::{name}: block_table must be a contiguous CUDA int32 (B={B}, max_pages) tensor")
    if pool.size(1) % PAGE_TILE:
        raise RuntimeError(f"nckv::{name}: page_tokens={pool.size(1)} must be a multiple of {PAGE_TILE}")
    return pool.stride(0), pool.stride(1)


def append_rope_norm_paged(q, k, v, k_pool, v_pool, block_table, cache_seqlens, cos, sin, qk_scale=QK_SCALE, eps=RMS_EPS):
    """``append_rope_norm`` into paged storage: k/v of row b's token at position p go to page
    ``block_table[b, p // page_tokens]``.  Returns q'."""
    name = "append_rope_norm_paged"
    _require_cuda(name, q, k, v, k_pool, v_pool, cache_seqlens, cos, sin)
    _require_bf16(name, q, k, v, k_pool, v_pool, cos, sin)
    if cache_seqlens.dtype != torch.int32:
        raise RuntimeError(f"nckv::{name}: cache_seqlens must be int32")
    B, T_new, Hq, D = q.shape
    Hkv = k.size(2)
    if k.shape != (B, T_new, Hkv, D) or v.shape != k.shape:
        raise RuntimeError(f"nckv::{name}: k/v shapes {tuple(k.shape)}/{tuple(v.shape)} do not match q {tuple(q.shape)}")
    if k_pool.shape != v_pool.shape or k_pool.stride() != v_pool.stride() or k_pool.size(2) != Hkv:
        raise RuntimeError(f"nckv::{name}: pools must share shape and strides and hold {Hkv} kv heads")
    sp, st = _pool_strides(name, k_pool, block_table, B)
    cos2, sin2 = cos.reshape(-1, D // 2), sin.reshape(-1, D // 2)
    if not (cos2.is_contiguous() and sin2.is_contiguous()):
        cos2, sin2 = cos2.contiguous(), sin2.contiguous()
    q, k, v = q.contiguous(), k.contiguous(), v.contiguous()
    q_out = torch.empty_like(q)
    idx, stream, ws = _launch_ctx(q, B, Hq, Hkv)
    with _device_guard(idx):
        _lib.call("nckv_append_rope_norm_paged", q.data_ptr(), k.data_ptr(), v.data_ptr(), q_out.data_ptr(),
                  k_pool.data_ptr(), v_pool.data_ptr(), block_table.data_ptr(), cache_seqlens.data_ptr(), cos2.data_ptr(),
                  sin2.data_ptr(), B, T_new, Hq, Hkv, D, k_pool.size(1), block_table.size(1), k_pool.size(0), sp, st,
                  cos2.size(0), qk_scale, eps, ws.data_ptr(), stream)
    return q_out


def decode_attention_paged(q, k_pool, v_pool, block_table, cache_seqlens, seqlen_offset=1, window_left=-1):
    """``decode_attention`` over paged storage. q: (B, Hq, D); returns (B, Hq, D) bf16."""
    name = "decode_attn_paged"
    _require_cuda(name, q, k_pool, v_pool, cache_seqlens)
    _require_bf16(name, q, k_pool, v_pool)
    if cache_seqlens.dtype != torch.int32:
        raise RuntimeError(f"nckv::{name}: cache_seqlens must be int32")
    if q.dim() != 3 or q.size(2) != HEAD_DIM:
        raise RuntimeError(f"nckv::{name}: q must be (B, Hq, {HEAD_DIM}), got {tuple(q.shape)}")
    B, Hq, D = q.shape
    Hkv = k_pool.size(2)
    if k_pool.shape != v_pool.shape or k_pool.stride() != v_pool.stride() or Hq % Hkv:
        raise RuntimeError(f"nckv::{name}: pools {tuple(k_pool.shape)} / {tuple(v_pool.shape)} do not fit q {tuple(q.shape)}")
    sp, st = _pool_strides(name, k_pool, block_table, B)
    q = q.contiguous()
    out = torch.empty_like(q)
    idx, stream, ws = _launch_ctx(q, B, Hq, Hkv)
    with _device_guard(idx):
        _lib.call("nckv_decode_attn_paged", q.data_ptr(), k_pool.data_ptr(), v_pool.data_ptr(), block_table.data_ptr(),
                  cache_seqlens.data_ptr(), out.data_ptr(), None, None, B, Hq, Hkv, D, k_pool.size(1), block_table.size(1),
                  k_pool.size(0), sp, st, seqlen_offset, window_left, ws.data_ptr(), ws.numel(), stream)
    return out


def paged_fill(src_k, src_v, k_pool, v_pool, jobs):
    """Copy runs of a batch-1 (L, 1, T, Hkv, D) cache into pages of (L, n_pages, page_tokens, Hkv, D)
    pools; ``jobs`` is a CUDA int32 (n_jobs, 3) tensor of (page, first source token, tokens)."""
    name = "paged_fill"
    _require_cuda(name, src_k, src_v, k_pool, v_pool, jobs)
    for t in (src_k, src_v, k_pool, v_pool):
        if t.dim() != 5 or not t.is_contiguous() or t.element_size() != 2 or t.dtype != k_pool.dtype:
            raise RuntimeError(f"nckv::{name}: caches must be contiguous 5-d tensors of one 16-bit dtype")
    L, n_pages, page_tokens, Hkv, D = k_pool.shape
    if src_k.shape != src_v.shape or v_pool.shape != k_pool.shape or src_k.size(0) != L or src_k.size(1) != 1 or \
            src_k.shape[3:] != k_pool.shape[3:]:
        raise RuntimeError(f"nckv::{name}: source {tuple(src_k.shape)} does not match pools {tuple(k_pool.shape)}")
    if jobs.dtype != torch.int32 or jobs.dim() != 2 or jobs.size(1) != 3 or not jobs.is_contiguous():
        raise RuntimeError(f"nckv::{name}: jobs must be a contiguous int32 (n, 3) tensor")
    if jobs.size(0) == 0:
        return
    with torch.cuda.device(k_pool.device):
        _lib.call("nckv_paged_fill", _ptr(src_k), _ptr(src_v), _ptr(k_pool), _ptr(v_pool), _ptr(jobs), jobs.size(0), L, Hkv, D,
                  src_k.size(2), page_tokens, n_pages, _stream(k_pool.device))


# ------------------------------------------------------------------------------------------------
# decode-time glue of the trunk (bit-exact fusions of the eager elementwise ops)
# ------------------------------------------------------------------------------------------------
def _rows(name, t, C):
    if not t.is_cuda or t.dtype != torch.bfloat16 or t.size(-1) != C or not t.is_contiguous():
        raise RuntimeError(f"nckv::{name} needs contiguous CUDA bfloat16 rows of {C} channels, got {tuple(t.shape)} "
                           f"{t.dtype} on {t.device}")
    return t.data_ptr()


def glue_mix_norm(x, add=None, x0=None, x_backout=None, resid_lambda=1.0, x0_lambda=0.0, backout_lambda=0.0,
                  want_sum=False, want_x=True, want_norm=True, eps=RMS_EPS):
    """One launch for the elementwise ops between two matrix products of the trunk, on (..., C) rows:
    ``a = x (+ add)``; then ``resid_lambda * a + x0_lambda * x0`` (when ``x0`` is given) or
    ``a - backout_lambda * x_backout`` (when ``x_backout`` is given); then rms-norm.  Every step
    rounds to bf16 like the eager op it stands for.  Returns (a or None, y or None, norm or None)."""
    name = "glue_mix_norm"
    C = x.size(-1)
    px = _rows(name, x, C)
    rows = x.numel() // C
    mode = 1 if x0 is not None else (2 if x_backout is not None else 0)
    out_sum = torch.empty_like(x) if (want_sum and add is not None) else None
    out_x = torch.empty_like(x) if want_x else None
    out_norm = torch.empty_like(x) if want_norm else None
    idx = x.device.index
    with _device_guard(idx):
        _lib.call("nckv_glue_mix_norm", px, _rows(name, add, C) if add is not None else None,
                  _rows(name, x0, C) if x0 is not None else None,
                  _rows(name, x_backout, C) if x_backout is not None else None,
                  _ptr(out_sum), _ptr(out_x), _ptr(out_norm), rows, C, mode, float(resid_lambda), float(x0_lambda),
                  float(backout_lambda), float(eps), torch.cuda.current_stream(idx).cuda_stream)
    return out_sum, out_x, out_norm


def glue_relu_sq(h):
    """relu(h)^2 in one launch (MLP.forward, gpt.py:136), bf16 rounding after each of the two eager ops."""
    if not h.is_cuda or h.dtype != torch.bfloat16 or not h.is_contiguous():
        raise RuntimeError("nckv::glue_relu_sq needs a contiguous CUDA bfloat16 tensor")
    out = torch.empty_like(h)
    idx = h.device.index
    with _device_guard(idx):
        _lib.call("nckv_glue_relu_sq", h.data_ptr(), out.data_ptr(), h.numel(), torch.cuda.current_stream(idx).cuda_stream)
    return out


def glue_ve_gate(v, gate_lin, ve):
    """v + 3 * sigmoid(gate_lin)[..., None] * ve in one launch (gpt.py:92-95); v, ve: (..., Hkv, 128),
    gate_lin: (..., Hkv) — the output of the gate's linear layer."""
    for t in (v, gate_lin, ve):
        if not t.is_cuda or t.dtype != torch.bfloat16:
            raise RuntimeError("nckv::glue_ve_gate needs CUDA bfloat16 tensors")
    Hkv, Dh = v.size(-2), v.size(-1)
    rows = v.numel() // (Hkv * Dh)
    if gate_lin.numel() != rows * Hkv or ve.numel() != v.numel():
        raise RuntimeError(f"nckv::glue_ve_gate: shapes {tuple(v.shape)} / {tuple(gate_lin.shape)} / {tuple(ve.shape)} do not match")
    # v may be a column slice of a projection output: (rows..., Hkv, D) with packed heads and one row stride
    row_stride = 0
    if not v.is_contiguous():
        lead = [(n, s) for n, s in zip(v.shape[:-2], v.stride()[:-2]) if n > 1]
        regular = v.stride(-1) == 1 and v.stride(-2) == Dh and all(
            lead[i][1] == lead[i + 1][0] * lead[i + 1][1] for i in range(len(lead) - 1))
        if regular and lead and lead[-1][1] % 8 == 0 and v.data_ptr() % 16 == 0:
            row_stride = lead[-1][1]
        else:
            v = v.contiguous()
    gate_lin, ve = gate_lin.contiguous(), ve.contiguous()
    out = torch.empty(v.shape, dtype=v.dtype, device=v.device)
    idx = v.device.index
    with _device_guard(idx):
        _lib.call("nckv_glue_ve_gate", v.data_ptr(), row_stride, gate_lin.data_ptr(), ve.data_ptr(), out.data_ptr(), rows,
                  Hkv, Dh, torch.cuda.current_stream(idx).cuda_stream)
    return out


class HostDecodeStep:
    """A decode step of one layer for activations that live in host memory.

    Owns the pinned host blocks and the device staging buffers of a fixed (B, Hq, Hkv) shape;
    ``run(k_cache, v_cache, cache_seqlens, window_left)`` copies ``self.q / self.k / self.v`` (views of
    one pinned block, fill them in place) to the device, runs the fused append and the decode
    attention, and returns ``self.out`` (pinned host, valid on return: the call synchronises).
    One C-ABI call per step (nckv_decode_step_host).  ``transfer="copy"`` enqueues an H2D and a D2H
    copy around the kernels; ``transfer="mapped"`` lets the kernels read the pinned inputs and write
    the pinned output themselves (same bytes over PCIe, two operations fewer in the stream)."""

    def __init__(self, B, Hq, Hkv, cos, sin, device, qk_scale=QK_SCALE, eps=RMS_EPS, transfer="copy"):
        if transfer not in ("copy", "mapped"):
            raise ValueError(f"transfer must be 'copy' or 'mapped', not {transfer!r}")
        self.transfer = transfer
        self.device = torch.device(device)
        if self.device.type != "cuda":
            raise RuntimeError("HostDecodeStep needs a CUDA device; the KV-cache decode path has no CPU implementation")
        self.B, self.Hq, self.Hkv = B, Hq, Hkv
        nq, nk = B * Hq * HEAD_DIM, B * Hkv * HEAD_DIM
        self.host_in = torch.empty(nq + 2 * nk, dtype=torch.bfloat16).pin_memory()
        self.q = self.host_in[:nq].view(B, Hq, HEAD_DIM)
        self.k = self.host_in[nq:nq + nk].view(B, Hkv, HEAD_DIM)
        self.v = self.host_in[nq + nk:].view(B, Hkv, HEAD_DIM)
        self.out = torch.empty(B, Hq, HEAD_DIM, dtype=torch.bfloat16).pin_memory()
        self._dev_in = torch.empty(nq + 2 * nk, dtype=torch.bfloat16, device=self.device)
        self._q_rot = torch.empty(B, Hq, HEAD_DIM, dtype=torch.bfloat16, device=self.device)
        self._out_dev = torch.empty_like(self._q_rot)
        _require_bf16("decode_step_host", cos, sin)
        self._cos = cos.reshape(-1, HEAD_DIM // 2).contiguous()
        self._sin = sin.reshape(-1, HEAD_DIM // 2).contiguous()
        self.qk_scale, self.eps = qk_scale, eps
        self._fn = _lib.lib.nckv_decode_step_host
        self._plans = {}
        self._ws_need = _lib.lib.nckv_workspace_bytes(B, Hq, Hkv, HEAD_DIM)

    def _make_plan(self, k_cache, v_cache, cache_seqlens):
        name = "decode_step_host"
        _require_cuda(name, k_cache, v_cache, cache_seqlens)
        _require_bf16(name, k_cache, v_cache)
        if k_cache.shape != v_cache.shape or k_cache.stride() != v_cache.stride():
            raise RuntimeError(f"nckv::{name}: k_cache and v_cache must share shape and strides")
        if k_cache.size(0) != self.B or k_cache.size(2) != self.Hkv or cache_seqlens.dtype != torch.int32:
            raise RuntimeError(f"nckv::{name}: cache {tuple(k_cache.shape)} / seqlens do not match B={self.B}, Hkv={self.Hkv}")
        sb, st = _cache_strides(name, k_cache)
        mapped = self.transfer == "mapped"
        head = (self.host_in.data_ptr(), None if mapped else self._dev_in.data_ptr(), self._q_rot.data_ptr(),
                None if mapped else self._out_dev.data_ptr(), self.out.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(),
                cache_seqlens.data_ptr(), self._cos.data_ptr(), self._sin.data_ptr())
        mid = (self.B, self.Hq, self.Hkv, HEAD_DIM, k_cache.size(1), sb, st, self._cos.size(0), self.qk_scale, self.eps)
        return k_cache.device.index, head, mid

    def run(self, k_cache, v_cache, cache_seqlens, window_left=-1):
        # argument checks and the constant part of the argument list are done once per distinct
        # (cache, seqlens) triple: a decode loop calls this with the same tensors every step
        key = (k_cache.data_ptr(), v_cache.data_ptr(), cache_seqlens.data_ptr(), k_cache.shape, k_cache.stride(0),
               k_cache.dtype, cache_seqlens.dtype)
        plan = self._plans.get(key)
        if plan is None:
            plan = self._make_plan(k_cache, v_cache, cache_seqlens)
            if len(self._plans) >= 64:
                self._plans.clear()
            self._plans[key] = plan
        idx, head, mid = plan
        stream = torch.cuda.current_stream(idx).cuda_stream
        ws = _workspaces.get((idx, stream))
        if ws is None or ws.numel() < self._ws_need:
            ws = workspace(k_cache.device, self.B, self.Hq, self.Hkv)
        with _device_guard(idx):
            rc = self._fn(*head, *mid, int(window_left), ws.data_ptr(), ws.numel(), stream)
        if rc < 0:
            _lib.check("nckv_decode_step_host", rc)
        return self.out
