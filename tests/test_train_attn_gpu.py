"""flash_attn_func with gradients: the library's forward (log-sum-exp kept) and backward kernels against
autograd through an fp32 masked softmax of the same bf16 inputs (what F.scaled_dot_product_attention
computes on the reference's path, flash_attention.py:107-128 reached from gpt.py:108).

Tolerances: the forward within 1e-2 of the fp32 result relative to its largest value; each gradient
within 2e-2 of the fp32 gradient relative to that gradient's largest value (bf16 P, dS and outputs).
"""
import math

import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda"
BF = torch.bfloat16


def _reference(q, k, v, window_left):
    """fp32 attention of bf16 inputs with the causal / left-window mask, differentiable."""
    B, T, Hq, D = q.shape
    Hkv = k.size(2)
    qf, kf, vf = (t.detach().float().requires_grad_(True) for t in (q, k, v))
    kr = kf.repeat_interleave(Hq // Hkv, dim=2)
    vr = vf.repeat_interleave(Hq // Hkv, dim=2)
    s = torch.einsum("bthd,bshd->bhts", qf, kr) / math.sqrt(D)
    pos = torch.arange(T, device=q.device)
    mask = pos[None, :] <= pos[:, None]
    if window_left >= 0:
        mask &= (pos[:, None] - pos[None, :]) <= window_left
    s = s.masked_fill(~mask, float("-inf"))
    p = torch.softmax(s, dim=-1)
    out = torch.einsum("bhts,bshd->bthd", p, vr)
    lse = torch.logsumexp(s, dim=-1)  # (B, Hq, T)
    return qf, kf, vf, out, lse


@pytest.mark.parametrize("B,T,Hq,Hkv,window", [
    (2, 256, 4, 4, -1),
    (1, 200, 8, 2, -1),      # GQA, T not a multiple of the tiles
    (2, 320, 4, 2, 96),      # sliding window
    (1, 1000, 2, 2, 256),
    (1, 64, 2, 1, -1),
    (3, 33, 2, 2, 7),
    (1, 1500, 8, 2, -1),     # a dozen 128-row blocks, four q heads per kv head
    (1, 2048, 4, 4, 1024),   # window wider than a block
    (2, 130, 4, 1, 128),     # a block and two rows, window of exactly one block
])
def test_flash_attn_func_forward_and_backward(B, T, Hq, Hkv, window):
    from nanochat_b200 import ops
    from nanochat_b200.flash_attention import flash_attn
    gen = torch.Generator(device=DEV).manual_seed(7 * T + Hq)
    q = torch.randn(B, T, Hq, 128, generator=gen, device=DEV).to(BF).requires_grad_(True)
    k = torch.randn(B, T, Hkv, 128, generator=gen, device=DEV).to(BF).requires_grad_(True)
    v = torch.randn(B, T, Hkv, 128, generator=gen, device=DEV).to(BF).requires_grad_(True)
    dout = torch.randn(B, T, Hq, 128, generator=gen, device=DEV).to(BF)

    out = flash_attn.flash_attn_func(q, k, v, causal=True, window_size=(window, 0))
    assert out.requires_grad and out.dtype == BF
    out.backward(dout)
    torch.cuda.synchronize()
    assert ops.read_status(DEV) == 0

    qf, kf, vf, out_ref, lse_ref = _reference(q, k, v, window)
    out_ref.backward(dout.float())
    assert (out.float() - out_ref).abs().max() <= 1e-2 * out_ref.abs().max()
    _, lse = ops.flash_attn_fwd(q.detach(), k.detach(), v.detach(), window)
    assert torch.allclose(lse, lse_ref, atol=2e-3, rtol=1e-3)
    for name, got, ref in (("dq", q.grad, qf.grad), ("dk", k.grad, kf.grad), ("dv", v.grad, vf.grad)):
        err = (got.float() - ref).abs().max().item()
        scale = ref.abs().max().item()
        assert err <= 2e-2 * scale, f"{name}: max error {err:.4g} against a largest value of {scale:.4g}"


def test_flash_attn_func_without_grad_takes_the_inference_path():
    from nanochat_b200.flash_attention import flash_attn
    gen = torch.Generator(device=DEV).manual_seed(3)
    q, k, v = (torch.randn(1, 130, 2, 128, generator=gen, device=DEV).to(BF) for _ in range(3))
    a = flash_attn.flash_attn_func(q, k, v, causal=True, window_size=(-1, 0))
    b = flash_attn.flash_attn_func(q.clone().requires_grad_(True), k, v, causal=True, window_size=(-1, 0))
    assert not a.requires_grad and b.requires_grad
    assert torch.equal(a, b.detach())  # the same kernel either way


def test_backward_is_deterministic():
    from nanochat_b200 import ops
    gen = torch.Generator(device=DEV).manual_seed(11)
    q = torch.randn(2, 300, 4, 128, generator=gen, device=DEV).to(BF)
    k = torch.randn(2, 300, 2, 128, generator=gen, device=DEV).to(BF)
    v = torch.randn(2, 300, 2, 128, generator=gen, device=DEV).to(BF)
    dout = torch.randn(2, 300, 4, 128, generator=gen, device=DEV).to(BF)
    out, lse = ops.flash_attn_fwd(q, k, v, -1)
    first = ops.flash_attn_bwd(q, k, v, out, dout, lse, -1)
    second = ops.flash_attn_bwd(q, k, v, out, dout, lse, -1)
    for a, b in zip(first, second):
        assert torch.equal(a.view(torch.int16), b.view(torch.int16))
