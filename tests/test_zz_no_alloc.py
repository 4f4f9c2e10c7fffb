"""nckv_decode_attn_static: the decode-attention entry point for callers that cannot allocate.

Some callers of this library have no way to get device memory when they call it: an inference
server that gave every free byte to the KV cache at start-up, or host code that is not allowed to
touch an allocator on its hot path.  For them the library carries its own scratch (a fixed device
array) and this entry point uses it.  The test calls it through the C ABI exactly as such a caller
would, twice in a row on the same shapes with different data, and checks each result against the
regular entry point (which is given a workspace) and against the numpy oracle, to the tolerance the
attention tests use.  The file is named so that pytest collects it last.
"""
import ctypes

import numpy as np
import pytest
import torch

from oracle import kv_oracle as O

pytestmark = pytest.mark.gpu
ATOL = RTOL = 1e-2  # the attention tolerance of tests/test_kernels_gpu.py


def _call(lib_call, name, q, kc, vc, seqlens, out, window, tail_args):
    B, Hq, D = q.shape
    Hkv, T_max = kc.size(2), kc.size(1)
    lib_call(name, q.data_ptr(), kc.data_ptr(), vc.data_ptr(), seqlens.data_ptr(), out.data_ptr(), None, None,
             B, Hq, Hkv, D, T_max, kc.stride(0), kc.stride(1), 1, window, 0, 0, *tail_args)


@pytest.mark.parametrize("Hq,Hkv,window", [(12, 12, -1), (16, 4, 40)])
def test_static_scratch_entry_point_matches_regular_one(Hq, Hkv, window):
    from nanochat_b200 import _lib, ops
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    B, T_max = 9, 700
    stream = torch.cuda.current_stream(dev).cuda_stream
    gen = torch.Generator(device=dev).manual_seed(1234 + Hq)
    ws = ops.workspace(dev, B, Hq, Hkv)
    status_ptr = ctypes.c_void_p(0)
    for call_no in range(2):  # two calls in a row: the second one meets the first one's leftovers
        seqlens = torch.randint(0, T_max - 1, (B,), generator=gen, device=dev, dtype=torch.int32)
        seqlens[0] = T_max - 1
        q = torch.randn(B, Hq, 128, generator=gen, device=dev).to(torch.bfloat16)
        kc = torch.randn(B, T_max, Hkv, 128, generator=gen, device=dev).to(torch.bfloat16)
        vc = torch.randn(B, T_max, Hkv, 128, generator=gen, device=dev).to(torch.bfloat16)
        expect = torch.empty_like(q)
        got = torch.full_like(q, float("nan"))
        _call(_lib.call, "nckv_decode_attn", q, kc, vc, seqlens, expect, window, (ws.data_ptr(), ws.numel(), stream))
        before = torch.cuda.memory_allocated(dev)
        _call(_lib.call, "nckv_decode_attn_static", q, kc, vc, seqlens, got, window, (ctypes.byref(status_ptr), stream))
        torch.cuda.synchronize(dev)
        assert torch.cuda.memory_allocated(dev) == before
        assert status_ptr.value, "the status word address was not reported"
        assert _lib.call("nckv_read_status", status_ptr, 1, stream) == 0
        assert not torch.isnan(got.float()).any(), f"call {call_no}: output rows were left unwritten"
        assert torch.allclose(got.float(), expect.float(), atol=ATOL, rtol=RTOL), \
            f"call {call_no}: max diff {(got.float() - expect.float()).abs().max().item()}"
        ref, _ = O.attention_kvcache(q.float().cpu().numpy()[:, None], kc.float().cpu().numpy(), vc.float().cpu().numpy(),
                                     seqlens.cpu().numpy(), window_left=window)
        assert np.allclose(got.float().cpu().numpy(), ref[:, 0], atol=ATOL, rtol=RTOL), f"call {call_no}: differs from the oracle"


def test_static_scratch_entry_point_rejects_oversized_shapes():
    from nanochat_b200 import _lib
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    B, Hq, Hkv, T_max = 2, 16, 1, 64  # group size 16 needs more scratch than the built-in array has
    q = torch.zeros(B, Hq, 128, device=dev, dtype=torch.bfloat16)
    kc = torch.zeros(B, T_max, Hkv, 128, device=dev, dtype=torch.bfloat16)
    seqlens = torch.zeros(B, device=dev, dtype=torch.int32)
    out = torch.zeros_like(q)
    with pytest.raises(_lib.NckvError) as e:
        _call(_lib.call, "nckv_decode_attn_static", q, kc, kc.clone(), seqlens, out, -1,
              (None, torch.cuda.current_stream(dev).cuda_stream))
    assert e.value.code == -3 and "scratch" in str(e.value)
