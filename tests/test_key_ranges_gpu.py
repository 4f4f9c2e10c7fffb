"""Integer parity of the device-side bookkeeping, bit-exact against the numpy restatement.

``nckv_decode_key_ranges`` dumps the per-row key ranges from the routine the decode kernels themselves
call (visible-key rule of nanochat/flash_attention.py:83-88 and :94-100); ``nckv_kv_split_plan`` dumps
the block-cyclic owner rule that the *_split kernels apply.  Both are compared with
``oracle.kv_oracle.visible_range`` / ``nanochat_b200.dist.owned_below`` for every benchmark
configuration's seeded lengths and for the edge lengths around each window.
"""
import numpy as np
import pytest
import torch

from oracle import kv_oracle as O

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _expected_ranges(lens, T_max, window, kv_begin, kv_end):
    lo_hi = []
    for L in lens:
        lo, hi = O.visible_range(int(L), 0, 1, window)   # the one new token of a decode step
        if kv_end > kv_begin:
            lo, hi = max(lo, kv_begin), min(hi, kv_end)
            hi = max(hi, lo)
        lo_hi.append((lo, hi))
    return np.array(lo_hi, dtype=np.int32)


def _seeded_lengths():
    """cache_seqlens of every benchmark configuration, drawn as its description says."""
    g = lambda s: torch.Generator().manual_seed(s)
    return {
        "configs[0] decode steps": (np.arange(32, 96, dtype=np.int32), 96),
        "configs[1]": (torch.randint(1, 2048, (32,), dtype=torch.int32, generator=g(2)).numpy(), 2048),
        "configs[2] mid generation": (np.full(64, 767, dtype=np.int32), 1024),
        "configs[3]": (torch.randint(128, 2049, (256,), dtype=torch.int32, generator=g(4)).numpy(), 4096),
        "configs[4]": (torch.randint(32768, 65536, (8,), dtype=torch.int32, generator=g(4)).numpy(), 65536),
    }


@pytest.mark.parametrize("window", [-1, 0, 8, 512, 1024, 2048, 4096])
def test_key_ranges_equal_the_visible_key_rule(window):
    from nanochat_b200 import ops
    cases = dict(_seeded_lengths())
    for T_max in (96, 2048, 4096):  # edge lengths around the window and at the end of the cache
        w = window if window >= 0 else T_max
        edge = sorted({0, 1, max(w - 1, 0), w, w + 1, T_max - 1} & set(range(T_max)))
        cases[f"edges T_max={T_max}"] = (np.array(edge, dtype=np.int32), T_max)
    for name, (lens, T_max) in cases.items():
        shards = [(0, 0), (0, T_max // 3), (T_max // 3, 2 * (T_max // 3)), (2 * (T_max // 3), T_max)]
        for kv_begin, kv_end in shards:
            lens_d = torch.from_numpy(lens).to(DEV)
            begin, end = ops.decode_key_ranges(lens_d, T_max, seqlen_offset=1, window_left=window,
                                               kv_begin=kv_begin, kv_end=kv_end)
            torch.cuda.synchronize()
            got = np.stack([begin.cpu().numpy(), end.cpu().numpy()], axis=1)
            want = _expected_ranges(lens, T_max, window, kv_begin, kv_end)
            assert np.array_equal(got, want), (name, window, kv_begin, kv_end, got[got != want][:8], want[got != want][:8])
            assert ops.read_status(DEV) == 0


def test_key_ranges_flag_and_clamp_invalid_lengths():
    from nanochat_b200 import ops
    lens = torch.tensor([5, -3, 100, 40], dtype=torch.int32, device=DEV)
    begin, end = ops.decode_key_ranges(lens, 64, seqlen_offset=1, window_left=-1)
    torch.cuda.synchronize()
    assert begin.tolist() == [0, 0, 0, 0] and end.tolist() == [6, 0, 64, 41]
    assert ops.read_status(DEV) == 1 | 4  # overflow and negative length, nothing trapped


@pytest.mark.parametrize("world", [1, 2, 3, 8])
@pytest.mark.parametrize("block", [32, 256, 1024])
def test_split_plan_and_split_key_ranges_equal_the_owner_rule(world, block):
    from nanochat_b200 import ops
    from nanochat_b200.dist import owned_below
    for name, (lens, T_max) in _seeded_lengths().items():
        extra = np.array([0, 1, block - 1, block, block + 1, block * world - 1, block * world, T_max - 1], dtype=np.int32)
        lens = np.concatenate([lens, extra[extra < T_max]])
        lens_d = torch.from_numpy(lens).to(DEV)
        for rank in range(world):
            local_len, slot = ops.kv_split_plan(lens_d, world, rank, block)
            cap = owned_below(T_max, world, rank, block)
            begin, end = ops.decode_key_ranges(lens_d, max(cap, 1), seqlen_offset=1, window_left=-1, split=(world, rank, block))
            torch.cuda.synchronize()
            want_len = np.array([owned_below(int(L) + 1, world, rank, block) for L in lens], dtype=np.int32)
            want_slot = np.array([owned_below(int(L), world, rank, block) if (int(L) // block) % world == rank else -1
                                  for L in lens], dtype=np.int32)
            assert np.array_equal(local_len.cpu().numpy(), want_len), (name, world, rank, block)
            assert np.array_equal(slot.cpu().numpy(), want_slot), (name, world, rank, block)
            # the decode kernel's own tables in split mode: local indices [0, keys this shard holds)
            assert begin.abs().sum().item() == 0
            assert np.array_equal(end.cpu().numpy(), np.minimum(want_len, max(cap, 1))), (name, world, rank, block)
            # every position has exactly one owner and local slots are dense
            if rank == 0:
                total = sum(np.array([owned_below(int(L) + 1, world, r, block) for L in lens]) for r in range(world))
                assert np.array_equal(total, lens.astype(np.int64) + 1)
        ops.read_status(DEV)  # lengths at T_max - 1 may legitimately clamp nothing; clear for the next test


def test_split_plan_output_is_complete_before_a_dependent_decode_reads_it():
    """The decode kernels read cache_seqlens before their grid-dependency wait, so whatever produces
    it must not release its dependents early.  Plan -> decode back to back, many times, into a
    poisoned length buffer: every result must equal the one computed from finished lengths."""
    from nanochat_b200 import _lib, ops
    gen = torch.Generator(device=DEV).manual_seed(5)
    B, Hq, Hkv, T, world, block = 16, 8, 2, 2048, 2, 64
    lens = torch.randint(100, T - 1, (B,), generator=gen, device=DEV, dtype=torch.int32)
    q = torch.randn(B, Hq, 128, generator=gen, device=DEV).to(torch.bfloat16)
    cap = T // world
    kc = torch.randn(B, cap, Hkv, 128, generator=gen, device=DEV).to(torch.bfloat16)
    vc = torch.randn(B, cap, Hkv, 128, generator=gen, device=DEV).to(torch.bfloat16)
    stream = torch.cuda.current_stream().cuda_stream
    want_len, _ = ops.kv_split_plan(lens, world, 1, block)
    want = ops.decode_attention(q, kc, vc, want_len, seqlen_offset=0)
    torch.cuda.synchronize()
    local_len = torch.empty_like(lens)
    slot = torch.empty_like(lens)
    for it in range(50):
        local_len.fill_(7 if it % 2 else 100000)  # stale or absurd lengths if read too early
        _lib.call("nckv_kv_split_plan", lens.data_ptr(), B, 1, world, 1, block, local_len.data_ptr(), slot.data_ptr(), stream)
        got = ops.decode_attention(q, kc, vc, local_len, seqlen_offset=0)
        assert torch.equal(got.view(torch.int16), want.view(torch.int16)), f"iteration {it}"
    torch.cuda.synchronize()
    assert ops.read_status(DEV) == 0
