"""Parity of the CUDA kernels (through the nckv custom ops / the C ABI) against the numpy oracle
and against the torch-eager restatement of the reference's bf16 GPU path."""
import os

import numpy as np
import pytest
import torch

from oracle import kv_oracle as O
from oracle import torch_ref as E

pytestmark = pytest.mark.gpu

DEV = "cuda"
BF = torch.bfloat16
# Tolerance of the reference's own differential tests (tests/test_attention_fallback.py:39-45).
ATOL = RTOL = 1e-2


def ops():
    from nanochat_b200 import ops as _ops
    return _ops


def bits(t):
    return t.contiguous().view(torch.int16)


def rel_err(got, ref):
    got, ref = got.double(), ref.double()
    return ((got - ref).abs().max() / ref.abs().max().clamp_min(1e-30)).item()


def make_cache(B, T_max, Hkv, seqlens, gen, layers=None):
    shape = (B, T_max, Hkv, 128) if layers is None else (layers, B, T_max, Hkv, 128)
    k = torch.randn(shape, generator=gen, device=DEV, dtype=torch.float32).to(BF)
    v = torch.randn(shape, generator=gen, device=DEV, dtype=torch.float32).to(BF)
    return k, v


# ------------------------------------------------------------------------------------------------
# (a) fused RoPE + QK-norm + scale + append
# ------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("B,T_new,Hq,Hkv,T_max", [(32, 1, 12, 12, 2048), (5, 1, 16, 4, 300), (3, 7, 4, 2, 64),
                                                  (1, 33, 2, 2, 40), (64, 1, 1, 1, 16)])
def test_append_rope_norm_bit_exact(B, T_new, Hq, Hkv, T_max):
    gen = torch.Generator(device=DEV).manual_seed(100 + B)
    cos, sin = E.rotary_tables(T_max + 8, 128, DEV, BF)
    seqlens = torch.randint(0, T_max - T_new + 1, (B,), generator=gen, device=DEV, dtype=torch.int32)
    seqlens[0] = T_max - T_new  # last slot of the cache
    if B > 1:
        seqlens[1] = 0
    q = torch.randn(B, T_new, Hq, 128, generator=gen, device=DEV).to(BF)
    k = torch.randn(B, T_new, Hkv, 128, generator=gen, device=DEV).to(BF) * 3.0
    v = torch.randn(B, T_new, Hkv, 128, generator=gen, device=DEV).to(BF)
    k_cache, v_cache = make_cache(B, T_max, Hkv, seqlens, gen)
    k_ref, v_ref = k_cache.clone(), v_cache.clone()

    q_out = ops().append_rope_norm(q, k, v, k_cache, v_cache, seqlens, cos, sin)
    assert ops().read_status(DEV) == 0

    # reference bf16 GPU path: eager ops, then the slice-assign, row by row
    q_ref = E.rope_norm_scale_rows(q, cos, sin, seqlens)
    k_new = E.rope_norm_scale_rows(k, cos, sin, seqlens)
    for b, L in enumerate(seqlens.tolist()):
        k_ref[b, L:L + T_new] = k_new[b]
        v_ref[b, L:L + T_new] = v[b]
    assert torch.equal(bits(v_cache), bits(v_ref)), "V bytes differ"
    n_bad_k = (bits(k_cache) != bits(k_ref)).sum().item()
    n_bad_q = (bits(q_out) != bits(q_ref)).sum().item()
    assert n_bad_k == 0, f"{n_bad_k} K cache elements differ from the eager bf16 path"
    assert n_bad_q == 0, f"{n_bad_q} q elements differ from the eager bf16 path"

    # numpy oracle (CPU restatement): identical up to isolated last-bit flips from rsqrt flavour
    cos_np, sin_np = cos[0, :, 0].float().cpu().numpy(), sin[0, :, 0].float().cpu().numpy()
    q_or = O.rope_norm_scale_rows(q.float().cpu().numpy(), cos_np, sin_np, seqlens.cpu().numpy(), bf16=True)
    bad = (O.f32_to_bf16_bits(q_or) != bits(q_out).cpu().numpy().view(np.uint16))
    assert bad.mean() < 1e-3
    assert np.abs(q_or - q_out.float().cpu().numpy()).max() <= 2.0 ** -6


def test_append_statistics_ten_million_elements():
    """Mismatch count against the eager bf16 path over > 10^7 elements (target 0)."""
    gen = torch.Generator(device=DEV).manual_seed(7)
    B, T_new, H = 64, 128, 12
    T_max = 128
    cos, sin = E.rotary_tables(T_max, 128, DEV, BF)
    seqlens = torch.zeros(B, device=DEV, dtype=torch.int32)
    total_bad = 0
    for scale in (1.0, 0.05, 30.0):
        q = (torch.randn(B, T_new, H, 128, generator=gen, device=DEV) * scale).to(BF)
        k = (torch.randn(B, T_new, H, 128, generator=gen, device=DEV) * scale).to(BF)
        v = torch.randn(B, T_new, H, 128, generator=gen, device=DEV).to(BF)
        k_cache = torch.zeros(B, T_max, H, 128, device=DEV, dtype=BF)
        v_cache = torch.zeros_like(k_cache)
        q_out = ops().append_rope_norm(q, k, v, k_cache, v_cache, seqlens, cos, sin)
        q_ref = E.rope_norm_scale(q, cos, sin)
        k_ref = E.rope_norm_scale(k, cos, sin)
        total_bad += (bits(q_out) != bits(q_ref)).sum().item() + (bits(k_cache) != bits(k_ref)).sum().item()
    print(f"append mismatches over {3 * 2 * B * T_new * H * 128} elements: {total_bad}")
    assert total_bad == 0


def test_append_overflow_sets_status_and_skips_row():
    gen = torch.Generator(device=DEV).manual_seed(3)
    B, Hkv, T_max = 3, 2, 8
    seqlens = torch.tensor([2, 8, 7], device=DEV, dtype=torch.int32)  # row 1 is full
    k = torch.randn(B, 1, Hkv, 128, generator=gen, device=DEV).to(BF)
    v = torch.randn(B, 1, Hkv, 128, generator=gen, device=DEV).to(BF)
    k_cache = torch.zeros(B, T_max + 1, Hkv, 128, device=DEV, dtype=BF)[:, :T_max]  # canary row behind each row
    v_cache = torch.zeros(B, T_max + 1, Hkv, 128, device=DEV, dtype=BF)[:, :T_max]
    ops().append_kv(k, v, k_cache, v_cache, seqlens)
    st = ops().read_status(DEV)
    assert st & 1, "overflow bit not set"
    assert ops().read_status(DEV) == 0, "status was not cleared"
    assert torch.equal(k_cache[0, 2], k[0, 0]) and torch.equal(k_cache[2, 7], k[2, 0])
    assert k_cache[1].abs().sum().item() == 0, "full row must be left untouched"
    base = k_cache._base if k_cache._base is not None else k_cache
    assert base[:, T_max].abs().sum().item() == 0, "canary row written"


# ------------------------------------------------------------------------------------------------
# (b) decode attention
# ------------------------------------------------------------------------------------------------
def run_decode_case(B, Hq, Hkv, T_max, seqlens, window, seed, kv_range=(0, 0), check_eager=True):
    gen = torch.Generator(device=DEV).manual_seed(seed)
    seqlens_t = torch.tensor(seqlens, device=DEV, dtype=torch.int32)
    q = torch.randn(B, Hq, 128, generator=gen, device=DEV).to(BF)
    k_cache, v_cache = make_cache(B, T_max, Hkv, seqlens_t, gen)
    partial = kv_range != (0, 0)
    res = ops().decode_attention(q, k_cache, v_cache, seqlens_t, seqlen_offset=1, window_left=window,
                                 kv_begin=kv_range[0], kv_end=kv_range[1], partial=partial)
    torch.cuda.synchronize()
    assert ops().read_status(DEV) == 0
    out = res[0] if partial else res
    ref, ref_lse = O.attention_kvcache(q.float().cpu().numpy()[:, None], k_cache.float().cpu().numpy(),
                                       v_cache.float().cpu().numpy(), np.array(seqlens), window_left=window,
                                       kv_begin=kv_range[0], kv_end=kv_range[1])
    ref = torch.from_numpy(ref[:, 0])
    got = out.float().cpu()
    assert not torch.isnan(got).any()
    assert torch.allclose(got, ref, atol=ATOL, rtol=RTOL), f"max diff {(got - ref).abs().max().item()}"
    assert rel_err(got, ref) <= 1e-2
    if partial:
        lse = res[2].float().cpu().numpy()
        ref_lse = ref_lse[:, 0]
        finite = np.isfinite(ref_lse)
        assert np.array_equal(np.isneginf(lse), ~finite)
        np.testing.assert_allclose(lse[finite], ref_lse[finite], rtol=1e-3, atol=2e-3)
        f32 = res[1].float().cpu()
        assert torch.allclose(f32, ref, atol=ATOL, rtol=RTOL)
    if check_eager and not partial:
        # the reference's own GPU path (SDPA on bf16), run row by row for ragged lengths
        eager = E.kvcache_attention(q[:, None], k_cache, v_cache, None, None, seqlens_t, window)[:, 0]
        assert torch.allclose(out.float(), eager.float(), atol=2e-2, rtol=2e-2)
    return out


@pytest.mark.parametrize("Hq,Hkv", [(2, 2), (12, 12), (16, 4), (8, 1), (16, 1), (24, 2)])
def test_decode_attention_ragged_groups(Hq, Hkv):
    rng = np.random.default_rng(Hq * 31 + Hkv)
    B, T_max = 6, 300
    seqlens = rng.integers(0, T_max - 1, size=B).tolist()
    seqlens[0], seqlens[1] = 0, T_max - 1  # a single key; the full cache
    run_decode_case(B, Hq, Hkv, T_max, seqlens, -1, seed=Hq)


@pytest.mark.parametrize("window", [8, 31, 32, 33, 1024])
def test_decode_attention_window_edges(window):
    w = window
    seqlens = [0, 1, max(w - 2, 0), w - 1, w, w + 1, 2 * w + 5, 70]
    T_max = max(seqlens) + 2
    run_decode_case(len(seqlens), 4, 2, T_max, seqlens, w, seed=window)


def test_decode_attention_config1_shape_and_split_invariance():
    """Benchmark configuration 1: B=32, 12/12 heads, capacity 2048, lengths uniform in [1, 2047] (seed 2)."""
    seqlens = torch.randint(1, 2048, (32,), dtype=torch.int32, generator=torch.Generator().manual_seed(2)).tolist()
    out = run_decode_case(32, 12, 12, 2048, seqlens, -1, seed=2)
    # same rows evaluated alone (different slicing of the tile sequence) must agree closely
    gen = torch.Generator(device=DEV).manual_seed(2)
    q = torch.randn(32, 12, 128, generator=gen, device=DEV).to(BF)
    k_cache, v_cache = make_cache(32, 2048, 12, None, gen)
    st = torch.tensor(seqlens, device=DEV, dtype=torch.int32)
    _, batch32, _ = ops().decode_attention(q, k_cache, v_cache, st, kv_begin=0, kv_end=2048, partial=True)
    for b in (0, 7, 31):
        alone, alone32, _ = ops().decode_attention(q[b:b + 1], k_cache[b:b + 1], v_cache[b:b + 1], st[b:b + 1],
                                                   kv_begin=0, kv_end=2048, partial=True)
        # fp32 outputs: only the bf16 rounding of P (taken against a different running max when the
        # tiles are cut differently) separates the two evaluations
        assert rel_err(alone32, batch32[b:b + 1]) <= 3e-3
        # bf16 outputs may differ by one unit in the last place (2^-8 relative to the largest element)
        assert rel_err(alone.float(), out[b:b + 1].float()) <= 1e-2


def test_decode_attention_long_rows_gqa():
    """configs[4]-like (scaled down): few rows, long keys, 16 q heads on 4 kv heads."""
    seqlens = [8191, 5000, 4097, 6143]
    run_decode_case(4, 16, 4, 8192, seqlens, -1, seed=44, check_eager=False)


def test_decode_attention_kv_shards_and_combine():
    """Sequence-split: per-shard partials merged by lse_combine equal the unsplit result."""
    B, Hq, Hkv, T_max = 5, 8, 2, 520
    seqlens = [519, 100, 0, 259, 260]
    full = run_decode_case(B, Hq, Hkv, T_max, seqlens, -1, seed=9)
    parts_o, parts_lse = [], []
    for lo, hi in [(0, 130), (130, 260), (260, 390), (390, 520)]:
        gen = torch.Generator(device=DEV).manual_seed(9)
        q = torch.randn(B, Hq, 128, generator=gen, device=DEV).to(BF)
        k_cache, v_cache = make_cache(B, T_max, Hkv, None, gen)
        st = torch.tensor(seqlens, device=DEV, dtype=torch.int32)
        _, o32, lse = ops().decode_attention(q, k_cache, v_cache, st, kv_begin=lo, kv_end=hi, partial=True)
        parts_o.append(o32)
        parts_lse.append(lse)
        run_decode_case(B, Hq, Hkv, T_max, seqlens, -1, seed=9, kv_range=(lo, hi))
    out, lse = ops().lse_combine(torch.stack(parts_o), torch.stack(parts_lse))
    assert rel_err(out.float(), full.float()) <= 4e-3
    ref_o, ref_lse = O.lse_combine(torch.stack(parts_o).cpu().numpy(), torch.stack(parts_lse).cpu().numpy())
    assert torch.allclose(out.float().cpu(), torch.from_numpy(ref_o), atol=1e-2, rtol=1e-2)
    np.testing.assert_allclose(lse.cpu().numpy(), ref_lse, rtol=1e-5, atol=1e-5)


def test_decode_attention_ignores_garbage_beyond_length():
    """Bytes past cache_seqlens (NaN/Inf patterns included) must not reach the output."""
    gen = torch.Generator(device=DEV).manual_seed(12)
    B, H, T_max = 3, 2, 100
    seqlens = [10, 40, 63]
    st = torch.tensor(seqlens, device=DEV, dtype=torch.int32)
    q = torch.randn(B, H, 128, generator=gen, device=DEV).to(BF)
    k_cache, v_cache = make_cache(B, T_max, H, None, gen)
    clean = ops().decode_attention(q, k_cache, v_cache, st)
    for b, L in enumerate(seqlens):
        k_cache[b, L + 1:] = float("nan")
        v_cache[b, L + 1:] = float("inf")
    dirty = ops().decode_attention(q, k_cache, v_cache, st)
    assert torch.equal(bits(clean), bits(dirty))


def test_workspace_ticket_counter_returns_to_zero():
    seqlens = [2000] * 4
    for _ in range(3):  # long rows on few pairs: every pair is split; repeated launches reuse the counter
        run_decode_case(4, 2, 2, 2048, seqlens, -1, seed=1)
    ws = ops().workspace(DEV, 4, 2, 2)
    torch.cuda.synchronize()
    assert ws[:256].view(torch.int32).abs().sum().item() == 0, "status word / ticket counter not back to zero"


@pytest.mark.parametrize("counted", [True, False])
def test_decode_right_behind_append_sees_the_appended_row(counted):
    """The attention kernels start while the append kernel in front of them may still be running
    and prefetch older keys early; the tile that holds the appended position must wait.  Lengths
    are multiples of the 48-key tile, the case in which the appended row is the last row of a full
    tile; ``counted``: cache_seqlens already counts the new token (seqlen_offset = 0, the
    sequence-split convention) or not (seqlen_offset = 1, the reference's convention)."""
    gen = torch.Generator(device=DEV).manual_seed(21)
    B, Hq, Hkv, T_max = 64, 4, 4, 480
    cos, sin = E.rotary_tables(T_max, 128, DEV, BF)
    after = torch.tensor([48 * (1 + (b % 9)) for b in range(B)], device=DEV, dtype=torch.int32)  # lengths incl. new token
    before = after - 1
    slots = before.clone()
    lens, offset = (after, 0) if counted else (before, 1)
    k_cache, v_cache = make_cache(B, T_max, Hkv, None, gen)
    q = torch.randn(B, 1, Hq, 128, generator=gen, device=DEV).to(BF)
    k = torch.randn(B, 1, Hkv, 128, generator=gen, device=DEV).to(BF)
    v = torch.randn(B, 1, Hkv, 128, generator=gen, device=DEV).to(BF)

    def pair():
        q2 = ops().append_rope_norm(q, k, v, k_cache, v_cache, before, cos, sin, write_slots=slots)
        return q2, ops().decode_attention(q2[:, 0], k_cache, v_cache, lens, seqlen_offset=offset)

    # the two calls back to back on the device (no host gap between the launches): a CUDA graph
    side = torch.cuda.Stream(DEV)
    with torch.cuda.stream(side):
        pair()
        side.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=side):
            q2, out = pair()
    torch.cuda.synchronize()
    for it in range(40):
        k.copy_(torch.randn(B, 1, Hkv, 128, generator=gen, device=DEV).to(BF) * (1 + it))
        v.copy_(torch.randn(B, 1, Hkv, 128, generator=gen, device=DEV).to(BF) * (1 + it))
        graph.replay()
        torch.cuda.synchronize()
        settled = ops().decode_attention(q2[:, 0], k_cache, v_cache, lens, seqlen_offset=offset)  # nothing in flight before it
        torch.cuda.synchronize()
        assert torch.equal(bits(out), bits(settled)), f"iteration {it}: attention ran ahead of the append"
    assert ops().read_status(DEV) == 0


def test_invalid_lengths_set_status_bits_and_spare_the_other_rows():
    """Negative and over-capacity cache_seqlens: the kernels flag them in the status word (bit 4 bad
    length, bit 1 overflow), touch nothing out of range, and the valid rows keep their results."""
    from nanochat_b200 import _lib
    gen = torch.Generator(device=DEV).manual_seed(31)
    B, Hq, Hkv, T_max = 6, 4, 2, 300
    good = [10, 0, 299, 150, 47, 48]
    lens_ok = torch.tensor(good, device=DEV, dtype=torch.int32)
    lens_bad = lens_ok.clone()
    lens_bad[1] = -7          # bad length
    lens_bad[3] = T_max + 50  # beyond the capacity
    q = torch.randn(B, Hq, 128, generator=gen, device=DEV).to(BF)
    k_cache, v_cache = make_cache(B, T_max, Hkv, None, gen)
    ref = ops().decode_attention(q, k_cache, v_cache, lens_ok, seqlen_offset=1)
    assert ops().read_status(DEV) & ~_lib.ST_OVERFLOW == 0  # row 2 (L + 1 == T_max) is legal
    ops().read_status(DEV)
    out = ops().decode_attention(q, k_cache, v_cache, lens_bad, seqlen_offset=1)
    torch.cuda.synchronize()
    st = ops().read_status(DEV)
    assert st & _lib.ST_BAD_SEQLEN and st & _lib.ST_OVERFLOW, st
    keep = [0, 2, 4, 5]
    assert torch.equal(bits(out[keep]), bits(ref[keep]))
    assert not torch.isnan(out.float()).any()
    # append: rows with a bad or overflowing position are skipped, the others written
    cos, sin = E.rotary_tables(T_max, 128, DEV, BF)
    kq = torch.randn(B, 1, Hq, 128, generator=gen, device=DEV).to(BF)
    kk = torch.randn(B, 1, Hkv, 128, generator=gen, device=DEV).to(BF)
    kv = torch.randn(B, 1, Hkv, 128, generator=gen, device=DEV).to(BF)
    kc2, vc2 = k_cache.clone(), v_cache.clone()
    ops().append_rope_norm(kq, kk, kv, kc2, vc2, lens_bad, cos, sin)
    torch.cuda.synchronize()
    st = ops().read_status(DEV)
    assert st & _lib.ST_BAD_SEQLEN and st & _lib.ST_OVERFLOW, st
    for b in (1, 3):
        assert torch.equal(bits(kc2[b]), bits(k_cache[b])) and torch.equal(bits(vc2[b]), bits(v_cache[b]))
    for b in (0, 4, 5):
        assert torch.equal(bits(vc2[b, good[b]]), bits(kv[b, 0]))
    # prefill attention
    T_new = 5
    pq = torch.randn(B, T_new, Hq, 128, generator=gen, device=DEV).to(BF)
    ops().prefill_attention(pq, k_cache, v_cache, lens_bad, -1)
    torch.cuda.synchronize()
    st = ops().read_status(DEV)
    assert st & _lib.ST_BAD_SEQLEN and st & _lib.ST_OVERFLOW, st
    assert ops().read_status(DEV) == 0


def test_decode_shapes_share_one_workspace():
    """Calls of different shapes through one workspace: the counter and the records of one call must
    not leak into the next."""
    lens32 = torch.randint(1, 2048, (32,), generator=torch.Generator().manual_seed(2)).tolist()
    for _ in range(2):
        run_decode_case(32, 12, 12, 2048, lens32, -1, seed=3, check_eager=False)
        run_decode_case(4, 16, 4, 4096, [4000, 17, 2500, 4095], -1, seed=4)
        run_decode_case(3, 2, 2, 2048, [2000, 1, 999], 512, seed=5)


# ------------------------------------------------------------------------------------------------
# reference fixtures through the public wrapper
# ------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("name", ["d128_single", "d128_single_window", "d128_gqa_single"])
def test_flash_attn_with_kvcache_golden_decode(golden_dir, name):
    from nanochat_b200.flash_attention import flash_attn
    g = np.load(os.path.join(golden_dir, "attn_kvcache_fp32.npz"))
    dev = lambda a: torch.from_numpy(a).to(DEV).to(BF)
    q, k, v = dev(g[f"{name}.q"]), dev(g[f"{name}.k"]), dev(g[f"{name}.v"])
    seqlens = torch.from_numpy(g[f"{name}.seqlens"]).to(DEV)
    window = int(g[f"{name}.window"])
    k_after, v_after = dev(g[f"{name}.k_cache_after"]), dev(g[f"{name}.v_cache_after"])
    L = int(seqlens[0])
    k_cache, v_cache = k_after.clone(), v_after.clone()
    k_cache[:, L:L + 1] = 0
    v_cache[:, L:L + 1] = 0
    before = seqlens.clone()
    out = flash_attn.flash_attn_with_kvcache(q, k_cache, v_cache, k=k, v=v, cache_seqlens=seqlens, causal=True,
                                             window_size=(window, 0))
    assert out.shape == q.shape
    assert torch.equal(seqlens, before), "cache_seqlens must not be advanced by the attention call"
    assert torch.equal(bits(k_cache), bits(k_after)) and torch.equal(bits(v_cache), bits(v_after))
    ref = torch.from_numpy(g[f"{name}.out"])
    # inputs were rounded to bf16 on the way in: compare loosely with the fp32 fixture and tightly
    # with the oracle evaluated on the rounded inputs
    assert torch.allclose(out.float().cpu(), ref, atol=3e-2, rtol=3e-2)
    o2, _ = O.attention_kvcache(q.float().cpu().numpy(), k_cache.float().cpu().numpy(), v_cache.float().cpu().numpy(),
                                before.cpu().numpy(), window_left=window)
    assert torch.allclose(out.float().cpu(), torch.from_numpy(o2), atol=ATOL, rtol=RTOL)


# ------------------------------------------------------------------------------------------------
# (c) prefill broadcast
# ------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("L,B,p,Hkv,T_src,T_dst", [(4, 4, 32, 2, 32, 96), (2, 7, 5, 3, 9, 11), (1, 64, 1024, 4, 1024, 1100),
                                                   (3, 2, 0, 1, 4, 4)])
def test_prefill_broadcast_bit_exact(L, B, p, Hkv, T_src, T_dst):
    gen = torch.Generator(device=DEV).manual_seed(L * 100 + B)
    src_k = torch.randn(L, 1, T_src, Hkv, 128, generator=gen, device=DEV).to(BF)
    src_v = torch.randn(L, 1, T_src, Hkv, 128, generator=gen, device=DEV).to(BF)
    dst_k = torch.full((L, B, T_dst, Hkv, 128), 7.0, device=DEV, dtype=BF)
    dst_v = torch.full((L, B, T_dst, Hkv, 128), -7.0, device=DEV, dtype=BF)
    seqlens = torch.zeros(B, device=DEV, dtype=torch.int32)
    ref_k, ref_v = dst_k.cpu().float().numpy(), dst_v.cpu().float().numpy()
    ref_s = np.zeros(B, dtype=np.int32)
    O.prefill_broadcast(src_k.cpu().float().numpy(), src_v.cpu().float().numpy(), ref_k, ref_v, ref_s, p)
    ops().prefill_broadcast(src_k, src_v, dst_k, dst_v, seqlens, p)
    assert np.array_equal(dst_k.cpu().float().numpy(), ref_k)
    assert np.array_equal(dst_v.cpu().float().numpy(), ref_v)
    assert np.array_equal(seqlens.cpu().numpy(), ref_s)


def test_lse_combine_matches_oracle():
    gen = torch.Generator(device=DEV).manual_seed(77)
    n, rows = 5, 37
    po = torch.randn(n, rows, 128, generator=gen, device=DEV)
    pl = torch.randn(n, rows, generator=gen, device=DEV) * 3
    pl[2, 5] = float("-inf")
    pl[:, 9] = float("-inf")  # a row nobody saw any key for
    out, lse = ops().lse_combine(po, pl)
    ro, rl = O.lse_combine(po.cpu().numpy(), pl.cpu().numpy())
    assert torch.allclose(out.float().cpu(), torch.from_numpy(ro), atol=1e-2, rtol=1e-2)
    assert np.array_equal(np.isneginf(lse.cpu().numpy()), np.isneginf(rl))
    fin = np.isfinite(rl)
    np.testing.assert_allclose(lse.cpu().numpy()[fin], rl[fin], rtol=1e-5, atol=1e-5)
    assert out[9].abs().sum().item() == 0


# ------------------------------------------------------------------------------------------------
# (d) dense prefill attention (tcgen05 / TMEM)
# ------------------------------------------------------------------------------------------------
def run_prefill_case(B, T_new, Hq, Hkv, T_k, prefix, window, seed, tol=ATOL):
    gen = torch.Generator(device=DEV).manual_seed(seed)
    seqlens = torch.tensor(prefix, device=DEV, dtype=torch.int32)
    q = torch.randn(B, T_new, Hq, 128, generator=gen, device=DEV).to(BF)
    k_cache, v_cache = make_cache(B, T_k, Hkv, None, gen)
    out = ops().prefill_attention(q, k_cache, v_cache, seqlens, window)
    torch.cuda.synchronize()
    assert ops().read_status(DEV) == 0
    ref, _ = O.attention_kvcache(q.float().cpu().numpy(), k_cache.float().cpu().numpy(), v_cache.float().cpu().numpy(),
                                 np.array(prefix), window_left=window)
    ref = torch.from_numpy(ref)
    got = out.float().cpu()
    assert not torch.isnan(got).any()
    assert torch.allclose(got, ref, atol=tol, rtol=tol), f"max diff {(got - ref).abs().max().item()}"
    assert rel_err(got, ref) <= 1e-2
    return out


@pytest.mark.parametrize("B,T_new,Hq,Hkv,T_k,prefix,window", [
    (2, 16, 2, 2, 48, [0, 0], -1),          # prefill into an empty cache (test_kvcache_prefill shape at D=128)
    (1, 128, 2, 2, 128, [0], -1),           # exactly one query tile, one and two key tiles
    (2, 200, 4, 2, 300, [0, 37], -1),       # ragged prefixes, partial tiles, GQA
    (1, 5, 4, 2, 40, [12], 6),              # chunk with a window (d128_gqa_chunk_window shape)
    (1, 300, 2, 1, 400, [90], 64),          # window shorter than a key tile's reach
    (2, 130, 2, 2, 260, [129, 1], 128),
    (1, 64, 16, 4, 1100, [1000], -1),       # long prefix, short chunk
])
def test_prefill_attention_matches_oracle(B, T_new, Hq, Hkv, T_k, prefix, window):
    run_prefill_case(B, T_new, Hq, Hkv, T_k, prefix, window, seed=T_new + Hq)


def test_prefill_attention_ignores_garbage_beyond_length():
    gen = torch.Generator(device=DEV).manual_seed(5)
    B, T_new, H, T_k = 1, 70, 2, 256
    q = torch.randn(B, T_new, H, 128, generator=gen, device=DEV).to(BF)
    k_cache, v_cache = make_cache(B, T_k, H, None, gen)
    st = torch.tensor([20], device=DEV, dtype=torch.int32)
    clean = ops().prefill_attention(q, k_cache, v_cache, st, -1)
    k_cache[:, 90:] = float("nan")
    v_cache[:, 90:] = float("inf")
    dirty = ops().prefill_attention(q, k_cache, v_cache, st, -1)
    assert torch.equal(bits(clean), bits(dirty))


@pytest.mark.parametrize("name", ["causal", "window", "window_ge_T"])
def test_flash_attn_func_golden(golden_dir, name):
    from nanochat_b200.flash_attention import flash_attn
    g = np.load(os.path.join(golden_dir, "attn_func_fp32.npz"))
    dev = lambda a: torch.from_numpy(a).to(DEV).to(BF)
    q, k, v = dev(g[f"{name}.q"]), dev(g[f"{name}.k"]), dev(g[f"{name}.v"])
    window = int(g[f"{name}.window"])
    out = flash_attn.flash_attn_func(q, k, v, causal=True, window_size=(window, 0))
    assert out.shape == q.shape
    assert torch.allclose(out.float().cpu(), torch.from_numpy(g[f"{name}.out"]), atol=3e-2, rtol=3e-2)
    ref = O.attention_nocache(q.float().cpu().numpy(), k.float().cpu().numpy(), v.float().cpu().numpy(), window_left=window)
    assert torch.allclose(out.float().cpu(), torch.from_numpy(ref), atol=ATOL, rtol=RTOL)


@pytest.mark.parametrize("name", ["d128_prefill", "d128_gqa_chunk_window", "d128_chunk_full"])
def test_flash_attn_with_kvcache_golden_prefill(golden_dir, name):
    from nanochat_b200.flash_attention import flash_attn
    g = np.load(os.path.join(golden_dir, "attn_kvcache_fp32.npz"))
    dev = lambda a: torch.from_numpy(a).to(DEV).to(BF)
    q, k, v = dev(g[f"{name}.q"]), dev(g[f"{name}.k"]), dev(g[f"{name}.v"])
    seqlens = torch.from_numpy(g[f"{name}.seqlens"]).to(DEV)
    window = int(g[f"{name}.window"])
    k_after, v_after = dev(g[f"{name}.k_cache_after"]), dev(g[f"{name}.v_cache_after"])
    L, T_new = int(seqlens[0]), q.size(1)
    k_cache, v_cache = k_after.clone(), v_after.clone()
    k_cache[:, L:L + T_new] = 0
    v_cache[:, L:L + T_new] = 0
    out = flash_attn.flash_attn_with_kvcache(q, k_cache, v_cache, k=k, v=v, cache_seqlens=seqlens, causal=True,
                                             window_size=(window, 0))
    assert torch.equal(bits(k_cache), bits(k_after)) and torch.equal(bits(v_cache), bits(v_after))
    assert torch.allclose(out.float().cpu(), torch.from_numpy(g[f"{name}.out"]), atol=3e-2, rtol=3e-2)


def test_prefill_then_decode_matches_eager_reference_path():
    """KVCache + two calls + advance, as tests/test_attention_fallback.py:292-334, against the eager bf16 path."""
    from nanochat_b200.engine import KVCache
    from nanochat_b200.flash_attention import flash_attn
    gen = torch.Generator(device=DEV).manual_seed(21)
    B, T_max, H = 2, 64, 4
    cache = KVCache(batch_size=B, num_heads=H, seq_len=T_max, head_dim=128, num_layers=1, device=DEV, dtype=BF)
    k_cache, v_cache = cache.get_layer_cache(0)
    ref_k, ref_v = k_cache.clone(), v_cache.clone()
    mk = lambda T: [torch.randn(B, T, H, 128, generator=gen, device=DEV).to(BF) for _ in range(3)]
    q, k, v = mk(16)
    y = flash_attn.flash_attn_with_kvcache(q, k_cache, v_cache, k=k, v=v, cache_seqlens=cache.cache_seqlens,
                                           causal=True, window_size=(T_max, 0))
    y_ref = E.kvcache_attention(q, ref_k, ref_v, k, v, cache.cache_seqlens, T_max)
    cache.advance(16)
    assert y.shape == (B, 16, H, 128) and cache.get_pos() == 16
    assert torch.allclose(y.float(), y_ref.float(), atol=2e-2, rtol=2e-2)
    q1, k1, v1 = mk(1)
    y1 = flash_attn.flash_attn_with_kvcache(q1, k_cache, v_cache, k=k1, v=v1, cache_seqlens=cache.cache_seqlens,
                                            causal=True, window_size=(T_max, 0))
    y1_ref = E.kvcache_attention(q1, ref_k, ref_v, k1, v1, cache.cache_seqlens, T_max)
    cache.advance(1)
    assert y1.shape == (B, 1, H, 128) and cache.get_pos() == 17
    assert torch.allclose(y1.float(), y1_ref.float(), atol=2e-2, rtol=2e-2)
    assert torch.equal(bits(k_cache), bits(ref_k)) and torch.equal(bits(v_cache), bits(ref_v))


def test_registered_custom_ops_dispatch():
    """torch.ops.nckv.* (the dispatcher route) gives the same results as the direct entry points."""
    gen = torch.Generator(device=DEV).manual_seed(31)
    B, H, T_max = 3, 4, 96
    st = torch.tensor([5, 50, 94], device=DEV, dtype=torch.int32)
    q = torch.randn(B, H, 128, generator=gen, device=DEV).to(BF)
    k_cache, v_cache = make_cache(B, T_max, H, None, gen)
    a = ops().decode_attention(q, k_cache, v_cache, st)
    b, e1, e2 = torch.ops.nckv.decode_attn(q, k_cache, v_cache, st, 1, -1, 0, 0, False)
    assert torch.equal(bits(a), bits(b)) and e1.numel() == 0 and e2.numel() == 0
    k = torch.randn(B, 1, H, 128, generator=gen, device=DEV).to(BF)
    kc2, vc2 = k_cache.clone(), v_cache.clone()
    torch.ops.nckv.append_kv(k, k, kc2, vc2, st)
    ops().append_kv(k, k, k_cache, v_cache, st)
    assert torch.equal(bits(kc2), bits(k_cache)) and torch.equal(bits(vc2), bits(v_cache))
    with pytest.raises(RuntimeError, match="CUDA"):
        torch.ops.nckv.decode_attn(q.cpu(), k_cache.cpu(), v_cache.cpu(), st.cpu(), 1, -1, 0, 0, False)


@pytest.mark.parametrize("transfer", ["copy", "mapped"])
def test_host_decode_step_matches_device_path(transfer):
    """nckv_decode_step_host (H2D + append + attention + D2H in one call, or the kernels reading and
    writing the pinned host blocks themselves) == the two device ops."""
    gen = torch.Generator(device=DEV).manual_seed(77)
    B, Hq, Hkv, T_max = 5, 8, 2, 200
    cos, sin = E.rotary_tables(T_max, 128, DEV, BF)
    st = torch.tensor([0, 17, 100, 198, 64], device=DEV, dtype=torch.int32)
    q = torch.randn(B, 1, Hq, 128, generator=gen, device=DEV).to(BF)
    k = torch.randn(B, 1, Hkv, 128, generator=gen, device=DEV).to(BF)
    v = torch.randn(B, 1, Hkv, 128, generator=gen, device=DEV).to(BF)
    k_cache, v_cache = make_cache(B, T_max, Hkv, None, gen)
    kc2, vc2 = k_cache.clone(), v_cache.clone()
    q2 = ops().append_rope_norm(q, k, v, k_cache, v_cache, st, cos, sin)
    ref = ops().decode_attention(q2[:, 0], k_cache, v_cache, st, window_left=50)
    step = ops().HostDecodeStep(B, Hq, Hkv, cos, sin, DEV, transfer=transfer)
    step.q.copy_(q[:, 0].cpu()); step.k.copy_(k[:, 0].cpu()); step.v.copy_(v[:, 0].cpu())
    out = step.run(kc2, vc2, st, 50)
    assert not out.is_cuda and torch.equal(bits(out), bits(ref.cpu()))
    assert torch.equal(bits(kc2), bits(k_cache)) and torch.equal(bits(vc2), bits(v_cache))
    assert ops().read_status(DEV) == 0


@pytest.mark.parametrize("transfer", ["copy", "mapped"])
def test_host_decode_step_replays_follow_the_callers_stream(transfer):
    """Six steps through the same HostDecodeStep (the first captures the step, the others replay it): new
    host inputs and cache_seqlens advanced on the caller's stream between steps; every step equals the device
    ops run on a copy of the cache."""
    gen = torch.Generator(device=DEV).manual_seed(78)
    B, Hq, Hkv, T_max = 4, 4, 4, 128
    cos, sin = E.rotary_tables(T_max, 128, DEV, BF)
    st = torch.tensor([3, 40, 0, 100], device=DEV, dtype=torch.int32)
    k_cache, v_cache = make_cache(B, T_max, Hkv, None, gen)
    kc2, vc2, st2 = k_cache.clone(), v_cache.clone(), st.clone()
    step = ops().HostDecodeStep(B, Hq, Hkv, cos, sin, DEV, transfer=transfer)
    for i in range(6):
        q = torch.randn(B, 1, Hq, 128, generator=gen, device=DEV).to(BF)
        k = torch.randn(B, 1, Hkv, 128, generator=gen, device=DEV).to(BF)
        v = torch.randn(B, 1, Hkv, 128, generator=gen, device=DEV).to(BF)
        q2 = ops().append_rope_norm(q, k, v, k_cache, v_cache, st, cos, sin)
        ref = ops().decode_attention(q2[:, 0], k_cache, v_cache, st)
        step.q.copy_(q[:, 0].cpu()); step.k.copy_(k[:, 0].cpu()); step.v.copy_(v[:, 0].cpu())
        out = step.run(kc2, vc2, st2)
        assert torch.equal(bits(out), bits(ref.cpu())), f"step {i}"
        st += 1
        st2 += 1  # enqueued on the caller's stream, not synchronised: the next step must come after it
    assert torch.equal(bits(kc2), bits(k_cache)) and torch.equal(bits(vc2), bits(v_cache))
    assert ops().read_status(DEV) == 0


def test_p2p_wait_runs_out_and_reports_instead_of_hanging():
    """A peer that never delivers: the wait/combine kernel gives up after its limit, sets the timeout
    bit, leaves the output untouched and the context usable.  (The failure is a flag nothing sets.)"""
    from nanochat_b200 import _lib
    rows, world = 12, 2
    nbytes = _lib.lib.nckv_p2p_buffer_bytes(world, rows, 128)
    assert nbytes > 0
    buf = torch.zeros((nbytes + 3) // 4, dtype=torch.float32, device=DEV)
    send = torch.randn(rows * 128 + rows, device=DEV)
    out = torch.full((rows, 128), 7.0, device=DEV, dtype=BF)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    stream = torch.cuda.current_stream().cuda_stream
    import ctypes
    ptrs = (ctypes.c_void_p * world)(buf.data_ptr(), buf.data_ptr())  # both "peers" map to the local buffer
    # only rank 0's part arrives (we push as rank 0); rank 1's flag is never set
    ctr = torch.zeros(2, dtype=torch.int32, device=DEV)
    _lib.call("nckv_p2p_push", send.data_ptr(), rows, 128, ptrs, 1, 0, ctr.data_ptr(), stream)
    t0 = torch.cuda.Event(enable_timing=True); t1 = torch.cuda.Event(enable_timing=True)
    t0.record()
    _lib.call("nckv_p2p_wait_combine", buf.data_ptr(), world, rows, 128, ctr.data_ptr(), out.data_ptr(), None,
              status.data_ptr(), 2_000_000, stream)  # 2 ms limit
    t1.record()
    torch.cuda.synchronize()
    assert status.item() & 2, "timeout bit not set"
    assert t0.elapsed_time(t1) < 200.0
    assert (out.float() == 7.0).all(), "output must be left untouched after a timeout"
    # the context is fine: complete the exchange properly (world = 1 view of the same buffer, step 2)
    status.zero_()
    buf.zero_()
    _lib.call("nckv_p2p_push", send.data_ptr(), rows, 128, ptrs, 1, 0, ctr.data_ptr(), stream)
    _lib.call("nckv_p2p_wait_combine", buf.data_ptr(), 1, rows, 128, ctr.data_ptr(), out.data_ptr(), None,
              status.data_ptr(), 0, stream)
    assert ctr.tolist() == [2, 0]
    torch.cuda.synchronize()
    assert status.item() == 0
    assert torch.allclose(out.float(), send[:rows * 128].view(rows, 128).to(BF).float(), atol=1e-2, rtol=1e-2)


def test_prefill_attention_random_shapes_match_fp32_and_repeat_bit_for_bit():
    """Sixty random (rows, tokens, heads, window, cached prefix, capacity) combinations of the dense kernel against
    an fp32 masked softmax of the same bf16 inputs (1e-2 of the largest output), each run twice: a persistent kernel
    with several asynchronous roles must return the same bytes every time."""
    import math
    import random
    rng = random.Random(0)
    for case in range(60):
        B = rng.choice([1, 2, 3, 5])
        T = rng.choice([1, 2, 7, 64, 100, 128, 129, 255, 256, 300, 511, 700, 1000, 1537])
        Hkv = rng.choice([1, 2, 4])
        Hq = Hkv * rng.choice([1, 2, 4])
        window = rng.choice([-1, -1, 0, 5, 63, 64, 200, 1024])
        prefix = rng.choice([0, 0, 1, 17, 128, 333])
        lens = torch.tensor([rng.randint(0, prefix) for _ in range(B)], dtype=torch.int32, device=DEV)
        Tk = int(lens.max()) + T + rng.choice([0, 3, 64])
        gen = torch.Generator(device=DEV).manual_seed(case)
        q = torch.randn(B, T, Hq, 128, generator=gen, device=DEV).to(BF)
        k = torch.randn(B, Tk, Hkv, 128, generator=gen, device=DEV).to(BF)
        v = torch.randn(B, Tk, Hkv, 128, generator=gen, device=DEV).to(BF)
        first = ops().prefill_attention(q, k, v, lens, window)
        second = ops().prefill_attention(q, k, v, lens, window)
        kf = k.float().repeat_interleave(Hq // Hkv, 2)
        vf = v.float().repeat_interleave(Hq // Hkv, 2)
        s = torch.einsum("bthd,bshd->bhts", q.float(), kf) / math.sqrt(128)
        pos = lens.view(B, 1) + torch.arange(T, device=DEV).view(1, T)
        key = torch.arange(Tk, device=DEV).view(1, 1, Tk)
        mask = key <= pos.unsqueeze(-1)
        if window >= 0:
            mask &= (pos.unsqueeze(-1) - key) <= window
        ref = torch.einsum("bhts,bshd->bthd", torch.softmax(s.masked_fill(~mask.unsqueeze(1), float("-inf")), -1), vf)
        what = dict(case=case, B=B, T=T, Hq=Hq, Hkv=Hkv, window=window, prefix=prefix, Tk=Tk)
        assert torch.equal(bits(first), bits(second)), what
        assert (first.float() - ref).abs().max() <= 1e-2 * ref.abs().max(), what
    assert ops().read_status(DEV) == 0
