"""Paged KV storage (page pools + block table) against the dense path and the numpy oracle."""
import numpy as np
import pytest
import torch

from oracle import kv_oracle as O
from oracle import torch_ref as E

pytestmark = pytest.mark.gpu
DEV = "cuda"
BF = torch.bfloat16


def _bits(t):
    return t.contiguous().view(torch.int16)


def _scatter_into_pages(dense, table, page_tokens, n_pages, lens):
    """Pool holding the first lens[b] tokens of every dense row at the places the table names; the rest NaN."""
    B, T, H, D = dense.shape
    pool = torch.full((n_pages, page_tokens, H, D), float("nan"), device=DEV, dtype=BF)
    for b in range(B):
        for i in range(-(-int(lens[b]) // page_tokens)):
            n = min(page_tokens, int(lens[b]) - i * page_tokens)
            pool[int(table[b, i]), :n] = dense[b, i * page_tokens:i * page_tokens + n]
    return pool


@pytest.mark.parametrize("Hq,Hkv,window,page_tokens", [(12, 12, -1, 192), (16, 4, -1, 48), (8, 2, 100, 96), (16, 1, 37, 48)])
def test_paged_decode_matches_dense_and_oracle(Hq, Hkv, window, page_tokens):
    from nanochat_b200 import ops
    gen = torch.Generator(device=DEV).manual_seed(Hq + page_tokens)
    B, T_max = 7, 960
    max_pages = T_max // page_tokens
    n_pages = B * max_pages + 3
    lens = torch.tensor([0, 1, 47, 48, 500, 959, 191], dtype=torch.int32)  # lengths before the new token
    q = torch.randn(B, Hq, 128, generator=gen, device=DEV).to(BF)
    kc = torch.randn(B, T_max, Hkv, 128, generator=gen, device=DEV).to(BF)
    vc = torch.randn(B, T_max, Hkv, 128, generator=gen, device=DEV).to(BF)
    # a scrambled table: pages of a row are neither contiguous nor ordered
    perm = torch.randperm(n_pages, generator=torch.Generator().manual_seed(1))[:B * max_pages].view(B, max_pages).to(torch.int32)
    kp = _scatter_into_pages(kc, perm, page_tokens, n_pages, lens + 1)
    vp = _scatter_into_pages(vc, perm, page_tokens, n_pages, lens + 1)
    table = perm.to(DEV)
    lens_d = lens.to(DEV)
    got = ops.decode_attention_paged(q, kp, vp, table, lens_d, seqlen_offset=1, window_left=window)
    dense = ops.decode_attention(q, kc, vc, lens_d, seqlen_offset=1, window_left=window)
    torch.cuda.synchronize()
    assert ops.read_status(DEV) == 0
    assert not torch.isnan(got.float()).any(), "stale bytes of a page reached the output"
    ref, _ = O.attention_kvcache(q.float().cpu().numpy()[:, None], kc.float().cpu().numpy(), vc.float().cpu().numpy(),
                                 lens.numpy(), window_left=window)
    assert np.allclose(got.float().cpu().numpy(), ref[:, 0], atol=1e-2, rtol=1e-2)
    if window < 0:  # same tile cuts as the dense kernel: the very same arithmetic
        assert torch.equal(_bits(got), _bits(dense))
    else:
        assert torch.allclose(got.float(), dense.float(), atol=1e-2, rtol=1e-2)


def test_paged_append_writes_through_the_table_bit_exactly():
    from nanochat_b200 import ops
    gen = torch.Generator(device=DEV).manual_seed(3)
    B, Hq, Hkv, page_tokens, max_pages = 6, 8, 2, 48, 5
    n_pages = B * max_pages
    T_max = page_tokens * max_pages
    cos, sin = E.rotary_tables(T_max, 128, DEV, BF)
    lens = torch.tensor([0, 47, 48, 100, 239, 95], dtype=torch.int32, device=DEV)
    table = torch.randperm(n_pages, generator=torch.Generator().manual_seed(2)).view(B, max_pages).to(torch.int32).to(DEV)
    q, k, v = (torch.randn(B, 1, h, 128, generator=gen, device=DEV).to(BF) for h in (Hq, Hkv, Hkv))
    kp = torch.zeros(n_pages, page_tokens, Hkv, 128, device=DEV, dtype=BF)
    vp = torch.zeros_like(kp)
    kd = torch.zeros(B, T_max, Hkv, 128, device=DEV, dtype=BF)
    vd = torch.zeros_like(kd)
    q_paged = ops.append_rope_norm_paged(q, k, v, kp, vp, table, lens, cos, sin)
    q_dense = ops.append_rope_norm(q, k, v, kd, vd, lens, cos, sin)
    torch.cuda.synchronize()
    assert ops.read_status(DEV) == 0
    assert torch.equal(_bits(q_paged), _bits(q_dense))
    for b, L in enumerate(lens.tolist()):
        page, off = int(table[b, L // page_tokens]), L % page_tokens
        assert torch.equal(_bits(kp[page, off]), _bits(kd[b, L])) and torch.equal(_bits(vp[page, off]), _bits(vd[b, L]))
    assert int((kp != 0).any(-1).any(-1).sum()) == B, "exactly one token per row may have been written"
    # a table entry outside the pool: flagged, row skipped, nothing else disturbed
    bad = table.clone()
    bad[2, 1] = n_pages + 5
    kp2 = torch.zeros_like(kp)
    ops.append_rope_norm_paged(q, k, v, kp2, torch.zeros_like(kp), bad, lens, cos, sin)
    torch.cuda.synchronize()
    assert ops.read_status(DEV) == 8
    assert int((kp2 != 0).any(-1).any(-1).sum()) == B - 1


def test_paged_cache_prefill_shares_prompt_pages_and_decodes_like_the_dense_cache():
    from nanochat_b200 import ops
    from nanochat_b200.engine import KVCache, PagedKVCache
    from nanochat_b200.gpt import kv_attention, precompute_rotary_embeddings
    gen = torch.Generator(device=DEV).manual_seed(11)
    L, B, Hq, Hkv, p, cap, pt = 3, 5, 8, 2, 250, 400, 96
    cos, sin = precompute_rotary_embeddings(cap, 128, device=DEV)
    prompt = KVCache(1, Hkv, p, 128, L, DEV, BF)
    prompt.k_cache.copy_(torch.randn(prompt.k_cache.shape, generator=gen, device=DEV))
    prompt.v_cache.copy_(torch.randn(prompt.v_cache.shape, generator=gen, device=DEV))
    prompt.advance(p)
    prompt.prev_embedding = torch.randn(1, 1, 64, generator=gen, device=DEV).to(BF)
    dense = KVCache(B, Hkv, cap, 128, L, DEV, BF)
    dense.prefill(prompt)
    n_shared = p // pt
    own = -(-cap // pt) - n_shared
    paged = PagedKVCache(B, Hkv, cap, 128, L, DEV, BF, page_tokens=pt, n_pages=n_shared + B * own)
    paged.prefill(prompt)
    torch.cuda.synchronize()
    assert paged.cache_seqlens.tolist() == [p] * B and paged.pages_in_use() == n_shared + B
    table = paged.block_table.cpu()
    assert all(torch.equal(table[b, :n_shared], table[0, :n_shared]) for b in range(B)), "full prompt pages are shared"
    assert len(set(table[:, n_shared].tolist())) == B, "the page with the prompt's tail is private to each row"
    assert torch.equal(paged.prev_embedding, dense.prev_embedding)
    # decode steps: each row gets its own tokens; outputs and the appended bytes must equal the dense cache's
    for step in range(pt + 3):  # crosses a page boundary
        paged.reserve(p + step + 1)
        for layer in range(L):
            q, k, v = (torch.randn(B, 1, h, 128, generator=gen, device=DEV).to(BF) for h in (Hq, Hkv, Hkv))
            w = (64, 0) if layer == 1 else (-1, 0)
            yd = kv_attention(q, k, v, (cos, sin), w, dense, layer)
            yp = kv_attention(q, k, v, (cos, sin), w, paged, layer)
            if w[0] < 0:
                assert torch.equal(_bits(yd), _bits(yp)), f"step {step} layer {layer}"
            else:
                assert torch.allclose(yd.float(), yp.float(), atol=1e-2, rtol=1e-2)
    torch.cuda.synchronize()
    ops.check_status(DEV)
    assert torch.equal(paged.cache_seqlens, dense.cache_seqlens)
    n = p + pt + 3
    table = paged.block_table.cpu()
    for b in (0, B - 1):
        for t in (0, p - 1, p, n - 1):
            page, off = int(table[b, t // pt]), t % pt
            assert torch.equal(_bits(paged.k_cache[:, page, off]), _bits(dense.k_cache[:, b, t]))
            assert torch.equal(_bits(paged.v_cache[:, page, off]), _bits(dense.v_cache[:, b, t]))
    used = paged.pages_in_use()
    paged.reset()
    assert paged.pages_in_use() == 0 and used == n_shared + B * (-(-n // pt) - n_shared)
    with pytest.raises(RuntimeError, match="exhausted"):
        small = PagedKVCache(2, Hkv, cap, 128, 1, DEV, BF, page_tokens=pt, n_pages=3)
        small.reserve(cap)


def test_engine_with_paged_cache_generates_the_tokens_of_the_dense_engine():
    from nanochat_b200.engine import Engine
    from tests.cpu_backend import SpecialsTokenizer
    from tests.test_e2e_gpu import _to_gpu
    from tests.test_host_logic import _config0_model
    model = _to_gpu(_config0_model(True))
    prompt = torch.randint(0, 32768, (70,), generator=torch.Generator().manual_seed(1)).tolist()
    want, _ = Engine(model, SpecialsTokenizer()).generate_batch(prompt, num_samples=4, max_tokens=60, temperature=0.0)
    got, _ = Engine(model, SpecialsTokenizer(), page_tokens=48).generate_batch(prompt, num_samples=4, max_tokens=60, temperature=0.0)
    assert got == want
    # sampled rows (each its own continuation) through the paged cache, eager and graph-replayed
    a, _ = Engine(model, SpecialsTokenizer(), page_tokens=48).generate_batch(prompt, num_samples=3, max_tokens=40, temperature=1.0, top_k=50, seed=7)
    b, _ = Engine(model, SpecialsTokenizer(), cuda_graph=False).generate_batch(prompt, num_samples=3, max_tokens=40, temperature=1.0, top_k=50, seed=7)
    assert a == b
