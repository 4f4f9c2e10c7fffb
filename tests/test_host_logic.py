"""Host-side logic on CPU: KVCache bookkeeping, module surface, the GPT glue and the Engine loop.
Attention itself is served by the oracle's torch port through tests/cpu_backend.py (test-only)."""
import os

import numpy as np
import pytest
import torch

from nanochat_b200 import flash_attention as fa
from nanochat_b200.engine import Engine, KVCache, sample_next_token, use_calculator
from nanochat_b200.gpt import GPT, GPTConfig, compute_window_sizes, precompute_rotary_embeddings
from tests.cpu_backend import SpecialsTokenizer, oracle_backend


# ------------------------------------------------------------------------------------------------
# KVCache (engine.py:82-137; the situations of tests/test_engine.py:84-155)
# ------------------------------------------------------------------------------------------------
def test_kvcache_shapes_and_bookkeeping():
    B, H, T, D, L = 2, 3, 32, 5, 6  # any head_dim: bookkeeping is shape-agnostic
    c = KVCache(batch_size=B, num_heads=H, seq_len=T, head_dim=D, num_layers=L, device="cpu", dtype=torch.float32)
    assert c.k_cache.shape == (L, B, T, H, D) and c.v_cache.shape == (L, B, T, H, D)
    assert c.cache_seqlens.dtype == torch.int32 and c.cache_seqlens.shape == (B,)
    assert (c.batch_size, c.max_seq_len, c.n_layers, c.n_heads, c.head_dim) == (B, T, L, H, D)
    assert c.get_pos() == 0 and c.prev_embedding is None
    c.advance(10)
    assert c.get_pos() == 10 and c.cache_seqlens.tolist() == [10, 10]
    c.advance(5)
    assert c.get_pos() == 15
    k3, v3 = c.get_layer_cache(3)
    assert k3.shape == (B, T, H, D)
    k3[0, 0, 0, 0] = 7.0  # a view, not a copy
    assert c.k_cache[3, 0, 0, 0, 0].item() == 7.0
    c.prev_embedding = torch.zeros(B, 1, 4)
    c.reset()
    assert c.get_pos() == 0 and c.prev_embedding is None


def test_kvcache_prefill_has_no_cpu_path_and_checks_preconditions(golden_dir):
    g = np.load(os.path.join(golden_dir, "kvcache_prefill.npz"))
    src = KVCache(1, 2, 6, 128, 3, "cpu", torch.float32)
    src.k_cache.copy_(torch.from_numpy(g["src_k"]))
    src.v_cache.copy_(torch.from_numpy(g["src_v"]))
    src.advance(6)
    src.prev_embedding = torch.arange(4.0).view(1, 1, 4)
    dst = KVCache(3, 2, 10, 128, 3, "cpu", torch.float32)
    with pytest.raises(RuntimeError, match="CUDA"):
        dst.prefill(src)  # the product path is the CUDA kernel only
    with oracle_backend():
        dst.prefill(src)
        assert np.array_equal(dst.k_cache.numpy(), g["dst_k"]) and np.array_equal(dst.v_cache.numpy(), g["dst_v"])
        assert np.array_equal(dst.cache_seqlens.numpy(), g["dst_seqlens"])
        assert dst.prev_embedding.shape == (3, 1, 4) and torch.equal(dst.prev_embedding[2], src.prev_embedding[0])
        with pytest.raises(AssertionError):
            dst.prefill(src)  # non-empty destination
        with pytest.raises(AssertionError):
            KVCache(3, 2, 4, 128, 3, "cpu", torch.float32).prefill(src)  # shorter than the source
        with pytest.raises(AssertionError):
            KVCache(3, 4, 10, 128, 3, "cpu", torch.float32).prefill(src)  # head count differs


# ------------------------------------------------------------------------------------------------
# module surface of flash_attention.py
# ------------------------------------------------------------------------------------------------
def test_flash_attention_module_surface():
    assert fa.HAS_FA3 is False and fa.USE_FA3 is False
    assert callable(fa.flash_attn.flash_attn_func) and callable(fa.flash_attn.flash_attn_with_kvcache)
    fa._override_impl = "sdpa"
    assert fa._resolve_use_fa3() is False
    fa._override_impl = "fa3"
    with pytest.raises(AssertionError):
        fa._resolve_use_fa3()
    fa._override_impl = None
    assert fa._resolve_use_fa3() == fa.HAS_FA3
    q = torch.zeros(1, 1, 2, 128)
    kc = torch.zeros(1, 4, 2, 128)
    with pytest.raises(RuntimeError, match="CUDA"):
        fa.flash_attn.flash_attn_with_kvcache(q, kc, kc.clone(), k=q, v=q, cache_seqlens=torch.zeros(1, dtype=torch.int32))
    with pytest.raises(ValueError):
        fa.flash_attn.flash_attn_with_kvcache(q, kc, kc.clone(), k=q, v=q)
    with pytest.raises(RuntimeError, match="CUDA"):  # training inputs take the library's own forward/backward: no CPU path
        fa.flash_attn.flash_attn_func(q.clone().requires_grad_(), q, q)


def test_window_sizes_and_rotary_tables_match_reference(golden_dir):
    g = np.load(os.path.join(golden_dir, "window_sizes.npz"))
    for key in g.files:
        seq_len, n_layer, pattern = key.split("_")
        assert np.array_equal(np.array(compute_window_sizes(int(seq_len), int(n_layer), pattern)), g[key])
    with pytest.raises(AssertionError):
        compute_window_sizes(2048, 4, "SQ")
    r = np.load(os.path.join(golden_dir, "rope_norm_fp32.npz"))
    rows = r["table_rows"]
    cos, sin = precompute_rotary_embeddings(4096, 128, device="cpu", dtype=torch.float32)
    assert np.array_equal(cos[0, rows, 0].numpy(), r["cos_rows"]) and np.array_equal(sin[0, rows, 0].numpy(), r["sin_rows"])
    cosb, sinb = precompute_rotary_embeddings(4096, 128, device="cpu", dtype=torch.bfloat16)
    assert np.array_equal(cosb[0, rows, 0].view(torch.int16).numpy(), r["cos_rows_bf16"])
    assert np.array_equal(sinb[0, rows, 0].view(torch.int16).numpy(), r["sin_rows_bf16"])


# ------------------------------------------------------------------------------------------------
# sampling and the Engine loop with a model that returns uniform logits
# (the situations of tests/test_engine.py:158-267)
# ------------------------------------------------------------------------------------------------
class UniformModel:
    """Returns all-zero logits and advances the cache like a real model would."""

    def __init__(self, vocab=262):
        self.vocab = vocab
        self.config = GPTConfig(sequence_len=64, vocab_size=vocab, n_layer=2, n_head=2, n_kv_head=2, n_embd=16)
        self._dev = torch.device("cpu")

    def get_device(self):
        return self._dev

    def forward(self, ids, kv_cache=None):
        B, T = ids.shape
        if kv_cache is not None:
            kv_cache.advance(T)
        return torch.zeros(B, T, self.vocab)


class ByteSpecials(SpecialsTokenizer):
    def __init__(self):
        super().__init__(base=256)


def _engine():
    return Engine(UniformModel(), ByteSpecials())


def test_sample_next_token_modes():
    logits = torch.tensor([[0.0, 5.0, 1.0], [9.0, 0.0, 1.0]])
    assert sample_next_token(logits, None, temperature=0.0).tolist() == [[1], [0]]
    rng = torch.Generator().manual_seed(0)
    out = sample_next_token(logits, rng, temperature=1.0, top_k=1)
    assert out.tolist() == [[1], [0]]  # top-1 sampling is argmax
    rng = torch.Generator().manual_seed(0)
    a = sample_next_token(torch.zeros(4, 50), rng, temperature=1.0)
    rng = torch.Generator().manual_seed(0)
    b = sample_next_token(torch.zeros(4, 50), rng, temperature=1.0)
    assert torch.equal(a, b) and a.shape == (4, 1)
    with pytest.raises(AssertionError):
        sample_next_token(logits, None, temperature=-1.0)


def test_engine_rows_sample_independently_and_seeds_reproduce():
    with oracle_backend():
        eng = _engine()
        prompt = [261, 72, 101, 108, 108, 111]
        first = {}
        res, masks = eng.generate_batch(prompt, num_samples=16, max_tokens=1, temperature=1.0, seed=42)
        first_tokens = [r[len(prompt)] for r in res if len(r) > len(prompt)]
        assert len(set(first_tokens)) > 1, "all rows drew the same first token: sampling was broadcast"
        again, _ = eng.generate_batch(prompt, num_samples=16, max_tokens=1, temperature=1.0, seed=42)
        assert again == res
        outs = {tuple(eng.generate_batch(prompt, max_tokens=5, temperature=1.0, seed=s)[0][0]) for s in (1, 42, 123, 999)}
        assert len(outs) > 1, "different seeds must be able to give different streams"
        assert all(len(m) == len(r) for m, r in zip(masks, res))


def test_engine_temperature_zero_max_tokens_and_num_samples():
    with oracle_backend():
        eng = _engine()
        prompt = [261, 72, 101]
        a, _ = eng.generate_batch(prompt, temperature=0.0, max_tokens=5, seed=1)
        b, _ = eng.generate_batch(prompt, temperature=0.0, max_tokens=5, seed=77)
        assert a == b
        for n in (1, 4, 16, 64):
            res, _ = eng.generate_batch(prompt, max_tokens=n, temperature=0.0)
            assert len(res[0]) - len(prompt) <= n
        for n in (1, 4, 9):
            res, _ = eng.generate_batch(prompt, num_samples=n, max_tokens=3, temperature=1.0)
            assert len(res) == n
        # the decode cache is sized prompt + max_tokens and the last append lands in its last slot
        steps = list(eng.generate(prompt, num_samples=2, max_tokens=4, temperature=0.0))
        assert len(steps) == 4 and all(len(col) == 2 for col, _ in steps)


def test_engine_calculator_tool_forces_tokens():
    assert use_calculator("2+3*4") == 14 and use_calculator("1,000+1") == 1001
    assert use_calculator("2**8") is None and use_calculator("__import__('os')") is None
    assert use_calculator("'strawberry'.count('r')") == 3 and use_calculator("'a'.upper()") is None

    tok = ByteSpecials()
    py_s, py_e = tok.encode_special("<|python_start|>"), tok.encode_special("<|python_end|>")
    o_s, o_e = tok.encode_special("<|output_start|>"), tok.encode_special("<|output_end|>")
    script = [py_s] + list(b"6*7") + [py_e]

    class Scripted(UniformModel):
        def __init__(self):
            super().__init__()
            self.step = 0

        def forward(self, ids, kv_cache=None):
            logits = super().forward(ids, kv_cache)
            want = script[self.step] if self.step < len(script) else 65
            self.step += 1
            logits[:, -1, want] = 10.0
            return logits

    with oracle_backend():
        res, masks = Engine(Scripted(), tok).generate_batch([261, 1, 2], max_tokens=12, temperature=0.0)
    gen, m = res[0][3:], masks[0][3:]
    assert gen[:5] == script
    assert gen[5:9] == [o_s] + list(b"42") + [o_e] and m[5:9] == [0, 0, 0, 0], "tool output must be forced tokens"
    assert m[:5] == [1] * 5 and m[9] == 1


# ------------------------------------------------------------------------------------------------
# GPT glue + Engine against the reference's own greedy streams (benchmark configuration 0)
# ------------------------------------------------------------------------------------------------
def _config0_model(binding):
    cfg = GPTConfig(sequence_len=2048, vocab_size=32768, n_layer=4, n_head=2, n_kv_head=2, n_embd=256,
                    window_pattern="SSSL")
    with torch.device("meta"):
        model = GPT(cfg)
    model.to_empty(device="cpu")
    torch.manual_seed(0)
    model.init_weights()
    if binding:
        torch.manual_seed(0)
        s = 3 ** 0.5 * cfg.n_embd ** -0.5
        for blk in model.transformer.h:
            torch.nn.init.uniform_(blk.attn.c_proj.weight, -s, s)
            torch.nn.init.uniform_(blk.mlp.c_proj.weight, -s, s)
        torch.nn.init.normal_(model.lm_head.weight, mean=0.0, std=0.02)
        model.smear_lambda.data.fill_(0.5)
    model.window_sizes = [(1024, 0), (1024, 0), (1024, 0), (2048, 0)]
    return model.eval()


@pytest.mark.parametrize("binding", [False, True])
def test_config0_greedy_streams_equal_reference(golden_dir, binding):
    g = np.load(os.path.join(golden_dir, "config0_streams.npz"))
    tag = "binding" if binding else "stock"
    torch.set_num_threads(1)
    model = _config0_model(binding)
    sd = model.state_dict()
    assert sorted(sd) == list(g["state_keys"]), "parameter names differ from the reference's state_dict"
    np.testing.assert_allclose([float(sd[k].double().sum()) for k in sorted(sd)], g[tag + "_wsum"], rtol=1e-12, atol=1e-9)
    np.testing.assert_allclose([float(sd[k].double().abs().sum()) for k in sorted(sd)], g[tag + "_wabs"], rtol=1e-12)
    prompt = g["prompt"].tolist()
    with oracle_backend():
        eng = Engine(model, SpecialsTokenizer())
        res, _ = eng.generate_batch(prompt, num_samples=4, max_tokens=64, temperature=0.0)
        assert np.array_equal(np.array(res), g[tag]), "Engine stream differs from the reference's"
        naive = prompt + list(model.generate(prompt, max_tokens=16, temperature=0.0))
        assert naive == g[tag + "_naive"][:len(naive)].tolist(), "cache-free generation differs from the reference's"
        model.window_sizes = [(8, 0), (8, 0), (8, 0), (2048, 0)]
        res, _ = eng.generate_batch(prompt, num_samples=2, max_tokens=24, temperature=0.0)
        assert np.array_equal(np.array(res), g[tag + "_w8"])


# ------------------------------------------------------------------------------------------------
# paged cache: host-side page bookkeeping (the copy kernel replaced by a torch stand-in)
# ------------------------------------------------------------------------------------------------
def test_paged_cache_tables_sharing_and_growth(monkeypatch):
    from nanochat_b200 import ops
    from nanochat_b200.engine import PagedKVCache

    def fill_on_host(src_k, src_v, k_pool, v_pool, jobs):
        for page, t0, n in jobs.tolist():
            k_pool[:, page, :n] = src_k[:, 0, t0:t0 + n]
            v_pool[:, page, :n] = src_v[:, 0, t0:t0 + n]

    monkeypatch.setattr(ops, "paged_fill", fill_on_host)
    L, B, H, D, pt, p, cap = 2, 3, 2, 8, ops.PAGE_TILE, 2 * ops.PAGE_TILE + 5, 5 * ops.PAGE_TILE
    prompt = KVCache(1, H, p, D, L, "cpu", torch.float32)
    prompt.k_cache.copy_(torch.randn(prompt.k_cache.shape))
    prompt.v_cache.copy_(torch.randn(prompt.v_cache.shape))
    prompt.advance(p)
    prompt.prev_embedding = torch.randn(1, 1, 4)
    cache = PagedKVCache(B, H, cap, D, L, "cpu", torch.float32, page_tokens=pt, n_pages=2 + B * 2 + 1)
    assert cache.block_table.shape == (B, 5) and cache.pages_in_use() == 0
    cache.prefill(prompt)
    t = cache.block_table
    assert cache.cache_seqlens.tolist() == [p] * B and cache.pages_in_use() == 2 + B
    assert all(t[b, :2].tolist() == t[0, :2].tolist() for b in range(B))           # full prompt pages: shared
    assert len(set(t[:, 2].tolist())) == B and (t[:, 3:] == -1).all()              # tail page: one per row
    for b in range(B):                                                              # every token readable through the table
        for tok in (0, pt - 1, pt, p - 1):
            page, off = int(t[b, tok // pt]), tok % pt
            assert torch.equal(cache.k_cache[:, page, off], prompt.k_cache[:, 0, tok])
            assert torch.equal(cache.v_cache[:, page, off], prompt.v_cache[:, 0, tok])
    assert cache.prev_embedding.shape == (B, 1, 4)
    cache.reserve(p + 1)                                                            # still inside the tail page
    assert cache.pages_in_use() == 2 + B
    cache.reserve(3 * pt + 1)                                                       # one more page per row
    assert cache.pages_in_use() == 2 + 2 * B and (cache.block_table[:, 3] >= 0).all()
    assert len(set(cache.block_table[cache.block_table >= 0].tolist())) == 2 + 2 * B  # no page handed out twice
    with pytest.raises(RuntimeError, match="exhausted"):
        cache.reserve(cap + 10 * pt)                                                # clamps to capacity: 5 pages per row, one page short
    with pytest.raises(AssertionError):
        cache.prefill(prompt)                                                       # not empty
    cache.reset()
    assert cache.pages_in_use() == 0 and (cache.block_table == -1).all() and cache.get_pos() == 0
    with pytest.raises(ValueError):
        PagedKVCache(1, H, cap, D, L, "cpu", torch.float32, page_tokens=pt + 1)
