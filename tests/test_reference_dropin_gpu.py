"""The drop-in, tested with the reference itself in the loop.

The unmodified reference modules (nanochat/gpt.py, engine.py, flash_attention.py, staged under
oracle/_ref by oracle/make_ref.py) run on the GPU in bf16.  Twice: as they are (their SDPA path, which
is what the reference executes on a B200), and with the two names this library replaces pointed at the
mirrors, exactly as an integrator would do it:

    nanochat.gpt.flash_attn   -> nanochat_b200.flash_attention.flash_attn
    nanochat.engine.KVCache   -> nanochat_b200.engine.KVCache

Model: benchmark configuration 0 (depth 4, 2 heads x 128, vocab 32768, SSSL), 32-token prompt, 4 samples,
64 greedy tokens; the stock initialisation and the "binding" one (c_proj re-drawn so that attention
reaches the logits).  These tests FAIL when oracle/_ref is missing; they do not skip.
"""
import contextlib

import numpy as np
import pytest
import torch

from tests.cpu_backend import SpecialsTokenizer

pytestmark = pytest.mark.gpu
DEV = "cuda"
BF = torch.bfloat16


def _ref():
    from oracle import ref_loader
    ref_loader.load("bfloat16")
    import nanochat.engine as ref_engine
    import nanochat.gpt as ref_gpt
    assert ref_gpt.COMPUTE_DTYPE == BF, "the reference must run its bf16 path here"
    return ref_gpt, ref_engine


@contextlib.contextmanager
def _mirrors_swapped_in(ref_gpt, ref_engine):
    from nanochat_b200.engine import KVCache
    from nanochat_b200.flash_attention import flash_attn
    saved = ref_gpt.flash_attn, ref_engine.KVCache
    ref_gpt.flash_attn, ref_engine.KVCache = flash_attn, KVCache
    try:
        yield
    finally:
        ref_gpt.flash_attn, ref_engine.KVCache = saved


def _config0(ref_gpt, binding, seed=0):
    cfg = ref_gpt.GPTConfig(sequence_len=2048, vocab_size=32768, n_layer=4, n_head=2, n_kv_head=2, n_embd=256,
                            window_pattern="SSSL")
    with torch.device("meta"):
        model = ref_gpt.GPT(cfg)
    model.to_empty(device=DEV)
    torch.manual_seed(seed)
    model.init_weights()
    if binding:
        torch.manual_seed(seed)
        s = 3 ** 0.5 * cfg.n_embd ** -0.5
        for blk in model.transformer.h:
            torch.nn.init.uniform_(blk.attn.c_proj.weight, -s, s)
            torch.nn.init.uniform_(blk.mlp.c_proj.weight, -s, s)
        torch.nn.init.normal_(model.lm_head.weight, mean=0.0, std=0.02)
        model.smear_lambda.data.fill_(0.5)
    model.window_sizes = [(1024, 0), (1024, 0), (1024, 0), (2048, 0)]
    return model.eval()


def _prompt():
    return torch.randint(0, 32768, (32,), generator=torch.Generator().manual_seed(1)).tolist()


@torch.inference_mode()
def _run(model, cache_cls, prompt, num_samples, forced=None, steps=64, dtype=BF):
    """Engine.generate's call sequence with the caches kept: batch-1 prefill, broadcast to num_samples rows,
    greedy steps (or the given continuation fed back).  Returns tokens, logits per step, seqlens per step, cache."""
    cfg = model.config
    geo = dict(num_heads=cfg.n_kv_head, head_dim=cfg.n_embd // cfg.n_head, num_layers=cfg.n_layer)
    pc = cache_cls(batch_size=1, seq_len=len(prompt), device=DEV, dtype=dtype, **geo)
    logits = model.forward(torch.tensor([prompt], dtype=torch.long, device=DEV), kv_cache=pc)[:, -1, :].expand(num_samples, -1)
    cache = cache_cls(batch_size=num_samples, seq_len=len(prompt) + steps, device=DEV, dtype=dtype, **geo)
    cache.prefill(pc)
    toks, all_logits, lens = [], [logits.float().clone()], [cache.cache_seqlens.clone()]
    for i in range(steps):
        nxt = torch.argmax(logits, dim=-1, keepdim=True) if forced is None else \
            torch.tensor([[forced[i]]] * num_samples, dtype=torch.long, device=DEV)
        toks.append(nxt[:, 0].tolist())
        logits = model.forward(nxt, kv_cache=cache)[:, -1, :]
        all_logits.append(logits.float().clone())
        lens.append(cache.cache_seqlens.clone())
    return toks, torch.stack(all_logits), lens, cache


@pytest.mark.parametrize("binding", [False, True])
def test_reference_engine_with_mirrors_swapped_in(binding):
    from nanochat_b200 import ops
    from nanochat_b200.engine import KVCache as OurCache
    ref_gpt, ref_engine = _ref()
    model = _config0(ref_gpt, binding)
    prompt = _prompt()
    tok = SpecialsTokenizer()

    # the reference's own generation loop, unpatched and patched
    ref_stream, _ = ref_engine.Engine(model, tok).generate_batch(prompt, num_samples=4, max_tokens=64, temperature=0.0)
    with _mirrors_swapped_in(ref_gpt, ref_engine):
        our_stream, _ = ref_engine.Engine(model, tok).generate_batch(prompt, num_samples=4, max_tokens=64, temperature=0.0)
    ops.check_status(DEV)
    assert all(r == our_stream[0] for r in our_stream) and all(r == ref_stream[0] for r in ref_stream)

    # the same sequence with the caches kept
    t_ref, l_ref, n_ref, c_ref = _run(model, ref_engine.KVCache, prompt, 4)
    with _mirrors_swapped_in(ref_gpt, ref_engine):
        t_our, l_our, n_our, c_our = _run(model, OurCache, prompt, 4)
    for a, b in zip(n_ref, n_our):
        assert torch.equal(a, b), "cache_seqlens differ"
    assert c_our.cache_seqlens.dtype == c_ref.cache_seqlens.dtype == torch.int32
    if not binding:
        # attention never reaches the residual stream (c_proj = 0): every layer's k/v is the same function of the
        # same inputs on both paths, so streams and all cache bytes must be identical
        assert our_stream == ref_stream
        assert torch.equal(c_our.k_cache.view(torch.int16), c_ref.k_cache.view(torch.int16))
        assert torch.equal(c_our.v_cache.view(torch.int16), c_ref.v_cache.view(torch.int16))
        return

    # binding weights: layer 0's keys/values do not depend on any attention output -> bit-exact while the streams agree
    gen_ref, gen_our = ref_stream[0][len(prompt):], our_stream[0][len(prompt):]
    same = next((i for i, (x, y) in enumerate(zip(gen_our, gen_ref)) if x != y), len(gen_ref))
    upto = len(prompt) + same
    assert torch.equal(c_our.k_cache[0, :, :upto].view(torch.int16), c_ref.k_cache[0, :, :upto].view(torch.int16))
    assert torch.equal(c_our.v_cache[0, :, :upto].view(torch.int16), c_ref.v_cache[0, :, :upto].view(torch.int16))

    # teacher-forced along the reference's stream: both bf16 paths against the reference computing in fp32
    forced = gen_ref
    _, a_ref, _, _ = _run(model, ref_engine.KVCache, prompt, 1, forced=forced)
    with _mirrors_swapped_in(ref_gpt, ref_engine):
        _, a_our, _, _ = _run(model, OurCache, prompt, 1, forced=forced)
    ref_gpt.COMPUTE_DTYPE = torch.float32
    try:
        m32 = _config0(ref_gpt, binding)  # same seed, fp32 compute; embeddings rounded like the bf16 model's
        sd = {k: v.float() for k, v in model.state_dict().items()}
        m32.load_state_dict(sd)
        _, a_32, _, _ = _run(m32, ref_engine.KVCache, prompt, 1, forced=forced, dtype=torch.float32)
    finally:
        ref_gpt.COMPUTE_DTYPE = BF
    err_ref = (a_ref - a_32).abs()
    err_our = (a_our - a_32).abs()
    print(f"teacher-forced logits vs fp32: reference bf16 max {err_ref.max():.4f} mean {err_ref.mean():.5f} | "
          f"this library max {err_our.max():.4f} mean {err_our.mean():.5f} | between the two bf16 paths "
          f"{(a_our - a_ref).abs().max():.4f}")
    # no worse than the reference's own bf16 path (25 % slack on the max, 10 % on the mean)
    assert err_our.max() <= 1.25 * err_ref.max() + 1e-3
    assert err_our.mean() <= 1.10 * err_ref.mean() + 1e-5
    if same < len(gen_ref):
        # the streams part ways: only legitimate where fp32 itself sees the two candidates within bf16 noise
        noise = max(err_ref.max().item(), err_our.max().item())
        gap = abs((a_32[same, 0, gen_ref[same]] - a_32[same, 0, gen_our[same]]).item())
        print(f"streams fork at generated token {same}: fp32 margin {gap:.4f}, bf16 noise {noise:.4f}")
        assert gap <= 2 * noise, f"fork at step {same} with a clear fp32 margin {gap}"


@pytest.mark.parametrize("B,T_new,Hq,Hkv", [(32, 1, 12, 12), (8, 1, 16, 4), (2, 37, 4, 2)])
def test_fused_append_bytes_equal_the_references_own_functions(B, T_new, Hq, Hkv):
    """q', k' and the cache rows written by the fused kernel against apply_rotary_emb / norm / * 1.2 of the
    reference module itself (gpt.py:42-63, 99-102) run on the GPU in bf16: zero differing bytes."""
    from nanochat_b200 import ops
    ref_gpt, _ = _ref()
    T_max = 2048
    gen = torch.Generator(device=DEV).manual_seed(100 + B)
    cos, sin = ref_gpt.GPT._precompute_rotary_embeddings(None, T_max, 128, device=DEV)
    assert cos.dtype == BF
    q = torch.randn(B, T_new, Hq, 128, generator=gen, device=DEV).to(BF)
    k = torch.randn(B, T_new, Hkv, 128, generator=gen, device=DEV).to(BF)
    v = torch.randn(B, T_new, Hkv, 128, generator=gen, device=DEV).to(BF)
    lens = torch.randint(0, T_max - T_new, (B,), generator=gen, device=DEV, dtype=torch.int32)
    kc = torch.zeros(B, T_max, Hkv, 128, device=DEV, dtype=BF)
    vc = torch.zeros_like(kc)
    q_out = ops.append_rope_norm(q, k, v, kc, vc, lens, cos, sin)
    torch.cuda.synchronize()
    assert ops.read_status(DEV) == 0
    bad = 0
    for b, L in enumerate(lens.tolist()):
        c, s = cos[:, L:L + T_new], sin[:, L:L + T_new]
        q_ref = ref_gpt.norm(ref_gpt.apply_rotary_emb(q[b:b + 1], c, s)) * 1.2
        k_ref = ref_gpt.norm(ref_gpt.apply_rotary_emb(k[b:b + 1], c, s)) * 1.2
        bad += (q_out[b:b + 1].view(torch.int16) != q_ref.view(torch.int16)).sum().item()
        bad += (kc[b:b + 1, L:L + T_new].view(torch.int16) != k_ref.view(torch.int16)).sum().item()
        bad += (vc[b:b + 1, L:L + T_new].view(torch.int16) != v[b:b + 1].view(torch.int16)).sum().item()
    assert bad == 0, f"{bad} elements differ from the reference's bf16 GPU path"


def test_reference_training_step_with_flash_attn_func_swapped_in():
    """The reference GPT's own training forward (gpt.py:416-472 with targets, attention through
    flash_attn_func at gpt.py:108) and loss.backward(), once on its SDPA path and once with flash_attn pointed
    at the mirror: the loss and every parameter gradient agree to bf16 accuracy.  Short windows on three of the
    four layers so that the sliding-window backward is exercised."""
    ref_gpt, ref_engine = _ref()
    model = _config0(ref_gpt, binding=True, seed=5)
    model.window_sizes = [(64, 0), (96, 0), (64, 0), (2048, 0)]
    gen = torch.Generator().manual_seed(9)
    idx = torch.randint(0, 32768, (2, 320), generator=gen).to(DEV)
    targets = torch.randint(0, 32768, (2, 320), generator=gen).to(DEV)

    def step():
        model.zero_grad(set_to_none=True)
        loss = model(idx, targets)
        loss.backward()
        return loss.detach().float().item(), {n: p.grad.detach().float().clone() for n, p in model.named_parameters()
                                             if p.grad is not None}

    loss_ref, g_ref = step()
    with _mirrors_swapped_in(ref_gpt, ref_engine):
        loss_our, g_our = step()
    from nanochat_b200 import ops
    assert ops.read_status(DEV) == 0
    assert abs(loss_our - loss_ref) <= 2e-3 * abs(loss_ref), (loss_our, loss_ref)
    assert g_our.keys() == g_ref.keys() and len(g_ref) > 10
    worst = 0.0
    for n in g_ref:
        denom = g_ref[n].norm().item()
        if denom == 0.0:
            assert g_our[n].norm().item() == 0.0, n
            continue
        rel = (g_our[n] - g_ref[n]).norm().item() / denom
        worst = max(worst, rel)
        assert rel <= 3e-2, f"{n}: gradient differs by {rel:.4f} of its norm"
    print(f"training step: loss {loss_our:.5f} vs {loss_ref:.5f}, worst relative gradient difference {worst:.4f}")
