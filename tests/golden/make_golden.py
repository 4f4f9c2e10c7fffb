"""Generate tests/golden/*.npz by importing and running the reference nanochat on CPU.

Run once in a container that has the reference checkout (it is not needed to run the tests):

    python tests/golden/make_golden.py <path of the reference checkout>

The reference's tokenizer module imports the `rustbpe` wheel, which this path never uses; a stub
module stands in for it.  Everything else is the reference's own code, unmodified: the functions
called are apply_rotary_emb / norm (gpt.py:42-63), flash_attn_func / flash_attn_with_kvcache
(flash_attention.py:107-177, SDPA branch), KVCache (engine.py:82-137), GPT (gpt.py) and
Engine.generate_batch (engine.py:282-304).  Seeds and shapes are fixed below so the files can be
regenerated bit for bit with the same torch build (written with torch 2.11, CPU).
"""
import os
import sys
import types

import numpy as np


def main(ref_root):
    sys.modules.setdefault("rustbpe", types.ModuleType("rustbpe"))
    sys.path.insert(0, ref_root)
    here = os.path.dirname(os.path.abspath(__file__))
    import torch

    torch.set_num_threads(1)  # fixed reduction order inside torch's CPU kernels

    # ------------------------------------------------------------------ bf16 q/k pipeline
    os.environ["NANOCHAT_DTYPE"] = "bfloat16"
    from nanochat.gpt import GPT, GPTConfig, apply_rotary_emb, norm
    import nanochat.gpt as ref_gpt
    from nanochat.engine import Engine, KVCache
    from nanochat.flash_attention import flash_attn

    def tables(seq_len, head_dim, dtype):
        # GPT._precompute_rotary_embeddings does not touch self when a device is passed
        ref_gpt.COMPUTE_DTYPE = dtype
        cos, sin = GPT._precompute_rotary_embeddings(None, seq_len, head_dim, device="cpu")
        return cos, sin

    g = torch.Generator().manual_seed(11)
    cos_b, sin_b = tables(4096, 128, torch.bfloat16)
    x = torch.randn(3, 5, 4, 128, generator=g).bfloat16()
    T0 = 37
    c, s = cos_b[:, T0:T0 + 5], sin_b[:, T0:T0 + 5]
    y = apply_rotary_emb(x, c, s)
    z = norm(y)
    out = z * 1.2
    np.savez_compressed(
        os.path.join(here, "rope_norm_bf16.npz"),
        x=x.view(torch.int16).numpy(), T0=np.int64(T0),
        cos=cos_b[0, :, 0].view(torch.int16).numpy()[:64], sin=sin_b[0, :, 0].view(torch.int16).numpy()[:64],
        rope=y.view(torch.int16).numpy(), norm=z.view(torch.int16).numpy(), out=out.view(torch.int16).numpy())

    cos_f, sin_f = tables(4096, 128, torch.float32)
    xf = torch.randn(2, 3, 2, 128, generator=g)
    yf = norm(apply_rotary_emb(xf, cos_f[:, 5:8], sin_f[:, 5:8])) * 1.2
    rows = [0, 1, 2, 17, 100, 1000, 2047, 4095]
    np.savez_compressed(
        os.path.join(here, "rope_norm_fp32.npz"), x=xf.numpy(), T0=np.int64(5), out=yf.numpy(),
        table_rows=np.array(rows), cos_rows=cos_f[0, rows, 0].numpy(), sin_rows=sin_f[0, rows, 0].numpy(),
        cos_rows_bf16=cos_b[0, rows, 0].view(torch.int16).numpy(),
        sin_rows_bf16=sin_b[0, rows, 0].view(torch.int16).numpy())

    # ------------------------------------------------------------------ attention (fp32, SDPA branch)
    ref_gpt.COMPUTE_DTYPE = torch.float32
    cases = {}

    def kv_case(name, B, T_max, Hq, Hkv, D, prefix, T_new, window, seed):
        gg = torch.Generator().manual_seed(seed)
        k_cache = torch.zeros(B, T_max, Hkv, D)
        v_cache = torch.zeros(B, T_max, Hkv, D)
        k_cache[:, :prefix] = torch.randn(B, prefix, Hkv, D, generator=gg)
        v_cache[:, :prefix] = torch.randn(B, prefix, Hkv, D, generator=gg)
        q = torch.randn(B, T_new, Hq, D, generator=gg)
        k = torch.randn(B, T_new, Hkv, D, generator=gg)
        v = torch.randn(B, T_new, Hkv, D, generator=gg)
        seqlens = torch.full((B,), prefix, dtype=torch.int32)
        out = flash_attn.flash_attn_with_kvcache(q, k_cache, v_cache, k=k, v=v, cache_seqlens=seqlens,
                                                 causal=True, window_size=(window, 0))
        # the cache before the call is the cache after it with rows [prefix, prefix + T_new) zeroed
        cases[name] = dict(q=q, k=k, v=v, k_cache_after=k_cache, v_cache_after=v_cache, seqlens=seqlens,
                           window=np.int64(window), out=out)

    # the shapes of tests/test_attention_fallback.py:132-213 ...
    kv_case("ref_prefill", 2, 64, 4, 4, 32, 0, 16, 64, 1)
    kv_case("ref_single", 2, 64, 4, 4, 32, 16, 1, 64, 2)
    kv_case("ref_single_window", 2, 64, 4, 4, 32, 32, 1, 8, 3)
    # ... and the same situations at the head_dim the kernels are built for, plus GQA and chunks
    kv_case("d128_prefill", 2, 48, 2, 2, 128, 0, 16, 48, 4)
    kv_case("d128_single", 2, 48, 2, 2, 128, 16, 1, 48, 5)
    kv_case("d128_single_window", 2, 48, 2, 2, 128, 32, 1, 8, 6)
    kv_case("d128_gqa_single", 2, 40, 8, 2, 128, 21, 1, -1, 7)
    kv_case("d128_gqa_chunk_window", 1, 40, 4, 2, 128, 12, 5, 6, 8)
    kv_case("d128_chunk_full", 1, 40, 2, 2, 128, 9, 7, -1, 9)
    flat = {}
    for name, d in cases.items():
        for key, val in d.items():
            flat[f"{name}.{key}"] = val.numpy() if hasattr(val, "numpy") else val
    np.savez_compressed(os.path.join(here, "attn_kvcache_fp32.npz"), **flat)

    gg = torch.Generator().manual_seed(21)
    flat = {}
    for name, (B, T, Hq, Hkv, D, window) in {"causal": (2, 24, 2, 2, 128, -1), "window": (1, 24, 4, 2, 128, 5),
                                             "window_ge_T": (1, 10, 2, 1, 128, 10)}.items():
        q = torch.randn(B, T, Hq, D, generator=gg)
        k = torch.randn(B, T, Hkv, D, generator=gg)
        v = torch.randn(B, T, Hkv, D, generator=gg)
        out = flash_attn.flash_attn_func(q, k, v, causal=True, window_size=(window, 0))
        flat.update({f"{name}.q": q.numpy(), f"{name}.k": k.numpy(), f"{name}.v": v.numpy(),
                     f"{name}.window": np.int64(window), f"{name}.out": out.numpy()})
    np.savez_compressed(os.path.join(here, "attn_func_fp32.npz"), **flat)

    # ------------------------------------------------------------------ KVCache.prefill
    gg = torch.Generator().manual_seed(31)
    src = KVCache(batch_size=1, num_heads=2, seq_len=6, head_dim=128, num_layers=3, device="cpu", dtype=torch.float32)
    src.k_cache.copy_(torch.randn(src.k_cache.shape, generator=gg))
    src.v_cache.copy_(torch.randn(src.v_cache.shape, generator=gg))
    src.advance(6)
    dst = KVCache(batch_size=3, num_heads=2, seq_len=10, head_dim=128, num_layers=3, device="cpu", dtype=torch.float32)
    dst.prefill(src)
    np.savez_compressed(os.path.join(here, "kvcache_prefill.npz"), src_k=src.k_cache.numpy(), src_v=src.v_cache.numpy(),
                        dst_k=dst.k_cache.numpy(), dst_v=dst.v_cache.numpy(), dst_seqlens=dst.cache_seqlens.numpy())

    # ------------------------------------------------------------------ window sizes
    win = {}
    for seq_len, n_layer, pattern in [(2048, 4, "SSSL"), (2048, 24, "SSSL"), (4096, 32, "SSSL"), (1024, 5, "SL"),
                                      (2048, 3, "L"), (640, 6, "sls")]:
        with torch.device("meta"):
            m = GPT(GPTConfig(sequence_len=seq_len, vocab_size=64, n_layer=n_layer, n_head=1, n_kv_head=1,
                              n_embd=128, window_pattern=pattern))
        win[f"{seq_len}_{n_layer}_{pattern}"] = np.array(m.window_sizes, dtype=np.int64)
    np.savez_compressed(os.path.join(here, "window_sizes.npz"), **win)

    # ------------------------------------------------------------------ configs[0] greedy streams
    class Tok:  # the six special ids Engine asks for, placed above the byte range
        names = ["<|bos|>", "<|python_start|>", "<|python_end|>", "<|output_start|>", "<|output_end|>",
                 "<|assistant_end|>"]

        def encode_special(self, s):
            return 32768 + 100 + self.names.index(s)  # never produced by a 32768-way argmax

        def get_bos_token_id(self):
            return self.encode_special("<|bos|>")

        def encode(self, s, prepend=None):
            return list(s.encode())

        def decode(self, ids):
            return bytes(i for i in ids if i < 256).decode("utf-8", "replace")

    def build(binding):
        cfg = GPTConfig(sequence_len=2048, vocab_size=32768, n_layer=4, n_head=2, n_kv_head=2, n_embd=256,
                        window_pattern="SSSL")
        with torch.device("meta"):
            model = GPT(cfg)
        model.to_empty(device="cpu")
        torch.manual_seed(0)
        model.init_weights()
        if binding:
            # stock init zeroes every c_proj and the smear weight, so attention never reaches the
            # logits; re-draw them so that a wrong attention result changes the token stream
            torch.manual_seed(0)
            s_ = 3 ** 0.5 * cfg.n_embd ** -0.5
            for blk in model.transformer.h:
                torch.nn.init.uniform_(blk.attn.c_proj.weight, -s_, s_)
                torch.nn.init.uniform_(blk.mlp.c_proj.weight, -s_, s_)
            torch.nn.init.normal_(model.lm_head.weight, mean=0.0, std=0.02)
            model.smear_lambda.data.fill_(0.5)
        model.window_sizes = [(1024, 0), (1024, 0), (1024, 0), (2048, 0)]
        model.eval()
        return model

    prompt = torch.randint(0, 32768, (32,), generator=torch.Generator().manual_seed(1)).tolist()
    streams = {"prompt": np.array(prompt)}
    for binding in (False, True):
        model = build(binding)
        eng = Engine(model, Tok())
        res, _ = eng.generate_batch(prompt, num_samples=4, max_tokens=64, temperature=0.0)
        tag = "binding" if binding else "stock"
        streams[tag] = np.array(res)
        # naive no-cache generation must agree (engine.py:307-357)
        naive = list(model.generate(prompt, max_tokens=64, temperature=0.0))
        streams[tag + "_naive"] = np.array(prompt + naive)
        # small-window variant so that the S layers bind inside 96 positions
        model.window_sizes = [(8, 0), (8, 0), (8, 0), (2048, 0)]
        res, _ = eng.generate_batch(prompt, num_samples=2, max_tokens=24, temperature=0.0)
        streams[tag + "_w8"] = np.array(res)
        # a few weight checksums so a restated init can be pinned without shipping 150 MB
        sd = model.state_dict()
        streams[tag + "_wsum"] = np.array([float(sd[k].double().sum()) for k in sorted(sd)])
        streams[tag + "_wabs"] = np.array([float(sd[k].double().abs().sum()) for k in sorted(sd)])
        if not binding:
            streams["state_keys"] = np.array(sorted(sd))
    np.savez_compressed(os.path.join(here, "config0_streams.npz"), **streams)
    for f in sorted(os.listdir(here)):
        if f.endswith(".npz"):
            print(f, os.path.getsize(os.path.join(here, f)))


if __name__ == "__main__":
    if len(sys.argv) != 2:
        raise SystemExit("usage: python tests/golden/make_golden.py <path of the reference checkout>")
    main(sys.argv[1])
