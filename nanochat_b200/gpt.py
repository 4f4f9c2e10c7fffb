"""Inference-side mirror of nanochat's GPT (nanochat/gpt.py) with the attention KV branch on the
fused sm_100a kernels.

Scope.  The reference's hot path runs through ``CausalSelfAttention.forward`` (gpt.py:82-126); what
this module replaces is its KV branch (gpt.py:97-121): RoPE, QK-norm, the 1.2 scale, the cache
append and the attention call become two kernel launches (``kv_attention``).  Everything around it
(embeddings, smear, residual lambdas, value embeddings, MLP, backout, logit softcap) is the same
sequence of torch ops as the reference, kept so that the path can be driven end to end by
``Engine`` on random-init or checkpointed weights; parameter names match the reference's
``state_dict`` so its checkpoints load unchanged.  Training (loss, optimizers, autograd through
attention) is out of scope and absent.
"""
from dataclasses import dataclass

import torch
import torch.nn as nn
import torch.nn.functional as F

from . import ops
from .flash_attention import flash_attn


# ------------------------------------------------------------------------------------------------
# pure-host helpers
# ------------------------------------------------------------------------------------------------
def precompute_rotary_embeddings(seq_len, head_dim, base=100000, device=None, dtype=torch.bfloat16):
    """cos/sin tables of shape (1, seq_len, 1, head_dim/2): the op sequence of
    GPT._precompute_rotary_embeddings (gpt.py:268-283), so the tables are bit-identical to the
    reference's when made on the same device with the same dtype."""
    channel_range = torch.arange(0, head_dim, 2, dtype=torch.float32, device=device)
    inv_freq = 1.0 / (base ** (channel_range / head_dim))
    t = torch.arange(seq_len, dtype=torch.float32, device=device)
    freqs = torch.outer(t, inv_freq)
    cos, sin = freqs.cos().to(dtype), freqs.sin().to(dtype)
    return cos[None, :, None, :], sin[None, :, None, :]


def compute_window_sizes(sequence_len, n_layer, window_pattern="SSSL"):
    """Per-layer (left, right) windows as GPT._compute_window_sizes (gpt.py:285-312): 'L' is
    sequence_len, 'S' is ceil(sequence_len / 4 / 128) * 128, the pattern is tiled over the
    layers and the last layer is always 'L'."""
    pattern = window_pattern.upper()
    assert pattern and all(c in "SL" for c in pattern), f"Invalid window_pattern: {pattern}. Use only S and L."
    long_window = sequence_len
    short_window = -(-long_window // 4 // 128) * 128
    sizes = [(long_window if pattern[i % len(pattern)] == "L" else short_window, 0) for i in range(n_layer)]
    sizes[-1] = (long_window, 0)
    return sizes


def kv_attention(q, k, v, cos_sin_tables, window_size, kv_cache, layer_idx):
    """The KV-cache branch of CausalSelfAttention.forward (gpt.py:97-121) in two launches.

    q: (B, T, Hq, D), k, v: (B, T, Hkv, D) straight from the projections (v already carries the
    value-embedding gate).  ``cos_sin_tables`` are the FULL tables (1, rope_len, 1, D/2): each row
    is rotated at its own position ``kv_cache.cache_seqlens[b] + t`` on the device, so no
    ``get_pos()`` synchronisation and no table slicing is needed.  Launch 1 applies RoPE, QK-norm
    and the 1.2 scale to q and k and appends k/v to the layer's cache; launch 2 attends.
    As in the reference the cache position is advanced once, after the last layer.
    Returns y of shape (B, T, Hq, D).
    """
    cos, sin = cos_sin_tables
    k_cache, v_cache = kv_cache.get_layer_cache(layer_idx)
    seqlens = kv_cache.cache_seqlens
    T = q.size(1)
    left = int(window_size[0])
    left = left if left >= 0 else -1
    if getattr(kv_cache, "paged", False):  # page pools + block table instead of dense rows
        if T != 1:
            raise NotImplementedError("a paged cache takes one new token per row; prefill the prompt into a dense "
                                      "batch-1 KVCache and hand it over with PagedKVCache.prefill")
        q2 = ops.append_rope_norm_paged(q, k, v, k_cache, v_cache, kv_cache.block_table, seqlens, cos, sin)
        y = ops.decode_attention_paged(q2[:, 0], k_cache, v_cache, kv_cache.block_table, seqlens, seqlen_offset=1,
                                       window_left=left).unsqueeze(1)
        if layer_idx == kv_cache.n_layers - 1:
            kv_cache.advance(T)
        return y
    q2 = ops.append_rope_norm(q, k, v, k_cache, v_cache, seqlens, cos, sin)
    if T == 1:
        y = ops.decode_attention(q2[:, 0], k_cache, v_cache, seqlens, seqlen_offset=1, window_left=left).unsqueeze(1)
    else:
        y = ops.prefill_attention(q2, k_cache, v_cache, seqlens, left)
    if layer_idx == kv_cache.n_layers - 1:
        kv_cache.advance(T)
    return y


# ------------------------------------------------------------------------------------------------
# model
# ------------------------------------------------------------------------------------------------
@dataclass
class GPTConfig:
    """Same fields and defaults as the reference's GPTConfig (gpt.py:28-39)."""
    sequence_len: int = 2048
    vocab_size: int = 32768
    n_layer: int = 12
    n_head: int = 6
    n_kv_head: int = 6
    n_embd: int = 768
    window_pattern: str = "SSSL"


def rms(x):
    """Parameter-free rms-norm over the last dim (gpt.py:42-43)."""
    return F.rms_norm(x, (x.size(-1),))


def layer_has_value_embedding(layer_idx, n_layer):
    """Alternating layers carry a value embedding, the last layer always does (gpt.py:53-55)."""
    return layer_idx % 2 == (n_layer - 1) % 2


class CastLinear(nn.Linear):
    """Bias-free linear whose weight is used in the activation's dtype (gpt.py:45-50).  The cast is
    skipped when the dtypes already agree, e.g. after ``model.to(torch.bfloat16)``."""

    def forward(self, x):
        w = self.weight if self.weight.dtype == x.dtype else self.weight.to(dtype=x.dtype)
        return F.linear(x, w)


class Attention(nn.Module):
    def __init__(self, config, layer_idx):
        super().__init__()
        self.layer_idx = layer_idx
        self.n_head, self.n_kv_head = config.n_head, config.n_kv_head
        assert config.n_embd % config.n_head == 0 and config.n_head % config.n_kv_head == 0
        self.head_dim = config.n_embd // config.n_head
        self.c_q = CastLinear(config.n_embd, self.n_head * self.head_dim, bias=False)
        self.c_k = CastLinear(config.n_embd, self.n_kv_head * self.head_dim, bias=False)
        self.c_v = CastLinear(config.n_embd, self.n_kv_head * self.head_dim, bias=False)
        self.c_proj = CastLinear(config.n_embd, config.n_embd, bias=False)
        self.ve_gate_channels = 12
        self.ve_gate = (CastLinear(self.ve_gate_channels, self.n_kv_head, bias=False)
                        if layer_has_value_embedding(layer_idx, config.n_layer) else None)
        self._qkv_cache = None

    def fused_qkv_weight(self, x):
        """[c_q; c_k; c_v] as one weight for activations like ``x`` (rows, n_embd), or None.

        One product over the stacked weight replaces three launches.  It is only used when it reproduces the
        three separate products bit for bit (the K/V bytes that reach the cache must be those of the
        reference's projections, gpt.py:88-90): that is checked once per (weights, dtype, row count) on
        random activations, outside stream capture; a step captured before the check has run keeps the three
        products.  Costs a second copy of the three weights.  (Stacking the value gate's rows as well, zero
        over the channels it does not read, was bit-identical only for some shapes and saved nothing measurable.)"""
        ws = (self.c_q.weight, self.c_k.weight, self.c_v.weight)
        rows = x.numel() // x.size(-1)
        key = tuple((w.data_ptr(), w._version) for w in ws) + (x.dtype, rows)
        if self._qkv_cache is None or self._qkv_cache[0] != key:
            if torch.cuda.is_current_stream_capturing():
                return None
            wq, wk, wv = (w.detach().to(x.dtype) for w in ws)
            stacked = torch.cat([wq, wk, wv], 0).contiguous()
            gen = torch.Generator(device=x.device).manual_seed(1234)
            same = True
            for _ in range(2):
                probe = torch.randn(rows, x.size(-1), generator=gen, device=x.device).to(x.dtype)
                apart = torch.cat([F.linear(probe, wq), F.linear(probe, wk), F.linear(probe, wv)], 1)
                same = same and torch.equal(F.linear(probe, stacked), apart)
            self._qkv_cache = (key, stacked if same else None)
        return self._qkv_cache[1]

    def forward(self, x, ve, rope_tables, window_size, kv_cache):
        B, T, _ = x.shape
        q = self.c_q(x).view(B, T, self.n_head, self.head_dim)
        k = self.c_k(x).view(B, T, self.n_kv_head, self.head_dim)
        v = self.c_v(x).view(B, T, self.n_kv_head, self.head_dim)
        if ve is not None:  # value residual with an input-dependent per-head gate (gpt.py:92-95)
            gate = 3 * torch.sigmoid(self.ve_gate(x[..., :self.ve_gate_channels]))
            v = v + gate.unsqueeze(-1) * ve.view(B, T, self.n_kv_head, self.head_dim)
        if kv_cache is not None:
            y = kv_attention(q, k, v, rope_tables, window_size, kv_cache, self.layer_idx)
        else:
            # no cache (naive generation): positions start at 0 for every row; RoPE / QK-norm are
            # plain torch ops here, the attention itself is the dense kernel
            cos, sin = rope_tables[0][:, :T], rope_tables[1][:, :T]
            q, k = _rope_norm_scale(q, cos, sin), _rope_norm_scale(k, cos, sin)
            y = flash_attn.flash_attn_func(q, k, v, causal=True, window_size=window_size)
        return self.c_proj(y.contiguous().view(B, T, -1))


def _rope_norm_scale(x, cos, sin):
    d = x.shape[3] // 2
    x1, x2 = x[..., :d], x[..., d:]
    y = torch.cat([x1 * cos + x2 * sin, x1 * (-sin) + x2 * cos], 3)
    return rms(y) * 1.2


class MLP(nn.Module):
    def __init__(self, config):
        super().__init__()
        self.c_fc = CastLinear(config.n_embd, 4 * config.n_embd, bias=False)
        self.c_proj = CastLinear(4 * config.n_embd, config.n_embd, bias=False)

    def forward(self, x):
        return self.c_proj(F.relu(self.c_fc(x)).square())


class Block(nn.Module):
    def __init__(self, config, layer_idx):
        super().__init__()
        self.attn = Attention(config, layer_idx)
        self.mlp = MLP(config)

    def forward(self, x, ve, rope_tables, window_size, kv_cache):
        x = x + self.attn(rms(x), ve, rope_tables, window_size, kv_cache)
        return x + self.mlp(rms(x))


class GPT(nn.Module):
    """Inference-only GPT with the reference's module tree and forward arithmetic (gpt.py:154-481)."""

    def __init__(self, config, pad_vocab_size_to=64, compute_dtype=None):
        super().__init__()
        self.config = config
        self.compute_dtype = compute_dtype  # resolved in init_weights / on first forward
        self.window_sizes = compute_window_sizes(config.sequence_len, config.n_layer, config.window_pattern)
        padded = -(-config.vocab_size // pad_vocab_size_to) * pad_vocab_size_to
        self.transformer = nn.ModuleDict({
            "wte": nn.Embedding(padded, config.n_embd),
            "h": nn.ModuleList([Block(config, i) for i in range(config.n_layer)]),
        })
        self.lm_head = CastLinear(config.n_embd, padded, bias=False)
        self.resid_lambdas = nn.Parameter(torch.ones(config.n_layer))
        self.x0_lambdas = nn.Parameter(torch.zeros(config.n_layer))
        self.smear_gate = CastLinear(24, 1, bias=False)
        self.smear_lambda = nn.Parameter(torch.zeros(1))
        self.backout_lambda = nn.Parameter(0.2 * torch.ones(1))
        head_dim = config.n_embd // config.n_head
        kv_dim = config.n_kv_head * head_dim
        self.value_embeds = nn.ModuleDict({str(i): nn.Embedding(padded, kv_dim) for i in range(config.n_layer)
                                           if layer_has_value_embedding(i, config.n_layer)})
        # Decode steps (one new token per row, CUDA, bf16) run the elementwise glue between the matrix
        # products through the fused kernels of libnckv (bit-identical to the eager ops); set False to
        # run the eager op sequence everywhere.
        self.fused_glue = True
        self.fused_qkv = True   # one [c_q; c_k; c_v] product per layer in the decode trunk where it is bit-identical
        self._lambda_cache = None
        self.rotary_seq_len = config.sequence_len * 10  # same over-allocation as gpt.py:195
        self.register_buffer("cos", torch.empty(0), persistent=False)
        self.register_buffer("sin", torch.empty(0), persistent=False)

    def get_device(self):
        return self.transformer.wte.weight.device

    def _resolve_dtype(self):
        if self.compute_dtype is None:
            self.compute_dtype = torch.bfloat16 if self.get_device().type == "cuda" else torch.float32
        return self.compute_dtype

    def build_rotary(self, seq_len=None):
        """(Re)build the cos/sin tables on the model's device in the compute dtype."""
        if seq_len is not None:
            self.rotary_seq_len = seq_len
        head_dim = self.config.n_embd // self.config.n_head
        self.cos, self.sin = precompute_rotary_embeddings(self.rotary_seq_len, head_dim, device=self.get_device(),
                                                          dtype=self._resolve_dtype())

    @torch.no_grad()
    def init_weights(self):
        """Random init that consumes the torch RNG in the reference's order (gpt.py:202-265), so the
        same seed gives the same weights."""
        cfg = self.config
        s = 3 ** 0.5 * cfg.n_embd ** -0.5
        nn.init.normal_(self.transformer.wte.weight, mean=0.0, std=0.8)
        nn.init.normal_(self.lm_head.weight, mean=0.0, std=0.001)
        for blk in self.transformer.h:
            for lin in (blk.attn.c_q, blk.attn.c_k, blk.attn.c_v):
                nn.init.uniform_(lin.weight, -s, s)
            nn.init.zeros_(blk.attn.c_proj.weight)
            nn.init.uniform_(blk.mlp.c_fc.weight, -s * 0.4, s * 0.4)
            nn.init.zeros_(blk.mlp.c_proj.weight)
        denom = max(cfg.n_layer - 1, 1)
        for i in range(cfg.n_layer):
            self.resid_lambdas.data[i] = 1.15 - (0.10 * i / denom)
        for i in range(cfg.n_layer):
            self.x0_lambdas.data[i] = 0.20 - (0.15 * i / denom)
        nn.init.zeros_(self.smear_lambda)
        nn.init.constant_(self.backout_lambda, 0.2)
        nn.init.uniform_(self.smear_gate.weight, 0.0, 0.02)
        for ve in self.value_embeds.values():
            nn.init.uniform_(ve.weight, -s, s)
        for blk in self.transformer.h:
            if blk.attn.ve_gate is not None:
                nn.init.uniform_(blk.attn.ve_gate.weight, 0.0, 0.02)
        self.build_rotary()
        dtype = self._resolve_dtype()
        if dtype != torch.float16:  # embeddings live in the compute dtype (gpt.py:259-265)
            self.transformer.wte.to(dtype=dtype)
            for ve in self.value_embeds.values():
                ve.to(dtype=dtype)

    @torch.inference_mode()
    def forward(self, idx, targets=None, kv_cache=None, loss_reduction="mean"):
        """Logits (B, T, vocab) in fp32.  Same arithmetic as gpt.py:416-472; ``targets`` is rejected
        (no training here)."""
        if targets is not None:
            raise NotImplementedError("this GPT is inference-only")
        B, T = idx.shape
        dtype = self._resolve_dtype()
        if self.cos.numel() == 0:
            self.build_rotary()
        assert T <= self.cos.size(1), f"Sequence length grew beyond the rotary embeddings cache: {T} > {self.cos.size(1)}"
        x = rms(self.transformer.wte(idx).to(dtype))
        if kv_cache is None:
            assert T > 1, "a forward pass without a KV cache needs T > 1"
            gate = self.smear_lambda.to(x.dtype) * torch.sigmoid(self.smear_gate(x[:, 1:, :24]))
            x = torch.cat([x[:, :1], x[:, 1:] + gate * x[:, :-1]], dim=1)
        else:
            prev = kv_cache.prev_embedding
            kv_cache.prev_embedding = x[:, -1:, :]
            if T > 1:
                gate = self.smear_lambda.to(x.dtype) * torch.sigmoid(self.smear_gate(x[:, 1:, :24]))
                x = torch.cat([x[:, :1], x[:, 1:] + gate * x[:, :-1]], dim=1)
            elif prev is not None:
                gate = self.smear_lambda.to(x.dtype) * torch.sigmoid(self.smear_gate(x[:, :, :24]))
                x = x + gate * prev
        x0 = x
        backout_at = self.config.n_layer // 2
        x_backout = None
        rope_tables = (self.cos, self.sin)
        if self.fused_glue and T == 1 and kv_cache is not None and x.is_cuda and x.dtype == torch.bfloat16:
            return self._decode_trunk_fused(idx, x, kv_cache, rope_tables)
        for i, block in enumerate(self.transformer.h):
            x = self.resid_lambdas[i] * x + self.x0_lambdas[i] * x0
            ve = self.value_embeds[str(i)](idx).to(x.dtype) if str(i) in self.value_embeds else None
            x = block(x, ve, rope_tables, self.window_sizes[i], kv_cache)
            if i == backout_at:
                x_backout = x
        if x_backout is not None:
            x = x - self.backout_lambda.to(x.dtype) * x_backout
        x = rms(x)
        logits = self.lm_head(x)[..., :self.config.vocab_size].float()
        return 15 * torch.tanh(logits / 15)

    def _lambdas(self):
        """Host copies of the per-layer scalars, read once (a device read per step would synchronise),
        rounded to bf16: the eager multiply converts a 0-dim parameter to the activation dtype before it
        multiplies (and gpt.py:467 casts the backout lambda explicitly)."""
        key = (self.resid_lambdas.data_ptr(), self.resid_lambdas._version, self.x0_lambdas._version,
               self.backout_lambda._version, self.resid_lambdas.dtype)
        if self._lambda_cache is None or self._lambda_cache[0] != key:
            as_bf16 = lambda t: t.detach().to(torch.bfloat16).float()
            self._lambda_cache = (key, as_bf16(self.resid_lambdas).tolist(), as_bf16(self.x0_lambdas).tolist(),
                                  float(as_bf16(self.backout_lambda).item()))
        return self._lambda_cache[1:]

    def _decode_trunk_fused(self, idx, x, kv_cache, rope_tables):
        """The layer loop of ``forward`` for one new token per row with the elementwise glue fused:
        per layer one launch for [previous MLP residual add + lambda mix + norm], one for [attention
        residual add + norm], one for relu^2 (and one for the value-embedding gate where a layer has
        one), instead of about a dozen eager launches.  Same matrix products, same roundings."""
        B = idx.size(0)
        C = x.size(-1)
        resid, x0l, backout = self._lambdas()
        n_layer = self.config.n_layer
        backout_at = n_layer // 2
        x = x.contiguous()
        x0 = x
        pending = None      # MLP output of the previous layer, not yet added to the residual stream
        x_backout = None
        for i, block in enumerate(self.transformer.h):
            # the residual stream after layer backout_at is needed later: keep the sum when the add happens
            x_sum, x, xn = ops.glue_mix_norm(x, add=pending, x0=x0, resid_lambda=resid[i], x0_lambda=x0l[i],
                                             want_sum=(i == backout_at + 1))
            if i == backout_at + 1:
                x_backout = x_sum
            attn = block.attn
            w_qkv = attn.fused_qkv_weight(xn) if self.fused_qkv else None
            if w_qkv is not None:  # one product; q, k, v are column slices of its output (the kernels take the stride)
                nq, nkv = attn.n_head * attn.head_dim, attn.n_kv_head * attn.head_dim
                qkv = F.linear(xn, w_qkv)
                q = qkv[..., :nq].view(B, 1, attn.n_head, attn.head_dim)
                k = qkv[..., nq:nq + nkv].view(B, 1, attn.n_kv_head, attn.head_dim)
                v = qkv[..., nq + nkv:].view(B, 1, attn.n_kv_head, attn.head_dim)
            else:
                q = attn.c_q(xn).view(B, 1, attn.n_head, attn.head_dim)
                k = attn.c_k(xn).view(B, 1, attn.n_kv_head, attn.head_dim)
                v = attn.c_v(xn).view(B, 1, attn.n_kv_head, attn.head_dim)
            if str(i) in self.value_embeds:
                ve = self.value_embeds[str(i)](idx).to(x.dtype)
                v = ops.glue_ve_gate(v, attn.ve_gate(xn[..., :attn.ve_gate_channels]), ve)
            y = kv_attention(q, k, v, rope_tables, self.window_sizes[i], kv_cache, i)
            _, x, xn = ops.glue_mix_norm(x, add=attn.c_proj(y.view(B, 1, C)))
            pending = block.mlp.c_proj(ops.glue_relu_sq(block.mlp.c_fc(xn)))
        if backout_at == n_layer - 1:  # only a one-layer model: the backout operand is the final sum itself
            x_backout, _, _ = ops.glue_mix_norm(x, add=pending, want_sum=True, want_x=False, want_norm=False)
            _, _, xn = ops.glue_mix_norm(x_backout, x_backout=x_backout, backout_lambda=backout, want_x=False)
        else:
            _, _, xn = ops.glue_mix_norm(x, add=pending, x_backout=x_backout, backout_lambda=backout, want_x=False)
        logits = self.lm_head(xn)[..., :self.config.vocab_size].float()
        return 15 * torch.tanh(logits / 15)

    @torch.inference_mode()
    def generate(self, tokens, max_tokens, temperature=1.0, top_k=None, seed=42):
        """Naive generation without a cache, one full forward per token (gpt.py:483-512); kept as
        the independent check of the cached path (engine.py:307-357)."""
        assert isinstance(tokens, list)
        device = self.get_device()
        rng = None
        if temperature > 0:
            rng = torch.Generator(device=device)
            rng.manual_seed(seed)
        ids = torch.tensor([tokens], dtype=torch.long, device=device)
        for _ in range(max_tokens):
            logits = self.forward(ids)[:, -1, :]
            if top_k is not None and top_k > 0:
                vals, _ = torch.topk(logits, min(top_k, logits.size(-1)))
                logits[logits < vals[:, [-1]]] = -float("inf")
            if temperature > 0:
                probs = F.softmax(logits / temperature, dim=-1)
                nxt = torch.multinomial(probs, num_samples=1, generator=rng)
            else:
                nxt = torch.argmax(logits, dim=-1, keepdim=True)
            ids = torch.cat((ids, nxt), dim=1)
            yield nxt.item()
