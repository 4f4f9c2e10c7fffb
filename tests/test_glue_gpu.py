"""The fused decode-time glue kernels against the eager bf16 op sequences they replace
(nanochat/gpt.py:457, 148-150, 466-468, 136, 92-95): bit-identical, element for element."""
import pytest
import torch
import torch.nn.functional as F

pytestmark = pytest.mark.gpu
DEV = "cuda"
BF = torch.bfloat16


def _bits(t):
    return t.contiguous().view(torch.int16)


def _rand(gen, *shape, scale=1.0):
    return (torch.randn(*shape, generator=gen, device=DEV) * scale).to(BF)


def _rms(x):
    return F.rms_norm(x, (x.size(-1),))


@pytest.mark.parametrize("C", [256, 768, 1536, 2048, 4096])
@pytest.mark.parametrize("lambda_dtype", [torch.float32, BF])
def test_mix_norm_is_bit_identical_to_the_eager_ops(C, lambda_dtype):
    from nanochat_b200 import ops
    gen = torch.Generator(device=DEV).manual_seed(C)
    rows = 257
    x, add, x0, xb = (_rand(gen, rows, 1, C, scale=s) for s in (1.0, 0.3, 1.0, 2.0))
    # parameters as the model holds them (fp32 by default, bf16 after model.to(bfloat16)); a 0-dim parameter is
    # converted to the activation dtype by the eager multiply, so the kernel takes the bf16-rounded value
    lam = torch.tensor([1.0826, 0.1337, 0.2], device=DEV).to(lambda_dtype)
    rl, xl, bl = lam[0], lam[1], lam[2:3]
    # lambda mix behind a residual add (a layer in the middle of the trunk)
    a = x + add
    y = rl * a + xl * x0
    got_sum, got_x, got_norm = ops.glue_mix_norm(x, add=add, x0=x0, resid_lambda=float(rl.to(BF).float()),
                                                 x0_lambda=float(xl.to(BF).float()), want_sum=True)
    assert torch.equal(_bits(got_sum), _bits(a))
    assert torch.equal(_bits(got_x), _bits(y))
    bad = (_bits(got_norm) != _bits(_rms(y))).sum().item()
    assert bad == 0, f"{bad} of {y.numel()} normalised elements differ"
    # first layer: no pending add
    y = rl * x + xl * x0
    _, got_x, got_norm = ops.glue_mix_norm(x, x0=x0, resid_lambda=float(rl.to(BF).float()), x0_lambda=float(xl.to(BF).float()))
    assert torch.equal(_bits(got_x), _bits(y)) and torch.equal(_bits(got_norm), _bits(_rms(y)))
    # attention residual + norm
    y = x + add
    _, got_x, got_norm = ops.glue_mix_norm(x, add=add)
    assert torch.equal(_bits(got_x), _bits(y)) and torch.equal(_bits(got_norm), _bits(_rms(y)))
    # end of the trunk: last residual add, backout, norm (the backout scalar is cast to bf16 first)
    y = (x + add) - bl.to(BF) * xb
    _, _, got_norm = ops.glue_mix_norm(x, add=add, x_backout=xb, backout_lambda=float(bl.to(BF).float()), want_x=False)
    assert torch.equal(_bits(got_norm), _bits(_rms(y)))


def test_norm_statistics_over_many_rows():
    """The order of the fp32 sum of squares decides the last bit of rstd; any other order shows up as a
    handful of differing bf16 outputs per million.  16.8 M elements of each trunk width, none may differ."""
    from nanochat_b200 import ops
    for C in (256, 1536, 2048):
        gen = torch.Generator(device=DEV).manual_seed(7 + C)
        x = _rand(gen, (1 << 24) // C, C, scale=3.0)
        _, _, got = ops.glue_mix_norm(x, want_x=False)
        bad = (_bits(got) != _bits(_rms(x))).sum().item()
        assert bad == 0, f"C={C}: {bad} of {x.numel()} elements differ from F.rms_norm"


def test_relu_sq_and_ve_gate_are_bit_identical_to_the_eager_ops():
    from nanochat_b200 import ops
    gen = torch.Generator(device=DEV).manual_seed(3)
    h = _rand(gen, 64, 1, 6144, scale=4.0)
    assert torch.equal(_bits(ops.glue_relu_sq(h)), _bits(F.relu(h).square()))
    B, Hkv = 64, 12
    v, ve = _rand(gen, B, 1, Hkv, 128), _rand(gen, B, 1, Hkv * 128)
    lin = _rand(gen, B, 1, Hkv, scale=3.0)
    gate = 3 * torch.sigmoid(lin)
    want = v + gate.unsqueeze(-1) * ve.view(B, 1, Hkv, 128)
    assert torch.equal(_bits(ops.glue_ve_gate(v, lin, ve)), _bits(want))


@pytest.mark.parametrize("shape", ["configs[0] binding", "d24 width, 3 layers", "two layers"])
def test_fused_trunk_gives_the_logits_and_cache_bytes_of_the_eager_trunk(shape):
    from nanochat_b200.engine import KVCache
    from nanochat_b200.gpt import GPT, GPTConfig
    from tests.test_e2e_gpu import _to_gpu
    from tests.test_host_logic import _config0_model
    if shape.startswith("configs[0]"):
        model = _to_gpu(_config0_model(True))  # fp32 parameters, bf16 activations: the reference's arrangement
    else:
        n_layer, n_embd, n_head = (3, 1536, 12) if shape.startswith("d24") else (2, 256, 2)
        cfg = GPTConfig(sequence_len=256, vocab_size=4096, n_layer=n_layer, n_head=n_head, n_kv_head=n_head, n_embd=n_embd)
        torch.manual_seed(5)
        with torch.device("meta"):
            model = GPT(cfg, compute_dtype=BF)
        model.to_empty(device=DEV)
        model.init_weights()
        s = 3 ** 0.5 * n_embd ** -0.5
        for blk in model.transformer.h:  # let attention and MLP reach the residual stream
            torch.nn.init.uniform_(blk.attn.c_proj.weight, -s, s)
            torch.nn.init.uniform_(blk.mlp.c_proj.weight, -s, s)
        torch.nn.init.normal_(model.lm_head.weight, mean=0.0, std=0.02)
        model.smear_lambda.data.fill_(0.5)
        model.to(BF)  # bf16 parameters, as the whole-model benchmark runs them
    cfg = model.config
    geo = dict(num_heads=cfg.n_kv_head, head_dim=cfg.n_embd // cfg.n_head, num_layers=cfg.n_layer)
    B, T0, steps = 5, 19, 12
    prompts = torch.randint(0, cfg.vocab_size, (B, T0), generator=torch.Generator().manual_seed(9)).to(DEV)
    runs = []
    for fused in (False, True):
        model.fused_glue = fused
        cache = KVCache(batch_size=B, seq_len=T0 + steps + 1, device=DEV, dtype=BF, **geo)
        logits = [model.forward(prompts, kv_cache=cache)[:, -1, :]]
        for _ in range(steps):
            logits.append(model.forward(logits[-1].argmax(-1, keepdim=True), kv_cache=cache)[:, -1, :])
        runs.append((torch.stack(logits), cache))
    (l_eager, c_eager), (l_fused, c_fused) = runs
    stacked = model.transformer.h[0].attn._qkv_cache
    print("stacked q/k/v projection in use:", stacked is not None and stacked[1] is not None)
    assert torch.equal(l_eager, l_fused), f"logits differ by {(l_eager - l_fused).abs().max().item()}"
    assert torch.equal(_bits(c_eager.k_cache), _bits(c_fused.k_cache)) and torch.equal(_bits(c_eager.v_cache), _bits(c_fused.v_cache))
    assert torch.equal(c_eager.cache_seqlens, c_fused.cache_seqlens)


def test_strided_qkv_slices_equal_packed_inputs():
    """q, k, v as column slices of one (B, 1, Nq + 2 Nkv) projection output: the append kernel and the value gate
    take the token stride and give the bytes they give for packed copies of the slices."""
    from nanochat_b200 import ops
    from oracle import torch_ref as E
    gen = torch.Generator(device=DEV).manual_seed(21)
    B, Hq, Hkv, T_max = 6, 8, 2, 96
    nq, nkv = Hq * 128, Hkv * 128
    qkv = torch.randn(B, 1, nq + 2 * nkv, generator=gen, device=DEV).to(BF)
    q = qkv[..., :nq].view(B, 1, Hq, 128)
    k = qkv[..., nq:nq + nkv].view(B, 1, Hkv, 128)
    v = qkv[..., nq + nkv:].view(B, 1, Hkv, 128)
    assert not q.is_contiguous() and not v.is_contiguous()
    gate = torch.randn(B, 1, Hkv, generator=gen, device=DEV).to(BF)
    ve = torch.randn(B, 1, Hkv, 128, generator=gen, device=DEV).to(BF)
    v_a = ops.glue_ve_gate(v, gate, ve)
    v_b = ops.glue_ve_gate(v.contiguous(), gate, ve)
    assert torch.equal(_bits(v_a), _bits(v_b))
    cos, sin = E.rotary_tables(T_max, 128, DEV, BF)
    lens = torch.tensor([0, 5, 17, 94, 33, 60], device=DEV, dtype=torch.int32)
    caches = []
    for strided in (True, False):
        kc = torch.zeros(B, T_max, Hkv, 128, device=DEV, dtype=BF)
        vc = torch.zeros_like(kc)
        args = (q, k, v) if strided else (q.contiguous(), k.contiguous(), v.contiguous())
        q_out = ops.append_rope_norm(*args, kc, vc, lens, cos, sin)
        caches.append((q_out, kc, vc))
    torch.cuda.synchronize()
    assert ops.read_status(DEV) == 0
    for a, b in zip(*caches):
        assert a.is_contiguous() and torch.equal(_bits(a), _bits(b))
