"""Benchmark of the KV-cache decode hot path (KV append + decode attention) on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--no-extras]

Headline workload (benchmark configuration 1, "configs[1]"): B=32 rows, 12 q heads, 12 kv heads, head_dim 128, cache
capacity 2048, cache_seqlens uniform in [1, 2047] (torch CPU generator, seed 2), caches and new
q/k/v ~ N(0,1) bf16, one new token per row, full causal.  One "step" is one pass of the hot path
over that batch: the fused RoPE + QK-norm + append launch followed by the split-KV decode
attention launch.  At N > 1 every rank runs the same workload on its own rows (sequences are
independent: no collective on the data path), so the headline scales weakly.

Timing: CUDA events on the launching stream, W warm-up steps, then a region of exactly K steps
bracketed by a barrier + device synchronisation on both sides, max over ranks.  The region is
repeated R >= 50 times (about a second of load, so that clock samples exist) and the MEDIAN region is
reported with its p10/p90, which makes a 20-step run agree with a 2000-step run.  Each step reads
a different one of NSETS cache sets (NSETS x 403 MB, far larger than the 126 MB L2) so KV bytes
come from HBM.
  value     steps replayed from a CUDA graph, inputs resident in HBM
  roofline  one nckv_decode_attn call alone (streaming kernel + its small merge kernel), launched
            K times per region through the C ABI; algorithmic bytes of the attention alone
  e2e       the public Python call with HOST inputs: H2D of q/k/v, both launches, D2H of the output
  cpu_baseline / --impl reference   the reference's CPU path (fp32, SDPA row by row): the staged
            reference modules (oracle/_ref) when present, else the torch port under oracle/
  gpu_reference   the reference's own GPU path (bf16 eager RoPE/norm ops, slice-assign append, SDPA)
            on the same device and data, beside the kernels that replace it

Two more legs ride in the same JSON line (skipped with --no-extras):
  long_context  benchmark configuration 4 ("configs[4]") (B=8, 16/4 heads, T_max=65536, lengths U[32768,65536]) with the keys
            split block-cyclically over the N ranks and the log-sum-exp exchange over NVLink peer memory
            (and over NCCL), checked in-run against the unsplit single-GPU result on the same data
  d24_sharded   benchmark configuration 2 ("configs[2]") (d24 model, 64 sequences, 512-token prompts, greedy decode) with the
            fixed batch sharded by sequence over the N ranks (strong scaling, weights replicated)
"""
import argparse
import json
import math
import os
import statistics
import subprocess
import sys
import threading
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

B, HQ, HKV, D, T_MAX = 32, 12, 12, 128, 2048
NSETS = 4
# dram__bytes_read.sum + dram__bytes_write.sum of one decode_attn_kernel launch on this workload
# (one `ncu --set full` capture of this file's default command, summarised beside the other kernel profiles)
TRAFFIC_BYTES_PER_LAUNCH = 202.63e6
TRAFFIC_CAPTURE = "ncu --set full capture of decode_attn_kernel<0,1,0> on this workload, 2026-11-25 (198.64 MB read + 4.00 MB written)"
METRIC = "decode tokens/s (KV append + decode attention, B=32 x 12 heads x 128, ragged cache)"
WORKLOAD = "configs[1]: op-level KV append + decode attention, B=32, 12q/12kv heads, D=128, T_max=2048, ragged seqlens seed 2"


def seqlens_cpu():
    return torch.randint(1, 2048, (B,), dtype=torch.int32, generator=torch.Generator().manual_seed(2))


def algorithmic_bytes(seqlens):
    """Bytes of one step (bf16).  Returns (K and V rows read, the attention call's other bytes: q in,
    out, cache_seqlens; the append's bytes: q/k/v read, q and the new k/v rows written, one cos and one
    sin row per batch row)."""
    n_keys = int((seqlens.long() + 1).sum())
    kv = 4 * HKV * D * n_keys
    attn_other = 2 * B * HQ * D * 2 + 4 * B
    append = 2 * B * (HQ + 2 * HKV) * D * 2 + B * D * 2
    return kv, attn_other, append


def config_dict(world):
    """Identical for both arms, so their lines compare like for like."""
    return {"workload": WORKLOAD, "rows_per_gpu": B, "rows_total": B * world,
            "l2": f"{NSETS} cache sets rotated, {NSETS * 2 * B * T_MAX * HKV * D * 2 / 1e6:.0f} MB > L2",
            "parallelism": f"{world} x independent sequences"}


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except Exception:
        return 6650.0, "fallback"


class ClockSampler:
    """nvidia-smi clock/throttle samples taken while the timed region runs."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index):
        self.gpu = gpu_index
        self.lines = []
        self.proc = None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-lms", "50", "-i", str(self.gpu)], stdout=subprocess.PIPE,
                                         stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._pump, daemon=True).start()
        except Exception:
            self.proc = None

    def _pump(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except Exception:
                pass
        sm, mx, reasons = [], [], set()
        for line in self.lines:
            f = [x.strip() for x in line.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1]))
                mx.append(float(f[2]))
            except ValueError:
                continue
            for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        return {"sm_mhz": statistics.median(sm), "sm_max_mhz": max(mx), "reasons": sorted(reasons), "samples": len(sm)}


def dist_setup(n_gpus):
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world > 1:
        import torch.distributed as dist
        torch.cuda.set_device(local)
        dist.init_process_group(backend="nccl", device_id=torch.device("cuda", local))
    return rank, world, local


def barrier(world):
    if world > 1:
        import torch.distributed as dist
        dist.barrier()
    torch.cuda.synchronize()


def max_over_ranks(x, world, device):
    if world == 1:
        return x
    import torch.distributed as dist
    t = torch.tensor(x if isinstance(x, (list, tuple)) else [x], dtype=torch.float64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return t.tolist() if isinstance(x, (list, tuple)) else float(t.item())


def timed_regions(region, repeats, world, dev):
    """Run ``region()`` (which enqueues one K-step region on the current stream) ``repeats`` times,
    each bracketed by barrier + device synchronisation and CUDA events on the launching stream.
    Returns the region times in ms, each the max over ranks."""
    events = []
    for _ in range(repeats):
        barrier(world)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        region()
        e1.record()
        events.append((e0, e1))
    barrier(world)
    return max_over_ranks([a.elapsed_time(b) for a, b in events], world, dev)


def spread(region_ms, per):
    """median / p10 / p90 of per-unit times (ms) over the repeated regions."""
    v = sorted(x / per for x in region_ms)
    pick = lambda f: v[min(len(v) - 1, max(0, int(round(f * (len(v) - 1)))))]
    return statistics.median(v), pick(0.1), pick(0.9)


REGIONS_OVERRIDE = None  # --regions: a fixed number of regions (profiling runs want few launches)


def repeats_for(region_s, target_s=1.0, lo=50, hi=3000):
    if REGIONS_OVERRIDE:
        return REGIONS_OVERRIDE
    return int(min(hi, max(lo, math.ceil(target_s / max(region_s, 1e-6)))))


# ------------------------------------------------------------------------------------------------
# CPU baseline: the reference's CPU path, fp32, all host threads
# ------------------------------------------------------------------------------------------------
def cpu_reference_run(steps, warmup, budget_s=25.0, rows=B):
    """configs[1] on the host cores, fp32.  With the staged reference (oracle/_ref) the functions timed
    are the reference's own apply_rotary_emb / norm / flash_attn_with_kvcache, called row by row (its
    SDPA fallback takes one length for the whole batch); otherwise the torch port of the same ops."""
    from oracle import ref_loader
    try:
        usable = len(os.sched_getaffinity(0))  # torchrun exports OMP_NUM_THREADS=1 to its ranks
    except AttributeError:
        usable = os.cpu_count() or 1
    torch.set_num_threads(max(usable, 1))
    threads = torch.get_num_threads()
    gen = torch.Generator().manual_seed(2)
    reps = max(1, rows // B)
    seqlens = seqlens_cpu().repeat(reps)
    k_cache = torch.randn(B, T_MAX, HKV, D, generator=gen).repeat(reps, 1, 1, 1)
    v_cache = torch.randn(B, T_MAX, HKV, D, generator=gen).repeat(reps, 1, 1, 1)
    q = torch.randn(B, 1, HQ, D, generator=gen).repeat(reps, 1, 1, 1)
    k = torch.randn(B, 1, HKV, D, generator=gen).repeat(reps, 1, 1, 1)
    v = torch.randn(B, 1, HKV, D, generator=gen).repeat(reps, 1, 1, 1)
    n_rows = B * reps
    if ref_loader.available():
        ref_loader.load("float32")
        import nanochat.gpt as ref_gpt
        from nanochat.flash_attention import flash_attn
        saved = ref_gpt.COMPUTE_DTYPE
        ref_gpt.COMPUTE_DTYPE = torch.float32
        cos, sin = ref_gpt.GPT._precompute_rotary_embeddings(None, T_MAX, D, device="cpu")
        ref_gpt.COMPUTE_DTYPE = saved
        kind = "reference"
        how = "the staged reference's apply_rotary_emb / norm / flash_attn_with_kvcache (SDPA fallback), one call per row"

        def step():
            outs = []
            for b in range(n_rows):
                L = int(seqlens[b])
                c, s_ = cos[:, L:L + 1], sin[:, L:L + 1]
                qb = ref_gpt.norm(ref_gpt.apply_rotary_emb(q[b:b + 1], c, s_)) * 1.2
                kb = ref_gpt.norm(ref_gpt.apply_rotary_emb(k[b:b + 1], c, s_)) * 1.2
                outs.append(flash_attn.flash_attn_with_kvcache(qb, k_cache[b:b + 1], v_cache[b:b + 1], k=kb, v=v[b:b + 1],
                                                               cache_seqlens=seqlens[b:b + 1], causal=True, window_size=(-1, 0)))
            return outs
    else:
        from oracle import torch_ref as R
        cos, sin = R.rotary_tables(T_MAX, D, "cpu", torch.float32)
        kind = "port"
        how = "torch port of the reference ops, SDPA row by row as the reference's CPU fallback does"

        def step():
            q2 = R.rope_norm_scale_rows(q, cos, sin, seqlens)
            k2 = R.rope_norm_scale_rows(k, cos, sin, seqlens)
            return R.kvcache_attention(q2, k_cache, v_cache, k2, v, seqlens, -1)

    with torch.inference_mode():
        for _ in range(max(warmup, 1)):
            step()
        t0 = time.perf_counter()
        done = 0
        while done < steps and (time.perf_counter() - t0) < budget_s:
            step()
            done += 1
        dt = time.perf_counter() - t0
    return {"value": n_rows * done / dt, "unit": "tokens/s", "cores": threads, "kind": kind,
            "sample": f"{done} full configs[1] steps of {n_rows} rows (fp32; {how}), {dt:.1f} s",
            "ms_per_step": 1e3 * dt / done}, done, dt


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    world = max(int(os.environ.get("WORLD_SIZE", "1")), 1)
    # the job of the other arm at this N is N x 32 rows: time the same number of rows on the host cores
    cb, done, dt = cpu_reference_run(args.steps, args.warmup, rows=B * world)
    line = {"impl": "reference", "metric": METRIC, "value": cb["value"], "unit": "tokens/s", "n_gpus": args.gpus,
            "steps": done, "warmup": args.warmup, "ms_per_step": cb["ms_per_step"], "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": config_dict(world), "device": "host CPU",
            "cpu_baseline": {k: cb[k] for k in ("value", "unit", "cores", "kind", "sample")},
            "e2e": {"value": cb["value"], "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0}
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------------------------------------------
# the reference's own GPU path on the same device (bf16 eager ops + SDPA), configs[1]
# ------------------------------------------------------------------------------------------------
def gpu_reference_leg(dev, sets, q, k, v, seqlens, cos, sin, steps):
    """What a B200 runs today without this library (flash_attention.py:155-177 and gpt.py:99-102 in bf16):
    row by row at the ragged lengths (the fallback takes row 0's length for the whole batch, so ragged rows
    need one call each) and batched with every row at the mean length."""
    from oracle import ref_loader
    lens_h = seqlens.cpu()
    mean_len = int(lens_h.float().mean().item())
    uniform = torch.full_like(seqlens, mean_len)
    if ref_loader.available():
        ref_loader.load("bfloat16")
        import nanochat.gpt as ref_gpt
        from nanochat.flash_attention import flash_attn
        source = "oracle/_ref (the reference's own functions)"

        def rope_norm(x, L):
            return ref_gpt.norm(ref_gpt.apply_rotary_emb(x, cos[:, L:L + x.size(1)], sin[:, L:L + x.size(1)])) * 1.2

        attend = lambda q_, kc, vc, k_, v_, lens_: flash_attn.flash_attn_with_kvcache(
            q_, kc, vc, k=k_, v=v_, cache_seqlens=lens_, causal=True, window_size=(-1, 0))
    else:
        from oracle import torch_ref as R
        source = "oracle/torch_ref.py (port of the same op sequence)"
        rope_norm = lambda x, L: R.rope_norm_scale(x, cos[:, L:L + x.size(1)], sin[:, L:L + x.size(1)])
        attend = lambda q_, kc, vc, k_, v_, lens_: R.kvcache_attention_row(q_, kc, vc, k_, v_, int(lens_[0]), -1)

    def ragged(i):
        kc, vc = sets[i % NSETS]
        for b in range(B):
            L = int(lens_h[b])
            attend(rope_norm(q[b:b + 1], L), kc[b:b + 1], vc[b:b + 1], rope_norm(k[b:b + 1], L), v[b:b + 1], seqlens[b:b + 1])

    def batched(i):
        kc, vc = sets[i % NSETS]
        attend(rope_norm(q, mean_len), kc, vc, rope_norm(k, mean_len), v, uniform)

    out = {"source": source, "dtype": "bf16"}
    with torch.inference_mode():
        for name, fn, n in (("ragged_row_by_row", ragged, max(3, min(steps, 20))), ("batched_uniform_mean_length", batched, max(5, min(steps, 100)))):
            for i in range(3):
                fn(i)
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for i in range(n):
                fn(i)
            e1.record()
            torch.cuda.synchronize()
            ms = e0.elapsed_time(e1) / n
            out[name] = {"ms_per_step": ms, "tokens_per_s": B / (ms * 1e-3), "steps": n}
    out["batched_uniform_mean_length"]["length"] = mean_len
    return out


# ------------------------------------------------------------------------------------------------
# configs[4]: long-context decode with the keys split over the ranks
# ------------------------------------------------------------------------------------------------
def long_context_leg(rank, world, dev, steps):
    from nanochat_b200 import ops
    from nanochat_b200.dist import KVSplitAttention
    from nanochat_b200.gpt import precompute_rotary_embeddings
    peak, peak_kind = peaks()
    Bc, Hq, Hkv, T, block, nsets = 8, 16, 4, 65536, 1024, 2
    lens = torch.randint(32768, 65536, (Bc,), dtype=torch.int32, generator=torch.Generator().manual_seed(4))
    lens_d = lens.to(dev)
    gen = torch.Generator(device=dev).manual_seed(4)  # the same seed on every rank: identical data everywhere
    bf = torch.bfloat16
    full_k = torch.randn(Bc, T, Hkv, D, generator=gen, device=dev, dtype=torch.float32).to(bf)
    full_v = torch.randn(Bc, T, Hkv, D, generator=gen, device=dev, dtype=torch.float32).to(bf)
    q = torch.randn(Bc, 1, Hq, D, generator=gen, device=dev).to(bf)
    k = torch.randn(Bc, 1, Hkv, D, generator=gen, device=dev).to(bf)
    v = torch.randn(Bc, 1, Hkv, D, generator=gen, device=dev).to(bf)
    cos, sin = precompute_rotary_embeddings(T, D, device=dev)
    # this rank's block-cyclic part of the keys, taken before the new token is appended anywhere
    pos = torch.arange(T, device=dev)
    mine = pos[(pos // block) % world == rank]
    sets = [(full_k[:, mine].contiguous(), full_v[:, mine].contiguous())]
    for _ in range(nsets - 1):
        sets.append((torch.randn(sets[0][0].shape, generator=gen, device=dev, dtype=torch.float32).to(bf),
                     torch.randn(sets[0][0].shape, generator=gen, device=dev, dtype=torch.float32).to(bf)))
    # unsplit result on this GPU from the same data: fused append into the full cache, attention over all keys
    q2 = ops.append_rope_norm(q, k, v, full_k, full_v, lens_d, cos, sin)
    want = ops.decode_attention(q2[:, 0], full_k, full_v, lens_d, seqlen_offset=1, window_left=-1).float()
    unsplit_s = _time_cuda(lambda i: ops.decode_attention(q2[:, 0], full_k, full_v, lens_d, 1, -1), max(5, min(steps, 20)))
    torch.cuda.synchronize()
    del full_k, full_v
    nbytes = 4 * Hkv * D * int((lens.long() + 1).sum()) + 4 * Bc * Hq * D + 4 * Bc
    out = {"workload": "configs[4]: B=8, 16q/4kv heads, D=128, T_max=65536, lengths U[32768,65536] seed 4, append + attention",
           "layout": f"block-cyclic, {block} keys per block", "keys_per_rank": int(mine.numel()), "scaling": "strong",
           "algorithmic_bytes": nbytes, "unsplit_single_gpu_us_per_call": unsplit_s * 1e6,
           "exchange_bytes_per_rank": Bc * Hq * (D + 1) * 4, "peak": peak, "peak_kind": f"of {peak_kind}"}
    side = torch.cuda.Stream(dev)
    for exch in (("p2p", "nccl") if world > 1 else ("nccl",)):
        key = exch if world > 1 else "single"
        try:
            att = KVSplitAttention(T, block=block, exchange=exch)
            got = att.append_and_attend(q, k, v, sets[0][0], sets[0][1], lens_d, cos, sin).float()
            torch.cuda.synchronize()
            err = ((got - want).abs().max() / want.abs().max()).item()
            with torch.cuda.stream(side):
                for i in range(2 * nsets):
                    att.append_and_attend(q, k, v, sets[i % nsets][0], sets[i % nsets][1], lens_d, cos, sin)
                side.synchronize()
                barrier(world)
                graph = torch.cuda.CUDAGraph()
                graph_steps = nsets * min(8, max(2, (steps + nsets - 1) // nsets))
                with torch.cuda.graph(graph, stream=side):
                    for i in range(graph_steps):
                        att.append_and_attend(q, k, v, sets[i % nsets][0], sets[i % nsets][1], lens_d, cos, sin)
            torch.cuda.synchronize()
            replays = max(1, (max(steps, 4) + graph_steps - 1) // graph_steps)
            for _ in range(3):
                graph.replay()
            region = lambda: [graph.replay() for _ in range(replays)]
            pilot = timed_regions(region, 3, world, dev)
            reps = repeats_for(statistics.median(pilot) * 1e-3, target_s=0.3, lo=20, hi=1000)
            reps = int(max_over_ranks(float(reps), world, dev))
            ms, p10, p90 = spread(timed_regions(region, reps, world, dev), replays * graph_steps)
            sec = ms * 1e-3
            out[key] = {"us_per_call": sec * 1e6, "us_p10": p10 * 1e3, "us_p90": p90 * 1e3, "repeats": reps,
                        "steps_per_region": replays * graph_steps, "kv_read_gbs": nbytes / sec / 1e9,
                        "frac_of_n_x_peak": nbytes / sec / 1e9 / (peak * world), "parity_max_rel_err": err,
                        "launch": f"CUDA graph; kernels per step: append, attention, merge{'+push' if exch == 'p2p' else ''}, "
                                  f"{'wait+combine' if exch == 'p2p' else ('all-gather (NCCL), combine' if world > 1 else 'combine')}"}
        except Exception as e:  # one exchange failing must not take the headline down with it
            out[key] = {"error": f"{type(e).__name__}: {e}"[:300]}
            torch.cuda.synchronize()
    best = out.get("p2p" if world > 1 else "single", {})
    for fld in ("us_per_call", "frac_of_n_x_peak", "parity_max_rel_err", "kv_read_gbs"):
        if fld in best:
            out[fld] = best[fld]
    out["device_status"] = ops.read_status(dev)
    return out


# ------------------------------------------------------------------------------------------------
# configs[2]: the d24 model, a fixed batch of 64 sequences sharded over the ranks
# ------------------------------------------------------------------------------------------------
def build_d24(dev, n_layer=24):
    from nanochat_b200.gpt import GPT, GPTConfig
    cfg = GPTConfig(sequence_len=2048, vocab_size=32768, n_layer=n_layer, n_head=12, n_kv_head=12, n_embd=1536)
    torch.manual_seed(3)
    with torch.device("meta"):
        model = GPT(cfg, compute_dtype=torch.bfloat16)
    model.to_empty(device=dev)
    model.init_weights()
    model.to(torch.bfloat16)
    model.window_sizes = [(1024, 0) if (i % 4) != 3 else (2048, 0) for i in range(n_layer)]
    model.window_sizes[-1] = (2048, 0)
    return model


def d24_sharded_leg(rank, world, dev, steps, small=False):
    from nanochat_b200 import ops
    from nanochat_b200.dist import shard_rows
    from nanochat_b200.engine import GraphedDecodeStep, KVCache
    peak, peak_kind = peaks()
    n_layer, rows_total, T0 = (4, 16, 64) if small else (24, 64, 512)
    n_new = 16 if small else 64
    model = build_d24(dev, n_layer)
    lo, hi = shard_rows(rows_total, rank, world)
    rows = hi - lo
    prompts = torch.randint(0, 32768, (rows_total, T0), generator=torch.Generator().manual_seed(3))[lo:hi].to(dev)
    cache = KVCache(batch_size=rows, num_heads=12, seq_len=T0 + n_new + 8, head_dim=128, num_layers=n_layer, device=dev,
                    dtype=torch.bfloat16)
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    ids = model.forward(prompts, kv_cache=cache)[:, -1, :].argmax(-1, keepdim=True)
    torch.cuda.synchronize()
    prefill_s = time.perf_counter() - t0
    graphed = GraphedDecodeStep(model, cache, ids)
    for _ in range(3):
        ids = graphed.step(ids).argmax(-1, keepdim=True)
    barrier(world)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(n_new):
        ids = graphed.step(ids).argmax(-1, keepdim=True)
    e1.record()
    barrier(world)
    ms = max_over_ranks(e0.elapsed_time(e1), world, dev) / n_new
    ctx = int(cache.cache_seqlens[0].item())
    kv_step = sum(4 * 12 * D * rows * min(ctx, w[0] + 1) for w in model.window_sizes)
    w_bytes = 2 * sum(p_.numel() for n_, p_ in model.named_parameters() if "wte" not in n_ and "value_embeds" not in n_)
    status = ops.read_status(dev)
    return {"workload": f"configs[2]: d{n_layer} (1536 wide, 12 heads), {rows_total} sequences, {T0}-token prompts, greedy, bf16 random init seed 3",
            "scaling": "strong", "rows_per_gpu": rows, "decode_steps": n_new, "context_at_end": ctx,
            "tokens_per_s": rows_total / (ms * 1e-3), "ms_per_step": ms, "prefill_s_rank0": prefill_s,
            "per_gpu_byte_floor_ms": (kv_step + w_bytes) / (peak * 1e9) * 1e3, "kv_bytes_per_step_per_gpu": kv_step,
            "weight_bytes_per_gpu": w_bytes, "peak": peak, "peak_kind": f"of {peak_kind}",
            "launch": "whole decode step replayed from a CUDA graph; weights replicated, rows sharded, no collective",
            "device_status": status}


# ------------------------------------------------------------------------------------------------
# our arm
# ------------------------------------------------------------------------------------------------
def run_ours(args):
    rank, world, local = dist_setup(args.gpus)
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (the hot path has no CPU implementation)")
    dev = torch.device("cuda", local)
    torch.cuda.set_device(dev)
    from nanochat_b200 import _lib, ops
    from nanochat_b200.gpt import precompute_rotary_embeddings

    seqlens_h = seqlens_cpu()
    kv_bytes, attn_other, append_bytes = algorithmic_bytes(seqlens_h)
    seqlens = seqlens_h.to(dev)
    gen = torch.Generator(device=dev).manual_seed(2 + rank)
    sets = []
    for _ in range(NSETS):
        kc = torch.randn(B, T_MAX, HKV, D, generator=gen, device=dev, dtype=torch.float32).to(torch.bfloat16)
        vc = torch.randn(B, T_MAX, HKV, D, generator=gen, device=dev, dtype=torch.float32).to(torch.bfloat16)
        sets.append((kc, vc))
    q = torch.randn(B, 1, HQ, D, generator=gen, device=dev).to(torch.bfloat16)
    k = torch.randn(B, 1, HKV, D, generator=gen, device=dev).to(torch.bfloat16)
    v = torch.randn(B, 1, HKV, D, generator=gen, device=dev).to(torch.bfloat16)
    cos, sin = precompute_rotary_embeddings(T_MAX, D, device=dev)
    K, W = args.steps, args.warmup

    def step(i):
        kc, vc = sets[i % NSETS]
        q2 = ops.append_rope_norm(q, k, v, kc, vc, seqlens, cos, sin)
        return ops.decode_attention(q2[:, 0], kc, vc, seqlens, seqlen_offset=1, window_left=-1)

    # ---- value: CUDA-graph replay of NSETS consecutive steps ------------------------------------
    for i in range(max(W, 3)):
        step(i)
    torch.cuda.synchronize()
    side = torch.cuda.Stream(dev)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.stream(side):
        for i in range(NSETS):
            step(i)  # allocate workspace for the side stream outside of capture
        side.synchronize()
        # one graph holds up to 64 consecutive steps (a multiple of the cache-set rotation): consecutive
        # launches inside a graph hand over like consecutive launches in a stream, separate replays do not
        graph_steps = NSETS * min(16, (K + NSETS - 1) // NSETS)
        with torch.cuda.graph(graph, stream=side):
            for i in range(graph_steps):
                step(i)
    replays = (K + graph_steps - 1) // graph_steps
    k_eff = replays * graph_steps
    for _ in range(max(1, (max(W, 3) + graph_steps - 1) // graph_steps)):
        graph.replay()

    def value_region():
        for _ in range(replays):
            graph.replay()

    pilot = timed_regions(value_region, 3, world, dev)
    r_value = int(max_over_ranks(float(repeats_for(statistics.median(pilot) * 1e-3)), world, dev))
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
        time.sleep(0.3)
    value_ms = timed_regions(value_region, r_value, world, dev)
    ms_step, ms_p10, ms_p90 = spread(value_ms, k_eff)
    value = world * B / (ms_step * 1e-3)

    # ---- roofline: the decode-attention call alone, through the C ABI ------------------------------
    q2 = ops.append_rope_norm(q, k, v, sets[0][0], sets[0][1], seqlens, cos, sin)[:, 0].contiguous()
    out = torch.empty_like(q2)

    def attn_only(i, raw_stream):
        kc, vc = sets[i % NSETS]
        _lib.call("nckv_decode_attn", q2.data_ptr(), kc.data_ptr(), vc.data_ptr(), seqlens.data_ptr(), out.data_ptr(),
                  None, None, B, HQ, HKV, D, T_MAX, kc.stride(0), kc.stride(1), 1, -1, 0, 0, ws.data_ptr(), ws.numel(),
                  raw_stream)

    # launched like the steps above: consecutive calls captured once, replayed to make a K-call region
    attn_graph = torch.cuda.CUDAGraph()
    with torch.cuda.stream(side):
        ws = ops.workspace(dev, B, HQ, HKV)  # the capture stream's own workspace
        for i in range(NSETS):
            attn_only(i, side.cuda_stream)
        side.synchronize()
        with torch.cuda.graph(attn_graph, stream=side):
            for i in range(graph_steps):
                attn_only(i, side.cuda_stream)

    def attn_region():
        for _ in range(replays):
            attn_graph.replay()

    for _ in range(3):
        attn_graph.replay()
    pilot = timed_regions(attn_region, 3, 1, dev)
    r_attn = repeats_for(statistics.median(pilot) * 1e-3, target_s=0.7)
    attn_ms, attn_p10, attn_p90 = spread(timed_regions(attn_region, r_attn, 1, dev), k_eff)
    status = ops.read_status(dev)
    with torch.cuda.stream(side):  # the graphs ran on the side stream, with that stream's workspace
        status |= ops.read_status(dev)
    clocks = sampler.stop() if rank == 0 else None

    # ---- e2e: public call, host buffers ------------------------------------------------------------
    # host side of a step: q, k, v of the new token in one pinned block (H2D), the output pinned (D2H);
    # one public call per step (ops.HostDecodeStep.run -> nckv_decode_step_host), which synchronises
    def time_host_steps(transfer):
        host_step = ops.HostDecodeStep(B, HQ, HKV, cos, sin, dev, transfer=transfer)
        host_step.q.copy_(q[:, 0].cpu())
        host_step.k.copy_(k[:, 0].cpu())
        host_step.v.copy_(v[:, 0].cpu())

        def region():
            for i in range(K):
                host_step.run(sets[i % NSETS][0], sets[i % NSETS][1], seqlens, -1)

        for i in range(max(W, 3)):
            host_step.run(sets[i % NSETS][0], sets[i % NSETS][1], seqlens, -1)
        reps = REGIONS_OVERRIDE or int(min(300, max(5, math.ceil(0.5 / (K * 80e-6)))))
        t0 = time.perf_counter()
        med, p10, p90 = spread(timed_regions(region, reps, world, dev), K)
        wall_ms = 1e3 * (time.perf_counter() - t0) / (reps * K)
        return med, p10, p90, wall_ms, reps, host_step.host_in.numel() * 2, host_step.out.numel() * 2

    # headline: explicit H2D / D2H copies around the kernels; beside it the mapped variant (the kernels
    # read the pinned inputs and write the pinned output over PCIe themselves: same bytes, no copy ops)
    e2e_ms, e2e_p10, e2e_p90, e2e_wall_ms, r_e2e, h2d, d2h = time_host_steps("copy")
    e2e_value = world * B / (e2e_ms * 1e-3)
    mapped_ms = time_host_steps("mapped")[0]

    # ---- the other legs ----------------------------------------------------------------------------
    extras = {}
    if not args.no_extras:
        if world == 1 and rank == 0:
            try:
                extras["gpu_reference"] = gpu_reference_leg(dev, sets, q, k, v, seqlens, cos, sin, K)
            except Exception as e:
                extras["gpu_reference"] = {"error": f"{type(e).__name__}: {e}"[:300]}
        del sets
        torch.cuda.empty_cache()
        for name, leg in (("long_context", long_context_leg), ("d24_sharded", d24_sharded_leg)):
            try:
                extras[name] = leg(rank, world, dev, K)
            except Exception as e:
                extras[name] = {"error": f"{type(e).__name__}: {e}"[:300]}
                torch.cuda.synchronize()
            torch.cuda.empty_cache()

    if rank == 0:
        peak, peak_kind = peaks()
        attn_bytes = kv_bytes + attn_other
        achieved = attn_bytes / (attn_ms * 1e-3) / 1e9
        cb = None
        if world == 1 and not args.no_cpu_baseline:
            cb_full, _, _ = cpu_reference_run(steps=100000, warmup=2, budget_s=12.0)
            cb = {k_: cb_full[k_] for k_ in ("value", "unit", "cores", "kind", "sample")}
        line = {
            "metric": METRIC, "value": value, "unit": "tokens/s", "n_gpus": world, "steps": k_eff, "warmup": W,
            "ms_per_step": ms_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "bf16", "data": "synthetic", "config": config_dict(world),
            "launch": f"CUDA graph replay of append + attention (3 kernels per step, {graph_steps} steps per graph)",
            "timing": {"regions": r_value, "steps_per_region": k_eff, "statistic": "median region, max over ranks per region",
                       "ms_per_step_p10": ms_p10, "ms_per_step_p90": ms_p90},
            "kv_read_gbs": world * kv_bytes / (ms_step * 1e-3) / 1e9,
            "step_frac_of_8000_nominal": (kv_bytes + attn_other + append_bytes) / (ms_step * 1e-3) / 1e9 / 8000.0,
            "roofline": {"bound": "hbm", "kernel": "decode_attn_kernel + decode_merge_kernel (one nckv_decode_attn call)", "achieved": achieved, "peak": peak,
                         "peak_kind": f"of {peak_kind}", "unit": "GB/s", "frac": achieved / peak,
                         "frac_of_8000_nominal": achieved / 8000.0, "us_per_launch": attn_ms * 1e3,
                         "us_per_launch_p10": attn_p10 * 1e3, "us_per_launch_p90": attn_p90 * 1e3, "regions": r_attn,
                         "launches_per_region": k_eff, "launch": "CUDA graph replay of the attention call", "algorithmic_bytes": attn_bytes,
                         "traffic": TRAFFIC_BYTES_PER_LAUNCH, "traffic_source": TRAFFIC_CAPTURE},
            "e2e": {"value": e2e_value, "unit": "tokens/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                    "ms_per_step": e2e_ms, "ms_per_step_p10": e2e_p10, "ms_per_step_p90": e2e_p90, "regions": r_e2e,
                    "wall_ms_per_step": e2e_wall_ms,
                    "mapped_host_memory": {"value": world * B / (mapped_ms * 1e-3), "ms_per_step": mapped_ms}},
            "gpu_launches": 3 * k_eff, "device_status": status, "clocks": clocks,
        }
        line.update(extras)
        if cb is not None:
            line["cpu_baseline"] = cb
        print(json.dumps(line), flush=True)
    if world > 1:
        import torch.distributed as dist
        dist.destroy_process_group()


# ------------------------------------------------------------------------------------------------
# secondary cases (one JSON line each): the other kernels and the other benchmark configurations, op level
# ------------------------------------------------------------------------------------------------
def _time_cuda(fn, iters, warmup=3):
    for i in range(warmup):
        fn(i)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(iters):
        fn(i)
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / iters * 1e-3  # seconds per call


def run_case_kv_split(args):
    """configs[4] with the keys split across the ranks (under torchrun), alone: the long_context leg."""
    rank, world, local = dist_setup(args.gpus)
    dev = torch.device("cuda", local)
    torch.cuda.set_device(dev)
    res = long_context_leg(rank, world, dev, args.steps)
    if rank == 0:
        res.update(case="decode_long", n_gpus=world, data="synthetic", dtype="bf16")
        print(json.dumps(res), flush=True)
    if world > 1:
        import torch.distributed as dist
        dist.destroy_process_group()


def run_case(args):
    if args.case == "decode_long" and int(os.environ.get("WORLD_SIZE", "1")) > 1:
        return run_case_kv_split(args)
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    from nanochat_b200 import ops
    from nanochat_b200.gpt import precompute_rotary_embeddings
    peak, peak_kind = peaks()
    gen = torch.Generator(device=dev).manual_seed(4)
    bf = torch.bfloat16
    rnd = lambda *shape: torch.randn(*shape, generator=gen, device=dev, dtype=torch.float32).to(bf)
    iters = max(args.steps, 3)
    out = {"case": args.case, "n_gpus": 1, "steps": iters, "data": "synthetic", "dtype": "bf16"}
    if args.case in ("decode_long", "decode_gqa", "decode_gqa_window", "decode_d24"):
        if args.case == "decode_long":      # configs[4]: long-context op-level decode
            Bc, Hq, Hkv, T, w, nsets = 8, 16, 4, 65536, -1, 2
            lens = torch.randint(32768, 65536, (Bc,), dtype=torch.int32, generator=torch.Generator().manual_seed(4))
        elif args.case == "decode_d24":     # one layer of configs[2] at mid generation
            Bc, Hq, Hkv, T, w, nsets = 64, 12, 12, 1024, -1, 2
            lens = torch.full((Bc,), 767, dtype=torch.int32)
        else:                               # one layer of configs[3]: GQA 16/4, ragged, capacity 4096
            Bc, Hq, Hkv, T, nsets = 256, 16, 4, 4096, 1
            w = 2048 if args.case.endswith("window") else -1
            lens = torch.randint(128, 4095, (Bc,), dtype=torch.int32, generator=torch.Generator().manual_seed(5))
        sets = [(rnd(Bc, T, Hkv, D), rnd(Bc, T, Hkv, D)) for _ in range(nsets)]
        q = rnd(Bc, Hq, D)
        lens_d = lens.to(dev)
        sec = _time_cuda(lambda i: ops.decode_attention(q, sets[i % nsets][0], sets[i % nsets][1], lens_d, 1, w), iters)
        n = lens.long() + 1
        if w >= 0:
            n = n.clamp(max=w + 1)
        nbytes = 4 * Hkv * D * int(n.sum()) + 4 * Bc * Hq * D + 4 * Bc
        out.update(metric="decode attention KV-read GB/s", value=nbytes / sec / 1e9, unit="GB/s", us_per_call=sec * 1e6,
                   algorithmic_bytes=nbytes, frac=nbytes / sec / 1e9 / peak, peak=peak, peak_kind=f"of {peak_kind}",
                   config={"B": Bc, "Hq": Hq, "Hkv": Hkv, "T_max": T, "window_left": w})
    elif args.case in ("engine_d24", "engine_d24_small"):
        # configs[2]: nanochat d24 (24 x 1536, 12 heads), random-init bf16, batch 64, prompts of 512 ids,
        # greedy decode; the whole forward (torch GEMMs + libnckv attention) replayed from a CUDA graph
        from nanochat_b200.engine import GraphedDecodeStep, KVCache
        from nanochat_b200.gpt import GPT, GPTConfig
        small = args.case.endswith("small")
        n_layer, Bc, T0 = (4, 8, 64) if small else (24, 64, 512)
        cfg = GPTConfig(sequence_len=2048, vocab_size=32768, n_layer=n_layer, n_head=12, n_kv_head=12, n_embd=1536)
        torch.manual_seed(3)
        with torch.device("meta"):
            model = GPT(cfg, compute_dtype=bf)
        model.to_empty(device=dev)
        model.init_weights()
        model.to(bf)
        model.window_sizes = [(1024, 0) if (i % 4) != 3 else (2048, 0) for i in range(n_layer)]
        model.window_sizes[-1] = (2048, 0)
        n_new = max(args.steps, 8)
        cache = KVCache(batch_size=Bc, num_heads=12, seq_len=T0 + n_new + 8, head_dim=128, num_layers=n_layer,
                        device=dev, dtype=bf)
        prompts = torch.randint(0, 32768, (Bc, T0), generator=torch.Generator().manual_seed(3)).to(dev)
        t0 = time.perf_counter()
        logits = model.forward(prompts, kv_cache=cache)[:, -1, :]
        torch.cuda.synchronize()
        prefill_s = time.perf_counter() - t0
        ids = logits.argmax(-1, keepdim=True)
        # eager steps (one host round trip per token, as Engine.generate does)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(4):
            ids = model.forward(ids, kv_cache=cache)[:, -1, :].argmax(-1, keepdim=True)
        e1.record()
        torch.cuda.synchronize()
        eager_ms = e0.elapsed_time(e1) / 4
        graphed = GraphedDecodeStep(model, cache, ids)
        for _ in range(3):
            ids = graphed.step(ids).argmax(-1, keepdim=True)
        torch.cuda.synchronize()
        e0.record()
        for _ in range(n_new - 8):
            ids = graphed.step(ids).argmax(-1, keepdim=True)
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1) / (n_new - 8)
        ctx = int(cache.cache_seqlens[0].item())
        kv_step = sum(4 * 12 * D * Bc * (min(ctx, w[0] + 1)) for w in model.window_sizes)
        w_bytes = 2 * sum(p_.numel() for n_, p_ in model.named_parameters() if "wte" not in n_ and "value_embeds" not in n_)
        out.update(metric="decode tokens/s (whole model, CUDA-graphed step)", value=Bc / (ms * 1e-3), unit="tokens/s",
                   ms_per_step=ms, eager_ms_per_step=eager_ms, prefill_s=prefill_s, context=ctx,
                   roofline_ms=(kv_step + w_bytes) / (peak * 1e9) * 1e3, kv_bytes_per_step=kv_step, weight_bytes=w_bytes,
                   config={"model": f"d{n_layer}", "B": Bc, "prompt": T0, "steps": n_new})
    elif args.case in ("engine_api_d24", "engine_api_small"):
        # configs[2] through the public generation loop (Engine.generate: one prompt, 64 samples, greedy):
        # per token one host round trip for the sampled ids and the Python row state machine, as in the
        # reference (engine.py:230-280); the decode step itself is replayed from a CUDA graph or run eagerly
        from nanochat_b200.engine import Engine
        from nanochat_b200.gpt import GPT, GPTConfig
        small = args.case.endswith("small")
        n_layer, Bc, T0 = (4, 8, 64) if small else (24, 64, 512)
        cfg = GPTConfig(sequence_len=2048, vocab_size=32768, n_layer=n_layer, n_head=12, n_kv_head=12, n_embd=1536)
        torch.manual_seed(3)
        with torch.device("meta"):
            model = GPT(cfg, compute_dtype=bf)
        model.to_empty(device=dev)
        model.init_weights()
        model.to(bf)
        model.window_sizes = [(1024, 0) if (i % 4) != 3 else (2048, 0) for i in range(n_layer)]
        model.window_sizes[-1] = (2048, 0)

        class _Specials:  # special ids lie outside the vocabulary: no row ever stops early
            def encode_special(self, name):
                return 40000 + (hash(name) % 1000)

            def get_bos_token_id(self):
                return 39999

            def encode(self, text):
                return []

            def decode(self, ids):
                return ""

        prompt = torch.randint(0, 32768, (T0,), generator=torch.Generator().manual_seed(3)).tolist()
        n_new = max(args.steps, 24)
        res = {}
        for mode in (True, False):
            eng = Engine(model, _Specials(), cuda_graph=mode)
            gen_ = eng.generate(prompt, num_samples=Bc, max_tokens=n_new + 8, temperature=0.0)
            for _ in range(8):  # prefill, first steps, graph capture
                next(gen_)
            torch.cuda.synchronize()
            t0 = time.perf_counter()
            for _ in range(n_new):
                next(gen_)
            torch.cuda.synchronize()
            res[mode] = (time.perf_counter() - t0) / n_new
            gen_.close()
        out.update(metric="tokens/s through Engine.generate (whole model, host loop included)",
                   value=Bc / res[True], unit="tokens/s", ms_per_step=res[True] * 1e3,
                   eager_ms_per_step=res[False] * 1e3, eager_tokens_per_s=Bc / res[False],
                   config={"model": f"d{n_layer}", "num_samples": Bc, "prompt": T0, "steps": n_new})
    elif args.case in ("engine_d32", "engine_d32_small"):
        # configs[3]: nanochat d32 with GQA (32 x 2048, 16 query / 4 kv heads), random-init bf16, 256 rows with
        # ragged prompt lengths U[128, 2048], capacity 4096, top-k 50 sampling at temperature 1; per-row
        # positions (the reference loop cannot run this batch), decode step replayed from a CUDA graph.
        # Prefill: uniform 2048-token chunks, each row then truncated to its own length (causal, so the cache
        # rows below that length are those of the shorter prompt).
        from nanochat_b200.engine import GraphedDecodeStep, KVCache, sample_next_token
        from nanochat_b200.gpt import GPT, GPTConfig, rms
        small = args.case.endswith("small")
        n_layer, Bc, Tp, cap, chunk = (4, 16, 256, 512, 8) if small else (32, 256, 2048, 4096, 16)
        cfg = GPTConfig(sequence_len=cap, vocab_size=32768, n_layer=n_layer, n_head=16, n_kv_head=4, n_embd=2048)
        torch.manual_seed(4)
        with torch.device("meta"):
            model = GPT(cfg, compute_dtype=bf)
        model.to_empty(device=dev)
        model.init_weights()
        model.to(bf)
        model.window_sizes = [(cap // 2, 0) if (i % 4) != 3 else (cap, 0) for i in range(n_layer)]
        model.window_sizes[-1] = (cap, 0)
        g4 = torch.Generator().manual_seed(4)
        lens = torch.randint(Tp // 16, Tp + 1, (Bc,), generator=g4, dtype=torch.int32)
        prompts = torch.randint(0, 32768, (Bc, Tp), generator=g4)
        cache = KVCache(batch_size=Bc, num_heads=4, seq_len=cap, head_dim=128, num_layers=n_layer, device=dev, dtype=bf)
        t0 = time.perf_counter()
        prev, first = [], []
        for r0 in range(0, Bc, chunk):
            part = KVCache(batch_size=chunk, num_heads=4, seq_len=Tp, head_dim=128, num_layers=n_layer, device=dev, dtype=bf)
            ids_c = prompts[r0:r0 + chunk].to(dev)
            logits_c = model.forward(ids_c, kv_cache=part)
            cache.k_cache[:, r0:r0 + chunk, :Tp] = part.k_cache
            cache.v_cache[:, r0:r0 + chunk, :Tp] = part.v_cache
            rows = torch.arange(chunk, device=dev)
            last = (lens[r0:r0 + chunk].to(dev) - 1).long()
            first.append(logits_c[rows, last])                      # logits at each row's own last prompt token
            prev.append(rms(model.transformer.wte(ids_c[rows, last]).to(bf)).unsqueeze(1))  # smear state of the model's forward
            del part, logits_c
        cache.cache_seqlens.copy_(lens.to(dev))
        cache.prev_embedding = torch.cat(prev, 0)
        torch.cuda.synchronize()
        prefill_s = time.perf_counter() - t0
        rng = torch.Generator(device=dev).manual_seed(4)
        ids = sample_next_token(torch.cat(first, 0).float(), rng, temperature=1.0, top_k=50)
        n_new = max(args.steps, 8)
        graphed = GraphedDecodeStep(model, cache, ids)
        for _ in range(3):
            ids = sample_next_token(graphed.step(ids).float(), rng, temperature=1.0, top_k=50)
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(n_new):
            ids = sample_next_token(graphed.step(ids).float(), rng, temperature=1.0, top_k=50)
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1) / n_new
        now = cache.cache_seqlens.long().cpu()
        kv_step = sum(4 * 4 * D * int(torch.clamp(now, max=w[0] + 1).sum()) for w in model.window_sizes)
        w_bytes = 2 * sum(p_.numel() for n_, p_ in model.named_parameters() if "wte" not in n_ and "value_embeds" not in n_)
        out.update(metric="decode tokens/s (whole model, ragged rows, top-k sampling, CUDA-graphed step)",
                   value=Bc / (ms * 1e-3), unit="tokens/s", ms_per_step=ms, prefill_s=prefill_s,
                   mean_context=float(now.float().mean()), roofline_ms=(kv_step + w_bytes) / (peak * 1e9) * 1e3,
                   kv_bytes_per_step=kv_step, weight_bytes=w_bytes,
                   config={"model": f"d{n_layer} GQA 16/4", "B": Bc, "prompt": f"U[{Tp // 16},{Tp}]", "capacity": cap,
                           "steps": n_new, "sampling": "top-k 50, temperature 1"})
    elif args.case == "prefill":            # dense causal attention, d24 shape: 12 heads, T=2048
        Bc, T, Hq, Hkv = 8, 2048, 12, 12
        q, k, v = rnd(Bc, T, Hq, D), rnd(Bc, T, Hkv, D), rnd(Bc, T, Hkv, D)
        sec = _time_cuda(lambda i: ops.prefill_attention(q, k, v, None, -1), iters)
        flops = 4.0 * D * Bc * Hq * (T * (T + 1) / 2)
        # the kernel the reference reaches on this GPU for the same call: torch SDPA, causal (flash_attention.py:79-80)
        qs, ks, vs = (t.transpose(1, 2) for t in (q, k, v))
        sdpa_sec = _time_cuda(lambda i: torch.nn.functional.scaled_dot_product_attention(qs, ks, vs, is_causal=True), iters)
        try:
            with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
                tpeak = float(json.load(f)["bf16_tflops"])
        except Exception:
            tpeak = 1590.0
        out.update(metric="prefill attention TFLOP/s (causal, useful FLOPs)", value=flops / sec / 1e12, unit="TFLOP/s",
                   us_per_call=sec * 1e6, frac=flops / sec / 1e12 / tpeak, peak=tpeak,
                   torch_sdpa={"us_per_call": sdpa_sec * 1e6, "tflops": flops / sdpa_sec / 1e12},
                   config={"B": Bc, "T": T, "Hq": Hq, "Hkv": Hkv})
    elif args.case == "train_attn":         # flash_attn_func forward + backward, d24 training shape
        Bc, T, Hq, Hkv = 8, 2048, 12, 12
        q, k, v = (rnd(Bc, T, Hq, D).requires_grad_(True), rnd(Bc, T, Hkv, D).requires_grad_(True),
                   rnd(Bc, T, Hkv, D).requires_grad_(True))
        dout = rnd(Bc, T, Hq, D)
        from nanochat_b200.flash_attention import flash_attn

        def ours(i):
            flash_attn.flash_attn_func(q, k, v, causal=True, window_size=(-1, 0)).backward(dout)
        o_, lse_ = ops.flash_attn_fwd(q.detach(), k.detach(), v.detach(), -1)
        sec = _time_cuda(ours, iters)
        bwd_sec = _time_cuda(lambda i: ops.flash_attn_bwd(q.detach(), k.detach(), v.detach(), o_, dout, lse_, -1), iters)
        qs, ks, vs = (t.detach().transpose(1, 2).requires_grad_(True) for t in (q, k, v))
        dts = dout.transpose(1, 2)

        def sdpa(i):  # what the reference runs on this GPU when training (flash_attention.py:122-128)
            torch.nn.functional.scaled_dot_product_attention(qs, ks, vs, is_causal=True).backward(dts)
        sdpa_sec = _time_cuda(sdpa, iters)
        flops = 3.5 * 4.0 * D * Bc * Hq * (T * (T + 1) / 2)  # forward 2 products, backward 5, causal half
        out.update(metric="attention forward + backward, us per call (causal, training shape)", value=sec * 1e6, unit="us",
                   backward_us=bwd_sec * 1e6, useful_tflops=flops / sec / 1e12,
                   torch_sdpa={"us_per_call": sdpa_sec * 1e6, "useful_tflops": flops / sdpa_sec / 1e12},
                   config={"B": Bc, "T": T, "Hq": Hq, "Hkv": Hkv})
    elif args.case == "broadcast":          # configs[4]: 8192-token block -> 64 sample rows, one layer
        L, Bc, p, Hkv = 1, 64, 8192, 4
        src_k, src_v = rnd(L, 1, p, Hkv, D), rnd(L, 1, p, Hkv, D)
        dst_k = torch.empty(L, Bc, p, Hkv, D, device=dev, dtype=bf)
        dst_v = torch.empty_like(dst_k)
        lens = torch.zeros(Bc, device=dev, dtype=torch.int32)
        sec = _time_cuda(lambda i: ops.prefill_broadcast(src_k, src_v, dst_k, dst_v, lens, p), iters)
        nbytes = 2 * L * (Bc + 1) * p * Hkv * D * 2
        out.update(metric="prefill broadcast GB/s (written + read)", value=nbytes / sec / 1e9, unit="GB/s",
                   us_per_call=sec * 1e6, algorithmic_bytes=nbytes, frac=nbytes / sec / 1e9 / peak, peak=peak,
                   peak_kind=f"of {peak_kind}", config={"L": L, "B": Bc, "p": p, "Hkv": Hkv})
    elif args.case == "decode_paged":       # one layer of configs[3] in pages of 192 tokens: same rows, scattered pages
        Bc, Hq, Hkv, T, pt = 256, 16, 4, 4096, 192
        lens = torch.randint(128, 4095, (Bc,), dtype=torch.int32, generator=torch.Generator().manual_seed(5))
        pages_of = [-(-(int(L) + 1) // pt) for L in lens.tolist()]
        n_pages = sum(pages_of)
        max_pages = -(-T // pt)
        perm = torch.randperm(n_pages, generator=torch.Generator().manual_seed(6)).to(torch.int32)
        table = torch.full((Bc, max_pages), -1, dtype=torch.int32)
        at = 0
        for b_, n_ in enumerate(pages_of):
            table[b_, :n_] = perm[at:at + n_]
            at += n_
        kp, vp = rnd(n_pages, pt, Hkv, D), rnd(n_pages, pt, Hkv, D)
        q = rnd(Bc, Hq, D)
        table_d, lens_d = table.to(dev), lens.to(dev)
        sec = _time_cuda(lambda i: ops.decode_attention_paged(q, kp, vp, table_d, lens_d, 1, -1), iters)
        nbytes = 4 * Hkv * D * int((lens.long() + 1).sum()) + 4 * Bc * Hq * D + 4 * Bc
        out.update(metric="decode attention KV-read GB/s (paged storage)", value=nbytes / sec / 1e9, unit="GB/s", us_per_call=sec * 1e6,
                   algorithmic_bytes=nbytes, frac=nbytes / sec / 1e9 / peak, peak=peak, peak_kind=f"of {peak_kind}",
                   pool_bytes=2 * n_pages * pt * Hkv * D * 2, dense_bytes=2 * Bc * T * Hkv * D * 2,
                   config={"B": Bc, "Hq": Hq, "Hkv": Hkv, "T_max": T, "page_tokens": pt, "pages": n_pages})
    elif args.case == "prefill_paged":      # configs[4] broadcast into a paged cache: prompt pages shared by the 64 rows
        from nanochat_b200.engine import KVCache, PagedKVCache
        L, Bc, p_, Hkv, pt, cap = 1, 64, 8192, 4, 192, 8192 + 1024
        prompt = KVCache(1, Hkv, p_, D, L, dev, bf)
        prompt.k_cache.copy_(rnd(*prompt.k_cache.shape))
        prompt.v_cache.copy_(rnd(*prompt.v_cache.shape))
        prompt.advance(p_)
        own = -(-cap // pt) - p_ // pt
        cache = PagedKVCache(Bc, Hkv, cap, D, L, dev, bf, page_tokens=pt, n_pages=p_ // pt + Bc * own)

        def fill(i):
            cache.reset()
            cache.prefill(prompt)

        sec = _time_cuda(fill, iters)
        written = 2 * L * cache.pages_in_use() * pt * Hkv * D * 2
        out.update(metric="prefill into a paged cache, us per call (host bookkeeping included)", value=sec * 1e6, unit="us",
                   bytes_written_upper_bound=written, dense_broadcast_bytes=2 * L * Bc * p_ * Hkv * D * 2,
                   pages_in_use=cache.pages_in_use(), config={"L": L, "B": Bc, "p": p_, "Hkv": Hkv, "page_tokens": pt})
    elif args.case == "append":             # configs[1] append alone
        kc, vc = rnd(B, T_MAX, HKV, D), rnd(B, T_MAX, HKV, D)
        q, k, v = rnd(B, 1, HQ, D), rnd(B, 1, HKV, D), rnd(B, 1, HKV, D)
        cos, sin = precompute_rotary_embeddings(T_MAX, D, device=dev)
        lens = seqlens_cpu().to(dev)
        sec = _time_cuda(lambda i: ops.append_rope_norm(q, k, v, kc, vc, lens, cos, sin), iters)
        nbytes = 2 * B * (HQ + 2 * HKV) * D * 2 + B * D * 2
        out.update(metric="append us per call", value=sec * 1e6, unit="us", algorithmic_bytes=nbytes,
                   config={"B": B, "Hq": HQ, "Hkv": HKV})
    else:
        raise SystemExit(f"unknown case {args.case}")
    out["device_status"] = ops.read_status(dev)
    print(json.dumps(out), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=2000)
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--regions", type=int, default=None,
                    help="time this many K-step regions instead of about a second's worth (at least 50)")
    ap.add_argument("--no-extras", action="store_true",
                    help="headline workload only: skip the long_context, d24_sharded and gpu_reference legs")
    ap.add_argument("--case", default=None,
                    help="secondary op-level measurement instead of the headline workload: decode_long, decode_gqa, "
                         "decode_gqa_window, decode_d24, decode_paged, prefill, prefill_paged, train_attn, broadcast, append, engine_d24, engine_d24_small, engine_d32, "
                         "engine_d32_small, engine_api_d24, engine_api_small")
    args = ap.parse_args()
    global REGIONS_OVERRIDE
    REGIONS_OVERRIDE = args.regions
    if args.case:
        run_case(args)
    elif args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
