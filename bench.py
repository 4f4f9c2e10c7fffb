"""Benchmark of the KV-cache decode hot path (KV append + decode attention) on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Workload (BASELINE.json configs[1]): B=32 rows, 12 q heads, 12 kv heads, head_dim 128, cache
capacity 2048, cache_seqlens uniform in [1, 2047] (torch CPU generator, seed 2), caches and new
q/k/v ~ N(0,1) bf16, one new token per row, full causal.  One "step" is one pass of the hot path
over that batch: the fused RoPE + QK-norm + append launch followed by the split-KV decode
attention launch.  At N > 1 every rank runs the same workload on its own rows (sequences are
independent: no collective on the data path), so scaling is weak.

Timing: CUDA events on the launching stream, W warm-up steps, K timed steps, barrier + device
synchronisation on both sides, max over ranks.  Each step reads a different one of NSETS cache
sets (NSETS x 403 MB, far larger than the 126 MB L2) so KV bytes come from HBM.
  value     steps replayed from a CUDA graph, inputs resident in HBM
  roofline  one nckv_decode_attn call alone (streaming kernel + its small merge kernel), launched
            K times through the C ABI
  e2e       the public Python call with HOST inputs: H2D of q/k/v, both launches, D2H of the output
  cpu_baseline / --impl reference   the torch-eager port of the reference's CPU path (fp32, SDPA)
"""
import argparse
import json
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
# dram__bytes_read.sum + dram__bytes_write.sum of one decode_attn_kernel launch on this workload, from the ncu
# capture summarised in profiles/decode_attn_config1.md
TRAFFIC_BYTES_PER_LAUNCH = 202.78e6
METRIC = "decode tokens/s (KV append + decode attention, B=32 x 12 heads x 128, ragged cache)"
WORKLOAD = "configs[1]: op-level KV append + decode attention, B=32, 12q/12kv heads, D=128, T_max=2048, ragged seqlens seed 2"


def seqlens_cpu():
    return torch.randint(1, 2048, (B,), dtype=torch.int32, generator=torch.Generator().manual_seed(2))


def algorithmic_bytes(seqlens):
    """Bytes one append + decode-attention call must move (bf16): visible K and V rows, q in/out,
    the new k/v read and written, cache_seqlens, one cos and one sin row per batch row."""
    n_keys = int((seqlens.long() + 1).sum())
    kv = 4 * HKV * D * n_keys
    other = 2 * B * HQ * D * 2 + 2 * B * HKV * D * 2 * 2 + 4 * B + B * D * 2
    return kv, other


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
    t = torch.tensor([x], dtype=torch.float64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


# ------------------------------------------------------------------------------------------------
# CPU baseline: the reference's CPU path (torch-eager port under oracle/), fp32, all host threads
# ------------------------------------------------------------------------------------------------
def cpu_reference_run(steps, warmup, budget_s=25.0):
    from oracle import torch_ref as R
    # all the host cores this process may use (torchrun exports OMP_NUM_THREADS=1 to its ranks)
    try:
        usable = len(os.sched_getaffinity(0))
    except AttributeError:
        usable = os.cpu_count() or 1
    torch.set_num_threads(max(usable, 1))
    threads = torch.get_num_threads()
    gen = torch.Generator().manual_seed(2)
    seqlens = seqlens_cpu()
    k_cache = torch.randn(B, T_MAX, HKV, D, generator=gen)
    v_cache = torch.randn(B, T_MAX, HKV, D, generator=gen)
    q = torch.randn(B, 1, HQ, D, generator=gen)
    k = torch.randn(B, 1, HKV, D, generator=gen)
    v = torch.randn(B, 1, HKV, D, generator=gen)
    cos, sin = R.rotary_tables(T_MAX, D, "cpu", torch.float32)

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
    return {"value": B * done / dt, "unit": "tokens/s", "cores": threads, "kind": "port",
            "sample": f"{done} full configs[1] steps (fp32, torch SDPA row by row as the reference's CPU fallback does), "
                      f"{dt:.1f} s", "ms_per_step": 1e3 * dt / done}, done, dt


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    cb, done, dt = cpu_reference_run(args.steps, args.warmup)
    line = {"impl": "reference", "metric": METRIC, "value": cb["value"], "unit": "tokens/s", "n_gpus": args.gpus,
            "steps": done, "warmup": args.warmup, "ms_per_step": cb["ms_per_step"], "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": WORKLOAD, "device": "host CPU"},
            "cpu_baseline": {k: cb[k] for k in ("value", "unit", "cores", "kind", "sample")},
            "e2e": {"value": cb["value"], "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0}
    print(json.dumps(line), flush=True)


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
    kv_bytes, other_bytes = algorithmic_bytes(seqlens_h)
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
        with torch.cuda.graph(graph, stream=side):
            for i in range(NSETS):
                out_graph = step(i)
    replays = (K + NSETS - 1) // NSETS
    k_eff = replays * NSETS
    for _ in range(max(1, (W + NSETS - 1) // NSETS)):
        graph.replay()
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
        time.sleep(0.5)
        for _ in range(200 if K >= 200 else 0):  # keep the GPU under load while the first samples are taken
            graph.replay()
    barrier(world)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(replays):
        graph.replay()
    e1.record()
    barrier(world)
    ms_total = max_over_ranks(e0.elapsed_time(e1), world, dev)
    ms_step = ms_total / k_eff
    value = world * B / (ms_step * 1e-3)

    # ---- roofline: the decode-attention kernel alone, through the C ABI ----------------------------
    q2 = ops.append_rope_norm(q, k, v, sets[0][0], sets[0][1], seqlens, cos, sin)[:, 0].contiguous()
    out = torch.empty_like(q2)
    ws = ops.workspace(dev, B, HQ, HKV)
    stream = torch.cuda.current_stream(dev)

    def attn_only(i):
        kc, vc = sets[i % NSETS]
        _lib.call("nckv_decode_attn", q2.data_ptr(), kc.data_ptr(), vc.data_ptr(), seqlens.data_ptr(), out.data_ptr(),
                  None, None, B, HQ, HKV, D, T_MAX, kc.stride(0), kc.stride(1), 1, -1, 0, 0, ws.data_ptr(), ws.numel(),
                  stream.cuda_stream)

    for i in range(max(W, 3)):
        attn_only(i)
    torch.cuda.synchronize()
    a0, a1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    n_attn = max(K, 200) if K >= 200 else max(K, 10)
    a0.record()
    for i in range(n_attn):
        attn_only(i)
    a1.record()
    torch.cuda.synchronize()
    attn_ms = a0.elapsed_time(a1) / n_attn
    status = ops.read_status(dev)
    clocks = sampler.stop() if rank == 0 else None

    # ---- e2e: public call, host buffers ------------------------------------------------------------
    # host side of a step: q, k, v of the new token in one pinned block (H2D), the output pinned (D2H);
    # one public call per step (ops.HostDecodeStep.run -> nckv_decode_step_host), which synchronises
    def time_host_steps(transfer):
        host_step = ops.HostDecodeStep(B, HQ, HKV, cos, sin, dev, transfer=transfer)
        host_step.q.copy_(q[:, 0].cpu())
        host_step.k.copy_(k[:, 0].cpu())
        host_step.v.copy_(v[:, 0].cpu())

        def e2e_step(i):
            kc, vc = sets[i % NSETS]
            return host_step.run(kc, vc, seqlens, -1)

        for i in range(max(W, 3)):
            e2e_step(i)
        barrier(world)
        t0 = time.perf_counter()
        c0, c1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        c0.record()
        for i in range(K):
            e2e_step(i)
        c1.record()
        barrier(world)
        dev_ms = max_over_ranks(c0.elapsed_time(c1), world, dev) / K
        wall_ms = max_over_ranks(1e3 * (time.perf_counter() - t0), world, dev) / K
        return dev_ms, wall_ms, host_step.host_in.numel() * 2, host_step.out.numel() * 2

    # headline: explicit H2D / D2H copies around the kernels; beside it the mapped variant (the kernels
    # read the pinned inputs and write the pinned output over PCIe themselves: same bytes, no copy ops)
    e2e_ms, e2e_wall_ms, h2d, d2h = time_host_steps("copy")
    e2e_value = world * B / (e2e_ms * 1e-3)
    mapped_ms, _, _, _ = time_host_steps("mapped")

    if rank == 0:
        peak, peak_kind = peaks()
        achieved = (kv_bytes + other_bytes) / (attn_ms * 1e-3) / 1e9
        cb = None
        if world == 1 and not args.no_cpu_baseline:
            cb_full, _, _ = cpu_reference_run(steps=100000, warmup=2, budget_s=12.0)
            cb = {k_: cb_full[k_] for k_ in ("value", "unit", "cores", "kind", "sample")}
        line = {
            "metric": METRIC, "value": value, "unit": "tokens/s", "n_gpus": world, "steps": k_eff, "warmup": W,
            "ms_per_step": ms_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "bf16", "data": "synthetic",
            "config": {"workload": WORKLOAD, "rows_per_gpu": B, "l2": f"{NSETS} cache sets rotated, {NSETS * 2 * B * T_MAX * HKV * D * 2 / 1e6:.0f} MB > L2",
                       "launch": "CUDA graph replay of append + attention (3 kernels per step)", "parallelism": f"{world} x independent sequences"},
            "kv_read_gbs": world * kv_bytes / (ms_step * 1e-3) / 1e9,
            "roofline": {"bound": "hbm", "kernel": "decode_attn_kernel + decode_merge_kernel (one nckv_decode_attn call)", "achieved": achieved, "peak": peak,
                         "peak_kind": f"of {peak_kind}", "unit": "GB/s", "frac": achieved / peak,
                         "frac_of_8000_nominal": achieved / 8000.0, "us_per_launch": attn_ms * 1e3,
                         "algorithmic_bytes": kv_bytes + other_bytes, "traffic": TRAFFIC_BYTES_PER_LAUNCH},
            "e2e": {"value": e2e_value, "unit": "tokens/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                    "ms_per_step": e2e_ms, "wall_ms_per_step": e2e_wall_ms,
                    "mapped_host_memory": {"value": world * B / (mapped_ms * 1e-3), "ms_per_step": mapped_ms}},
            "gpu_launches": 3 * k_eff, "device_status": status, "clocks": clocks,
        }
        if cb is not None:
            line["cpu_baseline"] = cb
        print(json.dumps(line), flush=True)
    if world > 1:
        import torch.distributed as dist
        dist.destroy_process_group()


# ------------------------------------------------------------------------------------------------
# secondary cases (one JSON line each): the other kernels and the other BASELINE configs, op level
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
    """configs[4] with the keys split across the ranks (torchrun): every rank attends over its key
    range of every row, one all-gather of the partials, LSE combine.  Strong scaling: total work fixed."""
    rank, world, local = dist_setup(args.gpus)
    dev = torch.device("cuda", local)
    torch.cuda.set_device(dev)
    from nanochat_b200 import ops
    from nanochat_b200.dist import KVSplitAttention
    peak, peak_kind = peaks()
    Bc, Hq, Hkv, T = 8, 16, 4, 65536
    lens = torch.randint(32768, 65536, (Bc,), dtype=torch.int32, generator=torch.Generator().manual_seed(4))
    # block-cyclic ownership (ragged rows stay balanced), exchange over NVLink peer memory
    att = KVSplitAttention(T, block=1024, exchange="p2p")
    gen = torch.Generator(device=dev).manual_seed(4)
    nsets = 2
    cap = att.local_capacity
    sets = [(torch.randn(Bc, cap, Hkv, D, generator=gen, device=dev).to(torch.bfloat16),
             torch.randn(Bc, cap, Hkv, D, generator=gen, device=dev).to(torch.bfloat16)) for _ in range(nsets)]
    q = torch.randn(Bc, Hq, D, generator=torch.Generator(device=dev).manual_seed(5), device=dev).to(torch.bfloat16)
    lens_d = lens.to(dev)
    iters = max(args.steps, 5)
    # the whole step (split-plan, attention over the local shard, merge, push to peers, wait + combine) is
    # kernels only, so nsets consecutive steps are replayed from one CUDA graph
    side = torch.cuda.Stream(dev)
    with torch.cuda.stream(side):
        for i in range(2 * nsets):
            att.attend(q, sets[i % nsets][0], sets[i % nsets][1], lens_d)
        side.synchronize()
        barrier(world)
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=side):
            for i in range(nsets):
                att.attend(q, sets[i][0], sets[i][1], lens_d)
    torch.cuda.synchronize()
    replays = (iters + nsets - 1) // nsets
    iters = replays * nsets
    for _ in range(3):
        graph.replay()
    barrier(world)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(replays):
        graph.replay()
    e1.record()
    barrier(world)
    sec = max_over_ranks(e0.elapsed_time(e1), world, dev) / iters * 1e-3
    status = ops.read_status(dev)
    if rank == 0:
        nbytes = 4 * Hkv * D * int((lens.long() + 1).sum()) + 4 * Bc * Hq * D + 4 * Bc
        print(json.dumps({"case": "decode_long", "n_gpus": world, "steps": iters, "scaling": "strong", "data": "synthetic",
                          "dtype": "bf16", "metric": "decode attention KV-read GB/s (keys split across GPUs, all-gather + LSE combine)",
                          "value": nbytes / sec / 1e9, "unit": "GB/s", "us_per_call": sec * 1e6, "algorithmic_bytes": nbytes,
                          "frac_of_n_x_peak": nbytes / sec / 1e9 / (peak * world), "peak": peak, "peak_kind": f"of {peak_kind}",
                          "exchange_bytes_per_rank": Bc * Hq * (D + 1) * 4,
                          "config": {"B": Bc, "Hq": Hq, "Hkv": Hkv, "T_max": T, "layout": "block-cyclic, 1024 keys", "keys_per_rank": cap,
                                     "launch": f"CUDA graph, exchange={att.exchange}"},
                          "device_status": status}), flush=True)
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
        try:
            with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
                tpeak = float(json.load(f)["bf16_tflops"])
        except Exception:
            tpeak = 1590.0
        out.update(metric="prefill attention TFLOP/s (causal, useful FLOPs)", value=flops / sec / 1e12, unit="TFLOP/s",
                   us_per_call=sec * 1e6, frac=flops / sec / 1e12 / tpeak, peak=tpeak,
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
    ap.add_argument("--case", default=None,
                    help="secondary op-level measurement instead of the headline workload: decode_long, decode_gqa, "
                         "decode_gqa_window, decode_d24, prefill, broadcast, append, engine_d24, engine_d24_small, engine_d32, "
                         "engine_d32_small, engine_api_d24, engine_api_small")
    args = ap.parse_args()
    if args.case:
        run_case(args)
    elif args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
