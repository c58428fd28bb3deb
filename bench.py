#!/usr/bin/env python
"""Benchmark of the attention hot path on B200.

Headline workload (`decode_ctx4096_36layers`): one decode token through the
36-layer decode-attention stack at context 4096 with Qwen3-8B attention shapes
(32 query heads, 8 KV heads, head_dim 128, Q8_0 KV cache). One step = for each
layer: Q norm+RoPE, KV write-back of the new token at row 4095, split-KV decode
attention over 4096 keys. The metric is achieved HBM GB/s = algorithmic cache
bytes read (2304 B per token per layer) / time.

  python bench.py --gpus 1 --steps 50 --warmup 5          # this implementation
  python bench.py --impl reference --steps 3 --warmup 1   # CPU restatement of the reference

With N > 1 ranks (torchrun) the KV heads are sharded over the ranks and the
per-head outputs are all-gathered with NCCL after every layer (strong scaling).

Prints ONE JSON line on rank 0.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

N_LAYER, N_HEAD, N_KV_HEAD, HEAD_DIM = 36, 32, 8, 128
Q_DIM, KV_DIM = N_HEAD * HEAD_DIM, N_KV_HEAD * HEAD_DIM
BYTES_PER_TOKEN_LAYER = 2 * (KV_DIM + KV_DIM // 32 * 4)  # 2304: K and V, int8 + f32 block scales
FALLBACK_HBM_GBS, FALLBACK_TFLOPS = 6650.0, 1590.0


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            d = json.load(f)
        return float(d["hbm_gbs"]), float(d["bf16_tflops"]), "measured"
    except Exception:
        return FALLBACK_HBM_GBS, FALLBACK_TFLOPS, "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while a region runs."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index, self.proc, self.file = index, None, None

    def start(self):
        try:
            self.file = tempfile.NamedTemporaryFile("w+", suffix=".csv", delete=False)
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-i", str(self.index), "-lms", "100"], stdout=self.file, stderr=subprocess.DEVNULL)
        except Exception:
            self.proc = None

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        self.file.flush()
        self.file.seek(0)
        sm, mx, reasons = [], [], set()
        for line in self.file.read().splitlines():
            f = [x.strip() for x in line.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1]))
                mx.append(float(f[2]))
            except ValueError:
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        try:
            os.unlink(self.file.name)
        except OSError:
            pass
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


# ----------------------------------------------------------------------------
# CPU side: the oracle timed as the baseline / the reference arm.
# ----------------------------------------------------------------------------
def cpu_decode_gbs(ctx_len, n_layers_sample, reps, seed=0):
    """Times the CPU restatement of attention_split + attention_merge (plus the
    two small kernels) on `n_layers_sample` layers of the workload, all host
    threads. Returns (GB/s, seconds per sample, threads)."""
    import numpy as np
    from bonsai_pot_b200 import synth
    from oracle import oracle as O
    try:
        O.lib(native=True)
        native = True
    except Exception:
        native = False
    sh = O.Shape(n_layer=n_layers_sample, n_head=N_HEAD, n_kv_head=N_KV_HEAD, max_seq=ctx_len)
    rope = O.rope_table_f16(sh)
    w = synth.ones_weight()
    kv_k, kv_v = sh.new_cache(), sh.new_cache()
    qs, ks, vs = [], [], []
    for il in range(n_layers_sample):
        O.quantize_rows(sh, synth.tensor(seed, 1, il, synth.T_K_PAST, (ctx_len - 1, sh.kv_dim)), kv_k, il, 0, ctx_len - 1)
        O.quantize_rows(sh, synth.tensor(seed, 1, il, synth.T_V_PAST, (ctx_len - 1, sh.kv_dim)), kv_v, il, 0, ctx_len - 1)
        qs.append(synth.tensor(seed, 1, il, synth.T_Q, (1, sh.q_dim)))
        ks.append(synth.tensor(seed, 1, il, synth.T_K_NEW, (1, sh.kv_dim)))
        vs.append(synth.tensor(seed, 1, il, synth.T_V_NEW, (1, sh.kv_dim)))
    best = None
    for _ in range(reps):
        t0 = time.perf_counter()
        for il in range(n_layers_sample):
            qn = O.q_norm_rope(sh, qs[il], w, rope, ctx_len - 1, 1, native=native)
            O.kv_writeback(sh, ks[il], vs[il], w, rope, kv_k, kv_v, il, ctx_len - 1, 1, native=native)
            O.attn_decode(sh, qn, kv_k, kv_v, il, ctx_len, native=native)
        dt = time.perf_counter() - t0
        best = dt if best is None else min(best, dt)
    gbs = n_layers_sample * ctx_len * BYTES_PER_TOKEN_LAYER / best / 1e9
    return gbs, best, O.num_threads(native)


def run_reference(args):
    """Reference arm: the reference's own engine (Rust + wgpu/Vulkan) cannot be
    built or run on this machine, so its CPU restatement (the oracle) is timed
    on the host cores with all threads, on the same workload and metric."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    n_sample = 4
    times = []
    gbs = 0.0
    threads = 1
    for i in range(args.warmup + args.steps):
        g, dt, threads = cpu_decode_gbs(args.ctx, n_sample, 1, seed=0) if i == 0 else cpu_decode_gbs_cached(args.ctx, n_sample)
        if i >= args.warmup:
            times.append(dt)
    dt = statistics.mean(times)
    gbs = n_sample * args.ctx * BYTES_PER_TOKEN_LAYER / dt / 1e9
    sample = f"{n_sample} of {N_LAYER} layers of the decode stack at ctx {args.ctx} per step"
    line = {
        "impl": "reference", "metric": "decode_attn_hbm_gbs", "value": round(gbs, 4), "unit": "GB/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(dt * 1e3, 3),
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": f"decode_ctx{args.ctx}_{N_LAYER}layers", "n_head": N_HEAD, "n_kv_head": N_KV_HEAD,
                   "head_dim": HEAD_DIM, "kv_cache": "Q8_0 (int8 + f32 block scales)"},
        "cpu_baseline": {"value": round(gbs, 4), "unit": "GB/s", "cores": threads, "kind": "port", "sample": sample},
        "e2e": {"value": round(gbs, 4), "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
        "note": "CPU restatement of the reference's WGSL math (the Rust/wgpu reference itself is unavailable on this box)",
    }
    print(json.dumps(line), flush=True)


_CPU_CACHE = {}


def cpu_decode_gbs_cached(ctx_len, n_layers_sample):
    """Same measurement as cpu_decode_gbs without regenerating the inputs."""
    import numpy as np
    from bonsai_pot_b200 import synth
    from oracle import oracle as O
    key = (ctx_len, n_layers_sample)
    if key not in _CPU_CACHE:
        sh = O.Shape(n_layer=n_layers_sample, n_head=N_HEAD, n_kv_head=N_KV_HEAD, max_seq=ctx_len)
        kv_k, kv_v = sh.new_cache(), sh.new_cache()
        rng = np.random.default_rng(0)
        # cache content does not change the CPU time: fill with plain random quants and scales
        for kv in (kv_k, kv_v):
            kv[:sh.d_total].view(np.float32)[:] = rng.random(sh.d_total // 4, dtype=np.float32) * 0.03
            kv[sh.d_total:] = rng.integers(0, 256, size=kv.size - sh.d_total, dtype=np.uint8)
        q = [O.q_norm_rope(sh, synth.tensor(0, 1, il, synth.T_Q, (1, sh.q_dim)), synth.ones_weight(),
                           O.rope_table_f16(sh), ctx_len - 1, 1) for il in range(n_layers_sample)]
        _CPU_CACHE[key] = (sh, kv_k, kv_v, q)
    sh, kv_k, kv_v, q = _CPU_CACHE[key]
    try:
        O.lib(native=True)
        native = True
    except Exception:
        native = False
    t0 = time.perf_counter()
    for il in range(n_layers_sample):
        O.attn_decode(sh, q[il], kv_k, kv_v, il, ctx_len, native=native)
    dt = time.perf_counter() - t0
    return n_layers_sample * ctx_len * BYTES_PER_TOKEN_LAYER / dt / 1e9, dt, O.num_threads(native)


# ----------------------------------------------------------------------------
# GPU side
# ----------------------------------------------------------------------------
def fill_cache(ctx, torch, n_layer, kv_dim, rows, gen):
    """Fills cache rows [0, rows) of every layer from seeded N(0,1) f16 data with
    the library's own write-back kernel (content does not affect timing)."""
    w = torch.ones(128, dtype=torch.float16, device="cuda")
    chunk = 4096
    for il in range(n_layer):
        for r0 in range(0, rows, chunk):
            m = min(chunk, rows - r0)
            k = torch.randn(m, kv_dim, generator=gen, device="cuda", dtype=torch.float32).half()
            v = torch.randn(m, kv_dim, generator=gen, device="cuda", dtype=torch.float32).half()
            ctx.dispatch_kv_writeback_fused(il, k, v, w, r0, m)
    torch.cuda.synchronize()


def graphed(torch, fn, stream):
    """Runs fn once eagerly, then captures it in a CUDA graph on `stream`; returns the replay callable.
    Host launch overhead (Python + ctypes) then stays out of the timed region."""
    with torch.cuda.stream(stream):
        fn()
        stream.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=stream):
            fn()
    torch.cuda.synchronize()
    return g.replay


def time_region(torch, fn, steps, stream):
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    start.record(stream)
    for _ in range(steps):
        fn()
    end.record(stream)
    torch.cuda.synchronize()
    return start.elapsed_time(end) / 1e3  # seconds


def run_ours(args):
    import torch
    import torch.distributed as dist

    import bonsai_pot_b200 as bp

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: there is no CPU path")
    torch.cuda.set_device(local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    assert N_KV_HEAD % world == 0, "KV heads shard over 1, 2, 4 or 8 ranks"
    nkv_l, nh_l = N_KV_HEAD // world, N_HEAD // world
    q_dim_l, kv_dim_l = nh_l * HEAD_DIM, nkv_l * HEAD_DIM
    ctx_len = args.ctx
    hbm_peak, tflops_peak, peak_kind = measured_peaks()

    ctx = bp.AttnContext(n_layer=N_LAYER, n_head=nh_l, n_kv_head=nkv_l, max_seq=ctx_len, n_shards=world, shard=rank,
                         device=local_rank)
    if args.decode_warps:
        ctx.set_option("decode_warps", args.decode_warps)
    if args.decode_hpc:
        ctx.set_option("decode_heads_per_cta", args.decode_hpc)
    if args.decode_uhpc:
        ctx.set_option("decode_umma_heads_per_cta", args.decode_uhpc)
    if args.no_pdl:
        ctx.set_option("dependent_launch", 0)
    if args.decode_ring:
        ctx.set_option("decode_ring", args.decode_ring)
    if args.separate_merge:
        ctx.set_option("decode_in_kernel_merge", 0)
    gen = torch.Generator(device="cuda")
    gen.manual_seed(1234 + rank)
    fill_cache(ctx, torch, N_LAYER, kv_dim_l, ctx_len - 1, gen)

    ctx.set_variant(args.variant)
    w = torch.ones(128, dtype=torch.float16, device="cuda")
    q_raw = torch.randn(N_LAYER, q_dim_l, generator=gen, device="cuda").half()
    k_new = torch.randn(N_LAYER, kv_dim_l, generator=gen, device="cuda").half()
    v_new = torch.randn(N_LAYER, kv_dim_l, generator=gen, device="cuda").half()
    q_work = q_raw.clone()
    out_local = torch.zeros(N_LAYER, q_dim_l, dtype=torch.float16, device="cuda")
    out_full = torch.zeros(N_LAYER, Q_DIM, dtype=torch.float16, device="cuda") if world > 1 else out_local
    # N > 1: the decode kernel's epilogue stores its heads straight into every rank's gathered buffer (peer
    # stores over NVLink, buffers from torch's symmetric-memory allocator) and one small kernel per token
    # waits for all ranks' arrivals. --nccl-gather keeps the plain NCCL all-gather after every layer instead.
    exchange = "none"
    if world > 1:
        exchange = "nccl all-gather per layer"
        if not args.nccl_gather and not args.separate and args.variant == 0:
            try:
                import torch.distributed._symmetric_memory as symm_mem
                out_full = symm_mem.empty((N_LAYER, Q_DIM), dtype=torch.float16, device=torch.device("cuda", local_rank))
                px_flags = symm_mem.empty((64,), dtype=torch.int32, device=torch.device("cuda", local_rank))
                out_full.zero_()
                px_flags.zero_()
                h_out = symm_mem.rendezvous(out_full, dist.group.WORLD)
                h_flag = symm_mem.rendezvous(px_flags, dist.group.WORLD)
                torch.cuda.synchronize()
                dist.barrier()
                ctx.set_peer_exchange(list(h_out.buffer_ptrs), list(h_flag.buffer_ptrs))
                exchange = "peer stores in the decode epilogue, ranks meet " + ("once per token" if args.sync_per_token else "after every layer")
            except Exception as e:  # no peer mapping on this box: fall back to NCCL
                print(f"[bench] symmetric memory unavailable ({type(e).__name__}: {e}); using NCCL all-gather", file=sys.stderr)
    use_px = exchange.startswith("peer")
    pos = ctx_len - 1
    stream = torch.cuda.Stream()
    launches_per_step = 0

    def one_token():
        nonlocal launches_per_step
        n = 0
        if args.separate:
            q_work.copy_(q_raw)  # q_norm_rope works in place; restore the raw activations (1 torch copy kernel)
        for il in range(N_LAYER):
            if args.separate:
                ctx.dispatch_q_norm_rope_fused(q_work[il], w, pos, 1, stream=stream)
                n += ctx.last_launch_count()
                ctx.dispatch_kv_writeback_fused(il, k_new[il], v_new[il], w, pos, 1, stream=stream)
                n += ctx.last_launch_count()
                ctx.dispatch_attention_decode(il, q_work[il], out_local[il], pos + 1, stream=stream)
                n += ctx.last_launch_count()
            else:  # the same layer step as one call (bp_attn_decode_layer)
                ctx.decode_layer(il, q_raw[il], w, k_new[il], v_new[il], w, pos, out_local[il], stream=stream)
                n += ctx.last_launch_count()
            if world > 1 and not use_px:
                dist.all_gather_into_tensor(out_full[il], out_local[il])
            if use_px and not args.sync_per_token:
                ctx.peer_sync(slot=il, stream=stream)  # the next operation of a decoder consumes this layer's gathered row
                n += 1
        if use_px and args.sync_per_token:
            ctx.peer_sync(slot=0, stream=stream)
            n += 1
        launches_per_step = n

    # Capture one token (36 dependent layers) in a CUDA graph: launch-bound otherwise.
    with torch.cuda.stream(stream):
        one_token()
        stream.synchronize()
        if use_px:
            # the gathered buffer must equal an NCCL all-gather of the ranks' local outputs
            dist.barrier()
            check = torch.zeros(N_LAYER, world, q_dim_l, dtype=torch.float16, device="cuda")
            for il in range(N_LAYER):
                dist.all_gather_into_tensor(check[il].reshape(-1), out_local[il])
            torch.cuda.synchronize()
            if not torch.equal(check.reshape(N_LAYER, Q_DIM), out_full):
                raise SystemExit("peer exchange: the gathered buffer differs from the NCCL all-gather")
            dist.barrier()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=stream):
            one_token()
    torch.cuda.synchronize()

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    with torch.cuda.stream(stream):
        for _ in range(args.warmup):
            graph.replay()
        barrier()
        sampler = ClockSampler(local_rank)
        if rank == 0:
            sampler.start()
        dt = time_region(torch, graph.replay, args.steps, stream)
        barrier()
        clocks = sampler.stop() if rank == 0 else None
    if world > 1:
        t = torch.tensor([dt], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        dt = float(t.item())
    sec_per_step = dt / args.steps
    bytes_per_step = N_LAYER * ctx_len * BYTES_PER_TOKEN_LAYER  # whole job, all ranks
    value = bytes_per_step / sec_per_step / 1e9

    # Roofline of the dominant kernel pair (split-KV pass + combine), timed alone
    # back to back over the 36 layers (340 MB of cache per sweep, larger than L2).
    def decode_only():
        for il in range(N_LAYER):
            ctx.dispatch_attention_decode(il, q_work[il], out_local[il], pos + 1, stream=stream)
    decode_graph = graphed(torch, decode_only, stream)
    with torch.cuda.stream(stream):
        for _ in range(3):
            decode_graph()
        reps = max(3, min(args.steps, 20))
        dt_k = time_region(torch, decode_graph, reps, stream) / (reps * N_LAYER)
    algo_bytes_launch = ctx_len * BYTES_PER_TOKEN_LAYER // world
    achieved = algo_bytes_launch / dt_k / 1e9
    # DRAM traffic per launch: one ncu capture of the decode kernel at ctx 32768 read 75.62 MB against
    # 75.50 MB of algorithmic bytes; reads grow in proportion to the tokens streamed, so the capture is
    # scaled by tokens. The split partials (tagged pairs, 8 bytes per value, written once and read back
    # from L2 by the merging warps) are added as written bytes.
    n_splits = ctx.decode_num_splits(pos + 1) if hasattr(ctx, "decode_num_splits") else 18
    traffic = int(75.62e6 * ctx_len / 32768 / world + n_splits * nh_l * 132 * 8) if args.variant == 0 else None
    roofline = {"bound": "hbm", "kernel": "decode_umma_kernel (splits merged in the kernel through tagged partials)", "achieved": round(achieved, 1),
                "peak": hbm_peak, "unit": "GB/s", "frac": round(achieved / hbm_peak, 4), "peak_kind": peak_kind,
                "us_per_launch": round(dt_k * 1e6, 3), "algorithmic_bytes_per_launch": algo_bytes_launch,
                "traffic": traffic, "frac_of_8000_spec": round(achieved / 8000.0, 4)}

    line = {
        "metric": "decode_attn_hbm_gbs", "value": round(value, 2), "unit": "GB/s", "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": round(sec_per_step * 1e3, 5), "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "f32 accumulate (int8 cache, f16 tensor-core operands)",
        "data": "synthetic",
        "config": {"workload": f"decode_ctx{ctx_len}_{N_LAYER}layers", "n_head": N_HEAD, "n_kv_head": N_KV_HEAD,
                   "head_dim": HEAD_DIM, "kv_cache": "Q8_0 (int8 + f32 block scales)", "bytes_per_token_layer": BYTES_PER_TOKEN_LAYER,
                   "parallelism": f"kv_head_shard{world}" if world > 1 else "single", "exchange": exchange,
                   "launch": "36 dependent layers in one CUDA graph, " + ("three dispatches per layer" if args.separate else "one bp_attn_decode_layer call per layer"), "l2": "working set 340 MB per step > 126 MB L2",
                   "us_per_layer": round(sec_per_step * 1e6 / N_LAYER, 3)},
        "roofline": roofline, "gpu_launches": launches_per_step * args.steps,
    }

    if rank == 0 and world == 1:
        # ---- e2e: host buffers through the C ABI, one call per token ----
        qh = q_raw.cpu().pin_memory(); kh = k_new.cpu().pin_memory(); vh = v_new.cpu().pin_memory()
        wh = w.cpu().pin_memory()
        oh = torch.zeros(N_LAYER, Q_DIM, dtype=torch.float16).pin_memory()
        def host_token():
            ctx.decode_token_host(qh.numpy(), kh.numpy(), vh.numpy(), wh.numpy(), wh.numpy(), pos, oh.numpy())
        for _ in range(3):
            host_token()
        e_steps = max(5, args.steps)
        t0 = time.perf_counter()
        for _ in range(e_steps):
            host_token()
        e_dt = (time.perf_counter() - t0) / e_steps
        line["e2e"] = {"value": round(bytes_per_step / e_dt / 1e9, 2), "unit": "GB/s",
                       "h2d_bytes_per_step": int(qh.numel() * 2 + kh.numel() * 2 + vh.numel() * 2 + 512),
                       "d2h_bytes_per_step": int(oh.numel() * 2), "ms_per_step": round(e_dt * 1e3, 4),
                       "call": "bp_decode_token_host (pinned host activations in, f16 outputs back, one sync per token)"}
        # ---- the other configurations, briefly ----
        if not args.no_extras:
            line["also"] = extras(torch, bp, stream, hbm_peak, tflops_peak, peak_kind, args)
        # ---- CPU baseline on this box's cores (bounded sample) ----
        if not args.no_cpu:
            try:
                g, t, th = cpu_decode_gbs(ctx_len, 4, 3)
                line["cpu_baseline"] = {"value": round(g, 4), "unit": "GB/s", "cores": th, "kind": "port",
                                        "sample": f"4 of {N_LAYER} layers at ctx {ctx_len}, best of 3 ({t*1e3:.1f} ms)"}
            except Exception as e:  # the oracle is optional for the bench
                line["cpu_baseline"] = {"value": None, "unit": "GB/s", "cores": 0, "kind": "port", "sample": f"failed: {e}"}
    if rank == 0:
        line["clocks"] = clocks
        print(json.dumps(line), flush=True)
    if world > 1:
        # The captured graphs hold NCCL work; tearing the process group down with them alive has
        # hung. Drop them, meet once more, and leave without the group's destructor.
        del graph, decode_graph
        torch.cuda.synchronize()
        dist.barrier()
        torch.cuda.synchronize()
        ctx.close()
        sys.stdout.flush()
        sys.stderr.flush()
        os._exit(0)
    ctx.close()


def prefill_bench(torch, bp, stream, tflops_peak, peak_kind, pp, nl):
    """One prefill pass per layer (Q norm+RoPE, KV write-back, causal attention) over `nl` layers."""
    gen = torch.Generator(device="cuda")
    gen.manual_seed(7 + pp)
    w = torch.ones(128, dtype=torch.float16, device="cuda")
    with bp.AttnContext(n_layer=nl, max_seq=pp) as c:
        q = torch.randn(nl, pp, Q_DIM, generator=gen, device="cuda").half()
        k = torch.randn(nl, pp, KV_DIM, generator=gen, device="cuda").half()
        v = torch.randn(nl, pp, KV_DIM, generator=gen, device="cuda").half()
        qw = q.clone()
        o = torch.zeros(nl, pp, Q_DIM, dtype=torch.float16, device="cuda")

        def full_pass():
            for il in range(nl):
                c.dispatch_q_norm_rope_fused(qw[il], w, 0, pp, stream=stream)
                c.dispatch_kv_writeback_fused(il, k[il], v[il], w, 0, pp, stream=stream)
                c.dispatch_attention(il, qw[il], o[il], pp, stream=stream)

        def attn_only():
            for il in range(nl):
                c.dispatch_attention(il, qw[il], o[il], pp, stream=stream)

        full_g, attn_g = graphed(torch, full_pass, stream), graphed(torch, attn_only, stream)
        with torch.cuda.stream(stream):
            for _ in range(3):
                full_g()
            reps = 10
            dt_full = time_region(torch, full_g, reps, stream) / (reps * nl)
            dt_attn = time_region(torch, attn_g, reps, stream) / (reps * nl)
        flops = 8192 * pp * (pp + 1)
        return {"us_per_layer_pass": round(dt_full * 1e6, 2), "us_per_layer_attention": round(dt_attn * 1e6, 2),
                "tflops_pass": round(flops / dt_full / 1e12, 2), "tflops_attention": round(flops / dt_attn / 1e12, 2),
                "frac_of_peak": round(flops / dt_attn / 1e12 / tflops_peak, 4), "peak_kind": peak_kind,
                "frac_of_2250_spec": round(flops / dt_attn / 1e12 / 2250.0, 4)}


def extras(torch, bp, stream, hbm_peak, tflops_peak, peak_kind, args):
    """Long-context decode (ctx 32768) and the prefill pass (pp 512 / 2048) on one GPU."""
    out = {}
    gen = torch.Generator(device="cuda")
    gen.manual_seed(99)
    w = torch.ones(128, dtype=torch.float16, device="cuda")
    # decode at 32K: 4 layers allocated and swept (302 MB > L2)
    nl, ctx_len = 4, 32768
    with bp.AttnContext(n_layer=nl, max_seq=ctx_len) as c:
        if args.decode_warps:
            c.set_option("decode_warps", args.decode_warps)
        if args.decode_hpc:
            c.set_option("decode_heads_per_cta", args.decode_hpc)
        if args.decode_uhpc:
            c.set_option("decode_umma_heads_per_cta", args.decode_uhpc)
        fill_cache(c, torch, nl, KV_DIM, ctx_len, gen)
        c.set_variant(args.variant)
        q = torch.randn(nl, Q_DIM, generator=gen, device="cuda").half()
        o = torch.zeros(nl, Q_DIM, dtype=torch.float16, device="cuda")
        sweeps = 9  # one graph = 36 decode calls back to back, like a token of the 36-layer stack
        def sweep():
            for _ in range(sweeps):
                for il in range(nl):
                    c.dispatch_attention_decode(il, q[il], o[il], ctx_len, stream=stream)
        sweep_g = graphed(torch, sweep, stream)
        with torch.cuda.stream(stream):
            for _ in range(3):
                sweep_g()
            dt = time_region(torch, sweep_g, 5, stream) / (5 * sweeps * nl)
        gbs = ctx_len * BYTES_PER_TOKEN_LAYER / dt / 1e9
        out["decode_ctx32768"] = {"us_per_layer": round(dt * 1e6, 2), "gbs": round(gbs, 1),
                                  "frac_of_peak": round(gbs / hbm_peak, 4), "peak_kind": peak_kind,
                                  "frac_of_8000_spec": round(gbs / 8000.0, 4), "splits": c.decode_num_splits(ctx_len)}
    for pp in (512, 2048):
        out[f"prefill_pp{pp}"] = prefill_bench(torch, bp, stream, tflops_peak, peak_kind, pp, 4)
    return out


def main():
    global N_LAYER
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--ctx", type=int, default=4096, help="context length of the decode stack")
    ap.add_argument("--layers", type=int, default=N_LAYER, help="layers of the stack (smaller only for profiler captures)")
    ap.add_argument("--decode-warps", type=int, default=0, help="override the decode kernel's compute warps per CTA")
    ap.add_argument("--decode-hpc", type=int, default=0, help="override the decode kernel's KV heads per CTA")
    ap.add_argument("--decode-uhpc", type=int, default=0, help="override the tcgen05 decode kernel's KV heads per CTA")
    ap.add_argument("--separate", action="store_true",
                    help="drive a layer with the reference's three dispatches instead of the one-call layer step")
    ap.add_argument("--separate-merge", action="store_true", help="merge the decode splits with a second kernel")
    ap.add_argument("--sync-per-token", action="store_true",
                    help="N > 1: the ranks meet once per token instead of after every layer")
    ap.add_argument("--nccl-gather", action="store_true", help="N > 1: all-gather the head outputs with NCCL after every layer")
    ap.add_argument("--decode-ring", type=int, default=0, help="override the decode kernel's ring: K stages * 16 + V slots")
    ap.add_argument("--no-pdl", action="store_true", help="launch the kernels without programmatic dependent launch")
    ap.add_argument("--variant", type=int, default=0, help="decode kernel family (0 = production)")
    ap.add_argument("--prefill-only", type=int, default=0, metavar="PP",
                    help="run only the prefill pass at this prompt length and print its JSON (profiler captures)")
    ap.add_argument("--no-extras", action="store_true", help="skip the ctx-32768 and prefill side measurements")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    args = ap.parse_args()
    N_LAYER = args.layers
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup
    if args.prefill_only:
        import torch
        import bonsai_pot_b200 as bp
        hbm_peak, tflops_peak, peak_kind = measured_peaks()
        torch.cuda.set_device(0)
        print(json.dumps(prefill_bench(torch, bp, torch.cuda.Stream(), tflops_peak, peak_kind, args.prefill_only, min(args.layers, 4))))
    elif args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
