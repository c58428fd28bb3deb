#!/usr/bin/env python
"""Benchmark of the attention hot path on B200.

Headline workload (`decode_ctx32768_36layers`): one decode token through the
36-layer decode-attention stack at context 32768 with Qwen3-8B attention shapes
(32 query heads, 8 KV heads, head_dim 128, Q8_0 KV cache; 2.7 GB of cache). One
step = for each layer: Q norm+RoPE, KV write-back of the new token at row 32767,
split-KV decode attention over 32768 keys (one bp_attn_decode_layer call). The
metric is achieved HBM GB/s = algorithmic cache bytes read (2304 B per token per
layer) / time.

  python bench.py --gpus 1 --steps 50 --warmup 5          # this implementation
  python bench.py --impl reference --steps 3 --warmup 1   # CPU restatement of the reference

With N > 1 ranks (torchrun) the KV heads are sharded over the ranks (strong
scaling: the same stack, 1/N of the heads per GPU). The all-gather of the head
outputs happens inside the decode kernel: its epilogue stores every output
element into every rank's gathered buffer (peer stores over NVLink), and the
next layer's decode kernel holds the ranks' meeting for that row (it signals
once its predecessors are complete and waits before it ends). `--exchange` selects the other
forms (a meeting kernel after every layer, one per token, or an NCCL all-gather
after every layer).

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
CPU_SAMPLE_LAYERS = 4
MIN_TIMED_SECONDS = 0.5
# DRAM bytes one decode launch at ctx 32768 read under ncu (profiles/decode_umma_kernel_ctx32768.md)
# against 75.50 MB of algorithmic bytes; reads grow in proportion to the tokens streamed.
CAPTURED_DRAM_BYTES_CTX32768 = 75.62e6


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            d = json.load(f)
        return float(d["hbm_gbs"]), float(d["bf16_tflops"]), "measured"
    except Exception:
        return FALLBACK_HBM_GBS, FALLBACK_TFLOPS, "fallback"


def workload_name(ctx_len):
    return f"decode_ctx{ctx_len}_{N_LAYER}layers"


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
# CPU side: the oracle timed as the baseline AND as the reference arm. One
# function, one set of inputs: both report the same measurement.
# ----------------------------------------------------------------------------
_CPU = {}


def cpu_sample(ctx_len):
    """One pass of the CPU restatement over CPU_SAMPLE_LAYERS layers of the workload: per layer
    q_norm_rope, kv_writeback at the last row, attention_split + attention_merge over ctx_len keys.
    All host cores (the thread count is set explicitly: a launcher's OMP_NUM_THREADS=1 does not apply).
    Returns (seconds, threads)."""
    import numpy as np
    from bonsai_pot_b200 import synth
    from oracle import oracle as O
    if "native" not in _CPU:
        try:
            O.lib(native=True)
            _CPU["native"] = True
        except Exception:
            _CPU["native"] = False
        O.set_threads(os.cpu_count() or 1, native=_CPU["native"])
    native = _CPU["native"]
    if ctx_len not in _CPU:
        nl = CPU_SAMPLE_LAYERS
        sh = O.Shape(n_layer=nl, n_head=N_HEAD, n_kv_head=N_KV_HEAD, max_seq=ctx_len)
        kv_k, kv_v = sh.new_cache(), sh.new_cache()
        rng = np.random.default_rng(0)
        # cache content does not change the CPU time: plain random quants and small positive scales
        for kv in (kv_k, kv_v):
            kv[:sh.d_total].view(np.float32)[:] = rng.random(sh.d_total // 4, dtype=np.float32) * 0.03
            kv[sh.d_total:] = rng.integers(0, 256, size=kv.size - sh.d_total, dtype=np.uint8)
        q = [synth.tensor(0, 3, il, synth.T_Q, (1, sh.q_dim)) for il in range(nl)]
        k = [synth.tensor(0, 3, il, synth.T_K_NEW, (1, sh.kv_dim)) for il in range(nl)]
        v = [synth.tensor(0, 3, il, synth.T_V_NEW, (1, sh.kv_dim)) for il in range(nl)]
        _CPU[ctx_len] = (sh, kv_k, kv_v, q, k, v, O.rope_table_f16(sh), synth.ones_weight())
    sh, kv_k, kv_v, q, k, v, rope, w = _CPU[ctx_len]
    t0 = time.perf_counter()
    for il in range(sh.n_layer):
        qn = O.q_norm_rope(sh, q[il], w, rope, ctx_len - 1, 1, native=native)
        O.kv_writeback(sh, k[il], v[il], w, rope, kv_k, kv_v, il, ctx_len - 1, 1, native=native)
        O.attn_decode(sh, qn, kv_k, kv_v, il, ctx_len, native=native)
    return time.perf_counter() - t0, O.num_threads(native)


def cpu_gbs(ctx_len, seconds):
    return CPU_SAMPLE_LAYERS * ctx_len * BYTES_PER_TOKEN_LAYER / seconds / 1e9


def cpu_sample_text(ctx_len):
    return (f"{CPU_SAMPLE_LAYERS} of {N_LAYER} layers of the decode stack at ctx {ctx_len} per step "
            "(q_norm_rope + kv_writeback + attention_split/merge per layer)")


def run_reference(args):
    """Reference arm: the reference's own engine (Rust + wgpu/Vulkan) cannot be built or run on this
    machine, so its CPU restatement (the oracle) is timed on the host cores with all threads, on the
    same workload and metric. Each step is a bounded sample (CPU_SAMPLE_LAYERS layers)."""
    if int(os.environ.get("RANK", "0")) != 0:
        return
    times, threads = [], 1
    for i in range(args.warmup + args.steps):
        dt, threads = cpu_sample(args.ctx)
        if i >= args.warmup:
            times.append(dt)
    dt = statistics.mean(times)
    gbs = cpu_gbs(args.ctx, dt)
    line = {
        "impl": "reference", "metric": "decode_attn_hbm_gbs", "value": round(gbs, 4), "unit": "GB/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(dt * 1e3, 3),
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": workload_name(args.ctx), "n_head": N_HEAD, "n_kv_head": N_KV_HEAD,
                   "head_dim": HEAD_DIM, "kv_cache": "Q8_0 (int8 + f32 block scales)"},
        "cpu_baseline": {"value": round(gbs, 4), "unit": "GB/s", "cores": threads, "kind": "port",
                         "sample": cpu_sample_text(args.ctx)},
        "e2e": {"value": round(gbs, 4), "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
        "note": "CPU restatement of the reference's WGSL math (the Rust/wgpu reference itself is unavailable on this box)",
    }
    print(json.dumps(line), flush=True)


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


def time_blocks(torch, fn, steps, stream, min_seconds=MIN_TIMED_SECONDS, max_blocks=400, n_blocks=None):
    """Times blocks of exactly `steps` calls of fn each with CUDA events on `stream`, back to back, until
    the region is at least min_seconds long (the block count comes from a first block, or from
    n_blocks). Returns (median seconds per block, blocks, seconds of the whole region)."""
    def block():
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record(stream)
        for _ in range(steps):
            fn()
        b.record(stream)
        return a, b
    torch.cuda.synchronize()
    if n_blocks is None:
        a, b = block()
        torch.cuda.synchronize()
        first = max(a.elapsed_time(b) / 1e3, 1e-6)
        n_blocks = int(min(max_blocks, max(3, -(-min_seconds // first))))
    evs = [block() for _ in range(n_blocks)]
    torch.cuda.synchronize()
    times = [a.elapsed_time(b) / 1e3 for a, b in evs]
    return statistics.median(times), n_blocks, sum(times)


def make_context(bp, args, n_layer, nh_l, nkv_l, ctx_len, world, rank, device):
    ctx = bp.AttnContext(n_layer=n_layer, n_head=nh_l, n_kv_head=nkv_l, max_seq=ctx_len, n_shards=world, shard=rank,
                         device=device, max_prefill=min(ctx_len, 2048))
    for name, value in (("decode_warps", args.decode_warps), ("decode_heads_per_cta", args.decode_hpc),
                        ("decode_umma_heads_per_cta", args.decode_uhpc), ("decode_ring", args.decode_ring)):
        if value:
            ctx.set_option(name, value)
    if args.no_pdl:
        ctx.set_option("dependent_launch", 0)
    if args.separate_merge:
        ctx.set_option("decode_in_kernel_merge", 0)
    if args.l2_promotion:
        ctx.set_option("tma_l2_promotion", args.l2_promotion)
    if args.no_v_preload:
        ctx.set_option("decode_v_preload", 0)
    return ctx


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

    ctx = make_context(bp, args, N_LAYER, nh_l, nkv_l, ctx_len, world, rank, local_rank)
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
    # N > 1: the gathered buffers and the meeting counters come from torch's symmetric-memory allocator
    # (peer-mapped over NVLink); the decode kernel stores into every rank's buffer itself.
    mode = args.exchange if world > 1 else "none"
    if world > 1 and (args.separate or args.variant != 0) and mode != "nccl":
        mode = "nccl"  # the exchange lives in the tcgen05 decode kernel
    if world > 1 and mode != "nccl":
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
            out_ptrs, flag_ptrs = list(h_out.buffer_ptrs), list(h_flag.buffer_ptrs)
        except Exception as e:  # no peer mapping on this box: fall back to NCCL
            print(f"[bench] symmetric memory unavailable ({type(e).__name__}: {e}); using NCCL all-gather", file=sys.stderr)
            mode = "nccl"
    exchange_text = {
        "none": "none",
        "kernel": "peer stores in the decode epilogue; the next layer's decode kernel holds the meeting (signal at its start, wait before its end), one meeting kernel per token for the last layer",
        "sync-kernel": "peer stores in the decode epilogue; a meeting kernel after every layer",
        "per-token": "peer stores in the decode epilogue; one meeting kernel per token",
        "nccl": "nccl all-gather per layer",
    }[mode]
    use_px = mode in ("kernel", "sync-kernel", "per-token")

    def exchange_on(on):
        if not use_px:
            return
        if on:
            ctx.set_peer_exchange(out_ptrs, flag_ptrs)
            ctx.set_option("peer_meet_in_kernel", 1 if mode == "kernel" else 0)
        else:
            ctx.set_peer_exchange([], [])
    exchange_on(True)
    pos = ctx_len - 1
    stream = torch.cuda.Stream()
    launches_per_step = 0
    last_slot = (N_LAYER - 1) % 64

    def one_token(exchange=True):
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
            if not exchange:
                continue
            if mode == "nccl":
                dist.all_gather_into_tensor(out_full[il], out_local[il])
            elif mode == "sync-kernel":
                ctx.peer_sync(slot=il % 64, stream=stream)  # the next operation of a decoder consumes this layer's gathered row
                n += 1
        if exchange and mode == "per-token":
            ctx.peer_sync(slot=0, stream=stream)
            n += 1
        if exchange and mode == "kernel":
            ctx.peer_sync(slot=last_slot, stream=stream)  # the last layer's row has no next layer to meet in
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

    def agree(value, op):  # one number for all ranks
        if world == 1:
            return value
        t = torch.tensor([float(value)], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=op)
        return float(t.item())

    with torch.cuda.stream(stream):
        for _ in range(args.warmup):
            graph.replay()
        barrier()
        # every rank must run the same number of blocks: the ranks wait for one another in every layer
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record(stream)
        for _ in range(args.steps):
            graph.replay()
        b.record(stream)
        torch.cuda.synchronize()
        first = agree(a.elapsed_time(b) / 1e3, dist.ReduceOp.MAX if world > 1 else None)
        n_blocks = int(min(400, max(3, -(-MIN_TIMED_SECONDS // max(first, 1e-6)))))
        barrier()
        sampler = ClockSampler(local_rank)
        if rank == 0:
            sampler.start()
        dt, n_blocks, region = time_blocks(torch, graph.replay, args.steps, stream, n_blocks=n_blocks)
        barrier()
        clocks = sampler.stop() if rank == 0 else None
    dt = agree(dt, dist.ReduceOp.MAX if world > 1 else None)
    sec_per_step = dt / args.steps
    bytes_per_step = N_LAYER * ctx_len * BYTES_PER_TOKEN_LAYER  # whole job, all ranks
    value = bytes_per_step / sec_per_step / 1e9

    # Multi-GPU: what the exchange costs. Compute only = the same stack with the exchange switched off
    # (no peer stores, no meeting); meeting only = 36 meeting kernels (signal + wait) and nothing else.
    scaling_detail = None
    if world > 1 and use_px:
        exchange_on(False)
        compute_g = graphed(torch, lambda: one_token(exchange=False), stream)
        exchange_on(True)

        def meetings():
            for il in range(N_LAYER):
                ctx.peer_sync(slot=il % 64, stream=stream)
        meet_g = graphed(torch, meetings, stream)
        with torch.cuda.stream(stream):
            barrier()
            for _ in range(3):
                compute_g()
            t_c, _, _ = time_blocks(torch, compute_g, args.steps, stream, n_blocks=5)
            barrier()
            for _ in range(3):
                meet_g()
            t_m, _, _ = time_blocks(torch, meet_g, args.steps, stream, n_blocks=5)
            barrier()
        t_c, t_m = agree(t_c, dist.ReduceOp.MAX), agree(t_m, dist.ReduceOp.MAX)
        scaling_detail = {"us_per_layer_with_exchange": round(sec_per_step * 1e6 / N_LAYER, 3),
                          "us_per_layer_compute_only": round(t_c / args.steps * 1e6 / N_LAYER, 3),
                          "us_per_meeting_kernel_alone": round(t_m / args.steps * 1e6 / N_LAYER, 3)}
        del compute_g, meet_g

    # Roofline of the dominant kernel (the decode kernel, splits merged inside it), timed alone back to
    # back over the 36 layers (each layer's cache is larger than what L2 keeps of it between sweeps).
    exchange_on(False)

    def decode_only():
        for il in range(N_LAYER):
            ctx.dispatch_attention_decode(il, q_work[il], out_local[il], pos + 1, stream=stream)
    decode_graph = graphed(torch, decode_only, stream)
    with torch.cuda.stream(stream):
        for _ in range(3):
            decode_graph()
        dt_k, _, _ = time_blocks(torch, decode_graph, 5, stream, n_blocks=5)
        dt_k /= 5 * N_LAYER
    exchange_on(True)
    algo_bytes_launch = ctx_len * BYTES_PER_TOKEN_LAYER // world
    achieved = algo_bytes_launch / dt_k / 1e9
    n_splits = ctx.decode_num_splits(pos + 1)
    # the tagged split partials (8 bytes per value, written once, read back from L2) are added as written bytes
    traffic = int(CAPTURED_DRAM_BYTES_CTX32768 * ctx_len / 32768 / world + n_splits * nh_l * 132 * 8) if args.variant == 0 else None
    roofline = {"bound": "hbm", "kernel": "decode_umma_kernel (splits merged in the kernel through tagged partials)",
                "achieved": round(achieved, 1), "peak": hbm_peak, "unit": "GB/s", "frac": round(achieved / hbm_peak, 4),
                "peak_kind": peak_kind, "us_per_launch": round(dt_k * 1e6, 3),
                "algorithmic_bytes_per_launch": algo_bytes_launch, "traffic": traffic,
                "traffic_source": "dram__bytes_read+write of one ncu capture of this kernel at ctx 32768 "
                                  "(profiles/decode_umma_kernel_ctx32768.md), scaled by the tokens of a launch",
                "frac_of_8000_spec": round(achieved / 8000.0, 4), "splits": n_splits}

    mb_step = bytes_per_step / 1e6
    line = {
        "metric": "decode_attn_hbm_gbs", "value": round(value, 2), "unit": "GB/s", "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": round(sec_per_step * 1e3, 5), "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": workload_name(ctx_len), "n_head": N_HEAD, "n_kv_head": N_KV_HEAD,
                   "head_dim": HEAD_DIM, "kv_cache": "Q8_0 (int8 + f32 block scales)", "bytes_per_token_layer": BYTES_PER_TOKEN_LAYER,
                   "arithmetic": "int8 tensor-core products (exact), f32 scales / softmax / accumulation, f16 in and out",
                   "parallelism": f"kv_head_shard{world}" if world > 1 else "single", "exchange": exchange_text,
                   "launch": f"{N_LAYER} dependent layers in one CUDA graph, " +
                             ("three dispatches per layer" if args.separate else "one bp_attn_decode_layer call per layer"),
                   "l2": f"working set {mb_step:.0f} MB per step > 126 MB L2",
                   "timing": f"median of {n_blocks} blocks of {args.steps} steps, {region:.2f} s timed",
                   "us_per_layer": round(sec_per_step * 1e6 / N_LAYER, 3)},
        "roofline": roofline, "gpu_launches": launches_per_step * args.steps * n_blocks,
    }
    if scaling_detail:
        line["exchange_cost"] = scaling_detail

    # ---- e2e: host buffers through the C ABI, one bp_decode_token_host call per token ----
    qh = q_raw.cpu().pin_memory(); kh = k_new.cpu().pin_memory(); vh = v_new.cpu().pin_memory()
    wh = w.cpu().pin_memory()
    oh = torch.zeros(N_LAYER, q_dim_l, dtype=torch.float16).pin_memory()
    gh = torch.zeros(N_LAYER, Q_DIM, dtype=torch.float16).pin_memory() if use_px else None

    def host_token(at):
        ctx.decode_token_host(qh.numpy(), kh.numpy(), vh.numpy(), wh.numpy(), wh.numpy(), at, oh.numpy())
        if use_px:
            # the gathered rows of all ranks, once every rank's stores have landed
            with torch.cuda.stream(stream):
                ctx.peer_sync(slot=last_slot if mode == "kernel" else 0, stream=stream)
                gh.copy_(out_full, non_blocking=True)
            stream.synchronize()
    if mode != "nccl":  # (the host entry point has no per-layer meeting kernel: the ranks meet once per token)
        # Successive positions, as a generation loop asks for them, ending at the benchmark's context length
        # (the library prepares its launches for the next position while the device works on the current one).
        e_steps = max(5, args.steps)
        first = max(0, pos - (e_steps + 3 - 1))
        at = [min(pos, first + i) for i in range(e_steps + 3)]
        barrier()
        for i in range(3):
            host_token(at[i])
        barrier()
        t0 = time.perf_counter()
        for i in range(e_steps):
            host_token(at[3 + i])
        e_dt = agree((time.perf_counter() - t0) / e_steps, dist.ReduceOp.MAX if world > 1 else None)
        e_keys = sum(a + 1 for a in at[3:]) / e_steps  # keys attended per layer, mean over the timed tokens
        line["e2e"] = {"value": round(N_LAYER * e_keys * BYTES_PER_TOKEN_LAYER / e_dt / 1e9, 2), "unit": "GB/s",
                       "h2d_bytes_per_step": int(qh.numel() * 2 + kh.numel() * 2 + vh.numel() * 2 + 512) * world,
                       "d2h_bytes_per_step": int(oh.numel() * 2 + (gh.numel() * 2 if gh is not None else 0)) * world,
                       "ms_per_step": round(e_dt * 1e3, 4),
                       "positions": f"{at[3]} .. {at[-1]}",
                       "call": "bp_decode_token_host (pinned host activations in, f16 outputs back, one sync per token)" +
                               ("; then the meeting and the gathered rows back to the host, on every rank" if use_px else "")}
    if rank == 0 and world == 1:
        # ---- the other configurations, briefly ----
        if not args.no_extras:
            line["also"] = extras(torch, bp, stream, hbm_peak, tflops_peak, peak_kind, args)
        # ---- CPU baseline on this box's cores (bounded sample; the reference arm runs the same function) ----
        if not args.no_cpu:
            try:
                cpu_sample(ctx_len)  # builds the inputs, warms the cores
                times = []
                for _ in range(3):
                    t, th = cpu_sample(ctx_len)
                    times.append(t)
                t = statistics.mean(times)
                line["cpu_baseline"] = {"value": round(cpu_gbs(ctx_len, t), 4), "unit": "GB/s", "cores": th, "kind": "port",
                                        "sample": cpu_sample_text(ctx_len) + f", mean of 3 ({t*1e3:.1f} ms)"}
            except Exception as e:  # the oracle is optional for the bench
                line["cpu_baseline"] = {"value": None, "unit": "GB/s", "cores": 0, "kind": "port", "sample": f"failed: {e}"}
    if world > 1 and not args.no_extras and use_px:
        pf = prefill_exchange_bench(torch, dist, bp, stream, args, world, rank, local_rank, tflops_peak, peak_kind)
        if rank == 0:
            line["also"] = {"prefill_pp2048_sharded": pf}
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
            dt_full, _, _ = time_blocks(torch, full_g, 10, stream, n_blocks=5)
            dt_attn, _, _ = time_blocks(torch, attn_g, 10, stream, n_blocks=5)
        dt_full /= 10 * nl
        dt_attn /= 10 * nl
        flops = 8192 * pp * (pp + 1)
        return {"us_per_layer_pass": round(dt_full * 1e6, 2), "us_per_layer_attention": round(dt_attn * 1e6, 2),
                "tflops_pass": round(flops / dt_full / 1e12, 2), "tflops_attention": round(flops / dt_attn / 1e12, 2),
                "frac_of_peak": round(flops / dt_attn / 1e12 / tflops_peak, 4), "peak_kind": peak_kind,
                "frac_of_2250_spec": round(flops / dt_attn / 1e12 / 2250.0, 4)}


def prefill_exchange_bench(torch, dist, bp, stream, args, world, rank, local_rank, tflops_peak, peak_kind):
    """Batched prefill at pp 2048 on KV-head shards: every rank's kernel stores its heads' outputs into
    every rank's gathered buffer (bp_set_prefill_exchange), the ranks meet once per layer."""
    import torch.distributed._symmetric_memory as symm_mem
    pp, nl = 2048, 4
    nkv_l, nh_l = N_KV_HEAD // world, N_HEAD // world
    gen = torch.Generator(device="cuda")
    gen.manual_seed(70 + rank)
    w = torch.ones(128, dtype=torch.float16, device="cuda")
    gathered = symm_mem.empty((pp, Q_DIM), dtype=torch.float16, device=torch.device("cuda", local_rank))
    flags = symm_mem.empty((64,), dtype=torch.int32, device=torch.device("cuda", local_rank))
    gathered.zero_()
    flags.zero_()
    h_g, h_f = symm_mem.rendezvous(gathered, dist.group.WORLD), symm_mem.rendezvous(flags, dist.group.WORLD)
    torch.cuda.synchronize()
    dist.barrier()
    with bp.AttnContext(n_layer=nl, n_head=nh_l, n_kv_head=nkv_l, max_seq=pp, n_shards=world, shard=rank,
                        device=local_rank) as c:
        q = torch.randn(nl, pp, nh_l * HEAD_DIM, generator=gen, device="cuda").half()
        k = torch.randn(nl, pp, nkv_l * HEAD_DIM, generator=gen, device="cuda").half()
        v = torch.randn(nl, pp, nkv_l * HEAD_DIM, generator=gen, device="cuda").half()
        o = torch.zeros(nl, pp, nh_l * HEAD_DIM, dtype=torch.float16, device="cuda")
        for il in range(nl):
            c.dispatch_q_norm_rope_fused(q[il], w, 0, pp, stream=stream)
            c.dispatch_kv_writeback_fused(il, k[il], v[il], w, 0, pp, stream=stream)
        torch.cuda.synchronize()

        def attn(exchange):
            for il in range(nl):
                c.dispatch_attention(il, q[il], o[il], pp, stream=stream)
                if exchange:
                    c.peer_sync(slot=il, stream=stream)
        res = {}
        for name, exchange in (("compute_only", False), ("with_exchange", True)):
            if exchange:
                c.set_peer_exchange([0] * world, list(h_f.buffer_ptrs))  # meeting counters only: decode is not run here
                c.set_prefill_exchange(list(h_g.buffer_ptrs))
            g = graphed(torch, lambda: attn(exchange), stream)
            with torch.cuda.stream(stream):
                dist.barrier()
                torch.cuda.synchronize()
                for _ in range(3):
                    g()
                dt, _, _ = time_blocks(torch, g, 5, stream, n_blocks=5)
                dist.barrier()
                torch.cuda.synchronize()
            t = torch.tensor([dt / (5 * nl)], device="cuda", dtype=torch.float64)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            res[name] = float(t.item())
            del g
        if not torch.equal(gathered[:, rank * nh_l * HEAD_DIM:(rank + 1) * nh_l * HEAD_DIM], o[nl - 1]):
            raise SystemExit("prefill exchange: this rank's columns of the gathered buffer differ from its local output")
        c.set_prefill_exchange([])
        c.set_peer_exchange([], [])
    flops = 8192 * pp * (pp + 1)  # whole job, all ranks
    return {"us_per_layer_compute_only": round(res["compute_only"] * 1e6, 2),
            "us_per_layer_with_exchange": round(res["with_exchange"] * 1e6, 2),
            "tflops_whole_job": round(flops / res["with_exchange"] / 1e12, 2),
            "frac_of_peak_per_gpu": round(flops / res["with_exchange"] / 1e12 / world / tflops_peak, 4), "peak_kind": peak_kind,
            "exchange": "peer stores in the prefill epilogue, one meeting kernel per layer"}


def extras(torch, bp, stream, hbm_peak, tflops_peak, peak_kind, args):
    """The 36-layer decode stack at ctx 4096 (BASELINE config 1) and the prefill pass (pp 512 / 2048) on one GPU."""
    out = {}
    gen = torch.Generator(device="cuda")
    gen.manual_seed(99)
    w = torch.ones(128, dtype=torch.float16, device="cuda")
    nl, ctx_len = N_LAYER, 4096
    if args.ctx != ctx_len:
        with make_context(bp, args, nl, N_HEAD, N_KV_HEAD, ctx_len, 1, 0, torch.cuda.current_device()) as c:
            fill_cache(c, torch, nl, KV_DIM, ctx_len - 1, gen)
            c.set_variant(args.variant)
            q = torch.randn(nl, Q_DIM, generator=gen, device="cuda").half()
            k = torch.randn(nl, KV_DIM, generator=gen, device="cuda").half()
            v = torch.randn(nl, KV_DIM, generator=gen, device="cuda").half()
            o = torch.zeros(nl, Q_DIM, dtype=torch.float16, device="cuda")

            def token():
                for il in range(nl):
                    c.decode_layer(il, q[il], w, k[il], v[il], w, ctx_len - 1, o[il], stream=stream)

            def kernel_only():
                for il in range(nl):
                    c.dispatch_attention_decode(il, q[il], o[il], ctx_len, stream=stream)
            token_g, kernel_g = graphed(torch, token, stream), graphed(torch, kernel_only, stream)
            with torch.cuda.stream(stream):
                for _ in range(3):
                    token_g()
                dt, _, _ = time_blocks(torch, token_g, 20, stream, n_blocks=5)
                dt_k, _, _ = time_blocks(torch, kernel_g, 20, stream, n_blocks=5)
            dt /= 20 * nl
            dt_k /= 20 * nl
            gbs = ctx_len * BYTES_PER_TOKEN_LAYER / dt / 1e9
            out[workload_name(ctx_len)] = {
                "us_per_layer": round(dt * 1e6, 3), "gbs": round(gbs, 1), "frac_of_peak": round(gbs / hbm_peak, 4),
                "peak_kind": peak_kind, "us_per_decode_kernel": round(dt_k * 1e6, 3),
                "kernel_frac_of_peak": round(ctx_len * BYTES_PER_TOKEN_LAYER / dt_k / 1e9 / hbm_peak, 4),
                "splits": c.decode_num_splits(ctx_len)}
    for pp in (512, 2048):
        out[f"prefill_pp{pp}"] = prefill_bench(torch, bp, stream, tflops_peak, peak_kind, pp, 4)
    try:
        out["e2e_bonsai8b_pp512_tg128"] = engine_bench(torch, bp)
    except Exception as e:  # a side measurement: it must not take the headline down
        out["e2e_bonsai8b_pp512_tg128"] = {"failed": f"{type(e).__name__}: {e}"}
    return out


def engine_bench(torch, bp, n_tokens=128, reps=3):
    """BASELINE config 4: a Bonsai-8B-shaped random-init model (Q1_0 signs Bernoulli(0.5), f16 block scales
    |N(0, 0.02)|, norms 1.0) written to a temporary model directory, loaded, prefilled with 512 tokens through
    the batched path and decoded greedily for 128 tokens through Session::generate, this library's attention
    inside. Tokens per second, whole engine (the CPU restatement of this size is hours of CPU time: the
    bit-for-bit comparison with it runs in the tests, at these widths on two layers and end to end on a small model)."""
    import shutil
    import tempfile
    import numpy as np
    from bonsai_pot_b200 import model_dir
    d = tempfile.mkdtemp(prefix="bonsai8b_synth_")
    try:
        model_dir.write_synthetic_model(d, shape=model_dir.BONSAI_8B, seed=1)
        with bp.Model(d, max_seq=1024) as m:
            prompt = np.random.default_rng(0).integers(0, model_dir.BONSAI_8B["n_vocab"], 512).tolist()
            greedy = bp.Sampler(temperature=0.0)
            sess = m.new_session()
            best_pp, best_tg, toks = None, None, None
            for _ in range(reps):
                sess.reset()
                torch.cuda.synchronize()
                t0 = time.perf_counter()
                first = sess.prefill(prompt, greedy)
                t_pp = time.perf_counter() - t0
                t0 = time.perf_counter()
                toks, _reason = sess.generate(first, bp.GenerateOptions(max_new_tokens=n_tokens, stop_pred=lambda _t: False, sampler=greedy))
                t_tg = time.perf_counter() - t0
                best_pp = t_pp if best_pp is None else min(best_pp, t_pp)
                best_tg = t_tg if best_tg is None else min(best_tg, t_tg)
            weights_mb = sum(os.path.getsize(os.path.join(d, f)) for f in os.listdir(d) if f.endswith(".bin")) / 1e6
        return {"pp512_tok_s": round(512 / best_pp, 1), "tg128_tok_s": round(n_tokens / best_tg, 1), "pp512_ms": round(best_pp * 1e3, 2),
                "tg128_ms_per_token": round(best_tg * 1e3 / n_tokens, 3), "generated_tokens": n_tokens, "weights_mb": round(weights_mb, 1), "tokens_emitted": len(toks),
                "weight_stream_gbs_decode": round(weights_mb / 1e3 / (best_tg / n_tokens), 1),
                "note": "whole engine through Session::prefill + Session::generate, host loop and sampling included"}
    finally:
        shutil.rmtree(d, ignore_errors=True)


def main():
    global N_LAYER
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--ctx", type=int, default=32768, help="context length of the decode stack")
    ap.add_argument("--layers", type=int, default=N_LAYER, help="layers of the stack (smaller only for profiler captures)")
    ap.add_argument("--decode-warps", type=int, default=0, help="override the decode kernel's compute warps per CTA")
    ap.add_argument("--decode-hpc", type=int, default=0, help="override the decode kernel's KV heads per CTA")
    ap.add_argument("--decode-uhpc", type=int, default=0, help="override the tcgen05 decode kernel's KV heads per CTA")
    ap.add_argument("--separate", action="store_true",
                    help="drive a layer with the reference's three dispatches instead of the one-call layer step")
    ap.add_argument("--separate-merge", action="store_true", help="merge the decode splits with a second kernel")
    ap.add_argument("--exchange", default="kernel", choices=["kernel", "sync-kernel", "per-token", "nccl"],
                    help="N > 1: how the ranks' head outputs are gathered (see the module docstring)")
    ap.add_argument("--decode-ring", type=int, default=0, help="override the decode kernel's ring: K stages * 16 + V slots")
    ap.add_argument("--l2-promotion", type=int, default=0, help="L2 promotion of the cache tensor maps: 0 = 256 B, 1 = 128 B, 2 = 64 B, 3 = none")
    ap.add_argument("--no-v-preload", action="store_true", help="request V tiles only when their job starts")
    ap.add_argument("--no-pdl", action="store_true", help="launch the kernels without programmatic dependent launch")
    ap.add_argument("--variant", type=int, default=0, help="decode kernel family (0 = production)")
    ap.add_argument("--prefill-only", type=int, default=0, metavar="PP",
                    help="run only the prefill pass at this prompt length and print its JSON (profiler captures)")
    ap.add_argument("--engine-only", type=int, default=0, metavar="TOKENS",
                    help="run only the whole-engine side measurement (512-token prefill, then this many generated tokens, "
                         "once) and print its JSON (profiler captures)")
    ap.add_argument("--no-extras", action="store_true", help="skip the ctx-4096 and prefill side measurements")
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
    elif args.engine_only:
        import torch
        import bonsai_pot_b200 as bp
        torch.cuda.set_device(0)
        print(json.dumps(engine_bench(torch, bp, n_tokens=args.engine_only, reps=1)))
    elif args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
