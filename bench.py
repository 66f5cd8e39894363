#!/usr/bin/env python3
"""Benchmark of the KV-cache hot path: quantized-KV decode attention at 128K context.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
                    [--workload decode128k|batch64|splitctx|appendsweep|prefill|pq2] [--mode planar4] [--ctx 131072]

A step is one decode token of one sequence through all 16 full-attention layers: per layer
one fused append (IMROPE + quantize + store of the new K/V rows) and one split-K decode
attention over the whole cache.  The default workload is the configuration the headline
metric is quoted on: planar4 cache, 24 q / 4 kv heads, head_dim 256, context 131072, batch 1,
seeded N(0,1) K/V with 1 % of the channels scaled x20.  Every step reads 16 x 138 MB of cache,
far more than the 126 MB L2, so no separate L2 flush is needed.

With N > 1 (torchrun, one rank per GPU) every rank decodes its own independent sequence of
the same shape: sequences shard across GPUs with no collective on the data path (weak
scaling); torch.distributed is used only for the barrier and the max over ranks.  After the
headline pass the same process group also runs the two configurations that shard ONE job over
the GPUs - 64 sequences split over the ranks, and one 262144-token sequence cut into context
chunks whose partial results meet through peer memory - for a few steps each and reports them
under `sharded` (with each one's own 1-GPU time measured on rank 0 in the same run, and a
small split-context self-check against a whole cache).  The split-context step is timed in two
forms: every layer's exchange completed before the next layer starts (what a model needs, the
headline of that workload), and all 16 layers scanned first with one exchange per token
(`layers_batched`, for callers whose layers do not depend on one another).

Prints one JSON line.  `value` is device-resident throughput (CUDA events on the library's
stream, max over ranks), `e2e` the same step through the host-buffer entry point
(bk_attn_step_host: pinned staging, H2D of q/k/v and D2H of the output inside the timed
region), `roofline` the decode kernel's algorithmic bytes / its measured launch time against
the measured HBM copy bandwidth, `cpu_baseline` the CPU oracle on a bounded sample.
"""
import argparse
import importlib
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))

NH, NKV, HD = 24, 4, 256
N_LAYERS = 16  # --layers overrides it for small profiling runs
FALLBACK_HBM_GBS = 6650.0


class Mode:
    """BONSAI_KV mode string -> (kind, bits, v_quant), the reference's table (src/kvquant.rs:515-543).
    Used by the reference arm, which must not load the CUDA library."""
    def __init__(self, text):
        t = text or ""
        self.kind, self.bits, self.v_quant = "f32", 0, False
        if t in ("f16", "fp16", "half"):
            self.kind = "f16"
            return
        k_only = t.endswith("k")
        body = t[:-1] if k_only else t
        for prefix in ("planar", "iso"):
            if body.startswith(prefix) and body[len(prefix):].isdigit() and 1 <= int(body[len(prefix):]) <= 8:
                self.kind, self.bits, self.v_quant = "planar", int(body[len(prefix):]), not k_only


def row_bytes(mode):
    if mode.kind == "f32":
        return 1024, 1024
    if mode.kind == "f16":
        return 512, 512
    k = 32 * mode.bits + 4
    return k, (k if mode.v_quant else 1024)


def attn_bytes(mode, n_pos):
    """Algorithmic bytes of one decode-attention launch: every cache byte once, q in, out out."""
    rk, rv = row_bytes(mode)
    return n_pos * NKV * (rk + rv) + 2 * NH * HD * 4


def append_bytes(mode, n_tok=1):
    rk, rv = row_bytes(mode)
    return n_tok * (2 * NKV * HD * 4 + NKV * (rk + rv))


def measured_peak():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except Exception:
        return FALLBACK_HBM_GBS, "fallback"


def synth_chunk(rng, n, channels):
    """N(0,1) K/V rows, the seeded outlier channels scaled x20."""
    k = rng.standard_normal((n, NKV, HD), dtype=np.float32)
    v = rng.standard_normal((n, NKV, HD), dtype=np.float32)
    k[:, :, channels] *= np.float32(20.0)
    v[:, :, channels] *= np.float32(20.0)
    return k, v


class ClockSampler:
    """nvidia-smi clocks and throttle reasons sampled every 50 ms while the timed region (and the per-launch pass after it) runs."""
    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, device):
        self.device, self.rows, self.proc = device, [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--id={self.device}", f"--query-gpu={self.FIELDS}",
                                          "--format=csv,noheader,nounits", "-lms", "50"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.25)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in self.rows:
            try:
                sm.append(float(r[0])); mx.append(float(r[1]))
            except Exception:
                continue
            for name, val in zip(names, r[2:6]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def dist_setup(n_gpus, need_nccl=False):
    """Returns (rank, world, local_rank, torch.distributed or None)."""
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if world <= 1:
        return 0, 1, 0, None
    import torch
    import torch.distributed as dist
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    # Workloads without a collective on the data path need torch.distributed only for the barrier
    # and the max over ranks; gloo does that without NCCL's helper threads, which cost the
    # host-buffer (e2e) path about 10 % when they share the cores.  NCCL is used when asked for
    # (BONSAI_BENCH_BACKEND=nccl), when the workload exchanges data through it, or if gloo fails.
    want = os.environ.get("BONSAI_BENCH_BACKEND", "nccl" if need_nccl else "gloo")
    if want == "gloo":
        os.environ.setdefault("GLOO_SOCKET_IFNAME", "lo")
        try:
            dist.init_process_group("gloo")
            return dist.get_rank(), world, local, dist
        except Exception as e:  # fall back rather than lose the run
            print(f"gloo rendezvous failed ({e}); using nccl", file=sys.stderr)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    return dist.get_rank(), world, local, dist


def max_over_ranks(dist, local, value):
    if dist is None:
        return value
    import torch
    dev = "cpu" if dist.get_backend() == "gloo" else f"cuda:{local}"
    t = torch.tensor([value], dtype=torch.float64, device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def barrier(dist):
    if dist is not None:
        dist.barrier()


# ---------------------------------------------------------------------------------------------
# reference arm: the reference's own CPU path (the C restatement; the Rust crate cannot be
# built here) on the host cores
# ---------------------------------------------------------------------------------------------

def cpu_fill(oracle, mode_tuple, chunks, n_pos):
    ref = oracle.cache(*mode_tuple)
    p = 0
    for k, v in chunks:
        for i in range(k.shape[0]):
            if p >= n_pos:
                return ref
            ref.append(0, k[i], v[i], p)
            p += 1
    return ref


def cpu_layer_step(ref, q, k, v, pos, threads):
    t0 = time.perf_counter()
    ref.step(0, q, k, v, pos, threads=threads)
    return time.perf_counter() - t0


def run_reference(args, mode, chunks_fn):
    from oracle_lib import MODE_F16, MODE_F32, MODE_PLANAR, load_oracle
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    oracle = load_oracle()
    kind = {"f32": MODE_F32, "f16": MODE_F16, "planar": MODE_PLANAR}[mode.kind]
    threads = oracle.lib.or_max_threads()
    n0 = args.ctx - (args.steps + args.warmup)
    chunks, extra = chunks_fn()
    ref = cpu_fill(oracle, (kind, mode.bits, mode.v_quant), chunks, n0)
    rng = np.random.default_rng(1234)
    times = []
    for s in range(args.warmup + args.steps):
        q = rng.standard_normal((NH, HD), dtype=np.float32)
        k, v = extra[0][s % extra[0].shape[0]], extra[1][s % extra[1].shape[0]]
        t = cpu_layer_step(ref, q, k, v, n0 + s, threads)
        if s >= args.warmup:
            times.append(t)
    t_layer = float(np.mean(times))
    tok_s = 1.0 / (t_layer * N_LAYERS)
    sample = (f"1 of {N_LAYERS} layers per step at the full context ({args.ctx} positions), append + attention, "
              f"time x{N_LAYERS}")
    line = {
        "impl": "reference", "metric": "quantized-KV decode attention tokens/s at 128K ctx", "value": tok_s,
        "unit": "tokens/s", "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": t_layer * N_LAYERS * 1e3, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "f32", "data": "synthetic",
        "config": workload_config(args, mode),
        "effective_gbs": attn_bytes(mode, args.ctx) / t_layer / 1e9,
        "cpu_baseline": {"value": tok_s, "unit": "tokens/s", "cores": min(threads, NH), "kind": "port",
                         "sample": sample},
        "e2e": {"value": tok_s, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


def workload_config(args, mode):
    return {"workload": f"decode128k: 1 sequence/GPU, {N_LAYERS} full-attention layers, context {args.ctx}, "
                        f"{args.mode} KV cache, {NH} q / {NKV} kv heads, head_dim {HD}",
            "kv_mode": args.mode, "context": args.ctx, "layers": N_LAYERS, "batch_per_gpu": 1,
            "step": ("bk_attn_layer_step (q|gate split, q/k RMSNorm, append, attention, sigmoid gate)"
                     if getattr(args, "step", "attn") == "layer" else "bk_attn_step (append + attention)"),
            "l2": ("each step streams %.2f GB of cache, larger than the 126 MB L2 (no flush needed)"
                   if N_LAYERS * attn_bytes(mode, args.ctx) > 2 * 126e6 else
                   "each step streams only %.2f GB of cache: it may stay in the 126 MB L2 between steps, so this is "
                   "not an HBM measurement") % (N_LAYERS * attn_bytes(mode, args.ctx) / 1e9)}


# ---------------------------------------------------------------------------------------------
# secondary workloads (the other sharded configurations; same JSON shape, no CPU arm)
# ---------------------------------------------------------------------------------------------


def build_batch64(bk, par, ctx, mode, rank, world, total_steps, mode_name):
    """64 sequences, contexts U[2048,16384] (seeded), sharded greedily by length over the ranks."""
    rng = np.random.default_rng(99)          # same plan and data on every rank
    channels = rng.choice(HD, size=3, replace=False)
    n_seqs = 64
    lens = rng.integers(2048, 16385, n_seqs)
    mine = par.shard_sequences(lens, world)[rank]
    n_local = len(mine)
    n_ctx = int(lens.max()) + total_steps
    cache = bk.AttnCache(ctx, mode, n_layers=N_LAYERS, n_seqs=max(n_local, 1), n_ctx=n_ctx)
    k, v = synth_chunk(rng, 16384, channels)
    dk, dv = ctx.to_device(k), ctx.to_device(v)
    for j, i in enumerate(mine):
        for il in range(N_LAYERS):
            cache.append_device(il, dk.ptr, dv.ptr, n_tokens=int(lens[i]), seq=j)
    ctx.synchronize()
    d_q = ctx.to_device(rng.standard_normal((N_LAYERS, max(n_local, 1), NH, HD), dtype=np.float32))
    d_out = ctx.alloc(max(n_local, 1) * NH * HD * 4)

    def step(_s):
        for il in range(N_LAYERS):
            if n_local:
                cache.step_batch_device(il, d_q.offset(il * n_local * NH * HD * 4), dk.ptr, dv.ptr, d_out.ptr, n_local)

    def cleanup():
        cache.close()
        for b in (dk, dv, d_q, d_out):
            b.free()
    step_bytes = N_LAYERS * sum(attn_bytes(mode, int(lens[i])) + append_bytes(mode) for i in range(n_seqs))
    cfg = {"workload": f"batch64: {n_seqs} sequences, contexts U[2048,16384] (seeded, mean {lens.mean():.0f}), "
                       f"{N_LAYERS} layers, {mode_name}; sequences sharded greedily over {world} GPU(s), no collective",
           "l2": "%.2f GB of cache per step, larger than L2" % (step_bytes / 1e9)}
    return step, step_bytes, n_seqs, "strong", cfg, cleanup


def build_splitctx(bk, par, ctx, mode, rank, world, local, dist, total_steps, mode_name, exchange):
    """One 262144-token sequence, contiguous context chunks per rank, the partial results exchanged per layer."""
    import torch
    rng = np.random.default_rng(99)
    channels = rng.choice(HD, size=3, replace=False)
    n_total = 262144
    chunks = par.split_context(n_total - total_steps, world)
    b, e = chunks[rank]
    owner = par.tail_owner(chunks)
    cache = bk.AttnCache(ctx, mode, n_layers=N_LAYERS, n_seqs=1, n_ctx=(e - b) + total_steps, rope_positions=n_total)
    k, v = synth_chunk(rng, 8192, channels)
    dk, dv = ctx.to_device(k), ctx.to_device(v)
    for il in range(N_LAYERS):
        p = b
        while p < e:
            n = min(8192, e - p)
            cache.append_device(il, dk.ptr, dv.ptr, n_tokens=n, pos=p)
            p += n
    ctx.synchronize()
    d_q = ctx.to_device(rng.standard_normal((N_LAYERS, NH, HD), dtype=np.float32))
    dev = torch.device("cuda", local)
    part = torch.zeros((NH, HD + 2), dtype=torch.float32, device=dev)
    out = torch.zeros((NH, HD), dtype=torch.float32, device=dev)
    gathered = torch.zeros((world, NH, HD + 2), dtype=torch.float32, device=dev)
    pos_now = [n_total - total_steps]
    lib_stream = torch.cuda.ExternalStream(ctx.stream, device=dev)
    split = par.ContextSplit(cache, dist, rank, world) if (world > 1 and exchange in ("p2p", "p2p_layers")) else None
    out_layers = None
    if split is not None and exchange == "p2p_layers":
        split.open_layers_mailbox(dist, N_LAYERS)
        out_layers = torch.zeros((N_LAYERS, NH, HD), dtype=torch.float32, device=dev)

    def step(_s):
        if out_layers is not None:  # all layers scanned back to back, ONE exchange of their partial rows per token
            own = rank == owner
            split.step_layers_device(d_q.ptr, dk.ptr if own else None, dv.ptr if own else None, out_layers.data_ptr(),
                                     q_pos=pos_now[0])
            pos_now[0] += 1
            return
        for il in range(N_LAYERS):
            if split is not None:  # one launch per rank and layer: append (tail owner), scan, exchange, merge
                own = rank == owner
                split.step_device(il, d_q.offset(il * NH * HD * 4), dk.ptr if own else None, dv.ptr if own else None,
                                  out.data_ptr(), q_pos=pos_now[0])
                continue
            if world == 1:
                cache.step_device(il, d_q.offset(il * NH * HD * 4), dk.ptr, dv.ptr, out.data_ptr(), pos_now[0])
                continue
            if rank == owner:
                cache.append_device(il, dk.ptr, dv.ptr, n_tokens=1, pos=pos_now[0])
            cache.decode_device(il, d_q.offset(il * NH * HD * 4), part.data_ptr(), q_pos=[pos_now[0]], partial=True)
            with torch.cuda.stream(lib_stream):     # NCCL orders itself against the library's stream:
                dist.all_gather_into_tensor(gathered.view(-1), part.view(-1))   # no host sync per layer
            ctx.check(ctx.lib.bk_lse_merge(ctx.h, world, NH, HD, gathered.data_ptr(), out.data_ptr()))
        pos_now[0] += 1

    def cleanup():
        if split is not None:
            split.close()
        cache.close()
        for bf in (dk, dv, d_q):
            bf.free()
    step_bytes = N_LAYERS * (attn_bytes(mode, n_total) + append_bytes(mode))
    cfg = {"workload": f"splitctx: 1 sequence, context {n_total}, {N_LAYERS} layers, {mode_name}; contiguous context "
                       f"chunks over {world} GPU(s); per layer the (acc, m, l) partials are exchanged "
                       + ("through peer memory in ONE call per token after all layers are scanned (bk_exchange_merge; "
                          "layers independent of one another)" if out_layers is not None else
                          "through peer memory inside the decode launch (bk_attn_step_split)" if split is not None
                          else ("by one NCCL all-gather, then bk_lse_merge" if world > 1 else "- one GPU, nothing to exchange")),
           "l2": "%.2f GB of cache per step over all GPUs" % (step_bytes / 1e9)}
    return step, step_bytes, 1, "strong", cfg, cleanup


def append_sweep(bk, ctx, mode, rng, channels, max_tokens=4096):
    """Append throughput for 1, 2, 4, ... tokens per call (one call per layer, 16 layers per measurement):
    the fused rope + quantize + store kernel alone, device-resident K/V, CUDA events, median of the repeats."""
    cache = bk.AttnCache(ctx, mode, n_layers=N_LAYERS, n_seqs=1, n_ctx=max_tokens * 2)
    k, v = synth_chunk(rng, max_tokens, channels)
    dk, dv = ctx.to_device(k), ctx.to_device(v)
    table = []
    n = 1
    while n <= max_tokens:
        reps = max(4, min(64, 8192 // n))
        ts = []
        for r in range(reps + 2):
            cache.reset()
            e0, e1 = ctx.event(), ctx.event()
            e0.record()
            for il in range(N_LAYERS):
                cache.append_device(il, dk.ptr, dv.ptr, n_tokens=n, pos=0)
            e1.record()
            ctx.synchronize()
            if r >= 2:
                ts.append(e0.elapsed_ms(e1))
        t = float(np.median(ts)) * 1e-3
        table.append({"tokens_per_call": n, "tokens_per_s": n / t, "gb_per_s": N_LAYERS * append_bytes(mode, n) / t / 1e9,
                      "us_per_call_all_layers": t * 1e6})
        n *= 2
    cache.close()
    dk.free()
    dv.free()
    return table


def timed_steps(ctx, dist, local, step, steps, warmup):
    """Device time of `steps` steps after `warmup`: CUDA events on the library's stream, barriers on both
    sides, max over the ranks.  Returns ms per step."""
    for s_ in range(warmup):
        step(s_)
    ctx.synchronize()
    barrier(dist)
    ev0, ev1 = ctx.event(), ctx.event()
    ev0.record()
    for s_ in range(steps):
        step(s_)
    ev1.record()
    ctx.synchronize()
    barrier(dist)
    return max_over_ranks(dist, local, ev0.elapsed_ms(ev1)) / steps


def splitctx_self_check(bk, par, ctx, dist, rank, world):
    """The split-context step against a whole cache, on a small side case (6003 rows, one layer, two steps):
    every rank's merged output is compared with rank 0's whole-cache output; returns the worst |difference|
    over the ranks (on every rank)."""
    rng = np.random.default_rng(3)       # same stream on every rank
    n0, steps = 6003, 2
    n_total = n0 + steps
    k = rng.standard_normal((n_total, NKV, HD), dtype=np.float32)
    v = rng.standard_normal((n_total, NKV, HD), dtype=np.float32)
    k[:, :, [9, 100, 222]] *= np.float32(20.0)
    v[:, :, [9, 100, 222]] *= np.float32(20.0)
    q = rng.standard_normal((steps, NH, HD), dtype=np.float32)
    chunks = par.split_context(n0, world)
    b, e = chunks[rank]
    owner = par.tail_owner(chunks)
    mode = bk.parse_mode("planar4")
    mine = bk.AttnCache(ctx, mode, n_layers=1, n_ctx=max(e - b, 0) + steps, rope_positions=n_total)
    # the whole cache goes through the f32 kernel (BONSAI_KV_GENERIC is read when a context is created), so the
    # difference measured is the split path's own error, not the sum of two tensor-core results
    ref_ctx = None
    if rank == 0:
        os.environ["BONSAI_KV_GENERIC"] = "1"
        ref_ctx = bk.Context(ctx.device)
        del os.environ["BONSAI_KV_GENERIC"]
    whole = bk.AttnCache(ref_ctx, mode, n_layers=1, n_ctx=n_total) if rank == 0 else None
    if e > b:
        mine.append(0, k[b:e], v[b:e], pos=b)
    if whole:
        whole.append(0, k[:n0], v[:n0])
    split = par.ContextSplit(mine, dist, rank, world)
    split.open_layers_mailbox(dist, 1)
    d_out = ctx.alloc(NH * HD * 4)
    worst = 0.0
    for s in range(steps):
        pos = n0 + s
        d_q, d_k, d_v = ctx.to_device(q[s]), ctx.to_device(k[pos]), ctx.to_device(v[pos])
        own = rank == owner
        if s == 0:   # the step whose exchange rides in the decode launch ...
            split.step_device(0, d_q.ptr, d_k.ptr if own else None, d_v.ptr if own else None, d_out.ptr, q_pos=pos)
        else:        # ... and the form that scans first and exchanges all (here: one) layers' rows in one call
            split.step_layers_device(d_q.ptr, d_k.ptr if own else None, d_v.ptr if own else None, d_out.ptr, q_pos=pos)
        got = d_out.download((NH, HD), np.float32)
        want = whole.step(0, q[s], k[pos], v[pos], pos) if whole else None
        box = [want]
        dist.broadcast_object_list(box, src=0)
        err = float(np.max(np.abs(got - box[0])))
        errs = [None] * world
        dist.all_gather_object(errs, err)
        worst = max(worst, max(errs))
        for bf in (d_q, d_k, d_v):
            bf.free()
    split.close()
    mine.close()
    if whole:
        whole.close()
        ref_ctx.close()
    return worst


def run_sharded(bk, ctx, mode, mode_name, rank, world, local, dist, steps=5, warmup=3):
    """The two configurations that shard one job over the ranks, each with its own 1-GPU time (rank 0 alone,
    same run) so that the speed-up needs no second record.  Returns the `sharded` object of the JSON line."""
    par = importlib.import_module("ternary-bonsai-inference_b200.parallel")
    total = steps + warmup
    out = {}
    for name in ("batch64", "splitctx"):
        def build(r, w, d):
            if name == "batch64":
                return build_batch64(bk, par, ctx, mode, r, w, total, mode_name)
            return build_splitctx(bk, par, ctx, mode, r, w, local, d, total, mode_name, "p2p")
        n1 = None
        if rank == 0:   # this workload on one GPU: rank 0 alone, the others wait at the barrier below
            step, step_bytes, tokens, _sc, _cfg, cleanup = build(0, 1, None)
            ms1 = timed_steps(ctx, None, local, step, steps, warmup)
            cleanup()
            n1 = {"tokens_per_s": tokens * 1e3 / ms1, "ms_per_step": ms1, "effective_gbs": step_bytes / ms1 / 1e6}
        entry = {"n1": n1}
        if world > 1:
            barrier(dist)
            step, step_bytes, tokens, scaling, cfg, cleanup = build(rank, world, dist)
            ms = timed_steps(ctx, dist, local, step, steps, warmup)
            cleanup()
            entry.update({"tokens_per_s": tokens * 1e3 / ms, "ms_per_step": ms, "effective_gbs": step_bytes / ms / 1e6,
                          "scaling": scaling, "workload": cfg["workload"], "steps": steps, "warmup": warmup})
            if n1:
                entry["speedup_vs_own_n1"] = n1["ms_per_step"] / ms
                entry["efficiency_vs_own_n1"] = n1["ms_per_step"] / ms / world
            if name == "splitctx":
                entry["exchange"] = "p2p"
                entry["form"] = "per-layer dependent: every layer's exchange completes before the next layer starts"
                # the other form: the 16 layers batched, one exchange per token (callers whose layers are independent)
                step, step_bytes, tokens, _sc, cfg, cleanup = build_splitctx(bk, par, ctx, mode, rank, world, local, dist, total,
                                                                             mode_name, "p2p_layers")
                ms_b = timed_steps(ctx, dist, local, step, steps, warmup)
                cleanup()
                entry["layers_batched"] = {"tokens_per_s": tokens * 1e3 / ms_b, "ms_per_step": ms_b,
                                           "effective_gbs": step_bytes / ms_b / 1e6, "workload": cfg["workload"]}
                if n1:
                    entry["layers_batched"]["speedup_vs_own_n1"] = n1["ms_per_step"] / ms_b
                    entry["layers_batched"]["efficiency_vs_own_n1"] = n1["ms_per_step"] / ms_b / world
                entry["check_max_abs"] = splitctx_self_check(bk, par, ctx, dist, rank, world)
        out[name] = entry
    return out


def run_other_workload(args):
    bk = importlib.import_module("ternary-bonsai-inference_b200")
    par = importlib.import_module("ternary-bonsai-inference_b200.parallel")
    mode = bk.parse_mode(args.mode)
    args.warmup = max(args.warmup, 3)
    rank, world, local, dist = dist_setup(args.gpus, need_nccl=(args.workload == "splitctx" and args.exchange == "nccl"))
    ctx = bk.Context(local)
    total_steps = args.steps + args.warmup
    rng = np.random.default_rng(99)          # same plan and data on every rank
    channels = rng.choice(HD, size=3, replace=False)
    line = {"metric": "quantized-KV decode attention tokens/s", "unit": "tokens/s", "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "higher_is_better": True, "vs_baseline": None,
            "dtype": "f32", "data": "synthetic"}

    if args.workload == "batch64":
        step, step_bytes, tokens_per_step, scaling, cfg, _cleanup = build_batch64(bk, par, ctx, mode, rank, world, total_steps, args.mode)
    elif args.workload == "prefill":
        # one prompt of `--ctx` tokens (default here 8192) through all layers in blocks of 512 tokens:
        # per block and layer one bulk append and one batched causal attention (bk_prefill_step)
        n_prompt = args.ctx if args.ctx != 131072 else 8192
        blk = 512
        cache = bk.AttnCache(ctx, mode, n_layers=N_LAYERS, n_seqs=1, n_ctx=n_prompt)
        k, v = synth_chunk(rng, n_prompt, channels)
        dk, dv = ctx.to_device(k), ctx.to_device(v)
        d_q = ctx.to_device(rng.standard_normal((blk, NH, HD), dtype=np.float32))
        d_out = ctx.alloc(blk * NH * HD * 4)

        def step(_s):
            cache.reset()
            for p0 in range(0, n_prompt, blk):
                m = min(blk, n_prompt - p0)
                for il in range(N_LAYERS):
                    cache.prefill_step_device(il, d_q.ptr, dk.offset(p0 * NKV * HD * 4), dv.offset(p0 * NKV * HD * 4),
                                              d_out.ptr, p0, m)
        # every block reads the rows before it once: about n^2 / (2 blk) row reads per layer
        rk, rv = row_bytes(mode)
        reads = sum(p0 + min(blk, n_prompt - p0) for p0 in range(0, n_prompt, blk))
        step_bytes = N_LAYERS * (reads * NKV * (rk + rv) + append_bytes(mode, n_prompt) + 2 * n_prompt * NH * HD * 4)
        tokens_per_step, scaling = n_prompt, "weak"
        flops = N_LAYERS * 4.0 * NH * HD * sum((p0 + i + 1) for p0 in range(0, n_prompt, blk) for i in range(min(blk, n_prompt - p0)))
        cfg = {"workload": f"prefill: one prompt of {n_prompt} tokens, blocks of {blk}, {N_LAYERS} layers, {args.mode}; "
                           f"per block and layer a bulk append and a batched causal attention over the quantized cache",
               "useful_tflop_per_step": flops / 1e12}
    elif args.workload == "splitctx":
        step, step_bytes, tokens_per_step, scaling, cfg, _cleanup = build_splitctx(bk, par, ctx, mode, rank, world, local, dist,
                                                                                   total_steps, args.mode, args.exchange)
    elif args.workload == "pq2":
        # The four PQ2_0 projections of a full-attention layer, one token: wq [12288 x 5120] (q | gate),
        # wk and wv [1024 x 5120], wo [5120 x 6144]; 16 layers with their own weights (446 MB, larger than L2).
        shapes = [("wq", 2 * NH * HD, 5120), ("wk", NKV * HD, 5120), ("wv", NKV * HD, 5120), ("wo", 5120, NH * HD)]
        n_tok = 1
        tensors, host_payloads = [], []
        for il in range(N_LAYERS):
            for name, n_rows, ne0 in shapes:
                nb = ne0 // 128
                raw = rng.integers(0, 256, size=(n_rows, nb, 34), dtype=np.uint8)
                raw[..., :2] = (0.01 + rng.random((n_rows, nb))).astype(np.float16).view(np.uint8).reshape(n_rows, nb, 2)
                tensors.append((bk.Pq2Tensor(ctx, raw.reshape(-1), ne0), n_rows, ne0))
                if il == 0:
                    host_payloads.append((raw.reshape(-1), n_rows, ne0))
        hx = {ne0: rng.standard_normal((n_tok, ne0), dtype=np.float32) for ne0 in (5120, NH * HD)}
        dx = {ne0: ctx.to_device(v) for ne0, v in hx.items()}
        d_y = ctx.alloc(n_tok * 2 * NH * HD * 4)

        d_yk, d_yv = ctx.alloc(n_tok * NKV * HD * 4), ctx.alloc(n_tok * NKV * HD * 4)

        def step(_s):
            # per layer two launches: q, k and v share their input and one launch; then the output projection
            for il in range(N_LAYERS):
                wq, wk, wv, wo = (t for t, _n, _e in tensors[4 * il:4 * il + 4])
                bk.pq2_matvec_multi_device(ctx, [wq, wk, wv], dx[5120].ptr, [d_y.ptr, d_yk.ptr, d_yv.ptr], n_tok)
                wo.matvec_device(dx[NH * HD].ptr, d_y.ptr, n_tok)
        step_bytes = world * sum(t.payload_bytes for t, _n, _e in tensors)   # every rank is a replica with its own token
        tokens_per_step, scaling = n_tok * world, "weak"
        cfg = {"workload": f"pq2: wq+wk+wv (one launch) and wo of {N_LAYERS} full-attention layers, {n_tok} token(s), weights resident "
                           f"({step_bytes / world / 1e6:.0f} MB streamed per step and GPU, larger than L2)"}

        def pq2_extras():
            """e2e through the host-buffer call, and the oracle's scalar matvec on one layer (x 16)."""
            for t, n_rows, ne0 in tensors[:4]:
                t.matmul_n(hx[ne0], n_tok)
            t0 = time.perf_counter()
            for _ in range(args.steps):
                for t, n_rows, ne0 in tensors:
                    t.matmul_n(hx[ne0], n_tok)
            e2e = args.steps * n_tok / (time.perf_counter() - t0)
            out = {"e2e": {"value": e2e, "unit": "tokens/s", "h2d_bytes_per_step": N_LAYERS * (3 * 5120 + NH * HD) * 4 * n_tok,
                           "d2h_bytes_per_step": N_LAYERS * sum(n for _p, n, _e in host_payloads) * 4 * n_tok}}
            if not args.no_cpu_baseline:
                sys.path.insert(0, os.path.join(ROOT, "tests"))
                from oracle_lib import load_oracle
                orc = load_oracle()
                t0 = time.perf_counter()
                for pl, n_rows, ne0 in host_payloads:
                    orc.pq2_matmul(pl, ne0, 0, n_rows, hx[ne0], n_tok)
                dt = time.perf_counter() - t0
                out["cpu_baseline"] = {"value": n_tok / (dt * N_LAYERS), "unit": "tokens/s", "cores": 1, "kind": "port",
                                       "sample": "the four tensors of one layer through the oracle's scalar row dot, time x 16"}
            return out
    else:  # appendsweep
        table = append_sweep(bk, ctx, mode, rng, channels)
        if rank == 0:
            line.update({"metric": "KV append throughput (fused rope+quantize+store)", "value": table[-1]["tokens_per_s"],
                         "ms_per_step": table[-1]["us_per_call_all_layers"] / 1e3, "scaling": "weak",
                         "config": {"workload": f"appendsweep: 1..4096 tokens per call, {N_LAYERS} layers, {args.mode}"},
                         "sweep": table})
            print(json.dumps(line), flush=True)
        if dist is not None:
            dist.destroy_process_group()
        return

    for s_ in range(args.warmup):
        step(s_)
    ctx.synchronize()
    barrier(dist)
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    launches0 = ctx.launch_count
    ev0, ev1 = ctx.event(), ctx.event()
    ev0.record()
    for s_ in range(args.steps):
        step(s_)
    ev1.record()
    ctx.synchronize()
    barrier(dist)
    ms_step = max_over_ranks(dist, local, ev0.elapsed_ms(ev1)) / args.steps
    clocks = sampler.stop() if rank == 0 else None
    if rank == 0:
        peak, peak_kind = measured_peak()
        gbs = step_bytes / (ms_step * 1e-3) / 1e9
        if args.workload == "prefill":
            line["metric"] = "quantized-KV prefill attention prompt tokens/s"
            line["useful_tflops"] = cfg["useful_tflop_per_step"] / (ms_step * 1e-3)
        if args.workload == "pq2":
            line["metric"] = "PQ2_0 attention-projection matvec tokens/s"
            if world == 1:   # the host-buffer loop and the CPU arm are single-process measurements
                line.update(pq2_extras())
        line.update({"value": tokens_per_step * 1e3 / ms_step, "ms_per_step": ms_step, "scaling": scaling, "config": cfg,
                     "effective_gbs": gbs, "gpu_launches": ctx.launch_count - launches0,
                     "roofline": {"bound": "hbm", "achieved": gbs / world, "peak": peak, "unit": "GB/s",
                                  "frac": gbs / world / peak, "peak_kind": f"of {peak_kind}", "traffic": None,
                                  "note": "whole step (append + decode of every layer) per GPU, not one kernel"},
                     "clocks": clocks})
        if args.workload == "pq2":
            line["roofline"]["note"] = ("pq2_matvec_kernel, every launch of the step: payload bytes (the algorithmic "
                                        "bytes: each weight byte once) over the step's device time")
            # not measured by this run: dram__bytes_read.sum + dram__bytes_write.sum of one layer's two launches
            # (19.55 + 8.41 MB, writes 0) from an ncu capture, times the layers of a step
            line["roofline"]["traffic"] = N_LAYERS * 27.96e6   # per GPU, like `achieved`
            line["roofline"]["traffic_source"] = "ncu capture of one layer (copied constant)"
        print(json.dumps(line), flush=True)
    if dist is not None:
        dist.destroy_process_group()


# ---------------------------------------------------------------------------------------------

def decode_kernel_name(mode_tag, ctx):
    """The kernel a decode launch of this workload runs (the library picks it by mode and length)."""
    if ctx >= 2048 and mode_tag == "planar4":
        return ("decode_p4_mma_kernel (split-K GQA decode attention over the 4-bit cache, with the one-token "
                "append fused in)")
    if ctx >= 2048 and mode_tag == "f16":
        return "decode_f16_mma_kernel (split-K GQA decode attention over the f16 cache, with the one-token append fused in)"
    return "decode_kernel (generic f32 split-K GQA decode attention), after append_kernel"


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--mode", default="planar4")
    ap.add_argument("--ctx", type=int, default=131072)
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-sharded", dest="sharded", action="store_false",
                    help="skip the batch64 / splitctx passes that follow the headline pass")
    ap.add_argument("--chunk", type=int, default=8192)
    ap.add_argument("--layers", type=int, default=16, help="full-attention layers (16 = qwen35; fewer only to keep a profiler capture small)")
    ap.add_argument("--exchange", default="p2p", choices=["p2p", "p2p_layers", "nccl"],
                    help="splitctx only: p2p = peer-memory exchange fused with the merge (bk_decode_attn_split); "
                         "nccl = all-gather of the partials + bk_lse_merge")
    ap.add_argument("--step", default="attn", choices=["attn", "layer"],
                    help="attn: bk_attn_step (the metric's step); layer: bk_attn_layer_step, which also does the "
                         "q|gate split, the per-head RMSNorm of q and k and the sigmoid gate in the same launch")
    ap.add_argument("--workload", default="decode128k", choices=["decode128k", "batch64", "splitctx", "appendsweep", "prefill", "pq2"],
                    help="decode128k: the headline (default).  batch64: 64 sequences, contexts U[2048,16384], sharded "
                         "over the ranks.  splitctx: one 262144-token sequence, context chunks per rank, LSE merge.  "
                         "appendsweep: append throughput for 1..4096 tokens per call")
    args = ap.parse_args()
    global N_LAYERS
    N_LAYERS = args.layers
    if args.workload != "decode128k" and args.impl == "ours":
        return run_other_workload(args)
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup

    mode = Mode(args.mode)                # (the reference arm runs without the CUDA library)
    total_steps = args.steps + args.warmup
    n0 = args.ctx - total_steps           # the context reaches args.ctx at the last step
    assert n0 > 0

    def make_chunks(seed=0):
        """Prefill rows for one layer (shared by all layers) + the rows appended by the steps."""
        rng = np.random.default_rng(seed)
        channels = rng.choice(HD, size=3, replace=False)
        chunks, left = [], n0
        while left > 0:
            n = min(args.chunk, left)
            chunks.append(synth_chunk(rng, n, channels))
            left -= n
        return chunks, synth_chunk(rng, total_steps, channels)

    if args.impl == "reference":
        run_reference(args, mode, make_chunks)
        return

    bk = importlib.import_module("ternary-bonsai-inference_b200")
    mode = bk.parse_mode(args.mode)
    rank, world, local, dist = dist_setup(args.gpus)
    ctx = bk.Context(local)
    cache = bk.AttnCache(ctx, mode, n_layers=N_LAYERS, n_seqs=1, n_ctx=args.ctx)
    chunks, (k_new, v_new) = make_chunks(seed=rank)

    # ---- prefill through the append kernel (not timed) ----------------------------------
    dk, dv = ctx.alloc(args.chunk * NKV * HD * 4), ctx.alloc(args.chunk * NKV * HD * 4)
    for k, v in chunks:
        dk.upload(k, sync=False)
        dv.upload(v, sync=True)
        for il in range(N_LAYERS):
            cache.append_device(il, dk.ptr, dv.ptr, n_tokens=k.shape[0])
        ctx.synchronize()
    dk.free(); dv.free()
    assert cache.n_pos(0) == n0

    # ---- step inputs, resident in HBM -------------------------------------------------------
    rng = np.random.default_rng(1234 + rank)
    layer_form = args.step == "layer"
    q_width = 2 * HD if layer_form else HD  # the layer form reads the interleaved [q | gate] projection output
    q_all = rng.standard_normal((total_steps, N_LAYERS, NH, q_width), dtype=np.float32)
    d_q = ctx.to_device(q_all)
    d_k = ctx.to_device(k_new)
    d_v = ctx.to_device(v_new)
    d_out = ctx.alloc(N_LAYERS * NH * HD * 4)
    q_stride, kv_stride, out_stride = NH * q_width * 4, NKV * HD * 4, NH * HD * 4
    norm_w = (1.0 + 0.1 * rng.standard_normal((2, HD))).astype(np.float32)
    d_w = ctx.to_device(norm_w)
    eps = 1e-6

    def device_step(s, events=None):
        # the reference's unit of work: one attention step per layer (append at pos, attend over pos+1)
        pos = cache.n_pos(0)
        for il in range(N_LAYERS):
            if events is not None:
                events[il][0].record()
            if layer_form:
                cache.layer_step_device(il, d_q.offset((s * N_LAYERS + il) * q_stride), d_k.offset(s * kv_stride),
                                        d_v.offset(s * kv_stride), d_w.ptr, d_w.offset(HD * 4), eps,
                                        d_out.offset(il * out_stride), pos)
            else:
                cache.step_device(il, d_q.offset((s * N_LAYERS + il) * q_stride), d_k.offset(s * kv_stride),
                                  d_v.offset(s * kv_stride), d_out.offset(il * out_stride), pos)
            if events is not None:
                events[il][1].record()

    for s in range(args.warmup):
        device_step(s)
    ctx.synchronize()
    barrier(dist)
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    ev0, ev1 = ctx.event(), ctx.event()
    launches0 = ctx.launch_count
    ev0.record()
    for s in range(args.warmup, total_steps):
        device_step(s)
    ev1.record()
    ctx.synchronize()
    barrier(dist)
    launches = ctx.launch_count - launches0
    ms_total = max_over_ranks(dist, local, ev0.elapsed_ms(ev1))
    ms_step = ms_total / args.steps
    final_ctx = cache.n_pos(0)

    # ---- roofline of the dominant kernel: per-launch events, steps replayed on the full cache ----
    for il in range(N_LAYERS):
        cache.set_n_pos(il, 0, final_ctx - args.steps)
    evs = [[(ctx.event(), ctx.event()) for _ in range(N_LAYERS)] for _ in range(args.steps)]
    for i, s in enumerate(range(args.warmup, total_steps)):
        device_step(s, evs[i])
    ctx.synchronize()
    dec_ms = [a.elapsed_ms(b) for step in evs for (a, b) in step]
    dec_ms_isolated = float(np.mean(dec_ms))       # each launch between its own pair of events (no overlap with its neighbours)
    clocks = sampler.stop() if rank == 0 else None
    peak, peak_kind = measured_peak()
    alg = attn_bytes(mode, args.ctx - args.steps // 2)
    # the kernel's average launch duration over the timed region.  On caches that take the fused kernel the step
    # is nothing but these launches (one per layer); elsewhere a layer is an append launch and a decode launch,
    # and the layer's whole time is charged to the decode kernel (its bytes over append + decode time)
    dec_ms_avg = ms_total / (args.steps * N_LAYERS)
    achieved = alg / (dec_ms_avg * 1e-3) / 1e9

    # ---- e2e: the same steps through the host-buffer entry point ---------------------------------
    for il in range(N_LAYERS):
        cache.set_n_pos(il, 0, final_ctx - args.steps)
    hq = ctx.pinned((N_LAYERS, NH * q_width), np.float32)
    hw = ctx.pinned((2, HD), np.float32)
    hw.array[:] = norm_w
    hk = ctx.pinned((NKV * HD,), np.float32)
    hv = ctx.pinned((NKV * HD,), np.float32)
    hout = ctx.pinned((N_LAYERS, NH * HD), np.float32)
    lib = ctx.lib
    barrier(dist)
    t0 = time.perf_counter()
    for s in range(args.warmup, total_steps):
        hq.array[:] = q_all[s].reshape(N_LAYERS, -1)
        hk.array[:] = k_new[s].ravel()
        hv.array[:] = v_new[s].ravel()
        pos = cache.n_pos(0)
        for il in range(N_LAYERS):
            if layer_form:
                ctx.check(lib.bk_attn_layer_step_host(cache.h, il, 0, pos, hq.ptr + il * q_stride, hk.ptr, hv.ptr,
                                                      hw.ptr, hw.ptr + HD * 4, eps, hout.ptr + il * out_stride))
            else:
                ctx.check(lib.bk_attn_step_host(cache.h, il, 0, pos, hq.ptr + il * q_stride, hk.ptr, hv.ptr,
                                                hout.ptr + il * out_stride))
    e2e_s = max_over_ranks(dist, local, time.perf_counter() - t0)
    barrier(dist)
    e2e_tok_s = world * args.steps / e2e_s
    checksum = float(np.abs(hout.array).sum())

    # ---- the configurations that shard one job over the GPUs (16 layers, planar cache) --------------
    sharded, sweep = None, None
    if args.sharded and mode.kind == "planar" and N_LAYERS == 16:
        cache.close()
        sharded = run_sharded(bk, ctx, mode, args.mode, rank, world, local, dist)
        if rank == 0 and world == 1:   # the append kernel on its own, 1 .. 4096 tokens per call
            r2 = np.random.default_rng(99)
            sweep = append_sweep(bk, ctx, mode, r2, r2.choice(HD, size=3, replace=False))

    if rank != 0:
        if dist is not None:
            dist.destroy_process_group()
        return

    # ---- CPU baseline (rank 0, N = 1 only): the oracle on one layer at the full context ----------
    cpu = None
    if world == 1 and not args.no_cpu_baseline:
        from oracle_lib import MODE_F16, MODE_F32, MODE_PLANAR, load_oracle
        oracle = load_oracle()
        kind = {"f32": MODE_F32, "f16": MODE_F16, "planar": MODE_PLANAR}[mode.kind]
        threads = oracle.lib.or_max_threads()
        ref = cpu_fill(oracle, (kind, mode.bits, mode.v_quant), chunks, n0)
        if layer_form:
            def cpu_one(s):
                t0 = time.perf_counter()
                ref.layer_step(0, q_all[s, 0], k_new[s], v_new[s], norm_w[0], norm_w[1], eps, n0 + s, threads=threads)
                return time.perf_counter() - t0
            ts = [cpu_one(s) for s in range(3)]
        else:
            ts = [cpu_layer_step(ref, q_all[s, 0], k_new[s], v_new[s], n0 + s, threads) for s in range(3)]
        t_layer = float(np.mean(ts[1:]))
        # the reference's own loop is single-threaded (src/forward.rs:297): one thread over a 1/8 slice of the
        # context (attention is linear in it), scaled back
        n_slice = max(n0 // 8, 1)
        t0 = time.perf_counter()
        ref.attend(0, q_all[0, 0][:, :HD] if layer_form else q_all[0, 0], n_slice - 1, n_slice, threads=1)
        t_one = (time.perf_counter() - t0) * (n0 / n_slice)
        cpu = {"value": 1.0 / (t_layer * N_LAYERS), "unit": "tokens/s", "cores": min(threads, NH), "kind": "port",
               "sample": f"1 of {N_LAYERS} layers at context {n0} (append + attention, 2 timed steps after 1 warm-up), "
                         f"time x{N_LAYERS}; q-heads spread over {min(threads, NH)} host threads",
               "ms_per_layer": t_layer * 1e3,
               "single_thread": {"value": 1.0 / (t_one * N_LAYERS), "unit": "tokens/s", "cores": 1,
                                 "ms_per_layer": t_one * 1e3,
                                 "sample": f"attention of 1 layer over the first {n_slice} of {n0} positions on one thread, "
                                           f"time x{n0 / n_slice:.0f} x{N_LAYERS}"}}

    tok_s = world * 1e3 / ms_step
    step_bytes = N_LAYERS * (attn_bytes(mode, args.ctx - args.steps // 2) + append_bytes(mode))
    line = {
        "metric": "quantized-KV decode attention tokens/s at 128K ctx",
        "value": tok_s, "unit": "tokens/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": ms_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": ("f16 tensor-core operands (centroid table and q as f16, q and V weights hi+lo), f32 accumulate and softmax"
                  if mode.kind != "f32" and args.ctx >= 2048 else "f32"),
        "data": "synthetic", "config": workload_config(args, mode),
        "effective_gbs": world * step_bytes / (ms_step * 1e-3) / 1e9,
        "gpu_launches": launches,
        "e2e": {"value": e2e_tok_s, "unit": "tokens/s",
                "h2d_bytes_per_step": N_LAYERS * ((NH * q_width + 2 * NKV * HD + (2 * HD if layer_form else 0)) * 4),
                "d2h_bytes_per_step": N_LAYERS * NH * HD * 4,
                "api": ("bk_attn_layer_step_host" if layer_form else "bk_attn_step_host") +
                       " per layer (host q/k/v in, host out; blocks per layer like the reference)",
                "out_checksum": checksum},
        "roofline": {"bound": "hbm", "kernel": decode_kernel_name(args.mode, args.ctx),
                     "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                     "peak_kind": f"of {peak_kind}",
                     # not measured by this run: dram__bytes_read.sum + dram__bytes_write.sum of one launch of this
                     # kernel at this workload, copied from an ncu capture (mean of the captured launches)
                     "traffic": {("planar4", 131072): 142.5e6, ("f16", 32768): 138.3e6}.get((args.mode, args.ctx)),
                     "traffic_source": "ncu capture of one layer of this workload (copied constant, see the profile summaries)",
                     "algorithmic_bytes_per_launch": alg, "avg_launch_ms": dec_ms_avg,
                     "avg_launch_ms_source": "timed region / (steps x layers): one decode launch per layer, overlapped by "
                                             "programmatic dependent launch"
                                             + ("" if launches == args.steps * N_LAYERS else
                                                "; this cache mode also launches an append kernel per layer, whose time is included"),
                     "isolated_launch_ms": dec_ms_isolated,
                     "frac_isolated": alg / (dec_ms_isolated * 1e-3) / 1e9 / peak,
                     "frac_of_8TBs_nominal": achieved / 8000.0},
        "cpu_baseline": cpu, "clocks": clocks, "sharded": sharded, "append_sweep": sweep,
    }
    print(json.dumps(line), flush=True)
    if dist is not None:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
