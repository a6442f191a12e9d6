"""Benchmark of the SQAttn hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]

One "step" is one call of the prefill operator (input preparation + windowed attention kernel, i.e.
``layer.prefill_attention(q, k, v, None)``) on one batch of synthetic input with the shapes of the
reference's Qwen2.5-7B attention call at a 131072-token context: batch 1, 28 query / 4 KV heads, head_dim 128,
bf16, Q,K,V ~ N(0,1) with four K channels scaled by 8, the reference's effective default window (sink 256,
int8/int4 window ratio 0.1).  The metric is TFLOP/s counted over the (query, key) pairs the kernel has to
visit (4*D flops per pair and head), never over padded tiles.  With N > 1 GPUs the SAME 131072-token sequence
is sharded by query rows (sequence parallel; K mean all-reduced, window halo of K/V exchanged over NCCL):
strong scaling.  The line also carries the 32768-token operator, dense causal attention, the 1M-token decode
step (on N GPUs: split-KV across the GPUs through both exchanges), the decoder stand-in's time to first token
and, for N > 1, the error of the N-rank results against the same computation on one GPU.

Prints ONE JSON line.  ``--impl reference`` times the CPU restatement of the reference's own path
(oracle/) on the host cores instead, on a bounded sample of the same workload.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import torch  # noqa: E402

HQ, HKV, D = 28, 4, 128
SEQ_TOTAL = 131072      # the context length the metric is quoted on
SEQ_SMALL = 32768       # the single-GPU prefill configuration, reported beside it
SINK, RATIO = 256, 0.1


# ----------------------------------------------------------------------------------------------- helpers
def visited_pairs(n: int, w: int, sink: int) -> int:
    """(query, key) pairs with non-zero weight per head for the relative-window schedule (BLOCK_M = 64)."""
    total = 0
    for qs in range(0, n, 64):
        qe = qs + 64
        l8 = max(sink, qe - w)
        total += 64 * min(sink, qs)            # sink stage
        if l8 < qs:
            total += 64 * (qs - l8)            # window stage
        total += 64 * 65 // 2                  # diagonal block
    return total


def window_size(ratio: float, kv_len: int) -> int:
    raw = int((torch.tensor(ratio, dtype=torch.float32) * torch.tensor(float(kv_len), dtype=torch.float32)).item())
    return (raw + 127) // 128 * 128


def load_peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        with open(p) as f:
            d = json.load(f)
        return {"tflops": float(d["bf16_tflops"]), "tflops_sustained": float(d.get("bf16_tflops_sustained", d["bf16_tflops"])),
                "hbm": float(d["hbm_gbs"]), "src": "measured"}
    return {"tflops": 1590.0, "tflops_sustained": 1400.0, "hbm": 6650.0, "src": "fallback"}


def captured_traffic_ratio():
    """DRAM bytes of the attention kernel's ncu capture over its algorithmic Q+K+V+O bytes, read from the committed
    summary of that capture (the table row `DRAM traffic ... | X MB = R x the algorithmic bytes`)."""
    import re
    path = os.path.join(ROOT, "profiles", "prefill_kernel_relative_window_32k.md")
    try:
        with open(path) as f:
            m = re.search(r"DRAM traffic[^|]*\|\s*([0-9.]+) MB = ([0-9.]+) x the algorithmic bytes", f.read())
        return float(m.group(2)), "profiles/prefill_kernel_relative_window_32k.md"
    except Exception:
        return None, None


class ClockSampler:
    """nvidia-smi clock / throttle-reason samples taken while the timed region runs."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.rows, self.proc, self.first = index, [], None, 0

    def start(self):
        """Start sampling and wait (at most 3 s) for the first row, so that a short timed region is covered; rows
        that arrived before the region starts are dropped."""
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-i", str(self.index), "-lms", "20"], stdout=subprocess.PIPE, text=True)
            threading.Thread(target=self._read, daemon=True).start()
            t0 = time.time()
            while not self.rows and time.time() - t0 < 3.0:
                time.sleep(0.01)
            self.first = len(self.rows)
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([x.strip() for x in line.split(",")])

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.05)
        self.proc.terminate()
        rows = self.rows[self.first:] or self.rows[-1:]
        sm = sorted(float(r[1]) for r in rows if len(r) > 8 and r[1].replace(".", "").isdigit())
        mx = [float(r[2]) for r in rows if len(r) > 8 and r[2].replace(".", "").isdigit()]
        reasons = set()
        for r in rows:
            if len(r) > 8:
                for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), r[5:9]):
                    if val.lower().startswith("active"):
                        reasons.add(name)
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": mx[0] if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}



def make_inputs(seed: int, n: int, device="cpu", hq: int = HQ, hkv: int = HKV, d: int = D, dtype=torch.bfloat16):
    """Seeded synthetic activations of one attention call: q [1,n,Hq,D], k/v [1,n,Hkv,D] ~ N(0,1), four of the K
    channels (the same four for every seed) scaled by 8."""
    g = torch.Generator(device=device).manual_seed(seed)
    q = torch.randn(1, n, hq, d, generator=g, device=device)
    k = torch.randn(1, n, hkv, d, generator=g, device=device)
    v = torch.randn(1, n, hkv, d, generator=g, device=device)
    ch = torch.randperm(d, generator=torch.Generator().manual_seed(0))[:4].to(k.device)
    k[..., ch] *= 8.0
    return q.to(dtype), k.to(dtype), v.to(dtype)


def block_pairs(blk: int, w: int, sink: int) -> int:
    """visited (query, key) pairs of the 64-row query block ``blk``"""
    qs, qe = blk * 64, blk * 64 + 64
    l8 = max(sink, qe - w)
    return 64 * min(sink, qs) + (64 * (qs - l8) if l8 < qs else 0) + 64 * 65 // 2


# ----------------------------------------------------------------------------------------------- CPU arm
def cpu_sample(seed: int, n: int, nblocks: int = 16, reps: int = 1):
    """Time the oracle (the reference's fake-quant SQAttn path restated on CPU) on a bounded sample of the
    workload: input preparation over a 4096-token slice (scaled to the full length: it is linear in tokens)
    and `nblocks` of the n/64 query blocks for all 28 heads."""
    from oracle import sqattn_oracle as so

    torch.set_num_threads(os.cpu_count() or 1)
    q, k, v = make_inputs(seed, n)
    groups = HQ // HKV
    sl = 4096
    t0 = time.perf_counter()
    so.prep_qkv(q[:, :sl], k[:, :sl], v[:, :sl], groups)
    t_prep = (time.perf_counter() - t0) * (n / sl)
    # kernel part on already prepared tensors (prep of the whole sequence is not repeated per block)
    q8, _, k8, _, v8 = so.prep_qkv(q, k, v, 1)  # GQA-native: the kernel indexes KV heads itself
    q8 = so.scale_q(q8, D)                       # the launcher's q scaling, once instead of once per call
    nblk = n // 64
    step = max(1, nblk // nblocks)
    blocks = list(range(step - 1, nblk, step))[:nblocks]
    w = window_size(RATIO, n)
    best = None
    for _ in range(reps):
        t0 = time.perf_counter()
        so.windowed_prefill(q8, k8, q8, k8, v8, [RATIO] * HQ, [RATIO] * HQ, SINK, mode="relative",
                            output_dtype=torch.bfloat16, blocks=blocks, q_is_scaled=True)
        dt = time.perf_counter() - t0
        best = dt if best is None else min(best, dt)
    flops = 4.0 * D * HQ * sum(block_pairs(b, w, SINK) for b in blocks)
    frac = len(blocks) / nblk
    total_t = best + t_prep * frac
    return {"value": flops / total_t / 1e12, "unit": "TFLOP/s", "cores": torch.get_num_threads(), "kind": "port",
            "sample": f"{len(blocks)} of {nblk} 64-row query blocks x {HQ} heads at N={n} (tile kernel {best:.2f}s) + "
                      f"the proportional share of input preparation ({t_prep:.2f}s for the full sequence, "
                      f"timed on a {sl}-token slice)"}


def cpu_config1():
    """The reference's CPU-runnable configuration exactly (batch 1, 28/4 heads, head_dim 128, 4096 tokens, fp32,
    causal, default window), best of 3 on all host cores: (i) the plain SDPA restatement (K centred like
    sdpa_reference, sqattn/attn_triton.py:324-357), (ii) the whole fake-quant SQAttn path (adapter + windowed kernel)."""
    from oracle import sqattn_oracle as so

    torch.set_num_threads(os.cpu_count() or 1)
    n = 4096
    q, k, v = make_inputs(0, n, dtype=torch.float32)
    qh, kh, vh = (t.permute(0, 2, 1, 3).contiguous() for t in (q, k, v))
    t_sdpa = t_fq = None
    for _ in range(3):
        t0 = time.perf_counter()
        so.sdpa_reference(qh, kh, vh, tensor_layout="HND", is_causal=True, center_k=True)
        dt = time.perf_counter() - t0
        t_sdpa = dt if t_sdpa is None else min(t_sdpa, dt)
        t0 = time.perf_counter()
        so.attention_fn(q, k, v, HQ // HKV, [RATIO] * HQ, [RATIO] * HQ, SINK)
        dt = time.perf_counter() - t0
        t_fq = dt if t_fq is None else min(t_fq, dt)
    dense = 4.0 * D * HQ * (n * (n + 1) / 2)
    win = 4.0 * D * HQ * visited_pairs(n, window_size(RATIO, n), SINK)
    return {"sdpa_fp32_4096": {"seconds": t_sdpa, "tflops_dense_causal": dense / t_sdpa / 1e12},
            "fake_quant_sqattn_fp32_4096": {"seconds": t_fq, "tflops_visited_pairs": win / t_fq / 1e12},
            "cores": torch.get_num_threads(), "best_of": 3}


def run_reference(args):
    """The reference arm: the CPU restatement of the reference's own path (oracle/), all host threads.  Inputs
    are generated and prepared once (the preparation is timed once and charged in proportion); every step
    then times the attention of ONE 64-row query block for all 28 heads, a different block each step, so that
    the whole run stays within a few minutes whatever --steps is."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    from oracle import sqattn_oracle as so

    torch.set_num_threads(os.cpu_count() or 1)
    n = SEQ_TOTAL
    t_all = time.perf_counter()
    q, k, v = make_inputs(0, n)
    sl = 4096
    t0 = time.perf_counter()
    so.prep_qkv(q[:, :sl], k[:, :sl], v[:, :sl], HQ // HKV)
    t_prep = (time.perf_counter() - t0) * (n / sl)
    q8, _, k8, _, v8 = so.prep_qkv(q, k, v, 1)
    q8 = so.scale_q(q8, D)   # the launcher's q scaling, once instead of once per call
    nblk = n // 64
    w = window_size(RATIO, n)
    vals, secs = [], []
    for i in range(args.warmup + args.steps):
        blk = (nblk - 1 - 37 * i) % nblk
        t0 = time.perf_counter()
        so.windowed_prefill(q8, k8, q8, k8, v8, [RATIO] * HQ, [RATIO] * HQ, SINK, mode="relative",
                            output_dtype=torch.bfloat16, blocks=[blk], q_is_scaled=True)
        dt = time.perf_counter() - t0 + t_prep / nblk
        if i >= args.warmup:
            vals.append(4.0 * D * HQ * block_pairs(blk, w, SINK) / dt / 1e12)
            secs.append(dt)
    wall = time.perf_counter() - t_all
    v_ = sum(vals) / len(vals)
    cb = {"value": v_, "unit": "TFLOP/s", "cores": torch.get_num_threads(), "kind": "port",
          "sample": f"one 64-row query block x {HQ} heads per step at N={n} (+ 1/{nblk} of the {t_prep:.2f}s input preparation)"}
    out = {"impl": "reference", "metric": "sqattn_prefill_tflops", "value": v_, "unit": "TFLOP/s", "n_gpus": args.gpus,
           "steps": args.steps, "warmup": args.warmup, "ms_per_step": sum(secs) / len(secs) * 1e3, "higher_is_better": True,
           "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
           "config": workload_config(n, args.gpus), "cpu_baseline": cb,
           "e2e": {"value": v_, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
           "wall_s": wall}
    print(json.dumps(out))


def workload_config(n, gpus):
    return {"workload": f"SQAttn prefill operator, batch 1, {HQ} q / {HKV} kv heads, head_dim {D}, seq {n}, causal, bf16, "
                        f"sink {SINK}, int8/int4 window ratio {RATIO} (the reference's effective default), K outlier channels x8",
            "seq_len": n, "parallelism": f"sp{gpus} (query rows sharded, work-balanced contiguous shards)" if gpus > 1 else "single",
            "l2": "inputs larger than L2 (Q alone is 940 MB at 131072 tokens); no flush needed"}


# ----------------------------------------------------------------------------------------------- GPU arm
class _Args:
    qk_qtype, v_qtype, use_relative_distance = "int", "int", True


class _Layer:
    num_key_value_groups = HQ // HKV


def bind_to_gpu_cpus(local_rank: int):
    """Run this process (and therefore allocate and first-touch its pinned host buffers) on the CPU cores next to
    its GPU: with several ranks on a two-socket host, pinned buffers on the far socket make every host copy cross
    the socket link.  Sets only this process's CPU affinity (what `numactl` would do); no GPU setting is touched.
    Returns the number of cores kept, or None when the topology cannot be read."""
    try:
        import pynvml
        pynvml.nvmlInit()
        h = pynvml.nvmlDeviceGetHandleByIndex(local_rank)
        words = (os.cpu_count() + 63) // 64
        mask = pynvml.nvmlDeviceGetCpuAffinity(h, words)
        cpus = {64 * w + b for w, m in enumerate(mask) for b in range(64) if (m >> b) & 1}
        cpus &= os.sched_getaffinity(0)
        if cpus:
            os.sched_setaffinity(0, cpus)
            return len(cpus)
    except Exception:
        pass
    return None


class _Ctx:
    """Rank, device and timing helpers shared by the legs of the GPU arm."""

    def __init__(self, args):
        import torch.distributed as dist
        self.dist = dist
        self.world = int(os.environ.get("WORLD_SIZE", "1"))
        self.rank = int(os.environ.get("RANK", "0"))
        self.local = int(os.environ.get("LOCAL_RANK", "0"))
        if args.gpus > 1 and self.world != args.gpus:
            raise SystemExit(f"--gpus {args.gpus} needs torchrun with {args.gpus} ranks (WORLD_SIZE={self.world})")
        torch.cuda.set_device(self.local)
        self.dev = torch.device("cuda", self.local)
        self.cpu_cores_bound = bind_to_gpu_cpus(self.local) if self.world > 1 else None
        if self.world > 1:
            dist.init_process_group("nccl", device_id=self.dev)
        self.peaks = load_peaks()

    def barrier(self):
        if self.world > 1:
            self.dist.barrier()
        torch.cuda.synchronize()

    def timed(self, fn, steps):
        """ms for `steps` calls: CUDA events on the launching stream, barrier + synchronize on both sides, max over ranks"""
        self.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            fn()
        e1.record()
        self.barrier()
        ms = torch.tensor([e0.elapsed_time(e1)], device=self.dev)
        if self.world > 1:
            self.dist.all_reduce(ms, op=self.dist.ReduceOp.MAX)
        return ms.item()

    def max_over_ranks(self, x: float) -> float:
        t = torch.tensor([x], device=self.dev, dtype=torch.float64)
        if self.world > 1:
            self.dist.all_reduce(t, op=self.dist.ReduceOp.MAX)
        return t.item()


def leg_decode_1m(ctx, extra):
    """One GPU: a 1M-token layer (K and V 1 GiB each) streamed per launch, four such layers in rotation (inputs exceed
    L2), eager and as a CUDA graph of one 28-layer step."""
    from longcontext_sqattn_paddle_b200 import ops
    dev, peaks = ctx.dev, ctx.peaks
    Lkv = 1 << 20
    layers = [(torch.randn(1, HKV, Lkv, D, device=dev, dtype=torch.bfloat16),
               torch.randn(1, HKV, Lkv, D, device=dev, dtype=torch.bfloat16)) for _ in range(4)]
    qd = torch.randn(1, HQ, 1, D, device=dev, dtype=torch.bfloat16)
    state = {"i": 0}

    def dec():
        kk, vv = layers[state["i"] % 4]
        state["i"] += 1
        ops.decode(qd, kk, vv, out_dtype=torch.bfloat16)

    for _ in range(4):
        dec()
    nl = 28
    dms_ = ctx.timed(dec, nl) / nl
    gbs = 2.0 * HKV * Lkv * D * 2 / (dms_ * 1e-3) / 1e9
    extra["decode_1m_eager"] = {"gb_per_s": gbs, "ms_per_layer": dms_}
    # one decode step = 28 layer launches; replayed from a CUDA graph so that host launch work (descriptors, ctypes)
    # is off the critical path
    graph = torch.cuda.CUDAGraph()
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        for _ in range(nl):
            dec()
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    with torch.cuda.graph(graph):
        for _ in range(nl):
            dec()
    for _ in range(2):
        graph.replay()
    reps = 5
    gms = ctx.timed(graph.replay, reps) / reps
    gbs_g = nl * 2.0 * HKV * Lkv * D * 2 / (gms * 1e-3) / 1e9
    extra["decode_1m"] = {"gb_per_s": gbs_g, "ms_per_step_28_layers": gms, "frac_of_measured_hbm": gbs_g / peaks["hbm"],
                          "frac_of_8tbs": gbs_g / 8000.0, "bytes_per_step": nl * 2 * HKV * Lkv * D * 2,
                          "launch": "CUDA graph replay of 28 layer calls (decode + merge kernels)", "gpu_launches_per_step": 2 * nl}


def leg_decode_1m_sp(ctx, extra, steps=5):
    """N GPUs: the 28-layer decode step at a 1,048,576-token context with the cache sharded by key ranges over the
    ranks (60 GB in all, 60/N GB per GPU): split-KV decode per rank, (partial O, LSE) exchange, merge.  Two routes:
    an NCCL all-gather + merge kernel (eager), and the fused peer-store exchange (two kernels per layer, the whole
    step replayed from a CUDA graph)."""
    from longcontext_sqattn_paddle_b200 import dist as sqdist
    dev, world, peaks = ctx.dev, ctx.world, ctx.peaks
    n_total, nl = 1 << 20, 28
    ls = n_total // world
    layers = [(torch.randn(1, HKV, ls, D, device=dev, dtype=torch.bfloat16),
               torch.randn(1, HKV, ls, D, device=dev, dtype=torch.bfloat16)) for _ in range(nl)]
    g = torch.Generator(device=dev).manual_seed(5)
    qd = torch.randn(1, HQ, 1, D, device=dev, dtype=torch.bfloat16, generator=g)
    nbytes = nl * 2.0 * HKV * n_total * D * 2
    res = {"context": n_total, "layers": nl, "kv_gb_total": nbytes / 1e9, "parallelism": f"kv-shard x{world}"}

    def step(ex):
        for kk, vv in layers:
            sqdist.sp_decode(qd, kk, vv, out_dtype=torch.bfloat16, exchange=ex)

    for _ in range(3):
        step(None)
    ms = ctx.timed(lambda: step(None), steps) / steps
    res["nccl"] = {"ms_per_token": ms, "aggregate_gb_per_s": nbytes / (ms * 1e-3) / 1e9,
                   "per_gpu_gb_per_s": nbytes / world / (ms * 1e-3) / 1e9,
                   "per_gpu_frac_of_measured_hbm": nbytes / world / (ms * 1e-3) / 1e9 / peaks["hbm"],
                   "launch": "eager: decode kernel, merge kernel, all_gather_into_tensor, merge kernel per layer"}
    ex = sqdist.PeerExchange(HQ, D)
    for _ in range(3):
        step(ex)
    graph = torch.cuda.CUDAGraph()
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        step(ex)
    torch.cuda.current_stream().wait_stream(side)
    ctx.barrier()
    with torch.cuda.graph(graph):
        step(ex)
    ctx.barrier()
    for _ in range(3):
        graph.replay()
    ms = ctx.timed(graph.replay, steps) / steps
    res["peer"] = {"ms_per_token": ms, "aggregate_gb_per_s": nbytes / (ms * 1e-3) / 1e9,
                   "per_gpu_gb_per_s": nbytes / world / (ms * 1e-3) / 1e9,
                   "per_gpu_frac_of_measured_hbm": nbytes / world / (ms * 1e-3) / 1e9 / peaks["hbm"],
                   "launch": "CUDA graph replay: decode kernel + one merge/peer-store/wait/merge kernel per layer"}
    extra["decode_1m_sp"] = res
    del layers


def leg_parity(ctx):
    """N > 1: max |difference| between what the N ranks compute together and the same computation on this GPU alone,
    on small seeded inputs every rank generates identically (4096 tokens for prefill, 16384 keys for decode)."""
    from longcontext_sqattn_paddle_b200 import _lib as L
    from longcontext_sqattn_paddle_b200 import dist as sqdist
    from longcontext_sqattn_paddle_b200 import ops
    from longcontext_sqattn_paddle_b200.sqattn.attn_replacer import mp_triton_wrapper
    dev, world, rank = ctx.dev, ctx.world, ctx.rank
    n = 4096
    q, k, v = make_inputs(77, n, device=dev)
    r8, r4 = [0.1] * HQ, [0.2] * HQ
    out = {}

    def rows(x, segs):
        return torch.cat([x[:, lo:hi] for lo, hi in segs], dim=1)

    single = mp_triton_wrapper(1, r8, r4, SINK, _Args())(_Layer(), q, k, v, None)
    for layout in ("balanced", "zigzag"):
        fn = sqdist.sp_prefill_wrapper(r8, r4, SINK, _Args(), seq_total=n, layout=layout)
        reach = sqdist._window_reach(r8, r4, True, n)
        segs = sqdist._resolve_layout(layout, n, world, reach, SINK).segments(rank)
        got = fn(_Layer(), rows(q, segs), rows(k, segs), rows(v, segs), None)
        out[f"prefill_windowed_{layout}"] = ctx.max_over_ranks((got.float() - rows(single, segs).float()).abs().max().item())
    dense_single = ops.prefill(q, k, q, k, v, mode=L.MODE_DENSE_CAUSAL, layout="NHD", out_dtype=torch.bfloat16).reshape(1, n, HQ * D)
    segs = sqdist.ShardLayout.zigzag(n, world).segments(rank)
    got = sqdist.sp_dense_wrapper(seq_total=n, layout="zigzag")(_Layer(), rows(q, segs), rows(k, segs), rows(v, segs), None)
    out["prefill_dense_zigzag"] = ctx.max_over_ranks((got.float() - rows(dense_single, segs).float()).abs().max().item())
    Lk = 16384
    g = torch.Generator(device=dev).manual_seed(78)
    qd = torch.randn(1, HQ, 1, D, device=dev, generator=g).to(torch.bfloat16)
    kd = torch.randn(1, HKV, Lk, D, device=dev, generator=g).to(torch.bfloat16)
    vd = torch.randn(1, HKV, Lk, D, device=dev, generator=g).to(torch.bfloat16)
    ref = ops.decode(qd, kd, vd, out_dtype=torch.bfloat16)
    ls = Lk // world
    ks, vs = kd[:, :, rank * ls:(rank + 1) * ls].contiguous(), vd[:, :, rank * ls:(rank + 1) * ls].contiguous()
    got = sqdist.sp_decode(qd, ks, vs, out_dtype=torch.bfloat16)
    out["decode_nccl"] = ctx.max_over_ranks((got.float() - ref.float()).abs().max().item())
    ex = sqdist.PeerExchange(HQ, D)
    for _ in range(3):     # both buffer parities
        got = sqdist.sp_decode(qd, ks, vs, out_dtype=torch.bfloat16, exchange=ex)
    out["decode_peer"] = ctx.max_over_ranks((got.float() - ref.float()).abs().max().item())
    torch.cuda.synchronize()
    ops.check_device_status()
    out["max"] = max(out.values())
    out["what"] = (f"max|dO| of the {world}-rank result against the same computation on one GPU; prefill: {n} tokens, "
                   f"windows 0.1/0.2, sink {SINK}; decode: {Lk} keys")
    return out


def leg_ttft(ctx, extra, steps=2):
    """The operator inside its caller: prefill of 131072 uniform-random token ids through the 28-layer decoder stand-in
    (random weights of the Qwen2.5-7B geometry; first and last layer dense causal, the others windowed, as the
    reference leaves them, sqattn/compress.py:162), to the first token's logits.  N > 1: zig-zag token shards."""
    ms = ttft_ms(ctx, SEQ_TOTAL, 28, warmup=1, steps=steps)
    extra["ttft_128k"] = {"ms": ms, "tokens_per_s": SEQ_TOTAL / (ms * 1e-3), "layers": 28, "seq_len": SEQ_TOTAL,
                          "dense_layers": [0, 27], "parallelism": f"sp{ctx.world} zig-zag" if ctx.world > 1 else "single",
                          "data": "uniform-random token ids, random weights", "steps": steps}


def ttft_ms(ctx, n_total, layers, warmup, steps):
    from longcontext_sqattn_paddle_b200 import ops
    from longcontext_sqattn_paddle_b200.model_hub import DecoderConfig, RandomInitDecoder, install_sequence_parallel
    from longcontext_sqattn_paddle_b200.sqattn import process_model
    world, rank, dev = ctx.world, ctx.rank, ctx.dev
    cfg = DecoderConfig.qwen2_5_7b(num_hidden_layers=layers)
    if n_total % (2 * world) or (world > 1 and (n_total // (2 * world)) % 128):
        raise SystemExit("--seq must split into 2 x gpus chunks of a multiple of 128 tokens")
    ns = n_total // world
    model = RandomInitDecoder(cfg, max_length=n_total + 8, device=dev, seed=0, seq_shard=(rank, world), shard_layout="zigzag")
    # the reference leaves the first and the last layer on dense attention (sqattn/compress.py:162)
    windows = {i: {"bit8": [RATIO] * HQ, "bit4": [RATIO] * HQ, "sink": SINK}
               for i in range(cfg.num_hidden_layers) if 0 < i < cfg.num_hidden_layers - 1}
    if world > 1:
        from longcontext_sqattn_paddle_b200.dist import ShardLayout
        install_sequence_parallel(model, windows, _Args())
        segs = ShardLayout.zigzag(n_total, world).segments(rank)
    else:
        process_model(model, "SQAttn", windows, _Args())
        segs = [(0, n_total)]
    g = torch.Generator().manual_seed(7)
    all_ids = torch.randint(0, cfg.vocab_size, (1, n_total), generator=g)
    ids = torch.cat([all_ids[:, lo:hi] for lo, hi in segs], dim=1).pin_memory()
    model.batch_size, model.max_new_length = 1, 8
    times = []
    for it in range(warmup + steps):
        model.init_kv_cache(ns, (0,))
        ctx.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        logits = model.prefill_forward(ids.to(dev, non_blocking=True))
        logits.argmax(dim=-1)
        e1.record()
        ctx.barrier()
        if it >= warmup:
            times.append(ctx.max_over_ranks(e0.elapsed_time(e1)))
        model.kv_cache = None
    ops.check_device_status()
    del model
    torch.cuda.empty_cache()
    return sum(times) / len(times)


def run_ours(args):
    from longcontext_sqattn_paddle_b200 import ops
    from longcontext_sqattn_paddle_b200 import _lib as L
    from longcontext_sqattn_paddle_b200.sqattn.attn_replacer import mp_triton_wrapper

    ctx = _Ctx(args)
    world, rank, dev, peaks, dist = ctx.world, ctx.rank, ctx.dev, ctx.peaks, ctx.dist
    n_total = SEQ_TOTAL
    r = [RATIO] * HQ
    w = window_size(RATIO, n_total)
    flops_total = 4.0 * D * HQ * visited_pairs(n_total, w, SINK)
    parity = leg_parity(ctx) if world > 1 else None

    if world == 1:
        fn = mp_triton_wrapper(1, r, r, SINK, _Args())
        op = lambda q, k, v: fn(_Layer(), q, k, v, None)
        segs = [(0, n_total)]
    else:
        from longcontext_sqattn_paddle_b200 import dist as sqdist
        spfn = sqdist.sp_prefill_wrapper(r, r, SINK, _Args(), seq_total=n_total, layout="balanced")
        op = lambda q, k, v: spfn(_Layer(), q, k, v, None)
        segs = sqdist.ShardLayout.balanced(n_total, world, w, SINK).segments(rank)
    launches_per_step = 6   # column sums (2), quantise V, K and Q, attention
    ns = sum(hi - lo for lo, hi in segs)

    # synthetic input: this rank's rows of the sequence, resident in HBM and mirrored in pinned host memory
    dq, dk, dv = make_inputs(1000 + rank, ns, device=dev)
    hq_, hk_, hv_ = (torch.empty(t.shape, dtype=t.dtype).pin_memory() for t in (dq, dk, dv))
    for h_, d_ in ((hq_, dq), (hk_, dk), (hv_, dv)):
        h_.copy_(d_)
    torch.cuda.synchronize()

    # ---- device-resident throughput
    for _ in range(max(args.warmup, 3)):
        out = op(dq, dk, dv)
    ops.check_device_status()
    sampler = ClockSampler(ctx.local)
    if rank == 0:
        sampler.start()
    ms = ctx.timed(lambda: op(dq, dk, dv), args.steps)
    clocks = sampler.stop() if rank == 0 else None
    ops.check_device_status()
    ms_per_step = ms / args.steps
    value = flops_total / (ms_per_step * 1e-3) / 1e12

    # ---- end to end: pinned host buffers in, host buffer out, copies inside the timed region
    hout = torch.empty(out.shape, dtype=out.dtype).pin_memory()
    if world == 1:
        from longcontext_sqattn_paddle_b200.sqattn import HostPrefillPipeline
        pipe = HostPrefillPipeline(r, r, SINK, _Args(), chunk_rows=8192)
        e2e_step = lambda: pipe(hq_, hk_, hv_, hout)
        e2e_api = "HostPrefillPipeline (chunked H2D / kernels / D2H on three streams)"
    else:
        sp_pipe = sqdist.SPHostPrefillPipeline(r, r, SINK, _Args(), seq_total=n_total, layout="balanced", chunk_rows=4096)
        e2e_step = lambda: sp_pipe(hq_, hk_, hv_, hout)
        e2e_api = "SPHostPrefillPipeline (K/V upload + exchange once, Q chunks / kernels / D2H overlapped on three streams)"
    for _ in range(2):
        e2e_step()
    torch.cuda.synchronize()
    e2e_ok = bool(torch.equal(hout, out.cpu()))
    e2e_steps = max(3, args.steps // 2)
    ms_e2e = ctx.timed(e2e_step, e2e_steps) / e2e_steps
    e2e = {"value": flops_total / (ms_e2e * 1e-3) / 1e12, "unit": "TFLOP/s", "ms_per_step": ms_e2e,
           "h2d_bytes_per_step": (dq.numel() + dk.numel() + dv.numel()) * 2, "d2h_bytes_per_step": out.numel() * 2,
           "bytes_are": "per rank", "api": e2e_api, "matches_device_path": e2e_ok, "steps": e2e_steps,
           "cpu_cores_bound_to_gpu": ctx.cpu_cores_bound}
    del hout

    # ---- roofline of the dominant kernel: the attention kernel alone on this rank's rows (events on its stream)
    extra = {}
    if world == 1:
        q8, _, k8, _, v8 = ops.prep_qkv(dq, dk, dv, skip_bit4=True)
        o4 = torch.empty(1, ns, HQ, D, dtype=torch.bfloat16, device=dev)
        kern = lambda: ops.prefill(q8, k8, q8, k8, v8, mode=L.MODE_RELATIVE_WINDOW, win8=r, win4=r, sink=SINK,
                                   q_is_scaled=True, out=o4, out_layout="NHD")
        my_flops = flops_total
    else:
        st = spfn.state      # the operator's own prepared K/V (own rows + halo) of the last call
        q8, _ = sqdist.CudaBackend().prep_q(dq, "int", False)
        be = sqdist.CudaBackend()
        kern = lambda: be.windowed_prefill(q8, None, st["k8"], None, st["v8"], r, r, SINK, segs, True, 0)
        my_flops = 4.0 * D * HQ * sum(block_pairs(b, w, SINK) for lo, hi in segs for b in range(lo // 64, hi // 64))
    for _ in range(3):
        kern()
    torch.cuda.synchronize()
    time.sleep(1.0)  # the kernel is timed alone: let the power-cap state of the preceding loops decay first
    rsampler = ClockSampler(ctx.local)
    if rank == 0:
        rsampler.start()
    # Two timings of the same launch.  Burst: three launches after the pause (about 70 ms of work, before the 1 kW power
    # cap pulls the clocks down), compared with the burst bf16 peak, which was measured the same way (sub-millisecond
    # GEMMs); sustained: a longer loop, compared with the peak measured in a seconds-long GEMM loop under the cap.
    ksteps = 3
    ctx.barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(ksteps):
        kern()
    e1.record()
    ctx.barrier()
    my_ms = e0.elapsed_time(e1) / ksteps
    rclocks = rsampler.stop() if rank == 0 else None
    lsteps = max(6, args.steps)
    for _ in range(lsteps // 2):
        kern()
    ssampler = ClockSampler(ctx.local)
    if rank == 0:
        ssampler.start()
    e0.record()
    for _ in range(lsteps):
        kern()
    e1.record()
    ctx.barrier()
    my_sus_ms = e0.elapsed_time(e1) / lsteps
    sus_ms = ctx.max_over_ranks(my_sus_ms)
    sus_ach = -ctx.max_over_ranks(-(my_flops / (my_sus_ms * 1e-3) / 1e12))   # the slowest GPU's rate
    sclocks = ssampler.stop() if rank == 0 else None
    ops.check_device_status()
    my_ach = my_flops / (my_ms * 1e-3) / 1e12
    worst = -ctx.max_over_ranks(-my_ach)          # the slowest GPU's rate
    kms = ctx.max_over_ranks(my_ms)
    # DRAM traffic of one launch: dram__bytes_read.sum + dram__bytes_write.sum of the ncu capture summarised in
    # profiles/ for this kernel (taken at 32768 tokens; its ratio to the algorithmic Q+K+V+O bytes is read from that file), scaled to
    # this launch by the algorithmic bytes, which grow with the rows like the traffic does
    alg_bytes = 2.0 * D * (2 * HQ * ns + 2 * HKV * min(n_total, ns + w + SINK))
    traffic_ratio, traffic_src = captured_traffic_ratio()
    roof = {"bound": "tensor", "kernel": "prefill_kernel<128> (relative windows)" + (", per GPU, slowest rank" if world > 1 else ""),
            "achieved": worst, "clocks": rclocks, "peak": peaks["tflops"], "unit": "TFLOP/s", "frac": worst / peaks["tflops"],
            "peak_source": peaks["src"], "ms_per_launch": kms, "seq_len": n_total, "rows_this_rank": ns,
            "algorithmic_bytes": alg_bytes, "traffic": (traffic_ratio * alg_bytes) if traffic_ratio else None,
            "traffic_unit": "bytes per launch (ncu capture at 32768 tokens scaled by algorithmic bytes)",
            "traffic_source": traffic_src,
            "timing": f"average of {ksteps} launches after a 1 s pause (burst)",
            "sustained": {"achieved": sus_ach, "ms_per_launch": sus_ms, "launches": lsteps, "peak": peaks["tflops_sustained"],
                          "clocks": sclocks, "frac": sus_ach / peaks["tflops_sustained"]}}
    del q8

    # ---- the other configurations of the metric, one key each
    if world == 1:
        del k8, v8, o4
        try:
            sq_, sk_, sv_ = make_inputs(2000, SEQ_SMALL, device=dev)
            for _ in range(3):
                op(sq_, sk_, sv_)
            sms = ctx.timed(lambda: op(sq_, sk_, sv_), args.steps) / args.steps
            sflops = 4.0 * D * HQ * visited_pairs(SEQ_SMALL, window_size(RATIO, SEQ_SMALL), SINK)
            q8, _, k8, _, v8 = ops.prep_qkv(sq_, sk_, sv_, skip_bit4=True)
            o4 = torch.empty(1, SEQ_SMALL, HQ, D, dtype=torch.bfloat16, device=dev)
            skern = lambda: ops.prefill(q8, k8, q8, k8, v8, mode=L.MODE_RELATIVE_WINDOW, win8=r, win4=r, sink=SINK,
                                        q_is_scaled=True, out=o4, out_layout="NHD")
            for _ in range(3):
                skern()
            torch.cuda.synchronize()
            time.sleep(1.0)   # like the headline kernel: a short run after a pause, compared with the burst peak
            ksteps32 = min(args.steps, 10)
            skms = ctx.timed(skern, ksteps32) / ksteps32
            extra["prefill_32k"] = {"operator_tflops": sflops / (sms * 1e-3) / 1e12, "operator_ms": sms,
                                    "kernel_tflops": sflops / (skms * 1e-3) / 1e12, "kernel_ms": skms,
                                    "kernel_frac_of_bf16_peak": sflops / (skms * 1e-3) / 1e12 / peaks["tflops"]}
            dense = lambda: ops.prefill(q8, k8, q8, k8, v8, mode=L.MODE_DENSE_CAUSAL, q_is_scaled=True, out=o4, out_layout="NHD")
            for _ in range(2):
                dense()
            torch.cuda.synchronize()
            time.sleep(1.0)
            dsteps = max(2, min(args.steps // 2, 5))
            dms = ctx.timed(dense, dsteps) / dsteps
            dflops = 4.0 * D * HQ * (SEQ_SMALL * (SEQ_SMALL + 1) / 2)
            extra["dense_causal"] = {"tflops": dflops / (dms * 1e-3) / 1e12, "ms": dms, "seq_len": SEQ_SMALL,
                                     "frac_of_bf16_peak": dflops / (dms * 1e-3) / 1e12 / peaks["tflops"]}
            del q8, k8, v8, o4, sq_, sk_, sv_
        except Exception as e:  # noqa: BLE001
            extra["prefill_32k"] = {"error": repr(e)}
    del dq, dk, dv, out
    torch.cuda.empty_cache()
    try:
        if world == 1:
            leg_decode_1m(ctx, extra)
        else:
            leg_decode_1m_sp(ctx, extra)
    except Exception as e:  # noqa: BLE001
        extra["decode_1m" if world == 1 else "decode_1m_sp"] = {"error": repr(e)}
    ops.check_device_status()
    torch.cuda.empty_cache()
    if not args.no_ttft:
        try:
            leg_ttft(ctx, extra)
        except Exception as e:  # noqa: BLE001
            extra["ttft_128k"] = {"error": repr(e)}

    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu:
        cpu = cpu_sample(0, n_total, nblocks=8)
        cpu["config1"] = cpu_config1()

    if rank == 0:
        res = {"metric": "sqattn_prefill_tflops", "value": value, "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps,
               "warmup": max(args.warmup, 3), "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "strong",
               "vs_baseline": None, "dtype": "bf16", "data": "synthetic", "config": workload_config(n_total, world),
               "clocks": clocks, "e2e": e2e, "gpu_launches": launches_per_step * args.steps,
               "roofline": roof, "cpu_baseline": cpu}
        if parity is not None:
            res["parity"] = parity
        res.update(extra)
        print(json.dumps(res))
    if world > 1:
        dist.destroy_process_group()


def run_kernel_only(args):
    """A few launches of one kernel on the bench's tensors: the command profiler captures are taken on."""
    from longcontext_sqattn_paddle_b200 import _lib as L
    from longcontext_sqattn_paddle_b200 import ops

    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    n = args.seq
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    if args.kernel_only == "decode":
        kk = torch.randn(1, HKV, n, D, device=dev, dtype=torch.bfloat16)
        vv = torch.randn(1, HKV, n, D, device=dev, dtype=torch.bfloat16)
        qd = torch.randn(1, HQ, 1, D, device=dev, dtype=torch.bfloat16)
        fn = lambda: ops.decode(qd, kk, vv, out_dtype=torch.bfloat16)
        work, unit = 2.0 * HKV * n * D * 2 / 1e9, "GB/s"
    elif args.kernel_only == "kmeans":
        # one Lloyd iteration (assign + exact re-check + member sums + update) of the clustering of --seq keys per KV head
        # of the Llama-3-8B geometry into seq/64 centroids: 2*T*K*D flops of assignment work per head
        from longcontext_sqattn_paddle_b200.cache_hub import kmeans as km
        from longcontext_sqattn_paddle_b200.cache_hub.retrieval import num_clusters_for
        g8, kc = 8, num_clusters_for(n)
        g = torch.Generator(device=dev).manual_seed(3)
        keys = torch.randn(g8, n, D, device=dev, dtype=torch.bfloat16, generator=g)
        cent = keys[:, km.init_centroid_indices(n, kc, dev)].contiguous()
        fn = lambda: km.k_means_train(keys, cent, True)
        work, unit = 2.0 * g8 * n * kc * D / 1e12, "TFLOP/s"
    elif args.kernel_only == "window":
        # the blockwise attention-energy histogram of one layer (28 heads) at --seq tokens: 2*D flops per causal pair
        from longcontext_sqattn_paddle_b200.sqattn import window_search as ws
        g = torch.Generator(device=dev).manual_seed(4)
        qw = torch.randn(HQ, n, D, device=dev, dtype=torch.bfloat16, generator=g)
        kw = torch.randn(HKV, n, D, device=dev, dtype=torch.bfloat16, generator=g)
        fn = lambda: ws.attention_histograms(qw, kw, relative=True, num_bins=200, sink_len=SINK)
        work, unit = 2.0 * 2 * D * HQ * (n * (n + 1) / 2) / 1e12, "TFLOP/s"    # two sweeps (maximum / sum, then weights)
    elif args.kernel_only == "retrieval":
        # select + gather + ragged decode for 4 clustered sequences of --seq tokens, 4096-token budget
        from longcontext_sqattn_paddle_b200.cache_hub import ClusteredKV, RaggedClusteredDecoder
        caches = [ClusteredKV(torch.randn(8, n, D, device=dev, dtype=torch.bfloat16),
                              torch.randn(8, n, D, device=dev, dtype=torch.bfloat16), 64, 3) for _ in range(4)]
        dec = RaggedClusteredDecoder(caches, budget=4096, p_fp8=True)
        qd = torch.randn(4, 32, 1, D, device=dev, dtype=torch.bfloat16)
        fn = lambda: dec.step(qd)
        work, unit = 4.0, "sequences"
    elif args.kernel_only == "merge":
        # split-KV decode with both merge kernels: the plain one, and the cross-GPU one run as a world of one rank (its
        # exchange buffers are ordinary local memory here), so that its instruction stream can be profiled on one GPU
        import ctypes as C
        kk = torch.randn(1, HKV, n, D, device=dev, dtype=torch.bfloat16)
        vv = torch.randn(1, HKV, n, D, device=dev, dtype=torch.bfloat16)
        qd = torch.randn(1, HQ, 1, D, device=dev, dtype=torch.bfloat16)
        data = torch.zeros(L.lib.sqattn_peer_merge_data_bytes(1, HQ, D) // 4, dtype=torch.int32, device=dev)
        flags = torch.zeros(L.lib.sqattn_peer_merge_flag_bytes(1, HQ) // 4, dtype=torch.int32, device=dev)
        epoch = torch.zeros(1, dtype=torch.int32, device=dev)
        outp = torch.empty(HQ, D, dtype=torch.bfloat16, device=dev)
        pa = L.PeerMergeArgs()
        pa.peer_data[0], pa.peer_flags[0] = data.data_ptr(), flags.data_ptr()
        pa.rank, pa.world, pa.rows, pa.rows_cap, pa.head_dim, pa.epoch = 0, 1, HQ, HQ, D, epoch.data_ptr()
        pa.out, pa.o_dtype = outp.data_ptr(), L.BF16

        def fn():
            ops.decode(qd, kk, vv, out_dtype=torch.bfloat16)
            ops.decode(qd, kk, vv, peer=pa)
        work, unit = 2 * 2.0 * HKV * n * D * 2 / 1e9, "GB/s"
    elif args.kernel_only == "prep":
        dq, dk, dv = make_inputs(1000, n, device=dev)
        fn = lambda: ops.prep_qkv(dq, dk, dv, skip_bit4=True)
        # one read and one write of Q, K and V (the K mean pass reads K once more)
        work, unit = 2.0 * 2 * n * (HQ + 2 * HKV) * D / 1e9, "GB/s"
    else:
        dq, dk, dv = make_inputs(1000, n, device=dev)
        q8, _, k8, _, v8 = ops.prep_qkv(dq, dk, dv, skip_bit4=True)
        del dq, dk, dv
        o4 = torch.empty(1, n, HQ, D, dtype=torch.bfloat16, device=dev)
        r = [RATIO] * HQ
        if args.kernel_only == "prefill":
            fn = lambda: ops.prefill(q8, k8, q8, k8, v8, mode=L.MODE_RELATIVE_WINDOW, win8=r, win4=r, sink=SINK,
                                     q_is_scaled=True, out=o4, out_layout="NHD")
            work = 4.0 * D * HQ * visited_pairs(n, window_size(RATIO, n), SINK) / 1e12
        else:
            fn = lambda: ops.prefill(q8, k8, q8, k8, v8, mode=L.MODE_DENSE_CAUSAL, q_is_scaled=True, out=o4,
                                     out_layout="NHD")
            work = 4.0 * D * HQ * (n * (n + 1) / 2) / 1e12
        unit = "TFLOP/s"
    for _ in range(args.warmup):
        fn()
    torch.cuda.synchronize()
    e0.record()
    for _ in range(args.steps):
        fn()
    e1.record()
    torch.cuda.synchronize()
    ops.check_device_status()
    ms = e0.elapsed_time(e1) / args.steps
    print(json.dumps({"kernel": args.kernel_only, "seq": n, "ms_per_launch": ms, "rate": work / (ms * 1e-3), "unit": unit}))


def run_decoder(args):
    """The operator inside its caller: a random-weight decoder of the Qwen2.5-7B geometry.
    --workload ttft: prefill of --seq uniform-random token ids (sharded over the ranks, sequence parallel), time to
    the first token's logits.  --workload decode_model: decode steps at a --seq-token context (cache filled with
    N(0,1) keys/values), one new token per step through all layers."""
    import torch.distributed as dist

    from longcontext_sqattn_paddle_b200.model_hub import DecoderConfig, RandomInitDecoder, install_sequence_parallel
    from longcontext_sqattn_paddle_b200.sqattn import process_model

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if args.gpus > 1 and world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} needs torchrun with {args.gpus} ranks (WORLD_SIZE={world})")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    cfg = DecoderConfig.qwen2_5_7b(num_hidden_layers=args.layers)
    n_total = args.seq

    class Args:
        qk_qtype, v_qtype, use_relative_distance = "int", "int", True

    def sync_all():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def max_ms(ms):
        t = torch.tensor([ms], device=dev)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return t.item()

    if args.workload == "ttft":
        ctx = _Ctx.__new__(_Ctx)   # the rank / device / timing helpers, on the process group initialised above
        ctx.dist, ctx.world, ctx.rank, ctx.local, ctx.dev, ctx.peaks = dist, world, rank, local, dev, load_peaks()
        ms = ttft_ms(ctx, n_total, cfg.num_hidden_layers, args.warmup, args.steps)
        if rank == 0:
            print(json.dumps({"workload": "decoder_prefill_ttft", "metric": "ttft_ms", "value": ms, "unit": "ms",
                              "higher_is_better": False, "n_gpus": world, "seq_len": n_total, "layers": cfg.num_hidden_layers,
                              "tokens_per_s": n_total / (ms * 1e-3), "steps": args.steps, "warmup": args.warmup,
                              "parallelism": f"sp{world} zig-zag" if world > 1 else "single",
                              "dense_layers": [0, cfg.num_hidden_layers - 1],
                              "data": "synthetic uniform-random token ids, random weights",
                              "window": {"sink": SINK, "ratio": RATIO}, "dtype": "bf16"}))
    else:
        new_tokens = args.warmup + 2 * args.steps + 8
        model = RandomInitDecoder(cfg, max_length=n_total + new_tokens, device=dev, seed=0)
        model.batch_size, model.max_new_length = 1, new_tokens
        model.init_kv_cache(n_total, (0,))
        kc = model.kv_cache
        if not kc.allocated:
            raise SystemExit("the cache does not fit this GPU")
        for ldx in range(cfg.num_hidden_layers):
            kc.key_cache[ldx].normal_()
            kc.value_cache[ldx].normal_()
        kc.valid_length = torch.full((1,), n_total, dtype=torch.int64, device=dev)
        kc.valid_length_host = [n_total]
        kc.context = n_total
        tok = torch.zeros(1, 1, dtype=torch.int64, device=dev)
        for _ in range(args.warmup):
            tok = model.decode_forward(tok).argmax(dim=-1)
        sync_all()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(args.steps):
            tok = model.decode_forward(tok).argmax(dim=-1)
        e1.record()
        sync_all()
        eager_ms = e0.elapsed_time(e1) / args.steps
        # the same step captured once and replayed: position, cache lengths and the write index advance on the GPU
        model.max_new_length += args.steps + 4
        model.capture_decode_step(1)
        for _ in range(2):
            tok = model.decode_forward_graph(tok).argmax(dim=-1)
        sync_all()
        e0.record()
        for _ in range(args.steps):
            tok = model.decode_forward_graph(tok).argmax(dim=-1)
        e1.record()
        sync_all()
        from longcontext_sqattn_paddle_b200 import ops
        ops.check_device_status()
        ms = e0.elapsed_time(e1) / args.steps
        kv_bytes = 2.0 * cfg.num_hidden_layers * HKV * D * 2 * n_total
        w_bytes = 2.0 * sum(t.numel() for l in model.layers for t in (l.wqkv, l.wo, l.gate_up_proj, l.down_proj)) \
            + 2.0 * model.lm_head.numel()
        print(json.dumps({"workload": "decoder_decode", "metric": "decode_ms_per_token", "value": ms, "unit": "ms",
                          "higher_is_better": False, "n_gpus": 1, "context": n_total, "layers": cfg.num_hidden_layers,
                          "tokens_per_s": 1e3 / ms, "hbm_gbs": (kv_bytes + w_bytes) / (ms * 1e-3) / 1e9,
                          "launch": "CUDA graph replay of the whole step", "eager_ms_per_token": eager_ms,
                          "kv_gb": kv_bytes / 1e9, "weights_gb": w_bytes / 1e9, "steps": args.steps,
                          "warmup": args.warmup, "data": "synthetic N(0,1) cache, random weights", "dtype": "bf16"}))
    if world > 1:
        dist.destroy_process_group()


def run_decode_variants(args):
    """Decode-side workloads next to the headline line.
    --workload decode_sp: one decode step = 28 layers of split-KV attention over a --seq-token context whose keys
      are sharded over the ranks (partial O + LSE per rank, one all-gather, one merge kernel per layer).
    --workload decode_hybrid: --layers layers of a --seq-token cache with 75 % of the blocks in pinned host memory,
      staged to the GPU by a side stream while the previous layer computes.
    --workload retrieval: ragged batch of 16 sequences (context log-uniform in [8K, 256K]), Llama-3-8B geometry,
      keys clustered per KV head into len/64 centroids (10 Lloyd iterations), 4096-token budget, FP8 P."""
    import math
    import torch.distributed as dist

    from longcontext_sqattn_paddle_b200 import dist as sqdist
    from longcontext_sqattn_paddle_b200 import ops
    from longcontext_sqattn_paddle_b200.cache_hub import ClusteredKV, HybridKVCache, RaggedClusteredDecoder

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)

    def sync_all():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(fn, steps):
        sync_all()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            fn()
        e1.record()
        sync_all()
        t = torch.tensor([e0.elapsed_time(e1) / steps], device=dev)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return t.item()

    res = None
    if args.workload == "decode_sp":
        n_total, nl = args.seq, args.layers
        ls = n_total // world
        layers = [(torch.randn(1, HKV, ls, D, device=dev, dtype=torch.bfloat16),
                   torch.randn(1, HKV, ls, D, device=dev, dtype=torch.bfloat16)) for _ in range(nl)]
        g = torch.Generator(device=dev).manual_seed(5)
        qd = torch.randn(1, HQ, 1, D, device=dev, dtype=torch.bfloat16, generator=g)

        ex = sqdist.PeerExchange(HQ, D) if (args.exchange == "peer" and world > 1) else None

        def step():
            for kk, vv in layers:
                sqdist.sp_decode(qd, kk, vv, out_dtype=torch.bfloat16, exchange=ex)

        for _ in range(max(args.warmup, 3)):
            step()
        ms = timed(step, args.steps)
        eager_ms = ms
        if ex is not None:
            # the whole step (28 x decode, split merge, step-counter advance, peer merge) replayed from a CUDA graph:
            # no host work and no collective-library call between the layers
            graph = torch.cuda.CUDAGraph()
            side = torch.cuda.Stream()
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side):
                step()
            torch.cuda.current_stream().wait_stream(side)
            sync_all()
            with torch.cuda.graph(graph):
                step()
            sync_all()
            for _ in range(3):
                graph.replay()
            ms = timed(graph.replay, args.steps)
        nbytes = nl * 2.0 * HKV * n_total * D * 2
        res = {"workload": "decode_split_kv", "metric": "decode_attention_ms_per_token", "value": ms, "unit": "ms",
               "higher_is_better": False, "n_gpus": world, "context": n_total, "layers": nl,
               "aggregate_gb_per_s": nbytes / (ms * 1e-3) / 1e9, "eager_ms": eager_ms,
               "launch": "CUDA graph replay" if ex is not None else "eager", "kv_gb_total": nbytes / 1e9, "steps": args.steps,
               "parallelism": f"kv-shard x{world}", "exchange": "peer stores in the merge kernel" if ex is not None else "nccl all-gather + merge kernel", "data": "synthetic N(0,1) cache", "dtype": "bf16"}
    elif args.workload == "decode_hybrid":
        n_total, nl = args.seq, args.layers
        cache = HybridKVCache(nl, 1, n_total, HKV, D, torch.bfloat16, gpu_fraction=0.25, device=dev)
        for ldx in range(nl):
            cache.k_res[ldx].normal_()
            cache.v_res[ldx].normal_()
            for host in (cache.k_host[ldx], cache.v_host[ldx]):  # filled from the GPU: a CPU generator is slow
                host.copy_(torch.randn(host.shape, device=dev, dtype=torch.bfloat16))
        qd = torch.randn(1, HQ, 1, D, device=dev, dtype=torch.bfloat16)

        def step():
            cache.prefetch(0)
            for ldx in range(nl):
                cache.decode_attention(qd, ldx)

        for _ in range(2):
            step()
        ms = timed(step, max(2, min(args.steps, 5)))
        host_bytes = nl * 2.0 * HKV * cache.host_tokens * D * 2
        res = {"workload": "decode_hybrid_cache", "metric": "decode_attention_ms_per_token", "value": ms, "unit": "ms",
               "higher_is_better": False, "n_gpus": 1, "context": n_total, "layers": nl, "host_fraction": cache.host_tokens / n_total,
               "host_gb_per_step": host_bytes / 1e9, "h2d_gb_per_s": host_bytes / (ms * 1e-3) / 1e9,
               "data": "synthetic N(0,1) cache", "dtype": "bf16"}
    else:
        hq, hkv = 32, 8
        g = torch.Generator().manual_seed(11)
        u = torch.rand(16, generator=g)
        lens = [int(math.exp(math.log(8192) + float(x) * (math.log(262144) - math.log(8192)))) // 64 * 64 for x in u]
        # The sequences are independent: with N ranks each rank clusters and serves its own (the longest are dealt
        # first, back and forth over the ranks, so that the token counts are close); no data-path collective.
        order = sorted(range(16), key=lambda i: -lens[i])
        mine = [i for pos, i in enumerate(order) if (pos % world if (pos // world) % 2 == 0 else world - 1 - pos % world) == rank]
        gens = {i: torch.Generator(device=dev).manual_seed(100 + i) for i in mine}
        kd = [(torch.randn(hkv, lens[i], D, device=dev, dtype=torch.bfloat16, generator=gens[i]),
               torch.randn(hkv, lens[i], D, device=dev, dtype=torch.bfloat16, generator=gens[i])) for i in mine]
        ClusteredKV(kd[0][0][:, :8192].contiguous(), kd[0][1][:, :8192].contiguous(), 64, 2)   # first-use set-up of the kernels
        sync_all()
        t0 = time.perf_counter()
        caches = [ClusteredKV(k_, v_, 64, 10) for k_, v_ in kd]
        torch.cuda.synchronize()
        tb = torch.tensor([time.perf_counter() - t0], device=dev)
        if world > 1:
            dist.all_reduce(tb, op=dist.ReduceOp.MAX)
        build_s = tb.item()
        del kd
        dec = RaggedClusteredDecoder(caches, budget=4096, p_fp8=True)
        qd = torch.randn(len(mine), hq, 1, D, device=dev, dtype=torch.bfloat16)
        for _ in range(max(args.warmup, 3)):
            dec.step(qd)
        ms = timed(lambda: dec.step(qd), args.steps)
        res = {"workload": "ragged_clustered_decode", "metric": "tokens_per_s", "value": 16 / (ms * 1e-3), "unit": "tokens/s",
               "higher_is_better": True, "n_gpus": world, "scaling": "strong", "ms_per_step": ms, "sequences": 16,
               "sequences_per_rank": "dealt by length, no collective on the data path", "context_lengths": lens,
               "geometry": "32 q / 8 kv heads, head_dim 128", "budget": 4096, "p_fp8": True,
               "cluster_build_s": build_s, "clustered_tokens": sum(lens), "attention_layers_per_step": 1,
               "data": "synthetic N(0,1) keys/values", "dtype": "bf16"}
    ops.check_device_status()
    if rank == 0:
        print(json.dumps(res))
    if world > 1:
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--no-ttft", action="store_true", help="skip the decoder stand-in's time-to-first-token leg")
    ap.add_argument("--kernel-only", choices=["prefill", "dense", "decode", "prep", "kmeans", "window", "retrieval", "merge"],
                    help="launch only this kernel --steps times on the bench tensors (for profiler captures)")
    ap.add_argument("--seq", type=int, default=None, help="sequence length for --kernel-only / --workload")
    ap.add_argument("--workload", default="operator", choices=["operator", "ttft", "decode_model", "decode_sp", "decode_hybrid", "retrieval"],
                    help="operator: the headline line; ttft / decode_model: the operator inside the decoder stand-in")
    ap.add_argument("--exchange", default="peer", choices=["peer", "nccl"], help="decode_sp: how the partials travel")
    ap.add_argument("--layers", type=int, default=28, help="decoder layers for --workload ttft / decode_model")
    args = ap.parse_args()
    if args.seq is None:
        args.seq = {"operator": SEQ_SMALL, "ttft": SEQ_TOTAL}.get(args.workload, 1048576)
    if args.kernel_only:
        run_kernel_only(args)
    elif args.workload in ("ttft", "decode_model"):
        run_decoder(args)
    elif args.workload != "operator":
        run_decode_variants(args)
    elif args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
