"""Benchmark of the SQAttn hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]

One "step" is one call of the prefill operator (input preparation + windowed attention kernel, i.e.
``layer.prefill_attention(q, k, v, None)``) on one batch of synthetic input with the shapes of the
reference's 32K-token Qwen2.5-7B attention call: batch 1, 28 query / 4 KV heads, head_dim 128, bf16,
Q,K,V ~ N(0,1) with four K channels scaled by 8, the reference's effective default window (sink 256,
int8/int4 window ratio 0.1).  The metric is TFLOP/s counted over the (query, key) pairs the kernel has to
visit (4*D flops per pair and head), never over padded tiles.  With N > 1 GPUs the sequence is N times
longer and sharded by query blocks (sequence parallel, K/V all-gathered over NCCL): weak scaling.

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
SEQ_PER_GPU = 32768
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
        return {"tflops": float(d["bf16_tflops"]), "hbm": float(d["hbm_gbs"]), "src": "measured"}
    return {"tflops": 1590.0, "hbm": 6650.0, "src": "fallback"}


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


# ----------------------------------------------------------------------------------------------- CPU arm
def cpu_sample(seed: int, n: int, nblocks: int = 16, reps: int = 1):
    """Time the oracle (the reference's fake-quant SQAttn path restated on CPU) on a bounded sample of the
    workload: input preparation over a 4096-token slice (scaled to the full length: it is linear in tokens)
    and `nblocks` of the n/64 query blocks for all 28 heads."""
    from oracle import sqattn_oracle as so

    torch.set_num_threads(os.cpu_count() or 1)
    q, k, v = so.make_inputs(seed, 1, n, HQ, HKV, D, torch.bfloat16)
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
    pairs = 0
    for b in blocks:
        qs, qe = b * 64, b * 64 + 64
        l8 = max(SINK, qe - w)
        pairs += 64 * min(SINK, qs) + (64 * (qs - l8) if l8 < qs else 0) + 64 * 65 // 2
    flops = 4.0 * D * HQ * pairs
    frac = len(blocks) / nblk
    total_t = best + t_prep * frac
    return {"value": flops / total_t / 1e12, "unit": "TFLOP/s", "cores": torch.get_num_threads(), "kind": "port",
            "sample": f"{len(blocks)} of {nblk} 64-row query blocks x {HQ} heads at N={n} (tile kernel {best:.2f}s) + "
                      f"the proportional share of input preparation ({t_prep:.2f}s for the full sequence, "
                      f"timed on a {sl}-token slice)",
            "seconds": total_t}


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
    n = SEQ_PER_GPU * args.gpus
    t_all = time.perf_counter()
    q, k, v = so.make_inputs(0, 1, n, HQ, HKV, D, torch.bfloat16)
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
        qs, qe = blk * 64, blk * 64 + 64
        l8 = max(SINK, qe - w)
        pairs = 64 * min(SINK, qs) + (64 * (qs - l8) if l8 < qs else 0) + 64 * 65 // 2
        if i >= args.warmup:
            vals.append(4.0 * D * HQ * pairs / dt / 1e12)
            secs.append(dt)
    wall = time.perf_counter() - t_all
    v_ = sum(vals) / len(vals)
    cb = {"value": v_, "unit": "TFLOP/s", "cores": torch.get_num_threads(), "kind": "port",
          "sample": f"one 64-row query block x {HQ} heads per step at N={n} (+ 1/{nblk} of the {t_prep:.2f}s input preparation)"}
    out = {"impl": "reference", "metric": "sqattn_prefill_tflops", "value": v_, "unit": "TFLOP/s", "n_gpus": args.gpus,
           "steps": args.steps, "warmup": args.warmup, "ms_per_step": sum(secs) / len(secs) * 1e3, "higher_is_better": True,
           "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
           "config": workload_config(n, args.gpus), "cpu_baseline": cb,
           "e2e": {"value": v_, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
           "wall_s": wall}
    print(json.dumps(out))


def workload_config(n, gpus):
    return {"workload": f"SQAttn prefill operator, batch 1, {HQ} q / {HKV} kv heads, head_dim {D}, seq {n}, causal, bf16, "
                        f"sink {SINK}, int8/int4 window ratio {RATIO} (the reference's effective default), K outlier channels x8",
            "seq_len": n, "parallelism": f"sp{gpus}" if gpus > 1 else "single",
            "l2": "inputs larger than L2 (Q alone is 235 MB per 32K tokens); no flush needed"}


# ----------------------------------------------------------------------------------------------- GPU arm
def run_ours(args):
    import torch.distributed as dist

    from longcontext_sqattn_paddle_b200 import ops
    from longcontext_sqattn_paddle_b200 import _lib as L
    from longcontext_sqattn_paddle_b200.sqattn.attn_replacer import mp_triton_wrapper
    from oracle import sqattn_oracle as so

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if args.gpus > 1 and world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} needs torchrun with {args.gpus} ranks (WORLD_SIZE={world})")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    n_total = SEQ_PER_GPU * world
    peaks = load_peaks()

    class Args:
        qk_qtype, v_qtype, use_relative_distance = "int", "int", True

    class Layer:
        num_key_value_groups = HQ // HKV

    r = [RATIO] * HQ
    if world == 1:
        fn = mp_triton_wrapper(1, r, r, SINK, Args())
        op = lambda q, k, v: fn(Layer(), q, k, v, None)
        launches_per_step = 6
    else:
        from longcontext_sqattn_paddle_b200 import dist as sqdist
        spfn = sqdist.sp_prefill_wrapper(r, r, SINK, Args(), seq_total=n_total)
        op = lambda q, k, v: spfn(Layer(), q, k, v, None)
        launches_per_step = 7

    # synthetic input: this rank's 32K-token shard of the sequence, pinned on the host and resident in HBM
    q, k, v = so.make_inputs(1000 + rank, 1, SEQ_PER_GPU, HQ, HKV, D, torch.bfloat16)
    hq_, hk_, hv_ = q.pin_memory(), k.pin_memory(), v.pin_memory()
    dq, dk, dv = hq_.to(dev), hk_.to(dev), hv_.to(dev)
    w = window_size(RATIO, n_total)
    flops_total = 4.0 * D * HQ * visited_pairs(n_total, w, SINK)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(fn_, steps):
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            fn_()
        e1.record()
        barrier()
        ms = torch.tensor([e0.elapsed_time(e1)], device=dev)
        if world > 1:
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        return ms.item()

    # ---- device-resident throughput
    for _ in range(max(args.warmup, 3)):
        out = op(dq, dk, dv)
    ops.check_device_status()
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    ms = timed(lambda: op(dq, dk, dv), args.steps)
    clocks = sampler.stop() if rank == 0 else None
    ops.check_device_status()
    ms_per_step = ms / args.steps
    value = flops_total / (ms_per_step * 1e-3) / 1e12

    # ---- end to end: pinned host buffers in, host buffer out, copies inside the timed region
    hout = torch.empty(out.shape, dtype=out.dtype).pin_memory()
    if world == 1:
        from longcontext_sqattn_paddle_b200.sqattn import HostPrefillPipeline
        pipe = HostPrefillPipeline(r, r, SINK, Args(), chunk_rows=4096)
        e2e_step = lambda: pipe(hq_, hk_, hv_, hout)
        e2e_api = "HostPrefillPipeline (chunked H2D / kernels / D2H on three streams)"
    else:
        def e2e_step():
            a, b_, c = hq_.to(dev, non_blocking=True), hk_.to(dev, non_blocking=True), hv_.to(dev, non_blocking=True)
            hout.copy_(op(a, b_, c), non_blocking=True)
        e2e_api = "copy in, sequence-parallel operator, copy out"

    for _ in range(2):
        e2e_step()
    torch.cuda.synchronize()
    e2e_ok = True
    if world == 1:
        e2e_ok = bool(torch.equal(hout, out.cpu()))
    ms_e2e = timed(e2e_step, args.steps) / args.steps
    e2e = {"value": flops_total / (ms_e2e * 1e-3) / 1e12, "unit": "TFLOP/s", "ms_per_step": ms_e2e,
           "h2d_bytes_per_step": (q.numel() + k.numel() + v.numel()) * 2, "d2h_bytes_per_step": out.numel() * 2,
           "api": e2e_api, "matches_device_path": e2e_ok}

    # ---- roofline of the dominant kernel (the attention kernel alone, events on its stream)
    roof = None
    extra = {}
    if world == 1:
        q8, _, k8, _, v8 = ops.prep_qkv(dq, dk, dv, skip_bit4=True)
        o4 = torch.empty(1, SEQ_PER_GPU, HQ, D, dtype=torch.bfloat16, device=dev)
        kern = lambda: ops.prefill(q8, k8, q8, k8, v8, mode=L.MODE_RELATIVE_WINDOW, win8=r, win4=r, sink=SINK,
                                   q_is_scaled=True, out=o4, out_layout="NHD")
        for _ in range(3):
            kern()
        torch.cuda.synchronize()
        time.sleep(1.0)  # the kernel is timed alone: let the power-cap state of the preceding loops decay first
        rsampler = ClockSampler(local)
        rsampler.start()
        kms = timed(kern, args.steps) / args.steps
        rclocks = rsampler.stop()
        ach = flops_total / (kms * 1e-3) / 1e12
        roof = {"bound": "tensor", "kernel": "prefill_kernel<128> (relative windows)", "achieved": ach, "clocks": rclocks,
                "peak": peaks["tflops"], "unit": "TFLOP/s", "frac": ach / peaks["tflops"], "peak_source": peaks["src"],
                "ms_per_launch": kms,
                # dram__bytes_read.sum + dram__bytes_write.sum of one launch from the ncu capture summarised in
                # profiles/prefill_kernel_relative_window_32k.md (algorithmic: Q+K+V+O = 537 MB)
                "traffic": 494.9e6, "traffic_unit": "bytes per launch"}
        # dense causal on the same tensors: the tensor-core-bound configuration
        dense = lambda: ops.prefill(q8, k8, q8, k8, v8, mode=L.MODE_DENSE_CAUSAL, q_is_scaled=True, out=o4, out_layout="NHD")
        for _ in range(2):
            dense()
        dms = timed(dense, max(2, args.steps // 2)) / max(2, args.steps // 2)
        dflops = 4.0 * D * HQ * (SEQ_PER_GPU * (SEQ_PER_GPU + 1) / 2)
        extra["dense_causal"] = {"tflops": dflops / (dms * 1e-3) / 1e12, "ms": dms,
                                 "frac_of_bf16_peak": dflops / (dms * 1e-3) / 1e12 / peaks["tflops"]}
        # decode: one 1M-token layer (K and V 1 GiB each) streamed per launch, four such layers in rotation
        try:
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
            dms_ = timed(dec, nl) / nl
            gbs = 2.0 * HKV * Lkv * D * 2 / (dms_ * 1e-3) / 1e9
            extra["decode_1m_eager"] = {"gb_per_s": gbs, "ms_per_layer": dms_}
            # one decode step = 28 layer launches; replayed from a CUDA graph so that host launch work
            # (descriptors, ctypes) is off the critical path
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
            gms = timed(graph.replay, reps) / reps
            gbs_g = nl * 2.0 * HKV * Lkv * D * 2 / (gms * 1e-3) / 1e9
            extra["decode_1m"] = {"gb_per_s": gbs_g, "ms_per_step_28_layers": gms, "frac_of_measured_hbm": gbs_g / peaks["hbm"],
                                  "frac_of_8tbs": gbs_g / 8000.0, "bytes_per_step": nl * 2 * HKV * Lkv * D * 2,
                                  "launch": "CUDA graph replay of 28 layer calls (decode + merge kernels)"}
            del layers
        except Exception as e:  # noqa: BLE001
            extra["decode_1m"] = {"error": repr(e)}
        ops.check_device_status()

    else:
        # every rank times the attention kernel on its own query shard against the gathered K/V; the slowest rank
        # sets the time, the figure is per GPU
        be = sqdist.CudaBackend()
        sums = be.k_column_sums(dk)
        dist.all_reduce(sums)
        q8, k8s, v8s = be.prep(dq, dk, dv, (sums / float(n_total)).contiguous(), "int", "int")
        k_full = torch.empty(1, n_total, HKV, D, dtype=k8s.dtype, device=dev)
        v_full = torch.empty(1, n_total, HKV, D, dtype=v8s.dtype, device=dev)
        dist.all_gather_into_tensor(k_full.view(n_total, HKV, D), k8s.view(SEQ_PER_GPU, HKV, D))
        dist.all_gather_into_tensor(v_full.view(n_total, HKV, D), v8s.view(SEQ_PER_GPU, HKV, D))
        kern = lambda: be.windowed_prefill(q8, k_full, v_full, r, r, SINK, rank * SEQ_PER_GPU, 0)
        for _ in range(3):
            kern()
        kms = timed(kern, args.steps) / args.steps
        ach = flops_total / world / (kms * 1e-3) / 1e12
        roof = {"bound": "tensor", "kernel": "prefill_kernel<128> (relative windows), per GPU, slowest rank",
                "achieved": ach, "peak": peaks["tflops"], "unit": "TFLOP/s", "frac": ach / peaks["tflops"],
                "peak_source": peaks["src"], "ms_per_launch": kms, "traffic": None}
        ops.check_device_status()

    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu:
        cpu = cpu_sample(0, SEQ_PER_GPU, nblocks=16)
        cpu.pop("seconds", None)

    if rank == 0:
        res = {"metric": "sqattn_prefill_tflops", "value": value, "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps,
               "warmup": max(args.warmup, 3), "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak",
               "vs_baseline": None, "dtype": "bf16", "data": "synthetic", "config": workload_config(n_total, world),
               "clocks": clocks, "e2e": e2e, "gpu_launches": launches_per_step * args.steps,
               "roofline": roof, "cpu_baseline": cpu}
        res.update(extra)
        print(json.dumps(res))
    if world > 1:
        dist.destroy_process_group()


def run_kernel_only(args):
    """A few launches of one kernel on the bench's tensors: the command profiler captures are taken on."""
    from longcontext_sqattn_paddle_b200 import _lib as L
    from longcontext_sqattn_paddle_b200 import ops
    from oracle import sqattn_oracle as so

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
    elif args.kernel_only == "prep":
        q, k, v = so.make_inputs(1000, 1, n, HQ, HKV, D, torch.bfloat16)
        dq, dk, dv = q.to(dev), k.to(dev), v.to(dev)
        fn = lambda: ops.prep_qkv(dq, dk, dv, skip_bit4=True)
        # one read and one write of Q, K and V (the K mean pass reads K once more)
        work, unit = 2.0 * 2 * n * (HQ + 2 * HKV) * D / 1e9, "GB/s"
    else:
        q, k, v = so.make_inputs(1000, 1, n, HQ, HKV, D, torch.bfloat16)
        q8, _, k8, _, v8 = ops.prep_qkv(q.to(dev), k.to(dev), v.to(dev), skip_bit4=True)
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
        if n_total % world or (world > 1 and (n_total // world) % 128):
            raise SystemExit("--seq must split into shards of a multiple of 128 tokens")
        ns = n_total // world
        model = RandomInitDecoder(cfg, max_length=n_total + 8, device=dev, seed=0, seq_shard=(rank, world))
        windows = {i: {"bit8": [RATIO] * HQ, "bit4": [RATIO] * HQ, "sink": SINK} for i in range(cfg.num_hidden_layers)}
        if world > 1:
            install_sequence_parallel(model, windows, Args())
        else:
            process_model(model, "SQAttn", windows, Args())
        g = torch.Generator().manual_seed(7)
        ids = torch.randint(0, cfg.vocab_size, (1, n_total), generator=g)[:, rank * ns:(rank + 1) * ns].pin_memory()
        model.batch_size, model.max_new_length = 1, 8
        times = []
        for it in range(args.warmup + args.steps):
            model.init_kv_cache(ns, (0,))
            sync_all()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            logits = model.prefill_forward(ids.to(dev, non_blocking=True))
            tok = logits.argmax(dim=-1)
            e1.record()
            sync_all()
            if it >= args.warmup:
                times.append(max_ms(e0.elapsed_time(e1)))
            model.kv_cache = None
        from longcontext_sqattn_paddle_b200 import ops
        ops.check_device_status()
        if rank == 0:
            ms = sum(times) / len(times)
            print(json.dumps({"workload": "decoder_prefill_ttft", "metric": "ttft_ms", "value": ms, "unit": "ms",
                              "higher_is_better": False, "n_gpus": world, "seq_len": n_total, "layers": cfg.num_hidden_layers,
                              "tokens_per_s": n_total / (ms * 1e-3), "steps": args.steps, "warmup": args.warmup,
                              "parallelism": f"sp{world}", "data": "synthetic uniform-random token ids, random weights",
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
        t0 = time.perf_counter()
        caches = []
        for ln in lens:
            caches.append(ClusteredKV(torch.randn(hkv, ln, D, device=dev, dtype=torch.bfloat16),
                                      torch.randn(hkv, ln, D, device=dev, dtype=torch.bfloat16), 64, 10))
        torch.cuda.synchronize()
        build_s = time.perf_counter() - t0
        dec = RaggedClusteredDecoder(caches, budget=4096, p_fp8=True)
        qd = torch.randn(16, hq, 1, D, device=dev, dtype=torch.bfloat16)
        for _ in range(max(args.warmup, 3)):
            dec.step(qd)
        ms = timed(lambda: dec.step(qd), args.steps)
        res = {"workload": "ragged_clustered_decode", "metric": "tokens_per_s", "value": 16 / (ms * 1e-3), "unit": "tokens/s",
               "higher_is_better": True, "n_gpus": 1, "ms_per_step": ms, "sequences": 16, "context_lengths": lens,
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
    ap.add_argument("--kernel-only", choices=["prefill", "dense", "decode", "prep"],
                    help="launch only this kernel --steps times on the bench tensors (for profiler captures)")
    ap.add_argument("--seq", type=int, default=None, help="sequence length for --kernel-only / --workload")
    ap.add_argument("--workload", default="operator", choices=["operator", "ttft", "decode_model", "decode_sp", "decode_hybrid", "retrieval"],
                    help="operator: the headline line; ttft / decode_model: the operator inside the decoder stand-in")
    ap.add_argument("--exchange", default="peer", choices=["peer", "nccl"], help="decode_sp: how the partials travel")
    ap.add_argument("--layers", type=int, default=28, help="decoder layers for --workload ttft / decode_model")
    args = ap.parse_args()
    if args.seq is None:
        args.seq = {"operator": SEQ_PER_GPU, "ttft": 131072}.get(args.workload, 1048576)
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
