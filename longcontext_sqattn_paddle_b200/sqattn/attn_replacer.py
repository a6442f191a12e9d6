"""The operator that replaces ``layer.prefill_attention`` (sqattn/attn_replacer.py:12-34, 296-454).

``process_model`` installs, and ``mp_triton_wrapper`` builds, an ``attention_fn(module, query, key, value,
attention_mask, dropout, scaling, sliding_window, **kwargs)`` with the reference's signature: query
[B,N,Hq,D], key/value [B,N,Hkv,D] in, [B,N,Hq*D] bf16 out; mask, dropout, scaling and sliding_window are
ignored and the softmax scale is always 1/sqrt(D), as in the reference."""
from __future__ import annotations

import types

import torch

from .. import _lib as L
from .. import ops


def process_model(model, method, window_sizes=None, args=None):
    """Install the SQAttn prefill operator on every layer listed in ``window_sizes``
    (``{layer: {"bit8": [...], "bit4": [...], "sink": 256}}``); the sink is fixed at 256 as in the reference."""
    if method == "SQAttn":
        for i in range(len(model.layers)):
            if i in window_sizes.keys():
                layer = model.layers[i]
                layer.prefill_attention = types.MethodType(
                    mp_triton_wrapper(i, args=args, bit8_window_sizes=window_sizes[i]["bit8"],
                                      bit4_window_sizes=window_sizes[i]["bit4"], sink_window_size=256), layer)
                model.layers[i] = layer
    elif method in ("SDPA", "FlashAttn"):
        pass
    else:
        raise ValueError(f"Unsupported attention type: {method}")
    return model


def _normalise_windows(bit8, bit4):
    """List/int normalisation of the factory arguments (attn_replacer.py:299-321)."""
    is_per_head = isinstance(bit8, list) or isinstance(bit4, list)
    if is_per_head:
        num_heads = len(bit8) if isinstance(bit8, list) else len(bit4)
        if isinstance(bit8, int):
            bit8 = [bit8] * num_heads
        if isinstance(bit4, int):
            bit4 = [bit4] * num_heads
        if bit8 is None:
            bit8 = [0] * num_heads
        if bit4 is None:
            bit4 = [0] * num_heads
    else:
        bit8 = bit8 or 0
        bit4 = bit4 or 0
    return bit8, bit4


def mp_triton_wrapper(layer_idx, bit8_window_sizes=0, bit4_window_sizes=0, sink_window_size=0, args=None,
                      p_fp8_mode="off"):
    bit8_window_sizes, bit4_window_sizes = _normalise_windows(bit8_window_sizes, bit4_window_sizes)
    fp8 = {"off": L.P_FP8_OFF, "all": L.P_FP8_ALL, "stage2": L.P_FP8_STAGE2}[p_fp8_mode]

    def attention_fn(module, query, key, value, attention_mask, dropout=0.0, scaling=1.0, sliding_window=None,
                     **kwargs):
        if args.qk_qtype not in L.QTYPE:
            raise ValueError(f"Invalid quantization type: {args.qk_qtype}")
        if args.v_qtype not in L.QTYPE:
            raise ValueError(f"Invalid quantization type: {args.v_qtype}")
        b, n, hq, d = query.shape
        relative = bool(args.use_relative_distance)
        # the relative launch never reads the int4 tensors (attn_triton_mix_relative.py:440-446): skip them
        q8, q4, k8, k4, v8 = ops.prep_qkv(query, key, value, qk_qtype=args.qk_qtype, v_qtype=args.v_qtype,
                                          skip_bit4=relative)
        out = torch.empty(b, n, hq * d, dtype=torch.bfloat16, device=query.device)
        o4 = out.view(b, n, hq, d)

        def per_head(w, conv):
            return [conv(w)] * hq if isinstance(w, (int, float)) else [conv(x) for x in w]

        if relative:
            ops.prefill(q8, k8, q8, k8, v8, mode=L.MODE_RELATIVE_WINDOW, win8=per_head(bit8_window_sizes, float),
                        win4=per_head(bit4_window_sizes, float), sink=sink_window_size, layout="HND",
                        p_fp8_mode=fp8, q_is_scaled=True, out=o4, out_layout="NHD")
        else:
            ops.prefill(q8, k8, q4, k4, v8, mode=L.MODE_ABSOLUTE_WINDOW, win8=per_head(bit8_window_sizes, int),
                        win4=per_head(bit4_window_sizes, int), sink=sink_window_size, layout="HND",
                        p_fp8_mode=fp8, q_is_scaled=True, out=o4, out_layout="NHD")
        return out

    return attention_fn


def chunk_bounds(n: int, chunk: int, edge: int):
    """Cuts ``n`` query rows into chunks for a copy / compute / copy pipeline: a short first chunk (``edge`` rows: its
    upload overlaps with nothing), full chunks of ``chunk`` rows, a short last chunk (its download overlaps with
    nothing).  Every chunk starts on a multiple of 128 rows; sequences of at most two chunks are cut evenly."""
    cuts = [0]
    if n > 2 * chunk:
        cuts.append(edge)
        r = chunk
        while r < n - chunk:
            cuts.append(r)
            r += chunk
        cuts.append(r)
        last = (n - edge) // 128 * 128   # a chunk starts on a multiple of 128 rows
        if last > r:
            cuts.append(last)
    else:
        r = chunk
        while r < n:
            cuts.append(r)
            r += chunk
    cuts.append(n)
    return [(cuts[i], cuts[i + 1]) for i in range(len(cuts) - 1) if cuts[i + 1] > cuts[i]]


class HostPrefillPipeline:
    """The same operator for callers whose activations live in PINNED HOST memory (layer-wise offloading runtimes
    such as the reference's, which keeps the KV cache on the host during prefill, cache_hub/flash_attn_cache.py):
    ``pipe(q_host, k_host, v_host, out_host)`` with q [1,N,Hq,D], k/v [1,N,Hkv,D] -> out [1,N,Hq*D].

    K goes first and whole (its centring needs the mean over the sequence); V and Q follow in chunks of query rows,
    in sequence order: a chunk of rows needs only the V rows up to its own end (causal), so its V rows travel with
    it, are prepared with it and the attention kernel (sqattn_prefill with q_row_offset) starts on the first chunk
    while the rest of V and Q is still on the bus and earlier outputs travel back.  The first and the last chunk are
    short, because the upload of the first and the download of the last cannot overlap with anything.  H2D copies
    and D2H copies have a stream each, and the chunks' kernels alternate between two streams, so that the attention
    CTAs of the next chunk fill the SMs the last wave of the previous chunk leaves idle.  Results are identical to the
    one-shot operator: chunks only partition the query rows."""

    def __init__(self, bit8_window_sizes=0, bit4_window_sizes=0, sink_window_size=0, args=None, chunk_rows=4096,
                 p_fp8_mode="off", device=None, edge_rows=2048):
        self.bit8, self.bit4 = _normalise_windows(bit8_window_sizes, bit4_window_sizes)
        self.sink, self.args, self.chunk = sink_window_size, args, int(chunk_rows)
        self.edge = min(int(edge_rows), self.chunk)
        if self.chunk % 128 or self.edge % 128 or self.edge <= 0:
            raise ValueError("chunk_rows and edge_rows must be positive multiples of 128")
        self.fp8 = {"off": L.P_FP8_OFF, "all": L.P_FP8_ALL, "stage2": L.P_FP8_STAGE2}[p_fp8_mode]
        self.device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
        self.s_in, self.s_out = torch.cuda.Stream(self.device), torch.cuda.Stream(self.device)
        self.s_run = [torch.cuda.Stream(self.device), torch.cuda.Stream(self.device)]   # kernels of even / odd chunks
        self._shape, self._buf = None, None

    def _bounds(self, n):
        """Row ranges of the chunks: a short first one, full chunks, a short last one."""
        return chunk_bounds(n, self.chunk, self.edge)

    def _buffers(self, n, hq, hkv, d, dtype):
        key = (n, hq, hkv, d, dtype)
        if self._shape != key:
            dev, c = self.device, min(self.chunk, n)
            self._buf = {
                "k": torch.empty(1, n, hkv, d, dtype=dtype, device=dev), "v": torch.empty(1, n, hkv, d, dtype=dtype, device=dev),
                # prepared K and V stay token-major, so that a chunk of V rows is one contiguous piece
                "k8": torch.empty(1, n, hkv, d, dtype=dtype, device=dev), "v8": torch.empty(1, n, hkv, d, dtype=torch.float16, device=dev),
                "q": [torch.empty(1, c, hq, d, dtype=dtype, device=dev) for _ in range(2)],
                "q8": [torch.empty(hq * c * d, dtype=dtype, device=dev) for _ in range(2)],
                "o": [torch.empty(1, c, hq * d, dtype=torch.bfloat16, device=dev) for _ in range(2)],
            }
            self._shape = key
        return self._buf

    def __call__(self, q_host, k_host, v_host, out_host=None):
        a = self.args
        if not a.use_relative_distance:
            raise ValueError("the host pipeline is implemented for relative windows")
        for t in (q_host, k_host, v_host):
            if t.is_cuda or not t.is_pinned():
                raise ValueError("q, k and v must be pinned host tensors")
        b, n, hq, d = q_host.shape
        hkv = k_host.shape[2]
        if b != 1:
            raise ValueError("the host pipeline takes one sequence (batch 1)")
        if out_host is None:
            out_host = torch.empty(1, n, hq * d, dtype=torch.bfloat16).pin_memory()
        buf = self._buffers(n, hq, hkv, d, q_host.dtype)
        cur = torch.cuda.current_stream(self.device)
        self.s_in.wait_stream(cur)
        self.s_out.wait_stream(cur)

        def per_head(w):
            return [float(w)] * hq if isinstance(w, (int, float)) else [float(x) for x in w]

        r8, r4 = per_head(self.bit8), per_head(self.bit4)
        with torch.cuda.stream(self.s_in):
            buf["k"].copy_(k_host, non_blocking=True)
            ev_k = torch.cuda.Event()
            ev_k.record(self.s_in)
        cur.wait_event(ev_k)
        ops.prep_qkv(None, buf["k"], None, qk_qtype=a.qk_qtype, v_qtype=a.v_qtype, skip_bit4=True, kv_out_nhd=True,
                     out={"k8": buf["k8"]})
        for st in self.s_run:
            st.wait_stream(cur)     # K is prepared, and everything the caller queued before this call is done
        q_free = [None, None]   # compute has finished reading q buffer s
        o_free = [None, None]   # the D2H copy has finished reading output buffer s
        ev_prep = None          # the previous chunk's V rows are prepared (the next chunk attends them too)
        for ci, (r0, r1) in enumerate(self._bounds(n)):
            rows, s = r1 - r0, ci & 1
            run = self.s_run[s]     # buffer s is only ever touched by the kernels of stream s
            with torch.cuda.stream(self.s_in):
                if q_free[s] is not None:
                    self.s_in.wait_event(q_free[s])
                buf["v"][:, r0:r1].copy_(v_host[:, r0:r1], non_blocking=True)
                buf["q"][s][:, :rows].copy_(q_host[:, r0:r1], non_blocking=True)
                ev_q = torch.cuda.Event()
                ev_q.record(self.s_in)
            with torch.cuda.stream(run):
                run.wait_event(ev_q)
                if o_free[s] is not None:
                    run.wait_event(o_free[s])
                q8 = buf["q8"][s][: hq * rows * d].view(1, hq, rows, d)
                ops.prep_qkv(buf["q"][s][:, :rows], None, buf["v"][:, r0:r1], qk_qtype=a.qk_qtype, v_qtype=a.v_qtype,
                             skip_bit4=True, kv_out_nhd=True, out={"q8": q8, "v8": buf["v8"][:, r0:r1]})
                this_prep = torch.cuda.Event()
                this_prep.record(run)
                if ev_prep is not None:
                    run.wait_event(ev_prep)
                ev_prep = this_prep
                o = buf["o"][s][:, :rows]
                ops.prefill(q8, buf["k8"], q8, buf["k8"], buf["v8"], mode=L.MODE_RELATIVE_WINDOW, win8=r8, win4=r4,
                            sink=self.sink, layout="HND", kv_layout="NHD", p_fp8_mode=self.fp8, q_is_scaled=True,
                            out=o.view(1, rows, hq, d), out_layout="NHD", q_row_offset=r0)
                ev_c = torch.cuda.Event()
                ev_c.record(run)
            q_free[s] = ev_c
            with torch.cuda.stream(self.s_out):
                self.s_out.wait_event(ev_c)
                out_host[:, r0:r1].copy_(o, non_blocking=True)
                ev_o = torch.cuda.Event()
                ev_o.record(self.s_out)
            o_free[s] = ev_o
        for st in self.s_run:
            cur.wait_stream(st)
        cur.wait_stream(self.s_out)
        return out_host
