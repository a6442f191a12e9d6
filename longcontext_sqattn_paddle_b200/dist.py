"""Multi-GPU partitioning of the attention path (one process per GPU, torch.distributed).

The reference has no multi-GPU path beyond layer-to-device placement (model_hub/qwen.py:203-267); these are the
two places where the path shards naturally:

* prefill: query rows are independent given K and V.  A ``ShardLayout`` says which token ranges of the sequence a
  rank owns: equal contiguous shards, contiguous shards cut so that the windowed attention work is equal
  (``balanced``), or the zig-zag split (rank r owns chunks r and 2G-1-r of 2G equal chunks) that balances dense
  causal work.  Exchange steps of a windowed layer: an all-reduce of the K column sums [B,Hkv,D] fp32 (the
  sequence mean that the adapter subtracts, sqattn/attn_replacer.py:338-339, is global) and a HALO exchange of
  the prepared K and V rows: a rank only needs the sink tokens and the ``reach`` (largest window) tokens in front
  of each of its row ranges, 13 440 tokens instead of 131 072 at the reference's default window, sent point to
  point.  The all-reduce runs while V is prepared and the halo exchange while Q is prepared, so neither is on
  the critical path.  A dense causal layer (the un-replaced first and last layer, model_hub/qwen.py:38-48)
  all-gathers the raw K and V.  Per-token Q/K scales and per-(token,channel) V scales are local to a shard.  The
  attention kernel then runs on the local query rows (one launch, one or two row ranges) against K/V in local
  memory; it never reads a peer's memory.
* decode: the cache is sharded by key ranges; every rank computes (partial O, LSE) over its keys, one
  all-gather of [B*Hq, D+1] floats, one merge kernel.

The collectives go through ``torch.distributed`` (NCCL on GPUs).  For decode, where the exchange is 14 KB per rank
and latency is everything, ``PeerExchange`` replaces the all-gather + merge by ONE kernel that stores the partials
into every rank's buffer over NVLink (plain peer stores into symmetric memory), flags, waits and merges
(csrc/peer_exchange.cuh).
The compute steps are taken from a ``backend`` object so that the partitioning logic can be exercised on CPU
ranks (gloo) with a stand-in backend; the default backend is the CUDA library and nothing else ships.
"""
from __future__ import annotations

from typing import List, Optional, Sequence, Tuple

import torch
import torch.distributed as dist

import ctypes as C
import os

from . import _lib as L


# ------------------------------------------------------------------------------------------- shard layouts
class ShardLayout:
    """Token ranges of a ``total``-token sequence owned by each of ``world`` ranks.  ``segments(rank)`` lists the
    rank's ranges [(lo, hi), ...] (one or two) in the order its local rows are stored; every range starts on a
    multiple of 128 rows and ends on one unless it ends the sequence."""

    def __init__(self, total: int, world: int, segments: List[List[Tuple[int, int]]], kind: str):
        self.total, self.world, self._segs, self.kind = int(total), int(world), segments, kind
        covered = sorted(s for segs in segments for s in segs)
        pos = 0
        for lo, hi in covered:
            if lo != pos or hi <= lo:
                raise ValueError(f"shard layout does not tile the sequence: {covered}")
            if lo % 128 or (hi % 128 and hi != total):
                raise ValueError(f"row range [{lo}, {hi}) is not aligned to 128 rows")
            pos = hi
        if pos != total:
            raise ValueError(f"shard layout covers {pos} of {total} tokens")
        if any(len(s) > 2 for s in segments):
            raise ValueError("at most two row ranges per rank")

    def segments(self, rank: int) -> List[Tuple[int, int]]:
        return list(self._segs[rank])

    def rows(self, rank: int) -> int:
        return sum(hi - lo for lo, hi in self._segs[rank])

    def owner_of_last_token(self) -> int:
        return next(r for r in range(self.world) if any(hi == self.total for _, hi in self._segs[r]))

    @classmethod
    def contiguous(cls, total: int, world: int) -> "ShardLayout":
        if total % world:
            raise ValueError(f"sequence length {total} is not divisible by the world size {world}")
        ns = total // world
        if world > 1 and ns % 128:
            raise ValueError(f"shard length {ns} must be a multiple of 128 query rows")
        return cls(total, world, [[(r * ns, (r + 1) * ns)] for r in range(world)], "contiguous")

    @classmethod
    def zigzag(cls, total: int, world: int) -> "ShardLayout":
        """Rank r owns chunks r and 2G-1-r of 2G equal chunks: under a causal mask the cheap early rows and the
        expensive late rows pair up, so every rank has the same dense-attention work."""
        if world == 1:
            return cls.contiguous(total, 1)
        if total % (2 * world) or (total // (2 * world)) % 128:
            raise ValueError(f"zig-zag sharding needs {total} tokens to split into {2 * world} chunks of a multiple of 128")
        c = total // (2 * world)
        return cls(total, world, [[(r * c, (r + 1) * c), ((2 * world - 1 - r) * c, (2 * world - r) * c)]
                                  for r in range(world)], "zigzag")

    @classmethod
    def balanced(cls, total: int, world: int, reach: int, sink: int) -> "ShardLayout":
        """Contiguous shards whose WINDOWED attention work is equal: a row attends to at most sink + reach + its
        diagonal block, the first rows to fewer, so the first rank takes more rows.  Cuts are multiples of 128."""
        nblk = (total + 127) // 128
        cost, acc = [], 0
        for b in range(nblk):
            qs = b * 128
            acc += min(sink, qs) + min(max(qs + 64 - sink, 0), reach) + 64
            cost.append(acc)
        cuts, b = [0], 0
        for r in range(1, world):
            target = acc * r / world
            while b < nblk and cost[b] < target:
                b += 1
            cuts.append(min(max(b + 1, cuts[-1] // 128 + 1), nblk - (world - r)) * 128)
        cuts.append(total)
        if any(cuts[i + 1] <= cuts[i] for i in range(world)):
            raise ValueError(f"{total} tokens are too few for {world} balanced shards")
        return cls(total, world, [[(cuts[r], cuts[r + 1])] for r in range(world)], "balanced")


def shard_range(rank: int, world: int, seq_total: int):
    """Token range [lo, hi) owned by ``rank`` under equal contiguous shards, each a multiple of 128 rows."""
    return ShardLayout.contiguous(seq_total, world).segments(rank)[0]


def halo_plan(layout: ShardLayout, reach: int, sink: int) -> List[Tuple[int, int, int, int]]:
    """Point-to-point transfers (src, dst, lo, hi) of key/value rows so that every rank holds, besides its own
    rows, the sink tokens [0, sink) and the ``reach`` tokens in front of each of its row ranges.  The same list is
    computed on every rank; ranges are cut at ownership boundaries."""
    owned = [(lo, hi, r) for r in range(layout.world) for lo, hi in layout.segments(r)]
    plan = []
    for dst in range(layout.world):
        need = []
        for lo, hi in layout.segments(dst):
            if sink > 0:
                need.append((0, min(sink, layout.total)))
            if reach > 0 and lo > 0:
                need.append((max(0, lo - reach), lo))
        need.sort()
        merged = []
        for lo, hi in need:                       # union of the needed ranges
            if merged and lo <= merged[-1][1]:
                merged[-1] = (merged[-1][0], max(merged[-1][1], hi))
            else:
                merged.append((lo, hi))
        for nlo, nhi in merged:
            for olo, ohi, src in owned:
                lo, hi = max(nlo, olo), min(nhi, ohi)
                if lo < hi and src != dst:
                    plan.append((src, dst, lo, hi))
    plan.sort()
    return plan


def _local_rows(segs: List[Tuple[int, int]], lo: int, hi: int) -> Tuple[int, int]:
    """Local row range of the global rows [lo, hi), which lie inside one of the rank's ranges."""
    base = 0
    for slo, shi in segs:
        if slo <= lo and hi <= shi:
            return base + lo - slo, base + hi - slo
        base += shi - slo
    raise ValueError(f"rows [{lo}, {hi}) are not owned by this rank")


# ------------------------------------------------------------------------------------------- compute backend
class CudaBackend:
    """The compute steps on the local GPU (libsqattn_b200.so)."""

    def k_column_sums(self, key):
        from . import ops
        return ops.k_column_sums(key)

    def empty_kv(self, total, hkv, d, dtype, like):
        return torch.empty(1, total, hkv, d, dtype=dtype, device=like.device)

    def prep_q(self, query, qk_qtype, need_bit4):
        """query [1,ns,Hq,D] -> (q_bit8, q_bit4 or None) [1,Hq,ns,D], already scaled."""
        from . import ops
        q8, q4, _, _, _ = ops.prep_qkv(query, None, None, qk_qtype=qk_qtype, skip_bit4=not need_bit4)
        return q8, q4

    def prep_k(self, key, k_mean, qk_qtype, out8, out4):
        """key [1,n,Hkv,D] minus the global mean, fake-quantised into the token-major views out8 (and out4)."""
        from . import ops
        ops.prep_qkv(None, key, None, qk_qtype=qk_qtype, skip_bit4=out4 is None, k_mean=k_mean, kv_out_nhd=True,
                     out={"k8": out8, "k4": out4})

    def prep_v(self, value, v_qtype, out):
        from . import ops
        ops.prep_qkv(None, None, value, v_qtype=v_qtype, skip_bit4=True, kv_out_nhd=True, out={"v8": out})

    def _segs(self, segs):
        if len(segs) == 1:
            return dict(q_row_offset=segs[0][0])
        return dict(q_row_offset=segs[0][0], q_split_rows=segs[0][1] - segs[0][0], q_row_offset2=segs[1][0])

    def windowed_prefill(self, q8, q4, k8, k4, v_full, win8, win4, sink, segs, relative, p_fp8_mode, out=None):
        from . import ops
        b, hq, n, d = q8.shape
        if out is None:
            out = torch.empty(b, n, hq * d, dtype=torch.bfloat16, device=q8.device)
        ops.prefill(q8, k8, q8 if q4 is None else q4, k8 if k4 is None else k4, v_full,
                    mode=L.MODE_RELATIVE_WINDOW if relative else L.MODE_ABSOLUTE_WINDOW, win8=win8, win4=win4, sink=sink,
                    layout="HND", kv_layout="NHD", p_fp8_mode=p_fp8_mode, q_is_scaled=True,
                    out=out.view(b, n, hq, d), out_layout="NHD", **self._segs(segs))
        return out

    def dense_prefill(self, query, k_full, v_full, segs):
        from . import ops
        b, n, hq, d = query.shape
        out = torch.empty(b, n, hq * d, dtype=query.dtype, device=query.device)
        ops.prefill(query, k_full, query, k_full, v_full, mode=L.MODE_DENSE_CAUSAL, layout="NHD", q_is_scaled=False,
                    out=out.view(b, n, hq, d), out_layout="NHD", **self._segs(segs))
        return out

    def decode_partial(self, q, k, v, kv_lens, p_fp8):
        from . import ops
        return ops.decode(q, k, v, partial=True, kv_lens=kv_lens, p_fp8=p_fp8)

    def merge(self, part_o, part_lse, out_dtype):
        from . import ops
        return ops.decode_merge(part_o, part_lse, out_dtype=out_dtype)


class PeerExchange:
    """Symmetric-memory buffers for the one-kernel cross-GPU merge (sqattn_decode_peer_merge).  Every rank
    allocates the same two buffers, the ranks exchange mappings once (torch symmetric memory), and each decode
    step is then a single kernel per rank with no NCCL call.  ``rows_cap`` = batch * query heads at most."""

    def __init__(self, rows_cap: int, head_dim: int, group=None, device=None):
        import torch.distributed._symmetric_memory as symm_mem
        if not dist.is_initialized():
            raise RuntimeError("PeerExchange needs an initialised process group")
        self.group = group if group is not None else dist.group.WORLD
        self.world, self.rank = dist.get_world_size(self.group), dist.get_rank(self.group)
        if self.world > 16:
            raise ValueError("PeerExchange supports at most 16 ranks")
        self.rows_cap, self.d = int(rows_cap), int(head_dim)
        dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
        # plain peer loads/stores only: no NVLink multicast object is needed for this exchange
        os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
        nd = L.lib.sqattn_peer_merge_data_bytes(self.world, self.rows_cap, self.d)
        nf = L.lib.sqattn_peer_merge_flag_bytes(self.world, self.rows_cap)
        self.data = symm_mem.empty(nd // 4, dtype=torch.float32, device=dev)
        self.flags = symm_mem.empty(nf // 4, dtype=torch.int32, device=dev)
        self.data.zero_()
        self.flags.zero_()
        self._hd = symm_mem.rendezvous(self.data, self.group)
        self._hf = symm_mem.rendezvous(self.flags, self.group)
        self.data_ptrs = [int(x) for x in self._hd.buffer_ptrs]
        self.flag_ptrs = [int(x) for x in self._hf.buffer_ptrs]
        torch.cuda.synchronize(dev)
        dist.barrier(self.group)   # everybody's buffers are zeroed before anybody's first store arrives
        self.epoch = torch.zeros(1, dtype=torch.int32, device=dev)   # advanced on the device by every call

    def _args(self, rows: int, out: torch.Tensor, lse: Optional[torch.Tensor]):
        a = L.PeerMergeArgs()
        for w in range(self.world):
            a.peer_data[w], a.peer_flags[w] = self.data_ptrs[w], self.flag_ptrs[w]
        a.rank, a.world, a.rows, a.rows_cap, a.head_dim, a.epoch = self.rank, self.world, rows, self.rows_cap, self.d, self.epoch.data_ptr()
        a.out = out.data_ptr()
        a.o_dtype = L.BF16 if out.dtype == torch.bfloat16 else L.F16
        a.lse = None if lse is None else lse.data_ptr()
        return a

    def merge(self, part_o: torch.Tensor, part_lse: torch.Tensor, out_dtype=torch.bfloat16, return_lse: bool = False):
        """part_o [rows, D] fp32, part_lse [rows] fp32 (this rank's partial) -> merged O [rows, D] on every rank."""
        rows, d = part_o.shape
        if d != self.d or rows > self.rows_cap:
            raise ValueError(f"partial of shape {tuple(part_o.shape)} does not fit an exchange of {self.rows_cap} x {self.d}")
        part_o, part_lse = part_o.contiguous(), part_lse.contiguous()
        out = torch.empty(rows, d, dtype=out_dtype, device=part_o.device)
        lse = torch.empty(rows, dtype=torch.float32, device=part_o.device) if return_lse else None
        a = self._args(rows, out, lse)
        a.part_o, a.part_lse = part_o.data_ptr(), part_lse.data_ptr()
        L.check(L.lib.sqattn_decode_peer_merge(C.byref(a), torch.cuda.current_stream().cuda_stream))
        return (out, lse) if return_lse else out

    def decode(self, q, k_shard, v_shard, *, kv_lens=None, out_dtype=torch.bfloat16, p_fp8: bool = False):
        """Split-KV decode of this rank's keys with the exchange fused behind it: two kernels per call (decode;
        split merge + peer stores + wait + merge across ranks).  q [B,Hq,1,D] -> O [B,Hq,1,D] on every rank."""
        from . import ops
        b, hq, _, d = q.shape
        rows = b * hq
        if d != self.d or rows > self.rows_cap:
            raise ValueError(f"{rows} rows x {d} do not fit an exchange of {self.rows_cap} x {self.d}")
        out = torch.empty(rows, d, dtype=out_dtype, device=q.device)
        a = self._args(rows, out, None)
        ops.decode(q, k_shard, v_shard, kv_lens=kv_lens, p_fp8=p_fp8, peer=a)
        return out.view(b, hq, 1, d)


# ------------------------------------------------------------------------------------------- prefill
def _group_info(group):
    if dist.is_initialized():
        return dist.get_world_size(group), dist.get_rank(group)
    return 1, 0


def _global_rank(group, r):
    return r if group is None else dist.get_global_rank(group, r)


def _resolve_layout(layout, total, world, reach, sink) -> ShardLayout:
    if isinstance(layout, ShardLayout):
        if layout.total != total or layout.world != world:
            raise ValueError(f"layout describes {layout.total} tokens on {layout.world} ranks, call has {total} on {world}")
        return layout
    if layout == "contiguous":
        return ShardLayout.contiguous(total, world)
    if layout == "zigzag":
        return ShardLayout.zigzag(total, world)
    if layout == "balanced":
        return ShardLayout.balanced(total, world, reach, sink)
    raise ValueError(f"unknown shard layout {layout!r}")


def _per_head(w, hq, conv):
    return [conv(w)] * hq if isinstance(w, (int, float)) else [conv(x) for x in w]


def _window_reach(win8, win4, relative, total) -> int:
    """Largest distance (in tokens) a query row looks back beyond its own 128-row block."""
    if relative:
        def size(r):
            raw = int((torch.tensor(r, dtype=torch.float32) * torch.tensor(float(total), dtype=torch.float32)).item())
            return (raw + 127) // 128 * 128
        return max(max(size(r) for r in win8), max(size(r) for r in win4), 0)
    return max(max(int(x) for x in win8), max(int(x) for x in win4), 0)


def _sp_kv_stage(state, backend, key, value, args, win8, win4, sink, total, world, rank, group, layout, exchange):
    """The K/V half of a sequence-parallel windowed layer: column sums, all-reduce, preparation of this rank's K/V
    rows into full-length buffers and the exchange of the rows other ranks need.  Returns (k8, k4, v8, segments,
    outstanding exchange handles); the caller waits on the handles before it launches attention."""
    relative = bool(args.use_relative_distance)
    b, ns, hkv, d = key.shape
    key_ = (total, world, hkv, d, key.dtype, key.device)
    if state.get("key") != key_:
        reach = _window_reach(win8, win4, relative, total)
        lay = _resolve_layout(layout, total, world, reach, sink)
        # a stage's 64-key tiles may run up to 63 keys past its end, as in the reference loops: the sink rounds up
        state.update(key=key_, layout=lay, plan=halo_plan(lay, reach, (sink + 63) // 64 * 64),
                     k8=backend.empty_kv(total, hkv, d, key.dtype, key),
                     k4=None if relative else backend.empty_kv(total, hkv, d, key.dtype, key),
                     v8=backend.empty_kv(total, hkv, d, torch.float16, key))
    lay, k8, k4, v8 = state["layout"], state["k8"], state["k4"], state["v8"]
    segs = lay.segments(rank)
    if lay.rows(rank) != ns:
        raise ValueError(f"rank {rank} holds {ns} tokens, its shard has {lay.rows(rank)}")
    # 1. global sequence mean of K: all-reduce of the shards' column sums (2 KB) while V is prepared
    sums = backend.k_column_sums(key)
    work = dist.all_reduce(sums, group=group, async_op=True) if world > 1 else None
    base = 0
    for lo, hi in segs:
        backend.prep_v(value[:, base:base + hi - lo], args.v_qtype, v8[:, lo:hi])
        base += hi - lo
    if work is not None:
        work.wait()
    k_mean = (sums / float(total)).contiguous()
    base = 0
    for lo, hi in segs:
        backend.prep_k(key[:, base:base + hi - lo], k_mean, args.qk_qtype, k8[:, lo:hi],
                       None if k4 is None else k4[:, lo:hi])
        base += hi - lo
    # 2. the rows other ranks need travel while Q is prepared
    works = []
    if world > 1 and exchange == "halo":
        p2p = []
        for src, dst, lo, hi in state["plan"]:
            for buf in (k8, k4, v8):
                if buf is None:
                    continue
                if src == rank:
                    p2p.append(dist.P2POp(dist.isend, buf[0, lo:hi], _global_rank(group, dst), group))
                elif dst == rank:
                    p2p.append(dist.P2POp(dist.irecv, buf[0, lo:hi], _global_rank(group, src), group))
        if p2p:
            works = dist.batch_isend_irecv(p2p)
    elif world > 1:
        if lay.kind != "contiguous":
            raise ValueError("exchange='allgather' needs equal contiguous shards")
        lo, hi = segs[0]
        for buf in (k8, k4, v8):
            if buf is not None:
                mine = buf[0, lo:hi].clone()
                works.append(dist.all_gather_into_tensor(buf.view(total, hkv, d), mine, group=group, async_op=True))
    return k8, k4, v8, segs, works


def sp_prefill_wrapper(bit8_window_sizes, bit4_window_sizes, sink_window_size, args, seq_total: Optional[int] = None,
                       group=None, backend=None, p_fp8_mode: int = 0, layout="contiguous", exchange: str = "halo"):
    """Sequence-parallel counterpart of ``mp_triton_wrapper`` (relative or absolute windows): returns
    attention_fn(module, query, key, value, attention_mask, ...) where query/key/value are THIS rank's token rows
    ([B=1, ns, H, D], its row ranges in ``layout`` order) and the result is this rank's [1, ns, Hq*D] rows of the
    output.  ``exchange``: "halo" sends every rank only the sink and window rows it needs, "allgather" gathers all
    prepared K/V (equal shards only)."""
    backend = backend or CudaBackend()
    state = {}

    def attention_fn(module, query, key, value, attention_mask=None, dropout=0.0, scaling=1.0, sliding_window=None,
                     **kwargs):
        if args.qk_qtype not in L.QTYPE:
            raise ValueError(f"Invalid quantization type: {args.qk_qtype}")
        if args.v_qtype not in L.QTYPE:
            raise ValueError(f"Invalid quantization type: {args.v_qtype}")
        relative = bool(args.use_relative_distance)
        world, rank = _group_info(group)
        b, ns, hq, d = query.shape
        if b != 1:
            raise ValueError("sequence-parallel prefill takes one sequence (batch 1), like the reference's cache")
        total = seq_total if seq_total is not None else ns * world
        win8 = _per_head(bit8_window_sizes, hq, float if relative else int)
        win4 = _per_head(bit4_window_sizes, hq, float if relative else int)
        k8, k4, v8, segs, works = _sp_kv_stage(state, backend, key, value, args, win8, win4, sink_window_size, total,
                                               world, rank, group, layout, exchange)
        q8, q4 = backend.prep_q(query, args.qk_qtype, not relative)
        for w in works:
            w.wait()
        return backend.windowed_prefill(q8, q4, k8, k4, v8, win8, win4, sink_window_size, segs, relative, p_fp8_mode)

    attention_fn.state = state
    return attention_fn


class SPHostPrefillPipeline:
    """The sequence-parallel operator for callers whose activations live in PINNED HOST memory (the counterpart of
    ``sqattn.HostPrefillPipeline`` on N ranks): ``pipe(q_host, k_host, v_host, out_host)`` with this rank's rows
    q [1,ns,Hq,D], k/v [1,ns,Hkv,D] -> its rows of the output [1,ns,Hq*D].  K and V are uploaded, prepared and
    exchanged once; Q is uploaded, prepared and attended in chunks of ``chunk_rows`` rows while the previous chunk's
    output travels back, so the two copy directions, the collectives and the kernels overlap.  Relative windows."""

    def __init__(self, bit8_window_sizes, bit4_window_sizes, sink_window_size, args, seq_total: int, layout="balanced",
                 chunk_rows: int = 4096, group=None, p_fp8_mode: int = 0, device=None, edge_rows: int = 1024):
        if chunk_rows % 128 or edge_rows % 128 or edge_rows <= 0:
            raise ValueError("chunk_rows and edge_rows must be positive multiples of 128")
        self.edge = min(int(edge_rows), int(chunk_rows))   # first and last chunk of a row range: their copies overlap with nothing
        if not args.use_relative_distance:
            raise ValueError("the host pipeline is implemented for relative windows")
        self.bit8, self.bit4, self.sink, self.args = bit8_window_sizes, bit4_window_sizes, sink_window_size, args
        self.total, self.layout, self.chunk, self.group, self.fp8 = int(seq_total), layout, int(chunk_rows), group, p_fp8_mode
        self.device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
        self.s_in, self.s_out = torch.cuda.Stream(self.device), torch.cuda.Stream(self.device)
        self.s_run = [torch.cuda.Stream(self.device), torch.cuda.Stream(self.device)]   # kernels of even / odd chunks
        self.backend, self.state, self._buf = CudaBackend(), {}, None

    def __call__(self, q_host, k_host, v_host, out_host):
        for t in (q_host, k_host, v_host, out_host):
            if t.is_cuda or not t.is_pinned():
                raise ValueError("q, k, v and out must be pinned host tensors")
        a, be, dev = self.args, self.backend, self.device
        world, rank = _group_info(self.group)
        b, ns, hq, d = q_host.shape
        hkv = k_host.shape[2]
        win8, win4 = _per_head(self.bit8, hq, float), _per_head(self.bit4, hq, float)
        if self._buf is None or self._buf["k"].shape != k_host.shape:
            c = min(self.chunk, ns)
            self._buf = {"k": torch.empty(k_host.shape, dtype=k_host.dtype, device=dev),
                         "v": torch.empty(v_host.shape, dtype=v_host.dtype, device=dev),
                         "q": [torch.empty(1, c, hq, d, dtype=q_host.dtype, device=dev) for _ in range(2)],
                         "o": [torch.empty(1, c, hq * d, dtype=torch.bfloat16, device=dev) for _ in range(2)]}
        buf = self._buf
        cur = torch.cuda.current_stream(dev)
        self.s_in.wait_stream(cur)
        self.s_out.wait_stream(cur)
        with torch.cuda.stream(self.s_in):
            buf["k"].copy_(k_host, non_blocking=True)
            buf["v"].copy_(v_host, non_blocking=True)
            ev_kv = torch.cuda.Event()
            ev_kv.record(self.s_in)
        cur.wait_event(ev_kv)
        k8, _, v8, segs, works = _sp_kv_stage(self.state, be, buf["k"], buf["v"], a, win8, win4, self.sink, self.total,
                                              world, rank, self.group, self.layout, "halo")
        q_free, o_free = [None, None], [None, None]
        ci, base, waited = 0, 0, [False, False]
        for st in self.s_run:
            st.wait_stream(cur)       # own K/V rows are prepared; the halo rows are waited for below
        from .sqattn.attn_replacer import chunk_bounds
        for lo, hi in segs:
            for r0, r1 in chunk_bounds(hi - lo, self.chunk, self.edge):
                rows, s = r1 - r0, ci & 1
                run = self.s_run[s]   # buffer s is only ever touched by the kernels of stream s; the two streams let
                                      # the next chunk's CTAs fill the last wave of the previous chunk
                with torch.cuda.stream(self.s_in):
                    if q_free[s] is not None:
                        self.s_in.wait_event(q_free[s])
                    buf["q"][s][:, :rows].copy_(q_host[:, base + r0:base + r0 + rows], non_blocking=True)
                    ev_q = torch.cuda.Event()
                    ev_q.record(self.s_in)
                with torch.cuda.stream(run):
                    run.wait_event(ev_q)
                    if o_free[s] is not None:
                        run.wait_event(o_free[s])
                    q8, _ = be.prep_q(buf["q"][s][:, :rows], a.qk_qtype, False)
                    if not waited[s]:       # the halo rows have to be in place before this stream's first attention launch
                        for w in works:
                            w.wait()
                        waited[s] = True
                    o = be.windowed_prefill(q8, None, k8, None, v8, win8, win4, self.sink, [(lo + r0, lo + r0 + rows)], True,
                                            self.fp8, out=buf["o"][s][:, :rows])
                    ev_c = torch.cuda.Event()
                    ev_c.record(run)
                q_free[s] = ev_c
                with torch.cuda.stream(self.s_out):
                    self.s_out.wait_event(ev_c)
                    out_host[:, base + r0:base + r0 + rows].copy_(o, non_blocking=True)
                    ev_o = torch.cuda.Event()
                    ev_o.record(self.s_out)
                o_free[s] = ev_o
                ci += 1
            base += hi - lo
        for st in self.s_run:
            cur.wait_stream(st)
        cur.wait_stream(self.s_out)
        return out_host


def sp_dense_wrapper(seq_total: Optional[int] = None, group=None, backend=None, layout="zigzag"):
    """Sequence-parallel dense causal attention for the layers the reference leaves un-replaced
    (model_hub/qwen.py:38-48; its first and last layer, sqattn/compress.py:162): the raw K and V shards are
    all-gathered into sequence order and every rank attends its own rows (``layout``: "zigzag" balances the causal
    work, "contiguous" does not).  Same calling convention as ``sp_prefill_wrapper``; output in the input dtype."""
    backend = backend or CudaBackend()
    state = {}

    def attention_fn(module, query, key, value, attention_mask=None, dropout=0.0, scaling=1.0, sliding_window=None,
                     **kwargs):
        world, rank = _group_info(group)
        b, ns, hq, d = query.shape
        hkv = key.shape[2]
        if b != 1:
            raise ValueError("sequence-parallel prefill takes one sequence (batch 1), like the reference's cache")
        total = seq_total if seq_total is not None else ns * world
        key_ = (total, world, hkv, d, key.dtype, key.device)
        if state.get("key") != key_:
            lay = _resolve_layout(layout, total, world, 0, 0)
            if lay.kind not in ("contiguous", "zigzag"):
                raise ValueError("dense sequence-parallel attention needs equal shards (contiguous or zig-zag)")
            state.update(key=key_, layout=lay, k=backend.empty_kv(total, hkv, d, key.dtype, key),
                         v=backend.empty_kv(total, hkv, d, value.dtype, key))
        lay, k_full, v_full = state["layout"], state["k"], state["v"]
        segs = lay.segments(rank)
        if lay.rows(rank) != ns:
            raise ValueError(f"rank {rank} holds {ns} tokens, its shard has {lay.rows(rank)}")
        if world == 1:
            return backend.dense_prefill(query, key, value, segs)
        works = []
        for full, mine in ((k_full, key), (v_full, value)):
            if lay.kind == "contiguous":
                works.append(dist.all_gather_into_tensor(full.view(total, hkv, d), mine[0].contiguous(), group=group,
                                                         async_op=True))
            else:
                c = ns // 2
                # first halves are chunks 0..G-1 in rank order; second halves are chunks 2G-1..G
                works.append(dist.all_gather_into_tensor(full[0, :total // 2], mine[0, :c].contiguous(), group=group,
                                                         async_op=True))
                outs = [full[0, (2 * world - 1 - r) * c:(2 * world - r) * c] for r in range(world)]
                works.append(dist.all_gather(outs, mine[0, c:].contiguous(), group=group, async_op=True))
        for w in works:
            w.wait()
        return backend.dense_prefill(query, k_full, v_full, segs)

    attention_fn.state = state
    return attention_fn


# ------------------------------------------------------------------------------------------- decode
def sp_decode(q, k_shard, v_shard, *, kv_lens: Optional[Sequence[int]] = None, out_dtype=torch.bfloat16,
              p_fp8: bool = False, group=None, backend=None, exchange: Optional[PeerExchange] = None):
    """Split-KV decode across ranks.  q [B,Hq,1,D] (replicated), k_shard/v_shard [B,Hkv,Ls,D]: this rank's keys
    (``kv_lens``: how many of them are valid per sequence).  Returns O [B,Hq,1,D] on every rank.  With
    ``exchange`` the partials travel by peer stores inside one merge kernel instead of an NCCL all-gather."""
    if exchange is not None:
        return exchange.decode(q, k_shard, v_shard, kv_lens=kv_lens, out_dtype=out_dtype, p_fp8=p_fp8)
    backend = backend or CudaBackend()
    world = dist.get_world_size(group) if dist.is_initialized() else 1
    b, hq, _, d = q.shape
    po, pl = backend.decode_partial(q, k_shard, v_shard, kv_lens, p_fp8)  # [B,Hq,D] fp32, [B,Hq] fp32
    rows = b * hq
    if world > 1:
        packed = torch.cat([po.reshape(rows, d), pl.reshape(rows, 1)], dim=1).contiguous()   # [rows, D+1]
        gathered = torch.empty(world, rows, d + 1, dtype=torch.float32, device=packed.device)
        dist.all_gather_into_tensor(gathered.view(world * rows, d + 1), packed, group=group)
        part_o = gathered[:, :, :d].contiguous()
        part_lse = gathered[:, :, d].contiguous()
    else:
        part_o, part_lse = po.reshape(1, rows, d), pl.reshape(1, rows)
    out = backend.merge(part_o, part_lse, out_dtype)
    return out.view(b, hq, 1, d)
