"""Multi-GPU partitioning of the attention path (one process per GPU, torch.distributed).

The reference has no multi-GPU path beyond layer-to-device placement (model_hub/qwen.py:203-267); these are the
two places where the path shards naturally:

* prefill: query rows are independent given K and V.  Rank r owns the tokens
  [r*Ns, (r+1)*Ns) of a sequence of world*Ns tokens.  Exchange steps: an all-reduce of the K column sums
  [B,Hkv,D] fp32 (the sequence mean that the adapter subtracts, sqattn/attn_replacer.py:338-339, is global)
  and an all-gather of the prepared K and V shards, written token-major so the gathered tensor is contiguous.
  Per-token Q/K scales and per-(token,channel) V scales are local to a shard.  The attention kernel then runs
  on the local query rows with q_row_offset = r*Ns against the gathered K/V in local memory.
* decode: the cache is sharded by key ranges; every rank computes (partial O, LSE) over its keys, one
  all-gather of [B*Hq, D+1] floats, one merge kernel.

The collectives go through ``torch.distributed`` (NCCL on GPUs) and the attention kernels only ever read local
memory.  For decode, where the exchange is 14 KB per rank and latency is everything, ``PeerExchange`` replaces
the all-gather + merge by ONE kernel that stores the partials into every rank's buffer over NVLink (plain peer
stores into symmetric memory), flags, waits and merges (csrc/peer_exchange.cuh).
The compute steps are taken from a ``backend`` object so that the partitioning logic can be exercised on CPU
ranks (gloo) with a stand-in backend; the default backend is the CUDA library and nothing else ships.
"""
from __future__ import annotations

from typing import Optional, Sequence

import torch
import torch.distributed as dist

import ctypes as C
import os

from . import _lib as L


class CudaBackend:
    """The compute steps on the local GPU (libsqattn_b200.so)."""

    def k_column_sums(self, key):
        from . import ops
        return ops.k_column_sums(key)

    def prep(self, query, key, value, k_mean, qk_qtype, v_qtype):
        from . import ops
        q8, _, k8, _, v8 = ops.prep_qkv(query, key, value, qk_qtype=qk_qtype, v_qtype=v_qtype, skip_bit4=True,
                                        k_mean=k_mean, kv_out_nhd=True)
        return q8, k8, v8

    def windowed_prefill(self, q8, k_full, v_full, win8, win4, sink, q_row_offset, p_fp8_mode):
        from . import ops
        b, hq, n, d = q8.shape
        out = torch.empty(b, n, hq * d, dtype=torch.bfloat16, device=q8.device)
        ops.prefill(q8, k_full, q8, k_full, v_full, mode=L.MODE_RELATIVE_WINDOW, win8=win8, win4=win4, sink=sink,
                    layout="HND", kv_layout="NHD", p_fp8_mode=p_fp8_mode, q_is_scaled=True,
                    out=out.view(b, n, hq, d), out_layout="NHD", q_row_offset=q_row_offset)
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


def shard_range(rank: int, world: int, seq_total: int):
    """Token range [lo, hi) owned by ``rank``: equal contiguous shards, each a multiple of 128 rows."""
    if seq_total % world:
        raise ValueError(f"sequence length {seq_total} is not divisible by the world size {world}")
    ns = seq_total // world
    if world > 1 and ns % 128:
        raise ValueError(f"shard length {ns} must be a multiple of 128 query rows")
    return rank * ns, (rank + 1) * ns


def sp_prefill_wrapper(bit8_window_sizes, bit4_window_sizes, sink_window_size, args, seq_total: Optional[int] = None,
                       group=None, backend=None, p_fp8_mode: int = 0):
    """Sequence-parallel counterpart of ``mp_triton_wrapper`` (relative windows): returns
    attention_fn(module, query, key, value, attention_mask, ...) where query/key/value are THIS rank's token
    shard ([B=1, Ns, H, D]) and the result is this rank's [1, Ns, Hq*D] slice of the output."""
    backend = backend or CudaBackend()

    def attention_fn(module, query, key, value, attention_mask=None, dropout=0.0, scaling=1.0, sliding_window=None,
                     **kwargs):
        if args.qk_qtype not in L.QTYPE:
            raise ValueError(f"Invalid quantization type: {args.qk_qtype}")
        if args.v_qtype not in L.QTYPE:
            raise ValueError(f"Invalid quantization type: {args.v_qtype}")
        if not args.use_relative_distance:
            raise ValueError("sequence-parallel prefill is implemented for relative windows")
        world = dist.get_world_size(group) if dist.is_initialized() else 1
        rank = dist.get_rank(group) if dist.is_initialized() else 0
        b, ns, hq, d = query.shape
        hkv = key.shape[2]
        if b != 1:
            raise ValueError("sequence-parallel prefill takes one sequence (batch 1), like the reference's cache")
        total = seq_total if seq_total is not None else ns * world
        lo, hi = shard_range(rank, world, total)
        if hi - lo != ns:
            raise ValueError(f"rank {rank} holds {ns} tokens, expected {hi - lo}")
        # global sequence mean of K: all-reduce the shards' column sums (2 KB), divide once
        sums = backend.k_column_sums(key)
        if world > 1:
            dist.all_reduce(sums, group=group)
        k_mean = (sums / float(total)).contiguous()
        q8, k8, v8 = backend.prep(query, key, value, k_mean, args.qk_qtype, args.v_qtype)  # k8/v8 [1,Ns,Hkv,D]
        if world > 1:
            k_full = torch.empty(1, total, hkv, d, dtype=k8.dtype, device=k8.device)
            v_full = torch.empty(1, total, hkv, d, dtype=v8.dtype, device=v8.device)
            dist.all_gather_into_tensor(k_full.view(total, hkv, d), k8.view(ns, hkv, d), group=group)
            dist.all_gather_into_tensor(v_full.view(total, hkv, d), v8.view(ns, hkv, d), group=group)
        else:
            k_full, v_full = k8, v8

        def per_head(w):
            return [float(w)] * hq if isinstance(w, (int, float)) else [float(x) for x in w]

        return backend.windowed_prefill(q8, k_full, v_full, per_head(bit8_window_sizes), per_head(bit4_window_sizes),
                                        sink_window_size, lo, p_fp8_mode)

    return attention_fn


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
