"""Clustered KV retrieval for decode: keys of every KV head are clustered once (segment_k_means), and each decode
step attends only to the tokens of the best-scoring clusters up to a token budget.  The reference ships the
clustering (cache_hub/kmeans.py) but not the retrieval its logs mention; this module completes that path on the
library's kernels (sqattn_retrieve_select, sqattn_gather_rows, sqattn_decode)."""
from __future__ import annotations

from typing import List, Sequence

import torch

from .. import _lib as L
from .. import ops
from ..ops import _dt, _stream
from .kmeans import segment_k_means


def num_clusters_for(num_tokens: int, tokens_per_cluster: int = 64) -> int:
    """len/64 centroids rounded to a multiple of 32 (the assign kernel's requirement, kmeans.py:146), at least 32."""
    k = int(round(num_tokens / tokens_per_cluster / 32.0)) * 32
    return max(32, k)


class ClusteredKV:
    """One sequence: key/value [Hkv, T, D] on the GPU, clustered per KV head."""

    def __init__(self, key: torch.Tensor, value: torch.Tensor, tokens_per_cluster: int = 64, num_iters: int = 10):
        assert key.dim() == 3 and key.is_cuda
        self.key, self.value = key.contiguous(), value.contiguous()
        self.hkv, self.tokens, self.d = key.shape
        self.k = num_clusters_for(self.tokens, tokens_per_cluster)
        self.centroids, self.value_sum, self.clusters, self.cluster_size = segment_k_means(self.key, self.value, self.k,
                                                                                            num_iters)
        self.max_cluster_size = self.clusters.shape[2]

    def select(self, q: torch.Tensor, budget: int, cap: int, out_idx=None, out_count=None):
        """q [Hq, D] (the group's query heads are consecutive) -> (idx [Hkv, cap] int32 ascending, count [Hkv])."""
        hq = q.shape[0]
        if out_idx is None:
            out_idx = torch.empty(self.hkv, cap, dtype=torch.int32, device=q.device)
            out_count = torch.empty(self.hkv, dtype=torch.int32, device=q.device)
        q = q.contiguous()
        L.check(L.lib.sqattn_retrieve_select(q.data_ptr(), self.centroids.data_ptr(), _dt(self.key.dtype),
                                             self.cluster_size.data_ptr(), self.clusters.data_ptr(), self.hkv,
                                             hq // self.hkv, self.k, self.d, self.max_cluster_size, self.tokens, budget,
                                             out_idx.data_ptr(), out_count.data_ptr(), cap, _stream()))
        return out_idx, out_count

    def gather(self, idx: torch.Tensor, count: torch.Tensor, cap: int, k_out: torch.Tensor, v_out: torch.Tensor):
        """k_out/v_out [Hkv, cap, D] <- rows idx[h, :count[h]] of this sequence's K and V."""
        for src, dst in ((self.key, k_out), (self.value, v_out)):
            L.check(L.lib.sqattn_gather_rows(src.data_ptr(), self.tokens * self.d, self.d, idx.data_ptr(), count.data_ptr(),
                                             self.hkv, cap, self.d, dst.data_ptr(), _stream()))


class RaggedClusteredDecoder:
    """A ragged batch of sequences with clustered caches.  ``step(q)`` with q [B, Hq, 1, D] retrieves up to
    ``budget`` tokens per (sequence, KV head), gathers them and attends with FP8-rounded P; every
    (sequence, KV head) pair is one row of a batched split-KV decode call."""

    def __init__(self, caches: Sequence[ClusteredKV], budget: int = 4096, p_fp8: bool = True, hq: int = 0):
        self.caches: List[ClusteredKV] = list(caches)
        self.budget, self.p_fp8 = budget, p_fp8
        c0 = self.caches[0]
        self.hkv, self.d, dev, dt = c0.hkv, c0.d, c0.key.device, c0.key.dtype
        self.cap = (budget + max(c.max_cluster_size for c in self.caches) + 63) // 64 * 64
        b = len(self.caches)
        self.idx = torch.empty(b, self.hkv, self.cap, dtype=torch.int32, device=dev)
        self.count = torch.empty(b, self.hkv, dtype=torch.int32, device=dev)
        self.k_sel = torch.empty(b * self.hkv, 1, self.cap, self.d, dtype=dt, device=dev)
        self.v_sel = torch.empty(b * self.hkv, 1, self.cap, self.d, dtype=dt, device=dev)
        self._q = None        # persistent copy of the step's queries: the item table below points into it
        self._items = None

    def _table(self, hq: int):
        """One sqattn_retrieve_item per sequence; every pointer in it stays valid for the decoder's lifetime."""
        b = len(self.caches)
        self._q = torch.empty(b, hq, 1, self.d, dtype=self.caches[0].key.dtype, device=self.idx.device)
        items = (L.RetrieveItem * b)()
        for i, c in enumerate(self.caches):
            it = items[i]
            it.q, it.centroids = self._q[i].data_ptr(), c.centroids.data_ptr()
            it.cluster_size, it.clusters = c.cluster_size.data_ptr(), c.clusters.data_ptr()
            it.num_clusters, it.max_cluster_size, it.num_tokens = c.k, c.max_cluster_size, c.tokens
            it.out_idx, it.out_count = self.idx[i].data_ptr(), self.count[i].data_ptr()
            it.k_src, it.v_src = c.key.data_ptr(), c.value.data_ptr()
            it.src_group_stride, it.src_row_stride = c.tokens * self.d, self.d
            it.k_dst = self.k_sel[i * self.hkv:(i + 1) * self.hkv].data_ptr()
            it.v_dst = self.v_sel[i * self.hkv:(i + 1) * self.hkv].data_ptr()
        self._items = items

    def step(self, q: torch.Tensor, out_dtype=None) -> torch.Tensor:
        """Four launches and no host synchronisation: select (all sequences), gather (all keys and values), split-KV
        decode with the retrieved counts read on the device, merge."""
        b, hq, _, d = q.shape
        groups = hq // self.hkv
        if self._items is None or self._q.shape[1] != hq:
            self._table(hq)
        self._q.copy_(q)
        L.check(L.lib.sqattn_retrieve_batch(self._items, b, _dt(q.dtype), self.hkv, groups, d, self.budget, self.cap,
                                            _stream()))
        qv = self._q.view(b * self.hkv, groups, 1, d)
        o = ops.decode(qv, self.k_sel, self.v_sel, out_dtype=out_dtype or q.dtype, p_fp8=self.p_fp8, kv_len=self.cap,
                       kv_lens_device=self.count.view(-1))
        return o.view(b, hq, 1, d)

    def step_unbatched(self, q: torch.Tensor, out_dtype=None) -> torch.Tensor:
        """The same through the per-sequence entry points (one select and two gathers per sequence, lengths read back
        to the host for the planner); kept as the cross-check of ``step``."""
        b, hq, _, d = q.shape
        groups = hq // self.hkv
        for i, c in enumerate(self.caches):
            c.select(q[i, :, 0], self.budget, self.cap, self.idx[i], self.count[i])
            c.gather(self.idx[i], self.count[i], self.cap, self.k_sel[i * self.hkv:(i + 1) * self.hkv, 0],
                     self.v_sel[i * self.hkv:(i + 1) * self.hkv, 0])
        lens = self.count.flatten().tolist()
        qv = q.reshape(b * self.hkv, groups, 1, d)
        o = ops.decode(qv, self.k_sel, self.v_sel, out_dtype=out_dtype or q.dtype, p_fp8=self.p_fp8, kv_lens=lens)
        return o.view(b, hq, 1, d)
