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
    """One sequence: key/value [Hkv, T, D], clustered per KV head, growing as tokens are decoded.

    ``capacity`` reserves room for appended tokens.  ``append`` stores a new token's key/value; it joins no cluster
    at once but is always attended (the retrieval step selects every token from ``clustered`` on), and after
    ``fold_every`` appended tokens ``fold`` assigns them to their best centroid (the exact arg-max rule of the
    clustering), recomputes the centroids as the means of their members (what the last Lloyd iteration leaves,
    cache_hub/kmeans.py:362-366), the value sums and the member lists.  Assignments of older tokens never change.

    ``host_rows``: a block-hybrid layout like the reference's CPU-GPU cache (cache_hub/cache.py,
    flash_attn_cache.py:128-141): the first ``split`` tokens stay on the GPU, the rest of K and V live in pinned
    host memory and the gather kernel reads the selected rows from there.  Clustering needs all keys once, so the
    host part is staged through the GPU for ``__init__`` and ``fold`` and released again."""

    def __init__(self, key: torch.Tensor, value: torch.Tensor, tokens_per_cluster: int = 64, num_iters: int = 10,
                 capacity: int = 0, fold_every: int = 256, split: int = -1):
        assert key.dim() == 3 and key.is_cuda
        self.hkv, self.tokens, self.d = key.shape
        self.capacity = max(int(capacity), self.tokens)
        self.fold_every = int(fold_every)
        self.k = num_clusters_for(self.tokens, tokens_per_cluster)
        key, value = key.contiguous(), value.contiguous()
        self.centroids, self.value_sum, self.clusters, self.cluster_size, self.assign = segment_k_means(
            key, value, self.k, num_iters, return_indices=True)
        self.max_cluster_size = self.clusters.shape[2]
        self.clustered = self.tokens                       # tokens [clustered, tokens) are the unclustered tail
        if self.capacity > self.tokens:
            pad = self.capacity - self.tokens
            self.assign = torch.cat([self.assign, torch.zeros(self.hkv, pad, dtype=torch.int32, device=key.device)], dim=1)
        # storage: [Hkv, split, 2, D] on the GPU and, for a hybrid layout, [Hkv, capacity - split, 2, D] in pinned host
        # memory.  A token's key row and value row sit next to each other (rows 2 * D elements apart in both views):
        # a retrieval step reads scattered tokens, and one 512-byte piece per token costs the DRAM half the page
        # openings of two 256-byte pieces in two arrays.
        self.split = self.capacity if split < 0 else min(int(split), self.tokens)
        dev_rows = self.split if split >= 0 else self.capacity
        self.kv = torch.empty(self.hkv, dev_rows, 2, self.d, dtype=key.dtype, device=key.device)
        self.key, self.value = self.kv[:, :, 0], self.kv[:, :, 1]
        n_dev = min(self.tokens, dev_rows)
        self.key[:, :n_dev], self.value[:, :n_dev] = key[:, :n_dev], value[:, :n_dev]
        self.key_host = self.value_host = None
        if split >= 0:
            rows = self.capacity - self.split
            self.kv_host = torch.empty(self.hkv, rows, 2, self.d, dtype=key.dtype, pin_memory=True)
            self.key_host, self.value_host = self.kv_host[:, :, 0], self.kv_host[:, :, 1]
            self.key_host[:, :self.tokens - self.split].copy_(key[:, self.split:])
            self.value_host[:, :self.tokens - self.split].copy_(value[:, self.split:])
            torch.cuda.synchronize(key.device)

    # ---- growth ---------------------------------------------------------------------------------------------
    def _rows(self, which: str, lo: int, hi: int) -> torch.Tensor:
        """tokens [lo, hi) of K or V as one device tensor [Hkv, hi-lo, D] (the host part is uploaded)"""
        dev = self.key if which == "k" else self.value
        host = self.key_host if which == "k" else self.value_host
        parts = []
        if lo < min(hi, self.split):
            parts.append(dev[:, lo:min(hi, self.split)])
        if host is not None and hi > self.split:
            parts.append(host[:, max(lo, self.split) - self.split:hi - self.split].to(dev.device, non_blocking=True))
        return parts[0] if len(parts) == 1 else torch.cat(parts, dim=1)

    def append(self, k_new: torch.Tensor, v_new: torch.Tensor):
        """k_new / v_new [Hkv, D]: the next token of this sequence."""
        if self.tokens >= self.capacity:
            raise ValueError(f"the clustered cache is full ({self.capacity} tokens)")
        t = self.tokens
        if t < self.split:
            self.key[:, t], self.value[:, t] = k_new, v_new
        else:
            self.key_host[:, t - self.split].copy_(k_new, non_blocking=True)
            self.value_host[:, t - self.split].copy_(v_new, non_blocking=True)
        self.tokens = t + 1
        if self.tokens - self.clustered >= self.fold_every:
            self.fold()

    def fold(self):
        """Give the tail tokens to their clusters and rebuild centroids, value sums and member lists."""
        if self.tokens == self.clustered:
            return
        from . import kmeans as km
        dev = self.key.device
        torch.cuda.current_stream(dev).synchronize()         # appended host rows have landed
        tail = self._rows("k", self.clustered, self.tokens).contiguous()
        n_tail = tail.shape[1]
        idx = torch.empty(self.hkv, n_tail, dtype=torch.int32, device=dev)
        need = L.lib.sqattn_kmeans_workspace_bytes(self.hkv, n_tail, self.k)
        ws = ops._workspace(need, dev)
        L.check(L.lib.sqattn_kmeans_assign(tail.data_ptr(), self.centroids.data_ptr(), _dt(tail.dtype), self.hkv, n_tail,
                                           self.k, self.d, idx.data_ptr(), None, None, ws.data_ptr(), need, _stream()))
        self.assign[:, self.clustered:self.tokens] = idx
        t = self.tokens
        assign = self.assign[:, :t].contiguous()
        keys, vals = self._rows("k", 0, t).contiguous(), self._rows("v", 0, t).contiguous()
        need = L.lib.sqattn_kmeans_workspace_bytes(self.hkv, t, self.k)
        ws = ops._workspace(need, dev)
        sums = torch.empty(self.hkv, self.k, self.d, dtype=torch.float64, device=dev)
        scratch16 = torch.empty(self.hkv, self.k, self.d, dtype=keys.dtype, device=dev)
        # exact member sums of the keys (fp64) -> centroid = sum / count, no normalisation (the final iteration's rule)
        L.check(L.lib.sqattn_kmeans_index_add(keys.data_ptr(), _dt(keys.dtype), assign.data_ptr(), self.hkv, t, self.k, self.d,
                                              sums.data_ptr(), scratch16.data_ptr(), ws.data_ptr(), need, _stream()))
        counts = torch.zeros(self.hkv, self.k, dtype=torch.int32, device=dev)
        counts.view(-1).index_add_(0, (assign.long() + torch.arange(self.hkv, device=dev)[:, None] * self.k).view(-1),
                                   torch.ones(assign.numel(), dtype=torch.int32, device=dev))
        L.check(L.lib.sqattn_kmeans_update(self.centroids.data_ptr(), _dt(keys.dtype), sums.data_ptr(), counts.data_ptr(),
                                           self.hkv, self.k, self.d, 0, _stream()))
        self.value_sum = km.index_add(vals, assign, self.k)
        self.max_cluster_size = int(counts.max().item())
        self.clusters, self.cluster_size = km.reverse_index(assign, self.k, self.max_cluster_size)
        self.clustered = t

    # ---- retrieval ------------------------------------------------------------------------------------------
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
                                             out_idx.data_ptr(), out_count.data_ptr(), cap, self.clustered, _stream()))
        return out_idx, out_count

    def gather(self, idx: torch.Tensor, count: torch.Tensor, cap: int, k_out: torch.Tensor, v_out: torch.Tensor):
        """k_out/v_out [Hkv, cap, D] <- rows idx[h, :count[h]] of this sequence's K and V (device-resident layouts)."""
        if self.key_host is not None:
            raise ValueError("hybrid layouts gather through RaggedClusteredDecoder.step (the batched entry point)")
        for src, dst in ((self.key, k_out), (self.value, v_out)):
            L.check(L.lib.sqattn_gather_rows(src.data_ptr(), src.stride(0), src.stride(1), idx.data_ptr(), count.data_ptr(),
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
        # room for the budget, the cluster that crosses it, and the unclustered tail between two folds
        self.cap = (budget + max(c.max_cluster_size for c in self.caches) + max(c.fold_every for c in self.caches)
                    + 63) // 64 * 64
        b = len(self.caches)
        self.idx = torch.empty(b, self.hkv, self.cap, dtype=torch.int32, device=dev)
        self.count = torch.empty(b, self.hkv, dtype=torch.int32, device=dev)
        self.k_sel = torch.empty(b * self.hkv, 1, self.cap, self.d, dtype=dt, device=dev)
        self.v_sel = torch.empty(b * self.hkv, 1, self.cap, self.d, dtype=dt, device=dev)
        self._q = None        # persistent copy of the step's queries: the item table below points into it
        self._items, self._state = None, None
        self._rows = None     # device arrays of the K / V base pointers of every (sequence, KV head), for in-place attention

    def _in_place(self) -> bool:
        """The selected rows can be attended where they lie when every cache is wholly on the device and all share a
        row stride (block-hybrid caches go through the packing kernel, which also reads the host part)."""
        return all(c.key_host is None for c in self.caches)

    def _table(self, hq: int):
        """One sqattn_retrieve_item per sequence; every pointer in it stays valid for the decoder's lifetime."""
        b = len(self.caches)
        in_place = self._in_place()
        self._q = torch.empty(b, hq, 1, self.d, dtype=self.caches[0].key.dtype, device=self.idx.device)
        items = (L.RetrieveItem * b)()
        for i, c in enumerate(self.caches):
            it = items[i]
            it.q, it.centroids = self._q[i].data_ptr(), c.centroids.data_ptr()
            it.cluster_size, it.clusters = c.cluster_size.data_ptr(), c.clusters.data_ptr()
            it.num_clusters, it.max_cluster_size, it.num_tokens = c.k, c.max_cluster_size, c.tokens
            it.tail_start = c.clustered
            it.out_idx, it.out_count = self.idx[i].data_ptr(), self.count[i].data_ptr()
            it.k_src, it.v_src = c.key.data_ptr(), c.value.data_ptr()
            it.src_group_stride, it.src_row_stride = c.key.stride(0), c.key.stride(1)
            if c.key_host is not None:      # hybrid layout: rows from `split` on are read from pinned host memory
                it.split_row, it.k_src2, it.v_src2 = c.split, c.key_host.data_ptr(), c.value_host.data_ptr()
                it.src2_group_stride = c.key_host.stride(0)
            if not in_place:   # no destination in any item: sqattn_retrieve_batch only selects
                it.k_dst = self.k_sel[i * self.hkv:(i + 1) * self.hkv].data_ptr()
                it.v_dst = self.v_sel[i * self.hkv:(i + 1) * self.hkv].data_ptr()
        self._items = items
        if in_place:
            esz = self.caches[0].key.element_size()
            kp = [c.key.data_ptr() + h * c.key.stride(0) * esz for c in self.caches for h in range(self.hkv)]
            vp = [c.value.data_ptr() + h * c.value.stride(0) * esz for c in self.caches for h in range(self.hkv)]
            dev = self.idx.device
            self._rows = (torch.tensor(kp, dtype=torch.int64, device=dev), torch.tensor(vp, dtype=torch.int64, device=dev))

    def step(self, q: torch.Tensor, out_dtype=None) -> torch.Tensor:
        """Three launches and no host synchronisation: select (all sequences), split-KV decode that copies the listed
        rows from the caches into shared memory itself (lengths read on the device), merge.  Block-hybrid caches add a
        launch that packs the rows (device and host part) first."""
        b, hq, _, d = q.shape
        groups = hq // self.hkv
        state = tuple((c.tokens, c.clustered, c.max_cluster_size, c.clusters.data_ptr()) for c in self.caches)
        if self._items is None or self._q.shape[1] != hq or state != self._state:
            if any(c.max_cluster_size + c.fold_every + self.budget > self.cap for c in self.caches):
                raise ValueError("a cluster outgrew the gather buffers: rebuild the decoder")
            self._table(hq)                 # the table holds sizes and pointers that appends and folds change
            self._state = state
        self._q.copy_(q)
        L.check(L.lib.sqattn_retrieve_batch(self._items, b, _dt(q.dtype), self.hkv, groups, d, self.budget, self.cap,
                                            _stream()))
        qv = self._q.view(b * self.hkv, groups, 1, d)
        if self._in_place():
            o = ops.decode_gather(qv, self.idx.view(b * self.hkv, self.cap), self.count.view(-1), self._rows[0], self._rows[1],
                                  self.caches[0].key.stride(1), q.dtype, out_dtype=out_dtype or q.dtype, p_fp8=self.p_fp8)
        else:
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
