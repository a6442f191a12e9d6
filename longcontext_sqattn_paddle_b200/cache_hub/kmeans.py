"""segment_k_means with the reference's signature and return values (cache_hub/kmeans.py:332-375), on the
library's clustering kernels.  Results do not depend on thread timing: assignments are exact (lowest index
on ties), member sums are exact, member lists are sorted by token index."""
from __future__ import annotations

import torch

from .. import _lib as L
from ..ops import _dt, _require_cuda, _stream, _workspace


def init_centroid_indices(num_tokens: int, num_centroids: int, device) -> torch.Tensor:
    """fp32 arange * (T/K) + T/K/2 truncated to int64 (kmeans.py:340-344)."""
    idx = torch.arange(num_centroids, dtype=torch.float32, device=device) * (num_tokens / num_centroids)
    idx += num_tokens / num_centroids / 2
    return idx.to(torch.int64)


def k_means_train(data: torch.Tensor, centroids: torch.Tensor, normalize_centroids: bool = True, scratch=None):
    """One assign + update pass (_triton_k_means_train, kmeans.py:127-196).
    Updates ``centroids`` in place; returns (centroids, max_idx, counts).  ``scratch`` (a dict) lets a loop of
    iterations reuse the index, sum and workspace buffers."""
    _require_cuda(data, centroids)
    g, t, d = data.shape
    k = centroids.shape[1]
    assert k % 32 == 0
    data = data.contiguous()
    assert centroids.is_contiguous()
    key = (g, t, k, d, data.device)
    if scratch is None or scratch.get("key") != key:
        need = L.lib.sqattn_kmeans_workspace_bytes(g, t, k)
        fresh = dict(key=key, idx=torch.empty(g, t, dtype=torch.int32, device=data.device),
                     sums=torch.empty(g, k, d, dtype=torch.float64, device=data.device),
                     counts=torch.empty(g, k, dtype=torch.int32, device=data.device), ws=_workspace(need, data.device), need=need)
        if scratch is None:
            scratch = fresh
        else:
            scratch.update(fresh)
    idx, sums, counts, ws = scratch["idx"], scratch["sums"], scratch["counts"], scratch["ws"]
    counts.zero_()
    L.check(L.lib.sqattn_kmeans_assign(data.data_ptr(), centroids.data_ptr(), _dt(data.dtype), g, t, k, d,
                                       idx.data_ptr(), sums.data_ptr(), counts.data_ptr(), ws.data_ptr(), scratch["need"],
                                       _stream()))
    L.check(L.lib.sqattn_kmeans_update(centroids.data_ptr(), _dt(data.dtype), sums.data_ptr(), counts.data_ptr(), g, k,
                                       d, int(normalize_centroids), _stream()))
    return centroids, idx, counts


def reverse_index(max_idx: torch.Tensor, num_centroids: int, max_cluster_size: int):
    g, t = max_idx.shape
    clusters = torch.zeros(g, num_centroids, max_cluster_size, dtype=torch.int32, device=max_idx.device)
    cluster_size = torch.zeros(g, num_centroids, dtype=torch.int32, device=max_idx.device)
    need = L.lib.sqattn_kmeans_workspace_bytes(g, t, num_centroids)
    ws = _workspace(need, max_idx.device)
    L.check(L.lib.sqattn_kmeans_reverse_index(max_idx.data_ptr(), g, t, num_centroids, max_cluster_size,
                                              clusters.data_ptr(), cluster_size.data_ptr(), ws.data_ptr(), need, _stream()))
    return clusters, cluster_size


def index_add(value: torch.Tensor, max_idx: torch.Tensor, num_centroids: int) -> torch.Tensor:
    g, t, d = value.shape
    value = value.contiguous()
    sums = torch.empty(g, num_centroids, d, dtype=torch.float64, device=value.device)
    out = torch.empty(g, num_centroids, d, dtype=value.dtype, device=value.device)
    need = L.lib.sqattn_kmeans_workspace_bytes(g, t, num_centroids)
    ws = _workspace(need, value.device)
    L.check(L.lib.sqattn_kmeans_index_add(value.data_ptr(), _dt(value.dtype), max_idx.data_ptr(), g, t, num_centroids, d,
                                          sums.data_ptr(), out.data_ptr(), ws.data_ptr(), need, _stream()))
    return out


def segment_k_means(key: torch.Tensor, value: torch.Tensor, num_centroids: int, num_iters: int = 10,
                    num_segments: int = 1, return_indices: bool = False):
    """key/value [G,T,D] -> (centroids, value_sum, clusters, cluster_size) (+ max_idx when asked)."""
    g, t, d = key.shape
    idx = init_centroid_indices(t, num_centroids, key.device)
    centroids = torch.index_select(key, 1, idx)
    assert num_centroids % num_segments == 0
    tps = t // num_segments
    cps = num_centroids // num_segments
    data = key[:, : tps * num_segments].reshape(-1, tps, d)
    centroids = centroids.reshape(-1, cps, d).contiguous()
    scratch = {}
    for _ in range(num_iters - 1):
        centroids, _, _ = k_means_train(data, centroids, True, scratch)
    data = key.reshape(-1, t, d)
    centroids = centroids.reshape(-1, num_centroids, d)
    centroids, max_idx, counts = k_means_train(data, centroids, False)
    mx = torch.zeros(1, dtype=torch.int32, device=key.device)
    L.check(L.lib.sqattn_kmeans_max_count(counts.data_ptr(), counts.numel(), mx.data_ptr(), _stream()))
    max_cluster_size = int(mx.item())  # the reference synchronises here too (kmeans.py:195)
    value_sum = index_add(value.reshape(-1, t, d), max_idx, num_centroids)
    clusters, cluster_size = reverse_index(max_idx, num_centroids, max_cluster_size)
    if return_indices:
        return centroids, value_sum, clusters, cluster_size, max_idx
    return centroids, value_sum, clusters, cluster_size
