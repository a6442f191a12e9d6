"""CPU oracle for the key clustering path (cache_hub/kmeans.py).

TEST INFRASTRUCTURE ONLY: the shipped package never imports this module.

The reference accumulates cluster sums with relaxed fp32 atomics, so its own
results depend on thread arrival order.  This restatement fixes the arithmetic
so that it has one answer that a GPU implementation can reproduce bit for bit:

* scores <k_t, x_c> are evaluated in fp64 (products of 16-bit inputs are exact,
  the sum is accurate to ~1e-16 relative); argmax ties go to the lowest centroid
  index, the reference's rule (kmeans.py:56-65: leftmost inside a chunk, strict
  ">" across chunks);
* member sums are exact (fp64 accumulation of 16-bit values; exact while the
  dynamic range of a cluster stays below 2^45) and rounded once to fp32;
* x = S/C in fp32 (kmeans.py:118-121); the optional normalisation divides by
  sqrt(sum_d x_d^2) with the sum taken in fp64 in index order and one rounding
  to fp32, then the centroid is stored in the key dtype (kmeans.py:122-124);
* member lists are sorted by token index (the reference's order is the atomic
  arrival order, kmeans.py:219-230).

Parity of this file against the reference is pinned up to those choices:
assignments and counts agree with the reference's assign/update kernels run by
Triton's CPU interpreter (tests/golden/kmeans.npz), and ``segment_k_means`` as a
whole (centroid initialisation, segmenting, the iteration schedule, value sums,
member lists) agrees with the reference's own function executed through a
``paddle`` module that forwards to torch (segment_kmeans.npz): cluster sizes and
sorted member lists exactly, centroids and value sums to one unit in the last
place of their 16-bit type.  ``select_clusters`` has no counterpart in the
reference (retrieval is not shipped there) and is unpinned.
"""
from __future__ import annotations

import torch


def init_centroid_indices(num_tokens: int, num_centroids: int) -> torch.Tensor:
    """kmeans.py:340-344: fp32 arange * (T/K) + T/K/2, truncated to int64."""
    idx = torch.arange(num_centroids, dtype=torch.float32) * (num_tokens / num_centroids)
    idx += num_tokens / num_centroids / 2
    return idx.to(torch.int64)


def assign(data: torch.Tensor, centroids: torch.Tensor) -> torch.Tensor:
    """argmax_c <k_t, x_c>, lowest index on ties (kmeans.py:56-66).
    data [G,T,D], centroids [G,K,D] -> int32 [G,T]."""
    scores = torch.matmul(data.double(), centroids.double().transpose(1, 2))  # [G,T,K]
    mx = scores.max(dim=-1, keepdim=True).values
    k = scores.shape[-1]
    idx = torch.where(scores == mx, torch.arange(k)[None, None, :], torch.tensor(k))
    return idx.min(dim=-1).values.to(torch.int32)


def cluster_sums(data: torch.Tensor, max_idx: torch.Tensor, num_centroids: int):
    """Exact member sums (rounded once to fp32) and int32 counts
    (kmeans.py:67-79 without the order dependence)."""
    g, t, d = data.shape
    s = torch.zeros(g, num_centroids, d, dtype=torch.float64)
    s.index_put_((torch.arange(g)[:, None].expand(g, t), max_idx.long()), data.double(), accumulate=True)
    c = torch.zeros(g, num_centroids, dtype=torch.int64)
    c.index_put_((torch.arange(g)[:, None].expand(g, t), max_idx.long()),
                 torch.ones(g, t, dtype=torch.int64), accumulate=True)
    return s.float(), c.to(torch.int32)


def update(centroids: torch.Tensor, s: torch.Tensor, c: torch.Tensor, normalize: bool) -> torch.Tensor:
    """x = S/C where C>0, optional L2 normalisation, stored in the centroid
    dtype; empty clusters keep their old centroid (kmeans.py:116-124)."""
    cf = c.float()[..., None]
    x = s / torch.where(cf > 0, cf, torch.ones_like(cf))
    if normalize:
        xd = x.double()
        sq = xd * xd
        nrm = torch.zeros(x.shape[:-1], dtype=torch.float64)
        for j in range(x.shape[-1]):  # index order, fp64
            nrm = nrm + sq[..., j]
        x = (xd / torch.sqrt(nrm)[..., None]).float()
    new = x.to(centroids.dtype)
    return torch.where((c > 0)[..., None], new, centroids)


def k_means_train(data, centroids, normalize_centroids=True):
    """_triton_k_means_train (kmeans.py:127-196) -> (centroids, max_idx, counts)."""
    max_idx = assign(data, centroids)
    s, c = cluster_sums(data, max_idx, centroids.shape[1])
    return update(centroids, s, c, normalize_centroids), max_idx, c


def reverse_index(max_idx: torch.Tensor, num_centroids: int, max_cluster_size: int):
    """triton_reverse_index (kmeans.py:233-262) with members sorted by token."""
    g, t = max_idx.shape
    clusters = torch.zeros(g, num_centroids, max_cluster_size, dtype=torch.int32)
    sizes = torch.zeros(g, num_centroids, dtype=torch.int32)
    for gi in range(g):
        order = torch.argsort(max_idx[gi].long() * t + torch.arange(t))
        sorted_c = max_idx[gi][order].long()
        counts = torch.bincount(sorted_c, minlength=num_centroids)
        sizes[gi] = counts.to(torch.int32)
        starts = torch.cumsum(counts, 0) - counts
        slot = torch.arange(t) - starts[sorted_c]
        clusters[gi, sorted_c, slot] = order.to(torch.int32)
    return clusters, sizes


def index_add(value: torch.Tensor, max_idx: torch.Tensor, num_centroids: int) -> torch.Tensor:
    """triton_index_add (kmeans.py:307-329): per-cluster value sums, exact then
    rounded to fp32 and cast to the value dtype."""
    s, _ = cluster_sums(value, max_idx, num_centroids)
    return s.to(value.dtype)


def segment_k_means(key, value, num_centroids: int, num_iters: int = 10, num_segments: int = 1):
    """segment_k_means (kmeans.py:332-375).
    key/value [G,T,D] -> (centroids [G,K,D], value_sum [G,K,D],
    clusters [G,K,max_cluster_size] int32, cluster_size [G,K] int32).
    Also returns max_idx [G,T] as a fifth element for checking."""
    g, t, d = key.shape
    assert num_centroids % 32 == 0  # kmeans.py:146
    idx = init_centroid_indices(t, num_centroids)
    centroids = key.index_select(1, idx)
    assert num_centroids % num_segments == 0
    tps = t // num_segments
    cps = num_centroids // num_segments
    data = key[:, : tps * num_segments].reshape(-1, tps, d)
    centroids = centroids.reshape(-1, cps, d)
    for _ in range(num_iters - 1):
        centroids, _, _ = k_means_train(data, centroids, True)
    data = key.reshape(-1, t, d)
    centroids = centroids.reshape(-1, num_centroids, d)
    centroids, max_idx, counts = k_means_train(data, centroids, False)
    max_cluster_size = int(counts.max().item())
    value_sum = index_add(value.reshape(-1, t, d), max_idx, num_centroids)
    clusters, cluster_size = reverse_index(max_idx, num_centroids, max_cluster_size)
    return centroids, value_sum, clusters, cluster_size, max_idx


def fold_tokens(key, value, assignments, centroids, num_clustered: int):
    """Growth of a clustered cache (no counterpart in the reference, which clusters once): the tokens from
    ``num_clustered`` on are assigned to their best centroid by the exact rule of ``assign``, older assignments stay,
    and centroids, value sums and member lists are recomputed from all assignments with the final iteration's rule
    (mean of the members, no normalisation, kmeans.py:362-366).
    key/value [G,T,D], assignments [G,num_clustered] -> (centroids, value_sum, clusters, cluster_size,
    assignments [G,T])."""
    g, t, d = key.shape
    k = centroids.shape[1]
    new = assign(key[:, num_clustered:], centroids) if t > num_clustered else assignments[:, :0]
    full = torch.cat([assignments[:, :num_clustered], new], dim=1)
    s, c = cluster_sums(key, full, k)
    cent = update(centroids, s, c, False)
    vsum = index_add(value, full, k)
    clusters, csize = reverse_index(full, k, int(c.max().item()))
    return cent, vsum, clusters, csize, full


def select_clusters(q_mean: torch.Tensor, centroids: torch.Tensor, cluster_size: torch.Tensor,
                    clusters: torch.Tensor, budget: int):
    """Centroid-scored retrieval (not in the reference; it completes the decode
    path its logs hint at): score_c = <q_mean, x_c> in fp64, clusters taken in
    descending score (ties: lowest index) until at least ``budget`` tokens are
    covered; returns per group the sorted selected token indices."""
    g = centroids.shape[0]
    out = []
    for gi in range(g):
        sc = torch.matmul(centroids[gi].double(), q_mean[gi].double())
        order = torch.argsort(-sc, stable=True)
        toks, total = [], 0
        for cidx in order.tolist():
            if total >= budget:
                break
            n = int(cluster_size[gi, cidx])
            if n == 0:
                continue
            toks.append(clusters[gi, cidx, :n])
            total += n
        sel = torch.sort(torch.cat(toks)).values if toks else torch.zeros(0, dtype=torch.int32)
        out.append(sel.to(torch.int32))
    return out
