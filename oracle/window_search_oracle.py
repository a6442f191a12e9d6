"""CPU oracle for the window calibration (sqattn/window_search.py).

TEST INFRASTRUCTURE ONLY: the shipped package never imports this module.  The reference has no test of this
code; it is pinned against outputs of the reference's own functions (cal_attn_weight, the histogram functions and
the two threshold searches) executed through a ``paddle`` module that forwards to torch
(tests/golden/make_golden.py, window_search.npz).
"""
from __future__ import annotations

import math

import numpy as np
import torch


def attention_map(q: torch.Tensor, k: torch.Tensor) -> torch.Tensor:
    """cal_attn_weight (sqattn/attn_replacer.py:253-278) in fp64: softmax(q k^T / sqrt(D)) with a causal mask.
    q [Hq,N,D], k [Hkv,N,D] -> [Hq,N,N]."""
    hq, n, d = q.shape
    groups = hq // k.shape[0]
    kk = k.repeat_interleave(groups, dim=0).double()
    s = torch.matmul(q.double(), kk.transpose(1, 2)) / math.sqrt(d)
    mask = torch.ones(n, n, dtype=torch.bool).tril()
    return torch.softmax(s.masked_fill(~mask, float("-inf")), dim=-1)


def relative_histogram_with_sink(a: torch.Tensor, num_bins: int = 200, sink_len: int = 128) -> np.ndarray:
    """compute_relative_attention_histogram_gpu_with_sink (window_search.py:244-283) for one [N,N] map."""
    n = a.shape[0]
    rows = torch.arange(n)[:, None]
    cols = torch.arange(n)[None, :]
    non_sink = torch.ones(n, n, dtype=torch.bool)
    non_sink[:, :sink_len] = False
    # distances, relative distances and bin indices in fp32 like the reference (bin edges depend on it)
    dist = (rows - cols).float()
    ctx = torch.clamp(rows.float() - sink_len, min=1)
    rel = dist / ctx
    rel[(rows.squeeze() <= sink_len)] = 0
    bins = torch.clamp((rel * num_bins).floor().long(), 0, num_bins - 1)
    w = a.double() * non_sink * (rel * num_bins + 1).double()
    m = torch.ones(n, n, dtype=torch.bool).tril() & non_sink
    return torch.bincount(bins[m], weights=w[m], minlength=num_bins).numpy()


def absolute_histogram_with_sink(a: torch.Tensor, max_len: int, sink_len: int = 0) -> np.ndarray:
    """compute_absolute_attention_histogram_gpu_with_sink (286-321); sink_len = 0 gives
    compute_attention_histogram_gpu (20-48)."""
    n = a.shape[0]
    rows = torch.arange(n)[:, None]
    cols = torch.arange(n)[None, :]
    non_sink = torch.ones(n, n, dtype=torch.bool)
    non_sink[:, :sink_len] = False
    dist = rows - cols
    w = a.double() * non_sink * dist.double()
    m = torch.ones(n, n, dtype=torch.bool).tril() & non_sink
    h = torch.bincount(dist[m], weights=w[m], minlength=max_len)
    return h[:max_len].numpy()


def find_optimal_relative_window(histogram: np.ndarray, threshold: float, num_bins: int = 100) -> float:
    """window_search.py:88-113."""
    total = np.sum(histogram)
    if total == 0:
        return 0.1
    cum, best = 0.0, 0
    for b in range(len(histogram)):
        cum += histogram[b]
        if cum >= threshold * total:
            best = b
            break
    return min((best + 1) / num_bins, 1.0)


def find_optimal_window(histogram: np.ndarray, threshold: float) -> int:
    """window_search.py:116-128 (128-token steps)."""
    total = np.sum(histogram)
    if total == 0:
        return 1
    cum = 0.0
    for d in range(0, len(histogram), 128):
        cum += sum(histogram[d:d + 128])
        if cum >= threshold * total:
            return d + 128
    return len(histogram)
