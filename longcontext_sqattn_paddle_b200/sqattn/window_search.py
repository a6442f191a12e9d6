"""Window calibration with the reference's function names and results (sqattn/window_search.py): histograms of
distance-weighted attention energy per head, and the smallest window that keeps a given share of it.  The
histograms come from q and k directly (sqattn_window_histogram): the reference first materialises the dense
[H, N, N] softmax map (cal_attn_weight), which limits it to a few thousand tokens."""
from __future__ import annotations

import json
from typing import Dict, List, Sequence

import numpy as np
import torch

from .. import _lib as L
from ..ops import _dt, _require_cuda, _stream


def attention_histograms(q: torch.Tensor, k: torch.Tensor, *, relative: bool, num_bins: int, sink_len: int,
                         out: torch.Tensor = None) -> torch.Tensor:
    """q [Hq,N,D], k [Hkv,N,D] (CUDA, 16-bit) -> fp64 [Hq, num_bins]; ``out`` accumulates over samples."""
    _require_cuda(q, k)
    hq, n, d = q.shape
    if out is None:
        out = torch.zeros(hq, num_bins, dtype=torch.float64, device=q.device)
    L.check(L.lib.sqattn_window_histogram(q.contiguous().data_ptr(), k.contiguous().data_ptr(), _dt(q.dtype), hq,
                                          k.shape[0], n, d, int(relative), num_bins, sink_len, out.data_ptr(), _stream()))
    return out


def find_optimal_relative_window(histogram: np.ndarray, threshold: float, num_bins: int = 100) -> float:
    """Smallest relative window keeping ``threshold`` of the energy; 0.1 when there is none (window_search.py:88-113)."""
    total = np.sum(histogram)
    if total == 0:
        return 0.1
    cum = np.cumsum(histogram)
    hit = np.nonzero(cum >= threshold * total)[0]
    best = int(hit[0]) if len(hit) else 0
    return min((best + 1) / num_bins, 1.0)


def find_optimal_window(histogram: np.ndarray, threshold: float) -> int:
    """Smallest absolute window in 128-token steps (window_search.py:116-128)."""
    total = np.sum(histogram)
    if total == 0:
        return 1
    cum = 0.0
    for d in range(0, len(histogram), 128):
        cum += float(np.sum(histogram[d:d + 128]))
        if cum >= threshold * total:
            return d + 128
    return len(histogram)


def calibrate_windows(samples: Sequence, args, max_len: int = 0):
    """calibrate_layer_windows (window_search.py:131-241) for one layer given its (q, k) samples
    (q [Hq,N,D], k [Hkv,N,D]): returns (bit8_max, bit4_max, windows) like the reference."""
    relative = bool(getattr(args, "use_relative_distance", False))
    num_bins = getattr(args, "relative_bins", 200) if relative else max_len
    sink_len = getattr(args, "sink_window_size", 256) if relative else 0
    hist = None
    for q, k in samples:
        hist = attention_histograms(q, k, relative=relative, num_bins=num_bins, sink_len=sink_len, out=hist)
    h = hist.cpu().numpy()
    windows: List[Dict] = []
    for head in range(h.shape[0]):
        if relative:
            windows.append({"head_idx": head,
                            "bit8_relative": find_optimal_relative_window(h[head], args.bit8_thres, num_bins),
                            "bit4_relative": find_optimal_relative_window(h[head], args.bit4_thres, num_bins),
                            "sink_len": sink_len})
        else:
            windows.append({"head_idx": head, "bit8": find_optimal_window(h[head], args.bit8_thres),
                            "bit4": find_optimal_window(h[head], args.bit4_thres)})
    k8, k4 = ("bit8_relative", "bit4_relative") if relative else ("bit8", "bit4")
    return max(w[k8] for w in windows), max(w[k4] for w in windows), windows


def bits_alloc_entry(windows: Sequence[Dict], relative: bool, sink: int = 256) -> Dict:
    """The per-layer dict process_model consumes: {"bit8": [...], "bit4": [...], "sink": 256} (compress.py:170-174)."""
    k8, k4 = ("bit8_relative", "bit4_relative") if relative else ("bit8", "bit4")
    return {"bit8": [w[k8] for w in windows], "bit4": [w[k4] for w in windows], "sink": sink}


def save_bits_alloc(path: str, bits_alloc: Dict[int, Dict]):
    with open(path, "w") as f:
        json.dump({str(k): v for k, v in bits_alloc.items()}, f, indent=1)


def load_bits_alloc(path: str) -> Dict[int, Dict]:
    with open(path) as f:
        return {int(k): v for k, v in json.load(f).items()}
