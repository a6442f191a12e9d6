"""Kernel launchers with the names, arguments and error behaviour of the reference's Python launchers:
attn_causal (sqattn/attn_triton.py:216-315), attn_hierarchical_relative_window
(sqattn/attn_triton_mix_relative.py:309-483), attn_hierarchical_window
(sqattn/attn_triton_mix_bad.py:285-426) and attn_unified (sqattn/attn_triton_decode.py:244-361).
They accept and return torch CUDA tensors; all arithmetic happens in libsqattn_b200.so."""
from __future__ import annotations

import torch
import torch.nn.functional as F

from .. import _lib as L
from .. import ops


def _pad_head_dim(ts):
    """head_dim < 64 -> 64, 64 < head_dim < 128 -> 128, > 128 rejected (attn_triton.py:236-244)."""
    d = ts[0].shape[-1]
    if d > 128:
        raise ValueError(f"Unsupported head_dim: {d}")
    tgt = 64 if d < 64 else (128 if 64 < d < 128 else d)
    if tgt == d:
        return list(ts), d
    return [F.pad(t, (0, tgt - d)) for t in ts], d


def _per_head(w, h, conv):
    if isinstance(w, (int, float)):
        return [conv(w)] * h
    if isinstance(w, torch.Tensor):
        w = w.detach().cpu().tolist()
    w = [conv(x) for x in w]
    if len(w) != h:
        raise ValueError(f"expected {h} per-head window entries, got {len(w)}")
    return w


def _slice_back(res, d_og):
    """o[..., :head_dim_og] (attn_triton.py:314); the LSE has no head_dim axis."""
    if isinstance(res, tuple):
        return (res[0] if res[0].shape[-1] == d_og else res[0][..., :d_og], res[1])
    return res if res.shape[-1] == d_og else res[..., :d_og]


def attn_hierarchical_relative_window(q_int8, k_int8, q_int4, k_int4, v, int8_window_ratios, int4_window_ratios,
                                      sink_size, tensor_layout="HND", output_dtype=torch.float16, return_lse=False,
                                      is_P_fp8_quant=False, p_fp8_mode=None, use_int4_operands=False):
    """Sink + hierarchical relative windows.  As in the reference launch (mix_relative.py:440-446) the int8
    tensors are read in both operand slots unless ``use_int4_operands`` is set."""
    if not isinstance(sink_size, int) or sink_size < 0:
        raise ValueError(f"sink_size must be a non-negative integer, got {sink_size}")
    (q_int8, k_int8, q_int4, k_int4, v), d_og = _pad_head_dim([q_int8, k_int8, q_int4, k_int4, v])
    h = q_int8.shape[1] if tensor_layout == "HND" else q_int8.shape[2]
    r8 = _per_head(int8_window_ratios, h, float)
    r4 = _per_head(int4_window_ratios, h, float)
    if not use_int4_operands:
        q_int4, k_int4 = q_int8, k_int8
    mode = L.P_FP8_ALL if is_P_fp8_quant else L.P_FP8_OFF
    if p_fp8_mode is not None:
        mode = {"off": L.P_FP8_OFF, "all": L.P_FP8_ALL, "stage2": L.P_FP8_STAGE2}[p_fp8_mode]
    # q is scaled inside the library (q_is_scaled=False), as the reference launchers do before the kernel call
    return _slice_back(ops.prefill(q_int8, k_int8, q_int4, k_int4, v, mode=L.MODE_RELATIVE_WINDOW, win8=r8, win4=r4,
                                   sink=sink_size, layout=tensor_layout, out_dtype=output_dtype, return_lse=return_lse,
                                   p_fp8_mode=mode, q_is_scaled=False, head_dim_og=d_og), d_og)


def attn_hierarchical_window(q_int8, k_int8, q_int4, k_int4, v, int8_window_sizes, int4_window_sizes, sink_size,
                             tensor_layout="HND", output_dtype=torch.float16, return_lse=False,
                             is_P_fp8_quant=False):
    """Sink + hierarchical absolute windows (BLOCK_M = 128, real int4 operands)."""
    if not isinstance(sink_size, int) or sink_size < 0:
        raise ValueError(f"sink_size must be a non-negative integer, got {sink_size}")
    (q_int8, k_int8, q_int4, k_int4, v), d_og = _pad_head_dim([q_int8, k_int8, q_int4, k_int4, v])
    h = q_int8.shape[1] if tensor_layout == "HND" else q_int8.shape[2]
    s8 = _per_head(int8_window_sizes, h, int)
    s4 = _per_head(int4_window_sizes, h, int)
    return _slice_back(ops.prefill(q_int8, k_int8, q_int4, k_int4, v, mode=L.MODE_ABSOLUTE_WINDOW, win8=s8, win4=s4,
                                   sink=sink_size, layout=tensor_layout, out_dtype=output_dtype, return_lse=return_lse,
                                   p_fp8_mode=L.P_FP8_ALL if is_P_fp8_quant else L.P_FP8_OFF, q_is_scaled=False,
                                   head_dim_og=d_og), d_og)


def attn_causal(q, k, v, tensor_layout="HND", output_dtype=torch.float16, return_lse=False, is_P_fp8_quant=False):
    """Dense causal GQA attention."""
    (q, k, v), d_og = _pad_head_dim([q, k, v])
    seq_dim = 1 if tensor_layout == "NHD" else 2
    assert q.shape[seq_dim] == k.shape[seq_dim], "qo_len and kv_len must be equal for causal attention"
    return _slice_back(ops.prefill(q, k, q, k, v, mode=L.MODE_DENSE_CAUSAL, layout=tensor_layout, out_dtype=output_dtype,
                                   return_lse=return_lse, p_fp8_mode=L.P_FP8_ALL if is_P_fp8_quant else L.P_FP8_OFF,
                                   q_is_scaled=False, head_dim_og=d_og), d_og)


def attn_unified(q, k, v, tensor_layout="HND", output_dtype=torch.float16, return_lse=False, is_P_fp8_quant=False,
                 center_k=True, kv_lens=None):
    """qo_len == 1 -> split-KV decode, otherwise dense causal prefill.  The reference subtracts the sequence
    mean from K on every call (attn_triton_decode.py:268-269); ``center_k=False`` skips that pass, which does
    not change a single-query softmax."""
    seq_dim = 1 if tensor_layout == "NHD" else 2
    if center_k:
        km = k.float().mean(dim=seq_dim, keepdim=True).to(k.dtype)
        k = k - km
    if q.shape[seq_dim] == 1:
        (qp, kp, vp), d_og = _pad_head_dim([q, k, v])
        return _slice_back(ops.decode(qp, kp, vp, layout=tensor_layout, out_dtype=output_dtype, return_lse=return_lse,
                                      p_fp8=is_P_fp8_quant, kv_lens=kv_lens, reference_tail=True, head_dim_og=d_og), d_og)
    return attn_causal(q, k, v, tensor_layout, output_dtype, return_lse, is_P_fp8_quant)
