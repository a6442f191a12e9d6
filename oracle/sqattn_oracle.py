"""CPU oracle for the SQAttn attention path (torch, CPU, fp32 arithmetic).

TEST INFRASTRUCTURE ONLY: the shipped package never imports this module.  It
restates, operation by operation, what the reference computes so that the CUDA
path can be checked against it.  Every function names the reference lines it
follows (paths are relative to the reference project root).

Pinning: the reference has no golden vectors of its own.  The tile kernels
below are pinned against outputs of the reference's unmodified ``@triton.jit``
kernels executed by Triton's CPU interpreter (fp16 inputs; the interpreter has
no bf16); see ``tests/golden/make_golden.py``.  The fake quantisers and the
adapter glue (repeat_kv, K centring, quantiser selection, the launchers'
padding / scaling / window tensors, the output transpose) are Paddle code; they
are pinned against outputs of that code itself, executed through a ``paddle``
module that forwards to torch (``tests/golden/paddle_torch_shim.py``): the
quantisers value for value in fp16 and bf16, ``attention_fn`` end to end.
What remains an ASSUMPTION, stated in that forwarder, are two Paddle
behaviours that cannot be observed without Paddle: ``paddle.round`` rounds
halves away from zero (a switch below selects ties-to-even), and
``bf16_tensor / fp32_tensor`` is evaluated in fp32.
"""
from __future__ import annotations

import math
from typing import Iterable, Optional, Sequence

import torch

LOG2E = 1.44269504  # literal used by the reference launchers
NEG_MASK = -1000000.0  # additive causal mask value used by the reference kernels
FP8_MAX = 448.0


# ----------------------------------------------------------------------------
# Fake quantisers  (sqattn/fake_quant.py)
# ----------------------------------------------------------------------------

def round_half_away(x: torch.Tensor) -> torch.Tensor:
    """Round to nearest, ties away from zero (the documented paddle.round)."""
    t = torch.trunc(x)
    d = x - t  # exact
    return t + torch.sign(x) * (d.abs() >= 0.5).to(x.dtype)


def _round(x: torch.Tensor, mode: str) -> torch.Tensor:
    if mode == "half_away":
        return round_half_away(x)
    if mode == "half_even":
        return torch.round(x)
    raise ValueError(f"unknown rounding mode {mode}")


def _minmax(xf: torch.Tensor, granularity: str):
    """fake_quant.py:23-38 (get_minmax_range): range in fp32."""
    if granularity == "per_tensor":
        return xf.min(), xf.max()
    if granularity == "per_channel":
        return xf.amin(dim=(0, 1), keepdim=True), xf.amax(dim=(0, 1), keepdim=True)
    return xf.amin(dim=-1, keepdim=True), xf.amax(dim=-1, keepdim=True)


def int_fake_quant(x: torch.Tensor, bits: int, granularity: str = "per_token",
                   symmetric: bool = True, round_mode: str = "half_away") -> torch.Tensor:
    """IntegerQuantizer.fake_quant_tensor (fake_quant.py:40-58, 80-86, 98-125).

    sym: absmax=max(|max|,|min|).clip(1e-5); scale=absmax/qmax;
    x_hat = clamp(round(x/scale), qmin, qmax)*scale, cast back to x.dtype.
    """
    org = x.dtype
    xf = x.float()
    mn, mx = _minmax(xf, granularity)
    if symmetric:
        qmin, qmax = -(2 ** (bits - 1)), 2 ** (bits - 1) - 1
        absmax = torch.maximum(mx.abs(), mn.abs()).clamp(min=1e-5)
        scale = absmax / qmax
        q = torch.clamp(_round(xf / scale, round_mode), qmin, qmax)
        out = q * scale
    else:
        qmin, qmax = 0.0, float(2 ** bits - 1)
        scale = (mx - mn).clamp(min=1e-5) / (qmax - qmin)
        zeros = torch.clamp(qmin - _round(mn / scale, round_mode), qmin, qmax)
        q = torch.clamp(_round(xf / scale, round_mode) + zeros, qmin, qmax)
        out = (q - zeros) * scale
    return out.to(org)


def float_quantize(x: torch.Tensor, e_bits: int, m_bits: int, round_mode: str = "half_away") -> torch.Tensor:
    """float_quantize (fake_quant.py:151-204), rounding="nearest", quirks kept:
    no subnormals, mantissa never carries into the next binade, and the
    exponent is clipped to 2**(e_bits-1)-1 (so e4m3 tops out at 240)."""
    bias = 2 ** (e_bits - 1) - 1
    eps = 2.0 ** (-m_bits)
    max_exp = 2 ** (e_bits - 1) - 1
    min_exp = 1 - bias
    sign = torch.sign(x)
    x = torch.abs(x)
    zero_mask = x == 0
    exp = torch.floor(torch.log2(x + 1e-30))
    frac = x / torch.exp2(exp) - 1.0
    exp_c = torch.clamp(exp, min_exp, max_exp)
    frac_q = _round(frac / eps, round_mode) * eps
    frac_q = torch.clamp(frac_q, 0.0, 1.0 - eps)
    x_q = (1.0 + frac_q) * torch.exp2(exp_c) * sign
    max_val = (2 - 2 ** (-m_bits)) * (2.0 ** max_exp)
    x_q = torch.clamp(x_q, -max_val, max_val)
    return torch.where(zero_mask, torch.zeros_like(x_q), x_q)


def float_fake_quant(x: torch.Tensor, kind: str, granularity: str = "per_token",
                     round_mode: str = "half_away") -> torch.Tensor:
    """FloatQuantizer.fake_quant_tensor (fake_quant.py:207-248): scale the
    range to +-448 (e4m3) / +-57344 (e5m2), clamp, float_quantize, rescale."""
    if kind == "e4m3":
        e_bits, m_bits, fmax = 4, 3, 448.0
    elif kind == "e5m2":
        e_bits, m_bits, fmax = 5, 2, 57344.0
    else:
        raise ValueError(f"Unsupported bit configuration: {kind}")
    org = x.dtype
    xf = x.float()
    mn, mx = _minmax(xf, granularity)
    absmax = torch.maximum(mx.abs(), mn.abs()).clamp(min=1e-5)
    scale = absmax / fmax
    scaled = torch.clamp(xf / scale, -fmax, fmax)
    q = float_quantize(scaled, e_bits, m_bits, round_mode)
    return (q * scale).to(org)


def make_quantizers(qk_qtype: str, v_qtype: str):
    """Quantiser selection of the adapter (attn_replacer.py:340-358)."""
    if qk_qtype == "int":
        q8 = lambda t, rm: int_fake_quant(t, 8, "per_token", True, rm)
    elif qk_qtype in ("e4m3", "e5m2"):
        q8 = lambda t, rm: float_fake_quant(t, qk_qtype, "per_token", rm)
    else:
        raise ValueError(f"Invalid quantization type: {qk_qtype}")
    q4 = lambda t, rm: int_fake_quant(t, 4, "per_token", True, rm)
    if v_qtype == "int":
        v8 = lambda t, rm: int_fake_quant(t, 8, "per_channel", True, rm)
    elif v_qtype in ("e4m3", "e5m2"):
        v8 = lambda t, rm: float_fake_quant(t, v_qtype, "per_channel", rm)
    else:
        raise ValueError(f"Invalid quantization type: {v_qtype}")
    return q8, q4, v8


# ----------------------------------------------------------------------------
# Adapter input preparation  (sqattn/attn_replacer.py:281-293, 334-366)
# ----------------------------------------------------------------------------

def repeat_kv(x: torch.Tensor, n_rep: int) -> torch.Tensor:
    """[B,N,Hkv,D] -> [B,Hkv*n_rep,N,D] (attn_replacer.py:281-293)."""
    b, n, hkv, d = x.shape
    x = x.permute(0, 2, 1, 3)
    if n_rep == 1:
        return x
    return x[:, :, None].expand(b, hkv, n_rep, n, d).reshape(b, hkv * n_rep, n, d)


def center_keys(key_hnd: torch.Tensor) -> torch.Tensor:
    """key - key.mean(dim=2, keepdim=True), both in key's dtype
    (attn_replacer.py:338-339).  The mean is accumulated in fp32 then rounded."""
    km = key_hnd.float().mean(dim=2, keepdim=True).to(key_hnd.dtype)
    return key_hnd - km


def prep_qkv(query, key, value, num_kv_groups: int, qk_qtype: str = "int", v_qtype: str = "int",
             round_mode: str = "half_away"):
    """Everything the adapter does before the kernel call
    (attn_replacer.py:334-365).  Inputs NHD, outputs HND with K/V GQA-expanded:
    returns (q_bit8, q_bit4, k_bit8, k_bit4, v_bit8)."""
    k = repeat_kv(key, num_kv_groups)
    v = repeat_kv(value, num_kv_groups)
    q = query.permute(0, 2, 1, 3)
    k = center_keys(k)
    f8, f4, fv = make_quantizers(qk_qtype, v_qtype)
    return f8(q, round_mode), f4(q, round_mode), f8(k, round_mode), f4(k, round_mode), fv(v, round_mode)


# ----------------------------------------------------------------------------
# Tile kernels
# ----------------------------------------------------------------------------

def scale_q(q: torch.Tensor, head_dim_og: int) -> torch.Tensor:
    """q * (1/sqrt(D) * 1.44269504) evaluated in q's dtype
    (attn_triton_mix_relative.py:383-385, attn_triton.py:249-253)."""
    sm_scale = 1.0 / head_dim_og ** 0.5 * LOG2E
    return (q.float() * torch.tensor(sm_scale, dtype=torch.float32)).to(q.dtype)


def p_fp8_round(p: torch.Tensor) -> torch.Tensor:
    """(p*448).to(float8e4nv).to(fp16)/448 in fp16 (attn_triton.py:81-83);
    the input is fp32 in [0,1], the result is returned as fp16."""
    p8 = (p * FP8_MAX).to(torch.float8_e4m3fn).to(torch.float16)
    # fp16 / fp16 correctly rounded: evaluate in fp32 and round once (24 >= 2*11+2 bits).
    return (p8.float() / FP8_MAX).to(torch.float16)


def relative_window_size(ratio, kv_len: int) -> int:
    """((int64)(ratio_f32 * kv_len) + 127)//128*128
    (attn_triton_mix_relative.py:43-46)."""
    prod = torch.tensor(float(ratio), dtype=torch.float32) * torch.tensor(float(kv_len), dtype=torch.float32)
    raw = int(prod.to(torch.int64).item())
    return (raw + 127) // 128 * 128


def stage_ranges(query_start: int, query_end: int, w8: int, w4: int, sink: int):
    """Key ranges [lo,hi) of the four stages for one query block
    (attn_triton_mix_relative.py:36-75, attn_triton_mix_bad.py:41-74).
    Returns a list of (stage, lo, hi); empty stages have lo == hi == 0."""
    out = [(1, 0, min(sink, query_start))]
    l4 = max(sink, query_end - w4)
    l8 = max(sink, query_end - w8)
    out.append((2, l4, l8) if l4 < l8 else (2, 0, 0))
    out.append((3, l8, query_start) if l8 < query_start else (3, 0, 0))
    out.append((4, query_start, query_end))
    return out


def _load_rows(x: torch.Tensor, start: int, count: int, limit: int) -> torch.Tensor:
    """x[..., start:start+count, :] with rows >= limit read as zero (masked loads)."""
    end = min(start + count, limit)
    part = x[..., start:end, :] if end > start else x[..., 0:0, :]
    if part.shape[-2] == count:
        return part
    pad = torch.zeros(*x.shape[:-2], count - part.shape[-2], x.shape[-1], dtype=x.dtype)
    return torch.cat([part, pad], dim=-2)


def _tile_step(state, q, k_t, v_t, row_idx, col_start, block_n, masked, fp8):
    """One iteration of the reference tile loop
    (attn_triton_mix_relative.py:76-98 == attn_triton.py:64-86).
    q [H,BM,D], k_t/v_t [H,BN,D]; state = (acc, l, m)."""
    acc, l_i, m_i = state
    qk = torch.matmul(q.float(), k_t.float().transpose(-1, -2))
    if masked:
        cols = col_start + torch.arange(block_n)
        causal = row_idx[:, None] >= cols[None, :]
        qk = qk + torch.where(causal, torch.tensor(0.0), torch.tensor(NEG_MASK))
    m_ij = torch.maximum(m_i, qk.max(dim=-1).values)
    p = torch.exp2(qk - m_ij[..., None])
    l_ij = p.sum(dim=-1)
    alpha = torch.exp2(m_i - m_ij)
    l_i = l_i * alpha + l_ij
    acc = acc * alpha[..., None]
    p16 = p_fp8_round(p) if fp8 else p.to(torch.float16)
    acc = acc + torch.matmul(p16.float(), v_t.to(torch.float16).float())
    return acc, l_i, m_ij


def _as_hnd(x: torch.Tensor, layout: str) -> torch.Tensor:
    if layout == "HND":
        return x
    if layout == "NHD":
        return x.permute(0, 2, 1, 3)
    raise ValueError(f"tensor_layout {layout} not supported")


def _pad_head_dim(ts: Sequence[torch.Tensor]):
    """head_dim < 64 -> 64, 64 < head_dim < 128 -> 128, > 128 rejected
    (attn_triton.py:236-244)."""
    d = ts[0].shape[-1]
    if d > 128:
        raise ValueError(f"Unsupported head_dim: {d}")
    tgt = 64 if d < 64 else (128 if 64 < d < 128 else d)
    if tgt == d:
        return list(ts), d
    return [torch.nn.functional.pad(t, (0, tgt - d)) for t in ts], d


def windowed_prefill(q_int8, k_int8, q_int4, k_int4, v, win8, win4, sink_size: int, *,
                     mode: str = "relative", tensor_layout: str = "HND",
                     output_dtype=torch.float16, return_lse: bool = False,
                     is_P_fp8_quant: bool = False, p_fp8_mode: Optional[str] = None,
                     use_int4_operands: Optional[bool] = None,
                     block_n: int = 64, blocks: Optional[Iterable[int]] = None, q_is_scaled: bool = False):
    """Sink + hierarchical-window causal attention.

    mode="relative": attn_hierarchical_relative_window
      (attn_triton_mix_relative.py:309-483): BLOCK_M=64, per-head fp32 ratios,
      windows rounded up to 128; as shipped the launch passes the int8 tensors
      in the int4 slots (440-446) -> use_int4_operands defaults to False.
    mode="absolute": attn_hierarchical_window (attn_triton_mix_bad.py:285-426):
      BLOCK_M=128, per-head int32 window sizes, real int4 operands.

    p_fp8_mode: "off", "all" (the reference's is_P_fp8_quant=True) or
      "stage2" (FP8 P only for the int4-window tiles).  ``blocks`` restricts
      the computation to those query-block indices (other rows are returned 0).
    Returns o [B,H,N,D] in ``tensor_layout`` (and lse [B,H,N] fp32).
    """
    if not isinstance(sink_size, int) or sink_size < 0:
        raise ValueError(f"sink_size must be a non-negative integer, got {sink_size}")
    if p_fp8_mode is None:
        p_fp8_mode = "all" if is_P_fp8_quant else "off"
    if mode == "relative":
        block_m = 64
        if use_int4_operands is None:
            use_int4_operands = False
    elif mode == "absolute":
        block_m = 128
        if use_int4_operands is None:
            use_int4_operands = True
    else:
        raise ValueError(mode)
    (q_int8, k_int8, q_int4, k_int4, v), d_og = _pad_head_dim([q_int8, k_int8, q_int4, k_int4, v])
    q8, q4 = _as_hnd(q_int8, tensor_layout), _as_hnd(q_int4, tensor_layout)
    if not q_is_scaled:
        q8, q4 = scale_q(q8, d_og), scale_q(q4, d_og)
    k8 = _as_hnd(k_int8, tensor_layout)
    k4 = _as_hnd(k_int4, tensor_layout)
    vv = _as_hnd(v, tensor_layout)
    if not use_int4_operands:
        q4, k4 = q8, k8
    b, h, n, d = q8.shape
    hkv, kv_len = k8.shape[1], k8.shape[2]
    groups = h // hkv

    def per_head(w):
        if isinstance(w, (int, float)):
            return [w] * h
        return [float(x) if mode == "relative" else int(x) for x in (w.tolist() if hasattr(w, "tolist") else w)]

    w8s, w4s = per_head(win8), per_head(win4)
    if mode == "relative":
        w8s = [relative_window_size(r, kv_len) for r in w8s]
        w4s = [relative_window_size(r, kv_len) for r in w4s]
    o = torch.zeros(b, h, n, d, dtype=output_dtype)   # rounded block by block: the same values as rounding at the end
    lse = torch.zeros(b, h, n, dtype=torch.float32)
    nblk = (n + block_m - 1) // block_m
    blk_list = list(range(nblk)) if blocks is None else list(blocks)
    # heads with identical windows share a schedule and are processed together
    sched = {}
    for hh in range(h):
        sched.setdefault((w8s[hh], w4s[hh]), []).append(hh)
    for (w8, w4), heads in sched.items():
        hq = torch.tensor(heads)
        hk = hq // groups
        for blk in blk_list:
            qs, qe = blk * block_m, (blk + 1) * block_m
            rows = torch.arange(qs, qe)
            q8b = _load_rows(q8, qs, block_m, n)[:, hq]
            q4b = _load_rows(q4, qs, block_m, n)[:, hq]
            acc = torch.zeros(b, len(heads), block_m, d)
            l_i = torch.ones(b, len(heads), block_m)
            m_i = torch.full((b, len(heads), block_m), float("-inf"))
            for stage, lo, hi in stage_ranges(qs, qe, w8, w4, sink_size):
                qb, kk = (q4b, k4) if stage == 2 else (q8b, k8)
                fp8 = p_fp8_mode == "all" or (p_fp8_mode == "stage2" and stage == 2)
                for start_n in range(lo, hi, block_n):
                    k_t = _load_rows(kk, start_n, block_n, kv_len)[:, hk]
                    v_t = _load_rows(vv, start_n, block_n, kv_len)[:, hk]
                    acc, l_i, m_i = _tile_step((acc, l_i, m_i), qb, k_t, v_t, rows, start_n,
                                               block_n, stage == 4, fp8)
            valid = min(qe, n) - qs
            o[:, hq, qs:qs + valid] = (acc / l_i[..., None])[:, :, :valid].to(output_dtype)
            lse[:, hq, qs:qs + valid] = (torch.log2(l_i) + m_i)[:, :, :valid]
    o = o[..., :d_og]
    if tensor_layout == "NHD":
        o = o.permute(0, 2, 1, 3)
    return (o, lse) if return_lse else o


def dense_causal(q, k, v, *, tensor_layout: str = "HND", output_dtype=torch.float16,
                 return_lse: bool = False, is_P_fp8_quant: bool = False, center_k: bool = False,
                 block_m: int = 128, block_n: int = 64, blocks: Optional[Iterable[int]] = None):
    """attn_causal (attn_triton.py:10-87, 90-213, 216-315): BLOCK_M=128,
    BLOCK_N=64, stage 1 = keys [0, 128*start_m), stage 2 = the diagonal block.
    ``center_k`` applies the K-mean subtraction that attn_unified does first
    (attn_triton_decode.py:268-269)."""
    (q, k, v), d_og = _pad_head_dim([q, k, v])
    qh, kh, vh = _as_hnd(q, tensor_layout), _as_hnd(k, tensor_layout), _as_hnd(v, tensor_layout)
    if center_k:
        kh = center_keys(kh)
    qh = scale_q(qh, d_og)
    b, h, n, d = qh.shape
    hkv, kv_len = kh.shape[1], kh.shape[2]
    assert n == kv_len, "qo_len and kv_len must be equal for causal attention"
    groups = h // hkv
    hk = torch.arange(h) // groups
    o = torch.zeros(b, h, n, d)
    lse = torch.zeros(b, h, n)
    nblk = (n + block_m - 1) // block_m
    for blk in (range(nblk) if blocks is None else blocks):
        qs, qe = blk * block_m, (blk + 1) * block_m
        rows = torch.arange(qs, qe)
        qb = _load_rows(qh, qs, block_m, n)
        acc = torch.zeros(b, h, block_m, d)
        l_i = torch.ones(b, h, block_m)
        m_i = torch.full((b, h, block_m), float("-inf"))
        for masked, lo, hi in ((False, 0, qs), (True, qs, qe)):
            for start_n in range(lo, hi, block_n):
                k_t = _load_rows(kh, start_n, block_n, kv_len)[:, hk]
                v_t = _load_rows(vh, start_n, block_n, kv_len)[:, hk]
                acc, l_i, m_i = _tile_step((acc, l_i, m_i), qb, k_t, v_t, rows, start_n, block_n,
                                           masked, is_P_fp8_quant)
        valid = min(qe, n) - qs
        o[:, :, qs:qs + valid] = (acc / l_i[..., None])[:, :, :valid]
        lse[:, :, qs:qs + valid] = (torch.log2(l_i) + m_i)[:, :, :valid]
    o = o.to(output_dtype)[..., :d_og]
    if tensor_layout == "NHD":
        o = o.permute(0, 2, 1, 3)
    return (o, lse) if return_lse else o


def decode(q, k, v, *, tensor_layout: str = "HND", output_dtype=torch.float16, return_lse: bool = False,
           is_P_fp8_quant: bool = False, center_k: bool = True, block_n: int = 64,
           kv_lens: Optional[Sequence[int]] = None, qk_in_input_dtype: bool = False,
           mask_tail: bool = False):
    """Single-query attention, attn_unified decode branch + _attn_decode_fwd
    (attn_triton_decode.py:175-241, 244-361): K re-centred over the sequence
    (268-269), q scaled in its dtype (270-271), 64-key online softmax with
    l initialised to 0, P optionally FP8-rounded, P*V in fp32 (234).
    ``kv_lens`` (one per batch row) extends it to ragged batches: rows at or
    beyond a sequence's length are masked like the kernel's kv_len mask.
    ``qk_in_input_dtype`` rounds each q*k product to the input dtype as the
    Triton elementwise multiply does (221); accumulation stays fp32.
    The reference loads keys past kv_len as zeros and does not mask their
    scores (215-221): the last tile is padded with keys of score 0 and value
    0, which this function reproduces; ``mask_tail=True`` masks them instead
    (exact softmax over the real keys, an option the CUDA path also has)."""
    (q, k, v), d_og = _pad_head_dim([q, k, v])
    qh, kh, vh = _as_hnd(q, tensor_layout), _as_hnd(k, tensor_layout), _as_hnd(v, tensor_layout)
    b, h, one, d = qh.shape
    assert one == 1
    hkv, kv_max = kh.shape[1], kh.shape[2]
    lens = [kv_max] * b if kv_lens is None else list(kv_lens)
    groups = h // hkv
    qh = scale_q(qh, d_og)
    o = torch.zeros(b, h, 1, d)
    lse = torch.zeros(b, h, 1)
    for bi in range(b):
        L = lens[bi]
        kb = kh[bi:bi + 1, :, :L]
        if center_k:
            kb = center_keys(kb)
        kb = kb[0]
        vb = vh[bi, :, :L]
        hk = torch.arange(h) // groups
        qv = qh[bi, :, 0]  # [H, D]
        m_i = torch.full((h,), float("-inf"))
        l_i = torch.zeros(h)
        acc = torch.zeros(h, d)
        for start_n in range(0, L, block_n):
            k_t = _load_rows(kb[hk], start_n, block_n, L)  # [H,BN,D]
            v_t = _load_rows(vb[hk], start_n, block_n, L)
            if qk_in_input_dtype:
                prod = (qv[:, None, :].float() * k_t.float()).to(qv.dtype).float()
                qk = prod.sum(-1)
            else:
                qk = torch.einsum("hd,hnd->hn", qv.float(), k_t.float())
            if mask_tail and start_n + block_n > L:
                qk[:, L - start_n:] = float("-inf")
            m_ij = torch.maximum(m_i, qk.max(dim=-1).values)
            p = torch.exp2(qk - m_ij[:, None])
            l_ij = p.sum(-1)
            alpha = torch.exp2(m_i - m_ij)
            l_i = l_i * alpha + l_ij
            acc = acc * alpha[:, None]
            if is_P_fp8_quant:
                p = p_fp8_round(p).float()
            acc = acc + torch.einsum("hn,hnd->hd", p, v_t.float())
            m_i = m_ij
        o[bi, :, 0] = acc / l_i[:, None]
        lse[bi, :, 0] = torch.log2(l_i) + m_i
    o = o.to(output_dtype)[..., :d_og]
    if tensor_layout == "NHD":
        o = o.permute(0, 2, 1, 3)
    return (o, lse) if return_lse else o


def merge_partials(o_parts: torch.Tensor, lse_parts: torch.Tensor):
    """Combine split-KV partial results (base-2 LSE, attn_triton.py:210-213):
    o_parts [S, ..., D] each already divided by its own l, lse_parts [S, ...].
    O = sum_i 2^(lse_i - lse_max) O_i / sum_i 2^(lse_i - lse_max)."""
    mx = lse_parts.max(dim=0).values
    w = torch.exp2(lse_parts - mx)
    den = w.sum(0)
    o = (w[..., None] * o_parts).sum(0) / den[..., None]
    return o, torch.log2(den) + mx


# ----------------------------------------------------------------------------
# The operator as installed on a layer  (attn_replacer.py:296-454)
# ----------------------------------------------------------------------------

def attention_fn(query, key, value, num_kv_groups: int, bit8_window_sizes, bit4_window_sizes,
                 sink_window_size: int, *, use_relative_distance: bool = True, qk_qtype: str = "int",
                 v_qtype: str = "int", p_fp8_mode: str = "off", round_mode: str = "half_away",
                 blocks: Optional[Iterable[int]] = None, output_dtype=torch.bfloat16) -> torch.Tensor:
    """mp_triton_wrapper.attention_fn for seq_len > 1: prep -> windowed kernel
    with output_dtype bf16 -> [B, N, Hq*D] (attn_replacer.py:334-365, 423-452)."""
    q8, q4, k8, k4, v8 = prep_qkv(query, key, value, num_kv_groups, qk_qtype, v_qtype, round_mode)
    o = windowed_prefill(q8, k8, q4, k4, v8, bit8_window_sizes, bit4_window_sizes, sink_window_size,
                         mode="relative" if use_relative_distance else "absolute",
                         tensor_layout="HND", output_dtype=output_dtype, p_fp8_mode=p_fp8_mode,
                         blocks=blocks)
    b, h, n, d = o.shape
    return o.transpose(1, 2).contiguous().view(b, n, h * d)


def sdpa_reference(q, k, v, *, tensor_layout: str = "HND", is_causal: bool = True, center_k: bool = True):
    """Plain softmax attention in fp32 with K-mean centring, the comparator the
    reference benches against (attn_triton.py:324-387)."""
    qh, kh, vh = (_as_hnd(t, tensor_layout).float() for t in (q, k, v))
    if center_k:
        kh = kh - kh.mean(dim=2, keepdim=True)
    groups = qh.shape[1] // kh.shape[1]
    kh = kh.repeat_interleave(groups, dim=1)
    vh = vh.repeat_interleave(groups, dim=1)
    s = torch.matmul(qh, kh.transpose(-1, -2)) / math.sqrt(qh.shape[-1])
    if is_causal:
        n, m = s.shape[-2:]
        mask = torch.ones(n, m, dtype=torch.bool).tril(diagonal=m - n)
        s = s.masked_fill(~mask, float("-inf"))
    o = torch.matmul(torch.softmax(s, dim=-1), vh)
    if tensor_layout == "NHD":
        o = o.permute(0, 2, 1, 3)
    return o


def visited_mask(n: int, w8: int, w4: int, sink: int, block_m: int, block_n: int = 64) -> torch.Tensor:
    """Boolean [n, n] map of the (query, key) pairs the windowed kernel visits
    with weight > 0 (stage 4 pairs above the diagonal excluded)."""
    mask = torch.zeros(n, n, dtype=torch.bool)
    for qs in range(0, n, block_m):
        qe = qs + block_m
        for stage, lo, hi in stage_ranges(qs, qe, w8, w4, sink):
            for start_n in range(lo, hi, block_n):
                c0, c1 = start_n, min(start_n + block_n, n)
                if c1 <= c0:
                    continue
                blk = torch.ones(min(qe, n) - qs, c1 - c0, dtype=torch.bool)
                if stage == 4:
                    rows = torch.arange(qs, min(qe, n))[:, None]
                    blk = rows >= torch.arange(c0, c1)[None, :]
                mask[qs:min(qe, n), c0:c1] |= blk
    return mask


def make_inputs(seed: int, batch: int, n: int, hq: int, hkv: int, d: int, dtype=torch.bfloat16,
                outlier_channels: int = 4, outlier_scale: float = 8.0):
    """Seeded synthetic Q,K,V (NHD) ~ N(0,1) with a few K channels scaled up,
    the input distribution the benchmark configurations describe."""
    g = torch.Generator().manual_seed(seed)
    q = torch.randn(batch, n, hq, d, generator=g)
    k = torch.randn(batch, n, hkv, d, generator=g)
    v = torch.randn(batch, n, hkv, d, generator=g)
    ch = torch.randperm(d, generator=g)[:outlier_channels]
    k[..., ch] *= outlier_scale
    return q.to(dtype), k.to(dtype), v.to(dtype)
