"""Tensor-level wrappers over the C ABI: they only translate torch tensors
(device memory, strides, the current stream) into the plain structs of
include/sqattn_b200.h.  No arithmetic happens on the Python side."""
from __future__ import annotations

import ctypes as C
from typing import Optional, Sequence

import torch

from . import _lib as L


def _dt(dtype: torch.dtype) -> int:
    if dtype == torch.float16:
        return L.F16
    if dtype == torch.bfloat16:
        return L.BF16
    raise ValueError(f"unsupported dtype {dtype}: float16 or bfloat16 expected")


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def _require_cuda(*ts):
    for t in ts:
        if t is not None and not t.is_cuda:
            raise RuntimeError("sqattn_b200 runs on CUDA tensors only (there is no CPU path)")


def _view(t: torch.Tensor, layout: str) -> L.Tensor:
    """Logical [B,H,N,D] view of a 4-D tensor stored HND or NHD."""
    assert t.dim() == 4 and t.stride(-1) == 1, "Last dim of qkv must be contiguous."
    if layout == "HND":
        return L.Tensor(t.data_ptr(), t.stride(0), t.stride(1), t.stride(2))
    if layout == "NHD":
        return L.Tensor(t.data_ptr(), t.stride(0), t.stride(2), t.stride(1))
    raise ValueError(f"tensor_layout {layout} not supported")


def _shape(t: torch.Tensor, layout: str):
    b, x, y, d = t.shape
    return (b, x, y, d) if layout == "HND" else (b, y, x, d)


_MIRRORS = {}


def poll_device_status(device=None):
    """Cheap, non-synchronising look at the failure word of ``device``: a pinned host int32 that a kernel whose bounded
    wait gave up also writes to (sqattn_set_status_mirror).  Raises SqattnError(ERR_DEVICE_TIMEOUT) once a failure has
    become visible; every operator below calls it on entry, so a caller of the drop-in operator hears about a timed-out
    wait at its next call at the latest (and meanwhile gets NaN, never stale memory).  The device-side word stays set,
    and later launches keep returning NaN, until ``check_device_status`` has cleared it."""
    idx = torch.cuda.current_device() if device is None or device.index is None else device.index
    ent = _MIRRORS.get(idx)
    if ent is None:
        if torch.cuda.is_current_stream_capturing():
            return
        word = torch.zeros(1, dtype=torch.int32).pin_memory()
        with torch.cuda.device(idx):
            L.check(L.lib.sqattn_set_status_mirror(word.data_ptr()))
        ent = _MIRRORS[idx] = (word, C.c_int32.from_address(word.data_ptr()))
    code = ent[1].value
    if code:
        raise L.SqattnError(L.ERR_DEVICE_TIMEOUT, f"a device-side wait gave up on cuda:{idx} (code {code}: 1xx prefill, "
                            "2xx decode, 3xx peer exchange); outputs since then are NaN; call check_device_status() to clear")


def _workspace(nbytes: int, device) -> Optional[torch.Tensor]:
    if nbytes == 0:
        return None
    ws = torch.empty(nbytes + 1024, dtype=torch.uint8, device=device)
    off = (-ws.data_ptr()) % 1024
    return ws[off:off + nbytes]


def prefill(q8, k8, q4, k4, v, *, mode: int, win8=None, win4=None, sink: int = 0, layout: str = "HND",
            out_dtype=torch.float16, return_lse: bool = False, p_fp8_mode: int = 0, q_is_scaled: bool = False,
            out: Optional[torch.Tensor] = None, out_layout: Optional[str] = None, kv_layout: Optional[str] = None,
            q_row_offset: int = 0, head_dim_og: int = 0, q_split_rows: int = 0, q_row_offset2: int = 0,
            q_fake_quant: Optional[str] = None, round_half_even: bool = False):
    """sqattn_prefill.  win8/win4: per-head sequences (floats for the relative mode, ints for the absolute).
    kv_layout: layout of k/v when it differs from q's; q_row_offset: first row of a query shard; head_dim_og: the
    head_dim before the caller zero-padded the tensors to 64 / 128 (the softmax scale follows it).  q_fake_quant
    ("int" / "e4m3" / "e5m2"): q8 is the raw query and the kernel fake-quantises and scales it tile by tile."""
    _require_cuda(q8, k8, q4, k4, v)
    poll_device_status(q8.device)
    b, hq, n, d = _shape(q8, layout)
    kv_layout = kv_layout or layout
    _, hkv, kv_len, _ = _shape(k8, kv_layout)
    if out is None:
        out = torch.empty(q8.shape, dtype=out_dtype, device=q8.device)
        out_layout = layout
    lse = torch.empty(b, hq, n, dtype=torch.float32, device=q8.device) if return_lse else None
    a = L.PrefillArgs()
    a.q_int8, a.k_int8 = _view(q8, layout), _view(k8, kv_layout)
    a.q_int4, a.k_int4 = _view(q4, layout), _view(k4, kv_layout)
    a.v, a.o = _view(v, kv_layout), _view(out, out_layout)
    a.q_row_offset, a.head_dim_og = int(q_row_offset), int(head_dim_og)
    a.q_split_rows, a.q_row_offset2 = int(q_split_rows), int(q_row_offset2)   # second row range of a shard, if any
    if q_fake_quant is not None:
        if q_fake_quant not in L.QTYPE:
            raise ValueError(f"Invalid quantization type: {q_fake_quant}")
        a.q_fake_quant, a.q_round_half_even = L.QTYPE[q_fake_quant] + 1, int(round_half_even)
    a.lse = lse.data_ptr() if lse is not None else None
    a.batch, a.num_q_heads, a.num_kv_heads, a.qo_len, a.kv_len, a.head_dim = b, hq, hkv, n, kv_len, d
    a.qk_dtype, a.v_dtype, a.o_dtype = _dt(q8.dtype), _dt(v.dtype), _dt(out.dtype)
    a.mode, a.sink_size, a.p_fp8_mode, a.q_is_scaled = mode, int(sink), int(p_fp8_mode), int(q_is_scaled)
    keep = []
    if mode == L.MODE_RELATIVE_WINDOW:
        r8 = (C.c_float * hq)(*[float(x) for x in win8])
        r4 = (C.c_float * hq)(*[float(x) for x in win4])
        a.win8_ratios, a.win4_ratios = r8, r4
        keep += [r8, r4]
    elif mode == L.MODE_ABSOLUTE_WINDOW:
        s8 = (C.c_int32 * hq)(*[int(x) for x in win8])
        s4 = (C.c_int32 * hq)(*[int(x) for x in win4])
        a.win8_sizes, a.win4_sizes = s8, s4
        keep += [s8, s4]
    need = L.lib.sqattn_prefill_workspace_bytes(C.byref(a))
    ws = _workspace(need, q8.device)
    a.workspace, a.workspace_bytes = (ws.data_ptr() if ws is not None else None), need
    L.check(L.lib.sqattn_prefill(C.byref(a), _stream()))
    return (out, lse) if return_lse else out


def prep_qkv(query, key, value, *, qk_qtype: str = "int", v_qtype: str = "int", round_half_even: bool = False,
             skip_bit4: bool = False, k_mean: Optional[torch.Tensor] = None, kv_out_nhd: bool = False,
             out: Optional[dict] = None):
    """sqattn_prep_qkv: NHD inputs -> (q_bit8, q_bit4, k_bit8, k_bit4, v_bit8) contiguous HND; q pre-scaled,
    K/V with their own Hkv heads, v_bit8 in fp16.  k_mean [B,Hkv,D] fp32 overrides the sequence mean of K;
    kv_out_nhd writes the K/V outputs token-major [B,N,Hkv,D].  Any of query/key/value may be None: only the
    tensors given are prepared (their outputs are returned, the others are None).  ``out`` may hold
    preallocated outputs under the keys q8, q4, k8, k4, v8."""
    given = [t for t in (query, key, value) if t is not None]
    _require_cuda(*given)
    if qk_qtype not in L.QTYPE:
        raise ValueError(f"Invalid quantization type: {qk_qtype}")
    if v_qtype not in L.QTYPE:
        raise ValueError(f"Invalid quantization type: {v_qtype}")
    ref = given[0]
    b, n, _, d = ref.shape
    dev, dt = ref.device, ref.dtype
    out = out or {}
    a = L.PrepArgs()
    q8 = q4 = k8 = k4 = v8 = None
    hq = hkv = 1
    if query is not None:
        hq = query.shape[2]
        q8 = out.get("q8") if out.get("q8") is not None else torch.empty(b, hq, n, d, dtype=dt, device=dev)
        q4 = None if skip_bit4 else (out.get("q4") if out.get("q4") is not None else torch.empty_like(q8))
        a.q, a.q_bit8, a.q_bit4 = _view(query, "NHD"), q8.data_ptr(), (None if q4 is None else q4.data_ptr())
        a.parts |= 1
    if key is not None or value is not None:
        hkv = (key if key is not None else value).shape[2]
    kv_shape = (b, n, hkv, d) if kv_out_nhd else (b, hkv, n, d)
    if key is not None:
        k8 = out.get("k8") if out.get("k8") is not None else torch.empty(kv_shape, dtype=dt, device=dev)
        k4 = None if skip_bit4 else (out.get("k4") if out.get("k4") is not None else torch.empty_like(k8))
        a.k, a.k_bit8, a.k_bit4 = _view(key, "NHD"), k8.data_ptr(), (None if k4 is None else k4.data_ptr())
        a.parts |= 2
    if value is not None:
        v8 = out.get("v8") if out.get("v8") is not None else torch.empty(kv_shape, dtype=torch.float16, device=dev)
        a.v, a.v_bit8 = _view(value, "NHD"), v8.data_ptr()
        a.parts |= 4
    a.batch, a.num_q_heads, a.num_kv_heads, a.seq_len, a.head_dim = b, hq, hkv, n, d
    a.dtype, a.qk_qtype, a.v_qtype = _dt(dt), L.QTYPE[qk_qtype], L.QTYPE[v_qtype]
    a.round_half_even, a.skip_bit4 = int(round_half_even), int(skip_bit4)
    a.kv_out_nhd = int(kv_out_nhd)
    if k_mean is not None:
        assert k_mean.dtype == torch.float32 and k_mean.is_contiguous() and k_mean.shape == (b, hkv, d)
        a.k_mean = k_mean.data_ptr()
    need = L.lib.sqattn_prep_workspace_bytes(C.byref(a))
    ws = _workspace(need, dev)
    a.workspace, a.workspace_bytes = ws.data_ptr(), need
    L.check(L.lib.sqattn_prep_qkv(C.byref(a), _stream()))
    return q8, q4, k8, k4, v8


def k_column_sums(key: torch.Tensor) -> torch.Tensor:
    """sqattn_k_column_sums: key [B,N,Hkv,D] -> fp32 [B,Hkv,D] sums over the sequence."""
    _require_cuda(key)
    b, n, hkv, d = key.shape
    sums = torch.empty(b, hkv, d, dtype=torch.float32, device=key.device)
    nbytes = b * hkv * 64 * d * 4
    ws = _workspace(nbytes, key.device)
    view = _view(key, "NHD")
    L.check(L.lib.sqattn_k_column_sums(C.byref(view), b, hkv, n, d, _dt(key.dtype), sums.data_ptr(), ws.data_ptr(),
                                       nbytes, _stream()))
    return sums


def decode(q, k, v, *, layout: str = "HND", out_dtype=torch.float16, return_lse: bool = False, p_fp8: bool = False,
           q_is_scaled: bool = False, kv_lens: Optional[Sequence[int]] = None, kv_len: Optional[int] = None,
           num_splits: int = 0, partial: bool = False, reference_tail: bool = False,
           kv_lens_device: Optional[torch.Tensor] = None, peer=None, head_dim_og: int = 0):
    """sqattn_decode.  q [B,Hq,1,D] (HND) or [B,1,Hq,D] (NHD); k/v caches of capacity >= kv_len.
    partial=True returns (O fp32 [B,Hq,D], LSE fp32 [B,Hq]) of these keys for a later merge.
    reference_tail=True reproduces the reference kernel's zero-score padding of the last 64-key tile.
    kv_lens_device (int32 [B] on the GPU): the lengths are read by the kernel at run time and ``kv_len`` is only the
    capacity the key ranges are planned for, so the call can sit in a CUDA graph that is replayed as the cache grows.
    peer: a filled ``_lib.PeerMergeArgs`` (dist.PeerExchange builds it): the merge of the split-KV partials, the
    exchange with the other GPUs and the merge across GPUs happen in one kernel; returns nothing (the result is
    written to peer.out)."""
    _require_cuda(q, k, v)
    poll_device_status(q.device)
    b, hq, one, d = _shape(q, layout)
    assert one == 1
    _, hkv, cap, _ = _shape(k, layout)
    a = L.DecodeArgs()
    a.q, a.k, a.v = _view(q, layout), _view(k, layout), _view(v, layout)
    a.batch, a.num_q_heads, a.num_kv_heads, a.head_dim, a.head_dim_og = b, hq, hkv, d, int(head_dim_og)
    a.kv_len = int(cap if kv_len is None else kv_len)
    lens = None
    if kv_lens is not None:
        lens = (C.c_int32 * b)(*[int(x) for x in kv_lens])
        a.kv_lens = lens
    a.dtype, a.p_fp8, a.q_is_scaled, a.num_splits = _dt(k.dtype), int(p_fp8), int(q_is_scaled), int(num_splits)
    a.reference_tail = int(reference_tail)
    if kv_lens_device is not None:
        if kv_lens is not None:
            raise ValueError("kv_lens and kv_lens_device are exclusive: device lengths are planned for kv_len")
        assert kv_lens_device.is_cuda and kv_lens_device.dtype == torch.int32 and kv_lens_device.numel() == b
        a.kv_lens_device = kv_lens_device.data_ptr()
    out = lse = po = pl = None
    if peer is not None:
        a.peer = C.addressof(peer)
        a.o_dtype = L.F16
    elif partial:
        po = torch.empty(b, hq, d, dtype=torch.float32, device=q.device)
        pl = torch.empty(b, hq, dtype=torch.float32, device=q.device)
        a.partial_o, a.partial_lse = po.data_ptr(), pl.data_ptr()
        a.o_dtype = L.F16
    else:
        out = torch.empty(q.shape, dtype=out_dtype, device=q.device)
        a.o = _view(out, layout)
        a.o_dtype = _dt(out_dtype)
        if return_lse:
            lse = torch.empty(b, hq, 1, dtype=torch.float32, device=q.device)
            a.lse = lse.data_ptr()
    need = L.lib.sqattn_decode_workspace_bytes(C.byref(a))
    if need == 0:  # the plan was rejected: let the entry point report why
        L.check(L.lib.sqattn_decode(C.byref(a), _stream()))
        raise ValueError("sqattn_decode: invalid arguments")
    ws = _workspace(need, q.device)
    a.workspace, a.workspace_bytes = ws.data_ptr(), need
    L.check(L.lib.sqattn_decode(C.byref(a), _stream()))
    if peer is not None:
        return None
    if partial:
        return po, pl
    return (out, lse) if return_lse else out


def decode_gather(q, idx, counts, k_rows, v_rows, row_stride: int, kv_dtype, *, out_dtype=torch.float16,
                  p_fp8: bool = False, q_is_scaled: bool = False, num_kv_heads: int = 1):
    """sqattn_decode over listed rows (sqattn_decode_args.gather): q [B,Hq,1,D]; key j of (sequence b, KV head h) is row
    idx[b*Hkv+h, j] of the matrix at k_rows[b*Hkv+h] / v_rows[b*Hkv+h] (int64 device tensors of device pointers), rows
    ``row_stride`` elements apart; counts (int32 [B] on the device) are the list lengths, idx.shape[1] the capacity the
    key ranges are planned for.  No host synchronisation."""
    _require_cuda(q, idx, counts, k_rows, v_rows)
    poll_device_status(q.device)
    b, hq, one, d = q.shape
    assert one == 1 and idx.dtype == torch.int32 and idx.is_contiguous() and idx.shape[0] == b * num_kv_heads
    assert counts.dtype == torch.int32 and counts.numel() == b
    assert k_rows.dtype == torch.int64 and v_rows.dtype == torch.int64 and k_rows.numel() == b * num_kv_heads == v_rows.numel()
    g = L.DecodeGather()
    g.idx, g.cap, g.k_rows, g.v_rows, g.row_stride = idx.data_ptr(), idx.shape[1], k_rows.data_ptr(), v_rows.data_ptr(), int(row_stride)
    a = L.DecodeArgs()
    a.q = _view(q, "HND")
    a.batch, a.num_q_heads, a.num_kv_heads, a.head_dim = b, hq, num_kv_heads, d
    a.kv_len = idx.shape[1]
    a.dtype, a.p_fp8, a.q_is_scaled = _dt(kv_dtype), int(p_fp8), int(q_is_scaled)
    a.kv_lens_device = counts.data_ptr()
    a.gather = C.addressof(g)
    out = torch.empty(q.shape, dtype=out_dtype, device=q.device)
    a.o = _view(out, "HND")
    a.o_dtype = _dt(out_dtype)
    need = L.lib.sqattn_decode_workspace_bytes(C.byref(a))
    if need == 0:  # the plan was rejected: let the entry point report why
        L.check(L.lib.sqattn_decode(C.byref(a), _stream()))
        raise ValueError("sqattn_decode: invalid arguments")
    ws = _workspace(need, q.device)
    a.workspace, a.workspace_bytes = ws.data_ptr(), need
    L.check(L.lib.sqattn_decode(C.byref(a), _stream()))
    return out


def decode_merge(part_o: torch.Tensor, part_lse: torch.Tensor, out_dtype=torch.float16, return_lse: bool = False):
    """sqattn_decode_merge: part_o [P, rows, D] fp32, part_lse [P, rows] fp32 -> O [rows, D]."""
    _require_cuda(part_o, part_lse)
    p, rows, d = part_o.shape
    out = torch.empty(rows, d, dtype=out_dtype, device=part_o.device)
    lse = torch.empty(rows, dtype=torch.float32, device=part_o.device) if return_lse else None
    L.check(L.lib.sqattn_decode_merge(part_o.contiguous().data_ptr(), part_lse.contiguous().data_ptr(), p, rows, d,
                                      out.data_ptr(), _dt(out_dtype), None if lse is None else lse.data_ptr(),
                                      _stream()))
    return (out, lse) if return_lse else out


def check_device_status():
    """Raise if a bounded device-side wait gave up since the last check (synchronises the stream); clears the
    device word and its host mirror, after which launches compute again."""
    ent = _MIRRORS.get(torch.cuda.current_device())
    try:
        L.check(L.lib.sqattn_check_device_status(_stream()))
    finally:
        if ent is not None:
            ent[1].value = 0


def decode_static_scratch(q, k, v, out, *, layout: str = "HND", lse: Optional[torch.Tensor] = None,
                          p_fp8: bool = False, q_is_scaled: bool = False, kv_lens: Optional[Sequence[int]] = None,
                          kv_len: Optional[int] = None, num_splits: int = 0, reference_tail: bool = False):
    """sqattn_decode_static_scratch: decode into the caller's ``out`` (and ``lse``) without any allocation, for
    callers inside a region where device memory may not be allocated.  The split-KV partials use the scratch
    array built into the library (4 MiB + 64 KiB); calls that need more are rejected, and calls must not overlap
    on the GPU.  Make the first call on a device outside stream capture."""
    _require_cuda(q, k, v, out)
    b, hq, one, d = _shape(q, layout)
    assert one == 1
    _, hkv, cap, _ = _shape(k, layout)
    a = L.DecodeArgs()
    a.q, a.k, a.v, a.o = _view(q, layout), _view(k, layout), _view(v, layout), _view(out, layout)
    a.lse = None if lse is None else lse.data_ptr()
    a.batch, a.num_q_heads, a.num_kv_heads, a.head_dim = b, hq, hkv, d
    a.kv_len = int(cap if kv_len is None else kv_len)
    if kv_lens is not None:
        lens = (C.c_int32 * b)(*[int(x) for x in kv_lens])
        a.kv_lens = lens
    a.dtype, a.o_dtype = _dt(k.dtype), _dt(out.dtype)
    a.p_fp8, a.q_is_scaled, a.num_splits, a.reference_tail = int(p_fp8), int(q_is_scaled), int(num_splits), int(reference_tail)
    L.check(L.lib.sqattn_decode_static_scratch(C.byref(a), _stream()))
    return out


def rmsnorm(x: torch.Tensor, weight: torch.Tensor, eps: float, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """sqattn_rmsnorm over the last dimension of x [..., dim] (rows may be strided); out may be x itself."""
    _require_cuda(x, weight)
    dim = x.shape[-1]
    x2 = x.reshape(-1, dim) if x.dim() != 2 else x
    assert x2.stride(1) == 1 and weight.is_contiguous() and weight.numel() == dim
    out = torch.empty(x.shape, dtype=x.dtype, device=x.device) if out is None else out
    o2 = out.reshape(-1, dim) if out.dim() != 2 else out
    assert o2.stride(1) == 1 and o2.shape == x2.shape
    assert o2.data_ptr() == out.data_ptr(), "out must be viewable as [rows, dim] without a copy"
    L.check(L.lib.sqattn_rmsnorm(x2.data_ptr(), weight.data_ptr(), o2.data_ptr(), x2.shape[0], dim, x2.stride(0),
                                 o2.stride(0), float(eps), _dt(x.dtype), _stream()))
    return out


def rope_qk(qkv: torch.Tensor, seq_len: int, num_heads: int, head_dim: int, cos_sin_cache: torch.Tensor, pos0: int,
            pos_device: Optional[torch.Tensor] = None):
    """sqattn_rope_qk: rotate the first num_heads heads of every row of the fused projection qkv [rows, width]
    in place; row r takes position pos0 + r % seq_len of cos_sin_cache [max_len, head_dim] (fp32).  With
    ``pos_device`` (int64 [1] on the GPU) that value is added to pos0 when the kernel runs."""
    _require_cuda(qkv, cos_sin_cache)
    assert qkv.dim() == 2 and qkv.stride(1) == 1
    assert cos_sin_cache.dtype == torch.float32 and cos_sin_cache.is_contiguous() and cos_sin_cache.shape[1] == head_dim
    if pos_device is not None:
        assert pos_device.is_cuda and pos_device.dtype == torch.int64
    L.check(L.lib.sqattn_rope_qk_devpos(qkv.data_ptr(), qkv.stride(0), qkv.shape[0], int(seq_len), int(num_heads),
                                        int(head_dim), cos_sin_cache.data_ptr(), cos_sin_cache.shape[0], int(pos0),
                                        None if pos_device is None else pos_device.data_ptr(), _dt(qkv.dtype), _stream()))
    return qkv


def silu_mul(x: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """sqattn_silu_mul: x [..., 2*inter] contiguous -> [..., inter]."""
    _require_cuda(x)
    assert x.is_contiguous() and x.shape[-1] % 2 == 0
    inter = x.shape[-1] // 2
    out = torch.empty(*x.shape[:-1], inter, dtype=x.dtype, device=x.device) if out is None else out
    assert out.is_contiguous()
    L.check(L.lib.sqattn_silu_mul(x.data_ptr(), out.data_ptr(), x.numel() // (2 * inter), inter, _dt(x.dtype), _stream()))
    return out
