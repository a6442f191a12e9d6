"""The operator that replaces ``layer.prefill_attention`` (sqattn/attn_replacer.py:12-34, 296-454).

``process_model`` installs, and ``mp_triton_wrapper`` builds, an ``attention_fn(module, query, key, value,
attention_mask, dropout, scaling, sliding_window, **kwargs)`` with the reference's signature: query
[B,N,Hq,D], key/value [B,N,Hkv,D] in, [B,N,Hq*D] bf16 out; mask, dropout, scaling and sliding_window are
ignored and the softmax scale is always 1/sqrt(D), as in the reference."""
from __future__ import annotations

import types

import torch

from .. import _lib as L
from .. import ops


def process_model(model, method, window_sizes=None, args=None):
    """Install the SQAttn prefill operator on every layer listed in ``window_sizes``
    (``{layer: {"bit8": [...], "bit4": [...], "sink": 256}}``); the sink is fixed at 256 as in the reference."""
    if method == "SQAttn":
        for i in range(len(model.layers)):
            if i in window_sizes.keys():
                layer = model.layers[i]
                layer.prefill_attention = types.MethodType(
                    mp_triton_wrapper(i, args=args, bit8_window_sizes=window_sizes[i]["bit8"],
                                      bit4_window_sizes=window_sizes[i]["bit4"], sink_window_size=256), layer)
                model.layers[i] = layer
    elif method in ("SDPA", "FlashAttn"):
        pass
    else:
        raise ValueError(f"Unsupported attention type: {method}")
    return model


def _normalise_windows(bit8, bit4):
    """List/int normalisation of the factory arguments (attn_replacer.py:299-321)."""
    is_per_head = isinstance(bit8, list) or isinstance(bit4, list)
    if is_per_head:
        num_heads = len(bit8) if isinstance(bit8, list) else len(bit4)
        if isinstance(bit8, int):
            bit8 = [bit8] * num_heads
        if isinstance(bit4, int):
            bit4 = [bit4] * num_heads
        if bit8 is None:
            bit8 = [0] * num_heads
        if bit4 is None:
            bit4 = [0] * num_heads
    else:
        bit8 = bit8 or 0
        bit4 = bit4 or 0
    return bit8, bit4


def mp_triton_wrapper(layer_idx, bit8_window_sizes=0, bit4_window_sizes=0, sink_window_size=0, args=None,
                      p_fp8_mode="off"):
    bit8_window_sizes, bit4_window_sizes = _normalise_windows(bit8_window_sizes, bit4_window_sizes)
    fp8 = {"off": L.P_FP8_OFF, "all": L.P_FP8_ALL, "stage2": L.P_FP8_STAGE2}[p_fp8_mode]

    def attention_fn(module, query, key, value, attention_mask, dropout=0.0, scaling=1.0, sliding_window=None,
                     **kwargs):
        if args.qk_qtype not in L.QTYPE:
            raise ValueError(f"Invalid quantization type: {args.qk_qtype}")
        if args.v_qtype not in L.QTYPE:
            raise ValueError(f"Invalid quantization type: {args.v_qtype}")
        b, n, hq, d = query.shape
        relative = bool(args.use_relative_distance)
        # the relative launch never reads the int4 tensors (attn_triton_mix_relative.py:440-446): skip them
        q8, q4, k8, k4, v8 = ops.prep_qkv(query, key, value, qk_qtype=args.qk_qtype, v_qtype=args.v_qtype,
                                          skip_bit4=relative)
        out = torch.empty(b, n, hq * d, dtype=torch.bfloat16, device=query.device)
        o4 = out.view(b, n, hq, d)

        def per_head(w, conv):
            return [conv(w)] * hq if isinstance(w, (int, float)) else [conv(x) for x in w]

        if relative:
            ops.prefill(q8, k8, q8, k8, v8, mode=L.MODE_RELATIVE_WINDOW, win8=per_head(bit8_window_sizes, float),
                        win4=per_head(bit4_window_sizes, float), sink=sink_window_size, layout="HND",
                        p_fp8_mode=fp8, q_is_scaled=True, out=o4, out_layout="NHD")
        else:
            ops.prefill(q8, k8, q4, k4, v8, mode=L.MODE_ABSOLUTE_WINDOW, win8=per_head(bit8_window_sizes, int),
                        win4=per_head(bit4_window_sizes, int), sink=sink_window_size, layout="HND",
                        p_fp8_mode=fp8, q_is_scaled=True, out=o4, out_layout="NHD")
        return out

    return attention_fn
