"""Generate golden vectors from the reference's own Triton kernels.

Run once, where the reference checkout is available:

    python tests/golden/make_golden.py /path/to/reference

Two kinds of vectors are produced, both by running the reference's code unmodified from its checkout:

* kernel vectors (relative, absolute, dense, decode, kmeans and their *_large variants): the ``@triton.jit``
  kernels executed on CPU tensors by Triton's interpreter (TRITON_INTERPRET=1), with the launch parameters (grid,
  BLOCK sizes, strides, q pre-scaling) restated from the launchers: attn_triton_mix_relative.py:383-475,
  attn_triton_mix_bad.py:359-422, attn_triton.py:249-310, attn_triton_decode.py:268-324, kmeans.py:127-196.
* glue vectors (fake_quant, adapter, window_search, segment_kmeans): the reference's Python code itself - the
  quantiser classes, ``mp_triton_wrapper`` with its launchers, the histogram and threshold functions, and
  ``segment_k_means`` - executed through ``paddle_torch_shim`` (a ``paddle`` module that forwards to torch; the
  two Paddle semantics it has to assume are stated there) with the kernels again on the interpreter.

Inputs are fp16 where a kernel is involved (the interpreter has no bf16); 16-bit arrays that numpy cannot hold
(bf16) are stored as their int16 bit patterns under a ``*_bf16bits`` key.  The vectors are written next to this
script as ``*.npz`` and are what the CPU tests pin the oracle against.

One repair is made to the interpreter (third-party tooling, not the reference):
its software fp32 -> float8e4nv conversion drops the carry when the mantissa
rounds up into the next binade (125.7 becomes 64 instead of 128) and rounds
halves up instead of to even.  The GPU instruction the compiled kernel uses
(cvt.rn.satfinite.e4m3x2.f32) is IEEE round-to-nearest-even, which is what
``torch.float8_e4m3fn`` casts implement, so that conversion is substituted.
"""
import os
import sys
import types

os.environ["TRITON_INTERPRET"] = "1"

import numpy as np  # noqa: E402
import torch  # noqa: E402

HERE = os.path.dirname(os.path.abspath(__file__))
LOG2E = 1.44269504


def _stub_modules(ref_root):
    sys.path.insert(0, HERE)
    import paddle_torch_shim
    paddle_torch_shim.install()
    sys.path.insert(0, ref_root)


def _repair_interpreter_fp8():
    import triton.language as tl
    from triton.runtime import interpreter as interp

    orig = interp._convert_float

    def convert(inp, in_dtype, out_dtype, rounding_mode):
        if out_dtype == tl.float8e4nv and in_dtype == tl.float32:
            t = torch.from_numpy(np.ascontiguousarray(inp).view(np.float32).copy())
            return t.to(torch.float8_e4m3fn).view(torch.uint8).numpy().reshape(inp.shape)
        return orig(inp, in_dtype, out_dtype, rounding_mode)

    interp._convert_float = convert


def _scale(q, d):
    return (q.float() * torch.tensor(1.0 / d ** 0.5 * LOG2E, dtype=torch.float32)).to(q.dtype)


def _randn(g, *shape, scale=1.0):
    return (torch.randn(*shape, generator=g) * scale).to(torch.float16)


def gen_relative(fp8):
    from sqattn.attn_triton_mix_relative import attn_prefill_fwd
    g = torch.Generator().manual_seed(11)
    b, hq, hkv, n, d, sink = 1, 4, 2, 300, 64, 64
    q = _randn(g, b, hq, n, d)
    k = _randn(g, b, hkv, n, d)
    k[..., 3] *= 8
    v = _randn(g, b, hkv, n, d)
    r8 = torch.tensor([0.2, 0.5, 0.3, 1.0], dtype=torch.float32)
    r4 = torch.tensor([0.6, 0.5, 0.9, 0.0], dtype=torch.float32)
    qs = _scale(q, d)
    o = torch.zeros_like(q)
    lse = torch.zeros(b, hq, n, dtype=torch.float32)
    grid = ((n + 63) // 64, hq, b)
    # as shipped the int8 tensors are passed in both operand slots (440-446)
    attn_prefill_fwd[grid](qs, k, qs, k, v, o, lse, r8, r4,
                           *qs.stride()[:3], *k.stride()[:3], *v.stride()[:3], *o.stride()[:3],
                           n, n, hq, hq // hkv, BLOCK_M=64, BLOCK_N=64, HEAD_DIM=d, STAGE=4,
                           RETURN_LSE=True, is_P_fp8_quant=fp8, SINK_SIZE=sink)
    return dict(q=q, k=k, v=v, r8=r8, r4=r4, sink=np.int32(sink), o=o, lse=lse)


def gen_absolute(fp8):
    from sqattn.attn_triton_mix_bad import _attn_prefill_fwd
    g = torch.Generator().manual_seed(12)
    b, hq, hkv, n, d, sink = 1, 2, 1, 512, 64, 64
    q8 = _randn(g, b, hq, n, d)
    k8 = _randn(g, b, hkv, n, d)
    q4 = (q8.float() + 0.05 * torch.randn(q8.shape, generator=g)).to(torch.float16)
    k4 = (k8.float() + 0.05 * torch.randn(k8.shape, generator=g)).to(torch.float16)
    v = _randn(g, b, hkv, n, d)
    w8 = torch.tensor([128, 192], dtype=torch.int32)
    w4 = torch.tensor([320, 256], dtype=torch.int32)
    q8s, q4s = _scale(q8, d), _scale(q4, d)
    o = torch.zeros_like(q8)
    lse = torch.zeros(b, hq, n, dtype=torch.float32)
    grid = ((n + 127) // 128, hq, b)
    _attn_prefill_fwd[grid](q8s, k8, q4s, k4, v, o, lse, w8, w4,
                            *q8s.stride()[:3], *k8.stride()[:3], *v.stride()[:3], *o.stride()[:3],
                            n, n, hq, hq // hkv, BLOCK_M=128, BLOCK_N=64, HEAD_DIM=d, STAGE=4,
                            RETURN_LSE=True, is_P_fp8_quant=fp8, SINK_SIZE=sink)
    return dict(q8=q8, k8=k8, q4=q4, k4=k4, v=v, w8=w8, w4=w4, sink=np.int32(sink), o=o, lse=lse)


def gen_dense(fp8):
    from sqattn.attn_triton import _attn_fwd
    g = torch.Generator().manual_seed(13)
    b, hq, hkv, n, d = 1, 2, 1, 320, 128
    q = _randn(g, b, hq, n, d)
    k = _randn(g, b, hkv, n, d)
    v = _randn(g, b, hkv, n, d)
    qs = _scale(q, d)
    o = torch.zeros_like(q)
    lse = torch.zeros(b, hq, n, dtype=torch.float32)
    grid = ((n + 127) // 128, hq, b)
    _attn_fwd[grid](qs, k, v, o, lse, *qs.stride()[:3], *k.stride()[:3], *v.stride()[:3], *o.stride()[:3],
                    n, n, hq, hq // hkv, BLOCK_M=128, BLOCK_N=64, HEAD_DIM=d, STAGE=3,
                    RETURN_LSE=True, is_P_fp8_quant=fp8)
    return dict(q=q, k=k, v=v, o=o, lse=lse)


def gen_decode(fp8):
    from sqattn.attn_triton_decode import _attn_decode_fwd
    g = torch.Generator().manual_seed(14)
    b, hq, hkv, L, d = 2, 4, 2, 600, 64
    q = _randn(g, b, hq, 1, d)
    k = _randn(g, b, hkv, L, d)
    v = _randn(g, b, hkv, L, d)
    # the launcher centres K and scales q first (attn_triton_decode.py:268-271)
    kc = k - k.float().mean(dim=2, keepdim=True).to(k.dtype)
    qs = _scale(q, d)
    o = torch.zeros_like(q)
    lse = torch.zeros(b, hq, 1, dtype=torch.float32)
    _attn_decode_fwd[(b, hq)](qs, kc, v, o, lse, *qs.stride()[:3], *kc.stride()[:3], *v.stride()[:3],
                              *o.stride()[:3], 1, L, hq, hq // hkv, BLOCK_N=64, HEAD_DIM=d,
                              RETURN_LSE=True, is_P_fp8_quant=fp8)
    return dict(q=q, k=k, v=v, o=o, lse=lse)


def gen_kmeans():
    from cache_hub.kmeans import _triton_assign_kernel, _triton_update_kernel
    g = torch.Generator().manual_seed(15)
    G, T, K, D = 2, 500, 64, 64
    data = _randn(g, G, T, D)
    cent = data[:, torch.linspace(3, T - 4, K).long()].clone()
    out = dict(data=data, cent0=cent.clone())
    for it, norm in enumerate((True, False)):
        s = torch.zeros(G, K, D, dtype=torch.float32)
        c = torch.zeros(G, K, dtype=torch.int32)
        m = torch.zeros(G, T, dtype=torch.int32)
        _triton_assign_kernel[((T + 127) // 128, G, 1)](
            data, cent, s, c, m, *data.stride(), *cent.stride(), *s.stride(), *c.stride(), *m.stride(),
            T, K, BLOCK_N=128, BLOCK_K=32, BLOCK_D=D)
        _triton_update_kernel[((K + 127) // 128, G, 1)](
            cent, s, c, *cent.stride(), *s.stride(), *c.stride(), K, BLOCK_K=128, BLOCK_D=D, NORMORLIZE=norm)
        out[f"idx{it}"] = m.clone()
        out[f"sum{it}"] = s.clone()
        out[f"cnt{it}"] = c.clone()
        out[f"cent{it + 1}"] = cent.clone()
    return out


def gen_relative_large(fp8):
    """The windowed kernel at head_dim 128, 1024 tokens, sink 256, GQA 7:1 with an outlier K channel."""
    from sqattn.attn_triton_mix_relative import attn_prefill_fwd
    g = torch.Generator().manual_seed(21)
    b, hq, hkv, n, d, sink = 1, 7, 1, 1024, 128, 256
    q = _randn(g, b, hq, n, d)
    k = _randn(g, b, hkv, n, d)
    k[..., 5] *= 8
    v = _randn(g, b, hkv, n, d)
    r8 = torch.tensor([0.1, 0.1, 0.25, 0.3, 0.05, 0.5, 0.2], dtype=torch.float32)
    r4 = torch.tensor([0.1, 0.3, 0.25, 0.6, 0.4, 0.5, 0.0], dtype=torch.float32)
    qs = _scale(q, d)
    o = torch.zeros_like(q)
    lse = torch.zeros(b, hq, n, dtype=torch.float32)
    grid = ((n + 63) // 64, hq, b)
    attn_prefill_fwd[grid](qs, k, qs, k, v, o, lse, r8, r4,
                           *qs.stride()[:3], *k.stride()[:3], *v.stride()[:3], *o.stride()[:3],
                           n, n, hq, hq // hkv, BLOCK_M=64, BLOCK_N=64, HEAD_DIM=d, STAGE=4,
                           RETURN_LSE=True, is_P_fp8_quant=fp8, SINK_SIZE=sink)
    return dict(q=q, k=k, v=v, r8=r8, r4=r4, sink=np.int32(sink), o=o, lse=lse)


def gen_decode_large(fp8):
    """The decode kernel at 4096 keys (64 tiles), head_dim 128, GQA 7:1."""
    from sqattn.attn_triton_decode import _attn_decode_fwd
    g = torch.Generator().manual_seed(24)
    b, hq, hkv, L, d = 1, 7, 1, 4096, 128
    q = _randn(g, b, hq, 1, d)
    k = _randn(g, b, hkv, L, d)
    v = _randn(g, b, hkv, L, d)
    kc = k - k.float().mean(dim=2, keepdim=True).to(k.dtype)
    qs = _scale(q, d)
    o = torch.zeros_like(q)
    lse = torch.zeros(b, hq, 1, dtype=torch.float32)
    _attn_decode_fwd[(b, hq)](qs, kc, v, o, lse, *qs.stride()[:3], *kc.stride()[:3], *v.stride()[:3],
                              *o.stride()[:3], 1, L, hq, hq // hkv, BLOCK_N=64, HEAD_DIM=d,
                              RETURN_LSE=True, is_P_fp8_quant=fp8)
    return dict(q=q, k=k, v=v, o=o, lse=lse)


def _bits(t):
    """bf16 tensor -> int16 bit patterns (numpy has no bf16)"""
    return t.view(torch.int16)


def gen_fake_quant():
    """IntegerQuantizer / FloatQuantizer of sqattn/fake_quant.py exactly as the adapter constructs them
    (attn_replacer.py:340-358), on [B, H, N, D] tensors in fp16 and bf16, with exact .5 ties of x/scale in the data."""
    from sqattn.fake_quant import FloatQuantizer, IntegerQuantizer
    g = torch.Generator().manual_seed(31)
    out = {}
    x = torch.randn(2, 3, 40, 64, generator=g)
    x[..., 7] *= 8                                   # an outlier channel
    x[0, 0, 0] = torch.arange(64) - 31.5             # absmax 32.5 -> scale 32.5/127: non-trivial ties elsewhere
    x[0, 0, 1] = (torch.arange(64) - 32).float() * 0.5   # absmax 16, 8-bit scale 16/127; 4-bit scale 16/7
    x[0, 0, 2] = 127.0 * torch.sign(torch.randn(64, generator=g)) * (torch.arange(64) % 5 + 0.5) / 127.0 * 2  # multiples of scale/2
    x[0, 0, 2, 0] = 127.0 * 2 / 127.0 * 4.5 * 0 + 9.0  # absmax 9 -> scale 9/127
    x[0, 1, 3] = 1e-7                                # below the 1e-5 clip of the range
    x[1, 2, 5] = 0.0
    quantisers = {
        "int8_token": IntegerQuantizer(8, True, "per_token"), "int4_token": IntegerQuantizer(4, True, "per_token"),
        "int8_channel": IntegerQuantizer(8, True, "per_channel"),
        "e4m3_token": FloatQuantizer("e4m3", True, "per_token"), "e5m2_token": FloatQuantizer("e5m2", True, "per_token"),
        "e4m3_channel": FloatQuantizer("e4m3", True, "per_channel"), "e5m2_channel": FloatQuantizer("e5m2", True, "per_channel"),
    }
    for dname, dt in (("f16", torch.float16), ("bf16", torch.bfloat16)):
        xin = x.to(dt)
        out[f"x_{dname}" if dt == torch.float16 else f"x_{dname}bits"] = xin if dt == torch.float16 else _bits(xin)
        for qname, qz in quantisers.items():
            y = qz.fake_quant_tensor(xin.clone())
            assert y.dtype == dt
            out[f"{qname}_{dname}" if dt == torch.float16 else f"{qname}_{dname}bits"] = y if dt == torch.float16 else _bits(y)
    return out


def gen_adapter():
    """mp_triton_wrapper(...).attention_fn of sqattn/attn_replacer.py end to end (repeat_kv, K centring, the five
    fake-quants, the launcher with its scaling and window tensors, the output transpose) for the relative and the
    absolute branch and for int / e4m3 operands.  Inputs fp16; the launcher's bf16 output is stored as fp16."""
    from sqattn.attn_replacer import mp_triton_wrapper
    # Triton's CPU interpreter cannot store bf16: the launcher's ``output_dtype=paddle.bfloat16`` becomes float16 for
    # this generator only (the inputs are fp16, so no other code path looks at the name)
    sys.modules["paddle"].bfloat16 = torch.float16
    g = torch.Generator().manual_seed(32)
    b, n, hq, hkv, d = 1, 320, 4, 2, 64
    q = _randn(g, b, n, hq, d)
    k = _randn(g, b, n, hkv, d)
    k[..., 9] *= 8
    k += 0.5                                         # a sequence mean for the centring to remove
    v = _randn(g, b, n, hkv, d)
    out = dict(q=q, k=k, v=v)
    layer = types.SimpleNamespace(num_key_value_groups=hq // hkv)
    cases = {
        "rel_int": (True, "int", "int", [0.2, 0.5, 0.3, 1.0], [0.6, 0.5, 0.9, 0.0], 64),
        "rel_e4m3": (True, "e4m3", "e4m3", [0.2, 0.5, 0.3, 1.0], [0.6, 0.5, 0.9, 0.0], 64),
        # the absolute branch only runs with one integer per window through this wrapper: a list reaches the launcher's
        # ``.to`` (attn_triton_mix_bad.py:317-332) and a tensor fails in ``or 0`` (attn_replacer.py:320)
        "abs_int": (False, "int", "int", 100, 192, 64),
        "abs_e5m2": (False, "e5m2", "int", 100, 192, 64),
    }
    for name, (rel, qk, vq, w8, w4, sink) in cases.items():
        args = types.SimpleNamespace(qk_qtype=qk, v_qtype=vq, use_relative_distance=rel)
        fn = mp_triton_wrapper(3, bit8_window_sizes=w8, bit4_window_sizes=w4, sink_window_size=sink, args=args)
        o = fn(layer, q.clone(), k.clone(), v.clone(), None)
        assert o.shape == (b, n, hq * d)
        out[f"o_{name}"] = o
        out[f"w8_{name}"], out[f"w4_{name}"] = np.asarray(w8, dtype=np.float64), np.asarray(w4, dtype=np.float64)
    out["sink"] = np.int32(64)
    sys.modules["paddle"].bfloat16 = torch.bfloat16
    return out


def gen_window_search():
    """cal_attn_weight (attn_replacer.py:253-278) and the histogram / threshold functions of
    sqattn/window_search.py (20-128, 244-321) on one head's softmax map."""
    from sqattn.attn_replacer import cal_attn_weight
    from sqattn import window_search as ws
    g = torch.Generator().manual_seed(33)
    n, hq, hkv, d = 300, 2, 1, 64
    q = torch.randn(1, n, hq, d, generator=g)
    k = torch.randn(1, n, hkv, d, generator=g)
    layer = types.SimpleNamespace(num_key_value_groups=hq // hkv)
    amap = cal_attn_weight(layer, q, k)               # [1, hq, n, n] fp32
    out = dict(q=q, k=k, attn=amap)
    for h in range(hq):
        a = amap[0, h]
        out[f"rel_hist_{h}"] = ws.compute_relative_attention_histogram_gpu_with_sink(a.clone(), num_bins=200, sink_len=64)
        out[f"abs_hist_{h}"] = ws.compute_absolute_attention_histogram_gpu_with_sink(a.clone(), max_len=n, sink_len=64)
        out[f"abs_hist_nosink_{h}"] = ws.compute_attention_histogram_gpu(a.clone(), max_len=n)
        out[f"rel_hist_nosink_{h}"] = ws.compute_relative_attention_histogram_gpu(a.clone(), num_bins=100)
    thr = [0.5, 0.9, 0.95, 0.99, 1.0]
    out["thresholds"] = np.asarray(thr)
    out["rel_windows"] = np.asarray([[ws.find_optimal_relative_window(out[f"rel_hist_{h}"], t, 200) for t in thr] for h in range(hq)])
    out["abs_windows"] = np.asarray([[ws.find_optimal_window(out[f"abs_hist_{h}"], t) for t in thr] for h in range(hq)])
    out["rel_window_empty"] = np.float64(ws.find_optimal_relative_window(np.zeros(200), 0.9, 200))
    out["abs_window_empty"] = np.int64(ws.find_optimal_window(np.zeros(300), 0.9))
    return out


def gen_segment_kmeans():
    """segment_k_means of cache_hub/kmeans.py:332-375 as a whole (centroid initialisation, segmenting, the Lloyd
    iterations with and without normalisation, value sums, member lists), 1 and 2 segments.  Member lists come out
    of the interpreter in program order; they are stored sorted, the order within a cluster being unspecified
    (atomic arrival order on a GPU)."""
    from cache_hub.kmeans import segment_k_means
    g = torch.Generator().manual_seed(34)
    G, T, K, D = 2, 512, 64, 64
    key = _randn(g, G, T, D)
    key[..., 11] *= 4
    value = _randn(g, G, T, D)
    out = dict(key=key, value=value)
    for seg in (1, 2):
        cent, vsum, clusters, csize = segment_k_means(key.clone(), value.clone(), K, num_iters=4, num_segments=seg)
        srt = torch.zeros_like(clusters)
        for gi in range(clusters.shape[0]):
            for c in range(K):
                m = int(csize[gi, c])
                srt[gi, c, :m] = torch.sort(clusters[gi, c, :m]).values
        out[f"centroids_{seg}"], out[f"value_sum_{seg}"] = cent, vsum
        out[f"clusters_{seg}"], out[f"cluster_size_{seg}"] = srt, csize
    return out


def _both(gen):
    """Run a generator with is_P_fp8_quant off and on; inputs stored once."""
    off, on = gen(False), gen(True)
    off["o_fp8"], off["lse_fp8"] = on["o"], on["lse"]
    return off


def main():
    if len(sys.argv) < 2:
        raise SystemExit("usage: python make_golden.py <path to a checkout of the reference repository>")
    ref_root = sys.argv[1]
    _stub_modules(ref_root)
    _repair_interpreter_fp8()
    cases = {
        "relative": lambda: _both(gen_relative),
        "absolute": lambda: _both(gen_absolute),
        "dense": lambda: _both(gen_dense),
        "decode": lambda: _both(gen_decode),
        "kmeans": gen_kmeans,
        "relative_large": lambda: _both(gen_relative_large),
        "decode_large": lambda: _both(gen_decode_large),
        "fake_quant": gen_fake_quant,
        "adapter": gen_adapter,
        "window_search": gen_window_search,
        "segment_kmeans": gen_segment_kmeans,
    }
    only = set(sys.argv[2:])
    for name, fn in cases.items():
        if only and name not in only:
            continue
        d = {k: (v.numpy() if isinstance(v, torch.Tensor) else v) for k, v in fn().items()}
        np.savez_compressed(os.path.join(HERE, f"{name}.npz"), **d)
        print(name, {k: getattr(v, "shape", ()) for k, v in d.items()})


if __name__ == "__main__":
    main()
