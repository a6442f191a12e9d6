"""Generate golden vectors from the reference's own Triton kernels.

Run once, where the reference checkout is available:

    python tests/golden/make_golden.py /path/to/reference

The reference's launchers need Paddle (not installable here), but its
``@triton.jit`` kernels do not: they are imported unmodified, with empty stub
modules standing in for ``paddle`` / ``paddle_utils``, and executed on CPU
tensors by Triton's interpreter (TRITON_INTERPRET=1).  Launch parameters
(grid, BLOCK sizes, strides, q pre-scaling) are restated from the launchers:
attn_triton_mix_relative.py:383-475, attn_triton_mix_bad.py:359-422,
attn_triton.py:249-310, attn_triton_decode.py:268-324, kmeans.py:127-196.
Inputs are fp16 (the interpreter has no bf16).  The vectors are written next
to this script as ``*.npz`` and are what the CPU tests pin the oracle against.

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
    pd = types.ModuleType("paddle")
    pd.float16, pd.bfloat16, pd.float32 = torch.float16, torch.bfloat16, torch.float32
    pd.Tensor = torch.Tensor
    pd.dtype = torch.dtype
    sys.modules["paddle"] = pd
    sys.modules["paddle_utils"] = types.ModuleType("paddle_utils")
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
    }
    for name, fn in cases.items():
        d = {k: (v.numpy() if isinstance(v, torch.Tensor) else v) for k, v in fn().items()}
        np.savez_compressed(os.path.join(HERE, f"{name}.npz"), **d)
        print(name, {k: getattr(v, "shape", ()) for k, v in d.items()})


if __name__ == "__main__":
    main()
