"""How far would REAL 8-bit tensor-core operands move the result?  (test infrastructure, CPU only)

The reference defines SQAttn through fake quantisation: Q and K become code * scale rounded to bf16
(sqattn/fake_quant.py:80-86, 114-125), q is multiplied by the softmax scale and rounded to bf16 again
(attn_triton_mix_relative.py:383-385), and the kernel multiplies those bf16 values.  An INT8 tensor-core product
would instead form the exact integer dot product of the codes and apply the per-token scales afterwards, i.e. it
skips both bf16 roundings.  ``exact_operand_variant`` evaluates that variant with the same tile loop as the oracle
(fp32 operands equal to code * scale, scaling in fp32; an fp32 dot product of such values differs from the exact
integer one by 2^-24 relative, three orders of magnitude below the bf16 effect being measured) so that the two can
be compared element by element.  V and the P*V product are the same in both."""
from __future__ import annotations

import torch

from . import sqattn_oracle as so


def exact_operand_variant(query, key, value, num_kv_groups, win8, win4, sink, **kw):
    """attention_fn with Q/K operands that are exactly code * scale (no bf16 rounding of the dequantised values
    or of q * softmax scale); K is still centred in the input dtype as the adapter does."""
    k_c = so.center_keys(so.repeat_kv(key, num_kv_groups)).float()
    q = query.permute(0, 2, 1, 3).float()
    v = so.repeat_kv(value, num_kv_groups)
    f8, f4, fv = so.make_quantizers(kw.get("qk_qtype", "int"), kw.get("v_qtype", "int"))
    q8, q4, k8, k4 = f8(q, "half_away"), f4(q, "half_away"), f8(k_c, "half_away"), f4(k_c, "half_away")
    v8 = fv(v, "half_away")
    o = so.windowed_prefill(q8, k8, q4, k4, v8, win8, win4, sink,
                            mode="relative" if kw.get("use_relative_distance", True) else "absolute",
                            tensor_layout="HND", output_dtype=torch.bfloat16, p_fp8_mode=kw.get("p_fp8_mode", "off"))
    b, h, n, d = o.shape
    return o.transpose(1, 2).contiguous().view(b, n, h * d)


def compare(seed=0, n=4096, hq=28, hkv=4, d=128, ratio=0.1, sink=256, p_fp8_mode="off"):
    """max and mean |dO| of the exact-operand variant against the reference's fake-quant emulation on seeded inputs
    of the benchmark distribution (N(0,1), four K channels x 8), bf16 inputs."""
    q, k, v = so.make_inputs(seed, 1, n, hq, hkv, d, torch.bfloat16)
    ref = so.attention_fn(q, k, v, hq // hkv, [ratio] * hq, [ratio] * hq, sink, p_fp8_mode=p_fp8_mode)
    var = exact_operand_variant(q, k, v, hq // hkv, [ratio] * hq, [ratio] * hq, sink, p_fp8_mode=p_fp8_mode)
    diff = (ref.float() - var.float()).abs()
    return {"max_abs": diff.max().item(), "mean_abs": diff.mean().item(), "max_abs_o": ref.float().abs().max().item()}


if __name__ == "__main__":
    for mode in ("off", "all"):
        print(mode, compare(p_fp8_mode=mode))
