"""The fused input preparation (K centring + fake quantisers + q scaling) against the oracle's restatement of
the adapter.  Integer grids make this almost always bit-exact; a value may land on the neighbouring grid point
when the fp32 K mean differs in its last bit (different summation order), so a tiny fraction of mismatches by
one quantisation step is allowed for K and none for Q and V."""
import pytest
import torch

from oracle import sqattn_oracle as so

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("n,hq,hkv,d", [(300, 4, 2, 128), (1024, 28, 4, 128), (77, 6, 3, 64)])
@pytest.mark.parametrize("qk_qtype,v_qtype", [("int", "int"), ("e4m3", "e5m2"), ("e5m2", "e4m3")])
def test_prep_matches_adapter(dtype, n, hq, hkv, d, qk_qtype, v_qtype):
    from longcontext_sqattn_paddle_b200 import ops
    q, k, v = so.make_inputs(3, 2, n, hq, hkv, d, dtype)
    q8, q4, k8, k4, v8 = (t.cpu() for t in ops.prep_qkv(q.cuda(), k.cuda(), v.cuda(), qk_qtype=qk_qtype, v_qtype=v_qtype))
    groups = hq // hkv
    r8, r4, rk8, rk4, rv8 = so.prep_qkv(q, k, v, groups, qk_qtype, v_qtype)
    r8, r4 = so.scale_q(r8, d), so.scale_q(r4, d)
    rk8, rk4, rv8 = rk8[:, ::groups], rk4[:, ::groups], rv8[:, ::groups]
    exact = qk_qtype == "int"

    def frac_bad(a, b):
        return (a.float() != b.float()).float().mean().item()

    assert frac_bad(q4, r4) == 0 and frac_bad(k4, rk4) < 2e-3
    if exact:
        assert frac_bad(q8, r8) == 0
        assert frac_bad(k8, rk8) < 2e-3
    else:  # emulated float formats go through log2/exp2: compare by value
        assert (q8.float() - r8.float()).abs().max().item() < 2e-2 * r8.float().abs().max().item()
        assert frac_bad(q8, r8) < 1e-3 and frac_bad(k8, rk8) < 3e-3
    if v_qtype == "int":
        assert frac_bad(v8, rv8.to(torch.float16)) == 0
    else:
        assert frac_bad(v8, rv8.to(torch.float16)) < 1e-3
    assert v8.dtype == torch.float16


def test_operator_boundary():
    """attention_fn installed with types.MethodType like the reference's process_model does."""
    from longcontext_sqattn_paddle_b200.sqattn import process_model
    hq, hkv, n, d = 8, 2, 700, 128

    class Layer:
        num_key_value_groups = hq // hkv

        def prefill_attention(self, q, k, v, mask):
            raise AssertionError("not replaced")

    class Model:
        layers = [Layer(), Layer(), Layer()]

    class Args:
        qk_qtype, v_qtype, use_relative_distance = "int", "int", True

    model = process_model(Model(), "SQAttn", {1: {"bit8": [0.2] * hq, "bit4": [0.4] * hq, "sink": 256}}, Args())
    q, k, v = so.make_inputs(5, 1, n, hq, hkv, d, torch.bfloat16)
    out = model.layers[1].prefill_attention(q.cuda(), k.cuda(), v.cuda(), None)
    assert out.shape == (1, n, hq * d) and out.dtype == torch.bfloat16
    ref = so.attention_fn(q, k, v, hq // hkv, [0.2] * hq, [0.4] * hq, 256)
    assert (out.float().cpu() - ref.float()).abs().max().item() < 2e-2
    with pytest.raises(AssertionError):
        model.layers[0].prefill_attention(q, k, v, None)
    with pytest.raises(ValueError):
        process_model(Model(), "Nope", {}, Args())

    class AbsArgs:
        qk_qtype, v_qtype, use_relative_distance = "int", "int", False

    model = process_model(Model(), "SQAttn", {2: {"bit8": [128] * hq, "bit4": [256] * hq, "sink": 256}}, AbsArgs())
    out = model.layers[2].prefill_attention(q.cuda(), k.cuda(), v.cuda(), None)
    ref = so.attention_fn(q, k, v, hq // hkv, [128] * hq, [256] * hq, 256, use_relative_distance=False)
    assert (out.float().cpu() - ref.float()).abs().max().item() < 2e-2


@pytest.mark.parametrize("n", [1280 + 384, 1700])
def test_host_pipeline_matches_operator(n):
    """Pinned host tensors in, pinned host tensor out, chunked over query rows: bit-identical to the one-shot
    operator (the last chunk is ragged; 1700 tokens: the sequence does not end on a 128-row tile either)."""
    from longcontext_sqattn_paddle_b200.sqattn import HostPrefillPipeline, mp_triton_wrapper
    hq, hkv, d = 8, 2, 128
    q, k, v = so.make_inputs(13, 1, n, hq, hkv, d, torch.bfloat16)

    class Layer:
        num_key_value_groups = hq // hkv

    class Args:
        qk_qtype, v_qtype, use_relative_distance = "int", "int", True

    ref = mp_triton_wrapper(0, [0.2] * hq, [0.4] * hq, 256, Args())(Layer(), q.cuda(), k.cuda(), v.cuda(), None)
    for edge in (512, 128):   # short first and last chunks
        pipe = HostPrefillPipeline([0.2] * hq, [0.4] * hq, 256, Args(), chunk_rows=512, edge_rows=edge)
        assert pipe._bounds(n)[0] == (0, edge) and pipe._bounds(n)[-1][1] == n
        for _ in range(2):   # buffers are reused across calls
            out = pipe(q.pin_memory(), k.pin_memory(), v.pin_memory())
            torch.cuda.synchronize()
            assert out.is_pinned() and torch.equal(out, ref.cpu())
    with pytest.raises(ValueError):
        pipe(q, k, v)   # pageable host memory


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("qtype", ["int", "e4m3", "e5m2"])
def test_q_fake_quant_inside_the_attention_kernel_is_bit_identical(dtype, qtype):
    """The operator hands the raw query to the attention kernel, which fake-quantises and scales every 128-row tile
    in shared memory; the result must be the one obtained from the stand-alone preparation of Q (same device
    functions), for a strided query view of a fused projection, a ragged last tile and a sharded launch."""
    from longcontext_sqattn_paddle_b200 import _lib as L, ops
    hq, hkv, n, d = 8, 2, 1000, 128
    q, k, v = so.make_inputs(17, 1, n, hq, hkv, d, dtype)
    fused = torch.zeros(1, n, (hq + 2 * hkv) * d, dtype=dtype, device="cuda")
    fused[..., :hq * d] = q.cuda().reshape(1, n, hq * d)
    query = fused[..., :hq * d].view(1, n, hq, d)                   # row stride (Hq + 2 Hkv) * D
    q8, _, k8, _, v8 = ops.prep_qkv(query, k.cuda(), v.cuda(), qk_qtype=qtype, skip_bit4=True)
    r8, r4 = [0.2] * hq, [0.4] * hq
    kw = dict(mode=L.MODE_RELATIVE_WINDOW, win8=r8, win4=r4, sink=128, out_dtype=dtype, return_lse=True, p_fp8_mode=L.P_FP8_STAGE2)
    o_ref, lse_ref = ops.prefill(q8, k8, q8, k8, v8, layout="HND", q_is_scaled=True, **kw)
    o, lse = ops.prefill(query, k8, query, k8, v8, layout="NHD", kv_layout="HND", q_fake_quant=qtype, **kw)
    assert torch.equal(o.permute(0, 2, 1, 3), o_ref) and torch.equal(lse, lse_ref)
    # a shard: rows [256, 768) of the sequence
    o, lse = ops.prefill(query[:, 256:768], k8, query[:, 256:768], k8, v8, layout="NHD", kv_layout="HND",
                         q_fake_quant=qtype, q_row_offset=256, **kw)
    assert torch.equal(o.permute(0, 2, 1, 3), o_ref[:, :, 256:768]) and torch.equal(lse, lse_ref[:, :, 256:768])
    with pytest.raises(ValueError):   # two operand sets (absolute windows) keep the stand-alone preparation
        ops.prefill(query, k8, q8.permute(0, 2, 1, 3), k8, v8, layout="NHD", kv_layout="HND", q_fake_quant=qtype, **kw)
    torch.cuda.synchronize()
    ops.check_device_status()
