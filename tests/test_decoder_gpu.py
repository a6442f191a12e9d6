"""The decoder stand-in (the operator's caller): row kernels against the op-by-op CPU restatement, and the layer
loops of a small random-weight model against the same loops run with the oracle's attention."""
import math
import types

import pytest
import torch

from oracle import decoder_oracle as DO
from oracle import sqattn_oracle as O


def _ulp_bf16(ref: torch.Tensor) -> torch.Tensor:
    return torch.clamp(ref.float().abs(), min=1e-30) * 2.0 ** -7


def test_yarn_table_matches_scalar_restatement():
    from longcontext_sqattn_paddle_b200.model_hub import yarn_cos_sin_cache
    d, base, maxpos, factor = 128, 1e6, 32768, 4.0
    table, scaling = yarn_cos_sin_cache(d, base, 40000, maxpos, factor)
    assert abs(scaling - (0.1 * math.log(4.0) + 1.0)) < 1e-12
    # scalar restatement of model_hub/qwen.py:133-197
    def corr(rot):
        return d * math.log(maxpos / (rot * 2 * math.pi)) / (2 * math.log(base))
    low, high = max(math.floor(corr(32)), 0), min(math.ceil(corr(1)), d - 1)
    for pos in (0, 1, 777, 39999):
        for i in (0, 5, low, (low + high) // 2, high, 63):
            f = base ** (2 * i / d)
            ramp = min(max((i - low) / (high - low), 0.0), 1.0)
            ext = 1 - ramp
            inv = (1 / (factor * f)) * (1 - ext) + (1 / f) * ext
            assert abs(table[pos, i].item() - math.cos(pos * inv) * scaling) < 2e-3 * max(1.0, pos * inv * 1e-3)
            assert abs(table[pos, 64 + i].item() - math.sin(pos * inv) * scaling) < 2e-3 * max(1.0, pos * inv * 1e-3)
    plain, s1 = yarn_cos_sin_cache(d, base, 4096, maxpos, factor)
    assert s1 == 1.0 and abs(plain[3, 1].item() - math.cos(3 / base ** (2 / d))) < 1e-6


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_rmsnorm_matches_op_chain(dtype):
    from longcontext_sqattn_paddle_b200 import ops
    torch.manual_seed(1)
    x = (torch.randn(300, 3584) * 3).to(dtype)
    w = (1 + 0.1 * torch.randn(3584)).to(dtype)
    ref = DO.rmsnorm(x, w, 1e-6)
    buf = torch.zeros(300, 4608, dtype=dtype, device="cuda")
    buf[:, :3584] = x.cuda()
    got = ops.rmsnorm(buf[:, :3584], w.cuda(), 1e-6).cpu()
    # the fp32 mean is accumulated in another order: a row whose variance or rsqrt sits on a rounding boundary
    # moves by one unit in the last place of the 16-bit type; everything else is identical
    ulp = 2.0 ** -7 if dtype == torch.bfloat16 else 2.0 ** -10
    err = (got.float() - ref.float()).abs()
    assert (err <= 2 * ulp * ref.float().abs() + 1e-6).all()
    assert (got == ref).float().mean() > 0.95
    # in place
    ops.rmsnorm(buf[:, :3584], w.cuda(), 1e-6, out=buf[:, :3584])
    assert torch.equal(buf[:, :3584].cpu(), got)


@pytest.mark.gpu
def test_rope_bit_exact():
    from longcontext_sqattn_paddle_b200 import ops
    from longcontext_sqattn_paddle_b200.model_hub import yarn_cos_sin_cache
    torch.manual_seed(2)
    b, s, hq, hkv, d = 2, 200, 6, 2, 128
    table, _ = yarn_cos_sin_cache(d, 1e6, 40000, 32768)
    qkv = torch.randn(b, s, (hq + 2 * hkv) * d).to(torch.bfloat16)
    q, k, v = qkv.split([hq * d, hkv * d, hkv * d], dim=-1)
    pos0 = 33000
    pos = (torch.arange(s) + pos0).unsqueeze(0).repeat(b, 1)
    rq, rk = DO.apply_rope(pos, q, k, d, table)
    dev = qkv.cuda()
    ops.rope_qk(dev.view(b * s, -1), s, hq + hkv, d, table.cuda(), pos0)
    got = dev.cpu()
    assert torch.equal(got[..., :hq * d], rq)
    assert torch.equal(got[..., hq * d:(hq + hkv) * d], rk)
    assert torch.equal(got[..., (hq + hkv) * d:], v)
    with pytest.raises(ValueError):
        ops.rope_qk(dev.view(b * s, -1), s, hq + hkv, d, table.cuda(), 40000 - s + 1)


@pytest.mark.gpu
def test_silu_mul_matches_op_chain():
    from longcontext_sqattn_paddle_b200 import ops
    torch.manual_seed(3)
    x = (torch.randn(257, 2 * 1024) * 2).to(torch.bfloat16)
    ref = DO.silu_and_mul(x)
    got = ops.silu_mul(x.cuda()).cpu()
    err = (got.float() - ref.float()).abs()
    assert (err <= _ulp_bf16(ref) + 1e-30).all()   # exp() differs in its last fp32 bit now and then
    assert (got == ref).float().mean() > 0.99


def _small_model(attention_type="SQAttn", layers=2, seed=5, max_length=1024):
    from longcontext_sqattn_paddle_b200.model_hub import DecoderConfig, RandomInitDecoder
    cfg = DecoderConfig(num_hidden_layers=layers, hidden_size=512, num_attention_heads=4, num_key_value_heads=2,
                        intermediate_size=1024, vocab_size=2048, model_size_b=0)
    return RandomInitDecoder(cfg, max_length=max_length, dtype=torch.bfloat16, device="cuda:0",
                             attention_type=attention_type, seed=seed)


def _weights(layer, eps):
    c = lambda t: t.detach().cpu()
    return DO.LayerWeights(wqkv=c(layer.wqkv), bqkv=c(layer.bqkv), wo=c(layer.wo), gate_up_proj=c(layer.gate_up_proj),
                           down_proj=c(layer.down_proj), input_ln=c(layer.input_layernorm_weight),
                           post_ln=c(layer.post_attention_layernorm_weight), eps=eps)


def _oracle_prefill(model, ids, attention_fn):
    h = torch.nn.functional.embedding(ids.cpu(), model.embed_tokens.cpu())
    table = model.cos_sin_cache.cpu()
    kvs = []
    for layer in model.layers:
        h, k, v = DO.layer_prefill(h, _weights(layer, model.config.rms_norm_eps), table, 0, model.num_heads,
                                   model.num_key_value_heads, model.head_dim, attention_fn)
        kvs.append((k, v))
    last = DO.rmsnorm(h[:, -1:, :], model.norm_weight.cpu(), model.norm_variance_epsilon)
    return torch.nn.functional.linear(last, model.lm_head.cpu()).float(), h, kvs


@pytest.mark.gpu
@pytest.mark.parametrize("method", ["dense", "SQAttn"])
def test_layer_prefill_loop_against_oracle(method):
    from longcontext_sqattn_paddle_b200.sqattn import process_model
    model = _small_model()
    n = 512
    g = torch.Generator().manual_seed(11)
    ids = torch.randint(0, model.vocab_size, (1, n), generator=g)
    if method == "SQAttn":
        args = types.SimpleNamespace(qk_qtype="int", v_qtype="int", use_relative_distance=True)
        windows = {i: {"bit8": [0.25] * 4, "bit4": [0.25] * 4, "sink": 256} for i in range(model.num_layers)}
        process_model(model, "SQAttn", windows, args)

        def attention_fn(q, k, v):
            return O.attention_fn(q, k, v, 2, [0.25] * 4, [0.25] * 4, 256, use_relative_distance=True)
    else:
        def attention_fn(q, k, v):
            b, s, hq, d = q.shape
            return O.dense_causal(q, k, v, tensor_layout="NHD", output_dtype=torch.bfloat16).reshape(b, s, hq * d)
    model.batch_size, model.max_new_length = 1, 4
    model.init_kv_cache(n, (0,))
    logits = model.prefill_forward(ids.cuda()).cpu()
    ref_logits, _, kvs = _oracle_prefill(model, ids, attention_fn)
    # 16-bit matrix products accumulate in another order on the GPU: tolerance, relative to the logit scale
    scale = ref_logits.abs().max().item()
    assert (logits - ref_logits).abs().max().item() < 0.05 * scale
    assert torch.argmax(logits) == torch.argmax(ref_logits) or \
        (ref_logits.flatten().topk(2).values.diff().abs().item() < 0.05 * scale)
    # first-layer keys go through rmsnorm -> projection -> rotation only: tight
    k0 = model.kv_cache.key_cache[0][0, :n].cpu().float()
    assert (k0 - kvs[0][0][0].float()).abs().max().item() < 0.05
    assert model.kv_cache.context == n and model.kv_cache.valid_length_host == [n]


@pytest.mark.gpu
def test_generate_decode_steps_against_oracle():
    model = _small_model(layers=2, seed=9)
    n, new = 300, 4
    g = torch.Generator().manual_seed(12)
    ids = torch.randint(0, model.vocab_size, (1, n), generator=g)
    out = model.generate("SQAttn", ids.cuda(), None, new)
    assert len(out) == 1 and len(out[0]) == new
    assert model.kv_cache.context == n + new - 1 and model.kv_cache.valid_length_host == [n + new - 1]

    # oracle: the same prefill, then one decode step with the token the model chose
    def dense(q, k, v):
        b, s, hq, d = q.shape
        return O.dense_causal(q, k, v, tensor_layout="NHD", output_dtype=torch.bfloat16).reshape(b, s, hq * d)

    def dec(q, k, v):
        return O.decode(q, k, v, tensor_layout="NHD", output_dtype=torch.bfloat16, center_k=False, mask_tail=True)

    ref_logits, h, kvs = _oracle_prefill(model, ids, dense)
    table = model.cos_sin_cache.cpu()
    tok = torch.tensor([[out[0][0]]])
    hd = torch.nn.functional.embedding(tok, model.embed_tokens.cpu())
    for li, layer in enumerate(model.layers):
        kc = torch.zeros(1, n + new, model.num_key_value_heads, model.head_dim, dtype=torch.bfloat16)
        vc = torch.zeros_like(kc)
        kc[:, :n], vc[:, :n] = kvs[li][0], kvs[li][1]
        hd = DO.layer_decode(hd, _weights(layer, model.config.rms_norm_eps), table, n, model.num_heads,
                             model.num_key_value_heads, model.head_dim, kc, vc, n, dec)
    ref = torch.nn.functional.linear(DO.rmsnorm(hd, model.norm_weight.cpu(), 1e-6), model.lm_head.cpu()).float()
    # re-run the model's first decode step from a fresh cache to read its logits
    model2 = _small_model(layers=2, seed=9)
    model2.batch_size, model2.max_new_length = 1, new
    model2.init_kv_cache(n, (0,))
    model2.prefill_forward(ids.cuda())
    model2.move()
    got = model2.decode_forward(tok.cuda()).cpu()
    scale = ref.abs().max().item()
    assert (got - ref).abs().max().item() < 0.05 * scale


@pytest.mark.gpu
def test_rope_with_device_position_matches_host_position():
    from longcontext_sqattn_paddle_b200 import ops
    from longcontext_sqattn_paddle_b200.model_hub import yarn_cos_sin_cache
    torch.manual_seed(4)
    table, _ = yarn_cos_sin_cache(128, 1e6, 5000, 32768)
    table = table.cuda()
    x = torch.randn(3, 6 * 128).to(torch.bfloat16).cuda()
    a, b = x.clone(), x.clone()
    ops.rope_qk(a, 1, 4, 128, table, 777)
    ops.rope_qk(b, 1, 4, 128, table, 0, pos_device=torch.tensor([777], dtype=torch.int64, device="cuda"))
    assert torch.equal(a, b)


@pytest.mark.gpu
def test_decode_with_device_lengths_matches_host_lengths():
    from longcontext_sqattn_paddle_b200 import ops
    torch.manual_seed(6)
    b, hq, hkv, cap, d = 3, 8, 2, 5000, 128
    q = torch.randn(b, 1, hq, d).to(torch.bfloat16).cuda()
    k = torch.randn(b, cap, hkv, d).to(torch.bfloat16).cuda()
    v = torch.randn(b, cap, hkv, d).to(torch.bfloat16).cuda()
    lens = [4999, 130, 2048]
    ref = ops.decode(q, k, v, layout="NHD", out_dtype=torch.bfloat16, kv_lens=lens)
    dev = torch.tensor(lens, dtype=torch.int32, device="cuda")
    got = ops.decode(q, k, v, layout="NHD", out_dtype=torch.bfloat16, kv_len=cap, kv_lens_device=dev)
    # the key ranges are planned for the capacity instead of the lengths: other split points, same attention
    assert (got.float() - ref.float()).abs().max().item() < 8e-3
    with pytest.raises(ValueError):
        ops.decode(q, k, v, layout="NHD", kv_lens=lens, kv_lens_device=dev)


@pytest.mark.gpu
def test_captured_decode_step_follows_the_eager_one():
    n, new = 300, 6
    g = torch.Generator().manual_seed(13)
    eager, graphed = _small_model(layers=2, seed=3), _small_model(layers=2, seed=3)
    ids = torch.randint(0, eager.vocab_size, (1, n), generator=g).cuda()
    for m in (eager, graphed):
        m.batch_size, m.max_new_length = 1, new + 2
        m.init_kv_cache(n, (0,))
        m.prefill_forward(ids)
        m.move()
    graphed.capture_decode_step(1)
    tok = torch.tensor([[5]], device="cuda")
    for step in range(new):
        le = eager.decode_forward(tok)
        lg = graphed.decode_forward_graph(tok)
        scale = le.abs().max().item()
        assert (le - lg).abs().max().item() < 0.03 * scale, f"step {step}"
        tok = le.argmax(dim=-1)
    torch.cuda.synchronize()
    assert graphed.kv_cache.context == eager.kv_cache.context == n + new
    assert graphed.kv_cache.valid_length_host == eager.kv_cache.valid_length_host
    assert torch.equal(graphed.kv_cache.valid_length, eager.kv_cache.valid_length)
    # the caches hold the same rows: the graph wrote each new key where the eager step did
    ke, kg = eager.kv_cache.key_cache[1][0, :n + new].float(), graphed.kv_cache.key_cache[1][0, :n + new].float()
    assert (ke - kg).abs().max().item() < 0.05
