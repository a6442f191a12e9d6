"""KV cache on the GPU: reference-compatible cache (device- and pinned-host-resident) and the block-hybrid
cache whose host part is staged by a side stream; decode results against the oracle."""
import pytest
import torch

from oracle import sqattn_oracle as so

pytestmark = pytest.mark.gpu


def _rand(shape, seed, dtype=torch.bfloat16):
    g = torch.Generator().manual_seed(seed)
    return torch.randn(*shape, generator=g).to(dtype)


@pytest.mark.parametrize("force_host", [False, True])
def test_reference_compatible_cache(force_host):
    from longcontext_sqattn_paddle_b200.cache_hub import flash_attn_cache
    layers, b, max_len, hkv, hq, d, n, vs = 2, 1, 700, 2, 8, 128, 600, 10
    cache = flash_attn_cache(vs, layers, b, max_len, hkv, hq, d, torch.bfloat16, force_host=force_host)
    assert cache.allocated == (not force_host)
    ks = [_rand((1, n, hkv, d), 10 + i).cuda() for i in range(layers)]
    vs_ = [_rand((1, n, hkv, d), 20 + i).cuda() for i in range(layers)]
    for i in range(layers):
        k_ret, v_ret = cache.prefill_update_kv_cache(None, ks[i], vs_[i], i, 0)
        assert k_ret.shape[1] == n - vs
    for i in range(layers):
        cache.sync(i)
    cache.move_gpu()
    torch.cuda.synchronize()
    valid = n - vs
    for i in range(layers):
        assert torch.equal(cache.key_cache[i][0, :valid].cpu(), ks[i][0, vs:].cpu())
        assert torch.equal(cache.value_cache[i][0, :valid].cpu(), vs_[i][0, vs:].cpu())
    # one decode step: append a token, attend over valid + 1 keys
    newk, newv = _rand((1, 1, hkv, d), 31).cuda(), _rand((1, 1, hkv, d), 32).cuda()
    q = _rand((1, 1, hq, d), 33).cuda()
    for i in range(layers):
        kc, vc = cache.decode_update_kv_cache(newk, newv, i)
        assert kc.shape == (b, max_len, hkv, d)
    assert int(cache.valid_length[0]) == valid + 1
    o = cache.decode_attention(q, 0, valid + 1)
    kfull = torch.cat([ks[0][:, vs:], newk], dim=1).cpu()
    vfull = torch.cat([vs_[0][:, vs:], newv], dim=1).cpu()
    ro = so.decode(q.cpu(), kfull, vfull, tensor_layout="NHD", output_dtype=torch.bfloat16, center_k=False, mask_tail=True)
    assert (o.float().cpu() - ro.float()).abs().max().item() < 2e-2


@pytest.mark.parametrize("frac", [0.25, 0.0, 1.0])
def test_hybrid_cache_decode(frac):
    from longcontext_sqattn_paddle_b200.cache_hub import HybridKVCache
    layers, b, tokens, hkv, hq, d = 3, 1, 5000, 4, 28, 128
    cache = HybridKVCache(layers, b, tokens, hkv, d, torch.bfloat16, gpu_fraction=frac, block_tokens=512)
    ks = [_rand((b, hkv, tokens, d), 40 + i) for i in range(layers)]
    vs = [_rand((b, hkv, tokens, d), 50 + i) for i in range(layers)]
    for i in range(layers):
        cache.load(i, ks[i], vs[i])
    q = _rand((b, hq, 1, d), 60)
    qc = q.cuda()
    for step in range(2):   # two decode steps: staging buffers are reused across steps
        cache.prefetch(0)
        for i in range(layers):
            o = cache.decode_attention(qc, i)
            ro = so.decode(q, ks[i], vs[i], output_dtype=torch.bfloat16, center_k=False, mask_tail=True)
            assert (o.float().cpu() - ro.float()).abs().max().item() < 2e-2, (step, i)
