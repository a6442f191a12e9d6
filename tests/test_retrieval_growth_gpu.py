"""The clustered cache while decoding: appended tokens are attended at once (the unclustered tail), folded into their
clusters every ``fold_every`` tokens, and the same retrieval works when most of K and V live in pinned host memory
(a block-hybrid layout like the reference's CPU-GPU cache).  Assignments, member lists, centroids, value sums and
selected token indices are compared bit for bit with the oracle."""
import pytest
import torch

from oracle import kmeans_oracle as ko
from oracle import sqattn_oracle as so

pytestmark = pytest.mark.gpu


def _data(g, n, d, seed, dtype):
    gen = torch.Generator().manual_seed(seed)
    x = torch.randn(g, n, d, generator=gen)
    x[..., 5] *= 4
    return x.to(dtype)


def _mean_query(q, hkv):
    hq, d = q.shape
    groups = hq // hkv
    qm = torch.zeros(hkv, d)
    for h in range(groups):          # fp32, heads added in order, one division
        qm = qm + q.view(hkv, groups, d)[:, h].float()
    return qm / float(groups)


def test_append_fold_and_tail_selection():
    from longcontext_sqattn_paddle_b200 import ops
    from longcontext_sqattn_paddle_b200.cache_hub import ClusteredKV, RaggedClusteredDecoder
    hq, hkv, d, t0, extra, fold_every, budget = 8, 2, 128, 2048, 300, 256, 512
    dtype = torch.bfloat16
    key, val = _data(hkv, t0 + extra, d, 1, dtype), _data(hkv, t0 + extra, d, 2, dtype)
    cache = ClusteredKV(key[:, :t0].cuda(), val[:, :t0].cuda(), num_iters=4, capacity=t0 + 1024, fold_every=fold_every)
    for t in range(t0, t0 + extra):
        cache.append(key[:, t].cuda(), val[:, t].cuda())
    assert cache.tokens == t0 + extra and cache.clustered == t0 + fold_every
    # oracle: clustering of the first t0 tokens, then one fold of the next fold_every
    cent, _, _, _, assign = ko.segment_k_means(key[:, :t0], val[:, :t0], cache.k, 4, 1)
    n1 = t0 + fold_every
    cent, vsum, clusters, csize, assign = ko.fold_tokens(key[:, :n1], val[:, :n1], assign, cent, t0)
    assert torch.equal(cache.assign[:, :n1].cpu(), assign)
    assert torch.equal(cache.cluster_size.cpu(), csize) and torch.equal(cache.clusters.cpu(), clusters)
    assert torch.equal(cache.centroids.cpu(), cent)
    assert torch.equal(cache.value_sum.cpu(), vsum)
    # retrieval: the oracle's clusters plus every token of the unclustered tail
    gen = torch.Generator().manual_seed(3)
    q = torch.randn(1, hq, 1, d, generator=gen).to(dtype)
    dec = RaggedClusteredDecoder([cache], budget=budget, p_fp8=False)
    out = dec.step(q.cuda()).cpu()
    sel = ko.select_clusters(_mean_query(q[0, :, 0], hkv), cent, csize, clusters, budget)
    tail = torch.arange(n1, t0 + extra, dtype=sel[0].dtype)
    groups = hq // hkv
    for h in range(hkv):
        want = torch.cat([sel[h], tail])
        cnt = int(dec.count[0, h])
        assert cnt == want.numel()
        assert torch.equal(dec.idx[0, h, :cnt].cpu(), want.to(torch.int32))
        kq, vq = key[h, want.long()][None, None], val[h, want.long()][None, None]
        ro = so.decode(q[:, h * groups:(h + 1) * groups], kq, vq, output_dtype=dtype, center_k=False, mask_tail=True)
        assert (out[0, h * groups:(h + 1) * groups].float() - ro[0].float()).abs().max().item() < 2e-2
    # a second fold through the explicit call: the tail empties
    cache.fold()
    assert cache.clustered == cache.tokens
    dec.step(q.cuda())
    torch.cuda.synchronize()
    ops.check_device_status()


def test_hybrid_layout_reads_selected_rows_from_pinned_host_memory():
    from longcontext_sqattn_paddle_b200 import ops
    from longcontext_sqattn_paddle_b200.cache_hub import ClusteredKV, RaggedClusteredDecoder
    hq, hkv, d, dtype = 16, 4, 128, torch.bfloat16
    lens, budget = [5000, 3000], 768
    keys = [_data(hkv, n, d, 10 + i, dtype) for i, n in enumerate(lens)]
    vals = [_data(hkv, n, d, 20 + i, dtype) for i, n in enumerate(lens)]
    on_gpu = [ClusteredKV(k.cuda(), v.cuda(), num_iters=3, capacity=n + 512) for k, v, n in zip(keys, vals, lens)]
    hybrid = [ClusteredKV(k.cuda(), v.cuda(), num_iters=3, capacity=n + 512, split=n // 4) for k, v, n in zip(keys, vals, lens)]
    for c in hybrid:
        assert c.key.shape[1] == c.split and c.key_host.is_pinned()
    gen = torch.Generator().manual_seed(5)
    q = torch.randn(len(lens), hq, 1, d, generator=gen).to(dtype).cuda()
    d_gpu, d_hyb = RaggedClusteredDecoder(on_gpu, budget=budget), RaggedClusteredDecoder(hybrid, budget=budget)
    a, b = d_gpu.step(q), d_hyb.step(q)
    assert torch.equal(d_gpu.count, d_hyb.count) and torch.equal(a, b)
    # growth on both layouts: appended rows land on the host side of the hybrid cache
    for step in range(40):
        for cg, ch, k, v in zip(on_gpu, hybrid, keys, vals):
            kn, vn = torch.roll(k[:, step], 1, dims=-1).cuda(), torch.roll(v[:, step], 1, dims=-1).cuda()
            cg.append(kn, vn)
            ch.append(kn, vn)
    a, b = d_gpu.step(q), d_hyb.step(q)
    assert torch.equal(d_gpu.count, d_hyb.count) and torch.equal(a, b)
    for cg, ch in zip(on_gpu, hybrid):
        cg.fold()
        ch.fold()
        assert torch.equal(cg.clusters, ch.clusters) and torch.equal(cg.centroids, ch.centroids)
    a, b = d_gpu.step(q), d_hyb.step(q)
    assert torch.equal(a, b)
    torch.cuda.synchronize()
    ops.check_device_status()
