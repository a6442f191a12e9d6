"""Clustering kernels against the CPU oracle: assignments, counts, member lists bit-exact; centroids and value
sums bit-exact as well (exact sums, one rounding)."""
import os

import numpy as np
import pytest
import torch

from oracle import kmeans_oracle as ko

pytestmark = pytest.mark.gpu


def _data(g, t, d, seed, dtype):
    gen = torch.Generator().manual_seed(seed)
    x = torch.randn(g, t, d, generator=gen)
    x[..., 5] *= 8
    return x.to(dtype)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("g,t,k,d", [(2, 500, 64, 64), (3, 4096, 96, 128), (1, 1000, 32, 128)])
def test_train_step(dtype, g, t, k, d):
    from longcontext_sqattn_paddle_b200.cache_hub import kmeans as km
    data = _data(g, t, d, 1, dtype)
    cent = data[:, ko.init_centroid_indices(t, k)].contiguous()
    cent[:, 3] = cent[:, 1]  # duplicate centroid: exact ties must go to the lower index
    for norm in (True, False):
        rc, ridx, rcnt = ko.k_means_train(data, cent, norm)
        dc = cent.clone().cuda()
        _, idx, cnt = km.k_means_train(data.cuda(), dc, norm)
        assert torch.equal(idx.cpu(), ridx)
        assert torch.equal(cnt.cpu(), rcnt)
        assert torch.equal(dc.cpu().view(torch.int16), rc.view(torch.int16))
        cent = rc


def test_segment_k_means_full():
    from longcontext_sqattn_paddle_b200.cache_hub import segment_k_means
    g, t, k, d = 4, 8192, 128, 128
    key, val = _data(g, t, d, 2, torch.bfloat16), _data(g, t, d, 3, torch.bfloat16)
    for segs in (1, 4):
        rc, rvs, rcl, rcs, ridx = ko.segment_k_means(key, val, k, 10, segs)
        c, vs, cl, cs, idx = segment_k_means(key.cuda(), val.cuda(), k, 10, segs, return_indices=True)
        assert torch.equal(idx.cpu(), ridx)
        assert torch.equal(cs.cpu(), rcs)
        assert torch.equal(cl.cpu(), rcl)
        assert torch.equal(c.cpu().view(torch.int16), rc.view(torch.int16))
        assert torch.equal(vs.cpu().view(torch.int16), rvs.view(torch.int16))


def test_kmeans_reference_golden(golden_dir):
    from longcontext_sqattn_paddle_b200.cache_hub import kmeans as km
    z = np.load(os.path.join(golden_dir, "kmeans.npz"))
    g = {n: torch.from_numpy(z[n]) for n in z.files}
    cent = g["cent0"].clone().cuda()
    for it, norm in enumerate((True, False)):
        _, idx, cnt = km.k_means_train(g["data"].cuda(), cent, norm)
        assert torch.equal(idx.cpu(), g[f"idx{it}"])
        assert torch.equal(cnt.cpu(), g[f"cnt{it}"])
        cent = g[f"cent{it + 1}"].clone().cuda()
