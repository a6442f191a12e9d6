"""Window calibration: threshold search on CPU (host logic) and the fused histogram kernel against the dense-map
restatement of the reference."""
import numpy as np
import pytest
import torch

from oracle import window_search_oracle as wo


def test_threshold_search_matches_reference_rules(tmp_path):
    from longcontext_sqattn_paddle_b200.sqattn import window_search as ws
    rng = np.random.default_rng(0)
    for _ in range(20):
        h = rng.random(200) * (rng.random(200) > 0.3)
        for thr in (0.5, 0.9, 0.99, 1.0):
            assert ws.find_optimal_relative_window(h, thr, 200) == wo.find_optimal_relative_window(h, thr, 200)
        h2 = rng.random(1000)
        for thr in (0.5, 0.95):
            assert ws.find_optimal_window(h2, thr) == wo.find_optimal_window(h2, thr)
    assert ws.find_optimal_relative_window(np.zeros(200), 0.9, 200) == 0.1   # the fallback the shipped reference always hits
    assert ws.find_optimal_window(np.zeros(10), 0.9) == 1
    alloc = {1: ws.bits_alloc_entry([{"bit8_relative": 0.1, "bit4_relative": 0.3}] * 4, True)}
    ws.save_bits_alloc(tmp_path / "b.json", alloc)
    assert ws.load_bits_alloc(tmp_path / "b.json") == alloc and alloc[1]["sink"] == 256


@pytest.mark.gpu
@pytest.mark.parametrize("relative,sink", [(True, 64), (True, 256), (False, 0), (False, 32)])
def test_histogram_kernel_matches_dense_map(relative, sink):
    from longcontext_sqattn_paddle_b200.sqattn import window_search as ws
    hq, hkv, n, d, bins = 4, 2, 700, 128, 200
    g = torch.Generator().manual_seed(1)
    q = torch.randn(hq, n, d, generator=g).to(torch.bfloat16)
    k = torch.randn(hkv, n, d, generator=g).to(torch.bfloat16)
    nb = bins if relative else n
    hist = ws.attention_histograms(q.cuda(), k.cuda(), relative=relative, num_bins=nb, sink_len=sink).cpu().numpy()
    a = wo.attention_map(q, k)
    for h in range(hq):
        ref = wo.relative_histogram_with_sink(a[h], bins, sink) if relative else wo.absolute_histogram_with_sink(a[h], n, sink)
        assert np.allclose(hist[h], ref, rtol=2e-3, atol=2e-3 * ref.max())
        for thr in (0.8, 0.95):
            if relative:
                assert abs(ws.find_optimal_relative_window(hist[h], thr, bins) - wo.find_optimal_relative_window(ref, thr, bins)) <= 1.0 / bins
            else:
                assert ws.find_optimal_window(hist[h], thr) == wo.find_optimal_window(ref, thr)

    class Args:
        use_relative_distance, bit8_thres, bit4_thres, relative_bins, sink_window_size = relative, 0.8, 0.95, bins, sink

    b8, b4, windows = ws.calibrate_windows([(q.cuda(), k.cuda())], Args(), max_len=n)
    assert len(windows) == hq and b8 <= b4
