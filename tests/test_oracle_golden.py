"""Pin the CPU oracle against vectors produced by running the reference's own code (tests/golden/make_golden.py):
its Triton kernels on Triton's interpreter and its Python glue (quantisers, adapter + launchers, window search,
segment_k_means) through a paddle-to-torch forwarder.  Tolerances: the interpreter and the oracle accumulate dot
products in different orders, so attention outputs agree to fp16 rounding (atol 2e-3 on O, 2e-3 on LSE); with FP8
rounding of P a rounding decision may flip for a few elements, which the looser bound covers.  Quantiser outputs,
window choices, kmeans assignments, counts and member lists are exact."""
import os

import numpy as np
import pytest
import torch

from oracle import kmeans_oracle as ko
from oracle import sqattn_oracle as so


def _load(golden_dir, name):
    z = np.load(os.path.join(golden_dir, name + ".npz"))
    def scalar(a):
        return int(a) if np.issubdtype(a.dtype, np.integer) else float(a)

    return {k: (torch.from_numpy(z[k]) if z[k].shape != () else scalar(z[k])) for k in z.files}


def _check(o, lse, go, glse, atol_o, atol_lse=2e-3):
    assert o.dtype == go.dtype
    assert (o.float() - go.float()).abs().max().item() <= atol_o
    assert (lse - glse).abs().max().item() <= atol_lse


@pytest.mark.parametrize("fp8", [False, True])
def test_relative_window_kernel(golden_dir, fp8):
    g = _load(golden_dir, "relative")
    o, lse = so.windowed_prefill(g["q"], g["k"], g["q"], g["k"], g["v"], g["r8"], g["r4"], g["sink"],
                                 mode="relative", output_dtype=torch.float16, return_lse=True,
                                 is_P_fp8_quant=fp8)
    _check(o, lse, g["o_fp8" if fp8 else "o"], g["lse_fp8" if fp8 else "lse"], 4e-3 if fp8 else 2e-3)


@pytest.mark.parametrize("fp8", [False, True])
def test_absolute_window_kernel(golden_dir, fp8):
    g = _load(golden_dir, "absolute")
    o, lse = so.windowed_prefill(g["q8"], g["k8"], g["q4"], g["k4"], g["v"], g["w8"], g["w4"], g["sink"],
                                 mode="absolute", output_dtype=torch.float16, return_lse=True,
                                 is_P_fp8_quant=fp8)
    _check(o, lse, g["o_fp8" if fp8 else "o"], g["lse_fp8" if fp8 else "lse"], 4e-3 if fp8 else 2e-3)


@pytest.mark.parametrize("fp8", [False, True])
def test_dense_causal_kernel(golden_dir, fp8):
    g = _load(golden_dir, "dense")
    o, lse = so.dense_causal(g["q"], g["k"], g["v"], output_dtype=torch.float16, return_lse=True,
                             is_P_fp8_quant=fp8)
    _check(o, lse, g["o_fp8" if fp8 else "o"], g["lse_fp8" if fp8 else "lse"], 4e-3 if fp8 else 2e-3)


@pytest.mark.parametrize("fp8", [False, True])
def test_decode_kernel(golden_dir, fp8):
    g = _load(golden_dir, "decode")
    o, lse = so.decode(g["q"], g["k"], g["v"], output_dtype=torch.float16, return_lse=True,
                       is_P_fp8_quant=fp8, center_k=True, qk_in_input_dtype=True)
    # the reference sums q*k products in 16-bit (tl.sum keeps the input dtype), the oracle in fp32
    _check(o, lse, g["o_fp8" if fp8 else "o"], g["lse_fp8" if fp8 else "lse"], 6e-3, 3e-2)


def test_kmeans_assign_update(golden_dir):
    g = _load(golden_dir, "kmeans")
    cent = g["cent0"]
    for it, norm in enumerate((True, False)):
        new, idx, cnt = ko.k_means_train(g["data"], cent, norm)
        assert torch.equal(idx, g[f"idx{it}"])
        assert torch.equal(cnt, g[f"cnt{it}"])
        s, _ = ko.cluster_sums(g["data"], idx, cent.shape[1])
        assert torch.allclose(s, g[f"sum{it}"], atol=1e-4, rtol=1e-5)
        # centroids are fp16: allow one ulp where the fp32 value sits on a rounding boundary
        diff = (new.float() - g[f"cent{it + 1}"].float()).abs()
        assert (diff <= 2e-3 * g[f"cent{it + 1}"].float().abs().clamp(min=0.1)).all()
        cent = g[f"cent{it + 1}"]


@pytest.mark.parametrize("fp8", [False, True])
def test_relative_window_kernel_large(golden_dir, fp8):
    """head_dim 128, 1024 tokens, sink 256, seven query heads on one KV head, per-head ratios, an outlier K channel"""
    g = _load(golden_dir, "relative_large")
    o, lse = so.windowed_prefill(g["q"], g["k"], g["q"], g["k"], g["v"], g["r8"], g["r4"], g["sink"],
                                 mode="relative", output_dtype=torch.float16, return_lse=True, is_P_fp8_quant=fp8)
    _check(o, lse, g["o_fp8" if fp8 else "o"], g["lse_fp8" if fp8 else "lse"], 4e-3 if fp8 else 2e-3)


@pytest.mark.parametrize("fp8", [False, True])
def test_decode_kernel_large(golden_dir, fp8):
    """4096 keys (64 tiles), head_dim 128, seven query heads on one KV head"""
    g = _load(golden_dir, "decode_large")
    o, lse = so.decode(g["q"], g["k"], g["v"], output_dtype=torch.float16, return_lse=True,
                       is_P_fp8_quant=fp8, center_k=True, qk_in_input_dtype=True)
    _check(o, lse, g["o_fp8" if fp8 else "o"], g["lse_fp8" if fp8 else "lse"], 6e-3, 3e-2)


def _golden16(g, name, dname):
    return g[f"{name}_f16"] if dname == "f16" else g[f"{name}_bf16bits"].view(torch.bfloat16)


@pytest.mark.parametrize("dname", ["f16", "bf16"])
def test_fake_quantisers_match_the_reference_classes(golden_dir, dname):
    """IntegerQuantizer / FloatQuantizer as the adapter builds them (sqattn/fake_quant.py, attn_replacer.py:340-358):
    every output value is identical (the reference produces -0.0 where the oracle has +0.0, hence values, not bits)."""
    g = _load(golden_dir, "fake_quant")
    x = _golden16(g, "x", dname)
    cases = {
        "int8_token": lambda t: so.int_fake_quant(t, 8, "per_token"),
        "int4_token": lambda t: so.int_fake_quant(t, 4, "per_token"),
        "int8_channel": lambda t: so.int_fake_quant(t, 8, "per_channel"),
        "e4m3_token": lambda t: so.float_fake_quant(t, "e4m3", "per_token"),
        "e5m2_token": lambda t: so.float_fake_quant(t, "e5m2", "per_token"),
        "e4m3_channel": lambda t: so.float_fake_quant(t, "e4m3", "per_channel"),
        "e5m2_channel": lambda t: so.float_fake_quant(t, "e5m2", "per_channel"),
    }
    for name, fn in cases.items():
        y, ref = fn(x), _golden16(g, name, dname)
        assert y.dtype == ref.dtype
        assert torch.equal(y.float(), ref.float()), name
    # ties-to-even rounding (the switch the oracle keeps for the other reading of paddle.round) does differ on this data
    assert dname != "f16" or not torch.equal(so.int_fake_quant(x, 8, "per_token", True, "half_even").float(), _golden16(g, "int8_token", dname).float())


@pytest.mark.parametrize("case", ["rel_int", "rel_e4m3", "abs_int", "abs_e5m2"])
def test_adapter_end_to_end(golden_dir, case):
    """mp_triton_wrapper(...).attention_fn of the reference (repeat_kv, K centring, five fake-quants, launcher, output
    transpose), fp16 in, output rounded to fp16 (the fixture generator's stand-in for the launcher's bf16)."""
    g = _load(golden_dir, "adapter")
    rel = case.startswith("rel")
    qk = {"rel_int": "int", "rel_e4m3": "e4m3", "abs_int": "int", "abs_e5m2": "e5m2"}[case]
    vq = "e4m3" if case == "rel_e4m3" else "int"
    w8, w4 = g[f"w8_{case}"], g[f"w4_{case}"]
    if rel:
        w8, w4 = [float(x) for x in w8], [float(x) for x in w4]
    else:
        w8, w4 = int(w8), int(w4)
    o = so.attention_fn(g["q"], g["k"], g["v"], 2, w8, w4, g["sink"], use_relative_distance=rel, qk_qtype=qk, v_qtype=vq,
                        output_dtype=torch.float16)
    ref = g[f"o_{case}"]
    assert o.shape == ref.shape and o.dtype == ref.dtype
    err = (o.float() - ref.float()).abs()
    # a handful of 8-bit codes of K may differ by one step where the fp32 sequence mean rounds differently
    assert err.max().item() <= 4e-3, err.max().item()
    assert (err > 2e-3).float().mean().item() < 1e-3


def test_window_search_functions(golden_dir):
    """cal_attn_weight, the four histogram functions and the two threshold searches of sqattn/window_search.py"""
    from oracle import window_search_oracle as wo
    g = _load(golden_dir, "window_search")
    q, k = g["q"][0].permute(1, 0, 2), g["k"][0].permute(1, 0, 2)            # [H, N, D]
    amap = wo.attention_map(q, k)
    assert (amap.float() - g["attn"][0]).abs().max().item() < 1e-6
    thr = g["thresholds"].tolist()
    for h in range(q.shape[0]):
        a = g["attn"][0, h]            # histograms of the reference's own fp32 map
        for mine, ref in ((wo.relative_histogram_with_sink(a, 200, 64), g[f"rel_hist_{h}"]),
                          (wo.absolute_histogram_with_sink(a, a.shape[0], 64), g[f"abs_hist_{h}"]),
                          (wo.absolute_histogram_with_sink(a, a.shape[0], 0), g[f"abs_hist_nosink_{h}"])):
            ref = ref.double().numpy()
            assert mine.shape == ref.shape
            assert np.allclose(mine, ref, rtol=1e-4, atol=1e-5)
        for i, t in enumerate(thr):
            assert wo.find_optimal_relative_window(g[f"rel_hist_{h}"].numpy(), t, 200) == float(g["rel_windows"][h, i])
            assert wo.find_optimal_window(g[f"abs_hist_{h}"].numpy(), t) == int(g["abs_windows"][h, i])
    assert wo.find_optimal_relative_window(np.zeros(200), 0.9, 200) == float(g["rel_window_empty"])
    assert wo.find_optimal_window(np.zeros(300), 0.9) == int(g["abs_window_empty"])


@pytest.mark.parametrize("segments", [1, 2])
def test_segment_k_means_whole(golden_dir, segments):
    """segment_k_means of cache_hub/kmeans.py:332-375 run as a whole by the reference's code: centroid initialisation,
    segmenting, Lloyd iterations, value sums and member lists (compared sorted: arrival order is unspecified)."""
    g = _load(golden_dir, "segment_kmeans")
    cent, vsum, clusters, csize, _ = ko.segment_k_means(g["key"], g["value"], 64, num_iters=4, num_segments=segments)
    assert torch.equal(csize, g[f"cluster_size_{segments}"])
    ref_clusters = g[f"clusters_{segments}"]
    assert clusters.shape == ref_clusters.shape
    srt = torch.zeros_like(clusters)
    for gi in range(clusters.shape[0]):
        for c in range(clusters.shape[1]):
            m = int(csize[gi, c])
            srt[gi, c, :m] = torch.sort(clusters[gi, c, :m]).values
    assert torch.equal(srt, ref_clusters)
    for mine, ref in ((cent, g[f"centroids_{segments}"]), (vsum, g[f"value_sum_{segments}"])):
        assert mine.dtype == ref.dtype
        diff = (mine.float() - ref.float()).abs()
        assert (diff <= 2e-3 * ref.float().abs().clamp(min=0.1)).all()   # fp16 values: one ulp at a rounding boundary
