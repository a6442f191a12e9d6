"""Pin the CPU oracle against vectors produced by the reference's own Triton
kernels (tests/golden/make_golden.py).  Tolerances: the interpreter and the
oracle accumulate dot products in different orders, so outputs agree to fp16
rounding (atol 2e-3 on O, 2e-3 on LSE); with FP8 rounding of P a rounding
decision may flip for a few elements, which the looser bound covers."""
import os

import numpy as np
import pytest
import torch

from oracle import kmeans_oracle as ko
from oracle import sqattn_oracle as so


def _load(golden_dir, name):
    z = np.load(os.path.join(golden_dir, name + ".npz"))
    return {k: (torch.from_numpy(z[k]) if z[k].shape != () else int(z[k])) for k in z.files}


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
