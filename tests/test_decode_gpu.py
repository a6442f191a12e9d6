"""Parity of the split-KV decode kernel with the CPU oracle.  Split-KV restarts the running maximum per key
range and P is rounded to the cache dtype for the tensor-core product, so parity is by tolerance:
max|dO| < 2e-2 (observed ~1e-3), LSE to 2e-3."""
import os

import numpy as np
import pytest
import torch

from oracle import sqattn_oracle as so

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ops():
    from longcontext_sqattn_paddle_b200 import ops
    yield ops
    torch.cuda.synchronize()
    ops.check_device_status()


def _rand(shape, seed, dtype):
    g = torch.Generator().manual_seed(seed)
    return torch.randn(*shape, generator=g).to(dtype)


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("b,hq,hkv,L,d", [(1, 28, 4, 5000, 128), (2, 4, 2, 600, 64), (3, 32, 8, 1, 128),
                                          (1, 8, 1, 64, 128), (2, 16, 1, 20000, 128)])
@pytest.mark.parametrize("fp8", [False, True])
@pytest.mark.parametrize("ref_tail", [True, False])
def test_decode(ops, dtype, b, hq, hkv, L, d, fp8, ref_tail):
    q, k, v = _rand((b, hq, 1, d), 1, dtype), _rand((b, hkv, L, d), 2, dtype), _rand((b, hkv, L, d), 3, dtype)
    o, lse = ops.decode(q.cuda(), k.cuda(), v.cuda(), out_dtype=dtype, return_lse=True, p_fp8=fp8,
                        reference_tail=ref_tail)
    ro, rlse = so.decode(q, k, v, output_dtype=dtype, return_lse=True, is_P_fp8_quant=fp8, center_k=False,
                         mask_tail=not ref_tail)
    assert torch.isfinite(o).all()
    assert (o.float().cpu() - ro.float()).abs().max().item() < 2e-2
    assert (lse.cpu() - rlse).abs().max().item() < 2e-3


def test_decode_full_size_1m_keys(ops):
    """One layer of the 1M-token configuration (28/4 heads, D=128, bf16, 2 x 1 GiB of keys and values): the
    length-aware planner at its largest single-GPU size (about 150 key ranges per KV head).  The tile-by-tile
    oracle needs a quarter of an hour for 16384 tiles, so this size is checked against the exact softmax in fp32
    (what the tiles add up to), with the tolerance of the tiled comparison."""
    dtype = torch.bfloat16
    b, hq, hkv, L, d = 1, 28, 4, 1 << 20, 128
    q, k, v = _rand((b, hq, 1, d), 7, dtype), _rand((b, hkv, L, d), 8, dtype), _rand((b, hkv, L, d), 9, dtype)
    o, lse = ops.decode(q.cuda(), k.cuda(), v.cuda(), out_dtype=dtype, return_lse=True)
    g = hq // hkv
    ro = torch.empty(b, hq, 1, d)
    rlse = torch.empty(b, hq, 1)
    for h in range(hkv):                                  # one KV head at a time: [g, L] scores in fp32
        s2 = (q[0, h * g:(h + 1) * g, 0].float() @ k[0, h].float().T) * (1.0 / d ** 0.5 * 1.44269504)
        m = s2.max(dim=-1, keepdim=True).values
        p = torch.exp2(s2 - m)
        l = p.sum(dim=-1, keepdim=True)
        ro[0, h * g:(h + 1) * g, 0] = (p @ v[0, h].float()) / l
        rlse[0, h * g:(h + 1) * g] = torch.log2(l) + m
    assert torch.isfinite(o).all()
    assert (o.float().cpu() - ro).abs().max().item() < 2e-2
    assert (lse.cpu() - rlse).abs().max().item() < 2e-3


def test_decode_ragged_nhd(ops):
    dtype = torch.bfloat16
    b, hq, hkv, cap, d = 5, 32, 8, 9000, 128
    lens = [9000, 1, 63, 4097, 2500]
    q, k, v = _rand((b, 1, hq, d), 4, dtype), _rand((b, cap, hkv, d), 5, dtype), _rand((b, cap, hkv, d), 6, dtype)
    # poison the unused tail of the cache: it must not leak into the result
    for i, n in enumerate(lens):
        k[i, n:] = float("nan")
        v[i, n:] = float("nan")
    o = ops.decode(q.cuda(), k.cuda(), v.cuda(), layout="NHD", out_dtype=dtype, kv_lens=lens)
    ro = so.decode(q, torch.nan_to_num(k), torch.nan_to_num(v), tensor_layout="NHD", output_dtype=dtype,
                   center_k=False, kv_lens=lens, mask_tail=True)
    assert torch.isfinite(o).all()
    assert (o.float().cpu() - ro.float()).abs().max().item() < 2e-2


def test_decode_partial_and_merge(ops):
    """Two key ranges computed separately (as two GPUs would) and merged equal one call over all keys."""
    dtype = torch.bfloat16
    b, hq, hkv, L, d = 2, 28, 4, 6000, 128
    q, k, v = _rand((b, hq, 1, d), 7, dtype).cuda(), _rand((b, hkv, L, d), 8, dtype).cuda(), _rand((b, hkv, L, d), 9, dtype).cuda()
    full, lse_full = ops.decode(q, k, v, out_dtype=dtype, return_lse=True)
    parts = [ops.decode(q, k[:, :, a:b_], v[:, :, a:b_], partial=True) for a, b_ in ((0, 2500), (2500, L))]
    po = torch.stack([p[0].reshape(b * hq, d) for p in parts])
    pl = torch.stack([p[1].reshape(b * hq) for p in parts])
    merged, lse = ops.decode_merge(po, pl, out_dtype=dtype, return_lse=True)
    assert (merged.view(b, hq, 1, d).float() - full.float()).abs().max().item() < 4e-3
    assert (lse.view(b, hq, 1) - lse_full).abs().max().item() < 1e-3
    ro, rl = so.merge_partials(po.cpu(), pl.cpu())
    assert (merged.float().cpu() - ro).abs().max().item() < 1e-2


@pytest.mark.parametrize("name", ["decode", "decode_large"])
@pytest.mark.parametrize("fp8", [False, True])
def test_decode_reference_golden(golden_dir, name, fp8):
    """attn_unified (K centred per call like the reference) against the reference kernel's own output.
    Bound 8e-3 on O, 3e-2 on LSE (the reference sums q*k products in 16 bits).  Observed on a B200 (max|dO| /
    max|dLSE|): decode (600 keys) 5.2e-4 / 2.5e-4, with P through e4m3 6.8e-3 / 2.5e-4; decode_large (4096 keys,
    64 tiles, 7:1 heads) 3.1e-4 / 1.9e-4, with P through e4m3 3.1e-3 / 1.9e-4."""
    from longcontext_sqattn_paddle_b200.sqattn import attn_unified
    z = np.load(os.path.join(golden_dir, name + ".npz"))
    q, k, v = (torch.from_numpy(z[n]).cuda() for n in ("q", "k", "v"))
    o, lse = attn_unified(q, k, v, "HND", torch.float16, True, fp8)
    go, gl = torch.from_numpy(z["o_fp8" if fp8 else "o"]), torch.from_numpy(z["lse_fp8" if fp8 else "lse"])
    assert (o.float().cpu() - go.float()).abs().max().item() < 8e-3
    assert (lse.cpu() - gl).abs().max().item() < 3e-2


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("fp8", [False, True])
@pytest.mark.parametrize("d", [128, 64])
def test_decode_over_listed_rows_equals_decode_over_packed_copies(dtype, fp8, d):
    """sqattn_decode_args.gather: attending rows of a cache through an index list gives the bits of attending a
    packed copy of those rows (the kernel's arithmetic is the same, only the producer differs); ragged list lengths,
    one of them empty-tailed inside a 64-key tile, caches with different lengths and a strided row layout."""
    from longcontext_sqattn_paddle_b200 import ops
    g = torch.Generator().manual_seed(21)
    b, groups, cap = 5, 4, 1408
    lens_cache = [3000, 777, 5000, 1500, 2048]
    counts = [1408, 300, 1000, 65, 640]
    caches = [(torch.randn(n, 2 * d, generator=g).to(dtype).cuda(), torch.randn(n, 2 * d, generator=g).to(dtype).cuda())
              for n in lens_cache]          # rows 2*d apart: the first d columns are the row
    idx = torch.zeros(b, cap, dtype=torch.int32)
    for i, (n, c) in enumerate(zip(lens_cache, counts)):
        idx[i, :c] = torch.sort(torch.randperm(n, generator=g)[:c]).values.to(torch.int32)
        idx[i, c:] = 2 ** 30                # never read
    idx = idx.cuda()
    cnt = torch.tensor(counts, dtype=torch.int32, device="cuda")
    q = torch.randn(b, groups, 1, d, generator=g).to(dtype).cuda()
    k_rows = torch.tensor([k.data_ptr() for k, _ in caches], dtype=torch.int64, device="cuda")
    v_rows = torch.tensor([v.data_ptr() for _, v in caches], dtype=torch.int64, device="cuda")
    out = ops.decode_gather(q, idx, cnt, k_rows, v_rows, 2 * d, dtype, out_dtype=dtype, p_fp8=fp8)
    k_sel = torch.zeros(b, 1, cap, d, dtype=dtype, device="cuda")
    v_sel = torch.zeros(b, 1, cap, d, dtype=dtype, device="cuda")
    for i, c in enumerate(counts):
        rows = idx[i, :c].long()
        k_sel[i, 0, :c] = caches[i][0][rows, :d]
        v_sel[i, 0, :c] = caches[i][1][rows, :d]
    ref = ops.decode(q, k_sel, v_sel, out_dtype=dtype, p_fp8=fp8, kv_len=cap, kv_lens_device=cnt)
    assert torch.isfinite(out.float()).all()
    assert torch.equal(out, ref)
