"""Sequence-parallel prefill and cross-GPU split-KV decode.  The two-rank run (windowed prefill in every shard layout,
dense causal layers, decode through the NCCL and the peer-store exchange) needs two GPUs and is skipped on a
single-GPU box; what a rank computes for its shard (one launch over one or two row ranges of the sequence against
K/V of the whole sequence) is checked on one GPU as well, and the partitioning logic by the gloo tests on CPU."""
import os

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import sqattn_oracle as so

pytestmark = pytest.mark.gpu


class _Args:
    qk_qtype, v_qtype, use_relative_distance = "int", "int", True


class _Layer:
    num_key_value_groups = 7


class _ArgsAbs:
    qk_qtype, v_qtype, use_relative_distance = "int", "int", False


def _cases(hq):
    return {
        "rel_contig_halo": (_Args, [0.1] * hq, [0.3] * hq, 256, "contiguous", "halo"),
        "rel_zigzag_halo": (_Args, [0.1 + 0.01 * h for h in range(hq)], [0.3] * hq, 128, "zigzag", "halo"),
        "rel_balanced_halo": (_Args, [0.125] * hq, [0.125] * hq, 256, "balanced", "halo"),
        "rel_contig_allgather": (_Args, [0.1] * hq, [0.3] * hq, 256, "contiguous", "allgather"),
        "abs_zigzag_halo": (_ArgsAbs, [100 + 8 * h for h in range(hq)], [300] * hq, 32, "zigzag", "halo"),
    }


def _rows(x, segs):
    return torch.cat([x[:, lo:hi] for lo, hi in segs], dim=1)


def _assemble(tmp_path, stem, world, n, width):
    full = torch.zeros(1, n, width, dtype=torch.bfloat16)
    for r in range(world):
        segs, out = torch.load(tmp_path / f"{stem}_{r}.pt")
        base = 0
        for lo, hi in segs:
            full[:, lo:hi] = out[:, base:base + hi - lo]
            base += hi - lo
    return full


def _worker(rank, world, port, tmp):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        from longcontext_sqattn_paddle_b200 import dist as sqdist, ops
        n, hq, hkv, d = 2048, 28, 4, 128
        q, k, v = so.make_inputs(21, 1, n, hq, hkv, d, torch.bfloat16)
        for name, (args, w8, w4, sink, layout, exchange) in _cases(hq).items():
            fn = sqdist.sp_prefill_wrapper(w8, w4, sink, args(), seq_total=n, layout=layout, exchange=exchange)
            reach = sqdist._window_reach(w8, w4, args.use_relative_distance, n)
            segs = sqdist._resolve_layout(layout, n, world, reach, sink).segments(rank)
            for _ in range(2):
                out = fn(_Layer(), _rows(q, segs).cuda(), _rows(k, segs).cuda(), _rows(v, segs).cuda(), None)
            torch.save((segs, out.cpu()), os.path.join(tmp, f"prefill_{name}_{rank}.pt"))
        # the same operator fed from pinned host buffers, chunked and overlapped: identical rows
        for layout in ("balanced", "zigzag"):
            w8, w4, sink = [0.125] * hq, [0.25] * hq, 128
            reach = sqdist._window_reach(w8, w4, True, n)
            segs = sqdist._resolve_layout(layout, n, world, reach, sink).segments(rank)
            ref = sqdist.sp_prefill_wrapper(w8, w4, sink, _Args(), seq_total=n, layout=layout)(
                _Layer(), _rows(q, segs).cuda(), _rows(k, segs).cuda(), _rows(v, segs).cuda(), None)
            pipe = sqdist.SPHostPrefillPipeline(w8, w4, sink, _Args(), seq_total=n, layout=layout, chunk_rows=256, edge_rows=128)
            hout = torch.empty(ref.shape, dtype=ref.dtype).pin_memory()
            for _ in range(2):
                pipe(_rows(q, segs).pin_memory(), _rows(k, segs).pin_memory(), _rows(v, segs).pin_memory(), hout)
                torch.cuda.synchronize()
                assert torch.equal(hout, ref.cpu()), layout
        for layout in ("contiguous", "zigzag"):
            fn = sqdist.sp_dense_wrapper(seq_total=n, layout=layout)
            segs = sqdist._resolve_layout(layout, n, world, 0, 0).segments(rank)
            out = fn(_Layer(), _rows(q, segs).cuda(), _rows(k, segs).cuda(), _rows(v, segs).cuda(), None)
            torch.save((segs, out.cpu()), os.path.join(tmp, f"dense_{layout}_{rank}.pt"))
        g = torch.Generator().manual_seed(5)
        b, L = 2, 4096
        qd = torch.randn(b, hq, 1, d, generator=g).to(torch.bfloat16)
        kd = torch.randn(b, hkv, L, d, generator=g).to(torch.bfloat16)
        vd = torch.randn(b, hkv, L, d, generator=g).to(torch.bfloat16)
        lens = [4096, 1500]
        ls = L // world
        mine = [max(0, min(x, (rank + 1) * ls) - rank * ls) for x in lens]
        od = sqdist.sp_decode(qd.cuda(), kd[:, :, rank * ls:(rank + 1) * ls].contiguous().cuda(),
                              vd[:, :, rank * ls:(rank + 1) * ls].contiguous().cuda(), kv_lens=mine)
        torch.cuda.synchronize()
        ops.check_device_status()
        torch.save(od.cpu(), os.path.join(tmp, f"decode_{rank}.pt"))
        # the same decode with the partials exchanged by peer stores inside one merge kernel; five steps with
        # different queries so that both buffer parities and growing epochs are used
        ex = sqdist.PeerExchange(rows_cap=b * hq, head_dim=d)
        outs = []
        for step in range(5):
            qs = (qd.float() * (1.0 + 0.25 * step)).to(torch.bfloat16).cuda()
            kk = kd[:, :, rank * ls:(rank + 1) * ls].contiguous().cuda()
            vv = vd[:, :, rank * ls:(rank + 1) * ls].contiguous().cuda()
            a = sqdist.sp_decode(qs, kk, vv, kv_lens=mine, exchange=ex)
            n_ = sqdist.sp_decode(qs, kk, vv, kv_lens=mine)
            outs.append((a.float() - n_.float()).abs().max().item())
        # the stand-alone exchange entry point on partials computed by a separate call
        po, pl = ops.decode(qs, kk, vv, partial=True, kv_lens=mine)
        m = ex.merge(po.reshape(b * hq, d), pl.reshape(b * hq)).view(b, hq, 1, d)
        outs.append((m.float() - n_.float()).abs().max().item())
        torch.cuda.synchronize()
        ops.check_device_status()
        torch.save(torch.tensor(outs), os.path.join(tmp, f"peer_{rank}.pt"))
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_two_gpu_prefill_and_decode(tmp_path):
    world, port = 2, 29600 + os.getpid() % 2000
    mp.spawn(_worker, args=(world, port, str(tmp_path)), nprocs=world, join=True)
    n, hq, hkv, d = 2048, 28, 4, 128
    q, k, v = so.make_inputs(21, 1, n, hq, hkv, d, torch.bfloat16)
    for name, (args, w8, w4, sink, _, _) in _cases(hq).items():
        ref = so.attention_fn(q, k, v, hq // hkv, w8, w4, sink, use_relative_distance=args.use_relative_distance)
        got = _assemble(tmp_path, f"prefill_{name}", world, n, hq * d)
        assert (got.float() - ref.float()).abs().max().item() < 2e-2, name
    refd = so.dense_causal(q, k, v, tensor_layout="NHD", output_dtype=torch.bfloat16).reshape(1, n, hq * d)
    for layout in ("contiguous", "zigzag"):
        got = _assemble(tmp_path, f"dense_{layout}", world, n, hq * d)
        assert (got.float() - refd.float()).abs().max().item() < 2e-2, layout
    g = torch.Generator().manual_seed(5)
    b, L = 2, 4096
    qd = torch.randn(b, hq, 1, d, generator=g).to(torch.bfloat16)
    kd = torch.randn(b, hkv, L, d, generator=g).to(torch.bfloat16)
    vd = torch.randn(b, hkv, L, d, generator=g).to(torch.bfloat16)
    refd = so.decode(qd, kd, vd, output_dtype=torch.bfloat16, center_k=False, kv_lens=[4096, 1500], mask_tail=True)
    for r in range(world):
        assert (torch.load(tmp_path / f"decode_{r}.pt").float() - refd.float()).abs().max().item() < 2e-2
        # peer-store exchange against the NCCL exchange: the same partials merged in another order, so the
        # difference is at most one unit in the last place of the 16-bit output
        assert torch.load(tmp_path / f"peer_{r}.pt").max().item() < 8e-3


@pytest.mark.parametrize("mode", ["relative", "absolute", "dense"])
def test_one_rank_of_a_zigzag_split_on_one_gpu(mode):
    """What rank 1 of 4 computes: its two row ranges (chunks 1 and 6 of 8) in ONE launch against K/V of the whole
    sequence, compared with the oracle's rows for the same blocks."""
    from longcontext_sqattn_paddle_b200 import _lib as L, dist as sqdist, ops
    n, hq, hkv, d, dtype = 2048, 4, 2, 128, torch.bfloat16
    g = torch.Generator().manual_seed(31)
    q = torch.randn(1, hq, n, d, generator=g).to(dtype)
    k = torch.randn(1, hkv, n, d, generator=g).to(dtype)
    v = torch.randn(1, hkv, n, d, generator=g).to(dtype)
    segs = sqdist.ShardLayout.zigzag(n, 4).segments(1)
    assert segs == [(256, 512), (1536, 1792)]
    q_loc = torch.cat([q[:, :, lo:hi] for lo, hi in segs], dim=2).cuda()
    kw = dict(q_row_offset=segs[0][0], q_split_rows=segs[0][1] - segs[0][0], q_row_offset2=segs[1][0], out_dtype=dtype,
              return_lse=True)
    if mode == "dense":
        o, lse = ops.prefill(q_loc, k.cuda(), q_loc, k.cuda(), v.cuda(), mode=L.MODE_DENSE_CAUSAL, **kw)
        ro, rlse = so.dense_causal(q, k, v, output_dtype=dtype, return_lse=True)
    elif mode == "relative":
        r8, r4 = [0.2, 0.1, 0.3, 0.5], [0.4, 0.1, 0.3, 0.6]
        o, lse = ops.prefill(q_loc, k.cuda(), q_loc, k.cuda(), v.cuda(), mode=L.MODE_RELATIVE_WINDOW, win8=r8, win4=r4,
                             sink=64, p_fp8_mode=L.P_FP8_STAGE2, **kw)
        ro, rlse = so.windowed_prefill(q, k, q, k, v, r8, r4, 64, mode="relative", output_dtype=dtype, return_lse=True,
                                       p_fp8_mode="stage2")
    else:
        s8, s4 = [100, 200, 64, 300], [150, 200, 500, 100]
        o, lse = ops.prefill(q_loc, k.cuda(), q_loc, k.cuda(), v.cuda(), mode=L.MODE_ABSOLUTE_WINDOW, win8=s8, win4=s4,
                             sink=32, **kw)
        ro, rlse = so.windowed_prefill(q, k, q, k, v, s8, s4, 32, mode="absolute", output_dtype=dtype, return_lse=True)
    torch.cuda.synchronize()
    ops.check_device_status()
    ro = torch.cat([ro[:, :, lo:hi] for lo, hi in segs], dim=2)
    rlse = torch.cat([rlse[:, :, lo:hi] for lo, hi in segs], dim=2)
    assert (o.float().cpu() - ro.float()).abs().max().item() < 2e-2
    assert (lse.cpu() - rlse).abs().max().item() < 2e-3
