"""World-size-2 gloo tests of the multi-GPU partitioning logic (dist.py) on CPU ranks.  The collectives, shard
layouts, halo plan, row offsets and the partial/merge protocol are the shipped code; the compute steps are
replaced by a stand-in backend built on the CPU oracle (the CUDA backend needs a GPU).  The sharded result must
match the single-process oracle.  Key/value buffers of the stand-in start as NaN, so a row that the halo
exchange failed to deliver would poison the result."""
import os

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import sqattn_oracle as so


class OracleBackend:
    """dist.CudaBackend's interface on top of the oracle, for CPU ranks."""

    def k_column_sums(self, key):
        return key.float().sum(dim=1)

    def empty_kv(self, total, hkv, d, dtype, like):
        return torch.full((1, total, hkv, d), float("nan"), dtype=dtype)

    def prep_q(self, query, qk_qtype, need_bit4):
        d = query.shape[-1]
        f8, f4, _ = so.make_quantizers(qk_qtype, "int")
        q = query.permute(0, 2, 1, 3)
        q8 = so.scale_q(f8(q, "half_away"), d)
        return q8, (so.scale_q(f4(q, "half_away"), d) if need_bit4 else None)

    def prep_k(self, key, k_mean, qk_qtype, out8, out4):
        f8, f4, _ = so.make_quantizers(qk_qtype, "int")
        k = key.permute(0, 2, 1, 3)
        kc = k - k_mean[:, :, None, :].to(k.dtype)
        out8.copy_(f8(kc, "half_away").permute(0, 2, 1, 3))
        if out4 is not None:
            out4.copy_(f4(kc, "half_away").permute(0, 2, 1, 3))

    def prep_v(self, value, v_qtype, out):
        _, _, fv = so.make_quantizers("int", v_qtype)
        out.copy_(fv(value.permute(0, 2, 1, 3), "half_away").to(torch.float16).permute(0, 2, 1, 3))

    @staticmethod
    def _scatter(x_local, segs, total):
        """local rows [b,h,ns,d] -> rows of the whole sequence (zeros elsewhere)"""
        b, h, _, d = x_local.shape
        full = torch.zeros(b, h, total, d, dtype=x_local.dtype)
        base = 0
        for lo, hi in segs:
            full[:, :, lo:hi] = x_local[:, :, base:base + hi - lo]
            base += hi - lo
        return full

    @staticmethod
    def _gather(o_full, segs):
        return torch.cat([o_full[:, :, lo:hi] for lo, hi in segs], dim=2)

    def windowed_prefill(self, q8, q4, k8, k4, v_full, win8, win4, sink, segs, relative, p_fp8_mode):
        b, hq, ns, d = q8.shape
        total = k8.shape[1]
        bm = 64 if relative else 128
        blocks = [blk for lo, hi in segs for blk in range(lo // bm, (hi + bm - 1) // bm)]
        q8f = self._scatter(q8, segs, total)
        q4f = q8f if q4 is None else self._scatter(q4, segs, total)
        kk8 = k8.permute(0, 2, 1, 3)
        kk4 = kk8 if k4 is None else k4.permute(0, 2, 1, 3)
        o = so.windowed_prefill(q8f, kk8, q4f, kk4, v_full.permute(0, 2, 1, 3), win8, win4, sink,
                                mode="relative" if relative else "absolute", output_dtype=torch.bfloat16, blocks=blocks,
                                q_is_scaled=True, p_fp8_mode={0: "off", 1: "all", 2: "stage2"}[p_fp8_mode])
        return self._gather(o, segs).transpose(1, 2).contiguous().view(b, ns, hq * d)

    def dense_prefill(self, query, k_full, v_full, segs):
        b, ns, hq, d = query.shape
        total = k_full.shape[1]
        qf = self._scatter(query.permute(0, 2, 1, 3), segs, total)
        blocks = [blk for lo, hi in segs for blk in range(lo // 128, (hi + 127) // 128)]
        o = so.dense_causal(qf, k_full.permute(0, 2, 1, 3), v_full.permute(0, 2, 1, 3), output_dtype=query.dtype,
                            blocks=blocks)
        return self._gather(o, segs).transpose(1, 2).contiguous().view(b, ns, hq * d)

    def decode_partial(self, q, k, v, kv_lens, p_fp8):
        b, hq, _, d = q.shape
        po, pl = torch.zeros(b, hq, d), torch.full((b, hq), float("-inf"))
        for i in range(b):
            n = k.shape[2] if kv_lens is None else kv_lens[i]
            if n == 0:
                continue
            o, lse = so.decode(q[i:i + 1], k[i:i + 1, :, :n], v[i:i + 1, :, :n], output_dtype=torch.float32,
                               return_lse=True, is_P_fp8_quant=p_fp8, center_k=False, mask_tail=True)
            po[i], pl[i] = o[0, :, 0], lse[0, :, 0]
        return po, pl

    def merge(self, part_o, part_lse, out_dtype):
        o, _ = so.merge_partials(part_o, part_lse)
        return o.to(out_dtype)


class _Args:
    qk_qtype, v_qtype, use_relative_distance = "int", "int", True


class _ArgsAbs:
    qk_qtype, v_qtype, use_relative_distance = "int", "int", False


class _Layer:
    num_key_value_groups = 2


PREFILL_CASES = {
    # name: (args, win8, win4, sink, layout, exchange)
    "rel_contig_halo": (_Args, [0.25] * 4, [0.5] * 4, 64, "contiguous", "halo"),
    "rel_zigzag_halo": (_Args, [0.25, 0.1, 0.3, 0.2], [0.25, 0.3, 0.3, 0.4], 128, "zigzag", "halo"),
    "rel_balanced_halo": (_Args, [0.125] * 4, [0.125] * 4, 64, "balanced", "halo"),
    "rel_contig_allgather": (_Args, [0.25] * 4, [0.5] * 4, 64, "contiguous", "allgather"),
    "abs_zigzag_halo": (_ArgsAbs, [100, 64, 200, 90], [150, 64, 300, 80], 32, "zigzag", "halo"),
}
N, HQ, HKV, D = 1024, 4, 2, 64


def _rows(x, segs):
    return torch.cat([x[:, lo:hi] for lo, hi in segs], dim=1)


def _worker(rank, world, port, tmp):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from longcontext_sqattn_paddle_b200 import dist as sqdist
        torch.set_num_threads(2)
        q, k, v = so.make_inputs(7, 1, N, HQ, HKV, D, torch.bfloat16)
        be = OracleBackend()
        # ---- sequence-parallel windowed prefill in every layout
        for name, (args, w8, w4, sink, layout, exchange) in PREFILL_CASES.items():
            fn = sqdist.sp_prefill_wrapper(w8, w4, sink, args(), seq_total=N, backend=be, layout=layout, exchange=exchange)
            segs = None
            for _ in range(2):          # the second call reuses the cached layout and buffers
                if segs is None:
                    reach = sqdist._window_reach(sqdist._per_head(w8, HQ, float), sqdist._per_head(w4, HQ, float),
                                                 args.use_relative_distance, N)
                    segs = sqdist._resolve_layout(layout, N, world, reach, sink).segments(rank)
                out = fn(_Layer(), _rows(q, segs), _rows(k, segs), _rows(v, segs), None)
            torch.save((segs, out), os.path.join(tmp, f"prefill_{name}_{rank}.pt"))
        # ---- sequence-parallel dense causal layer
        for layout in ("contiguous", "zigzag"):
            fn = sqdist.sp_dense_wrapper(seq_total=N, backend=be, layout=layout)
            segs = sqdist._resolve_layout(layout, N, world, 0, 0).segments(rank)
            out = fn(_Layer(), _rows(q, segs), _rows(k, segs), _rows(v, segs), None)
            torch.save((segs, out), os.path.join(tmp, f"dense_{layout}_{rank}.pt"))
        # ---- sharded decode (second sequence ends inside rank 0's range: rank 1 holds none of its keys)
        b, L = 2, 640
        g = torch.Generator().manual_seed(3)
        qd = torch.randn(b, HQ, 1, D, generator=g).to(torch.bfloat16)
        kd = torch.randn(b, HKV, L, D, generator=g).to(torch.bfloat16)
        vd = torch.randn(b, HKV, L, D, generator=g).to(torch.bfloat16)
        lens = [640, 200]
        ls = L // world
        mine = [max(0, min(x, (rank + 1) * ls) - rank * ls) for x in lens]
        od = sqdist.sp_decode(qd, kd[:, :, rank * ls:(rank + 1) * ls], vd[:, :, rank * ls:(rank + 1) * ls], kv_lens=mine,
                              backend=be)
        torch.save(od, os.path.join(tmp, f"decode_{rank}.pt"))
    finally:
        dist.destroy_process_group()


def _assemble(tmp_path, stem, world, width):
    full = torch.zeros(1, N, width, dtype=torch.bfloat16)
    seen = torch.zeros(N, dtype=torch.bool)
    for r in range(world):
        segs, out = torch.load(tmp_path / f"{stem}_{r}.pt")
        base = 0
        for lo, hi in segs:
            full[:, lo:hi] = out[:, base:base + hi - lo]
            seen[lo:hi] = True
            base += hi - lo
    assert seen.all()
    return full


def test_world2_sequence_parallel_prefill_and_sharded_decode(tmp_path):
    world, port = 2, 29500 + os.getpid() % 2000
    mp.spawn(_worker, args=(world, port, str(tmp_path)), nprocs=world, join=True)
    q, k, v = so.make_inputs(7, 1, N, HQ, HKV, D, torch.bfloat16)
    for name, (args, w8, w4, sink, _, _) in PREFILL_CASES.items():
        ref = so.attention_fn(q, k, v, HQ // HKV, w8, w4, sink, use_relative_distance=args.use_relative_distance)
        got = _assemble(tmp_path, f"prefill_{name}", world, HQ * D)
        assert torch.isfinite(got.float()).all(), name
        assert (got.float() - ref.float()).abs().max().item() < 2e-2, name
    refd = so.dense_causal(q, k, v, tensor_layout="NHD", output_dtype=torch.bfloat16).reshape(1, N, HQ * D)
    for layout in ("contiguous", "zigzag"):
        got = _assemble(tmp_path, f"dense_{layout}", world, HQ * D)
        assert (got.float() - refd.float()).abs().max().item() < 2e-2, layout
    b, L = 2, 640
    g = torch.Generator().manual_seed(3)
    qd = torch.randn(b, HQ, 1, D, generator=g).to(torch.bfloat16)
    kd = torch.randn(b, HKV, L, D, generator=g).to(torch.bfloat16)
    vd = torch.randn(b, HKV, L, D, generator=g).to(torch.bfloat16)
    refd = so.decode(qd, kd, vd, output_dtype=torch.bfloat16, center_k=False, kv_lens=[640, 200], mask_tail=True)
    for r in range(world):
        od = torch.load(tmp_path / f"decode_{r}.pt")
        assert (od.float() - refd.float()).abs().max().item() < 1e-2


def test_shard_layouts_and_halo_plan():
    from longcontext_sqattn_paddle_b200 import dist as sqdist
    assert sqdist.shard_range(1, 2, 512) == (256, 512)
    assert sqdist.shard_range(0, 1, 300) == (0, 300)
    with pytest.raises(ValueError):
        sqdist.shard_range(0, 3, 512)
    with pytest.raises(ValueError):
        sqdist.shard_range(0, 2, 200)   # 100-row shards: not a multiple of 128
    z = sqdist.ShardLayout.zigzag(4096, 4)
    assert z.segments(0) == [(0, 512), (3584, 4096)] and z.segments(3) == [(1536, 2048), (2048, 2560)]
    assert z.owner_of_last_token() == 0 and all(z.rows(r) == 1024 for r in range(4))
    # dense causal work (key positions visited) is equal across the ranks of a zig-zag split
    work = [sum(hi * (hi + 1) // 2 - lo * (lo + 1) // 2 for lo, hi in z.segments(r)) for r in range(4)]
    assert max(work) - min(work) <= 4096
    with pytest.raises(ValueError):
        sqdist.ShardLayout.zigzag(4096 + 128, 4)
    # balanced contiguous shards: the windowed work per rank is within one 128-row block of equal
    total, world, reach, sink = 131072, 8, 13184, 256
    bal = sqdist.ShardLayout.balanced(total, world, reach, sink)

    def cost(lo, hi):
        return sum(128 * (min(sink, qs) + min(max(qs + 64 - sink, 0), reach) + 64) for qs in range(lo, hi, 128))

    costs = [cost(*bal.segments(r)[0]) for r in range(world)]
    assert bal.rows(0) > bal.rows(world - 1)
    assert max(costs) / (sum(costs) / world) < 1.01
    # halo plan: every rank ends up with the sink and the `reach` rows in front of each of its ranges, nothing is sent twice
    for lay in (sqdist.ShardLayout.contiguous(8192, 4), z, sqdist.ShardLayout.balanced(8192, 4, 1024, 256)):
        for reach, sink in ((1024, 256), (3000, 0), (0, 64)):
            plan = sqdist.halo_plan(lay, reach, sink)
            for dst in range(lay.world):
                have = torch.zeros(lay.total, dtype=torch.int32)
                for lo, hi in lay.segments(dst):
                    have[lo:hi] += 1
                for src, d2, lo, hi in plan:
                    assert src != d2 and any(slo <= lo and hi <= shi for slo, shi in lay.segments(src))
                    if d2 == dst:
                        have[lo:hi] += 1
                assert have.max() <= 1
                for lo, hi in lay.segments(dst):
                    assert have[:min(sink, lay.total)].all() and have[max(0, lo - reach):lo].all()
