"""World-size-2 gloo tests of the multi-GPU partitioning logic (dist.py) on CPU ranks.  The collectives, shard
ranges, row offsets and the partial/merge protocol are the shipped code; the compute steps are replaced by a
stand-in backend built on the CPU oracle (the CUDA backend needs a GPU).  The sharded result must match the
single-process oracle."""
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

    def prep(self, query, key, value, k_mean, qk_qtype, v_qtype):
        d = query.shape[-1]
        q = query.permute(0, 2, 1, 3)
        k = key.permute(0, 2, 1, 3)
        v = value.permute(0, 2, 1, 3)
        kc = k - k_mean[:, :, None, :].to(k.dtype)
        f8, _, fv = so.make_quantizers(qk_qtype, v_qtype)
        q8 = so.scale_q(f8(q, "half_away"), d)
        k8 = f8(kc, "half_away").permute(0, 2, 1, 3).contiguous()
        v8 = fv(v, "half_away").to(torch.float16).permute(0, 2, 1, 3).contiguous()
        return q8, k8, v8

    def windowed_prefill(self, q8, k_full, v_full, win8, win4, sink, q_row_offset, p_fp8_mode):
        b, hq, ns, d = q8.shape
        total = k_full.shape[1]
        qfull = torch.zeros(b, hq, total, d, dtype=q8.dtype)
        qfull[:, :, q_row_offset:q_row_offset + ns] = q8
        k = k_full.permute(0, 2, 1, 3)
        v = v_full.permute(0, 2, 1, 3)
        blocks = range(q_row_offset // 64, (q_row_offset + ns) // 64)
        o = so.windowed_prefill(qfull, k, qfull, k, v, win8, win4, sink, mode="relative", output_dtype=torch.bfloat16,
                                blocks=blocks, q_is_scaled=True, p_fp8_mode={0: "off", 1: "all", 2: "stage2"}[p_fp8_mode])
        o = o[:, :, q_row_offset:q_row_offset + ns]
        return o.transpose(1, 2).contiguous().view(b, ns, hq * d)

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


class _Layer:
    num_key_value_groups = 2


def _worker(rank, world, port, tmp):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from longcontext_sqattn_paddle_b200 import dist as sqdist
        torch.set_num_threads(2)
        # ---- sequence-parallel prefill
        n, hq, hkv, d = 512, 4, 2, 64
        q, k, v = so.make_inputs(7, 1, n, hq, hkv, d, torch.bfloat16)
        lo, hi = sqdist.shard_range(rank, world, n)
        fn = sqdist.sp_prefill_wrapper([0.25] * hq, [0.5] * hq, 64, _Args(), seq_total=n, backend=OracleBackend())
        out = fn(_Layer(), q[:, lo:hi], k[:, lo:hi], v[:, lo:hi], None)
        torch.save(out, os.path.join(tmp, f"prefill_{rank}.pt"))
        # ---- sharded decode (second sequence ends inside rank 0's range: rank 1 holds none of its keys)
        b, L = 2, 640
        g = torch.Generator().manual_seed(3)
        qd = torch.randn(b, hq, 1, d, generator=g).to(torch.bfloat16)
        kd = torch.randn(b, hkv, L, d, generator=g).to(torch.bfloat16)
        vd = torch.randn(b, hkv, L, d, generator=g).to(torch.bfloat16)
        lens = [640, 200]
        ls = L // world
        mine = [max(0, min(x, (rank + 1) * ls) - rank * ls) for x in lens]
        od = sqdist.sp_decode(qd, kd[:, :, rank * ls:(rank + 1) * ls], vd[:, :, rank * ls:(rank + 1) * ls], kv_lens=mine,
                              backend=OracleBackend())
        torch.save(od, os.path.join(tmp, f"decode_{rank}.pt"))
    finally:
        dist.destroy_process_group()


def test_world2_sequence_parallel_prefill_and_sharded_decode(tmp_path):
    world, port = 2, 29500 + os.getpid() % 2000
    mp.spawn(_worker, args=(world, port, str(tmp_path)), nprocs=world, join=True)
    n, hq, hkv, d = 512, 4, 2, 64
    q, k, v = so.make_inputs(7, 1, n, hq, hkv, d, torch.bfloat16)
    ref = so.attention_fn(q, k, v, hq // hkv, [0.25] * hq, [0.5] * hq, 64)
    got = torch.cat([torch.load(tmp_path / f"prefill_{r}.pt") for r in range(world)], dim=1)
    assert got.shape == ref.shape
    assert (got.float() - ref.float()).abs().max().item() < 2e-2
    b, L = 2, 640
    g = torch.Generator().manual_seed(3)
    qd = torch.randn(b, hq, 1, d, generator=g).to(torch.bfloat16)
    kd = torch.randn(b, hkv, L, d, generator=g).to(torch.bfloat16)
    vd = torch.randn(b, hkv, L, d, generator=g).to(torch.bfloat16)
    refd = so.decode(qd, kd, vd, output_dtype=torch.bfloat16, center_k=False, kv_lens=[640, 200], mask_tail=True)
    for r in range(world):
        od = torch.load(tmp_path / f"decode_{r}.pt")
        assert (od.float() - refd.float()).abs().max().item() < 1e-2


def test_shard_range_errors():
    from longcontext_sqattn_paddle_b200 import dist as sqdist
    assert sqdist.shard_range(1, 2, 512) == (256, 512)
    assert sqdist.shard_range(0, 1, 300) == (0, 300)
    with pytest.raises(ValueError):
        sqdist.shard_range(0, 3, 512)
    with pytest.raises(ValueError):
        sqdist.shard_range(0, 2, 200)   # 100-row shards: not a multiple of 128
