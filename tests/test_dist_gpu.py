"""Two-GPU run of the sequence-parallel prefill and the cross-GPU split-KV decode (NCCL and peer-store exchange).  Skipped on a
single-GPU box; the partitioning logic itself is also covered by the gloo tests on CPU."""
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


def _worker(rank, world, port, tmp):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        from longcontext_sqattn_paddle_b200 import dist as sqdist, ops
        n, hq, hkv, d = 2048, 28, 4, 128
        q, k, v = so.make_inputs(21, 1, n, hq, hkv, d, torch.bfloat16)
        lo, hi = sqdist.shard_range(rank, world, n)
        fn = sqdist.sp_prefill_wrapper([0.1] * hq, [0.3] * hq, 256, _Args(), seq_total=n)
        out = fn(_Layer(), q[:, lo:hi].cuda(), k[:, lo:hi].cuda(), v[:, lo:hi].cuda(), None)
        torch.save(out.cpu(), os.path.join(tmp, f"prefill_{rank}.pt"))
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
    ref = so.attention_fn(q, k, v, hq // hkv, [0.1] * hq, [0.3] * hq, 256)
    got = torch.cat([torch.load(tmp_path / f"prefill_{r}.pt") for r in range(world)], dim=1)
    assert (got.float() - ref.float()).abs().max().item() < 2e-2
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
