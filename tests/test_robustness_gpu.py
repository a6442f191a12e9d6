"""Boundary behaviour around the kernels: head_dim padding like the reference launchers, rejected arguments, and the
failure path of a bounded device-side wait.  The failure is produced by a wait that simply runs out (a flag that
nobody sets); nothing faults, traps or hangs, and the context stays usable."""
import ctypes as C
import time

import pytest
import torch

from oracle import sqattn_oracle as so

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def pkg():
    from longcontext_sqattn_paddle_b200 import ops, sqattn
    yield ops, sqattn
    torch.cuda.synchronize()
    ops.check_device_status()


def _rand(shape, seed, dtype):
    g = torch.Generator().manual_seed(seed)
    return torch.randn(*shape, generator=g).to(dtype)


@pytest.mark.parametrize("d", [32, 80, 96])
def test_head_dim_is_padded_like_the_reference_launchers(pkg, d):
    """head_dim < 64 -> 64, 64 < head_dim < 128 -> 128, scaled with the ORIGINAL head_dim, output sliced back
    (sqattn/attn_triton.py:236-253, 314; attn_triton_mix_relative.py:369-385; attn_triton_decode.py:254-271)."""
    ops, sq = pkg
    dtype, n, hq, hkv = torch.bfloat16, 640, 4, 2
    q, k, v = _rand((1, hq, n, d), 1, dtype), _rand((1, hkv, n, d), 2, dtype), _rand((1, hkv, n, d), 3, dtype)
    o, lse = sq.attn_causal(q.cuda(), k.cuda(), v.cuda(), "HND", dtype, True, False)
    ro, rlse = so.dense_causal(q, k, v, output_dtype=dtype, return_lse=True)
    assert o.shape == q.shape
    assert (o.float().cpu() - ro.float()).abs().max().item() < 2e-2
    assert (lse.cpu() - rlse).abs().max().item() < 2e-3
    r8, r4 = [0.25] * hq, [0.5] * hq
    o = sq.attn_hierarchical_relative_window(q.cuda(), k.cuda(), q.cuda(), k.cuda(), v.cuda(), r8, r4, 64, "HND", dtype)
    ro = so.windowed_prefill(q, k, q, k, v, r8, r4, 64, mode="relative", output_dtype=dtype)
    assert o.shape == q.shape
    assert (o.float().cpu() - ro.float()).abs().max().item() < 2e-2
    o = sq.attn_hierarchical_window(q.cuda(), k.cuda(), q.cuda(), k.cuda(), v.cuda(), [200] * hq, [300] * hq, 32, "HND", dtype)
    ro = so.windowed_prefill(q, k, q, k, v, [200] * hq, [300] * hq, 32, mode="absolute", output_dtype=dtype)
    assert (o.float().cpu() - ro.float()).abs().max().item() < 2e-2
    qd = _rand((2, hq, 1, d), 4, dtype)
    kd, vd = _rand((2, hkv, 777, d), 5, dtype), _rand((2, hkv, 777, d), 6, dtype)
    od = sq.attn_unified(qd.cuda(), kd.cuda(), vd.cuda(), "HND", dtype, False, False)
    rod = so.decode(qd, kd, vd, output_dtype=dtype)
    assert od.shape == qd.shape
    assert (od.float().cpu() - rod.float()).abs().max().item() < 2e-2
    with pytest.raises(ValueError):
        sq.attn_causal(_rand((1, 1, 128, 160), 7, dtype).cuda(), _rand((1, 1, 128, 160), 8, dtype).cuda(),
                       _rand((1, 1, 128, 160), 9, dtype).cuda())


def test_decode_rejects_lengths_beyond_the_cache(pkg):
    ops, _ = pkg
    dtype = torch.bfloat16
    q, k, v = _rand((2, 4, 1, 128), 1, dtype).cuda(), _rand((2, 2, 512, 128), 2, dtype).cuda(), _rand((2, 2, 512, 128), 3, dtype).cuda()
    with pytest.raises(ValueError, match="cache holds"):
        ops.decode(q, k, v, kv_lens=[512, 513])
    ops.decode(q, k, v, kv_lens=[512, 1])


def _peer_args(L, world, rank, rows, d, data, flags, epoch, out, po, pl):
    a = L.PeerMergeArgs()
    for w in range(world):
        a.peer_data[w], a.peer_flags[w] = data[w].data_ptr(), flags[w].data_ptr()
    a.rank, a.world, a.rows, a.rows_cap, a.head_dim, a.epoch = rank, world, rows, rows, d, epoch.data_ptr()
    a.part_o, a.part_lse, a.out, a.o_dtype = po.data_ptr(), pl.data_ptr(), out.data_ptr(), L.BF16
    return a


def test_a_wait_that_runs_out_is_reported_and_poisons_nothing_silently(pkg):
    """The cross-GPU merge waits for the flag of every other rank.  Here "rank 1" is a second pair of buffers on the
    same GPU that no kernel ever publishes to, so rank 0's wait runs into its one-second limit: the kernel returns,
    its rows are NaN, the host mirror and sqattn_check_device_status report the timeout, launches made while the
    word is set return NaN instead of computing, and after the status has been read everything works again."""
    ops, _ = pkg
    from longcontext_sqattn_paddle_b200 import _lib as L
    dev = torch.device("cuda", 0)
    ops.poll_device_status(dev)            # installs the host mirror
    rows, d, world = 8, 128, 2
    nd = L.lib.sqattn_peer_merge_data_bytes(world, rows, d) // 4
    nf = L.lib.sqattn_peer_merge_flag_bytes(world, rows) // 4
    data = [torch.zeros(nd, dtype=torch.int32, device=dev) for _ in range(world)]
    flags = [torch.zeros(nf, dtype=torch.int32, device=dev) for _ in range(world)]
    epoch = torch.zeros(1, dtype=torch.int32, device=dev)
    po, pl = torch.randn(rows, d, device=dev), torch.randn(rows, device=dev)
    out = torch.zeros(rows, d, dtype=torch.bfloat16, device=dev)
    a = _peer_args(L, world, 0, rows, d, data, flags, epoch, out, po, pl)
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    L.check(L.lib.sqattn_decode_peer_merge(C.byref(a), torch.cuda.current_stream().cuda_stream))
    torch.cuda.synchronize()
    dt = time.perf_counter() - t0
    assert 0.9 < dt < 5.0, f"the wait should give up after about one second, took {dt:.2f}s"
    assert torch.isnan(out.float()).all()
    # while the word is set: the host mirror raises without a synchronisation, and kernels deliver NaN, not stale memory
    with pytest.raises(L.SqattnError) as ei:
        ops.poll_device_status(dev)
    assert ei.value.code == L.ERR_DEVICE_TIMEOUT
    dtype = torch.bfloat16
    q, k, v = _rand((1, 4, 256, 128), 1, dtype).cuda(), _rand((1, 2, 256, 128), 2, dtype).cuda(), _rand((1, 2, 256, 128), 3, dtype).cuda()
    ent = ops._MIRRORS[0]
    ent[1].value = 0                       # a caller that ignored the mirror and carried on
    o = ops.prefill(q, k, q, k, v, mode=L.MODE_DENSE_CAUSAL, out_dtype=dtype)
    od = ops.decode(q[:, :, :1], k, v, out_dtype=dtype)
    torch.cuda.synchronize()
    assert torch.isnan(o.float()).all() and torch.isnan(od.float()).all()
    with pytest.raises(L.SqattnError) as ei:
        ops.check_device_status()
    assert ei.value.code == L.ERR_DEVICE_TIMEOUT and "301" in str(ei.value)
    # cleared: the same calls compute again
    ops.check_device_status()
    o = ops.prefill(q, k, q, k, v, mode=L.MODE_DENSE_CAUSAL, out_dtype=dtype)
    od = ops.decode(q[:, :, :1], k, v, out_dtype=dtype)
    ro = so.dense_causal(q.cpu(), k.cpu(), v.cpu(), output_dtype=dtype)
    assert (o.float().cpu() - ro.float()).abs().max().item() < 2e-2
    assert torch.isfinite(od.float()).all()
    # and the exchange works once both "ranks" take part: two launches on one GPU must not wait for each other, so
    # rank 1's words are written by hand before rank 0's kernel runs
    data = [torch.zeros(nd, dtype=torch.int32, device=dev) for _ in range(world)]
    flags = [torch.zeros(nf, dtype=torch.int32, device=dev) for _ in range(world)]
    epoch.zero_()
    po1, pl1 = torch.randn(rows, d, device=dev), torch.randn(rows, device=dev)
    # [parity][source rank][row][D+1] words of {fp32 bits, step number}; the first call is step 1 and uses parity 1
    slot = data[0].view(2, world, rows, d + 1, 2)
    slot[1, 1, :, :d, 0], slot[1, 1, :, d, 0] = po1.view(torch.int32), pl1.view(torch.int32)
    slot[1, 1, :, :, 1] = 1
    a = _peer_args(L, world, 0, rows, d, data, flags, epoch, out, po, pl)
    L.check(L.lib.sqattn_decode_peer_merge(C.byref(a), torch.cuda.current_stream().cuda_stream))
    torch.cuda.synchronize()
    ops.check_device_status()
    ref = ops.decode_merge(torch.stack([po, po1]), torch.stack([pl, pl1]), out_dtype=torch.bfloat16)
    assert torch.equal(out, ref)


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_one_process_decodes_on_two_devices(pkg):
    """Function attributes (the decode kernel's dynamic shared memory) belong to a device: the second GPU of a
    single process (layer-to-device placement, model_hub/qwen.py:203-267) must work like the first."""
    ops, _ = pkg
    dtype = torch.bfloat16
    q, k, v = _rand((1, 28, 1, 128), 1, dtype), _rand((1, 4, 3000, 128), 2, dtype), _rand((1, 4, 3000, 128), 3, dtype)
    ro = so.decode(q, k, v, output_dtype=dtype, center_k=False)
    scratch_out = torch.empty(1, 28, 1, 128, dtype=dtype)
    for idx in (0, 1):
        with torch.cuda.device(idx):
            dev = torch.device("cuda", idx)
            o = ops.decode(q.to(dev), k.to(dev), v.to(dev), out_dtype=dtype)
            o2 = ops.decode_static_scratch(q.to(dev), k.to(dev), v.to(dev), scratch_out.to(dev))
            torch.cuda.synchronize(dev)
            ops.check_device_status()
            assert (o.float().cpu() - ro.float()).abs().max().item() < 2e-2
            assert torch.equal(o, o2)
