"""sqattn_decode_static_scratch: the decode entry point for callers that may not allocate device memory (it keeps
its split-KV partials in an array built into the library).  Called through the C ABI, twice in a row on
different inputs, its output must equal what sqattn_decode produces with a caller workspace (same kernels, same
order of operations: the tolerance of the other decode tests, 2e-2, is far from needed).  This file sorts last so
that a run stopping at the first failure has already run everything else."""
import ctypes as C

import pytest
import torch

pytestmark = pytest.mark.gpu


def _args(L, ops, q, k, v, out, lse, kv_lens=None, num_splits=0):
    b, hq, _, d = q.shape
    a = L.DecodeArgs()
    a.q, a.k, a.v, a.o = (ops._view(t, "HND") for t in (q, k, v, out))
    a.lse = lse.data_ptr()
    a.batch, a.num_q_heads, a.num_kv_heads, a.head_dim = b, hq, k.shape[1], d
    a.kv_len = k.shape[2]
    keep = None
    if kv_lens is not None:
        keep = (C.c_int32 * b)(*kv_lens)
        a.kv_lens = keep
    a.dtype = a.o_dtype = ops._dt(q.dtype)
    a.num_splits = num_splits
    return a, keep


def test_static_scratch_matches_workspace_entry_point_twice():
    from longcontext_sqattn_paddle_b200 import _lib as L, ops
    stream = torch.cuda.current_stream().cuda_stream
    for call, (b, hq, hkv, n, d, lens) in enumerate([(2, 28, 4, 7000, 128, None), (3, 32, 8, 3000, 128, [3000, 17, 1234])]):
        g = torch.Generator().manual_seed(100 + call)
        q = torch.randn(b, hq, 1, d, generator=g).to(torch.bfloat16).cuda()
        k = torch.randn(b, hkv, n, d, generator=g).to(torch.bfloat16).cuda()
        v = torch.randn(b, hkv, n, d, generator=g).to(torch.bfloat16).cuda()
        ref, ref_lse = torch.empty_like(q), torch.empty(b, hq, dtype=torch.float32, device="cuda")
        a, keep = _args(L, ops, q, k, v, ref, ref_lse, lens)
        need = L.lib.sqattn_decode_workspace_bytes(C.byref(a))
        ws = torch.empty(need + 256, dtype=torch.uint8, device="cuda")
        a.workspace = ws.data_ptr() + (-ws.data_ptr()) % 256
        a.workspace_bytes = need
        assert L.lib.sqattn_decode(C.byref(a), stream) == 0, L.lib.sqattn_last_error_string()

        out, out_lse = torch.full_like(q, float("nan")), torch.full_like(ref_lse, float("nan"))
        a2, keep2 = _args(L, ops, q, k, v, out, out_lse, lens)   # no workspace given
        before = torch.cuda.memory_allocated()
        assert L.lib.sqattn_decode_static_scratch(C.byref(a2), stream) == 0, L.lib.sqattn_last_error_string()
        torch.cuda.synchronize()
        assert torch.cuda.memory_allocated() == before
        assert torch.isfinite(out).all() and torch.isfinite(out_lse).all()
        assert (out.float() - ref.float()).abs().max().item() <= 2e-2
        assert torch.equal(out, ref) and torch.equal(out_lse, ref_lse)
    ops.check_device_status()


def test_static_scratch_rejects_oversized_calls():
    from longcontext_sqattn_paddle_b200 import _lib as L, ops
    b, hq, hkv, n, d = 64, 32, 8, 4096, 128
    q = torch.zeros(b, hq, 1, d, dtype=torch.bfloat16, device="cuda")
    k = torch.zeros(b, hkv, n, d, dtype=torch.bfloat16, device="cuda")
    out, lse = torch.empty_like(q), torch.empty(b, hq, dtype=torch.float32, device="cuda")
    a, _ = _args(L, ops, q, k, k, out, lse, num_splits=16)   # 64 x 16 ranges x 32 heads = 32768 partial rows
    rc = L.lib.sqattn_decode_static_scratch(C.byref(a), torch.cuda.current_stream().cuda_stream)
    assert rc == L.ERR_WORKSPACE
    assert b"built-in scratch" in L.lib.sqattn_last_error_string()
    with pytest.raises(L.SqattnError):
        ops.decode_static_scratch(q, k, k, out, num_splits=16)
