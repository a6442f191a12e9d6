"""How many FP8 rounding decisions of P differ between the CUDA prefill kernel and the reference rule.

The reference rounds P = exp2(S - m_running) through e4m3 tile by tile (sqattn/attn_triton.py:81-83).  The debug
build of the library dumps, for its first CTA, every S tile it computed and every P tile it handed to the tensor
core.  From those this test counts e4m3 codes that differ (a) from the rule applied on the CPU to the kernel's OWN S
(what the kernel's exponential and conversion instructions contribute) and (b) from the rule applied to S computed on
the CPU in fp32 (which adds the different summation order of Q K^T).  A differing code is always the neighbouring
e4m3 value: the decision flipped because p*448 sat on a rounding boundary to within the last bits of fp32."""
import ctypes as C
import importlib.util
import os

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
LOG2E = 1.44269504


@pytest.fixture(scope="module")
def dbg():
    spec = importlib.util.spec_from_file_location("_sqattn_build", os.path.join(ROOT, "longcontext_sqattn_paddle_b200", "build.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    lib = C.CDLL(mod.build_debug())
    from longcontext_sqattn_paddle_b200 import _lib as L
    lib.sqattn_debug_prefill_dump_sp.restype = C.c_int
    lib.sqattn_debug_prefill_dump_sp.argtypes = [C.POINTER(L.PrefillArgs), C.c_void_p, C.c_void_p, C.c_void_p]
    lib.sqattn_debug_schedule.restype = C.c_int
    lib.sqattn_debug_schedule.argtypes = [C.c_int] * 8 + [C.POINTER(C.c_int)]
    lib.sqattn_last_error_string.restype = C.c_char_p
    lib.sqattn_check_device_status.argtypes = [C.c_void_p]
    yield lib
    torch.cuda.synchronize()
    assert lib.sqattn_check_device_status(None) == 0


def _e4m3_codes(p):
    return (p * 448.0).to(torch.float8_e4m3fn).view(torch.uint8)


@pytest.mark.parametrize("mode,sink,w8,w4", [(0, 0, 0, 0), (2, 64, 300, 520)])
def test_fp8_rounding_decisions_of_p(dbg, mode, sink, w8, w4):
    from longcontext_sqattn_paddle_b200 import _lib as L, ops
    n, hq, hkv, d, dtype = 1536, 2, 1, 128, torch.bfloat16
    g = torch.Generator().manual_seed(41)
    q = torch.randn(1, hq, n, d, generator=g).to(dtype)
    k = torch.randn(1, hkv, n, d, generator=g).to(dtype)
    k[..., 17] *= 8
    v = torch.randn(1, hkv, n, d, generator=g).to(torch.float16)
    qs = (q.float() * torch.tensor(1.0 / d ** 0.5 * LOG2E, dtype=torch.float32)).to(dtype)   # the launcher's scaling
    blk = n // 128 - 1                                   # the kernel's first CTA takes the last query block of head 0
    sched = (C.c_int * 36)()
    nseg = dbg.sqattn_debug_schedule(mode, n, sink, w8, w4, 1, 1, blk, sched)
    steps = [(sched[3 * i] + 64 * t, sched[3 * i + 2]) for i in range(nseg) for t in range(sched[3 * i + 1])]
    dq, dk, dv = qs.cuda(), k.cuda(), v.cuda()
    out = torch.empty(1, hq, n, d, dtype=dtype, device="cuda")
    dump_s = torch.zeros(len(steps), 128, 64, device="cuda")
    dump_p = torch.zeros(len(steps), 128, 64, device="cuda")
    a = L.PrefillArgs()
    a.q_int8 = a.q_int4 = ops._view(dq, "HND")
    a.k_int8 = a.k_int4 = ops._view(dk, "HND")
    a.v, a.o = ops._view(dv, "HND"), ops._view(out, "HND")
    a.batch, a.num_q_heads, a.num_kv_heads, a.qo_len, a.kv_len, a.head_dim = 1, hq, hkv, n, n, d
    a.qk_dtype, a.v_dtype, a.o_dtype = L.BF16, L.F16, L.BF16
    a.mode, a.sink_size, a.p_fp8_mode, a.q_is_scaled = mode, sink, L.P_FP8_ALL, 1
    keep = ((C.c_int32 * hq)(*([w8] * hq)), (C.c_int32 * hq)(*([w4] * hq)))
    a.win8_sizes, a.win4_sizes = keep
    rc = dbg.sqattn_debug_prefill_dump_sp(C.byref(a), dump_s.data_ptr(), dump_p.data_ptr(), torch.cuda.current_stream().cuda_stream)
    assert rc == 0, dbg.sqattn_last_error_string()
    torch.cuda.synchronize()
    s_k, p_k = dump_s.cpu(), dump_p.cpu()
    rows = torch.arange(blk * 128, blk * 128 + 128)
    qrow = qs[0, 0, rows].float()
    m_own = torch.full((128,), float("-inf"))
    m_ref = torch.full((128,), float("-inf"))
    total = diff_own = diff_ref = far = 0
    for i, (key0, flags) in enumerate(steps):
        keys = torch.arange(key0, key0 + 64)
        s_ref = qrow @ k[0, 0, keys].float().T
        s_own = s_k[i].clone()
        if flags & 4:                                    # diagonal tile: additive causal mask
            mask = torch.where(rows[:, None] >= keys[None, :], 0.0, -1000000.0)
            s_ref, s_own = s_ref + mask, s_own + mask
        m_own = torch.maximum(m_own, s_own.max(dim=1).values)
        m_ref = torch.maximum(m_ref, s_ref.max(dim=1).values)
        c_kernel = _e4m3_codes(p_k[i])                   # p_k = f16(code) / 448: *448 gives the code's value back
        c_own = _e4m3_codes(torch.exp2(s_own - m_own[:, None]))
        c_ref = _e4m3_codes(torch.exp2(s_ref - m_ref[:, None]))
        total += c_kernel.numel()
        diff_own += (c_kernel != c_own).sum().item()
        diff_ref += (c_kernel != c_ref).sum().item()
        far += ((c_kernel.int() - c_ref.int()).abs() > 1).sum().item()
    f_own, f_ref = diff_own / total, diff_ref / total
    print(f"mode {mode}: {total} P elements; codes differing from the rule on the kernel's own S: {diff_own} ({f_own:.2e}); "
          f"from the rule on CPU fp32 S: {diff_ref} ({f_ref:.2e}); more than one code apart: {far}")
    assert far == 0
    assert f_own < 2e-3, f_own
    assert f_ref < 2e-2, f_ref
