"""Host logic of the KV cache: the reference's memory model and the block split of the hybrid cache."""
from longcontext_sqattn_paddle_b200.cache_hub import kv_memory_model, split_blocks


def test_memory_model_matches_reference_formula():
    # Qwen2.5-7B, 1M tokens, one 180 GB GPU: cache.py:45-83 / flash_attn_cache.py:128-141
    free, kv, fits = kv_memory_model(28, 1, 1048576, 4, 28, 128, 1, 7, 179.06)
    gb = 1024 ** 3
    per = 28 * 1048576 * 128 * 2 / gb
    prefill = 6 * per + (28 + 8) * 1048576 * 128 * 2 / gb
    assert abs(free - (179.06 - 14 - prefill)) < 1e-9
    assert abs(kv - 2 * 28 * 1048576 * 4 * 128 * 2 / gb) < 1e-9 and abs(kv - 56.0) < 1e-9
    assert fits == (free > kv * 1.3)
    assert kv_memory_model(28, 1, 131072, 4, 28, 128, 1, 7, 179.06)[2] is True
    assert kv_memory_model(28, 1, 1048576, 4, 28, 128, 1, 7, 80.0)[2] is False


def test_split_blocks():
    assert split_blocks(1048576, 4096, 0.25) == (262144, 786432)
    assert split_blocks(10000, 4096, 0.25) == (4096, 5904)   # 3 blocks, 1 resident
    assert split_blocks(10000, 4096, 1.0) == (10000, 0)
    assert split_blocks(10000, 4096, 0.0) == (0, 10000)
    assert split_blocks(100, 4096, 0.5) == (0, 100) or split_blocks(100, 4096, 0.5) == (100, 0)


def test_host_pipeline_chunk_bounds():
    """HostPrefillPipeline cuts the query rows into a short first chunk, full chunks and a short last chunk; every
    chunk starts on a multiple of 128 rows, none is longer than chunk_rows, together they cover the sequence once."""
    import types
    from longcontext_sqattn_paddle_b200.sqattn import HostPrefillPipeline
    for n, chunk, edge in ((131072, 8192, 2048), (32768, 8192, 2048), (16384, 8192, 2048), (8192, 8192, 2048),
                           (5000, 4096, 2048), (20000, 4096, 2048), (128, 4096, 2048), (131000, 8192, 2048), (1664, 512, 128)):
        cfg = types.SimpleNamespace(chunk=chunk, edge=min(edge, chunk))
        bounds = HostPrefillPipeline._bounds(cfg, n)
        assert bounds[0][0] == 0 and bounds[-1][1] == n
        assert all(a[1] == b[0] for a, b in zip(bounds, bounds[1:]))
        assert all(0 < r1 - r0 <= chunk and r0 % 128 == 0 for r0, r1 in bounds)
        if n > 2 * chunk:
            assert bounds[0][1] == cfg.edge and bounds[-1][1] - bounds[-1][0] <= cfg.edge + 127
